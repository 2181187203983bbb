"""Benchmark of the hot path: NVFP4 paged MLA decode at the headline shape (H=16, B=64, 64K-token contexts).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

One "step" is one decode call over the whole batch. With N > 1 (launched by torchrun, one rank per GPU) the batch is
sharded data-parallel: every rank holds its own B requests and their pages, nothing is exchanged, and the reported
value is the bytes all ranks streamed divided by the slowest rank's time (weak scaling). Rank 0 prints one JSON line.

  value      KV-cache bandwidth, 352 bytes per cached token / device time per step (CUDA events on the launching
             stream, inputs resident in HBM; the cache is far larger than L2, so no flush is needed)
  e2e        the same through the Python API with the per-step inputs (queries, page table, lengths) coming from
             pinned host memory (one packed buffer, one copy per step) and the output copied back to the host inside
             the timed region. The KV cache itself is device-resident state written by earlier steps of a serving
             engine, not a per-step input.
  roofline   the decode kernel alone (timed by the library's own event pair around it) against the measured HBM peak
  cpu_baseline / --impl reference
             the reference's CPU path (dequantize, then fp32 attention: its own torch functions from the unmodified
             package under baseline/_ref, else their numpy restatement oracle/mla_oracle.py), timed on this box's host
             cores over a bounded sample of the same workload
  reference_gpu (--reference-gpu)
             the reference's own CUDA kernel from baseline/_ref on the same GPU and inputs
"""
import argparse
import ctypes
import datetime
import json
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (batch, heads, kv_len, page_size, precision)
    "c2_h16_b64_64k": (64, 16, 65536, 64, "bf16"),   # the headline configuration: the shape the metric is quoted on
    "c1_h16_b32_8k": (32, 16, 8192, 64, "bf16"),     # a DeepSeek-V3 TP8 shard at 8K context
    "h16_b64_16k": (64, 16, 16384, 64, "bf16"),
    "h16_b8_64k": (8, 16, 65536, 64, "bf16"),        # small case for ncu captures (185 MB of KV, still larger than L2)
    "h16_b148_128": (148, 16, 128, 64, "bf16"),      # one 128-token tile per CTA: the fixed costs of a call
    "h128_b64_16k": (64, 128, 16384, 64, "bf16"),
    # the compute-bound configuration: ragged lengths drawn uniformly from [1024, 32768] (seeded, per rank), 8-bit mode; tensor-bound
    "c3_h128_b64_ragged_fp8": (64, 128, (1024, 32768), 64, "fp8"),
    "h128_b32_16k_fp8": (32, 128, 16384, 64, "fp8"),  # small case for ncu captures of the 128-head shape
    "c4_h128_b2_1m_seq": (2, 128, 1048576, 64, "bf16"),  # the long-context configuration: sequence-sharded, strong scaling
}
SEQUENCE_SHARDED = {"c4_h128_b2_1m_seq"}
TOKEN_BYTES = 352
# Published by the reference for this exact shape on B200: its SM100 tcgen05 kernel, 0.309 ms = 4.77 TB/s
# (README.md:194 and benchmarks/results/b200.csv:108 of the reference project).
BASELINE_TBPS = {"c2_h16_b64_64k": 4.77}
# DRAM bytes (read + write) per cached token of the H=16 decode kernels, from ncu captures of a smaller case of the same
# kernels (h16_b8_64k: 524 288 tokens); the kernels are persistent and stream each token once, so traffic grows with the
# token count and the benchmark scales it to its own workload (roofline.traffic_kind says so).
NCU_TRAFFIC_BYTES_PER_TOKEN = {"bf16": 401, "fp8": 398}


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def measured_tensor_peak(precision):
    """Dense tensor peak in TFLOP/s for the roofline of the 128-head shapes: the measured cuBLAS bf16 burst figure; the
    8-bit mode is held against twice that (E4M3 MMAs run at twice the 16-bit rate; no measured fp8 figure exists)."""
    p = ROOT / "MEASURED_PEAKS.json"
    bf16, kind = (float(json.loads(p.read_text())["bf16_tflops"]), "measured") if p.exists() else (1590.0, "fallback")
    return (bf16, f"of {kind} bf16") if precision == "bf16" else (2 * bf16, f"of 2 x {kind} bf16")


def request_lengths(kv_len, batch, seed):
    """kv_len is one length for every request, or (lo, hi) for seeded uniform ragged lengths."""
    if isinstance(kv_len, tuple):
        import numpy as np
        return [int(x) for x in np.random.default_rng(1234 + seed).integers(kv_len[0], kv_len[1] + 1, size=batch)]
    return [kv_len] * batch


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU with nvidia-smi.

    The process is started early (nvidia-smi needs a moment before its first sample) and runs until stop(); the
    benchmark marks the wall-clock window of its timed region and the summary uses the samples inside it. If the
    region is too short to hold three samples, the window is widened to everything from the first mark to stop()
    (warm-up, timed and end-to-end loops, all of them under the same load) and the summary says so."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    PERIOD_MS = 50

    def __init__(self, index):
        self.rows, self.proc, self.marks = [], None, {}
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", str(self.PERIOD_MS)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def mark(self, name):
        self.marks[name] = datetime.datetime.now()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        self.mark("stop")
        time.sleep(2.5 * self.PERIOD_MS / 1e3)  # let the last samples of the window arrive
        self.proc.terminate()
        self.thread.join(timeout=2)
        samples = []
        for r in self.rows:
            try:
                ts = datetime.datetime.strptime(r[0], "%Y/%m/%d %H:%M:%S.%f")
                samples.append((ts, float(r[1]), float(r[2]), float(r[3]), r[4:8]))
            except (ValueError, IndexError):
                continue

        def inside(a, b):
            return [x for x in samples if self.marks.get(a) and self.marks.get(b) and self.marks[a] <= x[0] <= self.marks[b]]
        chosen, window = inside("timed_begin", "timed_end"), "timed region"
        if len(chosen) < 3:
            chosen, window = inside("load_begin", "stop"), "warm-up, timed and end-to-end loops (timed region too short)"
        reasons = set()
        for x in chosen:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), x[4]):
                if v == "Active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(x[1] for x in chosen) if chosen else None,
                "sm_max_mhz": chosen[0][2] if chosen else None, "power_w_max": max((x[3] for x in chosen), default=None),
                "reasons": sorted(reasons), "samples": len(chosen), "window": window}


_REF_TESTING = None


def reference_torch_path():
    """The reference's own torch test path (`nvfp4_mla/testing.py`: dequantize, attention) from the unmodified package
    installed under baseline/_ref, or None if it is absent or does not import (the module imports flashinfer at its top)."""
    global _REF_TESTING
    if _REF_TESTING is None:
        _REF_TESTING = False
        f = ROOT / "baseline" / "_ref" / "nvfp4_mla" / "testing.py"
        if f.exists():
            try:
                import importlib.util
                spec = importlib.util.spec_from_file_location("nvfp4_mla_reference_testing", f)
                mod = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(mod)
                _REF_TESTING = mod
            except Exception:
                _REF_TESTING = False
    return _REF_TESTING or None


def cpu_reference_sample(cache, n_requests, repeats=1):
    """Times the reference's CPU path (dequantize + fp32 attention on host cores) on `n_requests` requests of the
    workload: the reference's own torch functions when baseline/_ref holds the package (kind "reference"), else the
    numpy port under oracle/ (kind "port").

    Returns (seconds per pass, KV bytes per pass, threads, kind). The sample's pages are copied to the host first; the
    copy is not timed."""
    import numpy as np
    import torch
    ps = cache.page_size
    reqs = list(range(min(n_requests, len(cache.kv_lens_list))))
    nbytes = TOKEN_BYTES * sum(cache.kv_lens_list[b] for b in reqs)
    ref = reference_torch_path()
    if ref is not None:
        inputs = []
        for b in reqs:
            L = cache.kv_lens_list[b]
            pages = cache.page_table[b, :(L + ps - 1) // ps].long()
            inputs.append((cache.q_nope[b:b + 1].cpu(), cache.q_pe[b:b + 1].cpu(), cache.ckv_cache[pages].cpu(),
                           cache.ckv_sf_cache[pages].cpu(), cache.kpe_cache[pages].cpu(),
                           torch.arange(pages.numel(), dtype=torch.int32)[None], torch.tensor([L], dtype=torch.int32)))
        t0 = time.perf_counter()
        for _ in range(repeats):
            for q_nope, q_pe, ckv8, sf8, kpe8, pt, lens in inputs:
                ckv, kpe = ref.dequantize(ckv8, sf8, kpe8, cache.ckv_scale, cache.kpe_scale)
                ref.attention(q_nope, q_pe, ckv, kpe, pt, lens, ref.SM_SCALE)
        dt = (time.perf_counter() - t0) / repeats
        return dt, nbytes, torch.get_num_threads(), "reference"
    sys.path.insert(0, str(ROOT / "oracle"))
    import mla_oracle as O
    inputs = []
    for b in reqs:
        L = cache.kv_lens_list[b]
        pages = cache.page_table[b, :(L + ps - 1) // ps].long()
        inputs.append(dict(
            q_nope=cache.q_nope[b:b + 1].float().cpu().numpy(), q_pe=cache.q_pe[b:b + 1].float().cpu().numpy(),
            ckv=cache.ckv_cache[pages].cpu().numpy(), sf=cache.ckv_sf_cache[pages].view(torch.uint8).cpu().numpy(),
            kpe=cache.kpe_cache[pages].view(torch.uint8).cpu().numpy(),
            pt=np.arange(pages.numel(), dtype=np.int32)[None], L=np.array([L], np.int32)))
    t0 = time.perf_counter()
    for _ in range(repeats):
        for a in inputs:
            ckv, kpe = O.dequantize(a["ckv"], a["sf"], a["kpe"], cache.ckv_scale, cache.kpe_scale)
            O.attention(a["q_nope"], a["q_pe"], ckv, kpe, a["pt"], a["L"], O.SM_SCALE)
    dt = (time.perf_counter() - t0) / repeats
    return dt, nbytes, os.cpu_count(), "port"


CPU_ARM_TEXT = {"reference": "the reference's own torch path (nvfp4_mla/testing.py from baseline/_ref) on host cores",
                "port": "numpy port of the reference torch path"}


def bench_writer(args):
    """`--workload writer_1m`: one step = quantise and append 1 048 576 new tokens (64 requests x 16 384) into an empty
    paged cache with the CUDA cache writer. HBM-bound: 1152 bytes read + 352 written per token. One GPU."""
    import numpy as np
    import torch
    import nvfp4_mla_b200 as mla
    B, L, ps = 64, 16384, 64
    nnz, bytes_per_token = B * L, 1152 + TOKEN_BYTES
    if args.impl == "reference" or not torch.cuda.is_available():
        # CPU arm: the numpy writer of the oracle on a sample of the tokens
        sys.path.insert(0, str(ROOT / "oracle"))
        import mla_oracle as O
        n = 16384
        rng = np.random.default_rng(0)
        ckv, kpe = rng.standard_normal((n, 512), dtype=np.float32), rng.standard_normal((n, 64), dtype=np.float32)
        t0 = time.perf_counter()
        O.quantize_ckv(ckv, 2.0 ** -9), O.quantize_kpe(kpe, 2.0 ** -6)
        dt = time.perf_counter() - t0
        val = n * bytes_per_token / dt / 1e9
        print(json.dumps({"impl": "reference", "metric": "nvfp4_mla_writer_bandwidth", "value": val, "unit": "GB/s", "n_gpus": 1,
                          "steps": 1, "warmup": 0, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": "writer_1m"},
                          "cpu_baseline": {"value": val, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
                                           "sample": f"{n} tokens, numpy writer of the oracle"},
                          "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    ckv = torch.randn(nnz, 512, generator=g, device=dev).bfloat16()
    kpe = torch.randn(nnz, 64, generator=g, device=dev).bfloat16()
    P = B * L // ps
    kv_indices = torch.randperm(P, generator=g, device=dev).int()
    kv_indptr = (torch.arange(B + 1, device=dev) * (L // ps)).int()
    lens = torch.full((B,), L, dtype=torch.int32, device=dev)
    bi, pos = mla.get_batch_indices_positions((torch.arange(B + 1, device=dev) * L).int(), lens, nnz)
    caches = (torch.zeros(P, ps, 256, dtype=torch.uint8, device=dev),
              torch.zeros(P, ps, 32, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn),
              torch.zeros(P, ps, 64, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn))

    def step():
        mla.quantize_append_paged_mla_kv_cache(ckv, kpe, bi, pos, *caches, kv_indices, kv_indptr, None, 2.0 ** -9, 2.0 ** -6)
    steps = min(args.steps, 200)
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.mark("load_begin"), sampler.mark("timed_begin")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    sampler.mark("timed_end")
    ms = e0.elapsed_time(e1) / steps
    # end to end: the new rows come from pinned host memory every step, a device-to-host read of one cache page ends it
    hc, hk = ckv.cpu().pin_memory(), kpe.cpu().pin_memory()
    page = torch.empty(ps, 256, dtype=torch.uint8).pin_memory()
    e0.record()
    for _ in range(3):
        ckv.copy_(hc, non_blocking=True), kpe.copy_(hk, non_blocking=True)
        step()
        page.copy_(caches[0][0], non_blocking=True)
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / 3
    peak, kind = measured_peak()
    val = nnz * bytes_per_token / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "nvfp4_mla_writer_bandwidth", "value": val, "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 arithmetic on bf16 inputs",
        "data": "synthetic",
        "config": {"workload": f"writer_1m: {nnz} new tokens (B={B} x {L}), page_size={ps}, shuffled pages",
                   "l2": "1.6 GB touched per step, larger than L2, no flush"},
        "e2e": {"value": nnz * bytes_per_token / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": nnz * 1152, "d2h_bytes_per_step": ps * 256},
        "gpu_launches": steps,
        "roofline": {"bound": "hbm", "achieved": val, "peak": peak, "unit": "GB/s", "frac": val / peak, "peak_kind": f"of {kind}",
                     "kernel": "mla_quantize_append_kernel", "algorithmic_bytes_per_launch": nnz * bytes_per_token, "traffic": None},
        "clocks": sampler.stop()}))


def bench_dequant(args):
    """`--workload dequant_1m`: one step = dequantise a cache of 1 048 576 tokens to BF16 with `dequantize` (the
    reference's `nvfp4_mla.dequantize`, csrc/mla_decode.cu:1101-1132). HBM-bound: 352 bytes read + 1152 written per token."""
    import numpy as np
    import torch
    import nvfp4_mla_b200 as mla
    P, ps = 16384, 64
    ntok, bytes_per_token = P * ps, TOKEN_BYTES + 1152
    if args.impl == "reference" or not torch.cuda.is_available():
        sys.path.insert(0, str(ROOT / "oracle"))
        import mla_oracle as O
        n = 256  # pages
        rng = np.random.default_rng(0)
        ckv = rng.integers(0, 256, (n, ps, 256), dtype=np.uint8)
        sf = rng.integers(0, 0x7F, (n, ps, 32), dtype=np.uint8)
        kpe = rng.integers(0, 0x7F, (n, ps, 64), dtype=np.uint8)
        t0 = time.perf_counter()
        O.dequantize(ckv, sf, kpe, 2.0 ** -9, 2.0 ** -6)
        dt = time.perf_counter() - t0
        val = n * ps * bytes_per_token / dt / 1e9
        print(json.dumps({"impl": "reference", "metric": "nvfp4_mla_dequantize_bandwidth", "value": val, "unit": "GB/s", "n_gpus": 1,
                          "steps": 1, "warmup": 0, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": "dequant_1m"},
                          "cpu_baseline": {"value": val, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
                                           "sample": f"{n * ps} tokens, numpy dequantize of the oracle"},
                          "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    ckv = torch.randint(0, 256, (P, ps, 256), generator=g, device=dev, dtype=torch.uint8)
    sf = torch.randint(0, 0x7F, (P, ps, 32), generator=g, device=dev, dtype=torch.uint8).view(torch.float8_e4m3fn)
    kpe = torch.randint(0, 0x7F, (P, ps, 64), generator=g, device=dev, dtype=torch.uint8).view(torch.float8_e4m3fn)

    def step():
        return mla.dequantize(ckv, sf, kpe, 2.0 ** -9, 2.0 ** -6)
    steps = min(args.steps, 200)
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.mark("load_begin"), sampler.mark("timed_begin")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = step()
    e1.record()
    torch.cuda.synchronize()
    sampler.mark("timed_end")
    ms = e0.elapsed_time(e1) / steps
    # end to end: the cache comes from pinned host memory every step, a device-to-host read of one page's values ends it
    host = [t.view(torch.uint8).cpu().pin_memory() for t in (ckv, sf, kpe)]
    page = torch.empty(ps, 512, dtype=torch.bfloat16).pin_memory()
    e0.record()
    for _ in range(3):
        for d, h in zip((ckv, sf, kpe), host):
            d.view(torch.uint8).copy_(h, non_blocking=True)
        out = step()
        page.copy_(out[0][0], non_blocking=True)
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / 3
    peak, kind = measured_peak()
    val = ntok * bytes_per_token / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "nvfp4_mla_dequantize_bandwidth", "value": val, "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 arithmetic, bf16 output",
        "data": "synthetic",
        "config": {"workload": f"dequant_1m: {ntok} tokens ({P} pages of {ps}), random bytes, BF16 output",
                   "l2": "1.6 GB touched per step, larger than L2, no flush"},
        "e2e": {"value": ntok * bytes_per_token / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": ntok * TOKEN_BYTES, "d2h_bytes_per_step": ps * 1024},
        "gpu_launches": steps,
        "roofline": {"bound": "hbm", "achieved": val, "peak": peak, "unit": "GB/s", "frac": val / peak, "peak_kind": f"of {kind}",
                     "kernel": "mla_dequant_kernel", "algorithmic_bytes_per_launch": ntok * bytes_per_token, "traffic": None},
        "clocks": sampler.stop()}))


LN2 = 0.6931471805599453


def parity_check(mla, mdist, cache, dargs, kw, out, precision, seq, rank, world, dev):
    """Outside the timed region: a sample of the step's output (first, middle and last request; 16 heads when there are
    more) against the streamed dequantise-then-attention reference in torch on the GPU. 16-bit mode: max-abs <= 2e-2 and,
    where the call returns it, natural-log LSE <= 1e-3; 8-bit mode: rel-L2 < 0.08. Sequence-sharded workloads: every
    rank computes the reference over its own slice of the sampled request, the slices are merged with the exact
    log-sum-exp weights on rank 0 and held against the merged output of the step. Returns a dict (rank 0 decides)."""
    import torch
    import torch.distributed as dist
    from nvfp4_mla_b200.testing import attention_paged_nvfp4, rel_l2
    B, H = cache.q_nope.shape[:2]
    reqs = [B - 1] if seq else sorted({0, B // 2, B - 1})
    heads = list(range(H)) if H <= 16 else list(range(3, H, H // 16))
    a = list(dargs)
    a[0], a[1] = cache.q_nope[:, heads].contiguous(), cache.q_pe[:, heads].contiguous()
    want, want_lse = attention_paged_nvfp4(*a, requests=reqs)
    lse_abs = None
    if seq and world > 1:
        ws = [torch.empty_like(want) for _ in range(world)]
        ls = [torch.empty_like(want_lse) for _ in range(world)]
        dist.all_gather(ws, want.contiguous())
        dist.all_gather(ls, want_lse.contiguous())
        ws, ls = torch.stack(ws).double(), torch.stack(ls).double()
        tot = torch.logsumexp(ls, 0)
        want = ((ls - tot).exp().unsqueeze(-1) * ws).sum(0).float()
    elif precision == "bf16":
        _, lse2 = mla.decode_partial(*dargs, **kw)
        lse_abs = (lse2[reqs][:, heads] * LN2 - want_lse).abs().max().item()
    got = out[reqs][:, heads].float()
    max_abs, rel = (got - want).abs().max().item(), rel_l2(got, want)
    if precision == "bf16":
        ok = max_abs <= 2e-2 and rel < 4e-3 and (lse_abs is None or lse_abs <= 1e-3)
    else:
        ok = rel < 0.08
    ok = ok and not bool(out.isnan().any())
    return {"requests": reqs, "heads_sampled": len(heads), "max_abs": max_abs, "rel_l2": rel, "lse_abs": lse_abs, "ok": bool(ok),
            "against": "streamed torch dequantise-then-attention on the GPU (the oracle's arithmetic), outside the timed region"}


def measure(args, workload, precision, steps, warmup, rank, world, dev, sampler, want_e2e=True):
    """Generates the workload on this rank, runs warm-up + two timed passes (+ the end-to-end loop), returns a dict."""
    import torch
    import torch.distributed as dist
    import nvfp4_mla_b200 as mla
    from nvfp4_mla_b200 import _lib
    from nvfp4_mla_b200 import dist as mdist
    from nvfp4_mla_b200.testing import SM_SCALE, SyntheticCache

    B, H, kv_len, ps, _ = WORKLOADS[workload]
    seq = workload in SEQUENCE_SHARDED
    if seq:
        # every rank holds a contiguous 1/world slice of each request's pages (generated directly as the local slice:
        # rank r's tokens are a seeded stream of their own), queries replicated
        local_len = mdist.shard_sequence(kv_len, ps, world)[rank][2]
        cache = SyntheticCache([local_len] * B, ps, H, 2.0 ** -9, 2.0 ** -6, seed=1000 + rank, device=dev)
        qsrc = SyntheticCache([ps] * B, ps, H, 1.0, 1.0, seed=7, device=dev)
        cache.q_nope, cache.q_pe = qsrc.q_nope, qsrc.q_pe
        kv_len_local = local_len
    else:
        cache = SyntheticCache(request_lengths(kv_len, B, rank), ps, H, None, None, seed=rank, device=dev)
        kv_len_local = kv_len[1] if isinstance(kv_len, tuple) else kv_len
    kv_bytes = cache.kv_bytes
    dargs = cache.args(SM_SCALE)
    kw = dict(max_kv_len=kv_len_local, num_splits=args.num_splits, precision=precision)
    if seq and world > 1:
        merger = mdist.PartialMerger(B, H, dev)

        def decode_fn(*a, **k):
            return mdist.decode_sequence_sharded(*a, merger=merger, **k)
    else:
        decode_fn = mla.decode

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(warmup):
        out = decode_fn(*dargs, **kw)
    sync_all()
    lib = _lib.load()
    if sampler:
        sampler.mark("timed_begin")
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # Inputs larger than twice the L2 evict themselves between steps; smaller workloads get an L2 flush (a 256 MB
    # write) before every step, and each step is then timed with its own event pair so that the flush is not counted.
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if kv_bytes < (256 << 20) else None
    l2 = ("inputs larger than L2 (126 MB), no flush" if flush is None else
          "256 MB written between timed steps (inputs smaller than 2 x L2); each step timed by its own event pair")
    pairs = None if flush is None else [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                                        for _ in range(steps)]

    def timed_pass(fn):
        """K steps; returns (total ms over the steps, last output)."""
        if flush is None:
            ev0.record()
            for _ in range(steps):
                o = fn()
            ev1.record()
            sync_all()
            return ev0.elapsed_time(ev1), o
        for a, b in pairs:
            flush.zero_()
            a.record()
            o = fn()
            b.record()
        sync_all()
        return sum(a.elapsed_time(b) for a, b in pairs), o

    # Pass 1, the reported step time: the call as a user makes it (its kernels chained by programmatic dependent
    # launch). Pass 2, the same K steps with the library's own event pair around the decode kernel (the roofline's
    # duration): those events sit between the kernels and undo the chaining, so this pass is not the one reported.
    total_ms, out = timed_pass(lambda: decode_fn(*dargs, **kw))
    _lib.check(lib.nvfp4_mla_profile_begin(steps))
    timed_pass(lambda: decode_fn(*dargs, **kw))
    if sampler:
        sampler.mark("timed_end")
    kern_ms = (ctypes.c_float * steps)()
    n_k = lib.nvfp4_mla_profile_end(kern_ms, steps)
    if n_k < 0:
        raise RuntimeError(lib.nvfp4_mla_last_error().decode())
    res = {"workload": workload, "precision": precision, "B": B, "H": H, "kv_len": kv_len, "ps": ps, "seq": seq, "l2": l2,
           "steps": steps, "kv_bytes": kv_bytes}
    res["ms_step"] = max_over_ranks(total_ms / steps)
    # kernels per decode call: 2 (decode, merge of the partials), 3 when a schedule kernel runs in front (large batches)
    res["launches_per_decode"] = lib.nvfp4_mla_decode_launches(len(cache.kv_lens_list), H, kv_len_local, args.num_splits,
                                                               0 if precision == "bf16" else 1)
    if res["launches_per_decode"] < 0:
        raise RuntimeError(lib.nvfp4_mla_last_error().decode())
    res["kernel_ms"] = max_over_ranks(sum(kern_ms[:n_k]) / max(n_k, 1))
    if seq and world > 1:  # the local split-KV decode alone (no exchange, no merge): what the exchange adds on top
        local_ms, _ = timed_pass(lambda: mla.decode_partial(*dargs, into=(merger.o, merger.lse), **kw))  # same buffers as the full step
        res["local_decode_ms"] = max_over_ranks(local_ms / steps)
        merger.check()  # raises if a hand-shake of the timed steps gave up waiting for a rank
        res["merge"] = {"peer-signal": "peer reads: the merge kernel announces this GPU's record, waits for the others' "
                                       "announcements (flag words in symmetric memory) and loads their records over NVLink",
                        "peer-barrier": "peer reads: one barrier between the GPUs, then the merge kernel loads the other GPUs' "
                                        "records over NVLink",
                        "all-gather": "one NCCL all-gather of the packed records, then the merge kernel"}[merger.mode]
    if world > 1:
        t = torch.tensor([float(kv_bytes)], dtype=torch.float64, device=dev)
        dist.all_reduce(t)
        res["kv_bytes_all"] = float(t.item())
    else:
        res["kv_bytes_all"] = float(kv_bytes)
    status = mla.workspace_status()
    if status != 0:
        raise SystemExit(f"decode failed: device-side status {status}")
    res["parity_check"] = parity_check(mla, mdist, cache, dargs, kw, out, precision, seq, rank, world, dev)

    if want_e2e:
        # ---- end to end through the public API, per-step inputs from pinned host memory ------------------------
        # The step's inputs sit back to back in ONE pinned host buffer (256-byte aligned pieces) and cross in one copy;
        # the tensors the decode call gets are views of the device copy.
        srcs = (cache.q_nope, cache.q_pe, cache.page_table, cache.kv_lens)
        offs, total = [], 0
        for t in srcs:
            offs.append(total)
            total += (t.numel() * t.element_size() + 255) // 256 * 256
        host_buf = torch.empty(total, dtype=torch.uint8).pin_memory()
        dev_buf = torch.empty(total, dtype=torch.uint8, device=dev)

        def views(buf):
            return [buf[o:o + t.numel() * t.element_size()].view(t.dtype).view(t.shape) for o, t in zip(offs, srcs)]

        for h, t in zip(views(host_buf), srcs):
            h.copy_(t.cpu())
        devbuf = views(dev_buf)
        out_host = torch.empty(B, H, 512, dtype=torch.bfloat16).pin_memory()
        res["h2d"] = sum(t.numel() * t.element_size() for t in srcs)
        res["d2h"] = out_host.numel() * out_host.element_size()

        def e2e_step():
            dev_buf.copy_(host_buf, non_blocking=True)
            o = decode_fn(devbuf[0], devbuf[1], cache.ckv_cache, cache.ckv_sf_cache, cache.kpe_cache, devbuf[2], devbuf[3],
                          SM_SCALE, cache.ckv_scale, cache.kpe_scale, **kw)
            out_host.copy_(o, non_blocking=True)
            return o

        for _ in range(warmup):
            e2e_step()
        sync_all()
        total_ms, _ = timed_pass(e2e_step)
        res["e2e_ms"] = max_over_ranks(total_ms / steps)
    del cache, out, flush
    torch.cuda.empty_cache()
    return res


def reference_gpu_kernel(workload, precision, steps=20, warmup=3):
    """Same-box timing of the reference's own CUDA kernel (its `mma.sync` split-KV decode, nvfp4_mla/csrc/mla_decode.cu),
    called through its public `nvfp4_mla.decode` on the inputs the product arm gets. The unmodified package is taken
    from baseline/_ref (installed there with pip, not part of this repository's sources) and JIT-compiles its
    extension for the GPU it finds on first use. Opt-in (`--reference-gpu`): the build takes a minute or two."""
    import importlib.util
    import torch
    import nvfp4_mla_b200 as mla
    from nvfp4_mla_b200.testing import SM_SCALE, SyntheticCache
    init = pathlib.Path(__file__).resolve().parent / "baseline" / "_ref" / "nvfp4_mla" / "__init__.py"
    if not init.exists():
        return {"unavailable": "baseline/_ref holds no installed reference package"}
    try:
        spec = importlib.util.spec_from_file_location("nvfp4_mla_reference", init, submodule_search_locations=[str(init.parent)])
        ref = importlib.util.module_from_spec(spec)
        sys.modules["nvfp4_mla_reference"] = ref
        spec.loader.exec_module(ref)
        B, H, kv_len, ps, _ = WORKLOADS[workload]
        c = SyntheticCache(request_lengths(kv_len, B, 0), ps, H, None, None, seed=0, device="cuda")
        max_len = max(c.kv_lens_list)
        call = lambda: ref.decode(c.q_nope, c.q_pe, c.ckv_cache, c.ckv_sf_cache, c.kpe_cache, c.page_table, c.kv_lens, SM_SCALE,
                                  c.ckv_scale, c.kpe_scale, max_kv_len=max_len, precision=precision)
        t_build = time.time()
        out_ref = call()
        torch.cuda.synchronize()
        t_build = time.time() - t_build
        for _ in range(warmup):
            call()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            call()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        ours = mla.decode(*c.args(), max_kv_len=max_len, precision=precision)
        diff = (ours.float() - out_ref.float()).abs().max().item()
        kv_bytes = TOKEN_BYTES * sum(c.kv_lens_list)
        return {"kernel": "the reference's CUDA kernel (mma.sync, nvfp4_mla/csrc/mla_decode.cu) through nvfp4_mla.decode, built on this box",
                "precision": precision, "ms_per_step": ms, "kv_tbps": kv_bytes / (ms * 1e-3) / 1e12, "steps": steps,
                "first_call_s": t_build, "max_abs_vs_this_library": diff}
    except Exception as e:  # a missing compiler, an unsupported GPU: report, do not fail the product arm
        return {"unavailable": f"{type(e).__name__}: {str(e)[:300]}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2_h16_b64_64k", choices=sorted(WORKLOADS) + ["writer_1m", "dequant_1m"])
    ap.add_argument("--num-splits", type=int, default=0)
    ap.add_argument("--precision", default=None, choices=["bf16", "fp8"], help="override the workload's precision mode")
    ap.add_argument("--cpu-sample-requests", type=int, default=16)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--reference-gpu", action="store_true",
                    help="also time the reference's own CUDA kernel from baseline/_ref on this GPU (one GPU only)")
    ap.add_argument("--no-seq-sharded", action="store_true",
                    help="skip the sequence-sharded long-context pass that the default workload appends")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.workload == "writer_1m":
        return bench_writer(args)
    if args.workload == "dequant_1m":
        return bench_dequant(args)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    B, H, kv_len, ps, precision = WORKLOADS[args.workload]
    precision = args.precision or precision
    seq = args.workload in SEQUENCE_SHARDED
    config = {"workload": f"{args.workload}: B={B} per GPU, H={H}, kv_len={kv_len}, page_size={ps}, precision={precision}, "
                          f"seeded N(0,1) latent KV quantised to NVFP4 (calibrated global scales), shuffled page table",
              "parallelism": f"batch-sharded dp{world}, no collective", "num_splits": args.num_splits,
              "l2": "inputs larger than L2 (126 MB), no flush" if TOKEN_BYTES * B * (kv_len if isinstance(kv_len, int) else kv_len[0]) >= (256 << 20)
                    else "256 MB written between timed steps (inputs smaller than 2 x L2); each step timed by its own event pair",
              "baseline": "reference SM100 tcgen05 kernel v3, 0.309 ms = 4.77 TB/s (published, B200)"}
    if seq:
        config["parallelism"] = f"sequence-sharded over {world} GPU(s): local split-KV decode, all-gather of (o, lse), merge"
        config["workload"] = config["workload"].replace(f"B={B} per GPU", f"B={B} in total (queries replicated, each rank holds 1/{world} of every context)")

    if args.impl == "reference":
        # The reference's CPU path on this box's host cores; rank 0 alone works.
        if rank != 0:
            return
        from nvfp4_mla_b200.testing import SyntheticCache
        n = args.cpu_sample_requests
        cache = SyntheticCache(request_lengths(kv_len, B, 0)[:n], ps, H, None, None, seed=0, device="cpu")
        for _ in range(min(args.warmup, 1)):
            cpu_reference_sample(cache, 1)
        times, budget_s = [], 90.0  # the CPU arm stops after about a minute and a half, whatever --steps asks for
        for _ in range(args.steps):
            dt, nbytes, threads, kind = cpu_reference_sample(cache, n)
            times.append(dt)
            if sum(times) + dt > budget_s:
                break
        t = sum(times) / len(times)
        val = nbytes / t / 1e12
        sample = f"{min(n, B)} of {B} requests per step ({nbytes // TOKEN_BYTES} tokens), {CPU_ARM_TEXT[kind]}"
        print(json.dumps({
            "impl": "reference", "metric": "nvfp4_mla_decode_kv_bandwidth", "value": val, "unit": "TB/s",
            "n_gpus": args.gpus, "steps": len(times), "steps_requested": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config,
            "cpu_baseline": {"value": val, "unit": "TB/s", "cores": threads, "kind": kind, "sample": sample},
            "e2e": {"value": val, "unit": "TB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    sampler = ClockSampler(local_rank) if rank == 0 else None  # started early: nvidia-smi takes a while to produce samples
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if sampler:
        sampler.mark("load_begin")

    m = measure(args, args.workload, precision, args.steps, args.warmup, rank, world, dev, sampler)
    clocks = sampler.stop() if sampler else None
    # The default (headline) run also times the one path that has a collective: the long-context configuration with
    # every request's pages cut over the ranks, local split-KV decode, all-gather of (o, lse) and merge.
    seq_extra = None
    if args.workload == "c2_h16_b64_64k" and not args.no_seq_sharded and args.precision is None:
        sm = measure(args, "c4_h128_b2_1m_seq", "bf16", max(3, min(args.steps, 100)), args.warmup, rank, world, dev, None, want_e2e=False)
        seq_extra = {"workload": "c4_h128_b2_1m_seq: B=2, H=128, kv_len=1048576 in total, bf16 mode, strong scaling",
                     "n_gpus": world, "steps": sm["steps"], "ms_per_step": sm["ms_step"], "decode_ms": sm["kernel_ms"],
                     "exchange_merge_us": (sm["ms_step"] - sm["local_decode_ms"]) * 1e3 if "local_decode_ms" in sm else 0.0,
                     "kv_tbps": sm["kv_bytes_all"] / (sm["ms_step"] * 1e-3) / 1e12, "parity_check": sm["parity_check"]}
        if "merge" in sm:
            seq_extra["merge"] = sm["merge"]

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak()
    kv_bytes, kernel_ms, ms_step = m["kv_bytes"], m["kernel_ms"], m["ms_step"]
    achieved = kv_bytes / (kernel_ms * 1e-3) / 1e9
    tokens = kv_bytes // TOKEN_BYTES
    kernel_name = ("mla_decode_hm_kernel" if (H % 128 == 0 and precision == "fp8") else
                   "mla_decode_vt_kernel" if precision == "bf16" else "mla_decode_kernel")
    if H >= 128:  # 2176 flop per token and head: the tensor pipe is the bound, the HBM figure becomes secondary
        tpeak, tkind = measured_tensor_peak(precision)
        tflops = 2176.0 * H * tokens / (kernel_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": tflops, "peak": tpeak, "unit": "TFLOP/s", "frac": tflops / tpeak,
                    "peak_kind": tkind, "kernel": kernel_name, "kernel_ms": kernel_ms,
                    "algorithmic_flops_per_launch": 2176.0 * H * tokens, "hbm_gbs": achieved, "traffic": None}
    else:
        per_token = NCU_TRAFFIC_BYTES_PER_TOKEN.get(precision)
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "peak_kind": f"of {peak_kind}", "kernel": kernel_name, "kernel_ms": kernel_ms,
                    "algorithmic_bytes_per_launch": kv_bytes,
                    "traffic": per_token * tokens if per_token else None,
                    "traffic_kind": f"ncu capture of h16_b8_64k ({precision} mode, {per_token} B per token) scaled by tokens"
                                    if per_token else None}
    value = m["kv_bytes_all"] / (ms_step * 1e-3) / 1e12
    config["l2"] = m["l2"]
    line = {
        "metric": "nvfp4_mla_decode_kv_bandwidth", "value": value, "unit": "TB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if seq else "weak",
        "vs_baseline": (value / world / BASELINE_TBPS[args.workload]) if args.workload in BASELINE_TBPS and world == 1 else None,
        "dtype": "QK^T: block-scaled e2m1 K (exact) x 4-term e2m1 query; PV: f16; f32 accumulate" if precision == "bf16" else "e4m3 operands, f32 accumulate",
        "data": "synthetic", "config": config,
        "decode_us": ms_step * 1e3, "frac_of_8tbps": value / world / 8.0,
        "e2e": {"value": m["kv_bytes_all"] / (m["e2e_ms"] * 1e-3) / 1e12, "unit": "TB/s", "ms_per_step": m["e2e_ms"],
                "h2d_bytes_per_step": m["h2d"], "d2h_bytes_per_step": m["d2h"]},
        "gpu_launches": (m["launches_per_decode"] + (1 if seq and world > 1 else 0)) * args.steps,
        "roofline": roofline,
        "parity_check": m["parity_check"],
        "clocks": clocks,
    }
    if seq and "local_decode_ms" in m:
        line["exchange_merge_us"] = (ms_step - m["local_decode_ms"]) * 1e3
        line["merge"] = m.get("merge")
    if seq_extra:
        line["seq_sharded"] = seq_extra
    if args.reference_gpu and world == 1:
        line["reference_gpu"] = reference_gpu_kernel(args.workload, precision)
    if world == 1 and not args.no_cpu_baseline:
        from nvfp4_mla_b200.testing import SyntheticCache
        n = args.cpu_sample_requests
        cache = SyntheticCache(request_lengths(kv_len, B, 0)[:n], ps, H, None, None, seed=0, device="cpu")
        dt, nbytes, threads, kind = cpu_reference_sample(cache, n)  # first pass: also sizes the timed one
        reps = max(1, min(8, int(10.0 / max(dt, 1e-3))))           # about ten seconds of CPU work, at most 8 passes
        if reps > 1:
            dt, nbytes, threads, kind = cpu_reference_sample(cache, n, repeats=reps)
        line["cpu_baseline"] = {"value": nbytes / dt / 1e12, "unit": "TB/s", "cores": threads, "kind": kind,
                                "seconds": dt * reps,
                                "sample": f"{min(n, B)} of {B} requests ({nbytes // TOKEN_BYTES} tokens) x {reps} pass(es), {CPU_ARM_TEXT[kind]}"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    bad = [k for k, pc in (("headline", line["parity_check"]), ("seq_sharded", (seq_extra or {}).get("parity_check"))) if pc and not pc["ok"]]
    if bad:
        raise SystemExit(f"parity check failed: {bad}")


if __name__ == "__main__":
    main()
