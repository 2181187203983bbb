"""Benchmark of the hot path: NVFP4 paged MLA decode at the headline shape (H=16, B=64, 64K-token contexts).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

One "step" is one decode call over the whole batch. With N > 1 (launched by torchrun, one rank per GPU) the batch is
sharded data-parallel: every rank holds its own B requests and their pages, nothing is exchanged, and the reported
value is the bytes all ranks streamed divided by the slowest rank's time (weak scaling). Rank 0 prints one JSON line.

  value      KV-cache bandwidth, 352 bytes per cached token / device time per step (CUDA events on the launching
             stream, inputs resident in HBM; the cache is far larger than L2, so no flush is needed)
  e2e        the same through the Python API with the per-step inputs (queries, page table, lengths) coming from
             pinned host memory and the output copied back to the host inside the timed region. The KV cache itself
             is device-resident state written by earlier steps of a serving engine, not a per-step input.
  roofline   the decode kernel alone (timed by the library's own event pair around it) against the measured HBM peak
  cpu_baseline / --impl reference
             the reference's CPU path (dequantize, then fp32 attention) as restated by oracle/mla_oracle.py, timed on
             this box's host cores over a bounded sample of the same workload
"""
import argparse
import ctypes
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
    "c2_h16_b64_64k": (64, 16, 65536, 64, "bf16"),   # BASELINE config 2, the shape the metric is quoted on
    "c1_h16_b32_8k": (32, 16, 8192, 64, "bf16"),     # BASELINE config 1
    "h16_b64_16k": (64, 16, 16384, 64, "bf16"),
    "h16_b8_64k": (8, 16, 65536, 64, "bf16"),        # small case for ncu captures (185 MB of KV, still larger than L2)
    "h128_b64_16k": (64, 128, 16384, 64, "bf16"),
    "c4_h128_b2_1m_seq": (2, 128, 1048576, 64, "bf16"),  # BASELINE config 4: sequence-sharded, strong scaling
}
SEQUENCE_SHARDED = {"c4_h128_b2_1m_seq"}
TOKEN_BYTES = 352
# Published by the reference for this exact shape on B200: its SM100 tcgen05 kernel, 0.309 ms = 4.77 TB/s
# (README.md:194 and benchmarks/results/b200.csv:108 of the reference project).
BASELINE_TBPS = {"c2_h16_b64_64k": 4.77}
# DRAM bytes (read + write) per cached token of the decode kernel, from the committed ncu capture of a smaller case
# (profiles/decode_kernel_h16_b8_64k_ncu_full.md: 208.6 MB for 524 288 tokens); traffic grows with the token count, so the
# benchmark scales it to its own workload.
NCU_TRAFFIC_BYTES_PER_TOKEN = 398
KERNELS_PER_DECODE = 3  # schedule, decode, combine


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.thread.join(timeout=2)
        clocks, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                clocks.append(float(r[0])), (mx := float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v == "Active":
                    reasons.add(name)
        busy = [c for c in clocks if mx and c > 0.5 * mx] or clocks
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(clocks)}


def cpu_reference_sample(cache, n_requests, repeats=1):
    """Times the oracle (dequantize + fp32 attention on host cores) on `n_requests` requests of the workload.

    Returns (seconds per pass, KV bytes per pass, threads). The sample's pages are copied to the host first; the
    copy is not timed."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import numpy as np
    import torch
    import mla_oracle as O
    ps = cache.page_size
    reqs = list(range(min(n_requests, len(cache.kv_lens_list))))
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
    nbytes = TOKEN_BYTES * sum(cache.kv_lens_list[b] for b in reqs)
    return dt, nbytes, os.cpu_count()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2_h16_b64_64k", choices=sorted(WORKLOADS))
    ap.add_argument("--num-splits", type=int, default=0)
    ap.add_argument("--precision", default=None, choices=["bf16", "fp8"], help="override the workload's precision mode")
    ap.add_argument("--cpu-sample-requests", type=int, default=4)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    B, H, kv_len, ps, precision = WORKLOADS[args.workload]
    precision = args.precision or precision
    config = {"workload": f"{args.workload}: B={B} per GPU, H={H}, kv_len={kv_len}, page_size={ps}, precision={precision}, "
                          f"seeded N(0,1) latent KV quantised to NVFP4 (calibrated global scales), shuffled page table",
              "parallelism": f"batch-sharded dp{world}, no collective", "num_splits": args.num_splits,
              "l2": "inputs larger than L2 (1.48 GB per GPU), no flush",
              "baseline": "reference SM100 tcgen05 kernel v3, 0.309 ms = 4.77 TB/s (published, B200)"}

    if args.impl == "reference":
        # The reference's CPU path on this box's host cores; rank 0 alone works.
        if rank != 0:
            return
        from nvfp4_mla_b200.testing import SyntheticCache
        n = args.cpu_sample_requests
        cache = SyntheticCache([kv_len] * n, ps, H, None, None, seed=0, device="cpu")
        for _ in range(min(args.warmup, 1)):
            cpu_reference_sample(cache, 1)
        times = []
        for _ in range(args.steps):
            dt, nbytes, threads = cpu_reference_sample(cache, n)
            times.append(dt)
        t = sum(times) / len(times)
        val = nbytes / t / 1e12
        sample = f"{n} of {B} requests per step ({n * kv_len} tokens), numpy port of the reference torch path"
        print(json.dumps({
            "impl": "reference", "metric": "nvfp4_mla_decode_kv_bandwidth", "value": val, "unit": "TB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config,
            "cpu_baseline": {"value": val, "unit": "TB/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "TB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    import nvfp4_mla_b200 as mla
    from nvfp4_mla_b200 import _lib
    from nvfp4_mla_b200.testing import SM_SCALE, SyntheticCache

    seq = args.workload in SEQUENCE_SHARDED
    if seq:
        # every rank holds a contiguous 1/world slice of each request's pages (generated directly as the local slice:
        # rank r's tokens are a seeded stream of their own), queries replicated
        from nvfp4_mla_b200 import dist as mdist
        local_len = mdist.shard_sequence(kv_len, ps, world)[rank][2]
        cache = SyntheticCache([local_len] * B, ps, H, 2.0 ** -9, 2.0 ** -6, seed=1000 + rank, device=dev)
        qsrc = SyntheticCache([ps] * B, ps, H, 1.0, 1.0, seed=7, device=dev)
        cache.q_nope, cache.q_pe = qsrc.q_nope, qsrc.q_pe
        config["parallelism"] = f"sequence-sharded over {world} GPU(s): local split-KV decode, all-gather of (o, lse), merge"
        kv_len_local = local_len
    else:
        cache = SyntheticCache([kv_len] * B, ps, H, None, None, seed=rank, device=dev)
        kv_len_local = kv_len
    kv_bytes = cache.kv_bytes
    dargs = cache.args(SM_SCALE)
    kw = dict(max_kv_len=kv_len_local, num_splits=args.num_splits, precision=precision)
    if seq:
        def decode_fn(*a, **k):
            return mdist.decode_sequence_sharded(*a, **k) if world > 1 else mla.decode(*a, **k)
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

    # ---- device-resident timing -------------------------------------------------------------------------------
    for _ in range(args.warmup):
        out = decode_fn(*dargs, **kw)
    sync_all()
    lib = _lib.load()
    _lib.check(lib.nvfp4_mla_profile_begin(args.steps))
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        out = decode_fn(*dargs, **kw)
    ev1.record()
    sync_all()
    clocks = sampler.stop() if sampler else None
    kern_ms = (ctypes.c_float * args.steps)()
    n_k = lib.nvfp4_mla_profile_end(kern_ms, args.steps)
    if n_k < 0:
        raise RuntimeError(lib.nvfp4_mla_last_error().decode())
    ms_step = max_over_ranks(ev0.elapsed_time(ev1) / args.steps)
    kernel_ms = max_over_ranks(sum(kern_ms[:n_k]) / max(n_k, 1))
    kv_bytes_all = kv_bytes
    if world > 1:
        t = torch.tensor([float(kv_bytes)], dtype=torch.float64, device=dev)
        dist.all_reduce(t)
        kv_bytes_all = float(t.item())
    else:
        kv_bytes_all = float(kv_bytes)
    status = mla.workspace_status()
    if status != 0 or bool(out.isnan().any()):
        raise SystemExit(f"decode failed: status {status}")

    # ---- end to end through the public API, per-step inputs from pinned host memory ---------------------------
    host = [t.cpu().pin_memory() for t in (cache.q_nope, cache.q_pe, cache.page_table, cache.kv_lens)]
    devbuf = [torch.empty_like(t, device=dev) for t in host]
    out_host = torch.empty(B, H, 512, dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = out_host.numel() * out_host.element_size()

    def e2e_step():
        for d, h in zip(devbuf, host):
            d.copy_(h, non_blocking=True)
        o = decode_fn(devbuf[0], devbuf[1], cache.ckv_cache, cache.ckv_sf_cache, cache.kpe_cache, devbuf[2], devbuf[3],
                      SM_SCALE, cache.ckv_scale, cache.kpe_scale, **kw)
        out_host.copy_(o, non_blocking=True)

    for _ in range(args.warmup):
        e2e_step()
    sync_all()
    ev0.record()
    for _ in range(args.steps):
        e2e_step()
    ev1.record()
    sync_all()
    e2e_ms = max_over_ranks(ev0.elapsed_time(ev1) / args.steps)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak()
    achieved = kv_bytes / (kernel_ms * 1e-3) / 1e9
    value = kv_bytes_all / (ms_step * 1e-3) / 1e12
    line = {
        "metric": "nvfp4_mla_decode_kv_bandwidth", "value": value, "unit": "TB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if seq else "weak",
        "vs_baseline": (value / world / BASELINE_TBPS[args.workload]) if args.workload in BASELINE_TBPS and world == 1 else None,
        "dtype": "f16 operands, f32 accumulate" if precision == "bf16" else "e4m3 operands, f32 accumulate",
        "data": "synthetic", "config": config,
        "decode_us": ms_step * 1e3, "frac_of_8tbps": value / world / 8.0,
        "e2e": {"value": kv_bytes_all / (e2e_ms * 1e-3) / 1e12, "unit": "TB/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": (KERNELS_PER_DECODE + (1 if seq and world > 1 else 0)) * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}", "kernel": "mla_decode_kernel", "kernel_ms": kernel_ms,
                     "algorithmic_bytes_per_launch": kv_bytes,
                     "traffic": (NCU_TRAFFIC_BYTES_PER_TOKEN * kv_bytes // TOKEN_BYTES) if NCU_TRAFFIC_BYTES_PER_TOKEN else None},
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu_baseline:
        n = args.cpu_sample_requests
        dt, nbytes, threads = cpu_reference_sample(cache, n)
        line["cpu_baseline"] = {"value": nbytes / dt / 1e12, "unit": "TB/s", "cores": threads, "kind": "port",
                                "seconds": dt,
                                "sample": f"{n} of {B} requests ({n * kv_len} tokens), numpy port of the reference torch path"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
