"""Seeded synthetic NVFP4 MLA caches for tests and benchmarks, plus torch reference helpers.

Plays the role of the reference's ``nvfp4_mla/testing.py`` (``RandomCache``, ``dequantize``, ``attention``,
``rel_l2``; nvfp4_mla/testing.py:15-125) without FlashInfer: the cache is written here by a torch restatement of
the NVFP4 writer (one E4M3 scale per 16 channels = amax / 6 in units of ``ckv_scale``; E2M1 codes rounded to
nearest, ties to even; kpe as E4M3 of x / ``kpe_scale``). Like the reference's generator, physical pages are
shuffled by a seeded permutation and every unused slot holds random bytes (NaN scales included), so a kernel that
reads past ``kv_lens`` or ignores the page table produces NaN or garbage.

Everything here is torch and device-agnostic: small cases are generated on the CPU (bit-reproducible from the seed)
and moved to the GPU, benchmark-sized caches are generated on the GPU request by request.
"""
import math

import torch

CKV, KPE = 512, 64
TOKEN_BYTES = CKV // 2 + CKV // 16 + KPE  # 352 bytes of cache per token
SM_SCALE = (128 + KPE) ** -0.5            # DeepSeek: qk_nope_head_dim 128 + qk_rope_head_dim 64
_E2M1 = [0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6]


def e2m1_codes(y):
    """Nearest E2M1 code (0..15) of fp32 ``y``: ties go to the even mantissa, magnitudes above 6 saturate."""
    a = y.abs()
    code = (a > 0.25).to(torch.uint8) + (a >= 0.75) + (a > 1.25) + (a >= 1.75) + (a > 2.5) + (a >= 3.5) + (a > 5.0)
    return code.to(torch.uint8) | (torch.signbit(y).to(torch.uint8) << 3)


def quantize_ckv(x, ckv_scale):
    """``[n, 512]`` float -> (``[n, 256]`` uint8 packed E2M1, ``[n, 32]`` float8_e4m3fn block scales)."""
    x = x.float().reshape(-1, CKV // 16, 16)
    amax = x.abs().amax(-1)
    sf8 = (amax / 6.0 / ckv_scale).clamp(max=448.0).to(torch.float8_e4m3fn)
    sf = sf8.float() * ckv_scale
    y = torch.where(sf[..., None] > 0, x / sf[..., None], torch.zeros_like(x))
    codes = e2m1_codes(y).reshape(-1, CKV)
    return codes[:, 0::2] | (codes[:, 1::2] << 4), sf8


def quantize_kpe(x, kpe_scale):
    return (x.float() / kpe_scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)


def dequantize(ckv_cache, ckv_sf_cache, kpe_cache, ckv_scale=1.0, kpe_scale=1.0):
    """fp32 ``[pages, page_size, 512]``, ``[pages, page_size, 64]``: ``e2m1 * block_scale * ckv_scale`` evaluated
    left to right, the multiply order the kernels' dequantize reproduces bit for bit."""
    lut = torch.tensor(_E2M1, device=ckv_cache.device)
    codes = torch.stack([ckv_cache & 15, ckv_cache >> 4], -1).flatten(-2).long()  # low nibble = even channel
    ckv = lut[codes] * ckv_sf_cache.float().repeat_interleave(16, -1) * ckv_scale
    return ckv, kpe_cache.float() * kpe_scale


def attention(q_nope, q_pe, ckv, kpe, page_table, kv_lens, sm_scale=SM_SCALE, return_lse=False):
    """fp32 absorbed-MLA decode (q_len = 1) over a dequantized cache, one request at a time.

    ``out[b, h] = softmax(q . [ckv | kpe]^T * sm_scale) @ ckv``; with ``return_lse`` also the natural-log
    log-sum-exp ``[batch, heads]``. Runs on whatever device the tensors are on.
    """
    ps, out, lse = ckv.shape[1], [], []
    for b, L in enumerate(kv_lens.tolist()):
        pages = page_table[b, :math.ceil(L / ps)].long()
        kc, kp = ckv[pages].reshape(-1, CKV)[:L].float(), kpe[pages].reshape(-1, KPE)[:L].float()
        s = (q_nope[b].float() @ kc.T + q_pe[b].float() @ kp.T) * sm_scale
        out.append(s.softmax(-1) @ kc)
        lse.append(torch.logsumexp(s, -1))
    return (torch.stack(out), torch.stack(lse)) if return_lse else torch.stack(out)


def attention_paged_nvfp4(q_nope, q_pe, ckv_cache, ckv_sf_cache, kpe_cache, page_table, kv_lens, sm_scale,
                          ckv_scale=1.0, kpe_scale=1.0, chunk_pages=256, requests=None):
    """The same dequantize-then-attention, streamed: dequantizes ``chunk_pages`` pages of one request at a time and
    merges with a running (max, sum, acc), so a 64K-token request never materialises more than a chunk in fp32.

    Used as the large-shape check on the GPU. Returns (out fp32, natural-log lse) for ``requests`` (default all).
    """
    ps = ckv_cache.shape[1]
    dev = q_nope.device
    reqs = list(range(q_nope.shape[0])) if requests is None else list(requests)
    H = q_nope.shape[1]
    outs, lses = [], []
    lens = kv_lens.tolist()
    for b in reqs:
        L = lens[b]
        m = torch.full((H, 1), -float("inf"), device=dev)
        l = torch.zeros(H, 1, device=dev)
        acc = torch.zeros(H, CKV, device=dev)
        n_pages = math.ceil(L / ps)
        for p0 in range(0, n_pages, chunk_pages):
            pages = page_table[b, p0:min(p0 + chunk_pages, n_pages)].long()
            kc, kp = dequantize(ckv_cache[pages], ckv_sf_cache[pages], kpe_cache[pages], ckv_scale, kpe_scale)
            n = min(L - p0 * ps, pages.numel() * ps)
            kc, kp = kc.reshape(-1, CKV)[:n], kp.reshape(-1, KPE)[:n]
            s = (q_nope[b].float() @ kc.T + q_pe[b].float() @ kp.T) * sm_scale
            m_new = torch.maximum(m, s.amax(-1, keepdim=True))
            c = torch.exp(m - m_new)
            p = torch.exp(s - m_new)
            l = l * c + p.sum(-1, keepdim=True)
            acc = acc * c + p @ kc
            m = m_new
        outs.append(acc / l)
        lses.append((m + torch.log(l))[:, 0])
    return torch.stack(outs), torch.stack(lses)


def rel_l2(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


class SyntheticCache:
    """Random q and random latent KV written into an NVFP4 paged cache (and optionally kept in BF16 as well).

    Args:
        kv_lens: tokens per request.
        page_size: power of two.
        heads: query heads.
        ckv_scale, kpe_scale: global scales; ``None`` calibrates them as a serving engine would
            (``amax / (6 * 448)`` and ``amax / 448``), which drives block scales to the E4M3 maximum.
        seed: everything (q, kv, page permutation, junk bytes) derives from it.
        device: where the tensors are generated. CPU generation is bit-reproducible; move with ``.to()``.
        keep_bf16: also keep the unquantized BF16 cache (``ckv_bf16`` / ``kpe_bf16``), for error baselines.
        extra_pages: unused physical pages appended to the pool (junk-filled).
    """

    def __init__(self, kv_lens, page_size, heads, ckv_scale=1.0, kpe_scale=1.0, seed=0, device="cpu",
                 keep_bf16=False, extra_pages=0):
        assert page_size & (page_size - 1) == 0, "page_size must be a power of two"
        dev = torch.device(device)
        g = torch.Generator(device=dev).manual_seed(seed)
        B, ps = len(kv_lens), page_size
        n_pages = [math.ceil(L / ps) for L in kv_lens]
        P = max(sum(n_pages) + extra_pages, 1)
        self.kv_lens_list = list(kv_lens)
        self.kv_lens = torch.tensor(kv_lens, dtype=torch.int32, device=dev)
        self.page_size, self.heads = ps, heads

        perm = torch.randperm(P, generator=g, device=dev).int()
        self.page_table = torch.zeros(B, max(max(n_pages), 1), dtype=torch.int32, device=dev)
        start = 0
        for b in range(B):
            self.page_table[b, :n_pages[b]] = perm[start:start + n_pages[b]]
            start += n_pages[b]

        rn = lambda *s: torch.randn(*s, generator=g, device=dev, dtype=torch.float32).bfloat16()
        self.q_nope, self.q_pe = rn(B, heads, CKV), rn(B, heads, KPE)

        junk = lambda n: torch.randint(0, 256, (P, ps, n), generator=g, device=dev, dtype=torch.uint8)
        self.ckv_cache = junk(CKV // 2)
        self.ckv_sf_cache = junk(CKV // 16).view(torch.float8_e4m3fn)
        self.kpe_cache = junk(KPE).view(torch.float8_e4m3fn)
        if keep_bf16:
            self.ckv_bf16 = torch.zeros(P, ps, CKV, dtype=torch.bfloat16, device=dev)
            self.kpe_bf16 = torch.zeros(P, ps, KPE, dtype=torch.bfloat16, device=dev)

        # per-request generators so that a calibration pass can replay exactly the same values
        seeds = [seed * 1000003 + 17 * b + 1 for b in range(B)]

        def kv_of(b):
            gb = torch.Generator(device=dev).manual_seed(seeds[b])
            L = kv_lens[b]
            ckv = torch.randn(L, CKV, generator=gb, device=dev, dtype=torch.float32).bfloat16()
            kpe = torch.randn(L, KPE, generator=gb, device=dev, dtype=torch.float32).bfloat16()
            return ckv, kpe

        if ckv_scale is None or kpe_scale is None:
            amax_c = amax_k = 0.0
            for b in range(B):
                if kv_lens[b] == 0:
                    continue
                ckv, kpe = kv_of(b)
                amax_c, amax_k = max(amax_c, ckv.abs().max().item()), max(amax_k, kpe.abs().max().item())
            ckv_scale = (amax_c / (6 * 448)) if ckv_scale is None else ckv_scale
            kpe_scale = (amax_k / 448) if kpe_scale is None else kpe_scale
        self.ckv_scale, self.kpe_scale = float(ckv_scale), float(kpe_scale)

        flat = lambda t: t.view(P * ps, t.shape[-1])
        for b in range(B):
            L = kv_lens[b]
            if L == 0:
                continue
            ckv, kpe = kv_of(b)
            t = torch.arange(L, device=dev)
            slots = self.page_table[b, (t // ps)].long() * ps + (t % ps)
            packed, sf8 = quantize_ckv(ckv, self.ckv_scale)
            flat(self.ckv_cache)[slots] = packed
            flat(self.ckv_sf_cache.view(torch.uint8))[slots] = sf8.view(torch.uint8)
            flat(self.kpe_cache.view(torch.uint8))[slots] = quantize_kpe(kpe, self.kpe_scale).view(torch.uint8)
            if keep_bf16:
                flat(self.ckv_bf16)[slots] = ckv
                flat(self.kpe_bf16)[slots] = kpe

    def to(self, device):
        for k, v in list(vars(self).items()):
            if isinstance(v, torch.Tensor):
                setattr(self, k, v.to(device))
        return self

    @property
    def max_kv_len(self):
        return max(self.kv_lens_list) if self.kv_lens_list else 0

    @property
    def kv_bytes(self):
        """Algorithmic bytes of one decode: 352 per token in use."""
        return TOKEN_BYTES * sum(self.kv_lens_list)

    def args(self, sm_scale=SM_SCALE):
        """Positional arguments of ``decode``."""
        return (self.q_nope, self.q_pe, self.ckv_cache, self.ckv_sf_cache, self.kpe_cache, self.page_table,
                self.kv_lens, sm_scale, self.ckv_scale, self.kpe_scale)

    def dequantize(self):
        return dequantize(self.ckv_cache, self.ckv_sf_cache, self.kpe_cache, self.ckv_scale, self.kpe_scale)

    def reference(self, sm_scale=SM_SCALE, return_lse=False):
        """fp32 attention over the dequantized NVFP4 cache: what the kernel should produce."""
        return attention(self.q_nope, self.q_pe, *self.dequantize(), self.page_table, self.kv_lens, sm_scale,
                         return_lse)

    def reference_bf16(self, sm_scale=SM_SCALE):
        """fp32 attention over the unquantized BF16 cache: the quantization-error baseline."""
        return attention(self.q_nope, self.q_pe, self.ckv_bf16, self.kpe_bf16, self.page_table, self.kv_lens,
                         sm_scale)


RandomCache = SyntheticCache  # the reference's name for this helper
