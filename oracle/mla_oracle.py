"""CPU oracle for NVFP4 paged MLA decode. TEST INFRASTRUCTURE ONLY.

This module restates, in plain numpy, the reference project's torch "dequantize, then fp32 attention" path and
the cache format it reads. It exists to check the CUDA kernels; nothing in the shipped package may import it
(only tests/, the smoke check and the benchmark's cpu_baseline / reference legs do).

What it follows in the reference (paths relative to the reference project root):
  * E2M1 code table and nibble order (low nibble = even channel): nvfp4_mla/testing.py:12, :76
  * dequantize(): ``lut[code] * block_scale * ckv_scale`` evaluated left to right in fp32, and
    ``kpe = fp8 * kpe_scale``: nvfp4_mla/testing.py:73-78 (same multiply order as the CUDA helper at
    nvfp4_mla/csrc/mla_decode.cu:44-63)
  * attention(): per request, pages = page_table[b, :ceil(L / page_size)], fp32
    ``softmax((q_nope @ ckv^T + q_pe @ kpe^T) * sm_scale) @ ckv``: nvfp4_mla/testing.py:81-89
  * split-KV partial / merge contract (o normalised by its own l, lse = m + log2(l) in log2 units, empty split
    lse = -inf with weight 0): nvfp4_mla/csrc/mla_decode.cu:478-492 and :933-966
  * fp8-mode arithmetic (per-row E4M3 query with 448 / amax, K and V rounded as e4m3((e2m1 * sf) / 8), E4M3 P):
    nvfp4_mla/csrc/mla_decode.cu:192-220, :425-457, :762-808

The cache WRITER is not part of the reference repository (it is FlashInfer's
``nvfp4_quantize_append_paged_mla_kv_cache``, flashinfer-python >= 0.7.0, pinned by the reference's
pyproject.toml:17). ``quantize_ckv`` / ``quantize_kpe`` restate its published format (one E4M3 scale per 16
channels equal to amax / 6 in units of ckv_scale, E2M1 codes rounded to nearest, ties to even; kpe as E4M3 of
x / kpe_scale). The reference's tests pin the writer only indirectly, so quantizer parity is UNPINNED (the E2M1
tie rule is an assumption). Decode parity does not depend on it: decode is defined on whatever bytes the cache
holds.

Pinning of the decode oracle itself: tests/golden/ holds outputs of the reference's own
nvfp4_mla.testing.dequantize / attention, produced by tests/golden/make_golden.py; tests/test_oracle.py checks
this module against them (dequantize bitwise, attention to 2e-6).
"""
import math

import numpy as np

CKV, KPE = 512, 64
TOKEN_BYTES = CKV // 2 + CKV // 16 + KPE  # 352
SM_SCALE = (128 + KPE) ** -0.5
LOG2E = 1.4426950408889634

E2M1_LUT = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)


def _e4m3_table():
    t = np.empty(256, dtype=np.float32)
    for b in range(256):
        s, e, m = b >> 7, (b >> 3) & 15, b & 7
        if e == 15 and m == 7:
            v = float("nan")
        elif e == 0:
            v = m * 2.0 ** -9
        else:
            v = (1 + m / 8.0) * 2.0 ** (e - 7)
        t[b] = -v if s else v
    return t


E4M3_LUT = _e4m3_table()


def e4m3_decode(b):
    """uint8 E4M3 (fn variant: no inf, 0x7f / 0xff = NaN) -> float32."""
    return E4M3_LUT[np.asarray(b, dtype=np.uint8)]


def e4m3_encode(x):
    """float32 -> uint8 E4M3, round to nearest even, saturating to +-448 (NaN -> 0x7f)."""
    x = np.asarray(x, dtype=np.float32)
    a = np.minimum(np.abs(x).astype(np.float64), 448.0)
    with np.errstate(divide="ignore", invalid="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.clip(e, -6, 8)                      # exponent of the binade; below 2^-6 the grid is the subnormal one
    q = np.rint(a / 2.0 ** (e - 3)) * 2.0 ** (e - 3)  # np.rint rounds half to even; spacing 2^(e-3)
    q = np.minimum(q, 448.0)
    # encode q (exactly representable) into bits
    with np.errstate(divide="ignore", invalid="ignore"):
        eq = np.floor(np.log2(np.where(q > 0, q, 1.0)))
    sub = q < 2.0 ** -6
    mant = np.where(sub, q / 2.0 ** -9, (q / 2.0 ** eq - 1.0) * 8.0)
    expo = np.where(sub, 0, eq + 7)
    bits = (expo.astype(np.int64) << 3) | np.rint(mant).astype(np.int64)
    bits = np.where(q == 0, 0, bits)
    bits |= (np.signbit(x).astype(np.int64) << 7)
    bits = np.where(np.isnan(x), 0x7F, bits)
    return bits.astype(np.uint8)


def e2m1_encode(x):
    """float32 -> E2M1 code 0..15, round to nearest, ties to even mantissa, saturating at 6."""
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x)
    # thresholds between 0,.5,1,1.5,2,3,4,6 ; ties go to the code with even mantissa bit (0,1,2,4 -> codes 0,2,4,6)
    code = np.zeros(a.shape, dtype=np.uint8)
    code = np.where(a > 0.25, 1, code)
    code = np.where(a >= 0.75, 2, code)
    code = np.where(a > 1.25, 3, code)
    code = np.where(a >= 1.75, 4, code)
    code = np.where(a > 2.5, 5, code)
    code = np.where(a >= 3.5, 6, code)
    code = np.where(a > 5.0, 7, code)
    return (code | (np.signbit(x).astype(np.uint8) << 3)).astype(np.uint8)


def bf16_round(x):
    """float32 -> nearest bfloat16 (ties to even), returned as float32."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = r.astype(np.uint32).view(np.float32)
    return np.where(np.isnan(x), np.float32("nan"), out)


def bf16_bits_to_f32(u16):
    return (np.asarray(u16, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x):
    return (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


# ---- cache format -----------------------------------------------------------------------------------------------

def unpack_codes(ckv_cache):
    """[..., 256] uint8 -> [..., 512] E2M1 codes; low nibble = even channel (testing.py:76)."""
    c = np.asarray(ckv_cache, dtype=np.uint8)
    return np.stack([c & 15, c >> 4], -1).reshape(*c.shape[:-1], CKV)


def dequantize(ckv_cache, ckv_sf_cache, kpe_cache, ckv_scale=1.0, kpe_scale=1.0):
    """fp32 ([pages, page_size, 512], [pages, page_size, 64]); follows testing.py:73-78 operation by operation."""
    val = E2M1_LUT[unpack_codes(ckv_cache)]
    sf = np.repeat(e4m3_decode(ckv_sf_cache), 16, axis=-1)
    with np.errstate(invalid="ignore", over="ignore"):
        ckv = (val * sf) * np.float32(ckv_scale)
        kpe = e4m3_decode(kpe_cache) * np.float32(kpe_scale)
    return ckv.astype(np.float32), kpe.astype(np.float32)


def quantize_ckv(x, ckv_scale):
    """[n, 512] float32 -> (packed [n, 256] uint8, scales [n, 32] uint8 E4M3). Writer restatement (unpinned)."""
    x = np.asarray(x, dtype=np.float32).reshape(-1, CKV // 16, 16)
    amax = np.abs(x).max(-1)
    sf8 = e4m3_encode(amax / np.float32(6.0) / np.float32(ckv_scale))
    sf = e4m3_decode(sf8) * np.float32(ckv_scale)
    with np.errstate(divide="ignore", invalid="ignore"):
        y = np.where(sf[..., None] > 0, x / sf[..., None], 0.0)
    codes = e2m1_encode(y).reshape(-1, CKV)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return packed, sf8


def quantize_kpe(x, kpe_scale):
    return e4m3_encode(np.asarray(x, dtype=np.float32) / np.float32(kpe_scale))


# ---- attention ---------------------------------------------------------------------------------------------------

def gather_request(ckv, kpe, page_table, b, L):
    ps = ckv.shape[1]
    pages = np.asarray(page_table[b, :math.ceil(L / ps)], dtype=np.int64)
    return ckv[pages].reshape(-1, CKV)[:L], kpe[pages].reshape(-1, KPE)[:L]


def attention(q_nope, q_pe, ckv, kpe, page_table, kv_lens, sm_scale=SM_SCALE, return_lse=False):
    """fp32 absorbed-MLA decode over a dequantized (or unquantized) cache; testing.py:81-89.

    q_nope [B, H, 512], q_pe [B, H, 64]: float32 arrays holding bf16-representable values.
    Returns out [B, H, 512] float32 and, with return_lse, the natural-log lse [B, H] (an addition: the reference's
    torch path does not return it; the kernels' unit is lse * log2(e), mla_decode.cu:478, :491).
    A request of length 0 gives out = 0 and lse = -inf.
    """
    B, H = q_nope.shape[:2]
    out = np.zeros((B, H, CKV), dtype=np.float32)
    lse = np.full((B, H), -np.inf, dtype=np.float32)
    for b, L in enumerate(np.asarray(kv_lens).tolist()):
        if L <= 0:
            continue
        kc, kp = gather_request(ckv, kpe, page_table, b, L)
        s = (q_nope[b].astype(np.float32) @ kc.T + q_pe[b].astype(np.float32) @ kp.T) * np.float32(sm_scale)
        m = s.max(-1, keepdims=True)
        p = np.exp(s - m)
        l = p.sum(-1, keepdims=True)
        out[b] = (p / l) @ kc
        lse[b] = (m + np.log(l))[:, 0]
    return (out, lse) if return_lse else out


def attention_partial(q_nope, q_pe, ckv, kpe, page_table, kv_lens, sm_scale, t_begin, t_end):
    """Attention restricted to tokens [t_begin, t_end) of every request: normalised o and lse in log2 units.

    This is the split-KV partial contract of mla_decode.cu:478-492 (o normalised by the split's own l,
    lse = m + log2(l) with scores in log2 units, -inf for an empty split).
    """
    B, H = q_nope.shape[:2]
    o = np.zeros((B, H, CKV), dtype=np.float32)
    lse2 = np.full((B, H), -np.inf, dtype=np.float32)
    for b, L in enumerate(np.asarray(kv_lens).tolist()):
        lo, hi = min(t_begin, L), min(t_end, L)
        if hi <= lo:
            continue
        kc, kp = gather_request(ckv, kpe, page_table, b, L)
        kc, kp = kc[lo:hi], kp[lo:hi]
        s = (q_nope[b] @ kc.T + q_pe[b] @ kp.T) * np.float32(sm_scale * LOG2E)
        m = s.max(-1, keepdims=True)
        p = np.exp2(s - m)
        l = p.sum(-1, keepdims=True)
        o[b] = (p / l) @ kc
        lse2[b] = (m + np.log2(l))[:, 0]
    return o, lse2


def combine(o_part, lse_part):
    """LSE merge of split partials; mla_decode.cu:933-966. o_part [S, B, H, 512], lse_part [S, B, H] (log2 units).

    Returns (out [B, H, 512] float32, lse [B, H] in log2 units). Rows whose every split is empty give 0 / -inf.
    """
    M = lse_part.max(0)
    with np.errstate(invalid="ignore"):
        w = np.where(np.isneginf(lse_part), 0.0, np.exp2(lse_part - np.where(np.isneginf(M), 0.0, M)))
    den = w.sum(0)
    with np.errstate(invalid="ignore", divide="ignore"):
        out = np.where(den[..., None] > 0, (w[..., None] * o_part).sum(0) / den[..., None], 0.0)
        lse = np.where(den > 0, M + np.log2(den), -np.inf)
    return out.astype(np.float32), lse.astype(np.float32)


# ---- fp8-mode model (what an E4M3 attention over this cache computes) ---------------------------------------------

def _e4m3_round(x):
    return e4m3_decode(e4m3_encode(x))


def attention_fp8_model(q_nope, q_pe, ckv_cache, ckv_sf_cache, kpe_cache, page_table, kv_lens, sm_scale,
                        ckv_scale, kpe_scale):
    """Model of the fp8 precision mode: E4M3 query rows (448 / amax, nope and rope parts separately), K and V
    rounded as e4m3((e2m1 * sf) / 8), raw E4M3 kpe bytes, fp32 accumulation, E4M3 P with an exact running max.

    Follows the reference's fp8 arithmetic (mla_decode.cu:192-220, :425-457, :762-808) except for the lazy
    (stale-max) rescale, which changes results only through the rounding of P. Used for error budgeting, not as
    the parity target: fp8-mode parity is the reference's own bound (rel-L2 < 0.08 against attention()).
    """
    B, H = q_nope.shape[:2]
    val = E2M1_LUT[unpack_codes(ckv_cache)] * np.repeat(e4m3_decode(ckv_sf_cache), 16, axis=-1) / np.float32(8)
    k8 = _e4m3_round(np.nan_to_num(val))
    kp8 = np.nan_to_num(e4m3_decode(kpe_cache))
    out = np.zeros((B, H, CKV), dtype=np.float32)
    for b, L in enumerate(np.asarray(kv_lens).tolist()):
        if L <= 0:
            continue
        kc, kp = gather_request(k8, kp8, page_table, b, L)
        an = np.maximum(np.abs(q_nope[b]).max(-1, keepdims=True), 1e-30).astype(np.float32)
        ap = np.maximum(np.abs(q_pe[b]).max(-1, keepdims=True), 1e-30).astype(np.float32)
        qn8 = _e4m3_round(q_nope[b] * (np.float32(448) / an))
        qp8 = _e4m3_round(q_pe[b] * (np.float32(448) / ap))
        s = (qn8 @ kc.T) * (an / 448 * np.float32(ckv_scale) * 8) + (qp8 @ kp.T) * (ap / 448 * np.float32(kpe_scale))
        s = s * np.float32(sm_scale * LOG2E)
        m = s.max(-1, keepdims=True)
        p = np.exp2(s - m)
        l = p.sum(-1, keepdims=True)
        out[b] = (_e4m3_round(p) @ kc) * (np.float32(ckv_scale) * 8) / l
    return out


def rel_l2(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))
