"""GPU parity tests of the CUDA path (through the ctypes C ABI) against the numpy oracle and the golden vectors.

Mirrors the reference's tests/test_decode.py: the same edge-case geometry (:17-24), split counts (:50), bitwise
dequantisation (:38-47), public-API behaviour (:106-115) and input rejection (:118-128).
Tolerances, bf16 mode: max-abs <= 2e-2 and rel-L2 < 4e-3 on the output, <= 1e-3 on the natural-log LSE.
"""
import math

import numpy as np
import pytest
import torch

import mla_oracle as O
import nvfp4_mla_b200 as mla
from nvfp4_mla_b200.testing import SM_SCALE, SyntheticCache, attention_paged_nvfp4, rel_l2
from util import GOLDEN_NAMES, load_golden, oracle_reference

pytestmark = pytest.mark.gpu
LN2 = math.log(2.0)

CASES = [  # (kv_lens, page_size, heads): the reference's list plus lengths around the 128-token tile
    ([1], 1, 16),
    ([17, 1, 64, 65], 16, 16),
    ([1000, 4097, 3, 64], 64, 16),
    ([513, 2048], 1, 128),
    ([4096, 1, 777, 5000], 64, 128),
    ([31, 33, 95, 97], 16, 16),
    ([1, 2, 63, 64, 65, 127, 128, 129, 255, 256, 257, 300, 513], 64, 16),
    ([0, 5, 0, 130], 32, 16),            # empty requests
    ([700, 129], 128, 32),               # page larger than a staging slot
    ([260, 1], 256, 16),
]


def check_status():
    assert mla.workspace_status() == 0, "device-side status word is set (a bounded wait gave up)"


def check(c, out, lse2=None, label=""):
    want, want_lse = oracle_reference(c)
    got = out.float().cpu().numpy()
    assert not np.isnan(got).any(), label
    nz = [b for b, L in enumerate(c.kv_lens_list) if L > 0]
    err = np.abs(got - want).max()
    rel = O.rel_l2(got[nz], want[nz]) if nz else 0.0
    print(f"{label}: max-abs {err:.2e} rel-L2 {rel:.2e}")
    assert err <= 2e-2, label
    assert rel < 4e-3, label
    for b, L in enumerate(c.kv_lens_list):
        if L == 0:
            assert (got[b] == 0).all(), label
    if lse2 is not None:
        got_lse = lse2.cpu().numpy() * LN2
        for b, L in enumerate(c.kv_lens_list):
            if L == 0:
                assert np.isneginf(got_lse[b]).all(), label
            else:
                assert np.abs(got_lse[b] - want_lse[b]).max() <= 1e-3, label


@pytest.mark.parametrize("ckv_scale,kpe_scale", [(1.0, 1.0), (0.37, 3.1)])
def test_dequantize_bitwise(ckv_scale, kpe_scale):
    c = SyntheticCache([100, 37], 16, 16, ckv_scale, kpe_scale, seed=11).to("cuda")
    ckv, kpe = mla.dequantize(c.ckv_cache, c.ckv_sf_cache, c.kpe_cache, ckv_scale, kpe_scale, dtype=torch.float32)
    got = torch.cat([ckv, kpe], -1).cpu().numpy()
    w_ckv, w_kpe = O.dequantize(c.ckv_cache.cpu().numpy(), c.ckv_sf_cache.view(torch.uint8).cpu().numpy(),
                                c.kpe_cache.view(torch.uint8).cpu().numpy(), ckv_scale, kpe_scale)
    want = np.concatenate([w_ckv, w_kpe], -1)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(want)
    assert np.array_equal(got.view(np.int32)[ok], want.view(np.int32)[ok])
    ckv16, kpe16 = mla.dequantize(c.ckv_cache, c.ckv_sf_cache, c.kpe_cache, ckv_scale, kpe_scale)
    got16 = torch.cat([ckv16, kpe16], -1)
    assert got16.dtype == torch.bfloat16
    want16 = torch.from_numpy(want).bfloat16()
    ok_t = torch.from_numpy(ok)
    assert torch.equal(got16.cpu()[ok_t], want16[ok_t])


def test_dequantize_golden():
    g, c = load_golden("tiny")
    c.to("cuda")
    ckv, kpe = mla.dequantize(c.ckv_cache, c.ckv_sf_cache, c.kpe_cache, c.ckv_scale, c.kpe_scale, dtype=torch.float32)
    for got, bits in ((ckv, g["deq_ckv_bits"]), (kpe, g["deq_kpe_bits"])):
        got = got.cpu().numpy()
        want = bits.view(np.float32)
        ok = ~np.isnan(want)
        assert np.array_equal(np.isnan(got), ~ok) and np.array_equal(got.view(np.int32)[ok], bits[ok])


def test_combine_vs_oracle():
    rng = np.random.default_rng(0)
    S, B, H = 5, 3, 16
    o = rng.standard_normal((S, B, H, 512)).astype(np.float32)
    lse = (rng.standard_normal((S, B, H)) * 4).astype(np.float32)
    lse[1, 0] = -np.inf            # an empty split
    lse[:, 2, 3] = -np.inf         # a row with no tokens at all
    want, want_lse = O.combine(o, lse)
    out, got_lse = mla.combine(torch.from_numpy(o).cuda(), torch.from_numpy(lse).cuda(), torch.float32, return_lse=True)
    assert np.abs(out.cpu().numpy() - want).max() < 1e-5
    g = got_lse.cpu().numpy()
    assert np.array_equal(np.isneginf(g), np.isneginf(want_lse))
    assert np.abs(g[np.isfinite(g)] - want_lse[np.isfinite(g)]).max() < 1e-5
    out16 = mla.combine(torch.from_numpy(o).cuda(), torch.from_numpy(lse).cuda())
    assert out16.dtype == torch.bfloat16 and np.abs(out16.float().cpu().numpy() - want).max() < 2e-2


def test_combine_records_equals_packed_merge():
    """The merge over records at unrelated addresses (what the cross-GPU merge reads from the peers' buffers) against the
    merge over one packed buffer, bit for bit, with an empty partial (lse = -inf) among them."""
    g = torch.Generator().manual_seed(5)
    rows, parts = 48, 5
    recs = [torch.empty(rows * 513, dtype=torch.float32, device="cuda") for _ in range(parts)]
    for i, r in enumerate(recs):
        r[:rows * 512] = torch.randn(rows * 512, generator=g).cuda()
        r[rows * 512:] = (torch.randn(rows, generator=g) * 3).cuda()
    recs[2][rows * 512:] = float("-inf")
    recs[2][:rows * 512] = float("nan")  # a partial of weight 0 may hold anything
    want = mla.combine_packed(torch.stack(recs), rows, torch.float32)
    got = mla.combine_records([r.data_ptr() for r in recs], rows, "cuda", torch.float32)
    torch.cuda.synchronize()
    assert not got.isnan().any()
    assert torch.equal(got, want)
    with pytest.raises(RuntimeError):
        mla.combine_records([r.data_ptr() for r in recs] * 4, rows, "cuda")  # 20 records: over the limit of 16


@pytest.mark.parametrize("rows", [48, 400])
def test_combine_records_signalled_on_one_gpu(rows):
    """The merge kernel that carries the GPUs' hand-shake, driven as "GPU 0 of 3" on one device: the words the other
    GPUs would write are set by the host. With all of them announced the result is the plain merge, bit for bit, and
    the kernel has announced itself in word 0 of every GPU's array; with one GPU missing the bounded wait runs out,
    status 4 is raised, and the context stays usable (a wait that ends by itself: nothing hangs or faults)."""
    g = torch.Generator().manual_seed(6)
    parts = 3
    recs = [torch.empty(rows * 513, dtype=torch.float32, device="cuda") for _ in range(parts)]
    for r in recs:
        r[:rows * 512] = torch.randn(rows * 512, generator=g).cuda()
        r[rows * 512:] = (torch.randn(rows, generator=g) * 3).cuda()
    want = mla.combine_records([r.data_ptr() for r in recs], rows, "cuda", torch.float32)
    flags = [torch.zeros(parts, dtype=torch.int32, device="cuda") for _ in range(parts)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ptrs, fptrs = [r.data_ptr() for r in recs], [f.data_ptr() for f in flags]
    epoch = 7
    flags[0][1], flags[0][2] = epoch, epoch + 1  # GPU 2 is one step ahead: allowed
    got = mla.combine_records_signalled(ptrs, fptrs, 0, epoch, rows, "cuda", torch.float32, status, wait_us=500_000)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and torch.equal(got, want)
    assert [int(f[0]) for f in flags] == [epoch] * parts and int(flags[1][1]) == 0
    # GPU 1 never announces the next step
    flags[0][2] = epoch + 1
    mla.combine_records_signalled(ptrs, fptrs, 0, epoch + 1, rows, "cuda", torch.float32, status, wait_us=2_000)
    torch.cuda.synchronize()
    assert int(status.item()) == 4
    assert torch.equal(mla.combine_records(ptrs, rows, "cuda", torch.float32), want)  # the context is intact
    with pytest.raises(RuntimeError):
        mla.combine_records_signalled(ptrs, fptrs, 3, epoch, rows, "cuda")  # rank outside [0, parts)
    with pytest.raises(RuntimeError):
        mla.combine_records_signalled(ptrs, fptrs, 0, epoch, rows, "cuda", wait_us=0)  # an unbounded wait is not offered


@pytest.mark.parametrize("parts,rows_shape", [(3, (2, 16)), (9, (40, 16)), (70, (2, 16)), (70, (40, 16))])
def test_combine_ignores_empty_partials(parts, rows_shape):
    """A partial of weight 0 (lse = -inf) may hold anything, NaN included: it must not reach the result. Covers the rows
    requested before the weights are known (the first eight per thread group) and the later batches, for few rows
    (four thread groups per row) and many (one group)."""
    rng = np.random.default_rng(parts)
    o = rng.standard_normal((parts, *rows_shape, 512)).astype(np.float32)
    lse = (rng.standard_normal((parts, *rows_shape)) * 4).astype(np.float32)
    dead = rng.random((parts, *rows_shape)) < 0.3
    dead[0] = False  # every row keeps at least one live partial
    lse[dead] = -np.inf
    want, want_lse = O.combine(np.where(dead[..., None], 0.0, o).astype(np.float32), lse)
    o[dead] = np.nan
    out, got_lse = mla.combine(torch.from_numpy(o).cuda(), torch.from_numpy(lse).cuda(), torch.float32, return_lse=True)
    got = out.cpu().numpy()
    assert not np.isnan(got).any()
    assert np.abs(got - want).max() < 1e-5
    assert np.abs(got_lse.cpu().numpy() - want_lse).max() < 1e-5


@pytest.mark.parametrize("num_splits", [0, 1, 3, 7])
@pytest.mark.parametrize("kv_lens,page_size,heads", CASES)
def test_decode(num_splits, kv_lens, page_size, heads):
    c = SyntheticCache(kv_lens, page_size, heads, 0.5, 2.0, seed=len(kv_lens) + page_size).to("cuda")
    out = mla.decode(*c.args(), max_kv_len=c.max_kv_len, num_splits=num_splits)
    o32, lse2 = mla.decode_partial(*c.args(), max_kv_len=c.max_kv_len, num_splits=num_splits)
    check_status()
    label = f"splits={num_splits} {kv_lens} ps={page_size} H={heads}"
    check(c, out, lse2, label)
    check(c, o32, None, label + " (f32)")


@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_decode_golden(name):
    """Against the reference's own torch output stored in tests/golden/."""
    g, c = load_golden(name)
    c.to("cuda")
    out = mla.decode(*c.args(), max_kv_len=c.max_kv_len)
    check_status()
    got = out.float().cpu().numpy()[:, ::int(g["head_stride"]), ::int(g["chan_stride"])]
    assert not np.isnan(got).any()
    assert np.abs(got - g["out"]).max() <= 2e-2
    assert O.rel_l2(got, g["out"]) < 4e-3


def test_calibrated_scales():
    """Global scales as a serving engine sets them: block scales reach the E4M3 maximum, e2m1 x scale reaches 2688."""
    c = SyntheticCache([300, 70, 1500], 64, 16, None, None, seed=5).to("cuda")
    out = mla.decode(*c.args(), max_kv_len=c.max_kv_len)
    check_status()
    check(c, out, None, "calibrated")


@pytest.mark.parametrize("factor", [8.0, 16.0])
def test_query_with_outlier_channels(factor):
    """The 16-bit mode multiplies QK^T with the query written as FP4 terms whose scales cover 32 channels each: a few
    channels far above the rest of their row (as absorbed queries have) must not cost the other channels their
    precision. Same bounds as every 16-bit case (max-abs 2e-2, rel-L2 4e-3, LSE 1e-3); at 32 times the LSE error measured
    1.2e-3 (output bounds still met): the coding keeps 2^-12 of a 32-channel group's maximum, not of each element."""
    c = SyntheticCache([2000, 777, 4096, 130], 64, 16, None, None, seed=11)
    g = torch.Generator().manual_seed(3)
    for b in range(c.q_nope.shape[0]):
        for h in range(16):
            idx = torch.randperm(512, generator=g)[:4]
            c.q_nope[b, h, idx] *= factor
    c.q_pe[:, ::3, :5] *= factor / 2
    c.to("cuda")
    out = mla.decode(*c.args(), max_kv_len=c.max_kv_len)
    _, lse2 = mla.decode_partial(*c.args(), max_kv_len=c.max_kv_len)
    check_status()
    check(c, out, lse2, f"outlier channels x{factor}")


@pytest.mark.parametrize("precision", ["bf16", "fp8"])
def test_schedule_inside_the_decode_kernel_and_in_front_of_it_agree(precision):
    """Up to one (request, split) pair per thread of a decode CTA the decode kernel derives the schedule by itself (two
    launches per call); beyond that a schedule kernel runs in front (three). Both must serve the same requests alike: a
    batch of 700 short ragged requests (some empty) takes the second path, its first 40 requests alone the first."""
    from nvfp4_mla_b200 import _lib
    lib = _lib.load()
    g = np.random.default_rng(11)
    lens = [int(x) for x in g.integers(0, 700, size=700)]
    lens[3] = lens[17] = 0
    c = SyntheticCache(lens, 64, 16, 0.5, 2.0, seed=4, device="cuda")
    prec = 0 if precision == "bf16" else 1
    assert lib.nvfp4_mla_decode_launches(700, 16, max(lens), 0, prec) == 3
    assert lib.nvfp4_mla_decode_launches(40, 16, max(lens), 0, prec) == 2
    assert lib.nvfp4_mla_decode_launches(0, 16, 128, 0, prec) == 0
    big = mla.decode(*c.args(SM_SCALE), max_kv_len=max(lens), precision=precision)
    a = list(c.args(SM_SCALE))

    def first(m):
        return mla.decode(a[0][:m].contiguous(), a[1][:m].contiguous(), a[2], a[3], a[4], a[5][:m].contiguous(),
                          a[6][:m].contiguous(), *a[7:], max_kv_len=max(lens), precision=precision)

    n = 40
    small = first(n)
    edge = 640 if precision == "bf16" else 512  # one pair per thread of the decode CTA: the largest batch of the first path
    assert lib.nvfp4_mla_decode_launches(edge, 16, max(lens), 0, prec) == 2
    assert lib.nvfp4_mla_decode_launches(edge + 1, 16, max(lens), 0, prec) == 3
    at_edge, past_edge = first(edge), first(edge + 1)
    torch.cuda.synchronize()
    assert mla.workspace_status() == 0
    assert float(big[3].abs().max()) == 0.0 and float(big[17].abs().max()) == 0.0
    want, _ = oracle_reference(c)
    tol = 4e-3 if precision == "bf16" else 0.08  # rel-L2 bounds of the two modes, as in the tests above
    for got, m in ((big.float().cpu().numpy(), 700), (small.float().cpu().numpy(), n),
                   (at_edge.float().cpu().numpy(), edge), (past_edge.float().cpu().numpy(), edge + 1)):
        assert not np.isnan(got).any()
        nz = [b for b in range(m) if lens[b] > 0]
        assert O.rel_l2(got[nz], want[nz]) < tol
    # the two schedules cut the requests at different tiles, so the results agree to rounding, not bit for bit
    assert float((big[:n].float() - small.float()).abs().max()) <= (2e-2 if precision == "bf16" else 0.2)


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_shapes_are_deterministic_and_clean(seed):
    """A dozen random (batch, heads, page size, lengths, splits) per seed, both modes: repeated calls give identical
    bits, the status word stays 0, and the 16-bit result of the smaller cases is held against the oracle."""
    import random
    rnd = random.Random(seed)
    for rep in range(12):
        B = rnd.choice([1, 2, 3, 8, 17, 32])
        H = rnd.choice([16, 16, 32, 128])
        ps = rnd.choice([16, 32, 64, 64, 128, 256])
        maxlen = rnd.choice([1, 130, 700, 4096, 9000])
        lens = [rnd.randint(0 if rnd.random() < 0.1 else 1, maxlen) for _ in range(B)]
        if H == 128:
            lens = lens[:3]
        c = SyntheticCache(lens, ps, H, None, None, seed=100 * seed + rep).to("cuda")
        for prec in ("bf16", "fp8"):
            splits = rnd.choice([0, 1, 2, 5])
            outs = [mla.decode(*c.args(), max_kv_len=max(lens + [1]), num_splits=splits, precision=prec) for _ in range(3)]
            check_status()
            assert not outs[0].isnan().any()
            assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]), (B, H, ps, prec, splits)
            if prec == "bf16" and sum(lens) * H <= 400000:
                check(c, outs[0], None, f"random shape B={B} H={H} ps={ps} splits={splits}")


SCALES = {"scale 0.5": (0.5, 2.0), "calibrated": (2.0 ** -9, 2.0 ** -6)}


@pytest.mark.parametrize("scales", SCALES.values(), ids=SCALES.keys())
@pytest.mark.parametrize("num_splits", [0, 3])
@pytest.mark.parametrize("kv_lens,page_size,heads", CASES[:6])
def test_decode_fp8(num_splits, kv_lens, page_size, heads, scales):
    """fp8 mode (E4M3 query rows, K, V and P): the reference's bounds (tests/test_decode.py:77-88): rel-L2 < 0.08 against
    the dequantised-cache oracle, and at most 1.2x the bf16 mode's error against the unquantised BF16 cache. Both the
    scale-0.5 and the calibrated global scales (block scales near 448: e2m1 x scale reaches 2688, the saturation guard)."""
    c = SyntheticCache(kv_lens, page_size, heads, *scales, seed=len(kv_lens) + page_size, keep_bf16=True).to("cuda")
    out = mla.decode(*c.args(), max_kv_len=c.max_kv_len, num_splits=num_splits, precision="fp8")
    out16 = mla.decode(*c.args(), max_kv_len=c.max_kv_len, num_splits=num_splits)
    check_status()
    assert not out.isnan().any()
    want, _ = oracle_reference(c)
    got = out.float().cpu().numpy()
    err = O.rel_l2(got, want)
    print(f"fp8 splits={num_splits} {kv_lens} ps={page_size} H={heads}: rel-L2 {err:.3e}")
    assert err < 0.08
    ref = c.reference_bf16().cpu().numpy()
    assert O.rel_l2(got, ref) < 1.2 * O.rel_l2(out16.float().cpu().numpy(), ref)


def test_fp8_streamed_reference_8k():
    c = SyntheticCache([8192] * 8, 64, 16, None, None, seed=4, device="cuda")
    out = mla.decode(*c.args(), max_kv_len=8192, precision="fp8")
    check_status()
    want, _ = attention_paged_nvfp4(*c.args(), requests=[0, 7])
    assert not out.isnan().any()
    assert rel_l2(out[[0, 7]], want) < 0.08


def test_max_kv_len_is_an_upper_bound():
    c = SyntheticCache([100, 900, 257], 64, 16, 0.5, 2.0, seed=9).to("cuda")
    a = mla.decode(*c.args(), max_kv_len=c.max_kv_len)
    b = mla.decode(*c.args(), max_kv_len=4096)
    d = mla.decode(*c.args())  # default: kv_lens.max()
    check_status()
    check(c, b, None, "max_kv_len=4096")
    assert torch.equal(a, d)


def test_cuda_graph_replay_with_new_lengths():
    """The launch shape depends on max_kv_len only: a captured decode replays correctly after kv_lens change."""
    big = SyntheticCache([1024, 1024, 1024], 64, 16, 0.5, 2.0, seed=21).to("cuda")  # every replayed length is written
    args = list(big.args())
    kv = big.kv_lens.clone()
    args[6] = kv
    mla.decode(*args, max_kv_len=1024)  # warm-up outside capture (one-time per-device setup)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = mla.decode(*args, max_kv_len=1024)
    for lens in ([1000, 700, 300], [5, 1024, 129], [640, 1, 0]):
        kv.copy_(torch.tensor(lens, dtype=torch.int32))
        graph.replay()
        torch.cuda.synchronize()
        big.kv_lens_list = lens
        big.kv_lens = kv
        check(big, out, None, f"graph replay {lens}")
    check_status()


def test_public_api():
    c = SyntheticCache([300, 70], 16, 16, 0.5, 2.0, seed=2).to("cuda")
    check(c, mla.decode(*c.args()), None, "decode defaults")
    assert mla.decode(*c.args(), precision="fp8").dtype == torch.bfloat16
    with pytest.raises(ValueError, match="precision"):
        mla.decode(*c.args(), precision="fp4-qk")
    with pytest.raises(ValueError, match="precision"):
        mla.decode(*c.args(), precision="int8")
    with pytest.raises(ValueError, match="dtype"):
        mla.dequantize(c.ckv_cache, c.ckv_sf_cache, c.kpe_cache, dtype=torch.float16)
    import nvfp4_mla
    assert nvfp4_mla.decode is mla.decode and nvfp4_mla.dequantize is mla.dequantize
    check_status()


def test_rejects_bad_inputs():
    c = SyntheticCache([64], 16, 16, seed=3).to("cuda")
    a = list(c.args())
    with pytest.raises(RuntimeError, match="bfloat16"):
        mla.decode(c.q_nope.half(), *a[1:])
    with pytest.raises(RuntimeError, match="multiple of 16"):
        mla.decode(c.q_nope[:, :8].contiguous(), c.q_pe[:, :8].contiguous(), *a[2:])
    with pytest.raises(RuntimeError, match="int32"):
        mla.decode(*a[:5], c.page_table.long(), *a[6:])
    with pytest.raises(RuntimeError, match="float8_e4m3fn"):
        mla.decode(*a[:3], c.ckv_sf_cache.view(torch.uint8), *a[4:])
    with pytest.raises(RuntimeError, match="positive"):
        mla.decode(*a[:8], 0.0, 1.0)


@pytest.mark.parametrize("precision,heads", [("bf16", 16), ("fp8", 16), ("fp8", 128)])
@pytest.mark.parametrize("page_size", [16, 64])
def test_page_ids_are_range_checked(page_size, precision, heads):
    """A page id outside [0, num_pages) must never be dereferenced. Beyond a request's live pages the table may hold
    anything (it is not read); inside the live range a bad id raises status 3 and the kernel loads nothing for it:
    with pages of a staging slot or more the rows read as zeros (finite output), smaller pages are left unloaded.
    The reference poisons everything out of range the same way (nvfp4_mla/testing.py:18-20, 47-50)."""
    c = SyntheticCache([300, 200], page_size, heads, 0.5, 2.0, seed=8).to("cuda")
    clean = mla.decode(*c.args(), max_kv_len=300, precision=precision)
    check_status()
    a = list(c.args())
    pt = torch.cat([c.page_table, torch.full((2, 3), 1 << 30, dtype=torch.int32, device="cuda")], 1).contiguous()
    n1 = math.ceil(200 / page_size)
    pt[1, n1:] = -7                      # the shorter request's unused entries
    a[5] = pt
    out = mla.decode(*a, max_kv_len=300, precision=precision)
    assert mla.workspace_status() == 0
    assert torch.equal(out, clean)
    pt[0, 1] = c.ckv_cache.shape[0]      # first id past the pool, inside request 0's live range
    pt[1, 0] = -1
    out = mla.decode(*a, max_kv_len=300, precision=precision)
    assert mla.workspace_status(clear=True) == 3
    if page_size >= 64:
        assert not out.isnan().any()
    assert mla.workspace_status() == 0


def test_config1_shape_streamed_reference():
    """B=32, H=16, kv=8192 (DeepSeek-V3 TP8 shard): checked against the streamed torch reference on the GPU for a
    sample of requests, and through the split-invariance property for all of them."""
    c = SyntheticCache([8192] * 32, 64, 16, None, None, seed=1, device="cuda")
    out = mla.decode(*c.args(), max_kv_len=8192)
    o32, lse2 = mla.decode_partial(*c.args(), max_kv_len=8192)
    check_status()
    reqs = [0, 13, 31]
    want, want_lse = attention_paged_nvfp4(*c.args(), requests=reqs)
    assert not out.isnan().any()
    assert (out[reqs].float() - want).abs().max().item() <= 2e-2
    assert rel_l2(out[reqs], want) < 4e-3
    assert (lse2[reqs] * LN2 - want_lse).abs().max().item() <= 1e-3
    o_split = mla.decode_partial(*c.args(), max_kv_len=8192, num_splits=5)[0]
    assert (o_split - o32).abs().max().item() <= 1e-3   # property: the result does not depend on the split
    check_status()


def test_config2_shape_streamed_reference():
    """B=64, H=16, kv=65536, bf16 mode: the configuration the headline metric is quoted on (1.48 GB of NVFP4 KV), at
    its own size. A sample of requests (first, middle, last) against the streamed dequantise-then-attention reference on
    the GPU, and the split-invariance property over all 64."""
    c = SyntheticCache([65536] * 64, 64, 16, None, None, seed=0, device="cuda")
    out = mla.decode(*c.args(), max_kv_len=65536)
    o32, lse2 = mla.decode_partial(*c.args(), max_kv_len=65536)
    check_status()
    assert not out.isnan().any()
    reqs = [0, 31, 63]
    want, want_lse = attention_paged_nvfp4(*c.args(), requests=reqs)
    err, rel = (out[reqs].float() - want).abs().max().item(), rel_l2(out[reqs], want)
    lse_err = (lse2[reqs] * LN2 - want_lse).abs().max().item()
    print(f"config 2: max-abs {err:.2e} rel-L2 {rel:.2e} lse {lse_err:.2e}")
    assert err <= 2e-2 and rel < 4e-3 and lse_err <= 1e-3
    o_split = mla.decode_partial(*c.args(), max_kv_len=65536, num_splits=3)[0]
    assert (o_split - o32).abs().max().item() <= 1e-3   # property: the result does not depend on the split
    check_status()


def test_config4_shape_one_gpu():
    """B=2, H=128, kv=1 048 576 each, bf16 mode (the long-context configuration on one GPU: page-table rows of 16 384
    entries, 8 192 tiles per request, P summed over a million tokens): request 1 against the streamed reference on a
    sample of 16 heads, plus split invariance over everything."""
    c = SyntheticCache([1048576] * 2, 64, 128, 2.0 ** -9, 2.0 ** -6, seed=4, device="cuda")
    out = mla.decode(*c.args(), max_kv_len=1048576)
    o32, lse2 = mla.decode_partial(*c.args(), max_kv_len=1048576)
    check_status()
    assert not out.isnan().any()
    heads = list(range(3, 128, 8))
    a = list(c.args())
    a[0], a[1] = c.q_nope[:, heads].contiguous(), c.q_pe[:, heads].contiguous()
    want, want_lse = attention_paged_nvfp4(*a, requests=[1])
    got = out[1:2, heads].float()
    err, rel = (got - want).abs().max().item(), rel_l2(got, want)
    lse_err = (lse2[1:2, heads] * LN2 - want_lse).abs().max().item()
    print(f"config 4: max-abs {err:.2e} rel-L2 {rel:.2e} lse {lse_err:.2e}")
    assert err <= 2e-2 and rel < 4e-3 and lse_err <= 1e-3
    o_split = mla.decode_partial(*c.args(), max_kv_len=1048576, num_splits=5)[0]
    assert (o_split - o32).abs().max().item() <= 1e-3
    check_status()


HM_CASES = [  # the 128-head 8-bit kernel (heads as M, CTA pairs): lengths around its 64-token tile, 256 heads, empty requests
    ([1, 31, 32, 33, 63, 64, 65, 127, 128, 129], 64, 128),
    ([0, 700, 0, 2050], 32, 128),
    ([300, 5000], 16, 256),
    ([9000], 128, 128),
    ([40, 3], 4, 128),
]


@pytest.mark.parametrize("num_splits", [0, 1, 7])
@pytest.mark.parametrize("kv_lens,page_size,heads", HM_CASES)
def test_decode_fp8_128_heads(num_splits, kv_lens, page_size, heads):
    c = SyntheticCache(kv_lens, page_size, heads, 2.0 ** -9, 2.0 ** -6, seed=3 + len(kv_lens), keep_bf16=True).to("cuda")
    out = mla.decode(*c.args(), max_kv_len=c.max_kv_len, num_splits=num_splits, precision="fp8")
    out16 = mla.decode(*c.args(), max_kv_len=c.max_kv_len, num_splits=num_splits)
    check_status()
    assert not out.isnan().any()
    want, _ = oracle_reference(c)
    got = out.float().cpu().numpy()
    live = [b for b, L in enumerate(kv_lens) if L > 0]
    for b, L in enumerate(kv_lens):
        if L == 0:
            assert (got[b] == 0).all()
    assert O.rel_l2(got[live], want[live]) < 0.08
    ref = c.reference_bf16().cpu().numpy()
    assert O.rel_l2(got[live], ref[live]) < 1.2 * O.rel_l2(out16.float().cpu().numpy()[live], ref[live])


def test_cuda_graph_replay_fp8_128_heads():
    """The 128-head kernel launches clusters of two CTAs with a programmatic dependency: it must capture and replay."""
    c = SyntheticCache([1500, 2048], 64, 128, 0.5, 2.0, seed=12, device="cuda")  # replayed with shorter lengths below
    args = c.args()
    mla.decode(*args, max_kv_len=2048, precision="fp8")  # set-up outside capture
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = mla.decode(*args, max_kv_len=2048, precision="fp8")
    c.kv_lens.copy_(torch.tensor([700, 2000], dtype=torch.int32))
    g.replay()
    torch.cuda.synchronize()
    c.kv_lens_list = [700, 2000]
    want, _ = oracle_reference(c)
    assert O.rel_l2(out.float().cpu().numpy(), want) < 0.08
    check_status()


def test_fp8_128_heads_config3_sizes_streamed_reference():
    """The compute-bound configuration's shape on a slice of its batch (128 heads, ragged lengths up to 32K, calibrated scales, 8-bit
    mode) against the streamed dequantise-then-attention reference, plus two size-independent properties at that size:
    the output does not depend on `num_splits`-style re-cutting beyond rounding, and permuting the physical pages (with
    the page table following) leaves it unchanged bit for bit."""
    lens = [32768, 1024, 17000, 9999, 31, 24576]
    c = SyntheticCache(lens, 64, 128, None, None, seed=21, device="cuda")
    out = mla.decode(*c.args(), max_kv_len=32768, precision="fp8")
    check_status()
    assert not out.isnan().any()
    want, _ = attention_paged_nvfp4(*c.args(), requests=[0, 2, 4])
    assert rel_l2(out[[0, 2, 4]], want) < 0.08
    out3 = mla.decode(*c.args(), max_kv_len=32768, num_splits=3, precision="fp8")
    assert rel_l2(out3, out.float()) < 2e-2
    # physical page permutation
    P = c.ckv_cache.shape[0]
    perm = torch.randperm(P, device="cuda")
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(P, device="cuda")
    out_p = mla.decode(c.q_nope, c.q_pe, c.ckv_cache[perm].contiguous(), c.ckv_sf_cache.view(torch.uint8)[perm].contiguous().view(torch.float8_e4m3fn),
                       c.kpe_cache.view(torch.uint8)[perm].contiguous().view(torch.float8_e4m3fn), inv[c.page_table.long()].int().contiguous(),
                       c.kv_lens, SM_SCALE, c.ckv_scale, c.kpe_scale, max_kv_len=32768, precision="fp8")
    assert torch.equal(out_p, out)
    check_status()
