"""GPU parity tests of the cache writer (quantise + append into the paged NVFP4 cache) against the numpy oracle.

The reference has no writer of its own (it calls FlashInfer's, nvfp4_mla/testing.py:38-53); the oracle restates the
published format (block scale = e4m3(amax / 6 / ckv_scale), nearest E2M1 codes, e4m3 rope) and the CUDA kernel must
produce the same bytes bit for bit, leave every slot it was not asked to write untouched, and feed decode.
"""
import math

import numpy as np
import pytest
import torch

import mla_oracle as O
import nvfp4_mla_b200 as mla
from nvfp4_mla_b200.testing import SM_SCALE, SyntheticCache

pytestmark = pytest.mark.gpu


def paged_tables(kv_lens, ps, g, device):
    n_pages = [math.ceil(L / ps) for L in kv_lens]
    P = sum(n_pages)
    kv_indices = torch.randperm(P, generator=g).int().to(device)
    kv_indptr = torch.tensor([0] + n_pages).cumsum(0).int().to(device)
    return P, kv_indices, kv_indptr


def oracle_write(ckv, kpe, bi, pos, ckv_cache, sf_cache, kpe_cache, kv_indices, kv_indptr, ckv_scale, kpe_scale):
    """numpy: the same append, on copies of the caches."""
    ps = ckv_cache.shape[1]
    packed, sf8 = O.quantize_ckv(ckv.float().cpu().numpy(), ckv_scale)
    k8 = O.quantize_kpe(kpe.float().cpu().numpy(), kpe_scale)
    c, s, k = (t.cpu().view(torch.uint8).numpy().copy() for t in (ckv_cache, sf_cache, kpe_cache))
    ki, kp = kv_indices.cpu().numpy(), kv_indptr.cpu().numpy()
    for i, (b, p) in enumerate(zip(bi.cpu().tolist(), pos.cpu().tolist())):
        page = ki[kp[b] + p // ps]
        c[page, p % ps], s[page, p % ps], k[page, p % ps] = packed[i], sf8[i], k8[i]
    return c, s, k


def special_rows(n, g):
    """bf16 rows that exercise ties, zeros, signed zeros, saturation and subnormal scales."""
    x = torch.randn(n, 512, generator=g)
    x[0] = 0.0
    x[1, ::2] = -0.0
    x[2] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] * 64)          # exact ties when the scale is 1
    x[3] = -x[2]
    x[4] *= 1e-4                                                                     # tiny blocks: subnormal scales
    x[5] *= 3e3                                                                      # scale saturates at 448
    x[6, :16] = torch.tensor([6.0] + [0.0] * 15)
    x[7] = torch.tensor([1.0, -1.0] * 256) * 2.0 ** -20
    return x.bfloat16()


@pytest.mark.parametrize("ps", [1, 16, 64])
@pytest.mark.parametrize("scales", [(1.0, 1.0), (0.37, 3.1), (2.0 ** -9, 2.0 ** -6)])
def test_writer_bytes_equal_oracle(ps, scales):
    dev = "cuda"
    g = torch.Generator().manual_seed(5 + ps)
    kv_lens = [37, 1, 130, 64]
    P, kv_indices, kv_indptr = paged_tables(kv_lens, ps, g, dev)
    nnz = sum(kv_lens)
    ckv = torch.cat([special_rows(8, g), torch.randn(nnz - 8, 512, generator=g).bfloat16()]).to(dev)
    kpe = (torch.randn(nnz, 64, generator=g) * 3).bfloat16().to(dev)
    append_indptr = torch.tensor([0] + kv_lens).cumsum(0).int().to(dev)
    bi, pos = mla.get_batch_indices_positions(append_indptr, torch.tensor(kv_lens, dtype=torch.int32, device=dev), nnz)
    junk = lambda n: torch.randint(0, 256, (P, ps, n), generator=g, dtype=torch.uint8).to(dev)
    ckv_cache, sf_cache, kpe_cache = junk(256), junk(32).view(torch.float8_e4m3fn), junk(64).view(torch.float8_e4m3fn)
    want = oracle_write(ckv, kpe, bi, pos, ckv_cache, sf_cache, kpe_cache, kv_indices, kv_indptr, *scales)
    mla.quantize_append_paged_mla_kv_cache(ckv, kpe, bi, pos, ckv_cache, sf_cache, kpe_cache, kv_indices, kv_indptr, None,
                                           *scales, check=True)
    for name, got, w in zip(("ckv", "sf", "kpe"), (ckv_cache, sf_cache, kpe_cache), want):
        got = got.cpu().view(torch.uint8).numpy()
        assert np.array_equal(got, w), f"{name}: {np.count_nonzero(got != w)} bytes differ"


def test_incremental_append_then_decode():
    """Prefill part of every request, append the rest one token per request and step (a decode loop), and compare the
    cache and the decode output with the cache SyntheticCache writes in one go."""
    dev = "cuda"
    kv_lens, ps, heads = [200, 65, 129], 64, 16
    ref = SyntheticCache(kv_lens, ps, heads, 0.5, 2.0, seed=3, device=dev, keep_bf16=True)
    B = len(kv_lens)
    pt = ref.page_table
    n_pages = [math.ceil(L / ps) for L in kv_lens]
    kv_indices = torch.cat([pt[b, :n_pages[b]] for b in range(B)]).contiguous()
    kv_indptr = torch.tensor([0] + n_pages, device=dev).cumsum(0).int()
    ckv_cache, sf_cache, kpe_cache = (torch.zeros_like(t.view(torch.uint8)) for t in (ref.ckv_cache, ref.ckv_sf_cache, ref.kpe_cache))
    sf_cache, kpe_cache = sf_cache.view(torch.float8_e4m3fn), kpe_cache.view(torch.float8_e4m3fn)

    def rows(b, lo, hi):  # the unquantised rows of request b, tokens [lo, hi)
        idx = torch.arange(lo, hi, device=dev)
        pages = pt[b, idx // ps].long()
        return ref.ckv_bf16[pages, idx % ps], ref.kpe_bf16[pages, idx % ps]

    prefill = [L - 5 for L in kv_lens]
    parts = [rows(b, 0, prefill[b]) for b in range(B)]
    ckv, kpe = torch.cat([p[0] for p in parts]), torch.cat([p[1] for p in parts])
    append_indptr = torch.tensor([0] + prefill, device=dev).cumsum(0).int()
    bi, pos = mla.get_batch_indices_positions(append_indptr, torch.tensor(prefill, dtype=torch.int32, device=dev), sum(prefill))
    mla.quantize_append_paged_mla_kv_cache(ckv, kpe, bi, pos, ckv_cache, sf_cache, kpe_cache, kv_indices, kv_indptr, None,
                                           ref.ckv_scale, ref.kpe_scale, check=True)
    for step in range(5):
        lens = [p + step + 1 for p in prefill]
        parts = [rows(b, lens[b] - 1, lens[b]) for b in range(B)]
        ckv, kpe = torch.cat([p[0] for p in parts]), torch.cat([p[1] for p in parts])
        bi, pos = mla.get_batch_indices_positions(torch.arange(B + 1, device=dev).int(),
                                                  torch.tensor(lens, dtype=torch.int32, device=dev), B)
        mla.quantize_append_paged_mla_kv_cache(ckv, kpe, bi, pos, ckv_cache, sf_cache, kpe_cache, kv_indices, kv_indptr, None,
                                               ref.ckv_scale, ref.kpe_scale, check=True)
    # live slots equal the one-shot writer's bytes
    for b, L in enumerate(kv_lens):
        idx = torch.arange(L, device=dev)
        pages = pt[b, idx // ps].long()
        for got, want in ((ckv_cache, ref.ckv_cache), (sf_cache, ref.ckv_sf_cache), (kpe_cache, ref.kpe_cache)):
            assert torch.equal(got.view(torch.uint8)[pages, idx % ps], want.view(torch.uint8)[pages, idx % ps])
    out = mla.decode(ref.q_nope, ref.q_pe, ckv_cache, sf_cache, kpe_cache, pt, ref.kv_lens, SM_SCALE, ref.ckv_scale, ref.kpe_scale)
    want = mla.decode(*ref.args())
    assert torch.equal(out, want)
    assert mla.workspace_status() == 0


def test_writer_rejects_bad_tables():
    dev = "cuda"
    ps, P = 16, 4
    ckv_cache = torch.zeros(P, ps, 256, dtype=torch.uint8, device=dev)
    sf_cache = torch.zeros(P, ps, 32, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    kpe_cache = torch.zeros(P, ps, 64, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    ckv, kpe = torch.ones(2, 512, dtype=torch.bfloat16, device=dev), torch.ones(2, 64, dtype=torch.bfloat16, device=dev)
    kv_indices = torch.tensor([0, 9], dtype=torch.int32, device=dev)   # page 9 does not exist
    kv_indptr = torch.tensor([0, 2], dtype=torch.int32, device=dev)
    bi = torch.zeros(2, dtype=torch.int32, device=dev)
    pos = torch.tensor([3, 17], dtype=torch.int32, device=dev)         # second token lands on the missing page
    with pytest.raises(RuntimeError, match="outside the tables"):
        mla.quantize_append_paged_mla_kv_cache(ckv, kpe, bi, pos, ckv_cache, sf_cache, kpe_cache, kv_indices, kv_indptr,
                                               check=True)
    assert int(ckv_cache[0, 3].count_nonzero()) > 0 and int(ckv_cache[1:].count_nonzero()) == 0  # first written, second skipped
    with pytest.raises(RuntimeError, match="bfloat16"):
        mla.quantize_append_paged_mla_kv_cache(ckv.float(), kpe, bi, pos, ckv_cache, sf_cache, kpe_cache, kv_indices, kv_indptr)
    with pytest.raises(RuntimeError, match="int32"):
        mla.quantize_append_paged_mla_kv_cache(ckv, kpe, bi.long(), pos, ckv_cache, sf_cache, kpe_cache, kv_indices, kv_indptr)
