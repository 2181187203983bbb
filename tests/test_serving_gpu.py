"""GPU tests of the callers around the decode path: multi-token (MTP / speculative verify) decode and the paged
latent-KV pool (append through the CUDA writer, decode, W_UV). Checked against the numpy oracle per query position."""
import numpy as np
import pytest
import torch

import mla_oracle as O
import nvfp4_mla_b200 as mla
from nvfp4_mla_b200 import serving
from nvfp4_mla_b200.testing import SM_SCALE, SyntheticCache
from util import oracle_reference

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("precision,tol", [("bf16", 4e-3), ("fp8", 0.08)])
def test_multi_token_decode_matches_oracle_per_position(precision, tol):
    kv_lens, ps, H, Q = [300, 2, 129, 1], 64, 16, 3
    c = SyntheticCache(kv_lens, ps, H, 0.5, 2.0, seed=11, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(1)
    q_nope = torch.randn(len(kv_lens), Q, H, 512, generator=g, device="cuda").bfloat16()
    q_pe = torch.randn(len(kv_lens), Q, H, 64, generator=g, device="cuda").bfloat16()
    out = serving.decode_multi_token(q_nope, q_pe, c.ckv_cache, c.ckv_sf_cache, c.kpe_cache, c.page_table, c.kv_lens, SM_SCALE,
                                     c.ckv_scale, c.kpe_scale, max_kv_len=max(kv_lens), precision=precision)
    assert out.shape == (len(kv_lens), Q, H, 512)
    for i in range(Q):
        lens_i = [max(L - (Q - 1 - i), 0) for L in kv_lens]
        ci = SyntheticCache.__new__(SyntheticCache)
        ci.__dict__.update(vars(c))
        ci.q_nope, ci.q_pe = q_nope[:, i].contiguous(), q_pe[:, i].contiguous()
        ci.kv_lens, ci.kv_lens_list = torch.tensor(lens_i, dtype=torch.int32), lens_i
        want, _ = oracle_reference(ci)
        got = out[:, i].float().cpu().numpy()
        live = [b for b, L in enumerate(lens_i) if L > 0]
        assert O.rel_l2(got[live], want[live]) < tol, (precision, i)
        for b, L in enumerate(lens_i):
            if L == 0:
                assert (got[b] == 0).all()
    assert mla.workspace_status() == 0


def test_pool_append_decode_loop():
    """Two requests: prefill different lengths, then decode steps that append one token each; every step's output
    must equal decode over a cache written in one go from the same rows, and W_UV must equal the einsum."""
    dev, ps, H = "cuda", 16, 16
    g = torch.Generator(device=dev).manual_seed(2)
    pool = serving.PagedLatentCache(num_pages=64, page_size=ps, max_requests=4, max_pages_per_request=16, ckv_scale=0.01,
                                    kpe_scale=0.02, device=dev)
    rows = {r: (torch.randn(120, 512, generator=g, device=dev).bfloat16(), (torch.randn(120, 64, generator=g, device=dev) * 2).bfloat16())
            for r in (0, 2)}
    have = {0: 37, 2: 81}
    pool.append([(0, 37), (2, 81)], torch.cat([rows[0][0][:37], rows[2][0][:81]]), torch.cat([rows[0][1][:37], rows[2][1][:81]]))
    w_uv = torch.randn(H, 512, 128, generator=g, device=dev).bfloat16()
    for step in range(20):
        new = [(r, 1) for r in (0, 2)]
        pool.append(new, torch.cat([rows[r][0][have[r]:have[r] + 1] for r in (0, 2)]),
                    torch.cat([rows[r][1][have[r]:have[r] + 1] for r in (0, 2)]))
        for r in (0, 2):
            have[r] += 1
        q_nope = torch.randn(2, H, 512, generator=g, device=dev).bfloat16()
        q_pe = torch.randn(2, H, 64, generator=g, device=dev).bfloat16()
        out = pool.decode([0, 2], q_nope, q_pe, SM_SCALE)
        # oracle over the pool's own bytes
        ckv, kpe = O.dequantize(pool.ckv_cache.cpu().numpy(), pool.ckv_sf_cache.view(torch.uint8).cpu().numpy(),
                                pool.kpe_cache.view(torch.uint8).cpu().numpy(), pool.ckv_scale, pool.kpe_scale)
        want = O.attention(q_nope.float().cpu().numpy(), q_pe.float().cpu().numpy(), ckv, kpe,
                           pool.page_table[[0, 2]].cpu().numpy(), np.array([have[0], have[2]], np.int32), O.SM_SCALE)
        assert np.abs(out.float().cpu().numpy() - want).max() <= 2e-2, step
        # and the bytes equal the oracle writer's, row by row
        if step in (0, 19):
            for r in (0, 2):
                packed, sf8 = O.quantize_ckv(rows[r][0][:have[r]].float().cpu().numpy(), pool.ckv_scale)
                t = torch.arange(have[r])
                pages = pool.page_table[r].cpu()[t // ps].long()
                assert np.array_equal(pool.ckv_cache.cpu()[pages, t % ps].numpy(), packed), (step, r)
                assert np.array_equal(pool.ckv_sf_cache.view(torch.uint8).cpu()[pages, t % ps].numpy(), sf8), (step, r)
    v = pool.decode([0, 2], q_nope, q_pe, SM_SCALE, w_uv=w_uv)
    assert torch.allclose(v.float(), torch.einsum("bhc,hcv->bhv", out, w_uv).float(), rtol=2e-2, atol=2e-2)
    used = pool.free_pages
    pool.release(0)
    assert pool.free_pages == used + -(-have[0] // ps) and int(pool.kv_lens[0]) == 0
    with pytest.raises(RuntimeError, match="out of cache pages"):
        pool.append([(1, 64 * ps + 1)], torch.zeros(64 * ps + 1, 512, dtype=torch.bfloat16, device=dev),
                    torch.zeros(64 * ps + 1, 64, dtype=torch.bfloat16, device=dev))
    assert mla.workspace_status() == 0
