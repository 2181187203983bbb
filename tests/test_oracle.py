"""CPU tests: the numpy oracle against the golden vectors produced by the reference's own torch path, and the
package's torch cache writer against the oracle's numpy one."""
import numpy as np
import pytest
import torch

import mla_oracle as O
from nvfp4_mla_b200 import testing as T
from util import GOLDEN_NAMES, load_golden, np_inputs


@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_oracle_dequantize_bitwise_vs_reference(name):
    g, c = load_golden(name)
    a = np_inputs(c)
    ckv, kpe = O.dequantize(a["ckv_cache"], a["ckv_sf_cache"], a["kpe_cache"], c.ckv_scale, c.kpe_scale)
    if "deq_pages" in g:
        ckv, kpe = ckv[g["deq_pages"]], kpe[g["deq_pages"]]
    for got, want_bits in ((ckv, g["deq_ckv_bits"]), (kpe, g["deq_kpe_bits"])):
        want = want_bits.view(np.float32)
        assert np.array_equal(np.isnan(got), np.isnan(want))
        ok = ~np.isnan(want)
        assert np.array_equal(got.view(np.int32)[ok], want_bits[ok])


@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_oracle_attention_vs_reference(name):
    g, c = load_golden(name)
    a = np_inputs(c)
    ckv, kpe = O.dequantize(a["ckv_cache"], a["ckv_sf_cache"], a["kpe_cache"], c.ckv_scale, c.kpe_scale)
    out, lse = O.attention(a["q_nope"], a["q_pe"], ckv, kpe, a["page_table"], a["kv_lens"], O.SM_SCALE, return_lse=True)
    want = g["out"]
    got = out[:, ::int(g["head_stride"]), ::int(g["chan_stride"])]
    assert not np.isnan(got).any() and np.isfinite(lse).all()
    assert np.abs(got - want).max() <= 2e-6 * max(1.0, np.abs(want).max())


def test_torch_helpers_match_oracle():
    """nvfp4_mla_b200.testing.dequantize / attention (torch) against the oracle on a stored-input case."""
    g, c = load_golden("tiny")
    ckv_t, kpe_t = c.dequantize()
    assert np.array_equal(ckv_t.view(torch.int32).numpy()[~np.isnan(ckv_t.numpy())],
                          g["deq_ckv_bits"][~np.isnan(ckv_t.numpy())])
    out, lse = c.reference(return_lse=True)
    a = np_inputs(c)
    ckv, kpe = O.dequantize(a["ckv_cache"], a["ckv_sf_cache"], a["kpe_cache"], c.ckv_scale, c.kpe_scale)
    o2, l2 = O.attention(a["q_nope"], a["q_pe"], ckv, kpe, a["page_table"], a["kv_lens"], return_lse=True)
    assert np.abs(out.numpy() - o2).max() < 2e-6 and np.abs(lse.numpy() - l2).max() < 2e-6
    o3, l3 = T.attention_paged_nvfp4(*c.args(), chunk_pages=2)
    assert np.abs(o3.numpy() - o2).max() < 2e-6 and np.abs(l3.numpy() - l2).max() < 2e-6


def test_stored_inputs_match_regenerated():
    g, c = load_golden("tiny")
    assert np.array_equal(g["ckv_cache"], c.ckv_cache.numpy())
    assert np.array_equal(g["page_table"], c.page_table.numpy())
    assert np.array_equal(g["q_nope"], c.q_nope.view(torch.int16).numpy())


def test_e4m3_codec_vs_torch():
    t = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    ok = ~np.isnan(t)
    assert np.array_equal(np.isnan(t), np.isnan(O.E4M3_LUT)) and np.array_equal(t[ok], O.E4M3_LUT[ok])
    rng = np.random.default_rng(0)
    x = np.clip(rng.standard_normal(100000) * np.exp(3 * rng.standard_normal(100000)), -448, 448).astype(np.float32)
    assert np.array_equal(O.e4m3_encode(x), torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy())


@pytest.mark.parametrize("scale", [1.0, 0.37, 2.0 ** -9])
def test_writer_torch_vs_oracle(scale):
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(257, 512, generator=g) * (scale * 300)).bfloat16().float()
    x[5] = 0
    packed, sf = T.quantize_ckv(x, scale)
    p2, s2 = O.quantize_ckv(x.numpy(), scale)
    assert np.array_equal(packed.numpy(), p2) and np.array_equal(sf.view(torch.uint8).numpy(), s2)
    k = torch.randn(100, 64, generator=g).bfloat16().float()
    assert np.array_equal(T.quantize_kpe(k, 0.01).view(torch.uint8).numpy(), O.quantize_kpe(k.numpy(), 0.01))


def test_writer_error_band():
    """NVFP4 vs the unquantized BF16 cache on config 0's shape: the reference reports 0.08-0.14 rel-L2."""
    c = T.SyntheticCache([1000, 3000], 64, 16, None, None, seed=0, keep_bf16=True)
    err = T.rel_l2(c.reference(), c.reference_bf16())
    assert 0.05 < err < 0.2


def test_partial_and_combine_identity():
    """Splitting the KV range and merging (o, lse) pairs reproduces whole-range attention; empty splits weigh 0."""
    g, c = load_golden("off_page")
    a = np_inputs(c)
    ckv, kpe = O.dequantize(a["ckv_cache"], a["ckv_sf_cache"], a["kpe_cache"], c.ckv_scale, c.kpe_scale)
    args = (a["q_nope"], a["q_pe"], ckv, kpe, a["page_table"], a["kv_lens"], O.SM_SCALE)
    whole, lse = O.attention(*args, return_lse=True)
    parts = [O.attention_partial(*args, lo, lo + 24) for lo in range(0, 96, 24)]
    out, lse2 = O.combine(np.stack([p[0] for p in parts]), np.stack([p[1] for p in parts]))
    assert np.abs(out - whole).max() < 2e-6
    assert np.abs(lse2 / O.LOG2E - lse).max() < 2e-6


def test_fp8_model_error_budget():
    """The fp8 arithmetic model stays inside the reference's fp8 bound (rel-L2 < 0.08) on both scale regimes."""
    for cs, ks in ((0.5, 2.0), (2.0 ** -9, 2.0 ** -6)):
        c = T.SyntheticCache([300, 70], 16, 16, cs, ks, seed=8)
        a = np_inputs(c)
        ckv, kpe = O.dequantize(a["ckv_cache"], a["ckv_sf_cache"], a["kpe_cache"], cs, ks)
        want = O.attention(a["q_nope"], a["q_pe"], ckv, kpe, a["page_table"], a["kv_lens"])
        got = O.attention_fp8_model(a["q_nope"], a["q_pe"], a["ckv_cache"], a["ckv_sf_cache"], a["kpe_cache"],
                                    a["page_table"], a["kv_lens"], O.SM_SCALE, cs, ks)
        assert O.rel_l2(got, want) < 0.08
