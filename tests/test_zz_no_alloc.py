"""The allocation-free decode entry point, called through the C ABI.

``nvfp4_mla_decode_static`` is for hosts that cannot give the library scratch memory at decode time (a server that has
already reserved the whole GPU for its own pool, a plugin that only receives its input and output buffers): it runs
the same kernels as ``nvfp4_mla_decode`` but keeps their scratch in a fixed array inside the library. This test
drives it with ctypes, twice in a row with different lengths so that the second call runs over what the first one
left in the array, and compares each result with the regular entry point's AND with the CPU oracle (tolerances of the
decode tests: max-abs <= 2e-2 and LSE <= 1e-3 in the 16-bit mode, rel-L2 < 0.08 in the 8-bit mode). The 8-bit mode is
covered at 16 and at 128 heads: there the regular entry point groups 128 heads per CTA pair, whose partial results
do not fit the built-in array, and the static one has to fall back to a narrower grouping. Collected last so that a
failure here cannot hide another test's result.
"""
import math

import numpy as np
import pytest
import torch

import mla_oracle as O
import nvfp4_mla_b200 as mla
from nvfp4_mla_b200 import _lib
from nvfp4_mla_b200.testing import SM_SCALE, SyntheticCache
from util import oracle_reference

pytestmark = pytest.mark.gpu
LN2 = math.log(2.0)


def decode_static(lib, c, kv_lens, max_kv_len, num_splits=0, precision=0):
    B, H = c.q_nope.shape[:2]
    out = torch.empty(B, H, 512, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(B, H, dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.nvfp4_mla_decode_static(
        c.q_nope.data_ptr(), c.q_pe.data_ptr(), c.ckv_cache.data_ptr(), c.ckv_sf_cache.data_ptr(), c.kpe_cache.data_ptr(),
        c.ckv_cache.shape[0], c.page_size, c.page_table.data_ptr(), c.page_table.stride(0), kv_lens.data_ptr(), B, H,
        SM_SCALE, c.ckv_scale, c.kpe_scale, max_kv_len, num_splits, precision, out.data_ptr(), None, lse.data_ptr(), stream)
    assert rc == 0, lib.nvfp4_mla_last_error().decode()
    return out, lse


def with_lengths(c, lens):
    """A view of cache `c` whose requests are `lens` tokens long (a prefix of what was written)."""
    v = SyntheticCache.__new__(SyntheticCache)
    v.__dict__.update(vars(c))
    v.kv_lens_list = list(lens)
    v.kv_lens = torch.tensor(lens, dtype=torch.int32, device=c.kv_lens.device)
    return v


def test_static_scratch_matches_regular_entry_point_twice():
    lib = _lib.load()
    assert lib.nvfp4_mla_decode_static_capacity() == 9 << 20
    c = SyntheticCache([3000, 1500, 700, 4096], 64, 16, 0.5, 2.0, seed=31).to("cuda")
    for lens, splits in (([3000, 1500, 700, 4096], 0), ([129, 1, 640, 2000], 3)):  # second call: shorter, extra splits
        v = with_lengths(c, lens)
        want = mla.decode(*v.args(), max_kv_len=4096, num_splits=splits)
        _, want_lse = mla.decode_partial(*v.args(), max_kv_len=4096, num_splits=splits)
        got, got_lse = decode_static(lib, v, v.kv_lens, 4096, splits)
        torch.cuda.synchronize()
        assert lib.nvfp4_mla_decode_static_status(None) == 0
        assert not got.isnan().any()
        assert (got.float() - want.float()).abs().max().item() <= 2e-2
        assert (got_lse - want_lse).abs().max().item() <= 1e-3
        ref, ref_lse = oracle_reference(v)
        assert np.abs(got.float().cpu().numpy() - ref).max() <= 2e-2
        assert np.abs(got_lse.cpu().numpy() * LN2 - ref_lse).max() <= 1e-3


@pytest.mark.parametrize("heads", [16, 128])
def test_static_scratch_8bit_mode(heads):
    """8-bit mode, two calls in a row; at 128 heads the static entry point runs a narrower head grouping than the
    regular one (another kernel), so both are held against the oracle with the mode's own bound."""
    lib = _lib.load()
    c = SyntheticCache([2000, 300, 4096, 65], 64, heads, 2.0 ** -9, 2.0 ** -6, seed=32).to("cuda")
    for lens, splits in (([2000, 300, 4096, 65], 0), ([1, 300, 1000, 64], 2)):
        v = with_lengths(c, lens)
        want = mla.decode(*v.args(), max_kv_len=4096, num_splits=splits, precision="fp8")
        got, _ = decode_static(lib, v, v.kv_lens, 4096, splits, precision=1)
        torch.cuda.synchronize()
        assert lib.nvfp4_mla_decode_static_status(None) == 0
        assert not got.isnan().any()
        ref, _ = oracle_reference(v)
        assert O.rel_l2(got.float().cpu().numpy(), ref) < 0.08
        assert O.rel_l2(want.float().cpu().numpy(), ref) < 0.08
        assert O.rel_l2(got.float().cpu().numpy(), want.float().cpu().numpy()) < 0.08


def test_static_scratch_rejects_oversized_problems():
    lib = _lib.load()
    c = SyntheticCache([64] * 4, 64, 16, seed=1).to("cuda")
    out = torch.empty(4, 16, 512, dtype=torch.bfloat16, device="cuda")
    rc = lib.nvfp4_mla_decode_static(
        c.q_nope.data_ptr(), c.q_pe.data_ptr(), c.ckv_cache.data_ptr(), c.ckv_sf_cache.data_ptr(), c.kpe_cache.data_ptr(),
        c.ckv_cache.shape[0], c.page_size, c.page_table.data_ptr(), c.page_table.stride(0), c.kv_lens.data_ptr(), 4, 16,
        SM_SCALE, 1.0, 1.0, 64, 200, 0, out.data_ptr(), None, None, None)   # 4 x 1 x 200 items: over the capacity
    assert rc != 0
    assert "too large for the built-in scratch" in lib.nvfp4_mla_last_error().decode()
