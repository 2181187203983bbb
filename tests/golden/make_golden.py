"""Regenerates tests/golden/*.npz from the reference project's own torch path.

Run where the reference project is checked out, with $NVFP4_MLA_REFERENCE pointing at it:

    NVFP4_MLA_REFERENCE=<path to elwhyjay/nvfp4-mla> python tests/golden/make_golden.py

Inputs come from nvfp4_mla_b200.testing.SyntheticCache on the CPU (bit-reproducible from the seed); outputs are
what the reference's nvfp4_mla.testing.dequantize / attention return for them on CPU tensors. Small cases store
their inputs; larger ones store a SHA-256 of the regenerated cache bytes and a strided sample of the output.
"""
import hashlib
import os
import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
if "NVFP4_MLA_REFERENCE" not in os.environ:
    raise SystemExit("set NVFP4_MLA_REFERENCE to a checkout of the reference project")
sys.path.insert(0, os.environ["NVFP4_MLA_REFERENCE"])

import nvfp4_mla.testing as ref  # noqa: E402  (the reference; needs flashinfer importable, no GPU)
from nvfp4_mla_b200.testing import SyntheticCache  # noqa: E402

# name -> (kv_lens, page_size, heads, ckv_scale, kpe_scale, seed, store_inputs, head_stride, chan_stride)
CASES = {
    "tiny":        ([21, 9], 8, 16, 0.37, 3.1, 1, True, 1, 1),
    "config0":     ([1000, 3000], 64, 16, None, None, 0, False, 1, 1),          # the CPU-runnable reference configuration (calibrated scales)
    "ps1_len1":    ([1], 1, 16, 0.5, 2.0, 2, True, 1, 1),
    "off_page":    ([17, 1, 64, 65], 16, 16, 0.5, 2.0, 3, False, 1, 1),
    "mixed":       ([1000, 4097, 3, 64], 64, 16, 0.5, 2.0, 4, False, 1, 2),
    "ps1_h128":    ([513, 2048], 1, 128, 0.5, 2.0, 5, False, 8, 4),
    "h128":        ([4096, 1, 777, 5000], 64, 128, 0.5, 2.0, 6, False, 8, 4),
    "around_tile": ([31, 33, 95, 97, 127, 128, 129, 255, 257], 16, 16, 0.5, 2.0, 7, False, 1, 2),
    "calibrated":  ([300, 70], 16, 16, 2.0 ** -9, 2.0 ** -6, 8, False, 1, 1),
}


def sha(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def main():
    torch.manual_seed(0)
    for name, (lens, ps, H, cs, ks, seed, store, hs, chs) in CASES.items():
        c = SyntheticCache(lens, ps, H, cs, ks, seed=seed, device="cpu")
        ckv, kpe = ref.dequantize(c.ckv_cache, c.ckv_sf_cache, c.kpe_cache, c.ckv_scale, c.kpe_scale)
        out = ref.attention(c.q_nope, c.q_pe, ckv, kpe, c.page_table, c.kv_lens, ref.SM_SCALE)
        d = dict(kv_lens=np.array(lens, np.int32), page_size=ps, heads=H, ckv_scale=c.ckv_scale,
                 kpe_scale=c.kpe_scale, seed=seed, head_stride=hs, chan_stride=chs,
                 out=out[:, ::hs, ::chs].numpy(),
                 input_sha=sha(c.q_nope, c.q_pe, c.ckv_cache, c.ckv_sf_cache, c.kpe_cache, c.page_table))
        if store:
            d.update(q_nope=c.q_nope.view(torch.int16).numpy(), q_pe=c.q_pe.view(torch.int16).numpy(),
                     ckv_cache=c.ckv_cache.numpy(), ckv_sf_cache=c.ckv_sf_cache.view(torch.uint8).numpy(),
                     kpe_cache=c.kpe_cache.view(torch.uint8).numpy(), page_table=c.page_table.numpy(),
                     deq_ckv_bits=ckv.view(torch.int32).numpy(), deq_kpe_bits=kpe.view(torch.int32).numpy())
        else:
            # dequantize is pinned on a sample of pages for the larger cases
            d.update(deq_pages=np.arange(min(2, ckv.shape[0])),
                     deq_ckv_bits=ckv[:2].view(torch.int32).numpy(), deq_kpe_bits=kpe[:2].view(torch.int32).numpy())
        np.savez_compressed(HERE / f"{name}.npz", **d)
        print(name, "out", tuple(out.shape), "stored", d["out"].shape, "ckv_scale", c.ckv_scale)


if __name__ == "__main__":
    main()
