"""Shared helpers of the test-suite: golden fixtures and conversions between torch tensors and the numpy oracle."""
import hashlib
import pathlib

import numpy as np
import torch

from nvfp4_mla_b200.testing import SyntheticCache

GOLDEN = pathlib.Path(__file__).resolve().parent / "golden"
GOLDEN_NAMES = sorted(p.stem for p in GOLDEN.glob("*.npz"))


def sha(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def load_golden(name):
    """Returns (fixture dict, SyntheticCache regenerated on the CPU from the fixture's seed)."""
    g = dict(np.load(GOLDEN / f"{name}.npz", allow_pickle=False))
    c = SyntheticCache(g["kv_lens"].tolist(), int(g["page_size"]), int(g["heads"]), float(g["ckv_scale"]),
                       float(g["kpe_scale"]), seed=int(g["seed"]), device="cpu")
    got = sha(c.q_nope, c.q_pe, c.ckv_cache, c.ckv_sf_cache, c.kpe_cache, c.page_table)
    assert got == str(g["input_sha"]), f"regenerated inputs of golden case {name!r} differ from the recorded ones"
    return g, c


def np_inputs(c):
    """SyntheticCache (CPU) -> numpy arrays in the oracle's conventions (q as float32, caches as uint8)."""
    return dict(q_nope=c.q_nope.float().numpy(), q_pe=c.q_pe.float().numpy(), ckv_cache=c.ckv_cache.numpy(),
                ckv_sf_cache=c.ckv_sf_cache.view(torch.uint8).numpy(), kpe_cache=c.kpe_cache.view(torch.uint8).numpy(),
                page_table=c.page_table.numpy(), kv_lens=c.kv_lens.numpy())


def oracle_reference(c, sm_scale=None, return_lse=True):
    """Oracle output (fp32 out, natural-log lse) for a SyntheticCache living on any device."""
    import mla_oracle as O
    cpu = SyntheticCache.__new__(SyntheticCache)
    cpu.__dict__.update({k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in vars(c).items()})
    a = np_inputs(cpu)
    ckv, kpe = O.dequantize(a["ckv_cache"], a["ckv_sf_cache"], a["kpe_cache"], c.ckv_scale, c.kpe_scale)
    return O.attention(a["q_nope"], a["q_pe"], ckv, kpe, a["page_table"], a["kv_lens"],
                       O.SM_SCALE if sm_scale is None else sm_scale, return_lse=return_lse)
