"""Host-side logic of the multi-GPU paths on CPU: world_size-2 gloo ranks exchange oracle partials and merge them.

The merge itself runs in the library's CUDA kernel on a GPU box; here a torch restatement of the same formula stands
in for it, so that what is tested is the sharding arithmetic and the gather plumbing of nvfp4_mla_b200.dist."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import mla_oracle as O
from nvfp4_mla_b200 import dist as mdist
from nvfp4_mla_b200.testing import SyntheticCache
from util import np_inputs


def torch_combine(o_part, lse_part, out_dtype):
    M = lse_part.max(0).values
    w = torch.where(torch.isneginf(lse_part), torch.zeros_like(lse_part),
                    torch.exp2(lse_part - torch.where(torch.isneginf(M), torch.zeros_like(M), M)))
    den = w.sum(0)
    out = (w[..., None] * o_part).sum(0) / den.clamp_min(1e-38)[..., None]
    return torch.where(den[..., None] > 0, out, torch.zeros_like(out)).to(out_dtype)


def test_shard_batch_balances_tokens():
    lens = [32768, 1024, 9000, 20000, 4096, 30000, 2048, 15000]
    shards = mdist.shard_batch(lens, 4)
    assert sorted(sum(shards, [])) == list(range(len(lens)))
    loads = [sum(lens[b] for b in s) for s in shards]
    assert max(loads) - min(loads) <= max(lens)
    assert mdist.shard_batch([5, 5], 4)[2:] == [[], []]


def test_shard_sequence_covers_every_token_once():
    for kv_len, ps, world in [(1048576, 64, 8), (1000, 64, 4), (63, 64, 2), (0, 64, 2), (129, 1, 3)]:
        parts = mdist.shard_sequence(kv_len, ps, world)
        assert sum(t for _, _, t in parts) == kv_len
        nxt = 0
        for p0, n, t in parts:
            assert p0 == nxt or n == 0
            nxt = p0 + n if n else nxt
            assert 0 <= t <= n * ps


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lens = [300, 77, 129]
        c = SyntheticCache(lens, 16, 16, 0.5, 2.0, seed=13)
        a = np_inputs(c)
        ckv, kpe = O.dequantize(a["ckv_cache"], a["ckv_sf_cache"], a["kpe_cache"], c.ckv_scale, c.kpe_scale)
        args = (a["q_nope"], a["q_pe"], ckv, kpe, a["page_table"], a["kv_lens"], O.SM_SCALE)
        # this rank's contiguous token range of every request (page aligned, as shard_sequence cuts it)
        o = np.zeros((len(lens), 16, 512), np.float32)
        lse = np.full((len(lens), 16), -np.inf, np.float32)
        for b, L in enumerate(lens):
            p0, n, t = mdist.shard_sequence(L, 16, world)[rank]
            ob, lb = O.attention_partial(*args, p0 * 16, p0 * 16 + t)
            o[b], lse[b] = ob[b], lb[b]
        out = mdist.merge_partials(torch.from_numpy(o), torch.from_numpy(lse), None, torch_combine, torch.float32)
        want = O.attention(*args)
        err = float(np.abs(out.numpy() - want).max())
        # the packed path: the partial is written into the merger's send record, one all-gather, merge from the records
        mg = mdist.PartialMerger(len(lens), 16, "cpu")
        mg.o.copy_(torch.from_numpy(o)), mg.lse.copy_(torch.from_numpy(lse))

        def packed_combine(recv, rows, out_dtype):
            return torch_combine(recv[:, :rows * 512].reshape(-1, rows, 512), recv[:, rows * 512:], out_dtype)
        out2 = mg.merge(torch.float32, packed_combine)
        ret[rank] = max(err, float(np.abs(out2.numpy() - want).max()))
    finally:
        dist.destroy_process_group()


def test_sequence_sharded_merge_two_ranks():
    world, port = 2, _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_rank, args=(world, port, ret), nprocs=world, join=True)
        assert len(ret) == world and all(v < 5e-6 for v in ret.values()), dict(ret)
