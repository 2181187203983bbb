"""Multi-GPU paths on real devices: two NCCL ranks (skipped on a box with fewer than two GPUs).

Sequence sharding: every rank holds a contiguous slice of each request's pages, decodes it with the normal split-KV
kernel in partial mode, and the (o, lse) pairs are merged with the library's combine kernels (peers' records read in place with the hand-shake in
the merge kernel or a barrier in front of it, or one all-gather); the result
must match whole-sequence attention (oracle) within the bf16-mode tolerances. Batch sharding: each rank decodes its own
requests; no collective."""
import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _local_slice(c, rank, world):
    """Local cache tensors, page table and lengths of `rank` for the sequence-sharded layout."""
    import nvfp4_mla_b200.dist as mdist
    ps = c.page_size
    B = len(c.kv_lens_list)
    parts = [mdist.shard_sequence(L, ps, world)[rank] for L in c.kv_lens_list]
    n_local = max(sum(n for _, n, _ in parts), 1)
    ckv = torch.zeros(n_local, ps, 256, dtype=torch.uint8)
    sf = torch.zeros(n_local, ps, 32, dtype=torch.uint8)
    kpe = torch.zeros(n_local, ps, 64, dtype=torch.uint8)
    pt = torch.zeros(B, max(max(n for _, n, _ in parts), 1), dtype=torch.int32)
    nxt = 0
    for b, (p0, n, _) in enumerate(parts):
        src = c.page_table[b, p0:p0 + n].long()
        ckv[nxt:nxt + n], sf[nxt:nxt + n], kpe[nxt:nxt + n] = c.ckv_cache[src], c.ckv_sf_cache.view(torch.uint8)[src], c.kpe_cache.view(torch.uint8)[src]
        pt[b, :n] = torch.arange(nxt, nxt + n, dtype=torch.int32)
        nxt += n
    lens = torch.tensor([t for _, _, t in parts], dtype=torch.int32)
    return ckv, sf.view(torch.float8_e4m3fn), kpe.view(torch.float8_e4m3fn), pt, lens


def _rank(rank, world, port, ret):
    import sys
    import pathlib
    root = pathlib.Path(__file__).resolve().parent.parent
    for p in (root, root / "oracle", root / "tests"):
        sys.path.insert(0, str(p))
    import torch.distributed as dist
    import nvfp4_mla_b200 as mla
    import nvfp4_mla_b200.dist as mdist
    from nvfp4_mla_b200.testing import SM_SCALE, SyntheticCache
    from util import oracle_reference
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = torch.device("cuda", rank)
        c = SyntheticCache([5000, 131, 64, 9000], 64, 16, 0.5, 2.0, seed=17)   # identical on every rank
        want, _ = oracle_reference(c)
        # ---- sequence sharded
        ckv, sf, kpe, pt, lens = [t.to(dev) for t in _local_slice(c, rank, world)]
        out = mdist.decode_sequence_sharded(c.q_nope.to(dev), c.q_pe.to(dev), ckv, sf, kpe, pt, lens, SM_SCALE, c.ckv_scale,
                                            c.kpe_scale, max_kv_len=int(lens.max()), out_dtype=torch.float32)
        torch.cuda.synchronize()
        err_seq = float(np.abs(out.cpu().numpy() - want).max())
        # the same through preallocated buffers, every way of merging: the peers' records read where they were written
        # (symmetric memory, hand-shake inside the merge kernel or as a barrier in front of it; falls back to the
        # collective by itself where that cannot be set up) and one packed all-gather per step. Five steps each: the
        # buffers are reused, the peer records alternate.
        modes = []
        for peer in (True, "barrier", False):
            mg = mdist.PartialMerger(len(c.kv_lens_list), 16, dev, peer=peer)
            modes.append(mg.mode)
            for step in range(5):
                if rank == step % world:
                    torch.cuda._sleep(2_000_000)  # about a millisecond: the ranks reach the merge at different times
                out = mdist.decode_sequence_sharded(c.q_nope.to(dev), c.q_pe.to(dev), ckv, sf, kpe, pt, lens, SM_SCALE, c.ckv_scale,
                                                    c.kpe_scale, max_kv_len=int(lens.max()), out_dtype=torch.float32, merger=mg)
                if step % 2:  # odd steps are queued behind the even ones without a host synchronisation in between
                    torch.cuda.synchronize()
                    mg.check()
                    err_seq = max(err_seq, float(np.abs(out.cpu().numpy() - want).max()))
            torch.cuda.synchronize()
            mg.check()
        if rank == 0:
            print("merge modes exercised:", modes)
        # ---- batch sharded: this rank's requests only
        mine = mdist.shard_batch(c.kv_lens_list, world)[rank]
        sub = SyntheticCache.__new__(SyntheticCache)
        sub.__dict__.update(vars(c))
        cg = sub.to(dev)
        idx = torch.tensor(mine, device=dev)
        out_b = mla.decode(cg.q_nope[idx], cg.q_pe[idx], cg.ckv_cache, cg.ckv_sf_cache, cg.kpe_cache, cg.page_table[idx].contiguous(),
                           cg.kv_lens[idx].contiguous(), SM_SCALE, c.ckv_scale, c.kpe_scale)
        torch.cuda.synchronize()
        err_batch = float(np.abs(out_b.float().cpu().numpy() - want[mine]).max()) if mine else 0.0
        ret[rank] = (err_seq, err_batch, mla.workspace_status())
    finally:
        dist.destroy_process_group()


def test_two_gpu_sequence_and_batch_sharding():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world, port = 2, _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_rank, args=(world, port, ret), nprocs=world, join=True)
        assert len(ret) == world
        for err_seq, err_batch, status in ret.values():
            assert status == 0
            assert err_seq <= 2e-2 and err_batch <= 2e-2, dict(ret)
