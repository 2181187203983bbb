"""Multi-GPU use of the decode path: one process per GPU, ``torch.distributed`` for the plumbing.

Two shardings follow the path's natural units (the reference itself is single-GPU):

* **Batch sharding** (data parallel). Requests are independent, so each rank decodes its own requests against its own
  pages and nothing is exchanged. ``shard_batch`` assigns requests to ranks by token count, which matters for ragged
  batches.
* **Sequence sharding** for very long single contexts. The pages of every request are cut into contiguous ranges, one
  per rank; each rank runs the normal split-KV decode over its range in "partial" mode, producing for every
  (request, head) an output normalised by its own softmax sum and a log2-domain log-sum-exp, exactly the pair the
  in-GPU split merge consumes (reference contract: nvfp4_mla/csrc/mla_decode.cu:478-492). The pairs (513 KiB per GPU at
  B=2, H=128) are all-gathered over NCCL / NVLink and merged on every rank with the library's combine kernel.
"""
import math

import torch
import torch.distributed as dist


def shard_batch(kv_lens, world_size):
    """Greedy longest-first assignment of requests to ranks balancing the token count.

    Returns a list of ``world_size`` lists of request indices (each sorted ascending)."""
    loads = [0] * world_size
    shards = [[] for _ in range(world_size)]
    for b in sorted(range(len(kv_lens)), key=lambda i: -int(kv_lens[i])):
        r = min(range(world_size), key=lambda i: (loads[i], i))
        shards[r].append(b)
        loads[r] += int(kv_lens[b])
    return [sorted(s) for s in shards]


def shard_sequence(kv_len, page_size, world_size):
    """Cuts a request of ``kv_len`` tokens into ``world_size`` contiguous page ranges of near-equal size.

    Returns a list of ``(first_page, n_pages, n_tokens)`` per rank; trailing ranks may be empty."""
    n_pages = math.ceil(kv_len / page_size)
    per = math.ceil(n_pages / world_size) if n_pages else 0
    out = []
    for r in range(world_size):
        p0 = min(r * per, n_pages)
        p1 = min(p0 + per, n_pages)
        tokens = max(0, min(kv_len, p1 * page_size) - p0 * page_size)
        out.append((p0, p1 - p0, tokens))
    return out


def merge_partials(o, lse, group=None, combine=None, out_dtype=torch.bfloat16):
    """All-gathers this rank's partial ``(o [..., 512] float32, lse [...] float32 log2 units)`` over ``group`` and merges
    them. ``combine(o_part [ranks, ..., 512], lse_part [ranks, ...], out_dtype)`` defaults to the library's kernel.
    Every rank returns the full result."""
    world = dist.get_world_size(group)
    o_all = torch.empty((world,) + tuple(o.shape), dtype=o.dtype, device=o.device)
    lse_all = torch.empty((world,) + tuple(lse.shape), dtype=lse.dtype, device=lse.device)
    dist.all_gather_into_tensor(o_all.view(-1), o.contiguous().view(-1), group=group)  # flat: rank r's record is slice r
    dist.all_gather_into_tensor(lse_all.view(-1), lse.contiguous().view(-1), group=group)
    if combine is None:
        from . import combine as combine  # the CUDA kernel; there is no host implementation
    return combine(o_all, lse_all, out_dtype)


class PartialMerger:
    """Buffers of the cross-GPU merge, allocated once and reused by every decode step.

    ``send`` is this rank's packed record ``[o (batch x heads x 512) | lse (batch x heads)]`` (float32); the decode
    kernels write their partial result straight into it (``o`` and ``lse`` are views). ``recv [world, record]`` is the
    target of ONE ``all_gather_into_tensor`` per step (the exchange is latency-bound: 513 KiB per rank at B=2, H=128),
    and the library's combine kernel merges the records where they landed."""

    def __init__(self, batch, heads, device, group=None):
        self.group, self.rows = group, batch * heads
        self.world = dist.get_world_size(group)
        n = self.rows * 513
        self.send = torch.empty(n, dtype=torch.float32, device=device)
        self.recv = torch.empty(self.world, n, dtype=torch.float32, device=device)
        self.o = self.send[:self.rows * 512].view(batch, heads, 512)
        self.lse = self.send[self.rows * 512:].view(batch, heads)

    def merge(self, out_dtype=torch.bfloat16, combine_packed=None):
        """One all-gather, one merge kernel. ``combine_packed(recv, rows, out_dtype)`` defaults to the library's kernel."""
        if combine_packed is None:
            from . import combine_packed  # the CUDA kernel; there is no host implementation
        dist.all_gather_into_tensor(self.recv.view(-1), self.send, group=self.group)
        return combine_packed(self.recv, self.rows, out_dtype).view(*self.o.shape)


def decode_sequence_sharded(q_nope, q_pe, ckv_cache, ckv_sf_cache, kpe_cache, page_table, kv_lens, sm_scale,
                            ckv_scale=1.0, kpe_scale=1.0, max_kv_len=None, num_splits=0, precision="bf16", group=None,
                            out_dtype=torch.bfloat16, merger=None):
    """Decode when each rank holds a contiguous slice of every request's KV.

    ``ckv_cache`` / ``ckv_sf_cache`` / ``kpe_cache`` / ``page_table`` / ``kv_lens`` describe the LOCAL slice (local page
    ids, local token counts; a rank may hold zero tokens of a request); the queries are replicated. Returns the full
    ``[batch, heads, 512]`` output on every rank. Pass a ``PartialMerger`` to reuse its buffers across steps (one
    packed all-gather per step); without one the (o, lse) pair is gathered into fresh tensors."""
    from . import decode_partial
    if merger is not None:
        decode_partial(q_nope, q_pe, ckv_cache, ckv_sf_cache, kpe_cache, page_table, kv_lens, sm_scale, ckv_scale, kpe_scale,
                       max_kv_len, num_splits, precision, into=(merger.o, merger.lse))
        return merger.merge(out_dtype)
    o, lse = decode_partial(q_nope, q_pe, ckv_cache, ckv_sf_cache, kpe_cache, page_table, kv_lens, sm_scale, ckv_scale,
                            kpe_scale, max_kv_len, num_splits, precision)
    return merge_partials(o, lse, group, None, out_dtype)
