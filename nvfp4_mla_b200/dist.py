"""Multi-GPU use of the decode path: one process per GPU, ``torch.distributed`` for the plumbing.

Two shardings follow the path's natural units (the reference itself is single-GPU):

* **Batch sharding** (data parallel). Requests are independent, so each rank decodes its own requests against its own
  pages and nothing is exchanged. ``shard_batch`` assigns requests to ranks by token count, which matters for ragged
  batches.
* **Sequence sharding** for very long single contexts. The pages of every request are cut into contiguous ranges, one
  per rank; each rank runs the normal split-KV decode over its range in "partial" mode, producing for every
  (request, head) an output normalised by its own softmax sum and a log2-domain log-sum-exp, exactly the pair the
  in-GPU split merge consumes (reference contract: nvfp4_mla/csrc/mla_decode.cu:478-492). The pairs (513 KiB per GPU at
  B=2, H=128) are merged on every rank with the library's combine kernel, which reads the other GPUs' records over
  NVLink where they were written (symmetric memory; the ranks' hand-shake runs inside that kernel), or after one NCCL
  all-gather where that cannot be set up.
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

    A rank's partial result is one packed record ``[o (batch x heads x 512) | lse (batch x heads)]`` (float32) that the
    decode kernels write directly (``o`` and ``lse`` are views of it). Two ways to merge the ranks' records:

    * **peer reads** (default where it can be set up): the records live in symmetric memory, every rank maps every
      other rank's buffer, and the library's merge kernel reads the peers' records over NVLink with ordinary loads
      where their owners wrote them: no collective, no copy. The ranks' hand-shake ("my record of this step is
      written") runs inside the merge kernel itself (``nvfp4_mla_combine_records_signalled``: one flag word per pair of
      ranks in symmetric memory, a bounded wait), or, with ``peer="barrier"``, as symmetric memory's own barrier launched
      in front of the plain merge kernel. Two records alternate from step to step, so that a rank that is one step
      ahead never writes what a slower rank still reads (the hand-shake of step s + 1 is passed only when every rank
      has finished the merge of step s).
    * **all-gather** (``peer=False``, or when symmetric memory is unavailable: one GPU, a gloo group, an older torch):
      ONE ``all_gather_into_tensor`` of the record per step into ``recv [world, record]``, merged where it landed.

    The exchange is latency-bound either way (513 KiB per rank at B=2, H=128). ``check()`` synchronises and raises if a
    hand-shake ever ran out of time (a rank that never arrived)."""

    def __init__(self, batch, heads, device, group=None, peer=None, wait_us=10_000_000):
        import os
        self.group, self.rows, self.shape = group, batch * heads, (batch, heads)
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device)
        self.wait_us = wait_us
        n = self.rows * 513
        self.step, self.handles, self.flag_ptrs, self.status = 0, None, None, None
        if peer is None:
            env = os.environ.get("NVFP4_MLA_PEER_MERGE", "1")
            peer = False if env == "0" else ("barrier" if env == "barrier" else True)
        if peer and self.world > 1 and self.world <= 16 and self.device.type == "cuda":
            try:
                import torch.distributed._symmetric_memory as symm
                g = group if group is not None else dist.group.WORLD
                bufs = [symm.empty(n, dtype=torch.float32, device=self.device) for _ in range(2)]
                self.handles = [symm.rendezvous(b, g) for b in bufs]
                self.records = bufs
                self.peer_ptrs = [[int(h.buffer_ptrs[r]) for r in range(self.world)] for h in self.handles]
                if peer != "barrier":
                    self.flags = symm.empty(32, dtype=torch.int32, device=self.device)
                    self.flags.zero_()
                    fh = symm.rendezvous(self.flags, g)
                    self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
                    torch.cuda.synchronize(self.device)
                    dist.barrier(group)  # every rank's words are zero before anyone announces a step
                    self.flag_ptrs = [int(fh.buffer_ptrs[r]) for r in range(self.world)]
                    self._flag_handle = fh
            except Exception:  # no symmetric memory on this system / backend: the collective does the exchange
                self.handles, self.flag_ptrs = None, None
        if self.handles is None:
            self.records = [torch.empty(n, dtype=torch.float32, device=device)]
            self.recv = torch.empty(self.world, n, dtype=torch.float32, device=device)

    @property
    def mode(self):
        """How the ranks' records meet: "peer-signal", "peer-barrier" or "all-gather"."""
        if self.handles is None:
            return "all-gather"
        return "peer-signal" if self.flag_ptrs is not None else "peer-barrier"

    def check(self):
        """Synchronises and raises if a hand-shake of the in-kernel merge gave up waiting for another rank."""
        if self.status is not None:
            st = int(self.status.item())
            if st:
                raise RuntimeError(f"cross-GPU merge: status {st} (4 = a rank's record was not announced within {self.wait_us} us)")

    @property
    def send(self):
        """The record the current step's decode writes."""
        return self.records[self.step % len(self.records)]

    @property
    def o(self):
        return self.send[:self.rows * 512].view(*self.shape, 512)

    @property
    def lse(self):
        return self.send[self.rows * 512:].view(*self.shape)

    def merge(self, out_dtype=torch.bfloat16, combine_packed=None):
        """Merges the ranks' records of the current step; every rank returns the full ``[batch, heads, 512]`` result.
        ``combine_packed(recv, rows, out_dtype)`` replaces the library's kernel on the all-gather path (tests)."""
        if self.handles is not None and combine_packed is None:
            from . import combine_records, combine_records_signalled
            k = self.step % 2
            if self.flag_ptrs is not None:  # announce, wait and merge in one kernel
                out = combine_records_signalled(self.peer_ptrs[k], self.flag_ptrs, self.rank, self.step + 1, self.rows,
                                                self.device, out_dtype, self.status, self.wait_us)
            else:
                self.handles[k].barrier()  # every rank's record of this step is written and visible
                out = combine_records(self.peer_ptrs[k], self.rows, self.device, out_dtype)
            self.step += 1
            return out.view(*self.shape, 512)
        if combine_packed is None:
            from . import combine_packed  # the CUDA kernel; there is no host implementation
        if self.handles is not None:  # a caller-supplied merge on the peer set-up: gather the records first
            recv = torch.empty(self.world, self.rows * 513, dtype=torch.float32, device=self.device)
        else:
            recv = self.recv
        dist.all_gather_into_tensor(recv.view(-1), self.send, group=self.group)
        self.step += 1 if self.handles is not None else 0
        return combine_packed(recv, self.rows, out_dtype).view(*self.shape, 512)


def decode_sequence_sharded(q_nope, q_pe, ckv_cache, ckv_sf_cache, kpe_cache, page_table, kv_lens, sm_scale,
                            ckv_scale=1.0, kpe_scale=1.0, max_kv_len=None, num_splits=0, precision="bf16", group=None,
                            out_dtype=torch.bfloat16, merger=None):
    """Decode when each rank holds a contiguous slice of every request's KV.

    ``ckv_cache`` / ``ckv_sf_cache`` / ``kpe_cache`` / ``page_table`` / ``kv_lens`` describe the LOCAL slice (local page
    ids, local token counts; a rank may hold zero tokens of a request); the queries are replicated. Returns the full
    ``[batch, heads, 512]`` output on every rank. Pass a ``PartialMerger`` to reuse its buffers across steps (peer
    reads of the records, or one packed all-gather per step); without one the (o, lse) pair is gathered into fresh
    tensors."""
    from . import decode_partial
    if merger is not None:
        decode_partial(q_nope, q_pe, ckv_cache, ckv_sf_cache, kpe_cache, page_table, kv_lens, sm_scale, ckv_scale, kpe_scale,
                       max_kv_len, num_splits, precision, into=(merger.o, merger.lse))
        return merger.merge(out_dtype)
    o, lse = decode_partial(q_nope, q_pe, ckv_cache, ckv_sf_cache, kpe_cache, page_table, kv_lens, sm_scale, ckv_scale,
                            kpe_scale, max_kv_len, num_splits, precision)
    return merge_partials(o, lse, group, None, out_dtype)
