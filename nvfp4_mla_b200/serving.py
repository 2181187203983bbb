"""The callers either side of the decode path, as a serving engine would use them: a paged latent-KV pool that appends
through the CUDA cache writer and decodes through the decode kernel, multi-token (speculative / MTP verify) decode, and
the W_UV projection after the latent output.

The reference lists these as what comes next around its kernel (README.md:88, 118-119, 414-415 of the reference
project): it has none of them, so there is no reference code to mirror; the arithmetic is the decode path's own and is
checked against the oracle per query position.
"""
import torch

from . import CKV, KPE, decode, get_batch_indices_positions, quantize_append_paged_mla_kv_cache


def decode_multi_token(q_nope, q_pe, ckv_cache, ckv_sf_cache, kpe_cache, page_table, kv_lens, sm_scale,
                       ckv_scale=1.0, kpe_scale=1.0, max_kv_len=None, num_splits=0, precision="bf16"):
    """Decode ``Q`` query tokens per request against one cache (speculative or multi-token-prediction verify).

    ``q_nope [batch, Q, heads, 512]``, ``q_pe [batch, Q, heads, 64]``; ``kv_lens [batch]`` counts the tokens in the
    cache INCLUDING the ``Q`` new ones, which are its last ``Q`` positions. Query ``i`` attends causally to the first
    ``kv_lens - (Q - 1 - i)`` tokens. Returns ``[batch, Q, heads, 512]`` bfloat16.

    Each query position runs as a request of its own that shares the original's pages (its row of the page table is
    repeated), so the launch shape stays fixed by ``max_kv_len`` and nothing synchronises; the ``Q`` reads of a request's
    cache are scheduled next to each other and the later ones are served from L2.
    """
    if q_nope.dim() != 4 or q_pe.dim() != 4:
        raise RuntimeError("q_nope must be [batch, Q, heads, 512] and q_pe [batch, Q, heads, 64]")
    B, Q, H = q_nope.shape[:3]
    if tuple(q_pe.shape) != (B, Q, H, KPE) or q_nope.shape[3] != CKV:
        raise RuntimeError("q_nope must be [batch, Q, heads, 512] and q_pe [batch, Q, heads, 64]")
    if kv_lens.dim() != 1 or kv_lens.shape[0] != B or kv_lens.dtype != torch.int32:
        raise RuntimeError("kv_lens must be int32 [batch]")
    back = torch.arange(Q - 1, -1, -1, dtype=torch.int32, device=kv_lens.device)  # Q-1 .. 0 tokens not yet visible
    lens = (kv_lens[:, None] - back[None, :]).clamp_(min=0).reshape(B * Q).contiguous()
    table = page_table.repeat_interleave(Q, dim=0).contiguous()
    out = decode(q_nope.reshape(B * Q, H, CKV).contiguous(), q_pe.reshape(B * Q, H, KPE).contiguous(), ckv_cache,
                 ckv_sf_cache, kpe_cache, table, lens, sm_scale, ckv_scale, kpe_scale, max_kv_len, num_splits, precision)
    return out.view(B, Q, H, CKV)


class PagedLatentCache:
    """A fixed pool of NVFP4 latent-KV pages with per-request page lists: what a serving engine keeps per layer.

    Pages are handed out on the host (a free list), the page table and lengths live on the device, and every append
    goes through the CUDA cache writer. ``max_pages_per_request`` fixes the page-table width, ``max_kv_len`` the decode
    launch shape, so a decode step can be captured in a CUDA graph once the pages of the step have been reserved.
    """

    def __init__(self, num_pages, page_size, max_requests, max_pages_per_request, ckv_scale, kpe_scale, device="cuda"):
        dev = torch.device(device)
        self.page_size, self.ckv_scale, self.kpe_scale = page_size, float(ckv_scale), float(kpe_scale)
        self.ckv_cache = torch.zeros(num_pages, page_size, CKV // 2, dtype=torch.uint8, device=dev)
        self.ckv_sf_cache = torch.zeros(num_pages, page_size, CKV // 16, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        self.kpe_cache = torch.zeros(num_pages, page_size, KPE, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        self.page_table = torch.zeros(max_requests, max_pages_per_request, dtype=torch.int32, device=dev)
        self.kv_lens = torch.zeros(max_requests, dtype=torch.int32, device=dev)
        self.max_kv_len = max_pages_per_request * page_size
        self._free = list(range(num_pages - 1, -1, -1))
        self._pages = [[] for _ in range(max_requests)]   # host mirror of the page lists
        self._lens = [0] * max_requests                   # host mirror of the lengths

    @property
    def free_pages(self):
        return len(self._free)

    def release(self, request):
        """Returns the request's pages to the pool."""
        self._free.extend(reversed(self._pages[request]))
        self._pages[request], self._lens[request] = [], 0
        self.kv_lens[request] = 0

    def append(self, requests, ckv, kpe):
        """Appends ``counts[i]`` new tokens to ``requests[i]``: ``requests`` is a list of ``(request, count)`` pairs and
        ``ckv [sum(counts), 512]`` / ``kpe [sum(counts), 64]`` (bfloat16) hold their latent rows in that order."""
        dev = self.ckv_cache.device
        new_rows = []
        for r, n in requests:
            need = -(-(self._lens[r] + n) // self.page_size) - len(self._pages[r])
            if need > len(self._free) or len(self._pages[r]) + need > self.page_table.shape[1]:
                raise RuntimeError("out of cache pages")
            for _ in range(need):
                new_rows.append((r, len(self._pages[r]), self._free.pop()))
                self._pages[r].append(new_rows[-1][2])
            self._lens[r] += n
        if new_rows:
            idx = torch.tensor(new_rows, dtype=torch.int64, device=dev)
            self.page_table[idx[:, 0], idx[:, 1]] = idx[:, 2].int()
        reqs = [r for r, _ in requests]
        counts = torch.tensor([0] + [n for _, n in requests], device=dev)
        nnz = int(counts.sum())
        lens = torch.tensor([self._lens[r] for r in reqs], dtype=torch.int32, device=dev)
        self.kv_lens[torch.tensor(reqs, device=dev)] = lens
        bi, pos = get_batch_indices_positions(counts.cumsum(0).int(), lens, nnz)
        # the writer addresses pages through (kv_indices, kv_indptr): the rows of the page table of the named requests
        width = self.page_table.shape[1]
        kv_indices = self.page_table[torch.tensor(reqs, device=dev)].reshape(-1).contiguous()
        kv_indptr = (torch.arange(len(reqs) + 1, device=dev) * width).int()
        quantize_append_paged_mla_kv_cache(ckv, kpe, bi, pos, self.ckv_cache, self.ckv_sf_cache, self.kpe_cache, kv_indices,
                                           kv_indptr, None, self.ckv_scale, self.kpe_scale)

    def decode(self, requests, q_nope, q_pe, sm_scale, w_uv=None, precision="bf16"):
        """One decode step for ``requests`` (a list of request ids): ``q_nope [len(requests), heads, 512]``,
        ``q_pe [len(requests), heads, 64]``. Returns the latent output ``[n, heads, 512]``, or, with
        ``w_uv [heads, 512, v_head_dim]``, the value-space output ``[n, heads, v_head_dim]`` (the absorbed W_UV applied
        after attention)."""
        idx = torch.tensor(requests, device=self.ckv_cache.device)
        out = decode(q_nope, q_pe, self.ckv_cache, self.ckv_sf_cache, self.kpe_cache, self.page_table[idx].contiguous(),
                     self.kv_lens[idx].contiguous(), sm_scale, self.ckv_scale, self.kpe_scale, max_kv_len=self.max_kv_len,
                     precision=precision)
        return out if w_uv is None else torch.einsum("bhc,hcv->bhv", out, w_uv.to(out.dtype))
