"""MLA decode attention that reads the FlashInfer NVFP4 paged latent-KV cache directly, for B200 (sm_100a).

Drop-in for the reference project's ``nvfp4_mla`` package (nvfp4_mla/__init__.py:13, :47-92): the same ``decode`` and
``dequantize`` signatures, defaults, exception types and messages. The work is done by hand-written CUDA kernels in
``libnvfp4_mla_b200.so`` behind a C ABI (``include/nvfp4_mla_b200.h``); torch only owns the memory and the stream.
"""
import torch

from . import _lib

__all__ = ["decode", "dequantize", "decode_partial", "combine", "combine_packed", "combine_records", "combine_records_signalled", "workspace_status", "quantize_append_paged_mla_kv_cache",
           "get_batch_indices_positions"]
__version__ = "0.1.0"

CKV, KPE = 512, 64
_PRECISIONS = {"bf16": 0, "fp8": 1}
_LN2 = 0.6931471805599453

_workspaces = {}  # (device index, stream handle) -> uint8 tensor; the first int32 is the sticky status word


def _ptr(t):
    return None if t is None else t.data_ptr()


def _check_cache(ckv, sf, kpe):
    """The reference's check_cache (nvfp4_mla/csrc/mla_decode.cu:970-982), same messages."""
    if not (ckv.is_cuda and sf.device == ckv.device and kpe.device == ckv.device):
        raise RuntimeError("caches must be on the same CUDA device")
    if ckv.dtype != torch.uint8:
        raise RuntimeError("ckv_cache must be uint8 (packed E2M1)")
    if sf.dtype != torch.float8_e4m3fn or kpe.dtype != torch.float8_e4m3fn:
        raise RuntimeError("ckv_sf_cache and kpe_cache must be float8_e4m3fn")
    if ckv.dim() != 3 or ckv.shape[2] != CKV // 2:
        raise RuntimeError("ckv_cache must be [pages, page_size, 256]")
    if sf.dim() != 3 or sf.shape[2] != CKV // 16:
        raise RuntimeError("ckv_sf_cache must be [pages, page_size, 32]")
    if kpe.dim() != 3 or kpe.shape[2] != KPE:
        raise RuntimeError("kpe_cache must be [pages, page_size, 64]")
    if sf.shape[:2] != ckv.shape[:2] or kpe.shape[:2] != ckv.shape[:2]:
        raise RuntimeError("ckv_cache, ckv_sf_cache and kpe_cache must have the same [pages, page_size]")
    if not (ckv.is_contiguous() and sf.is_contiguous() and kpe.is_contiguous()):
        raise RuntimeError("caches must be contiguous")


def _workspace(device, stream, nbytes):
    key = (device.index, stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _decode(q_nope, q_pe, ckv_cache, ckv_sf_cache, kpe_cache, page_table, kv_lens, sm_scale, ckv_scale, kpe_scale,
            max_kv_len, num_splits, precision, want_out, want_partial, partial_into=None):
    _check_cache(ckv_cache, ckv_sf_cache, kpe_cache)
    if q_nope.dim() != 3 or q_nope.shape[2] != CKV:
        raise RuntimeError("q_nope must be [batch, heads, 512]")
    B, H = q_nope.shape[:2]
    if q_pe.dim() != 3 or tuple(q_pe.shape) != (B, H, KPE):
        raise RuntimeError("q_pe must be [batch, heads, 64]")
    if q_nope.dtype != torch.bfloat16 or q_pe.dtype != torch.bfloat16:
        raise RuntimeError("q must be bfloat16")
    if H % 16 != 0:
        raise RuntimeError("heads must be a multiple of 16")
    if page_table.dim() != 2 or page_table.shape[0] != B or page_table.dtype != torch.int32:
        raise RuntimeError("page_table must be int32 [batch, max_pages]")
    if kv_lens.dim() != 1 or kv_lens.shape[0] != B or kv_lens.dtype != torch.int32:
        raise RuntimeError("kv_lens must be int32 [batch]")
    for t in (q_nope, q_pe, page_table, kv_lens):
        if t.device != ckv_cache.device or not t.is_contiguous():
            raise RuntimeError("inputs must be contiguous and on the cache device")
    if not (ckv_scale > 0 and kpe_scale > 0):
        raise RuntimeError("ckv_scale and kpe_scale must be positive")
    ps = ckv_cache.shape[1]
    if ps & (ps - 1):
        raise RuntimeError("page_size must be a power of two")
    if max_kv_len is None:
        max_kv_len = int(kv_lens.max()) if B else 0  # device sync; pass max_kv_len to avoid it
    lib = _lib.load()
    dev = ckv_cache.device
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        nbytes = lib.nvfp4_mla_decode_workspace_bytes(B, H, int(num_splits))
        if nbytes < 0:
            raise RuntimeError(lib.nvfp4_mla_last_error().decode())
        ws = _workspace(dev, stream, nbytes)
        out = torch.empty(B, H, CKV, dtype=torch.bfloat16, device=dev) if want_out else None
        if partial_into is not None:
            o32, lse = partial_into
            if not (o32.dtype == lse.dtype == torch.float32 and tuple(o32.shape) == (B, H, CKV) and tuple(lse.shape) == (B, H)
                    and o32.is_contiguous() and lse.is_contiguous() and o32.device == dev and lse.device == dev):
                raise RuntimeError("into must be contiguous float32 ([batch, heads, 512], [batch, heads]) tensors on the cache device")
        else:
            o32 = torch.empty(B, H, CKV, dtype=torch.float32, device=dev) if want_partial else None
            lse = torch.empty(B, H, dtype=torch.float32, device=dev) if want_partial else None
        _lib.check(lib.nvfp4_mla_decode(
            _ptr(q_nope), _ptr(q_pe), _ptr(ckv_cache), _ptr(ckv_sf_cache), _ptr(kpe_cache), ckv_cache.shape[0], ps,
            _ptr(page_table), page_table.stride(0), _ptr(kv_lens), B, H, float(sm_scale), float(ckv_scale),
            float(kpe_scale), int(max_kv_len), int(num_splits), int(precision), _ptr(out), _ptr(o32), _ptr(lse),
            _ptr(ws), ws.numel(), stream))
    return out, o32, lse


def decode(q_nope, q_pe, ckv_cache, ckv_sf_cache, kpe_cache, page_table, kv_lens, sm_scale,
           ckv_scale=1.0, kpe_scale=1.0, max_kv_len=None, num_splits=0, precision="bf16"):
    """Absorbed-MLA decode (one query token per request) on an NVFP4 paged KV cache.

    Args:
        q_nope: ``[batch, heads, 512]`` bfloat16, the absorbed no-RoPE query. ``heads`` must be a multiple of 16.
        q_pe: ``[batch, heads, 64]`` bfloat16, the RoPE query.
        ckv_cache: ``[pages, page_size, 256]`` uint8, packed E2M1 (low nibble = even channel).
        ckv_sf_cache: ``[pages, page_size, 32]`` float8_e4m3fn, one scale per 16 channels.
        kpe_cache: ``[pages, page_size, 64]`` float8_e4m3fn. ``page_size`` must be a power of two.
        page_table: ``[batch, max_pages]`` int32, page ids of each request.
        kv_lens: ``[batch]`` int32, tokens per request (slots past it are never used).
        sm_scale: softmax scale applied to ``q . k``.
        ckv_scale, kpe_scale: the global scales used when the cache was written.
        max_kv_len: an upper bound of ``kv_lens``. Pass it to avoid a device sync and to keep the launch shape fixed
            under CUDA graphs. Default: ``kv_lens.max()``.
        num_splits: extra KV cuts per request. 0 (default) lets the device-side schedule balance 128-token tiles over
            all SMs; ``n > 0`` additionally cuts every request at multiples of ``ceil(max_kv_len / n)`` tokens
            (rounded up to 128).
        precision: arithmetic of the attention, not of the cache: ``"bf16"`` (16-bit operands, exact K and V) or
            ``"fp8"`` (E4M3 query, K, V and P).

    Returns:
        ``[batch, heads, 512]`` bfloat16 attention output (the latent value; apply W_UV outside).
    """
    if precision not in _PRECISIONS:
        raise ValueError(f"precision must be one of {list(_PRECISIONS)}, got {precision!r}")
    return _decode(q_nope, q_pe, ckv_cache, ckv_sf_cache, kpe_cache, page_table, kv_lens, sm_scale, ckv_scale,
                   kpe_scale, max_kv_len, num_splits, _PRECISIONS[precision], True, False)[0]


def decode_partial(q_nope, q_pe, ckv_cache, ckv_sf_cache, kpe_cache, page_table, kv_lens, sm_scale,
                   ckv_scale=1.0, kpe_scale=1.0, max_kv_len=None, num_splits=0, precision="bf16", into=None):
    """As ``decode`` but returns ``(o [batch, heads, 512] float32, lse [batch, heads] float32)`` with ``lse`` the
    log2-domain log-sum-exp of the scaled scores: the (o, lse) pair that ``combine`` merges, e.g. across GPUs that
    each hold a slice of one long context. A request with ``kv_len == 0`` gives ``o = 0`` and ``lse = -inf``.
    ``into=(o, lse)`` writes into caller-owned tensors (e.g. the send buffer of a collective) instead of new ones."""
    if precision not in _PRECISIONS:
        raise ValueError(f"precision must be one of {list(_PRECISIONS)}, got {precision!r}")
    _, o, lse = _decode(q_nope, q_pe, ckv_cache, ckv_sf_cache, kpe_cache, page_table, kv_lens, sm_scale, ckv_scale,
                        kpe_scale, max_kv_len, num_splits, _PRECISIONS[precision], False, True, into)
    return o, lse


def combine_packed(packed, rows, out_dtype=torch.bfloat16):
    """Merge of ``packed [parts, rows * 513]`` float32, one record ``[o (rows x 512) | lse (rows)]`` per part: the
    receive buffer of an all-gather of the ranks' partial results, merged in place of unpacking it. Returns
    ``[rows, 512]`` in ``out_dtype``."""
    if packed.dtype != torch.float32 or packed.dim() != 2 or packed.shape[1] != rows * (CKV + 1) or not packed.is_contiguous():
        raise RuntimeError("packed must be a contiguous float32 [parts, rows * 513] tensor")
    if not packed.is_cuda:
        raise RuntimeError("packed must be a CUDA tensor")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"out_dtype must be bfloat16 or float32, got {out_dtype}")
    dev = packed.device
    out = torch.empty(rows, CKV, dtype=out_dtype, device=dev)
    lib = _lib.load()
    stride = rows * (CKV + 1)
    with torch.cuda.device(dev):
        _lib.check(lib.nvfp4_mla_combine_strided(
            packed.data_ptr(), packed.data_ptr() + rows * CKV * 4, packed.shape[0], rows, stride, stride,
            _ptr(out) if out_dtype == torch.bfloat16 else None, _ptr(out) if out_dtype == torch.float32 else None, None,
            torch.cuda.current_stream(dev).cuda_stream))
    return out


def combine_records(record_ptrs, rows, device, out_dtype=torch.bfloat16):
    """Merge of packed records ``[o (rows x 512) | lse (rows)]`` (float32) given by their device addresses, one per
    part (at most 16): the partial results of the GPUs of a sequence-sharded decode, read where their owners wrote them
    (addresses of peers' symmetric-memory buffers included). The caller orders the call after the owners' writes.
    Returns ``[rows, 512]`` in ``out_dtype`` on ``device``."""
    import ctypes
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"out_dtype must be bfloat16 or float32, got {out_dtype}")
    dev = torch.device(device)
    out = torch.empty(rows, CKV, dtype=out_dtype, device=dev)
    ptrs = (ctypes.c_void_p * len(record_ptrs))(*[int(p) for p in record_ptrs])
    lib = _lib.load()
    with torch.cuda.device(dev):
        _lib.check(lib.nvfp4_mla_combine_records(
            ptrs, len(record_ptrs), rows, _ptr(out) if out_dtype == torch.bfloat16 else None,
            _ptr(out) if out_dtype == torch.float32 else None, None, torch.cuda.current_stream(dev).cuda_stream))
    return out


def combine_records_signalled(record_ptrs, flag_ptrs, rank, epoch, rows, device, out_dtype=torch.bfloat16, status=None,
                              wait_us=10_000_000):
    """``combine_records`` with the hand-shake between the GPUs inside the merge kernel (no barrier in front of it).
    ``flag_ptrs[g]`` is the address, in this process, of GPU ``g``'s array of ``len(record_ptrs)`` uint32 words (zero
    before the first call); the call announces this GPU's record of step ``epoch`` (1, 2, 3, ... on every GPU alike) in
    word ``rank`` of every array, waits at most ``wait_us`` microseconds for the other GPUs' announcements and merges.
    ``status``: int32 CUDA tensor of one element that receives 4 when the wait ran out (the output is then not to be
    used). Returns ``[rows, 512]`` in ``out_dtype`` on ``device``."""
    import ctypes
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"out_dtype must be bfloat16 or float32, got {out_dtype}")
    if len(flag_ptrs) != len(record_ptrs):
        raise ValueError("one flag array per record")
    dev = torch.device(device)
    if status is not None and not (status.is_cuda and status.dtype == torch.int32 and status.numel() >= 1):
        raise RuntimeError("status must be an int32 CUDA tensor")
    out = torch.empty(rows, CKV, dtype=out_dtype, device=dev)
    recs = (ctypes.c_void_p * len(record_ptrs))(*[int(p) for p in record_ptrs])
    flags = (ctypes.c_void_p * len(flag_ptrs))(*[int(p) for p in flag_ptrs])
    lib = _lib.load()
    with torch.cuda.device(dev):
        _lib.check(lib.nvfp4_mla_combine_records_signalled(
            recs, flags, int(rank), int(epoch) & 0xFFFFFFFF, int(wait_us), len(record_ptrs), rows,
            _ptr(out) if out_dtype == torch.bfloat16 else None, _ptr(out) if out_dtype == torch.float32 else None, None,
            _ptr(status), torch.cuda.current_stream(dev).cuda_stream))
    return out


def combine(o_part, lse_part, out_dtype=torch.bfloat16, return_lse=False):
    """Log-sum-exp merge of partial results: ``o_part [parts, ..., 512]`` float32 (each normalised by its own softmax
    sum) and ``lse_part [parts, ...]`` float32 in log2 units. Returns ``[..., 512]`` in ``out_dtype`` (bfloat16 or
    float32), and the merged lse with ``return_lse``."""
    if o_part.dtype != torch.float32 or lse_part.dtype != torch.float32:
        raise RuntimeError("o_part and lse_part must be float32")
    if o_part.shape[-1] != CKV or tuple(o_part.shape[:-1]) != tuple(lse_part.shape) or o_part.dim() < 2:
        raise RuntimeError("o_part must be [parts, ..., 512] and lse_part [parts, ...]")
    if not (o_part.is_cuda and o_part.is_contiguous() and lse_part.is_contiguous() and lse_part.device == o_part.device):
        raise RuntimeError("o_part and lse_part must be contiguous CUDA tensors on one device")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"out_dtype must be bfloat16 or float32, got {out_dtype}")
    parts, inner = o_part.shape[0], tuple(o_part.shape[1:-1])
    rows = lse_part[0].numel()
    dev = o_part.device
    out = torch.empty(*inner, CKV, dtype=out_dtype, device=dev)
    lse = torch.empty(inner, dtype=torch.float32, device=dev) if return_lse else None
    lib = _lib.load()
    with torch.cuda.device(dev):
        _lib.check(lib.nvfp4_mla_combine(_ptr(o_part), _ptr(lse_part), parts, rows,
                                         _ptr(out) if out_dtype == torch.bfloat16 else None,
                                         _ptr(out) if out_dtype == torch.float32 else None, _ptr(lse),
                                         torch.cuda.current_stream(dev).cuda_stream))
    return (out, lse) if return_lse else out


def dequantize(ckv_cache, ckv_sf_cache, kpe_cache, ckv_scale=1.0, kpe_scale=1.0, dtype=torch.bfloat16):
    """Dequantize a whole NVFP4 MLA cache to ``(ckv [pages, page_size, 512], kpe [pages, page_size, 64])``.

    ``dtype`` is bfloat16 or float32. The float32 result equals ``e2m1 * block_scale * ckv_scale`` evaluated left to
    right bit for bit; BF16 is exact when ``ckv_scale`` and ``kpe_scale`` are powers of two.
    """
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
    _check_cache(ckv_cache, ckv_sf_cache, kpe_cache)
    P, ps = ckv_cache.shape[:2]
    dev = ckv_cache.device
    ckv = torch.empty(P, ps, CKV, dtype=dtype, device=dev)
    kpe = torch.empty(P, ps, KPE, dtype=dtype, device=dev)
    lib = _lib.load()
    with torch.cuda.device(dev):
        _lib.check(lib.nvfp4_mla_dequantize(_ptr(ckv_cache), _ptr(ckv_sf_cache), _ptr(kpe_cache), P * ps,
                                            float(ckv_scale), float(kpe_scale), int(dtype == torch.bfloat16),
                                            _ptr(ckv), _ptr(kpe), torch.cuda.current_stream(dev).cuda_stream))
    return ckv, kpe


def get_batch_indices_positions(append_indptr, seq_lens, nnz):
    """``(batch_indices [nnz], positions [nnz])`` int32 of appended tokens, FlashInfer's helper of the same name
    (used by the reference at ``nvfp4_mla/testing.py:36``): request ``b`` appends tokens
    ``append_indptr[b] .. append_indptr[b + 1]``, which become the last positions of its ``seq_lens[b]`` tokens."""
    append_indptr, seq_lens = append_indptr.to(torch.int64), seq_lens.to(torch.int64)
    counts = append_indptr[1:] - append_indptr[:-1]
    bi = torch.repeat_interleave(torch.arange(counts.numel(), device=counts.device), counts, output_size=nnz)
    pos = torch.arange(nnz, device=counts.device) - append_indptr[:-1][bi] + (seq_lens - counts)[bi]
    return bi.to(torch.int32), pos.to(torch.int32)


def quantize_append_paged_mla_kv_cache(ckv, kpe, batch_indices, positions, ckv_cache, ckv_sf_cache, kpe_cache,
                                       kv_indices, kv_indptr, kv_last_page_len=None, ckv_scale=1.0, kpe_scale=1.0,
                                       check=False):
    """Quantises new tokens to NVFP4 / E4M3 and writes them into the paged cache, in place.

    Same arguments as FlashInfer's ``nvfp4_quantize_append_paged_mla_kv_cache``, the writer the reference uses
    (``nvfp4_mla/testing.py:51-53``): ``ckv [nnz, 512]`` and ``kpe [nnz, 64]`` bfloat16, ``batch_indices`` /
    ``positions`` ``[nnz]`` int32, the three cache tensors, the page list ``kv_indices`` with ``kv_indptr [B + 1]``;
    ``kv_last_page_len`` is accepted and not needed. ``check=True`` synchronises and raises if a token pointed
    outside the tables (such tokens are skipped)."""
    _check_cache(ckv_cache, ckv_sf_cache, kpe_cache)
    nnz = ckv.shape[0]
    if ckv.dtype != torch.bfloat16 or kpe.dtype != torch.bfloat16:
        raise RuntimeError("ckv and kpe must be bfloat16")
    if tuple(ckv.shape) != (nnz, CKV) or tuple(kpe.shape) != (nnz, KPE) or not (ckv.is_contiguous() and kpe.is_contiguous()):
        raise RuntimeError("ckv must be a contiguous [nnz, 512] and kpe a contiguous [nnz, 64] tensor")
    for name, t, n in (("batch_indices", batch_indices, nnz), ("positions", positions, nnz), ("kv_indices", kv_indices, None),
                       ("kv_indptr", kv_indptr, None)):
        if t.dtype != torch.int32 or t.dim() != 1 or not t.is_contiguous() or (n is not None and t.numel() != n):
            raise RuntimeError(f"{name} must be a contiguous 1-D int32 tensor" + (f" of {n} elements" if n is not None else ""))
    P, ps = ckv_cache.shape[:2]
    dev = ckv_cache.device
    status = torch.zeros(1, dtype=torch.int32, device=dev) if check else None
    lib = _lib.load()
    with torch.cuda.device(dev):
        _lib.check(lib.nvfp4_mla_quantize_append(
            _ptr(ckv), _ptr(kpe), _ptr(batch_indices), _ptr(positions), nnz, _ptr(ckv_cache), _ptr(ckv_sf_cache),
            _ptr(kpe_cache), P, ps, _ptr(kv_indices), _ptr(kv_indptr), kv_indptr.numel() - 1, float(ckv_scale),
            float(kpe_scale), _ptr(status) if check else None, torch.cuda.current_stream(dev).cuda_stream))
    if check and int(status.item()) != 0:
        raise RuntimeError("quantize_append: a token named a request, position or page outside the tables")


def workspace_status(device=None, clear=False):
    """Synchronises and returns the worst device-side status of the decode workspaces of ``device`` (0 = fine,
    1 = a bounded wait inside the decode kernel gave up, 2 = schedule capacity exceeded, 3 = a page id inside a request's
    live range lies outside the cache; the id was not dereferenced). The status word is sticky; ``clear=True`` zeroes
    it after reading. For tests and debugging."""
    lib = _lib.load()
    worst = 0
    for (idx, stream), ws in list(_workspaces.items()):
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        with torch.cuda.device(idx):
            torch.cuda.synchronize(idx)
            st = lib.nvfp4_mla_workspace_status(_ptr(ws), None)
            if st < 0:
                raise RuntimeError(lib.nvfp4_mla_last_error().decode())
            if clear and st:
                ws[:4].zero_()
                torch.cuda.synchronize(idx)
            worst = max(worst, st)
    return worst
