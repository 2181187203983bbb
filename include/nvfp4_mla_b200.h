/* C ABI of the B200 (sm_100a) NVFP4 paged MLA decode library, libnvfp4_mla_b200.so.
 *
 * Every entry point takes plain device pointers and sizes plus a CUDA stream handle (cudaStream_t passed as void*;
 * NULL = the legacy default stream), launches asynchronously on that stream and never synchronises the device,
 * allocates nothing and keeps no reference to its arguments. Functions returning int return 0 on success; on
 * failure nothing was launched and nvfp4_mla_last_error() describes why (thread-local, valid until the thread's
 * next call). All pointers must belong to the device that is current when the call is made.
 *
 * Each function names the interface of the reference project (elwhyjay/nvfp4-mla) that it replaces, by the file's
 * path inside that project.
 */
#ifndef NVFP4_MLA_B200_H_
#define NVFP4_MLA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define NVFP4_MLA_API __attribute__((visibility("default")))
#else
#define NVFP4_MLA_API
#endif

#define NVFP4_MLA_PRECISION_BF16 0 /* exact FP16 K/V operands, FP16 P, fp32 accumulation */
#define NVFP4_MLA_PRECISION_FP8 1  /* E4M3 query rows, K, V and P, fp32 accumulation */

/* Library version as major * 10000 + minor * 100 + patch. */
NVFP4_MLA_API int nvfp4_mla_version(void);

/* Message of the calling thread's most recent failed call ("" if none). */
NVFP4_MLA_API const char* nvfp4_mla_last_error(void);

/* Kernels one nvfp4_mla_decode call with these arguments launches on the current device: 2 (decode, merge of the
 * partials) when the decode kernel derives the split-KV schedule by itself (batch x splits up to its thread count),
 * 3 with the schedule kernel in front (larger batches); 0 for batch 0, -1 on invalid arguments. For launch accounting;
 * the reference's launcher (nvfp4_mla/csrc/mla_decode.cu:1042-1069) launches its split and merge kernels likewise. */
NVFP4_MLA_API int nvfp4_mla_decode_launches(int batch, int heads, int max_kv_len, int num_splits, int precision);

/* Bytes of scratch nvfp4_mla_decode needs for this problem on the current device. `num_splits` as in the decode
 * call. Replaces the torch::empty of o_part / lse_part inside the reference launcher
 * (nvfp4_mla/csrc/mla_decode.cu:1042-1047). Returns -1 on invalid arguments. */
NVFP4_MLA_API int64_t nvfp4_mla_decode_workspace_bytes(int batch, int heads, int num_splits);

/* Absorbed-MLA decode, one query token per request, over the NVFP4 paged latent-KV cache.
 * Replaces the pybind `decode` of the reference (nvfp4_mla/csrc/mla_decode.cu:1063-1085, launcher :984-1061), which
 * nvfp4_mla.decode calls (nvfp4_mla/__init__.py:47-81).
 *
 *   q_nope       [batch, heads, 512] bfloat16, contiguous        q_pe  [batch, heads, 64] bfloat16, contiguous
 *   ckv_cache    [num_pages, page_size, 256] uint8   packed E2M1, low nibble = even channel
 *   ckv_sf_cache [num_pages, page_size, 32]  E4M3    one scale per 16 channels
 *   kpe_cache    [num_pages, page_size, 64]  E4M3
 *   page_table   [batch, page_table_stride] int32 page ids (only the first ceil(kv_len / page_size) are read)
 *   kv_lens      [batch] int32; read on the device, never on the host
 *   heads        a multiple of 16;  page_size a power of two;  ckv_scale, kpe_scale > 0
 *   max_kv_len   upper bound of kv_lens: with num_splits it fixes the launch shape, so the same call can be
 *                captured in a CUDA graph and replayed with other kv_lens below the bound
 *   num_splits   0 = one KV range per request (work is still balanced over all SMs tile by tile);
 *                n > 0 = cut every request at multiples of round_up(ceil(max_kv_len / n), 128) tokens as well
 *   precision    NVFP4_MLA_PRECISION_*
 *   out          [batch, heads, 512] bfloat16 or NULL
 *   out_f32      [batch, heads, 512] float or NULL: the same result unrounded (for merging across GPUs)
 *   lse          [batch, heads] float or NULL: log2-domain log-sum-exp of the scaled scores, i.e.
 *                log2(sum_t exp(score_t)), -inf for kv_len 0 (the unit of the reference's split partials,
 *                nvfp4_mla/csrc/mla_decode.cu:478-492)
 *   workspace    at least nvfp4_mla_decode_workspace_bytes() bytes, 256-byte aligned; its first int32 is a sticky
 *                device-side status word that the caller zeroes once (see nvfp4_mla_workspace_status)
 */
NVFP4_MLA_API int nvfp4_mla_decode(const void* q_nope, const void* q_pe, const uint8_t* ckv_cache, const uint8_t* ckv_sf_cache,
                     const uint8_t* kpe_cache, int64_t num_pages, int page_size, const int32_t* page_table,
                     int64_t page_table_stride, const int32_t* kv_lens, int batch, int heads, float sm_scale,
                     float ckv_scale, float kpe_scale, int max_kv_len, int num_splits, int precision, void* out,
                     float* out_f32, float* lse, void* workspace, int64_t workspace_bytes, void* stream);

/* nvfp4_mla_decode for callers that have no way to hand over scratch memory. (No counterpart in the reference, whose
 * launcher always allocates its partial buffers through torch.)
 *
 * Some hosts of this library cannot allocate device memory at the point where they decode: an inference server that
 * reserved the whole GPU for its own pool at start-up and has nothing left for cudaMalloc to hand out, a plugin that is
 * only given its input and output buffers, or code running where an allocation would stall the device for every other
 * stream. For them the library carries its own scratch: a fixed 9 MiB array inside the library's device image
 * (nvfp4_mla_decode_static_capacity() bytes, held by every GPU that loads the library until the process exits).
 * Arguments and results are those of nvfp4_mla_decode, without `workspace` / `workspace_bytes`.
 *
 *   - Limit: the partial results take 2 KB per head, CTA and work item, so the call fails, launching nothing, when
 *     (SMs + batch * (heads / 16) * max(num_splits, 1)) * 32.1 KB exceeds the capacity: on a 148-SM B200 that allows
 *     batch * (heads / 16) * max(num_splits, 1) up to about 138 in either precision, e.g. batch 64 with 16 heads, or
 *     batch 16 with 128 heads. The 8-bit mode normally groups 32 or 128 heads per CTA, which needs more scratch than
 *     that; this entry point uses the widest grouping that fits and falls back to 16 heads per CTA (same results
 *     within the mode's tolerance, slower at 128 heads).
 *   - Nothing is allocated or freed here, by CUDA or by any library, on any call.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress) and does the one-time
 *     kernel set-up; make that first call outside any stream capture.
 *   - All calls on a device share the one array. Calls that can overlap on the GPU (different streams, or graphs
 *     replayed concurrently) race on it and corrupt each other's results: serialise them, or give the concurrent
 *     ones their own workspace through nvfp4_mla_decode.
 *   - The array keeps what the previous call wrote. Nothing in it has to be cleared between calls: every record the
 *     kernels read is rewritten by the call itself first (by its schedule kernel, or by the decode CTAs that derive
 *     the schedule themselves). The device-side status word is zero when the
 *     library is loaded and sticky afterwards: nvfp4_mla_decode_static_status(stream) synchronises `stream`, returns
 *     the status of all static calls since it last reported a non-zero one (same codes as nvfp4_mla_workspace_status)
 *     and, if it was non-zero, clears the word. */
NVFP4_MLA_API int nvfp4_mla_decode_static(const void* q_nope, const void* q_pe, const uint8_t* ckv_cache,
                                          const uint8_t* ckv_sf_cache, const uint8_t* kpe_cache, int64_t num_pages,
                                          int page_size, const int32_t* page_table, int64_t page_table_stride,
                                          const int32_t* kv_lens, int batch, int heads, float sm_scale, float ckv_scale,
                                          float kpe_scale, int max_kv_len, int num_splits, int precision, void* out,
                                          float* out_f32, float* lse, void* stream);
NVFP4_MLA_API int64_t nvfp4_mla_decode_static_capacity(void);
NVFP4_MLA_API int nvfp4_mla_decode_static_status(void* stream);

/* Synchronises `stream` and returns the status word of a decode workspace: 0 = every kernel ran to completion,
 * 1 = a bounded wait inside the decode kernel gave up (results invalid), 2 = batch * num_splits too large for the
 * schedule kernel, 3 = a page id inside a request's live range lies outside [0, num_pages) (it was not dereferenced:
 * pages of 64 tokens or more read as zeros, smaller pages keep whatever the staging buffer held; results invalid);
 * negative = CUDA error (see nvfp4_mla_last_error). No counterpart in the reference, whose kernels
 * have no bounded waits. */
NVFP4_MLA_API int nvfp4_mla_workspace_status(const void* workspace, void* stream);

/* Measurement aid: between nvfp4_mla_profile_begin(capacity) and nvfp4_mla_profile_end, every nvfp4_mla_decode call
 * made by this thread (up to `capacity` of them) brackets its main decode kernel, and only that kernel, with a pair
 * of CUDA events on the call's stream. profile_end waits for them, writes the kernel durations in milliseconds to
 * ms[0 .. min(calls, capacity)) and returns how many it wrote (negative on error). The only entry points that create
 * CUDA objects; not meant for stream capture. Stands where the reference times kernels with CUPTI
 * (benchmarks/baselines.py:168-187). */
NVFP4_MLA_API int nvfp4_mla_profile_begin(int capacity);
NVFP4_MLA_API int nvfp4_mla_profile_end(float* ms, int capacity);

/* Whole-cache dequantisation: ckv = e2m1 * block_scale * ckv_scale, kpe = e4m3 * kpe_scale, in that multiply
 * order, to float (out_bf16 = 0) or bfloat16 (out_bf16 = 1). num_tokens = num_pages * page_size. ckv_cache must be
 * 4-byte aligned, kpe_cache 2-byte, ckv_out 16-byte and kpe_out 8-byte aligned (checked; a misaligned pointer is an error
 * return, never a device fault).
 * Replaces the pybind `dequantize` (nvfp4_mla/csrc/mla_decode.cu:1113-1132; nvfp4_mla/__init__.py:84-92). */
NVFP4_MLA_API int nvfp4_mla_dequantize(const uint8_t* ckv_cache, const uint8_t* ckv_sf_cache, const uint8_t* kpe_cache,
                         int64_t num_tokens, float ckv_scale, float kpe_scale, int out_bf16, void* ckv_out,
                         void* kpe_out, void* stream);

/* Cache writer: quantises `nnz` new tokens (ckv [nnz, 512] and kpe [nnz, 64], bfloat16) and appends them to the paged
 * cache. Token i belongs to request batch_indices[i] at position positions[i]; its slot is page
 * kv_indices[kv_indptr[b] + position / page_size], row position % page_size. Per 16 latent channels the block scale is
 * e4m3(amax / 6 / ckv_scale), the codes are the nearest E2M1 of x / (scale * ckv_scale) (ties to even, saturating),
 * packed low nibble = even channel; rope is e4m3(kpe / kpe_scale). `status` (optional device word) is set to 1 if a
 * token names a request, position or page outside the tables; such a token is skipped.
 * The reference has no writer of its own: it calls FlashInfer's nvfp4_quantize_append_paged_mla_kv_cache with these
 * arguments (nvfp4_mla/testing.py:51-53, README.md:77-79); this entry point takes the same tables so that it can stand
 * in for that call. */
NVFP4_MLA_API int nvfp4_mla_quantize_append(const void* ckv, const void* kpe, const int32_t* batch_indices,
                              const int32_t* positions, int64_t nnz, uint8_t* ckv_cache, uint8_t* ckv_sf_cache,
                              uint8_t* kpe_cache, int64_t num_pages, int page_size, const int32_t* kv_indices,
                              const int32_t* kv_indptr, int batch, float ckv_scale, float kpe_scale, int32_t* status,
                              void* stream);

/* Log-sum-exp merge of `parts` partial results: o_part [parts, rows, 512] float (each normalised by its own
 * softmax sum), lse_part [parts, rows] float in log2 units (-inf = empty partial, weight 0); parts <= 512. Any of out
 * (bfloat16 [rows, 512]), out_f32 (float [rows, 512]) and lse (float [rows]) may be NULL.
 * Replaces the pybind `combine` (nvfp4_mla/csrc/mla_decode.cu:1281-1294, kernel :933-966); also the merge step of
 * sequence-sharded decode across GPUs. */
NVFP4_MLA_API int nvfp4_mla_combine(const float* o_part, const float* lse_part, int parts, int64_t rows, void* out, float* out_f32,
                      float* lse, void* stream);

/* nvfp4_mla_combine over partials that are not densely stacked: part i has its o rows at o_part + i * o_part_stride
 * floats and its lse values at lse_part + i * lse_part_stride floats. This is the shape of an all-gather of one packed
 * [o | lse] record per GPU (sequence-sharded decode: o_part = buffer, lse_part = buffer + rows * 512, both strides
 * rows * 513), merged without unpacking. o_part_stride must be a multiple of 4. Same reference counterpart as
 * nvfp4_mla_combine (nvfp4_mla/csrc/mla_decode.cu:933-966, :1281-1294). */
NVFP4_MLA_API int nvfp4_mla_combine_strided(const float* o_part, const float* lse_part, int parts, int64_t rows,
                                            int64_t o_part_stride, int64_t lse_part_stride, void* out, float* out_f32,
                                            float* lse, void* stream);

/* The same merge over `parts` (at most 16) packed records [o (rows x 512) | lse (rows)] at unrelated addresses:
 * records is a HOST array of device pointers, 16-byte aligned, which may point into other GPUs' memory mapped into this
 * process (peer access, symmetric memory). Used by the sequence-sharded decode to merge the GPUs' partial results where
 * their owners wrote them, without a collective; the caller orders this call after the owners' writes (a barrier
 * between the GPUs on the stream). Same reference counterpart as nvfp4_mla_combine. */
NVFP4_MLA_API int nvfp4_mla_combine_records(const float* const* records, int parts, int64_t rows, void* out, float* out_f32,
                                            float* lse, void* stream);

/* nvfp4_mla_combine_records with the hand-shake between the GPUs inside the kernel, so that no barrier has to be
 * launched in front of it. GPU `rank` (0 <= rank < parts) owns an array of `parts` 32-bit words that every GPU can
 * write (flags[g] = address, in this process, of GPU g's array; flags is a HOST array), zero before the first call.
 * The call announces "my record of step `epoch` is written" by storing `epoch` into word `rank` of every GPU's array,
 * waits until all `parts` words of its own array carry `epoch` or a later one, and then merges. Every GPU makes the
 * same sequence of calls with epoch = 1, 2, 3, ... (wrap-around is handled). A GPU may overwrite the record it
 * announced at step s once its own call of step s + 1 has completed (work queued behind that call on the same stream
 * qualifies): every GPU has finished reading step s by then, so two records that alternate are enough. The
 * wait gives up after wait_us microseconds (> 0): the kernel then raises status 4 (peer time-out) in *status (device
 * int, may be NULL; the larger of the old and new value is kept) and merges whatever the records hold, so the
 * context stays usable. The reference is single-GPU: no counterpart. */
NVFP4_MLA_API int nvfp4_mla_combine_records_signalled(const float* const* records, uint32_t* const* flags, int rank,
                                                      uint32_t epoch, int64_t wait_us, int parts, int64_t rows, void* out,
                                                      float* out_f32, float* lse, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NVFP4_MLA_B200_H_ */
