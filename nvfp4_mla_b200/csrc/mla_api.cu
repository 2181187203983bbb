// C ABI of libnvfp4_mla_b200.so: argument validation, the TMA descriptor of the cache, and kernel launches.
// Declarations and their documentation: include/nvfp4_mla_b200.h.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/nvfp4_mla_b200.h"
#include "mla_common.cuh"
#include "mla_decode_sm100.cuh"
#include "mla_decode_vt_sm100.cuh"
#include "mla_decode_hm_sm100.cuh"
#include "mla_dequant.cuh"
#include "mla_quantize.cuh"
#include "mla_schedule.cuh"

namespace {

thread_local char g_error[512] = "";

int fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
  return 1;
}
#define MLA_CHECK(cond, ...) \
  do {                       \
    if (!(cond)) return fail(__VA_ARGS__); \
  } while (0)
#define MLA_CUDA(expr)                                                                   \
  do {                                                                                   \
    cudaError_t e_ = (expr);                                                             \
    if (e_ != cudaSuccess) return fail("%s failed: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

constexpr int kMaxDevices = 64;
struct DeviceInfo {
  bool ready = false;
  int sm_count = 0;
  int hm_pairs = 0;  // CTA pairs (clusters of two) of the heads-as-M kernel that can be resident at once; 0 = do not use it
};
std::mutex g_mutex;
DeviceInfo g_devices[kMaxDevices];

using DecodeKernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const mla::DecodeParams);
// staging slots of 64 tokens next to the V tile (one FP16 tile of 128 KB, or two E4M3 tiles of 64 KB)
constexpr int kRawSlots8 = 3;
constexpr int kRawSlotsHm = 4;  // heads-as-M kernel: staging slots of 32 tokens
// Heads per CTA (the N of both MMAs). One conversion of a tile serves all of the CTA's heads, so more heads per CTA
// means less conversion work per head; 32 fit next to the tiles only in the 8-bit mode (tensor memory and shared memory).
// With 128 heads per request the 8-bit mode runs the heads-as-M kernel: a pair of CTAs per 128 heads (each CTA
// accumulates half of the output channels), scheduled as one unit, so the schedule sees half as many "CTAs".
// `limit` caps the grouping (a caller with little scratch asks for a narrower one: the partial results of a CTA take
// 2 KB per head).
int heads_per_cta(int heads, int precision, const DeviceInfo& d, int limit = 128) {
  if (precision != NVFP4_MLA_PRECISION_FP8) return 16;
  return heads % 128 == 0 && d.hm_pairs > 0 && limit >= 128 ? 128 : heads % 32 == 0 && limit >= 32 ? 32 : 16;
}
int schedule_units(const DeviceInfo& d, int hpc) { return hpc == 128 ? d.hm_pairs : d.sm_count; }
int ctas_per_unit(int hpc) { return hpc == 128 ? 2 : 1; }
DecodeKernel decode_kernel(int precision, int hpc) {
  if (precision == NVFP4_MLA_PRECISION_FP8)
    return hpc == 128  ? mla::mla_decode_hm_kernel<kRawSlotsHm>
           : hpc == 32 ? mla::mla_decode_kernel<32, kRawSlots8, true>
                       : mla::mla_decode_kernel<16, kRawSlots8, true>;
  return mla::mla_decode_vt_kernel;
}
unsigned decode_threads(int precision, int hpc) {
  if (precision == NVFP4_MLA_PRECISION_FP8) return hpc == 128 ? mla::kHmThreads : mla::kDecodeThreads;
  return mla::kVtThreads;
}
size_t decode_smem(int precision, int hpc) {
  if (precision == NVFP4_MLA_PRECISION_FP8)
    return hpc == 128  ? mla::hm_smem_bytes<kRawSlotsHm>()
           : hpc == 32 ? mla::decode_smem_bytes<32, kRawSlots8, true>()
                       : mla::decode_smem_bytes<16, kRawSlots8, true>();
  return mla::vt_smem_bytes();
}
static_assert(mla::hm_smem_bytes<kRawSlotsHm>() <= 232448, "heads-as-M kernel exceeds the shared memory a CTA can opt in to");
static_assert(mla::decode_smem_bytes<32, kRawSlots8, true>() <= 232448 && mla::decode_smem_bytes<16, kRawSlots8, true>() <= 232448 &&
                  mla::vt_smem_bytes() <= 232448,
              "decode kernel exceeds the 227 KB of shared memory a CTA can opt in to");

// Per-device one-time setup (SM count, opt-in shared memory). Must first run outside stream capture.
int device_info(DeviceInfo** out) {
  int dev = 0;
  MLA_CUDA(cudaGetDevice(&dev));
  MLA_CHECK(dev >= 0 && dev < kMaxDevices, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceInfo& d = g_devices[dev];
  if (!d.ready) {
    int major = 0;
    MLA_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    MLA_CHECK(major == 10, "nvfp4_mla_b200 needs an sm_100a GPU (B200), found compute capability %d.x", major);
    MLA_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
    for (int prec : {NVFP4_MLA_PRECISION_BF16, NVFP4_MLA_PRECISION_FP8})
      for (int hpc : {16, 32, 128})
        MLA_CUDA(cudaFuncSetAttribute(decode_kernel(prec, hpc), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      int(decode_smem(prec, hpc))));
    {  // clusters of two need both SMs in one GPC: ask how many can be resident rather than assuming sm_count / 2
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(unsigned(d.sm_count / 2 * 2)), cfg.blockDim = dim3(mla::kHmThreads);
      cfg.dynamicSmemBytes = decode_smem(NVFP4_MLA_PRECISION_FP8, 128);
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr, cfg.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, decode_kernel(NVFP4_MLA_PRECISION_FP8, 128), &cfg) != cudaSuccess) {
        (void)cudaGetLastError();
        clusters = 0;
      }
      d.hm_pairs = clusters < d.sm_count / 2 ? clusters : d.sm_count / 2;
      if (getenv("NVFP4_MLA_DEBUG"))
        fprintf(stderr, "nvfp4_mla_b200: device %d: %d SMs, %d resident CTA pairs for the 128-head kernel\n", dev, d.sm_count, d.hm_pairs);
    }
    d.ready = true;
  }
  *out = &d;
  return 0;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
int encode_fn(EncodeTiledFn* out) {
  static EncodeTiledFn fn = nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    MLA_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    MLA_CHECK(p != nullptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is not available in this driver");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  *out = fn;
  return 0;
}

// ckv_cache as a 2-D byte tensor [num_pages * page_size, 256]; a box is min(page_size, 64) token rows by 128 bytes,
// written to shared memory with the 128-byte swizzle that makes thread-per-token reads conflict free.
// 2-D byte map over one of the cache tensors seen as [rows = pages * page_size, row_bytes]; a box is `box_bytes` of up
// to `slot_rows` rows (one staging slot, or one page if pages are smaller), written to shared memory with the given swizzle.
int make_row_map(const uint8_t* base, int64_t rows, int row_bytes, int box_bytes, int page_size, int slot_rows,
                 CUtensorMapSwizzle swizzle, CUtensorMap* map) {
  EncodeTiledFn encode;
  if (encode_fn(&encode)) return 1;
  const cuuint64_t dims[2] = {cuuint64_t(row_bytes), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(row_bytes)};
  const cuuint32_t box[2] = {cuuint32_t(box_bytes), cuuint32_t(page_size < slot_rows ? page_size : slot_rows)};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(base), dims, strides, box, elem_strides,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MLA_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with CUresult %d", int(r));
  return 0;
}

// Optional per-call timing of the decode kernel alone (see nvfp4_mla_profile_begin).
struct Profile {
  std::vector<cudaEvent_t> start, stop;
  int used = 0;
};
thread_local Profile* g_profile = nullptr;

// Launch with programmatic stream serialization: the kernel may start while its predecessor in the stream is still
// running; it must execute griddepcontrol.wait before touching anything the predecessor writes. Used for the
// schedule -> decode -> combine chain so that launch latency and prologues overlap the previous kernel.
// `cluster` > 1 launches thread-block clusters of that many consecutive CTAs (the grid must be a multiple of it).
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, unsigned cluster,
                                     Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  if (cluster > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster, attr[1].val.clusterDim.y = 1, attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  return launch_dependent_cluster(kernel, grid, block, smem, st, 1u, static_cast<Args&&>(args)...);
}

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

int problem_of(int batch, int heads, int max_kv_len, int num_splits, int n_cta, int hpc, mla::Problem* pb) {
  MLA_CHECK(batch >= 0, "batch must be non-negative");
  MLA_CHECK(heads > 0 && heads % 16 == 0, "heads must be a multiple of 16, got %d", heads);
  MLA_CHECK(num_splits >= 0, "num_splits must be non-negative");
  const int splits = num_splits > 0 ? num_splits : 1;
  const long long len = max_kv_len > 1 ? max_kv_len : 1;
  const long long chunk = ((len + splits - 1) / splits + mla::TILE - 1) / mla::TILE * mla::TILE;
  pb->batch = batch, pb->heads = heads, pb->heads_per_cta = hpc, pb->head_groups = heads / hpc;
  pb->splits = splits, pb->chunk = int(chunk), pb->n_cta = n_cta;
  MLA_CHECK((long long)batch * splits <= mla::kSchedMaxBZ, "batch * num_splits = %lld exceeds %d", (long long)batch * splits,
            mla::kSchedMaxBZ);
  MLA_CHECK(splits + n_cta <= 512, "num_splits %d too large (at most %d)", splits, 512 - n_cta);
  return 0;
}

}  // namespace

extern "C" {

int nvfp4_mla_version(void) { return 100; }

const char* nvfp4_mla_last_error(void) { return g_error; }

// Whether the decode kernel derives the schedule by itself (one thread per (request, split) pair, 32-bit tile counts)
// or reads the output of a schedule kernel launched in front of it.
static bool schedules_itself(const mla::Problem& pb, int precision, int hpc) {
  const long long bz = (long long)pb.batch * pb.splits;
  return bz <= (long long)decode_threads(precision, hpc) &&
         bz * ((pb.chunk + mla::TILE - 1) / mla::TILE + 1) * pb.head_groups < (1ll << 31);
}

// workspace of one precision mode (the modes may group the heads differently); negative on error
static int64_t workspace_bytes_of(int batch, int heads, int num_splits, int precision, int hpc_limit = 128) {
  DeviceInfo* d;
  if (device_info(&d)) return -1;
  mla::Problem pb;
  const int hpc = heads_per_cta(heads, precision, *d, hpc_limit);
  if (problem_of(batch, heads, 1, num_splits, schedule_units(*d, hpc), hpc, &pb)) return -1;
  return int64_t(mla::ws_layout(pb.n_cta, pb.items(), pb.heads_per_cta).total);
}

int nvfp4_mla_decode_launches(int batch, int heads, int max_kv_len, int num_splits, int precision) {
  g_error[0] = 0;
  if (precision != NVFP4_MLA_PRECISION_BF16 && precision != NVFP4_MLA_PRECISION_FP8) {
    fail("precision must be 0 (bf16) or 1 (fp8), got %d", precision);
    return -1;
  }
  DeviceInfo* d;
  if (device_info(&d)) return -1;
  mla::Problem pb;
  const int hpc = heads_per_cta(heads, precision, *d, 128);
  if (problem_of(batch, heads, max_kv_len, num_splits, schedule_units(*d, hpc), hpc, &pb)) return -1;
  if (batch == 0) return 0;
  return schedules_itself(pb, precision, hpc) ? 2 : 3;
}

int64_t nvfp4_mla_decode_workspace_bytes(int batch, int heads, int num_splits) {
  // the size covers either precision mode
  const int64_t a = workspace_bytes_of(batch, heads, num_splits, NVFP4_MLA_PRECISION_BF16);
  const int64_t b = workspace_bytes_of(batch, heads, num_splits, NVFP4_MLA_PRECISION_FP8);
  return a < 0 || b < 0 ? -1 : (a > b ? a : b);
}

// The decode call proper; `hpc_limit` caps the heads per CTA (see heads_per_cta).
static int decode_impl(const void* q_nope, const void* q_pe, const uint8_t* ckv_cache, const uint8_t* ckv_sf_cache,
                       const uint8_t* kpe_cache, int64_t num_pages, int page_size, const int32_t* page_table,
                       int64_t page_table_stride, const int32_t* kv_lens, int batch, int heads, float sm_scale, float ckv_scale,
                       float kpe_scale, int max_kv_len, int num_splits, int precision, void* out, float* out_f32, float* lse,
                       void* workspace, int64_t workspace_bytes, void* stream, int hpc_limit) {
  g_error[0] = 0;
  MLA_CHECK(precision == NVFP4_MLA_PRECISION_BF16 || precision == NVFP4_MLA_PRECISION_FP8,
            "precision must be 0 (bf16) or 1 (fp8), got %d", precision);
  MLA_CHECK(page_size > 0 && (page_size & (page_size - 1)) == 0, "page_size must be a power of two, got %d", page_size);
  MLA_CHECK(num_pages > 0 && num_pages * page_size < (int64_t(1) << 31), "num_pages * page_size must be in [1, 2^31)");
  MLA_CHECK(ckv_scale > 0.f && kpe_scale > 0.f, "ckv_scale and kpe_scale must be positive");
  MLA_CHECK(q_nope && q_pe && ckv_cache && ckv_sf_cache && kpe_cache && page_table && kv_lens && workspace, "null pointer argument");
  MLA_CHECK(out || out_f32 || lse, "at least one of out, out_f32 and lse must be given");
  MLA_CHECK(aligned(q_nope, 16) && aligned(q_pe, 16) && aligned(ckv_cache, 16) && aligned(ckv_sf_cache, 16) &&
                aligned(kpe_cache, 16) && aligned(workspace, 256) && aligned(out, 16) && aligned(out_f32, 16),
            "q, caches and outputs must be 16-byte aligned and the workspace 256-byte aligned");
  MLA_CHECK(page_table_stride >= 0, "page_table_stride must be non-negative");
  DeviceInfo* d;
  if (device_info(&d)) return 1;
  mla::Problem pb;
  const int hpc = heads_per_cta(heads, precision, *d, hpc_limit);
  if (problem_of(batch, heads, max_kv_len, num_splits, schedule_units(*d, hpc), hpc, &pb)) return 1;
  if (batch == 0) return 0;
  const mla::WsLayout L = mla::ws_layout(pb.n_cta, pb.items(), pb.heads_per_cta);
  MLA_CHECK(workspace_bytes >= int64_t(L.total), "workspace too small: %lld bytes given, %lld needed", (long long)workspace_bytes,
            (long long)L.total);

  CUtensorMap ckv_map, sf_map, kpe_map;
  const int slot_rows = hpc == 128 ? mla::kHmRows : mla::HALF;  // tokens per staging slot of the kernel that will run
  if (make_row_map(ckv_cache, num_pages * page_size, 256, 128, page_size, slot_rows, CU_TENSOR_MAP_SWIZZLE_128B, &ckv_map)) return 1;
  if (make_row_map(ckv_sf_cache, num_pages * page_size, 32, 32, page_size, slot_rows, CU_TENSOR_MAP_SWIZZLE_32B, &sf_map)) return 1;
  if (make_row_map(kpe_cache, num_pages * page_size, 64, 64, page_size, slot_rows, CU_TENSOR_MAP_SWIZZLE_64B, &kpe_map)) return 1;

  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int* header = reinterpret_cast<int*>(ws + L.header);
  int2* cta_range = reinterpret_cast<int2*>(ws + L.cta_range);
  int2* item_range = reinterpret_cast<int2*>(ws + L.item_range);
  mla::Seg* segs = reinterpret_cast<mla::Seg*>(ws + L.segs);
  float* lse_part = reinterpret_cast<float*>(ws + L.lse_part);
  float* o_part = reinterpret_cast<float*>(ws + L.o_part);
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  // The decode kernels derive their schedule by themselves when one thread per (request, split) pair is enough; larger
  // batches read the output of the schedule kernel.
  const bool inline_sched = schedules_itself(pb, precision, hpc);
  if (!inline_sched) {
    mla::mla_schedule_kernel<<<1, mla::kSchedThreads, 0, st>>>(kv_lens, pb, header, cta_range, item_range, segs);
    MLA_CUDA(cudaGetLastError());
  }

  mla::DecodeParams P;
  P.q_nope = static_cast<const __nv_bfloat16*>(q_nope), P.q_pe = static_cast<const __nv_bfloat16*>(q_pe);
  P.ckv = ckv_cache, P.sf = ckv_sf_cache, P.kpe = kpe_cache, P.page_table = page_table, P.pt_stride = page_table_stride;
  P.page_shift = __builtin_ctz(unsigned(page_size)), P.num_pages = int(num_pages), P.heads = heads, P.heads_per_cta = hpc;
  P.sf_swz_mask = page_size >= slot_rows ? 1u : 0u, P.kpe_swz_mask = page_size >= slot_rows ? 3u : 0u;
  P.sm_scale_log2 = sm_scale * 1.4426950408889634f, P.ckv_scale = ckv_scale, P.kpe_scale = kpe_scale;
  P.cta_range = cta_range, P.segs = segs, P.lse_part = lse_part, P.o_part = o_part, P.header = header;
  P.kv_lens = kv_lens, P.pb = pb, P.inline_sched = inline_sched ? 1 : 0, P.item_range = item_range;
  P.cta_range_out = cta_range, P.segs_out = segs;
  Profile* prof = g_profile && g_profile->used < int(g_profile->start.size()) ? g_profile : nullptr;
  if (prof) MLA_CUDA(cudaEventRecord(prof->start[prof->used], st));
  MLA_CUDA(launch_dependent_cluster(decode_kernel(precision, hpc), dim3(pb.n_cta * ctas_per_unit(hpc)),
                                    dim3(decode_threads(precision, hpc)), decode_smem(precision, hpc), st,
                                    unsigned(ctas_per_unit(hpc)), ckv_map, sf_map, kpe_map, P));
  if (prof) MLA_CUDA(cudaEventRecord(prof->stop[prof->used++], st));

  // few rows: four thread groups share a row's partials; many rows: one group per row keeps the CTAs small
  const unsigned rows = unsigned(batch) * unsigned(heads);
  if (rows <= 2u * unsigned(d->sm_count))
    MLA_CUDA(launch_dependent(mla::mla_combine_sched_kernel<4>, dim3(rows), dim3(512), 0, st, pb,
                              static_cast<const int2*>(item_range), static_cast<const int*>(inline_sched ? kv_lens : nullptr),
                              static_cast<const float*>(lse_part),
                              static_cast<const float*>(o_part), out, out_f32, lse));
  else
    MLA_CUDA(launch_dependent(mla::mla_combine_sched_kernel<1>, dim3(rows), dim3(128), 0, st, pb,
                              static_cast<const int2*>(item_range), static_cast<const int*>(inline_sched ? kv_lens : nullptr),
                              static_cast<const float*>(lse_part),
                              static_cast<const float*>(o_part), out, out_f32, lse));
  return 0;
}

int nvfp4_mla_decode(const void* q_nope, const void* q_pe, const uint8_t* ckv_cache, const uint8_t* ckv_sf_cache,
                     const uint8_t* kpe_cache, int64_t num_pages, int page_size, const int32_t* page_table,
                     int64_t page_table_stride, const int32_t* kv_lens, int batch, int heads, float sm_scale, float ckv_scale,
                     float kpe_scale, int max_kv_len, int num_splits, int precision, void* out, float* out_f32, float* lse,
                     void* workspace, int64_t workspace_bytes, void* stream) {
  return decode_impl(q_nope, q_pe, ckv_cache, ckv_sf_cache, kpe_cache, num_pages, page_size, page_table, page_table_stride, kv_lens,
                     batch, heads, sm_scale, ckv_scale, kpe_scale, max_kv_len, num_splits, precision, out, out_f32, lse, workspace,
                     workspace_bytes, stream, 128);
}

// ---- decode without caller-provided scratch -----------------------------------------------------------------------
// Scratch for nvfp4_mla_decode_static: lives in the library's own device image, so no allocation ever happens for it.
// Every GPU that loads the library holds these bytes until the process exits.
constexpr size_t kStaticScratchBytes = size_t(9) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
void* g_static_scratch_ptr[kMaxDevices] = {};  // device address of g_static_scratch, per device (set up on first use)

// The array's name is only a host-side handle; kernels need its device address, which differs per device.
int static_scratch(void** out) {
  int dev = 0;
  MLA_CUDA(cudaGetDevice(&dev));
  MLA_CHECK(dev >= 0 && dev < kMaxDevices, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_static_scratch_ptr[dev]) {
    void* p = nullptr;
    MLA_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    MLA_CHECK(p != nullptr, "cudaGetSymbolAddress returned a null address for the static scratch");
    g_static_scratch_ptr[dev] = p;
  }
  *out = g_static_scratch_ptr[dev];
  return 0;
}
}  // namespace

int64_t nvfp4_mla_decode_static_capacity(void) { return int64_t(kStaticScratchBytes); }

int nvfp4_mla_decode_static(const void* q_nope, const void* q_pe, const uint8_t* ckv_cache, const uint8_t* ckv_sf_cache,
                            const uint8_t* kpe_cache, int64_t num_pages, int page_size, const int32_t* page_table,
                            int64_t page_table_stride, const int32_t* kv_lens, int batch, int heads, float sm_scale,
                            float ckv_scale, float kpe_scale, int max_kv_len, int num_splits, int precision, void* out,
                            float* out_f32, float* lse, void* stream) {
  g_error[0] = 0;
  MLA_CHECK(precision == NVFP4_MLA_PRECISION_BF16 || precision == NVFP4_MLA_PRECISION_FP8,
            "precision must be 0 (bf16) or 1 (fp8), got %d", precision);
  // The widest grouping of heads per CTA whose partial results fit the array: the 8-bit mode prefers 128 or 32 heads
  // per CTA (2 KB of partial result per head and CTA), which needs more scratch than 16 heads per CTA do.
  int limit = 128;
  int64_t need = -1;
  for (; limit >= 16; limit = limit == 128 ? 32 : limit == 32 ? 16 : 0) {
    need = workspace_bytes_of(batch, heads, num_splits, precision, limit);
    if (need < 0) return 1;  // message already set
    if (need <= int64_t(kStaticScratchBytes)) break;
  }
  MLA_CHECK(limit >= 16,
            "problem too large for the built-in scratch: batch %d x heads %d x num_splits %d needs %lld bytes, the library holds "
            "%lld; use nvfp4_mla_decode with a caller-provided workspace",
            batch, heads, num_splits, (long long)need, (long long)kStaticScratchBytes);
  void* scratch = nullptr;
  if (static_scratch(&scratch)) return 1;
  // Nothing of the array has to be cleared per call: the schedule kernel rewrites every record the other kernels read,
  // and the status word (zero when the library is loaded) is sticky until nvfp4_mla_decode_static_status clears it.
  return decode_impl(q_nope, q_pe, ckv_cache, ckv_sf_cache, kpe_cache, num_pages, page_size, page_table, page_table_stride, kv_lens,
                     batch, heads, sm_scale, ckv_scale, kpe_scale, max_kv_len, num_splits, precision, out, out_f32, lse, scratch,
                     int64_t(kStaticScratchBytes), stream, limit);
}

int nvfp4_mla_decode_static_status(void* stream) {
  g_error[0] = 0;
  void* scratch = nullptr;
  if (static_scratch(&scratch)) return -1;
  const int status = nvfp4_mla_workspace_status(scratch, stream);
  if (status > 0) {  // reported once: start the next run of calls from a clean word
    cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(int), static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return -fail("clearing the status word failed: %s", cudaGetErrorString(e));
  }
  return status;
}

int nvfp4_mla_profile_begin(int capacity) {
  g_error[0] = 0;
  MLA_CHECK(capacity > 0 && capacity <= (1 << 20), "capacity must be in [1, 2^20]");
  MLA_CHECK(g_profile == nullptr, "a profile is already open on this thread");
  Profile* p = new Profile;
  p->start.resize(capacity), p->stop.resize(capacity);
  for (int i = 0; i < capacity; ++i) {
    MLA_CUDA(cudaEventCreate(&p->start[i]));
    MLA_CUDA(cudaEventCreate(&p->stop[i]));
  }
  g_profile = p;
  return 0;
}

int nvfp4_mla_profile_end(float* ms, int capacity) {
  g_error[0] = 0;
  Profile* p = g_profile;
  if (!p) return -fail("no profile is open on this thread");
  g_profile = nullptr;
  int n = p->used < capacity ? p->used : capacity, rc = n;
  for (int i = 0; i < p->used; ++i) {
    cudaError_t e = cudaEventSynchronize(p->stop[i]);
    if (e == cudaSuccess && i < n) e = cudaEventElapsedTime(&ms[i], p->start[i], p->stop[i]);
    if (e != cudaSuccess) rc = -fail("reading kernel timings failed: %s", cudaGetErrorString(e));
  }
  for (size_t i = 0; i < p->start.size(); ++i) cudaEventDestroy(p->start[i]), cudaEventDestroy(p->stop[i]);
  delete p;
  return rc;
}

int nvfp4_mla_workspace_status(const void* workspace, void* stream) {
  g_error[0] = 0;
  if (!workspace) return -fail("null workspace");
  int status = 0;
  cudaError_t e = cudaMemcpyAsync(&status, workspace, sizeof status, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return -fail("reading the workspace status failed: %s", cudaGetErrorString(e));
  return status;
}

int nvfp4_mla_dequantize(const uint8_t* ckv_cache, const uint8_t* ckv_sf_cache, const uint8_t* kpe_cache, int64_t num_tokens,
                         float ckv_scale, float kpe_scale, int out_bf16, void* ckv_out, void* kpe_out, void* stream) {
  g_error[0] = 0;
  MLA_CHECK(num_tokens >= 0, "num_tokens must be non-negative");
  if (num_tokens == 0) return 0;
  MLA_CHECK(ckv_cache && ckv_sf_cache && kpe_cache && ckv_out && kpe_out, "null pointer argument");
  MLA_CHECK(aligned(ckv_cache, 4) && aligned(kpe_cache, 2) && aligned(ckv_out, 16) && aligned(kpe_out, 8),
            "ckv_cache must be 4-byte and kpe_cache 2-byte aligned, ckv_out 16-byte and kpe_out 8-byte aligned");
  DeviceInfo* d;
  if (device_info(&d)) return 1;
  const long long warps_per_block = mla::kDequantThreads / 32;
  long long blocks = (num_tokens + warps_per_block - 1) / warps_per_block;
  const long long cap = (long long)d->sm_count * 32;  // grid-stride beyond 32 CTAs per SM
  if (blocks > cap) blocks = cap;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_bf16)
    mla::mla_dequant_kernel<__nv_bfloat16><<<unsigned(blocks), mla::kDequantThreads, 0, st>>>(
        ckv_cache, ckv_sf_cache, kpe_cache, ckv_scale, kpe_scale, static_cast<__nv_bfloat16*>(ckv_out),
        static_cast<__nv_bfloat16*>(kpe_out), num_tokens);
  else
    mla::mla_dequant_kernel<float><<<unsigned(blocks), mla::kDequantThreads, 0, st>>>(
        ckv_cache, ckv_sf_cache, kpe_cache, ckv_scale, kpe_scale, static_cast<float*>(ckv_out), static_cast<float*>(kpe_out),
        num_tokens);
  MLA_CUDA(cudaGetLastError());
  return 0;
}

int nvfp4_mla_quantize_append(const void* ckv, const void* kpe, const int32_t* batch_indices, const int32_t* positions,
                              int64_t nnz, uint8_t* ckv_cache, uint8_t* ckv_sf_cache, uint8_t* kpe_cache, int64_t num_pages,
                              int page_size, const int32_t* kv_indices, const int32_t* kv_indptr, int batch, float ckv_scale,
                              float kpe_scale, int32_t* status, void* stream) {
  g_error[0] = 0;
  MLA_CHECK(nnz >= 0 && batch >= 0, "nnz and batch must be non-negative");
  MLA_CHECK(page_size > 0 && (page_size & (page_size - 1)) == 0, "page_size must be a power of two, got %d", page_size);
  MLA_CHECK(num_pages > 0 && num_pages * page_size < (int64_t(1) << 31), "num_pages * page_size must be in [1, 2^31)");
  MLA_CHECK(ckv_scale > 0.f && kpe_scale > 0.f, "ckv_scale and kpe_scale must be positive");
  if (nnz == 0) return 0;
  MLA_CHECK(ckv && kpe && batch_indices && positions && ckv_cache && ckv_sf_cache && kpe_cache && kv_indices && kv_indptr,
            "null pointer argument");
  MLA_CHECK(aligned(ckv, 16) && aligned(kpe, 4) && aligned(ckv_cache, 8) && aligned(kpe_cache, 2),
            "ckv must be 16-byte, kpe 4-byte, ckv_cache 8-byte and kpe_cache 2-byte aligned");
  DeviceInfo* d;
  if (device_info(&d)) return 1;
  const long long warps_per_block = mla::kQuantThreads / 32;
  long long blocks = (nnz + warps_per_block - 1) / warps_per_block;
  const long long cap = (long long)d->sm_count * 32;  // grid-stride beyond 32 CTAs per SM
  if (blocks > cap) blocks = cap;
  mla::mla_quantize_append_kernel<<<unsigned(blocks), mla::kQuantThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(ckv), static_cast<const __nv_bfloat16*>(kpe), batch_indices, positions, nnz, ckv_cache,
      ckv_sf_cache, kpe_cache, num_pages, __builtin_ctz(unsigned(page_size)), kv_indices, kv_indptr, batch, ckv_scale, kpe_scale,
      status);
  MLA_CUDA(cudaGetLastError());
  return 0;
}

int nvfp4_mla_combine_strided(const float* o_part, const float* lse_part, int parts, int64_t rows, int64_t o_part_stride,
                              int64_t lse_part_stride, void* out, float* out_f32, float* lse, void* stream) {
  g_error[0] = 0;
  MLA_CHECK(parts > 0 && rows >= 0, "parts must be positive and rows non-negative");
  MLA_CHECK(parts <= mla::kCombineMaxParts, "at most %d partials per row, got %d", mla::kCombineMaxParts, parts);
  if (rows == 0) return 0;
  MLA_CHECK(o_part && lse_part, "null pointer argument");
  MLA_CHECK(out || out_f32 || lse, "at least one of out, out_f32 and lse must be given");
  MLA_CHECK(aligned(o_part, 16) && aligned(out, 8) && aligned(out_f32, 16), "o_part and out_f32 must be 16-byte, out 8-byte aligned");
  MLA_CHECK(o_part_stride >= rows * mla::CKV && o_part_stride % 4 == 0 && lse_part_stride >= rows,
            "o_part_stride must be a multiple of 4 floats and at least rows * 512, lse_part_stride at least rows");
  MLA_CHECK(rows < (int64_t(1) << 31), "rows must be below 2^31");
  if (rows <= 296)
    mla::mla_combine_dense_kernel<4><<<unsigned(rows), 512, 0, static_cast<cudaStream_t>(stream)>>>(
        o_part, lse_part, parts, rows, o_part_stride, lse_part_stride, out, out_f32, lse);
  else
    mla::mla_combine_dense_kernel<1><<<unsigned(rows), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        o_part, lse_part, parts, rows, o_part_stride, lse_part_stride, out, out_f32, lse);
  MLA_CUDA(cudaGetLastError());
  return 0;
}

int nvfp4_mla_combine_records(const float* const* records, int parts, int64_t rows, void* out, float* out_f32, float* lse,
                              void* stream) {
  g_error[0] = 0;
  MLA_CHECK(parts > 0 && rows >= 0, "parts must be positive and rows non-negative");
  MLA_CHECK(parts <= mla::kCombineMaxRecords, "at most %d records, got %d", mla::kCombineMaxRecords, parts);
  if (rows == 0) return 0;
  MLA_CHECK(records, "null pointer argument");
  MLA_CHECK(out || out_f32 || lse, "at least one of out, out_f32 and lse must be given");
  MLA_CHECK(aligned(out, 8) && aligned(out_f32, 16), "out_f32 must be 16-byte, out 8-byte aligned");
  MLA_CHECK(rows < (int64_t(1) << 31), "rows must be below 2^31");
  mla::RecordPtrs recs = {};
  for (int i = 0; i < parts; ++i) {
    MLA_CHECK(records[i] && aligned(records[i], 16), "record %d is null or not 16-byte aligned", i);
    recs.p[i] = records[i];
  }
  if (rows <= 296)
    mla::mla_combine_records_kernel<4><<<unsigned(rows), 512, 0, static_cast<cudaStream_t>(stream)>>>(recs, parts, rows, out, out_f32, lse);
  else
    mla::mla_combine_records_kernel<1><<<unsigned(rows), 128, 0, static_cast<cudaStream_t>(stream)>>>(recs, parts, rows, out, out_f32, lse);
  MLA_CUDA(cudaGetLastError());
  return 0;
}

int nvfp4_mla_combine_records_signalled(const float* const* records, uint32_t* const* flags, int rank, uint32_t epoch,
                                        int64_t wait_us, int parts, int64_t rows, void* out, float* out_f32, float* lse,
                                        int* status, void* stream) {
  g_error[0] = 0;
  MLA_CHECK(parts > 0 && rows > 0, "parts and rows must be positive (every GPU has to run the hand-shake)");
  MLA_CHECK(parts <= mla::kCombineMaxRecords, "at most %d records, got %d", mla::kCombineMaxRecords, parts);
  MLA_CHECK(rank >= 0 && rank < parts, "rank %d outside [0, %d)", rank, parts);
  MLA_CHECK(wait_us > 0, "wait_us must be positive: an unbounded wait is not offered");
  MLA_CHECK(records && flags, "null pointer argument");
  MLA_CHECK(out || out_f32 || lse, "at least one of out, out_f32 and lse must be given");
  MLA_CHECK(aligned(out, 8) && aligned(out_f32, 16), "out_f32 must be 16-byte, out 8-byte aligned");
  MLA_CHECK(aligned(status, 4), "status must be 4-byte aligned");
  MLA_CHECK(rows < (int64_t(1) << 31), "rows must be below 2^31");
  mla::RecordPtrs recs = {};
  mla::FlagPtrs fl = {};
  for (int i = 0; i < parts; ++i) {
    MLA_CHECK(records[i] && aligned(records[i], 16), "record %d is null or not 16-byte aligned", i);
    MLA_CHECK(flags[i] && aligned(flags[i], 4), "flag array %d is null or not 4-byte aligned", i);
    recs.p[i] = records[i], fl.p[i] = flags[i];
  }
  const unsigned long long wait_ns = (unsigned long long)wait_us * 1000ull;
  auto st = static_cast<cudaStream_t>(stream);
  if (rows <= 296)
    mla::mla_combine_records_signalled_kernel<4><<<unsigned(rows), 512, 0, st>>>(recs, fl, rank, epoch, wait_ns, parts, rows, out, out_f32, lse, status);
  else
    mla::mla_combine_records_signalled_kernel<1><<<unsigned(rows), 128, 0, st>>>(recs, fl, rank, epoch, wait_ns, parts, rows, out, out_f32, lse, status);
  MLA_CUDA(cudaGetLastError());
  return 0;
}

int nvfp4_mla_combine(const float* o_part, const float* lse_part, int parts, int64_t rows, void* out, float* out_f32, float* lse,
                      void* stream) {
  return nvfp4_mla_combine_strided(o_part, lse_part, parts, rows, rows * mla::CKV, rows, out, out_f32, lse, stream);
}

}  // extern "C"
