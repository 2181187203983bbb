// Split-KV schedule, computed on the device from kv_lens so that the launch shape of the decode kernel never
// depends on host-visible lengths (no host sync, CUDA-graph safe).
//
// The (request, split, head-group) items are laid end to end in units of 128-token tiles and the flattened tile
// range is cut into n_cta equal pieces, one per decode CTA: every SM streams the same number of tiles whatever the
// mix of request lengths. A CTA whose piece spans several items produces one partial (o, lse) per item it touches;
// the partial of (cta, item w) lives in slot cta + w, which is unique because both indices only grow along the cut.
#pragma once
#include "mla_common.cuh"
#include "ptx_sm100.cuh"

namespace mla {

constexpr int kSchedThreads = 1024;
constexpr int kSchedMaxBZ = 8192;  // batch * splits the single-block scan holds in shared memory

__global__ void __launch_bounds__(kSchedThreads, 1)
mla_schedule_kernel(const int* __restrict__ kv_lens, Problem pb, int* header, int2* cta_range, int2* item_range, Seg* segs) {
  __shared__ int tiles[kSchedMaxBZ];      // tiles of (b, z), then its exclusive prefix
  __shared__ int warp_sums[kSchedThreads / 32];
  __shared__ int total_bz;
  ptx::grid_launch_dependents();  // the decode kernel may start its prologue; it waits for this grid before reading
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int BZ = pb.batch * pb.splits;
  if (BZ > kSchedMaxBZ) {
    if (tid == 0) header[0] = kBadSchedule;
    return;
  }
  const int HG = pb.head_groups;

  // ---- tiles per (b, z) and their exclusive prefix (block scan, kSchedMaxBZ / kSchedThreads entries per thread)
  constexpr int PER = kSchedMaxBZ / kSchedThreads;
  int local[PER], sum = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int bz = tid * PER + j;
    int t = 0;
    if (bz < BZ) {
      const int b = bz / pb.splits, z = bz % pb.splits;
      const int len = kv_lens[b];
      const long long lo = (long long)z * pb.chunk;
      long long n = (long long)len - lo;
      n = n < 0 ? 0 : (n > pb.chunk ? pb.chunk : n);
      t = int((n + TILE - 1) / TILE);
    }
    local[j] = sum;
    sum += t;
  }
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(~0u, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int v = warp_sums[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(~0u, v, o);
      if (lane >= o) v += u;
    }
    warp_sums[lane] = v;  // inclusive over warps
    if (lane == 31) total_bz = v;
  }
  __syncthreads();
  const int base = incl - sum + (warp ? warp_sums[warp - 1] : 0);
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int bz = tid * PER + j;
    if (bz < BZ) tiles[bz] = base + local[j];  // exclusive prefix of tiles over (b, z)
  }
  __syncthreads();
  const long long T = (long long)total_bz * HG;
  const int q = int(T > 0 ? (T + pb.n_cta - 1) / pb.n_cta : 1);
  if (tid == 0) header[1] = int(T), header[2] = q;
  auto prefix = [&](int bz) { return bz < BZ ? tiles[bz] : total_bz; };  // exclusive prefix, in (b, z) tiles
  auto tiles_of = [&](int bz) { return prefix(bz + 1) - prefix(bz); };

  // ---- invalidate every slot, then fill the live ones
  const long long W = pb.items();
  for (long long i = tid; i < W + pb.n_cta; i += kSchedThreads) segs[i].cta = -1, segs[i].ntiles = 0;
  __syncthreads();

  // ---- per CTA: the items its tile range [c * q, (c + 1) * q) touches
  for (int c = tid; c < pb.n_cta; c += kSchedThreads) {
    const long long g0 = (long long)c * q, g1 = (g0 + q < T ? g0 + q : T);
    int2 r = make_int2(0, 0);
    if (g0 < g1) {
      auto item_of = [&](long long g) {  // item containing flat tile g
        int lo = 0, hi = BZ - 1;         // last bz with HG * prefix(bz) <= g
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if ((long long)HG * prefix(mid) <= g) lo = mid; else hi = mid - 1;
        }
        const int t = tiles_of(lo);
        const int hg = t > 0 ? int((g - (long long)HG * prefix(lo)) / t) : 0;
        return lo * HG + hg;
      };
      r = make_int2(item_of(g0), item_of(g1 - 1) + 1);
    }
    cta_range[c] = r;
  }

  // ---- per item: the CTAs that hold a piece of it, and one Seg per piece
  for (long long w = tid; w < W; w += kSchedThreads) {
    const int bz = int(w / HG), hg = int(w % HG);
    const int t = tiles_of(bz);
    if (t == 0) {
      item_range[w] = make_int2(0, -1);
      continue;
    }
    const int b = bz / pb.splits, z = bz % pb.splits;
    const long long P = (long long)HG * prefix(bz) + (long long)hg * t;
    const int c0 = int(P / q), c1 = int((P + t - 1) / q);
    item_range[w] = make_int2(c0, c1);
    const int len = kv_lens[b];
    const long long end = (long long)(z + 1) * pb.chunk;
    for (int c = c0; c <= c1; ++c) {
      const long long lo = ((long long)c * q > P ? (long long)c * q : P) - P;
      const long long hi = ((long long)(c + 1) * q < P + t ? (long long)(c + 1) * q : P + t) - P;
      Seg s;
      s.b = b, s.hg = hg, s.tok0 = z * pb.chunk + int(lo) * TILE, s.ntiles = int(hi - lo);
      s.tok_end = int(end < len ? end : len), s.w = int(w), s.cta = c, s.pad = 0;
      segs[c + w] = s;
    }
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------------------------------------------
// Merge of the partials of one output row (b, h): out = sum_i 2^(lse_i - M) o_i / sum_i 2^(lse_i - M).
// One CTA per row: GROUPS groups of 128 threads, each thread owns 4 channels; group g takes the partials
// i = g, g + GROUPS, ... in batches of 8 independent 16-byte loads (a row with a hundred partials, one long request
// spread over every SM, is a chain of memory latencies otherwise), and the groups' sums meet in shared memory. The
// host picks GROUPS = 4 when there are few rows (their CTAs cannot fill the GPU anyway) and 1 when there are many. Log-sum-exp
// weights are computed by the lanes of a warp in parallel (one partial per lane) and reduced with shuffles; every
// warp repeats that small reduction so the warps only meet once.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kCombineMaxGroups = 4;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(~0u, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(~0u, v, o);
  return v;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

// Shared tail: `n_parts` partials whose (lse, o-row) addresses are produced by `lse_of(i)` / `o_of(i)`.
// `weights` and `partial` are shared-memory scratch of at least n_parts (up to kCombineMaxParts) and 3 x 128 x 4 floats.
constexpr int kCombineMaxParts = 512;
template <int GROUPS, class LseOf, class OOf>
__device__ __forceinline__ void merge_row(int n_parts, LseOf lse_of, OOf o_of, long long row, void* out_bf16,
                                          float* out_f32, float* lse_out, float* weights, float4* partial) {
  const int lane = threadIdx.x & 31, grp = threadIdx.x >> 7, t = threadIdx.x & 127;
  // The first batch of rows is requested before the weights are known (they need the lse values, another round trip to
  // memory): a row with a handful of partials, the common case, then costs one memory latency instead of two. A partial
  // of weight 0 may hold anything, so its values are dropped by a select, not multiplied away.
  float4 v0[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int i = grp + j * GROUPS;
    v0[j] = i < n_parts ? reinterpret_cast<const float4*>(o_of(i))[t] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float M = -INFINITY;
  for (int i = lane; i < n_parts; i += 32) M = fmaxf(M, lse_of(i));
  M = warp_max(M);
  float den = 0.f;
  for (int i = lane; i < n_parts; i += 32) {
    const float wl = M > -INFINITY ? exp2f(lse_of(i) - M) : 0.f;  // lse = -inf (empty partial) gives weight 0
    den += wl;
    if (threadIdx.x < 32 && i < kCombineMaxParts) weights[i] = wl;
  }
  den = warp_sum(den);
  __syncthreads();
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  auto add = [&](float w, const float4& v) {
    if (w != 0.f) acc.x += w * v.x, acc.y += w * v.y, acc.z += w * v.z, acc.w += w * v.w;
  };
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int i = grp + j * GROUPS;
    add(i < n_parts ? weights[i] : 0.f, v0[j]);
  }
  for (int i0 = grp + 8 * GROUPS; i0 < n_parts; i0 += 8 * GROUPS) {
    float4 v[8];
    float w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = i0 + j * GROUPS;
      w[j] = i < n_parts ? weights[i] : 0.f;
      v[j] = w[j] != 0.f ? reinterpret_cast<const float4*>(o_of(i))[t] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) add(w[j], v[j]);
  }
  if (GROUPS > 1) {
    if (grp > 0) partial[(grp - 1) * 128 + t] = acc;
    __syncthreads();
    if (grp > 0) return;
#pragma unroll
    for (int g = 0; g < GROUPS - 1; ++g) {
      const float4 o = partial[g * 128 + t];
      acc.x += o.x, acc.y += o.y, acc.z += o.z, acc.w += o.w;
    }
  }
  const float s = den > 0.f ? 1.f / den : 0.f;
  acc.x *= s, acc.y *= s, acc.z *= s, acc.w *= s;
  if (out_bf16)
    reinterpret_cast<uint2*>(out_bf16)[row * (CKV / 4) + t] = make_uint2(pack_bf16x2(acc.x, acc.y), pack_bf16x2(acc.z, acc.w));
  if (out_f32) reinterpret_cast<float4*>(out_f32)[row * (CKV / 4) + t] = acc;
  if (lse_out && t == 0) lse_out[row] = den > 0.f ? M + log2f(den) : -INFINITY;
}

// Partials addressed through the schedule (what the decode kernel wrote).
template <int GROUPS>
__global__ void __launch_bounds__(128 * GROUPS)
mla_combine_sched_kernel(Problem pb, const int2* __restrict__ item_range, const int* __restrict__ kv_lens,
                         const float* __restrict__ lse_part, const float* __restrict__ o_part, void* out_bf16, float* out_f32,
                         float* lse_out) {
  __shared__ int slots[kCombineMaxParts];
  __shared__ int n_parts_s;
  __shared__ float weights[kCombineMaxParts];
  __shared__ float4 partial[GROUPS > 1 ? (GROUPS - 1) * 128 : 1];
  // Launched as a programmatic dependent of the decode kernel, which lets its dependents start only after it has seen
  // the schedule kernel complete: the schedule kernel's output (item_range) may be read at once, the partials (and an
  // item_range written by the decode kernel itself) only after the wait.
  const long long row = blockIdx.x;
  const int b = int(row / pb.heads), h = int(row % pb.heads);
  const int N = pb.heads_per_cta, hg = h / N, n = h % N;
  if (threadIdx.x < 32) {  // enumerate the row's partial slots: splits z, CTAs c0..c1 of item (b, z, hg)
    // Without a schedule kernel (kv_lens given: the decode kernel derived its schedule by itself) the CTA that holds
    // the first tile of an item has written the item's CTA range; an item without tiles has none, which the lengths tell.
    int count = 0;
    for (int z0 = 0; z0 < pb.splits; z0 += 32) {
      const int z = z0 + threadIdx.x;
      int c0 = 0, c1 = -1;
      long long w = 0;
      if (z < pb.splits) w = ((long long)b * pb.splits + z) * pb.head_groups + hg;
      if (kv_lens) {
        // the two loads are independent (a stale range is read and dropped): one memory latency, not two in a row
        const int t = z < pb.splits ? sched_tiles(kv_lens, pb, b * pb.splits + z) : 0;
        ptx::grid_dependency_wait();  // item_range is the decode kernel's output here
        const int2 r = z < pb.splits ? item_range[w] : make_int2(0, -1);
        if (t > 0) c0 = r.x, c1 = r.y;
      } else if (z < pb.splits) {
        const int2 r = item_range[w];
        c0 = r.x, c1 = r.y;
      }
      const int mine = c1 >= c0 ? c1 - c0 + 1 : 0;
      int incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(~0u, incl, o);
        if (int(threadIdx.x) >= o) incl += v;
      }
      int pos = count + incl - mine;
      for (int c = c0; c <= c1; ++c, ++pos)
        if (pos < kCombineMaxParts) slots[pos] = int(c + w);
      count += __shfl_sync(~0u, incl, 31);
    }
    if (threadIdx.x == 0) n_parts_s = count < kCombineMaxParts ? count : kCombineMaxParts;
  }
  __syncthreads();
  const int n_parts = n_parts_s;
  ptx::grid_dependency_wait();
  merge_row<GROUPS>(
      n_parts, [&](int i) { return lse_part[(long long)slots[i] * N + n]; },
      [&](int i) { return o_part + ((long long)slots[i] * N + n) * CKV; }, row, out_bf16, out_f32, lse_out, weights, partial);
}

// Dense partials: part i holds o rows at o_part + i * o_stride (floats) and lse values at lse_part + i * lse_stride. The
// merge a caller runs on (o, lse) pairs gathered from several GPUs (one packed [o | lse] record per GPU) or produced by
// its own splits ([parts, rows, 512] / [parts, rows]).
template <int GROUPS>
__global__ void __launch_bounds__(128 * GROUPS)
mla_combine_dense_kernel(const float* __restrict__ o_part, const float* __restrict__ lse_part, int parts, long long rows,
                         long long o_stride, long long lse_stride, void* out_bf16, float* out_f32, float* lse_out) {
  __shared__ float weights[kCombineMaxParts];
  __shared__ float4 partial[GROUPS > 1 ? (GROUPS - 1) * 128 : 1];
  const long long row = blockIdx.x;
  merge_row<GROUPS>(
      parts, [&](int i) { return lse_part[(long long)i * lse_stride + row]; },
      [&](int i) { return o_part + (long long)i * o_stride + row * CKV; }, row, out_bf16, out_f32, lse_out, weights, partial);
}

// The same merge over packed records [o (rows x 512) | lse (rows)] that live at unrelated addresses, one per part: the
// partial results of the GPUs of a sequence-sharded decode, read where their owners wrote them (a peer's record is read
// over NVLink with ordinary loads; the caller orders the reads after the writes, e.g. with a barrier between the GPUs).
constexpr int kCombineMaxRecords = 16;
struct RecordPtrs {
  const float* p[kCombineMaxRecords];
};
template <int GROUPS>
__global__ void __launch_bounds__(128 * GROUPS)
mla_combine_records_kernel(RecordPtrs recs, int parts, long long rows, void* out_bf16, float* out_f32, float* lse_out) {
  __shared__ float weights[kCombineMaxParts];
  __shared__ float4 partial[GROUPS > 1 ? (GROUPS - 1) * 128 : 1];
  const long long row = blockIdx.x;
  merge_row<GROUPS>(
      parts, [&](int i) { return recs.p[i][rows * CKV + row]; }, [&](int i) { return recs.p[i] + row * CKV; }, row, out_bf16,
      out_f32, lse_out, weights, partial);
}

// The same merge with the hand-shake between the GPUs inside the kernel: no barrier launch in front of it. GPU `rank`
// owns a word per GPU (`flags.p[rank][r]` is written by GPU r alone); the first CTA of each GPU's merge stores the
// step's epoch into its word on every GPU (release at system scope: the record this GPU's earlier kernels wrote is
// visible to whoever then reads the word), every CTA polls this GPU's own words until all of them carry the epoch,
// and then reads the records. Epochs only grow, so a GPU that is one step ahead passes the test as well; it cannot be
// two ahead, because its next merge waits for this GPU's next epoch. The wait is bounded by `wait_ns` of the global
// timer: when it runs out the CTA raises kPeerTimeout in *status and merges what is there, so that the context stays
// usable and the host learns of the missing GPU from the status word.
struct FlagPtrs {
  uint32_t* p[kCombineMaxRecords];
};
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
template <int GROUPS>
__global__ void __launch_bounds__(128 * GROUPS)
mla_combine_records_signalled_kernel(RecordPtrs recs, FlagPtrs flags, int rank, uint32_t epoch, unsigned long long wait_ns,
                                     int parts, long long rows, void* out_bf16, float* out_f32, float* lse_out, int* status) {
  __shared__ float weights[kCombineMaxParts];
  __shared__ float4 partial[GROUPS > 1 ? (GROUPS - 1) * 128 : 1];
  if (int(threadIdx.x) < parts) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.p[threadIdx.x] + rank), "r"(epoch) : "memory");
    }
    const uint32_t* mine = flags.p[rank] + threadIdx.x;
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (int(v - epoch) >= 0) break;
      if (global_timer_ns() - t0 > wait_ns) {
        if (status) atomicMax(status, int(kPeerTimeout));
        break;
      }
    }
  }
  __syncthreads();
  const long long row = blockIdx.x;
  merge_row<GROUPS>(
      parts, [&](int i) { return recs.p[i][rows * CKV + row]; }, [&](int i) { return recs.p[i] + row * CKV; }, row, out_bf16,
      out_f32, lse_out, weights, partial);
}

}  // namespace mla
