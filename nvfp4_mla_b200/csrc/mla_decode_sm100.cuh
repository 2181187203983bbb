// Weight-absorbed MLA decode over the NVFP4 paged latent-KV cache for sm_100a: the 8-bit mode at 16 or 32 heads per
// CTA (the 16-bit mode is mla_decode_vt_sm100.cuh, 128 heads in the 8-bit mode mla_decode_hm_sm100.cuh; this header
// also holds what the three share: DecodeParams, the segment batch, the query's per-row maxima).
//
// Data path (one CTA per SM, persistent over the work the schedule kernel assigned to it):
//
//   HBM --TMA--> raw ring (smem) --convert warps--> K as E4M3 in TENSOR MEMORY (tokens = lanes)  --QK^T--> S^T (TMEM)
//                                              \--> V as E4M3 in smem, [token][channel]           --PV----> O^T (TMEM)
//
// Tokens are the M dimension of both MMAs (128 per tile); the heads of the CTA are N (16 or 32), so 16 heads are
// never padded to the MMA's minimum M.
//   QK^T : S^T[token, head] = K[token, 576] . Q^T          A = K from tensor memory, B = Q^T from smem (K-major)
//   PV   : O^T[chan, head] += V^T[chan, token] . P^T       A = V from smem read MN-major (the [token][channel] tile
//          IS V^T with M contiguous), B = P^T from smem (K-major), 4 blocks of 128 channels
// One dequantisation (thread = token, registers = channels) feeds both: K, V = E4M3((e2m1 x scale) / 8), the reference's
// 8-bit rounding. Phase A of a tile converts the token row and writes it to tensor memory with tcgen05.st, chunk by
// chunk, so QK^T chases the conversion. Phase B copies the same values from tensor memory to one of two swizzled V
// tiles (tcgen05.ld + st.shared): the arithmetic never waits for the V buffer.
// The template parameter P8 (8-bit operands) is always true in the instantiations that are built; its `false`
// branches are the layout rules of the FP16 form of this data path (K 288 columns, one 128 KB V tile), which the
// 16-bit mode used before it got a kernel of its own.
//
// Warp roles (512 threads): 0-3 softmax + epilogue (thread = token row of S^T / channel row of O^T),
// 4-11 dequantise (warp%4 = TMEM lane quadrant, two warps per quadrant split the channel panels), 12 QK^T issue,
// 13 TMA producer, 14 PV issue. QK^T and PV have their own issuing warps so that the tensor pipe interleaves
// QK^T of tile j+1 (as its chunks are converted) with PV of tile j (as softmax and the V copy finish); S^T and P^T
// are double buffered. Softmax keeps one running max per head shared by all 128 token rows and rescales O^T in
// tensor memory only when some score outgrows it by 2^8 (a CTA-wide vote per tile), so the common tile has no
// cross-thread traffic except that vote.
//
// Every wait is bounded (ptx::mbar_wait): a protocol error sets an abort flag, every role leaves its loop, the CTA
// frees its tensor memory and the kernel reports kWaitTimeout in the workspace header.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "mla_common.cuh"
#include "ptx_sm100.cuh"

namespace mla {

constexpr int kDecodeThreads = 512;
constexpr int kSegBatch = 32;
constexpr int kRawSlotBytes = HALF * TOKEN_BYTES;  // 22528: ckv lo | ckv hi | sf | kpe
constexpr int kRawCkvHi = HALF * 128, kRawSf = 2 * HALF * 128, kRawKpe = kRawSf + HALF * 32;
constexpr int kVPanelBytes = TILE * 128;  // one 64-channel panel of the FP16 V tile
constexpr int kTmemCols = 512;

struct DecodeParams {
  const __nv_bfloat16* q_nope;
  const __nv_bfloat16* q_pe;
  const uint8_t* ckv;
  const uint8_t* sf;
  const uint8_t* kpe;
  const int* page_table;
  long long pt_stride;
  int page_shift;  // log2(page_size)
  int num_pages;   // page ids outside [0, num_pages) are never dereferenced: the rows stay unloaded and kBadPage is reported
  // Pages of at least a staging slot (64 tokens) arrive through swizzled tensor maps: the 32-byte scale rows with the
  // 32-byte swizzle (16-byte chunk ^= row / 4 % 2), the 64-byte rope rows with the 64-byte swizzle (chunk ^= row / 2 % 4),
  // so that 32 threads reading the same chunk of 32 consecutive rows touch every bank once. Smaller pages arrive
  // through linear bulk copies (a box of fewer than 128 bytes cannot be a TMA tile destination): masks 0.
  uint32_t sf_swz_mask, kpe_swz_mask;
  int heads, heads_per_cta;
  float sm_scale_log2, ckv_scale, kpe_scale;
  const int2* cta_range;
  const Seg* segs;
  float* lse_part;
  float* o_part;
  int* header;
  // Schedule computed by the decode kernel itself (16-bit kernel, batch * splits up to its thread count): every CTA
  // scans the lengths and derives its own items; cta_range and segs are then unused and no schedule kernel runs.
  const int* kv_lens;
  Problem pb;
  int inline_sched;
  int2* item_range;  // written by the CTA that holds an item's first tile (read by the combine kernel)
  int2* cta_range_out;
  Seg* segs_out;
};

// ---------------------------------------------------------------------------------------------------------------
// The schedule, derived by every decode CTA (or CTA pair: `unit`) for itself, so that no schedule kernel runs in
// front of the decode kernel. Thread bz takes the (request, split) pair bz; a block scan gives the exclusive prefix
// of their tile counts; the unit's piece [unit q, (unit + 1) q) of the flattened (pair, head group) tile range gives
// its items. The unit's part of the schedule goes to the workspace in the form mla_schedule_kernel writes (its
// cta_range entry, one Seg per item of its range in slot unit + w, and the CTA range of every item whose first tile it
// holds, for the combine kernel), and the roles read it from there as they do after a schedule kernel: writes and
// reads of one CTA, ordered by the CTA-wide barrier (the two CTAs of a pair write the same values). 32-bit arithmetic:
// the host takes this path only when batch * splits <= THREADS and the flattened tile count is below 2^31.
// `scratch`: THREADS + THREADS / 32 + 4 ints of shared memory that nothing else uses yet (a staging buffer).
// ---------------------------------------------------------------------------------------------------------------
template <int THREADS>
__device__ __forceinline__ void publish_own_schedule(int* scratch, const DecodeParams& P, int unit) {
  int* pre = scratch;                     // [BZ + 1] exclusive prefix of the tiles of the (request, split) pairs
  int* warp_tot = scratch + THREADS + 1;  // [THREADS / 32]
  int* misc = warp_tot + THREADS / 32;    // first item, last item + 1, tiles per unit
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int BZ = P.pb.batch * P.pb.splits, HG = P.pb.head_groups;
  const int t = tid < BZ ? sched_tiles(P.kv_lens, P.pb, tid) : 0;
  int incl = t;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(~0u, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  int base = 0, total = 0;
  for (int i = 0; i < THREADS / 32; ++i) {
    const int v = warp_tot[i];
    base += i < warp ? v : 0, total += v;
  }
  const int mine = base + incl - t;
  if (tid < BZ) pre[tid] = mine;
  const uint32_t T = uint32_t(total) * uint32_t(HG);
  const uint32_t q = T > 0 ? (T + P.pb.n_cta - 1) / P.pb.n_cta : 1u;
  const uint32_t g0 = uint32_t(unit) * q, g1 = g0 + q < T ? g0 + q : T;
  if (tid == 0) {
    pre[BZ] = total, misc[2] = int(q);
    if (g0 >= g1) misc[0] = 0, misc[1] = 0;
  }
  if (g0 < g1 && t > 0) {
    const uint32_t lo = uint32_t(HG) * uint32_t(mine), hi = lo + uint32_t(HG) * uint32_t(t);
    if (g0 >= lo && g0 < hi) misc[0] = tid * HG + int((g0 - lo) / uint32_t(t));
    if (g1 - 1 >= lo && g1 - 1 < hi) misc[1] = tid * HG + int((g1 - 1 - lo) / uint32_t(t)) + 1;
  }
  __syncthreads();
  const int2 range = make_int2(misc[0], misc[1]);
  for (int w = range.x + tid; w < range.y; w += THREADS) {
    const int bz = w / HG, hg = w % HG, tw = pre[bz + 1] - pre[bz];
    const int b = bz / P.pb.splits, z = bz % P.pb.splits;
    Seg g;
    g.b = b, g.hg = hg, g.tok0 = 0, g.ntiles = 0, g.tok_end = 0, g.w = w, g.cta = unit, g.pad = 0;
    if (tw > 0) {
      const uint32_t Pw = uint32_t(HG) * uint32_t(pre[bz]) + uint32_t(hg) * uint32_t(tw);
      const uint32_t lo = (g0 > Pw ? g0 : Pw) - Pw, hi = (g0 + q < Pw + tw ? g0 + q : Pw + tw) - Pw;
      if (hi > lo) {
        if (lo == 0) P.item_range[w] = make_int2(unit, int((Pw + tw - 1) / q));
        const int len = P.kv_lens[b];
        const long long end = (long long)(z + 1) * P.pb.chunk;
        g.tok0 = z * P.pb.chunk + int(lo) * TILE, g.ntiles = int(hi - lo), g.tok_end = int(end < len ? end : len);
      }
    }
    P.segs_out[(long long)unit + w] = g;
  }
  if (tid == 0) P.cta_range_out[unit] = range;
  __syncthreads();
}

template <int N, int RAW_SLOTS, bool P8>
struct DecodeSmem {
  // Operand tiles, all with the 128-byte swizzle, one 128-byte row per token (V) or head (Q^T, P^T).
  //   16-bit mode: a row holds 64 elements. V: 8 panels of 64 channels; Q^T: 8 latent panels + rope; P^T: 2 panels of 64 tokens
  //   8-bit mode : a row holds 128 elements. V: 4 panels of 128 channels; Q^T: 4 latent panels + rope (half a row); P^T: 1 panel
  static constexpr int VBUFS = P8 ? 2 : 1;          // the 8-bit V tile is small enough to double buffer
  alignas(1024) uint8_t v16[VBUFS][P8 ? 4 : 8][kVPanelBytes];
  alignas(1024) uint8_t q[P8 ? 5 : 9][N * 128];
  alignas(1024) uint8_t p[2][P8 ? 1 : 2][N * 128];  // double buffered
  alignas(1024) uint8_t raw[RAW_SLOTS][kRawSlotBytes];
  Seg segs[kSegBatch];
  float qa[4][N], qb[4][N];                         // per-head score scales (latent, rope), ring indexed by segment count
  float red[4][N];                                  // softmax group: per-warp partial reductions
  float corr[N];                                    // softmax group: per-head rescale factors of the current tile
  unsigned int qamax[N], qamax_pe[N];
  alignas(8) uint64_t raw_full[RAW_SLOTS];
  uint64_t raw_empty[RAW_SLOTS];
  // K chunk in tensor memory: [tile parity][0..3 = latent panels {g, g+4}, 4 = rope], one phase per two tiles. Two sets,
  // because in the 16-bit mode the convert warps publish the rope chunk and chunk 0 of tile it + 1 (which have their
  // own columns) while QK^T may not yet have looked at tile it's barriers.
  uint64_t k_full[2][5];
  // QK^T of the tile has finished reading K and Q^T. 16-bit mode: one barrier per tile parity, one phase per two
  // tiles; 8-bit mode: one barrier, one phase per tile (each measured faster in its mode by 1-2 %).
  uint64_t k_done[2];
  static constexpr bool kDoneTwo = !P8;
  __device__ __forceinline__ uint64_t* kdone_bar(uint32_t tile) { return &k_done[kDoneTwo ? tile & 1 : 0]; }
  __device__ static __forceinline__ uint32_t kdone_phase(uint32_t tile) { return kDoneTwo ? (tile >> 1) & 1 : tile & 1; }
  uint64_t v_full[2];                               // V buffer b is written (one phase per tile that uses the buffer)
  // 16-bit mode (single V tile): per 128-channel block mb = panels {mb, mb + 4}, one phase per tile. PV of a tile chases
  // the copy block by block, and the copy of the next tile chases PV.
  uint64_t vb_full[4], vb_free[4];
  // S^T and P^T are double buffered; each of these barriers belongs to one buffer and completes once per two tiles, so
  // a waiter that runs up to two tiles ahead or behind can never mistake one phase for another of the same parity.
  uint64_t s_full[2], s_free[2];                    // S^T written by QK^T / read by softmax
  uint64_t p_full[2], p_free[2];                    // P^T written by softmax / read by PV (= PV of that tile complete)
  uint32_t tmem_base;
  int abort_flag;
};

template <int N, int RAW_SLOTS, bool P8>
constexpr size_t decode_smem_bytes() { return sizeof(DecodeSmem<N, RAW_SLOTS, P8>) + 1024; }

// tensor-memory columns. K: one token row per lane, PANEL columns per 64-channel panel (2 FP16 or 4 E4M3 per column).
template <int N, bool P8> struct Cols {
  static constexpr uint32_t PANEL = P8 ? 16 : 32, K = 0, KROPE = 8 * PANEL, S = 9 * PANEL, O = S + 4 * N;
  __host__ __device__ static constexpr uint32_t sn(uint32_t buf) { return S + buf * 2 * N; }      // latent part of the scores
  __host__ __device__ static constexpr uint32_t sp(uint32_t buf) { return S + buf * 2 * N + N; }  // rope part
  static_assert(O + 4 * N <= kTmemCols, "tensor memory overflow");
  // 16-bit mode with 16 heads: 96 columns are left over. They give the rope chunk and the first latent chunk (panels
  // 0 and 4) of ODD tiles a home of their own, so that the conversion of a tile can start before QK^T of the tile
  // before it has finished with K (the wait moves from the first chunk to the second).
  static constexpr bool kTwoHomes = !P8 && O + 4 * N + 3 * PANEL <= kTmemCols;
  static constexpr uint32_t SPARE = O + 4 * N;
  // (In the 8-bit mode with 16 heads the whole of K would fit a second time; measured, it gains nothing: that kernel is
  // paced by the conversion arithmetic, not by this wait.)
  __host__ __device__ static constexpr uint32_t krope(uint32_t parity) { return kTwoHomes && parity ? SPARE : KROPE; }
  __host__ __device__ static constexpr uint32_t kpanel(uint32_t p, uint32_t parity) {
    return kTwoHomes && parity && (p & 3) == 0 ? SPARE + PANEL + (p >> 2) * PANEL : K + PANEL * p;
  }
};

// ---------------------------------------------------------------------------------------------------------------
// role: TMA producer (one warp; lane 0 issues, all lanes help with page ids)
// ---------------------------------------------------------------------------------------------------------------
// Smem: any struct with raw[RAW_SLOTS][kRawSlotBytes], raw_full / raw_empty[RAW_SLOTS], segs[] and abort_flag.
template <int RAW_SLOTS, class Smem>
__device__ __forceinline__ void producer_role(Smem& s, const DecodeParams& P, const CUtensorMap* ckv_map,
                                              const CUtensorMap* sf_map, const CUtensorMap* kpe_map, int n_segs, uint32_t& hcount) {
  const int lane = ptx::lane_id();
  const int ps = 1 << P.page_shift;
  for (int si = 0; si < n_segs; ++si) {
    const Seg seg = s.segs[si];
    if (seg.ntiles <= 0) continue;
    const int* pt = P.page_table + (long long)seg.b * P.pt_stride;
    for (int hk = 0; hk < 2 * seg.ntiles; ++hk, ++hcount) {
      const int slot = hcount % RAW_SLOTS;
      const uint32_t use = hcount / RAW_SLOTS;
      bool ok = ptx::mbar_wait(&s.raw_empty[slot], (use & 1) ^ 1, &s.abort_flag);
      if (!__all_sync(~0u, ok)) return;
      const int tok = seg.tok0 + hk * HALF;
      int nvalid = seg.tok_end - tok;
      nvalid = nvalid < 0 ? 0 : (nvalid > HALF ? HALF : nvalid);
      uint8_t* dst = s.raw[slot];
      uint64_t* bar = &s.raw_full[slot];
      if (nvalid == 0) {
        if (lane == 0) ptx::mbar_arrive(bar);
      } else if (ps >= HALF) {
        if (lane == 0) {
          const int page = pt[tok >> P.page_shift];
          // A stale or corrupt id is never dereferenced: the boxes are taken beyond the last row of the cache instead,
          // where TMA fills zeros (scale 0: the rows contribute score 0 and value 0), and the call is flagged.
          const bool bad = uint32_t(page) >= uint32_t(P.num_pages);
          if (bad) atomicExch(P.header, int(kBadPage));
          const int row = bad ? (P.num_pages << P.page_shift) : (page << P.page_shift) + (tok & (ps - 1));
          ptx::mbar_arrive_expect_tx(bar, HALF * TOKEN_BYTES);
          ptx::tma_load_2d(dst, ckv_map, 0, row, bar);
          ptx::tma_load_2d(dst + kRawCkvHi, ckv_map, 128, row, bar);
          ptx::tma_load_2d(dst + kRawSf, sf_map, 0, row, bar);
          ptx::tma_load_2d(dst + kRawKpe, kpe_map, 0, row, bar);
          // L2 prefetch a few slots ahead (the ring itself is too shallow to cover HBM latency)
          const int tok_pf = tok + 6 * HALF;
          if (tok_pf < seg.tok_end) {
            const int page2 = pt[tok_pf >> P.page_shift];
            if (uint32_t(page2) < uint32_t(P.num_pages)) {
              const int row2 = (page2 << P.page_shift) + (tok_pf & (ps - 1));
              ptx::tma_prefetch_l2_2d(ckv_map, 0, row2);
              ptx::tma_prefetch_l2_2d(ckv_map, 128, row2);
              ptx::tma_prefetch_l2_2d(sf_map, 0, row2);
              ptx::tma_prefetch_l2_2d(kpe_map, 0, row2);
            }
          }
        }
      } else {
        // small pages: one box per page that holds a valid token, lanes share the pages (at most 64 pages per slot)
        const int npages = (nvalid + ps - 1) >> P.page_shift;
        int page[2];
        uint32_t good = 0;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int pi = lane + 32 * k;
          page[k] = pi < npages ? pt[(tok >> P.page_shift) + pi] : -1;
          const bool ok_page = pi < npages && uint32_t(page[k]) < uint32_t(P.num_pages);
          if (pi < npages && !ok_page) atomicExch(P.header, int(kBadPage));
          if (!ok_page) page[k] = -1;
          good += __popc(__ballot_sync(~0u, ok_page));
        }
        if (lane == 0) {
          if (good) ptx::mbar_arrive_expect_tx(bar, good * ps * TOKEN_BYTES);
          else ptx::mbar_arrive(bar);
        }
        __syncwarp();
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          if (page[k] < 0) continue;
          const int row = page[k] << P.page_shift, r0 = (lane + 32 * k) << P.page_shift;
          ptx::tma_load_2d(dst + r0 * 128, ckv_map, 0, row, bar);
          ptx::tma_load_2d(dst + kRawCkvHi + r0 * 128, ckv_map, 128, row, bar);
          ptx::bulk_load(dst + kRawSf + r0 * 32, P.sf + (long long)row * 32, ps * 32, bar);
          ptx::bulk_load(dst + kRawKpe + r0 * 64, P.kpe + (long long)row * 64, ps * 64, bar);
        }
      }
      __syncwarp();
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// role: dequantise (8 warps). cw = warp - 4: quadrant = cw % 4 (tensor-memory lanes), hf = cw / 4 (panel parity).
// ---------------------------------------------------------------------------------------------------------------
template <int N, int RAW_SLOTS, bool P8>
__device__ __forceinline__ void load_query(DecodeSmem<N, RAW_SLOTS, P8>& s, const DecodeParams& P, const Seg& seg, int ct, int par) {
  // ct = 0..255. Pass 1: per-row amax (positive floats compare as unsigned ints), latent and rope parts separately.
  // Pass 2, 16-bit mode: scale the row by 2^(14 - e) so its largest magnitude lies in [2^14, 2^15), convert to FP16
  // (exact), store swizzled; the score scale undoes it. 8-bit mode: E4M3 of q * 448 / amax, each part with its own amax
  // (the reference's fp8 query, nvfp4_mla/csrc/mla_decode.cu:425-457); K is stored as value / 8, hence the 8.
  if (ct < N) s.qamax[ct] = 0, s.qamax_pe[ct] = 0;
  ptx::bar_sync(2, 256);
  const long long row0 = (long long)seg.b * P.heads + (long long)seg.hg * N;
  constexpr int CH = (CKV + KPE) / 8;              // 72 chunks of 8 channels per row
  constexpr int PER = (N * CH + 255) / 256;        // chunks per thread: all loaded up front (one memory latency), kept for pass 2
  const int lane_of_warp = ptx::lane_id();
  uint4 q8[PER];
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int i = ct + 256 * k, n = i / CH, c = i % CH;
    q8[k] = make_uint4(0, 0, 0, 0);
    if (i < N * CH)
      q8[k] = c < 64 ? reinterpret_cast<const uint4*>(P.q_nope + (row0 + n) * CKV)[c]
                     : reinterpret_cast<const uint4*>(P.q_pe + (row0 + n) * KPE)[c - 64];
  }
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int i = ct + 256 * k, n = i / CH, c = i % CH;
    if (i >= N * CH) continue;
    const uint32_t w[4] = {q8[k].x, q8[k].y, q8[k].z, q8[k].w};
    unsigned int m = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const unsigned int lo = (w[j] << 16) & 0x7FFFFFFFu, hi = w[j] & 0x7FFF0000u;
      m = max(m, max(lo, hi));
    }
    // One shared-memory atomic per (row, part) and warp instead of one per thread: the lanes that hold chunks of the
    // same row part (a warp's 32 consecutive chunks belong to at most three) reduce among themselves first.
    if (m >= 0x7F800000u) m = 0;  // ignore inf / nan for the scale
    const bool pe = P8 && c >= 64;
    const unsigned peers = __match_any_sync(__activemask(), 2 * n + int(pe));
    m = __reduce_max_sync(peers, m);
    if (lane_of_warp == __ffs(peers) - 1) atomicMax(pe ? &s.qamax_pe[n] : &s.qamax[n], m);
  }
  ptx::bar_sync(2, 256);
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int i = ct + 256 * k, n = i / CH, c = i % CH;
    if (i >= N * CH) continue;
    const uint32_t w[4] = {q8[k].x, q8[k].y, q8[k].z, q8[k].w};
    if constexpr (!P8) {
      int e = int(s.qamax[n] >> 23) - 127;       // floor(log2(amax)); -127 for 0 / subnormal rows
      e = e < -100 ? -100 : e;
      const float up = __uint_as_float(uint32_t(14 - e + 127) << 23);  // 2^(14 - e), exact
      uint32_t h[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        h[j] = ptx::f32x2_to_f16x2(__uint_as_float(w[j] << 16) * up, __uint_as_float(w[j] & 0xFFFF0000u) * up);
      const int panel = c >> 3, cc = c & 7;
      *reinterpret_cast<uint4*>(s.q[panel] + n * 128 + ((cc ^ (n & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
      if (c == 0) {
        const float down = __uint_as_float(uint32_t(e - 14 + 127) << 23);  // 2^(e - 14)
        s.qa[par][n] = P.sm_scale_log2 * P.ckv_scale * down;
        s.qb[par][n] = P.sm_scale_log2 * P.kpe_scale * down;
      }
    } else {
      const float an = fmaxf(__uint_as_float(s.qamax[n]), 1e-30f), ap = fmaxf(__uint_as_float(s.qamax_pe[n]), 1e-30f);
      const float inv = __fdividef(448.f, c < 64 ? an : ap);  // (2 ulp: it only steers the rounding of the codes; the score scale below is exact)
      uint32_t b[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint32_t lo = ptx::f32x2_to_e4m3x2(__uint_as_float(w[2 * j] << 16) * inv, __uint_as_float(w[2 * j] & 0xFFFF0000u) * inv);
        const uint32_t hi = ptx::f32x2_to_e4m3x2(__uint_as_float(w[2 * j + 1] << 16) * inv, __uint_as_float(w[2 * j + 1] & 0xFFFF0000u) * inv);
        b[j] = lo | (hi << 16);
      }
      // 8 channels = 8 bytes: panel = 128 channels (rope: panel 4), 16-byte chunk (c % 16) / 2, half c % 2
      const int panel = c >> 4, cc = (c & 15) >> 1;
      *reinterpret_cast<uint2*>(s.q[panel] + n * 128 + ((cc ^ (n & 7)) << 4) + (c & 1) * 8) = make_uint2(b[0], b[1]);
      if (c == 0) {
        s.qa[par][n] = P.sm_scale_log2 * P.ckv_scale * 8.f * (an / 448.f);
        s.qb[par][n] = P.sm_scale_log2 * P.kpe_scale * (ap / 448.f);
      }
    }
  }
  ptx::fence_proxy_async_smem();
}

// One pipeline step of a convert thread, in two parts.
//   Part B (tile it - 1): copy the thread's FP16 / E4M3 row from tensor memory into the V tile and publish it. It
//   comes first: it needs nothing from QK^T of tile it - 1, whose last MMAs are still in flight when the step starts,
//   and it lets PV of tile it - 1 start (and finish) early in the step instead of colliding with the next QK^T tail.
//   Part A (tile it): dequantise the thread's share of the token row into tensor memory, chunk by chunk, so that QK^T
//   chases the conversion; the publish of a chunk is deferred until the next chunk's values have been computed, so the
//   latency of the tensor-memory store hides behind arithmetic.
// FULL = every row of tile `it` is a live token (no masking). Returns false if a wait gave up.
template <int N, int RAW_SLOTS, bool P8, bool FULL, bool has_a, bool has_b>
__device__ __forceinline__ bool convert_step(DecodeSmem<N, RAW_SLOTS, P8>& s, const DecodeParams& P, const Seg& seg, int t, uint32_t it,
                                             int lane, int quad, int hf) {
  const int r = quad * 32 + lane;        // token row of the tile = tensor-memory lane
  const int half = r >> 6, rr = r & 63;
  const uint32_t tm_lane = s.tmem_base + (uint32_t(quad * 32) << 16);
  constexpr int W = Cols<N, P8>::PANEL;  // 32-bit words of one converted panel row: 32 (FP16) or 16 (E4M3)
  bool ok;

  // ------------------------------------------------------------------------------------------------ part B
  if (has_b) {
    constexpr uint32_t VB = DecodeSmem<N, RAW_SLOTS, P8>::VBUFS;
    const uint32_t tb = it - 1, vbuf = tb % VB;  // the tile being copied and its V buffer
    const uint32_t swz_v = uint32_t(r & 7) << 4;
    uint32_t hb[2][W];
    ptx::tmem_ldn(tm_lane + Cols<N, P8>::kpanel(4 * hf, tb & 1), hb[0]);
    // the PV that last read this V buffer (tile tb - VB) must have finished
    ok = tb < VB || ptx::mbar_wait(&s.p_free[(tb - VB) & 1], ((tb - VB) >> 1) & 1, &s.abort_flag);
    if (!__all_sync(~0u, ok)) return false;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int p = g + 4 * hf;  // 64-channel panel; 16-bit mode: V panel p, 8-bit mode: half p % 2 of V panel p / 2
      ptx::tmem_wait_ld();
      if (g < 3) ptx::tmem_ldn(tm_lane + Cols<N, P8>::kpanel(p + 1, tb & 1), hb[(g + 1) & 1]);
      const uint32_t* v = hb[g & 1];
      uint8_t* vrow = (P8 ? s.v16[vbuf][p >> 1] : s.v16[vbuf][p]) + r * 128;
#pragma unroll
      for (int c = 0; c < W / 4; ++c) {
        const uint32_t chunk = P8 ? uint32_t(4 * (p & 1) + c) : uint32_t(c);
        *reinterpret_cast<uint4*>(vrow + ((chunk << 4) ^ swz_v)) = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
      }
    }
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(&s.v_full[vbuf]);  // for tile it - 1
  }
  if (!has_a) return true;

  // ------------------------------------------------------------------------------------------------ part A
  const uint32_t hidx = 2 * it + half;
  const int slot = hidx % RAW_SLOTS;
  const uint8_t* raw = s.raw[slot];
  const uint32_t swz = uint32_t(rr & 7) << 4;
  ok = ptx::mbar_wait(&s.raw_full[slot], (hidx / RAW_SLOTS) & 1, &s.abort_flag);
  if (!__all_sync(~0u, ok)) return false;
  const bool valid = FULL || (seg.tok0 + t * TILE + r < seg.tok_end);
  const uint4 sf16 = *reinterpret_cast<const uint4*>(raw + kRawSf + rr * 32 + ((uint32_t(hf) ^ ((rr >> 2) & P.sf_swz_mask)) << 4));  // the 16 block scales of this half row
  {  // ---- rope chunk: 32 channels of this thread's half
    const uint32_t kswz = (rr >> 1) & P.kpe_swz_mask;
    const uint4 rope0 = *reinterpret_cast<const uint4*>(raw + kRawKpe + rr * 64 + ((uint32_t(2 * hf) ^ kswz) << 4));
    const uint4 rope1 = *reinterpret_cast<const uint4*>(raw + kRawKpe + rr * 64 + ((uint32_t(2 * hf + 1) ^ kswz) << 4));
    // K of the previous tile may be overwritten once its QK^T has finished (the copy above has already read it)
    ok = it == 0 || ptx::mbar_wait(s.kdone_bar(it - 1), s.kdone_phase(it - 1), &s.abort_flag);
    if (!__all_sync(~0u, ok)) return false;
    ptx::tc_fence_after_sync();
    const uint32_t rw[8] = {rope0.x, rope0.y, rope0.z, rope0.w, rope1.x, rope1.y, rope1.z, rope1.w};
    if constexpr (!P8) {
      uint32_t h[16];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        h[2 * j] = valid ? ptx::e4m3x2_to_f16x2(uint16_t(rw[j] & 0xFFFF)) : 0u;
        h[2 * j + 1] = valid ? ptx::e4m3x2_to_f16x2(uint16_t(rw[j] >> 16)) : 0u;
      }
      ptx::tmem_st16(tm_lane + Cols<N, P8>::krope(it & 1) + 16 * hf, h);
    } else {  // the rope bytes are E4M3 already
      uint32_t h[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) h[j] = valid ? rw[j] : 0u;
      ptx::tmem_st8(tm_lane + Cols<N, P8>::krope(it & 1) + 8 * hf, h);
    }
  }
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int p = g + 4 * hf;  // 64-channel panel = bytes [32p, 32p + 32) of the 256-byte row; hf = its 128-byte half
    uint32_t h[W];
    const uint8_t* base = raw + hf * kRawCkvHi + rr * 128;
    const uint32_t c0 = uint32_t(2 * g) << 4;
    const uint4 n0 = *reinterpret_cast<const uint4*>(base + (c0 ^ swz));
    const uint4 n1 = *reinterpret_cast<const uint4*>(base + ((c0 + 16) ^ swz));
    const uint32_t sfw = g == 0 ? sf16.x : g == 1 ? sf16.y : g == 2 ? sf16.z : sf16.w;
    if (g == 3) {  // last read of the raw slot by this thread
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&s.raw_empty[slot]);
    }
    // block scales: 4 E4M3 bytes -> four FP16 pairs (s, s); the 8-bit mode stores (e2m1 x s) / 8 so that the product
    // (up to 2688) stays inside E4M3's range, and undoes the 8 in the score scale and the output
    uint32_t s01 = ptx::e4m3x2_to_f16x2(uint16_t(sfw & 0xFFFF)), s23 = ptx::e4m3x2_to_f16x2(uint16_t(sfw >> 16));
    if constexpr (P8) s01 = ptx::hmul2(s01, 0x30003000u), s23 = ptx::hmul2(s23, 0x30003000u);  // x 1/8, exact
    const uint32_t sc[4] = {__byte_perm(s01, s01, 0x1010), __byte_perm(s01, s01, 0x3232), __byte_perm(s23, s23, 0x1010),
                            __byte_perm(s23, s23, 0x3232)};
    const uint32_t wds[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {  // word j = channels [8j, 8j + 8) of the panel, scale block j / 2
      uint32_t e[4];
      ptx::e2m1x8_to_f16x8(wds[j], e);
      if constexpr (!P8) {
#pragma unroll
        for (int i = 0; i < 4; ++i) h[4 * j + i] = valid ? ptx::hmul2(e[i], sc[j >> 1]) : 0u;
      } else {  // the FP16 product is exact; the only rounding is the conversion to E4M3
        const uint32_t b01 = ptx::f16x4_to_e4m3x4(ptx::hmul2(e[0], sc[j >> 1]), ptx::hmul2(e[1], sc[j >> 1]));
        const uint32_t b23 = ptx::f16x4_to_e4m3x4(ptx::hmul2(e[2], sc[j >> 1]), ptx::hmul2(e[3], sc[j >> 1]));
        h[2 * j] = valid ? b01 : 0u;
        h[2 * j + 1] = valid ? b23 : 0u;
      }
    }
    // publish the previous chunk (rope for g = 0): its store has been in flight during the arithmetic above
    ptx::tmem_wait_st();
    ptx::tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(&s.k_full[it & 1][g == 0 ? 4 : g - 1]);
    ptx::tmem_stn(tm_lane + Cols<N, P8>::kpanel(p, it & 1), h);
  }
  ptx::tmem_wait_st();
  ptx::tc_fence_before_sync();
  __syncwarp();
  if (lane == 0) ptx::mbar_arrive(&s.k_full[it & 1][3]);
  return true;
}

// A warp whose wait gave up does not leave at once: the 256 convert threads meet at a named barrier at the start of
// every segment, so it carries on (skipping the work) to the next such barrier, where the failure is OR-reduced and
// all eight warps leave together.
template <int N, int RAW_SLOTS, bool P8>
__device__ __forceinline__ void convert_role(DecodeSmem<N, RAW_SLOTS, P8>& s, const DecodeParams& P, int n_segs, uint32_t& it,
                                             uint32_t& seg_count) {
  const int lane = ptx::lane_id();
  const int cw = (threadIdx.x >> 5) - 4, quad = cw & 3, hf = cw >> 2;
  bool dead = false, pending = false;  // pending: tile it - 1 still has to be copied into the V tile
  Seg seg = s.segs[0];
  for (int si = 0; si < n_segs; ++si) {
    seg = s.segs[si];
    if (seg.ntiles <= 0) continue;
    // the previous tile's QK^T must be done reading Q^T before the new query overwrites it
    const bool ok = !dead && (it == 0 || ptx::mbar_wait(s.kdone_bar(it - 1), s.kdone_phase(it - 1), &s.abort_flag));
    if (ptx::bar_red_or(2, 256, !ok)) return;
    load_query<N, RAW_SLOTS, P8>(s, P, seg, cw * 32 + lane, seg_count & 3);
    ++seg_count;
    for (int t = 0; t < seg.ntiles; ++t, ++it) {
      const bool full = seg.tok0 + (t + 1) * TILE <= seg.tok_end;
      bool ok_s;
      // double-buffered V tile: copy first, then convert
      ok_s = !pending ? convert_step<N, RAW_SLOTS, P8, false, true, false>(s, P, seg, t, it, lane, quad, hf)
             : full   ? convert_step<N, RAW_SLOTS, P8, true, true, true>(s, P, seg, t, it, lane, quad, hf)
                      : convert_step<N, RAW_SLOTS, P8, false, true, true>(s, P, seg, t, it, lane, quad, hf);
      pending = true;
      if (!ok_s) {
        dead = true;
        break;
      }
    }
  }
  // drain: the batch's last tile still has to reach the V tile
  if (pending && !dead) {
    convert_step<N, RAW_SLOTS, P8, true, false, true>(s, P, seg, 0, it, lane, quad, hf);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// roles: MMA issue (one warp for QK^T, one for PV). The whole warp runs the loop so that every operand is
// warp-uniform (descriptors then live in uniform registers and an MMA costs a couple of instructions); one elected
// lane issues. A tcgen05.commit tracks only the MMAs of the thread that executes it, so each role's barriers speak
// for its own MMAs.
// ---------------------------------------------------------------------------------------------------------------
template <int N, int RAW_SLOTS, bool P8>
__device__ __forceinline__ void qk_role(DecodeSmem<N, RAW_SLOTS, P8>& s, const DecodeParams& P, int n_segs, uint32_t& it) {
  const bool leader = ptx::elect_one();
  const uint32_t tm = s.tmem_base;
  constexpr uint32_t FMT = P8 ? ptx::FMT_E4M3 : ptx::FMT_F16;
  constexpr int KSTEPS = P8 ? 2 : 4;            // MMAs per 64-channel panel (K = 32 E4M3 or 16 FP16 per MMA, 8 columns)
  const uint32_t idesc = ptx::instr_desc(128, N, FMT, FMT, false, false);
  const uint64_t q_desc = ptx::smem_desc_sw128(ptx::smem_u32(s.q[0]), 16, 1024);
  // byte offset of (64-channel panel p, K step ks) inside Q^T: 16-bit: panel p, 32 bytes per step;
  // 8-bit: 128-channel panel p / 2, half p % 2 (64 bytes), 32 bytes per step. Rope = panel 8.
  auto q_off = [](int p, int ks) { return P8 ? ((p >> 1) * N * 128 + (p & 1) * 64 + ks * 32) : (p * N * 128 + ks * 32); };
  auto mma = [&](uint32_t d, uint32_t a, uint64_t b, uint32_t accum) {
    if constexpr (P8) ptx::mma_f8_ts(d, a, b, idesc, accum); else ptx::mma_f16_ts(d, a, b, idesc, accum);
  };
  for (int si = 0; si < n_segs; ++si) {
    const int ntiles = s.segs[si].ntiles;
    for (int t = 0; t < ntiles; ++t, ++it) {
      const uint32_t par = it & 1, buf = it & 1;
      // softmax of tile it - 2 must have read this S^T buffer
      if (!__all_sync(~0u, it < 2 || ptx::mbar_wait(&s.s_free[buf], ((it >> 1) - 1) & 1, &s.abort_flag))) return;
      // ---- S^T = K . Q^T : rope chunk into SP, latent chunks into SN
      if (!__all_sync(~0u, ptx::mbar_wait(&s.k_full[par][4], (it >> 1) & 1, &s.abort_flag))) return;
      ptx::tc_fence_after_sync();
      if (leader) {
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks)
          mma(tm + Cols<N, P8>::sp(buf), tm + Cols<N, P8>::krope(par) + 8 * ks, q_desc + (q_off(8, ks) >> 4), ks > 0);
      }
      // rolled loops (one panel per trip): fully unrolled, the operand sets would occupy ~100 registers of a warp
      // group that has given most of its registers away
#pragma unroll 1
      for (int g = 0; g < 4; ++g) {
        if (!__all_sync(~0u, ptx::mbar_wait(&s.k_full[par][g], (it >> 1) & 1, &s.abort_flag))) return;
        ptx::tc_fence_after_sync();
        if (leader) {
#pragma unroll 1
          for (int half = 0; half < 2; ++half) {
            const int p = g + 4 * half;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks)
              mma(tm + Cols<N, P8>::sn(buf), tm + Cols<N, P8>::kpanel(p, par) + 8 * ks, q_desc + (q_off(p, ks) >> 4), (g | half | ks) != 0);
          }
          if (g == 3) ptx::mma_commit(s.kdone_bar(it)), ptx::mma_commit(&s.s_full[buf]);
        }
      }
    }
  }
}

template <int N, int RAW_SLOTS, bool P8>
__device__ __forceinline__ void pv_role(DecodeSmem<N, RAW_SLOTS, P8>& s, const DecodeParams& P, int n_segs, uint32_t& it) {
  const bool leader = ptx::elect_one();
  const uint32_t tm = s.tmem_base;
  constexpr uint32_t FMT = P8 ? ptx::FMT_E4M3 : ptx::FMT_F16;
  const uint32_t idesc = ptx::instr_desc(128, N, FMT, FMT, true, false);
  // MN-major A, block mb of 128 channels. 16-bit: panels {mb, mb + 4} (channels [64mb, +64) and [256 + 64mb, +64)), so the
  // second 128-byte run along M is 4 panels away (LBO); 8-bit: panel mb alone (one 128-byte run, LBO unused).
  const uint64_t v_desc0 = ptx::smem_desc_sw128(ptx::smem_u32(s.v16[0][0]), P8 ? 16 : 4 * kVPanelBytes, 1024);
  constexpr uint32_t VB = DecodeSmem<N, RAW_SLOTS, P8>::VBUFS;
  constexpr int KROWS = P8 ? 32 : 16;  // tokens per MMA
  for (int si = 0; si < n_segs; ++si) {
    const int ntiles = s.segs[si].ntiles;
    for (int t = 0; t < ntiles; ++t, ++it) {
      const uint32_t par = it & 1, buf = it & 1;
      const uint64_t p_desc = ptx::smem_desc_sw128(ptx::smem_u32(s.p[buf][0]), 16, 1024);
      const uint64_t v_desc = v_desc0 + (((it % VB) * sizeof(s.v16[0])) >> 4);
      // ---- O^T += V^T . P^T
      if (!__all_sync(~0u, ptx::mbar_wait(&s.p_full[buf], (it >> 1) & 1, &s.abort_flag))) return;
      constexpr bool kVBlock = !P8;  // 16-bit mode: the single V tile is handed over per 128-channel block
      if (!kVBlock && !__all_sync(~0u, ptx::mbar_wait(&s.v_full[it % VB], (it / VB) & 1, &s.abort_flag))) return;
      ptx::tc_fence_after_sync();
#pragma unroll 1
      for (int mb = 0; mb < 4; ++mb) {
        if (kVBlock) {
          if (!__all_sync(~0u, ptx::mbar_wait(&s.vb_full[mb], par, &s.abort_flag))) return;
          ptx::tc_fence_after_sync();
        }
        if (leader) {
#pragma unroll 1
          for (int kh = 0; kh < (P8 ? 1 : 2); ++kh) {  // one P^T panel (128 bytes of tokens) per trip
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              const int row = (4 * kh + ks) * KROWS;  // first token of this K step
              if constexpr (P8)
                ptx::mma_f8_ss(tm + Cols<N, P8>::O + mb * N, v_desc + ((mb * kVPanelBytes + row * 128) >> 4),
                               p_desc + ((ks * 32) >> 4), idesc, (t | ks) != 0);
              else
                ptx::mma_f16_ss(tm + Cols<N, P8>::O + mb * N, v_desc + ((mb * kVPanelBytes + row * 128) >> 4),
                                p_desc + ((kh * N * 128 + ks * 32) >> 4), idesc, (t | kh | ks) != 0);
            }
          }
          if (kVBlock) ptx::mma_commit(&s.vb_free[mb]);
          if (mb == 3) ptx::mma_commit(&s.p_free[buf]);
        }
      }
    }
  }
}

// Reduces 16 (or 32) per-lane values over the warp in 16 (31) shuffles instead of 80 (160): every step exchanges the
// half of the values that the partner lane keeps. With 16 values lane l ends with the result of value (l / 2) % 16
// (lanes l and l ^ 1 hold the same one), with 32 values with that of value l. Deterministic. A shuffle costs about eight
// instructions of code here, and the kernel's code size shows in its speed (instruction fetch).
template <class Op>
__device__ __forceinline__ float warp_reduce16(const float (&x)[16], int lane, Op op) {
  float a[8], b[4], c[2];
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4, b1 = lane & 2;
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = op(b4 ? x[j + 8] : x[j], __shfl_xor_sync(~0u, b4 ? x[j] : x[j + 8], 16));
#pragma unroll
  for (int j = 0; j < 4; ++j) b[j] = op(b3 ? a[j + 4] : a[j], __shfl_xor_sync(~0u, b3 ? a[j] : a[j + 4], 8));
#pragma unroll
  for (int j = 0; j < 2; ++j) c[j] = op(b2 ? b[j + 2] : b[j], __shfl_xor_sync(~0u, b2 ? b[j] : b[j + 2], 4));
  const float d = op(b1 ? c[1] : c[0], __shfl_xor_sync(~0u, b1 ? c[0] : c[1], 2));
  return op(d, __shfl_xor_sync(~0u, d, 1));
}
template <class Op>
__device__ __forceinline__ float warp_reduce32(const float (&x)[32], int lane, Op op) {
  float a[16], b[8], c[4], d[2];
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4, b1 = lane & 2, b0 = lane & 1;
#pragma unroll
  for (int j = 0; j < 16; ++j) a[j] = op(b4 ? x[j + 16] : x[j], __shfl_xor_sync(~0u, b4 ? x[j] : x[j + 16], 16));
#pragma unroll
  for (int j = 0; j < 8; ++j) b[j] = op(b3 ? a[j + 8] : a[j], __shfl_xor_sync(~0u, b3 ? a[j] : a[j + 8], 8));
#pragma unroll
  for (int j = 0; j < 4; ++j) c[j] = op(b2 ? b[j + 4] : b[j], __shfl_xor_sync(~0u, b2 ? b[j] : b[j + 4], 4));
#pragma unroll
  for (int j = 0; j < 2; ++j) d[j] = op(b1 ? c[j + 2] : c[j], __shfl_xor_sync(~0u, b1 ? c[j] : c[j + 2], 2));
  return op(b0 ? d[1] : d[0], __shfl_xor_sync(~0u, b0 ? d[0] : d[1], 1));
}
// stores the warp's reduction of the N per-lane values x[] to dst[0 .. N)
template <int N, class Op>
__device__ __forceinline__ void warp_reduce_to(float* dst, const float (&x)[N], int lane, Op op) {
  static_assert(N == 16 || N == 32, "16 or 32 values");
  if constexpr (N == 16) {
    const float v = warp_reduce16(x, lane, op);
    if ((lane & 1) == 0) dst[(lane >> 1) & 15] = v;
  } else {
    dst[lane] = warp_reduce32(x, lane, op);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// role: softmax + epilogue (4 warps; thread r = token row of S^T and channel row of O^T)
// ---------------------------------------------------------------------------------------------------------------
template <int N, int RAW_SLOTS, bool P8>
__device__ __forceinline__ void softmax_role(DecodeSmem<N, RAW_SLOTS, P8>& s, const DecodeParams& P, int n_segs, uint32_t& it,
                                             uint32_t& seg_count) {
  const int lane = ptx::lane_id(), warp = threadIdx.x >> 5;
  const int r = threadIdx.x;  // 0..127
  const uint32_t tm_lane = s.tmem_base + (uint32_t(warp * 32) << 16);
  constexpr float kGrow = 8.f;  // rescale only when a score exceeds the running max by 2^8 (P stays <= 256)
  // P^T[head h][token r], row h = 128 bytes. 16-bit: panel r / 64, 16-byte chunk (r % 64) / 8; 8-bit: chunk r / 16.
  // The chunk index is swizzled by h % 8.
  const uint32_t p_off = P8 ? uint32_t(r & 15) : uint32_t(r >> 6) * (N * 128) + (r & 7) * 2;
  const uint32_t p_chunk = (P8 ? uint32_t(r >> 4) : uint32_t((r & 63) >> 3)) << 4;
  for (int si = 0; si < n_segs; ++si) {
    const Seg seg = s.segs[si];
    if (seg.ntiles <= 0) continue;
    const int par_q = seg_count & 3;
    ++seg_count;
    float m[N], lsum[N];
#pragma unroll
    for (int h = 0; h < N; ++h) m[h] = -INFINITY, lsum[h] = 0.f;
    // per-head score scales: kept in registers for 16 heads, read from shared memory (broadcast) for more
    constexpr bool kScalesInRegs = N <= 16;
    bool scales_loaded = false;
    float qa_r[kScalesInRegs ? N : 1], qb_r[kScalesInRegs ? N : 1];

    for (int t = 0; t < seg.ntiles; ++t, ++it) {
      const uint32_t buf = it & 1;
      bool ok = ptx::mbar_wait(&s.s_full[buf], (it >> 1) & 1, &s.abort_flag);
      ptx::tc_fence_after_sync();
      float x[N];
      if (kScalesInRegs && !scales_loaded) {  // written by the convert warps before the segment's first K chunk was published
#pragma unroll
        for (int h = 0; h < (kScalesInRegs ? N : 0); ++h) qa_r[h] = s.qa[par_q][h], qb_r[h] = s.qb[par_q][h];
        scales_loaded = true;
      }
      if (ok) {
        const bool valid = seg.tok0 + t * TILE + r < seg.tok_end;
#pragma unroll
        for (int c0 = 0; c0 < N; c0 += 16) {
          uint32_t sn[16], sp[16];
          ptx::tmem_ld16(tm_lane + Cols<N, P8>::sn(buf) + c0, sn);
          ptx::tmem_ld16(tm_lane + Cols<N, P8>::sp(buf) + c0, sp);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float qa = kScalesInRegs ? qa_r[kScalesInRegs ? c0 + j : 0] : s.qa[par_q][c0 + j];
            const float qb = kScalesInRegs ? qb_r[kScalesInRegs ? c0 + j : 0] : s.qb[par_q][c0 + j];
            const float v = fmaf(__uint_as_float(sp[j]), qb, __uint_as_float(sn[j]) * qa);
            x[c0 + j] = valid ? v : -INFINITY;
          }
        }
      } else {
#pragma unroll
        for (int h = 0; h < N; ++h) x[h] = -INFINITY;
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&s.s_free[buf]);  // QK^T of tile it + 2 may overwrite this S^T buffer
      bool need = !ok;
#pragma unroll
      for (int h = 0; h < N; ++h) need |= x[h] > m[h] + kGrow;
      if (ptx::bar_red_or(1, 128, need)) {
        if (ptx::bar_red_or(1, 128, s.abort_flag != 0)) return;  // uniform decision, whoever raised the flag
        // new running max per head over the 128 token rows
        warp_reduce_to<N>(s.red[warp], x, lane, [](float p, float q) { return fmaxf(p, q); });
        ptx::bar_sync(1, 128);
        // The correction factors are the same in every thread (the running max is shared by all rows); they are parked
        // in shared memory (every thread stores the same values and reads back its own store) to keep this rare path
        // from raising the role's register need.
        bool any_scale = false;
#pragma unroll
        for (int h = 0; h < N; ++h) {
          const float mx = fmaxf(fmaxf(s.red[0][h], s.red[1][h]), fmaxf(s.red[2][h], s.red[3][h]));
          const float mn = fmaxf(m[h], mx);
          const float c = (m[h] == -INFINITY) ? 0.f : ptx::ex2(m[h] - mn);  // mn = -inf only if m = -inf
          any_scale |= c != 1.f;
          lsum[h] *= c;
          m[h] = mn;
          s.corr[h] = c;
        }
        // O^T *= corr per head (column): after the previous tile's PV has finished; this tile's PV is not issued
        // before this thread arrives on p_full.
        if (t > 0 && any_scale) {
          const bool okv = ptx::mbar_wait(&s.p_free[buf ^ 1], ((it - 1) >> 1) & 1, &s.abort_flag);  // PV of tile it - 1
          if (ptx::bar_red_or(1, 128, !okv)) return;
          ptx::tc_fence_after_sync();
#pragma unroll 1
          for (int mb = 0; mb < 4; ++mb) {
#pragma unroll
            for (int c0 = 0; c0 < N; c0 += 16) {
              uint32_t o[16];
              ptx::tmem_ld16(tm_lane + Cols<N, P8>::O + mb * N + c0, o);
              ptx::tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * s.corr[c0 + j]);
              ptx::tmem_st16(tm_lane + Cols<N, P8>::O + mb * N + c0, o);
            }
          }
          ptx::tmem_wait_st();
        }
      }
      // PV of tile it - 2 must have read this P^T buffer
      // (if this wait gives up the abort flag is raised and the next vote or the epilogue ends the role for all)
      if (it >= 2) ptx::mbar_wait(&s.p_free[buf], ((it >> 1) - 1) & 1, &s.abort_flag);
      // P^T[head][token] = 2^(x - m) as FP16, and the row's share of the softmax denominators
      uint8_t* const p_base = s.p[buf][0] + p_off;
#pragma unroll
      for (int h = 0; h < N; ++h) {
        const float pv = ptx::ex2(x[h] - (m[h] == -INFINITY ? 0.f : m[h]));  // x = -inf gives 0
        lsum[h] += pv;
        if constexpr (P8)
          *(p_base + h * 128 + (p_chunk ^ (uint32_t(h & 7) << 4))) = uint8_t(ptx::f32x2_to_e4m3x2(pv, 0.f));
        else
          *reinterpret_cast<__half*>(p_base + h * 128 + (p_chunk ^ (uint32_t(h & 7) << 4))) = __float2half_rn(pv);
      }
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&s.p_full[buf]);
    }

    // ---- segment epilogue: wait for the last PV, reduce the denominators, write the normalised partial
    bool ok = ptx::mbar_wait(&s.p_free[(it - 1) & 1], ((it - 1) >> 1) & 1, &s.abort_flag);  // PV of the last tile
    if (ptx::bar_red_or(1, 128, !ok)) return;
    ptx::tc_fence_after_sync();
    warp_reduce_to<N>(s.red[warp], lsum, lane, [](float p, float q) { return p + q; });
    ptx::bar_sync(1, 128);
    float inv[N];
#pragma unroll
    for (int h = 0; h < N; ++h) {
      const float l = (s.red[0][h] + s.red[1][h]) + (s.red[2][h] + s.red[3][h]);
      inv[h] = l > 0.f ? __fdividef((P8 ? 8.f : 1.f) * P.ckv_scale, l) : 0.f;  // (2 ulp; an IEEE division is twenty instructions, N times)
      lsum[h] = l;
    }
    const long long slot = (long long)seg.cta + seg.w;
    float* obase = P.o_part + slot * N * CKV;
#pragma unroll 1
    for (int mb = 0; mb < 4; ++mb) {
#pragma unroll
      for (int c0 = 0; c0 < N; c0 += 16) {
        uint32_t o[16];
        ptx::tmem_ld16(tm_lane + Cols<N, P8>::O + mb * N + c0, o);
        ptx::tmem_wait_ld();
        // lane r of block mb is channel 64mb + r (r < 64) or 256 + 64mb + r - 64 in 16-bit mode, 128mb + r in 8-bit mode
        const int ch = P8 ? 128 * mb + r : 64 * mb + (r & 63) + 256 * (r >> 6);
#pragma unroll
        for (int j = 0; j < 16; ++j) obase[(long long)(c0 + j) * CKV + ch] = __uint_as_float(o[j]) * inv[c0 + j];
      }
    }
    if (r < N) {
      float l = 0.f, mm = 0.f;
#pragma unroll
      for (int h = 0; h < N; ++h)
        if (h == r) l = lsum[h], mm = m[h];
      P.lse_part[slot * N + r] = l > 0.f ? mm + log2f(l) : -INFINITY;
    }
    ptx::tc_fence_before_sync();
    ptx::bar_sync(1, 128);  // s.red is reused by the next segment
  }
}

// ---------------------------------------------------------------------------------------------------------------
// The CTA's segments are staged through shared memory in batches; every thread takes part in the two CTA-wide
// barriers around a batch, whatever its role.
// ---------------------------------------------------------------------------------------------------------------
enum Role { kRoleSoftmax, kRoleConvert, kRoleQk, kRoleProducer, kRolePv, kRoleIdle };

template <int N, int RAW_SLOTS, bool P8, int ROLE>
__device__ __forceinline__ void run_role(DecodeSmem<N, RAW_SLOTS, P8>& s, const DecodeParams& P, const CUtensorMap* ckv_map,
                                         const CUtensorMap* sf_map, const CUtensorMap* kpe_map) {
  const int2 range = P.cta_range[blockIdx.x];
  uint32_t it = 0, seg_count = 0, hcount = 0;  // every role advances its own copies identically
  for (int w0 = range.x; w0 < range.y; w0 += kSegBatch) {
    const int n_segs = range.y - w0 < kSegBatch ? range.y - w0 : kSegBatch;
    if (ROLE == kRoleSoftmax && int(threadIdx.x) < n_segs) {
      Seg g = P.segs[(long long)blockIdx.x + w0 + threadIdx.x];
      if (g.cta != int(blockIdx.x) || g.w != w0 + int(threadIdx.x)) g.ntiles = 0;  // empty item or foreign slot
      s.segs[threadIdx.x] = g;
    }
    __syncthreads();
    if (ROLE == kRoleSoftmax) softmax_role<N, RAW_SLOTS, P8>(s, P, n_segs, it, seg_count);
    if (ROLE == kRoleConvert) convert_role<N, RAW_SLOTS, P8>(s, P, n_segs, it, seg_count);
    if (ROLE == kRoleQk) qk_role<N, RAW_SLOTS, P8>(s, P, n_segs, it);
    if (ROLE == kRoleProducer) producer_role<RAW_SLOTS>(s, P, ckv_map, sf_map, kpe_map, n_segs, hcount);
    if (ROLE == kRolePv) pv_role<N, RAW_SLOTS, P8>(s, P, n_segs, it);
    __syncthreads();
    if (s.abort_flag) break;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------------------------------------------
template <int N, int RAW_SLOTS, bool P8>
__global__ void __launch_bounds__(kDecodeThreads, 1)
mla_decode_kernel(const __grid_constant__ CUtensorMap ckv_map, const __grid_constant__ CUtensorMap sf_map,
                  const __grid_constant__ CUtensorMap kpe_map, const DecodeParams P) {
  static_assert(P8, "only the 8-bit mode is built from this template: the 16-bit mode is mla_decode_vt_kernel");
  extern __shared__ uint8_t smem_raw[];
  using Smem = DecodeSmem<N, RAW_SLOTS, P8>;
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    for (int i = 0; i < RAW_SLOTS; ++i) ptx::mbar_init(&s.raw_full[i], 1), ptx::mbar_init(&s.raw_empty[i], 4);
    for (int i = 0; i < 5; ++i) ptx::mbar_init(&s.k_full[0][i], 8), ptx::mbar_init(&s.k_full[1][i], 8);
    ptx::mbar_init(&s.k_done[0], 1), ptx::mbar_init(&s.k_done[1], 1);
    ptx::mbar_init(&s.v_full[0], 8), ptx::mbar_init(&s.v_full[1], 8);
    for (int i = 0; i < 4; ++i) ptx::mbar_init(&s.vb_full[i], 8), ptx::mbar_init(&s.vb_free[i], 1);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&s.s_full[i], 1), ptx::mbar_init(&s.s_free[i], 4);  // one arrival per softmax warp
      ptx::mbar_init(&s.p_full[i], 4), ptx::mbar_init(&s.p_free[i], 1);
    }
    s.abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&ckv_map), ptx::prefetch_tensormap(&sf_map), ptx::prefetch_tensormap(&kpe_map);
  }
  if (warp == 12) {
    ptx::tmem_alloc(&s.tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  ptx::grid_dependency_wait();  // whatever precedes the call in the stream (the lengths' producer, a schedule kernel, the
                                // previous call's use of the workspace) is settled
  // The combine kernel may be scheduled from here on: it reads a schedule kernel's output at once (settled, as this
  // grid has just seen) and waits for this grid before it reads partials.
  ptx::grid_launch_dependents();
  if (P.inline_sched) publish_own_schedule<kDecodeThreads>(reinterpret_cast<int*>(s.raw[0]), P, blockIdx.x);

  // Each role lives entirely inside its own branch, so that the register budget set at the top of the branch
  // (setmaxnreg) governs the role's code: the light issue / producer warps hand registers to the softmax and convert
  // warp groups. Registers are granted per warp group (4 warps): 0-3 softmax, 4-7 and 8-11 convert, 12-15 the rest.
  // The pool is the launch allocation (512 threads x 128): 4 x softmax + 8 x convert + 4 x 64 <= 16 x 128.
  constexpr int kSoftmaxRegs = N > 16 ? 200 : 168, kConvertRegs = N > 16 ? 120 : 136;
  static_assert(4 * kSoftmaxRegs + 8 * kConvertRegs + 4 * 64 <= 16 * 128, "register budgets exceed the CTA's allocation");
  if (warp < 4) {
    ptx::reg_alloc<kSoftmaxRegs>();
    run_role<N, RAW_SLOTS, P8, kRoleSoftmax>(s, P, &ckv_map, &sf_map, &kpe_map);
  } else if (warp < 12) {
    if constexpr (kConvertRegs >= 128) ptx::reg_alloc<kConvertRegs>(); else ptx::reg_dealloc<kConvertRegs>();
    run_role<N, RAW_SLOTS, P8, kRoleConvert>(s, P, &ckv_map, &sf_map, &kpe_map);
  } else {
    ptx::reg_dealloc<64>();
    if (warp == 12) run_role<N, RAW_SLOTS, P8, kRoleQk>(s, P, &ckv_map, &sf_map, &kpe_map);
    else if (warp == 13) run_role<N, RAW_SLOTS, P8, kRoleProducer>(s, P, &ckv_map, &sf_map, &kpe_map);
    else if (warp == 14) run_role<N, RAW_SLOTS, P8, kRolePv>(s, P, &ckv_map, &sf_map, &kpe_map);
    else run_role<N, RAW_SLOTS, P8, kRoleIdle>(s, P, &ckv_map, &sf_map, &kpe_map);
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 12) ptx::tmem_dealloc(s.tmem_base, kTmemCols);
  if (threadIdx.x == 0 && s.abort_flag) atomicExch(P.header, int(kWaitTimeout));
}

}  // namespace mla
