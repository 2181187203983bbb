// Weight-absorbed MLA decode, 16-bit mode, 16 heads per CTA: QK^T runs on the cache's own bytes, PV on V^T in TENSOR
// MEMORY; no 16-bit copy of a tile ever touches shared memory and K is never dequantised by a thread.
//
//   HBM --TMA--> raw ring (smem) --------------------------------> A operand of QK^T (packed E2M1, as stored)
//                               \--K warps--> cache block scales -> tensor memory (the MMA's scale factors of A)
//                               \--V warps--> V^T as FP16 in tensor memory, lanes = channel pairs --PV--> O^T (TMEM)
//
//   QK^T : S^T[token, head] = K[token, 512] . Q^T with tcgen05.mma kind::mxf4nvf4 (block-scaled FP4 x FP4, fp32
//          accumulation): A = the packed ckv bytes exactly as TMA delivered them (K-major, 128-byte swizzle), its scale
//          factors = the cache's E4M3 block scales, so K enters the product EXACTLY (e2m1 x e4m3, no rounding). The
//          BF16 query cannot be an FP4 operand as it is; it is written once per request as a sum of four E2M1 terms,
//          q * 2^k = sum_t s_t . c_t, with E4M3 scales s_t per row, term and 32-channel group (a quarter of the group's
//          residual maximum, so the codes stay in [-4, 4] where E2M1 is spaced by at most 1) and c_t the nearest E2M1
//          codes of the residual: the residual shrinks by 8 per term, four terms reproduce q to 2^-12 of the group's
//          maximum (the rounding of an FP16 operand is 2^-11 of the element), and the terms are MMA chains into one
//          accumulator, two terms stacked along N per chain.
//          The rope part (64 E4M3 channels) is converted to FP16 and multiplied with kind::f16 into the same
//          accumulator, with the rope rows of Q pre-multiplied by kpe_scale / ckv_scale.
//   PV   : a byte of the cache holds one token's channels 2c and 2c + 1, and the conversion instruction turns it
//          into the FP16 pair (V[t, 2c], V[t, 2c + 1]) (times the block scale: exact in FP16). That pair is stored as
//          ONE 32-bit column entry of lane c, i.e. the contraction index is k = 2 t + parity, and the parity is sorted
//          out on the B side:
//              O^T[c, 2h + e] = sum_{t, par} A[c, 2t + par] . B[2t + par, 2h + e],   B[2t + par, 2h + e] = P[t, h] (par == e)
//          so N = 32 (head, channel parity), M = 128 channel pairs per block (two blocks), and no value is ever
//          shuffled between registers: thread data from a transposing 8-bit ldmatrix goes straight through
//          convert-multiply into a 16-lane tcgen05.st. The softmax threads write P twice (as (p, 0) and (0, p)).
//   Tokens inside a 32-token group are stored in the column order the ldmatrix / tcgen05.st fragments give
//   (column 16 tg + 4 (t % 4) + (t % 16) / 4 for token 16 tg + t % 16); P^T uses the same order, and a contraction
//   does not care about the order of its index.
//
// Tensor memory (all 512 columns): V^T ring 8 x 32 | rope K 32 | scale factors of A 2 x 32 | of B 32 | S^T 2 x 32 | O^T 2 x 32.
//   V^T is a ring of eight slots of 32 tokens x 128 channel pairs = one tile: V^T(j) can be complete before P(j)
//   exists, and the V warps of tile j + 1 follow PV of tile j half by half (64 tokens). Scale factors: the word of the
//   four blocks of one K = 64 step of operand row r sits in lane r % 32 of every lane quadrant, column 4 step + r / 32
//   (A side); the B side has a word per row, pass and 128-channel quarter at column 16 pass + 4 quarter.
// Shared memory: raw ring of three 128-token tiles (packed low / high halves, block scales, rope), the query terms,
//   P^T (two tiles), and the block scales as FP16 pairs (s, s) for the V warps: two tables of a whole tile
//   ([quarter][block][32 token slots] each), written by the K warps; rows beyond the request's end get scale 0 there,
//   so V is 0 and finite wherever P is 0.
//
// Warp roles (640 threads): 0-3 softmax + epilogue, 4-7 K side (thread = token: scale factors and rope into tensor
// memory, scale table for the V warps; the query terms at the start of a request), 8-15 V^T conversion (warp % 4 = lane
// quadrant = 32 channel pairs of each block, warps 8-11 the first 64 tokens of a tile, 12-15 the second), 16 QK^T
// issue, 17 TMA producer, 18 PV issue.
// Every wait is bounded; a wait that gives up raises the CTA's abort flag and the kernel reports kWaitTimeout.
#pragma once
#include "mla_decode_sm100.cuh"

namespace mla {

constexpr int kVtRawSlots = 3;   // raw tiles in flight
constexpr int kVtRing = 8;       // V^T slots (32 tokens x 128 channel pairs, 32 columns): one tile
constexpr int kVtScRing = 2;     // scale tables of whole tiles (16 KB each)
constexpr int kVtTerms = 4;      // E2M1 terms of the query (even: two terms share an MMA)
constexpr int kVtPasses = kVtTerms / 2;
static_assert(kVtTerms % 2 == 0, "terms are stacked in pairs along N");
constexpr int kVtThreads = 640;  // 20 warps: 4 softmax, 4 K side, 8 V^T conversion, QK^T / producer / PV issue, one spare
// raw tile of 128 tokens: packed low halves | packed high halves | block scales | rope
constexpr int kVtRawHi = TILE * 128, kVtRawSf = 2 * TILE * 128, kVtRawKpe = kVtRawSf + TILE * 32;
constexpr int kVtRawTileBytes = TILE * TOKEN_BYTES;
static_assert(kVtRawTileBytes % 1024 == 0, "raw tile alignment");

struct VtCols {
  // V^T ring | rope K | scale factors of A (two tiles) | scale factors of B (per pass: four channel quarters x four columns) | S^T (two tiles) | O^T
  static constexpr uint32_t VT = 0, KROPE = 32 * kVtRing, SFA = KROPE + 32, SFB = SFA + 64, S = SFB + 16 * kVtPasses, O = S + 64;
  __host__ __device__ static constexpr uint32_t vt(uint32_t ring) { return VT + 32 * ring; }
  __host__ __device__ static constexpr uint32_t sfa(uint32_t buf) { return SFA + 32 * buf; }
  __host__ __device__ static constexpr uint32_t s(uint32_t buf) { return S + 32 * buf; }
  __host__ __device__ static constexpr uint32_t o(uint32_t mb) { return O + 32 * mb; }
  static_assert(O + 64 <= kTmemCols, "tensor memory overflow");
  static_assert(SFA % 4 == 0 && SFB % 4 == 0 && kVtPasses == 2, "scale-factor columns must be multiples of four (the B side is stored as 32 columns)");
};

struct VtSmem {
  alignas(1024) uint8_t q4[kVtPasses][2][32 * 128]; // query terms: packed E2M1, row 16 (term % 2) + head of pass term / 2, two 256-channel
                                                    // panels, K-major, 128-byte swizzle
  alignas(1024) uint8_t qrope[16 * 128];            // rope part of Q^T as FP16
  alignas(1024) uint8_t p[2][4][32 * 128];          // P^T: [buffer][32-token group][row 2h + parity], 128-byte swizzle
  alignas(1024) uint8_t raw[kVtRawSlots][kVtRawTileBytes];
  alignas(16) uint32_t sc[kVtScRing][4][32][32];    // block scales as FP16 pairs (s, s): [tile][quarter][block][token slot], the slot
                                                    // of token 16 h + 4 q + i of the quarter being 8 q + 4 h + i
  Seg segs[kSegBatch];
  alignas(16) float qa[4][16];                      // per-head score scale, ring indexed by segment count
  float red[4][16];
  float corr[16];
  uint32_t sfb[kVtTerms][4][16];                    // scale word of (term, channel quarter, head) on its way to tensor memory
  alignas(8) uint64_t raw_full[kVtRawSlots];
  uint64_t raw_empty[kVtRawSlots];
  uint64_t k_full[2], k_free[2];                    // K side of the tile in tensor memory / QK^T of the tile complete
  uint64_t rope_free;                               // QK^T's rope MMAs of the tile complete (rope K is single-buffered)
  uint64_t s_full[2], s_free[2];
  uint64_t p_full[2], p_free[2];
  uint64_t vt_full[2], vt_free[2];                  // halves of the V^T ring (64 tokens each)
  uint64_t sc_full[kVtScRing], sc_free[kVtScRing];
  uint32_t tmem_base;
  int abort_flag;
};
constexpr size_t vt_smem_bytes() { return sizeof(VtSmem) + 1024; }

// ---------------------------------------------------------------------------------------------------------------
// role: TMA producer (one warp; lane 0 issues, all lanes help with the page ids of small pages)
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void vt_producer_role(VtSmem& s, const DecodeParams& P, const CUtensorMap* ckv_map, const CUtensorMap* sf_map,
                                                 const CUtensorMap* kpe_map, int n_segs, uint32_t& it) {
  const int lane = ptx::lane_id();
  const int ps = 1 << P.page_shift;
  for (int si = 0; si < n_segs; ++si) {
    const Seg seg = s.segs[si];
    if (seg.ntiles <= 0) continue;
    const int* pt = P.page_table + (long long)seg.b * P.pt_stride;
    // page ids of a tile's two half tiles and of the two that are prefetched into L2 (three tiles ahead: the ring itself
    // is too shallow to cover HBM latency); read one tile ahead of their use so that nothing ever waits for them
    auto fetch_ids = [&](int tk0, int (&pg)[2], int (&pf)[2]) {
      pg[0] = pg[1] = 0, pf[0] = pf[1] = -1;
      if (ps >= HALF && lane == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int tk = tk0 + h * HALF;
          if (tk < seg.tok_end) pg[h] = pt[tk >> P.page_shift];
          if (tk + 3 * TILE < seg.tok_end) pf[h] = pt[(tk + 3 * TILE) >> P.page_shift];
        }
      }
    };
    int page_nx[2], pf_nx[2];
    fetch_ids(seg.tok0, page_nx, pf_nx);
    for (int t = 0; t < seg.ntiles; ++t, ++it) {
      const int slot = it % kVtRawSlots;
      const int tok = seg.tok0 + t * TILE;
      int nvalid = seg.tok_end - tok;
      nvalid = nvalid < 0 ? 0 : (nvalid > TILE ? TILE : nvalid);
      const int page[2] = {page_nx[0], page_nx[1]}, page_pf[2] = {pf_nx[0], pf_nx[1]};
      if (t + 1 < seg.ntiles) fetch_ids(tok + TILE, page_nx, pf_nx);
      if (ps >= HALF) {
        // The pages of the tile three ahead, into L2, by plain prefetch instructions of all lanes: a tensor-map prefetch
        // costs the TMA unit as much as the load itself (it walks the box row by row), and the TMA unit is what
        // bounds this warp. A page's 64 tokens are contiguous in each of the three arrays. Not waiting for the slot.
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int pf = __shfl_sync(~0u, page_pf[h], 0);
          if (uint32_t(pf) < uint32_t(P.num_pages)) {
            const long long row2 = ((long long)pf << P.page_shift) + ((tok + h * HALF + 3 * TILE) & (ps - 1));
            const uint8_t* c = P.ckv + row2 * 256 + lane * 128;  // 16 KB = 128 lines
#pragma unroll
            for (int k = 0; k < 4; ++k) ptx::prefetch_l2(c + k * 4096);
            ptx::prefetch_l2(P.kpe + row2 * 64 + lane * 128);    // 4 KB = 32 lines
            if (lane < 16) ptx::prefetch_l2(P.sf + row2 * 32 + lane * 128);  // 2 KB = 16 lines
          }
        }
      }
      const bool ok = ptx::mbar_wait(&s.raw_empty[slot], ((it / kVtRawSlots) & 1) ^ 1, &s.abort_flag);
      if (!__all_sync(~0u, ok)) return;
      uint8_t* dst = s.raw[slot];
      uint64_t* bar = &s.raw_full[slot];
      if (nvalid == 0) {
        ptx::mbar_arrive_if(bar, lane == 0);
      } else if (ps >= HALF) {
        if (lane == 0) {
          const int nh = nvalid > HALF ? 2 : 1;  // half tiles that hold a live token
          ptx::mbar_arrive_expect_tx(bar, uint32_t(nh) * HALF * TOKEN_BYTES);
          for (int h = 0; h < nh; ++h) {
            const int tk = tok + h * HALF;
            // A stale or corrupt id is never dereferenced: the boxes are taken beyond the last row of the cache instead,
            // where TMA fills zeros (scale 0: the rows contribute score 0 and value 0), and the call is flagged.
            const bool bad = uint32_t(page[h]) >= uint32_t(P.num_pages);
            if (bad) atomicExch(P.header, int(kBadPage));
            const int row = bad ? (P.num_pages << P.page_shift) : (page[h] << P.page_shift) + (tk & (ps - 1));
            ptx::tma_load_2d(dst + h * HALF * 128, ckv_map, 0, row, bar);
            ptx::tma_load_2d(dst + kVtRawHi + h * HALF * 128, ckv_map, 128, row, bar);
            if (!bad) {
              // scales and rope: the half tile's rows are contiguous, one linear copy each (a tiled copy costs the TMA
              // unit one request per ROW, however short the row)
              ptx::bulk_load(dst + kVtRawSf + h * HALF * 32, P.sf + (long long)row * 32, HALF * 32, bar);
              ptx::bulk_load(dst + kVtRawKpe + h * HALF * 64, P.kpe + (long long)row * 64, HALF * 64, bar);
            } else {
              ptx::tma_load_2d(dst + kVtRawSf + h * HALF * 32, sf_map, 0, row, bar);  // zeros (in any layout)
              ptx::tma_load_2d(dst + kVtRawKpe + h * HALF * 64, kpe_map, 0, row, bar);
            }
          }
        }
      } else {
        // small pages: one box per page that holds a live token (at most 128 per tile), lanes share the pages;
        // scales and rope arrive through linear bulk copies (unswizzled)
        const int npages = (nvalid + ps - 1) >> P.page_shift;
        int page[4];
        uint32_t good = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
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
        for (int k = 0; k < 4; ++k) {
          if (page[k] < 0) continue;
          const int row = page[k] << P.page_shift, r0 = (lane + 32 * k) << P.page_shift;
          ptx::tma_load_2d(dst + r0 * 128, ckv_map, 0, row, bar);
          ptx::tma_load_2d(dst + kVtRawHi + r0 * 128, ckv_map, 128, row, bar);
          ptx::bulk_load(dst + kVtRawSf + r0 * 32, P.sf + (long long)row * 32, ps * 32, bar);
          ptx::bulk_load(dst + kVtRawKpe + r0 * 64, P.kpe + (long long)row * 64, ps * 64, bar);
        }
      }
      __syncwarp();
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// role: K side (4 warps; thread = token row of the tile)
// ---------------------------------------------------------------------------------------------------------------
// The query of a segment, by the 128 K threads: row n = thread / 8, channels [64 sub, 64 sub + 64) with sub = thread % 8.
// The row (latent part, and rope part times kpe_scale / ckv_scale) is scaled by 2^(9 - e), e = floor(log2(row maximum)).
// Latent part: E2M1 terms. A term has sixteen E4M3 scales per row: one per (128-channel quarter, position j of the
// 16-channel block inside its 64-channel MMA step), i.e. per 32 channels {128 qd + 64 a + 16 j ..}: that is how far the
// 32 tensor-memory columns left for the B side's scale factors go (the MMA takes a scale word per step; a quarter's two
// steps share theirs). A scale is a quarter of its group's residual maximum, rounded; the codes are the nearest E2M1 of
// residual / scale (saturating), and the residual is updated with what the codes decode to, so every term corrects the
// rounding of the ones before it, and an outlier channel coarsens only its own group.
// Rope part: FP16, K-major with the 128-byte swizzle.
// `must_wait`: QK^T of the previous tile (barrier `prev_done`, `prev_parity`) still reads the old query; the rows are
// fetched and scaled first, and the wait sits before the first store. Returns false if the wait gave up (`dead`: an
// earlier one already has).
__device__ __forceinline__ bool vt_load_query(VtSmem& s, const DecodeParams& P, const Seg& seg, int kt, int par, int lane, int quad,
                                              bool dead, bool must_wait, uint64_t* prev_done, uint32_t prev_parity) {
  const int n = kt >> 3, sub = kt & 7;
  const long long row = (long long)seg.b * P.heads + (long long)seg.hg * 16 + n;
  float r[64];
  {
    uint4 qn[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) qn[k] = reinterpret_cast<const uint4*>(P.q_nope + row * CKV)[8 * sub + k];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t w[4] = {qn[k].x, qn[k].y, qn[k].z, qn[k].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) r[8 * k + 2 * j] = __uint_as_float(w[j] << 16), r[8 * k + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
  }
  const uint4 qp = reinterpret_cast<const uint4*>(P.q_pe + row * KPE)[sub];
  const float ratio = P.kpe_scale / P.ckv_scale;
  auto finite = [](float v) { const uint32_t b = __float_as_uint(v) & 0x7FFFFFFFu; return b < 0x7F800000u ? b : 0u; };  // inf / nan do not set the scale
  auto row_max = [&](uint32_t m) {
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) m = max(m, __shfl_xor_sync(~0u, m, o));
    return m;
  };
  float pe[8];
  uint32_t m_pe = 0, m = 0;
  {
    const uint32_t w[4] = {qp.x, qp.y, qp.z, qp.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      pe[2 * j] = __uint_as_float(w[j] << 16) * ratio, pe[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u) * ratio;
      m_pe = max(m_pe, max(finite(pe[2 * j]), finite(pe[2 * j + 1])));
    }
  }
#pragma unroll
  for (int i = 0; i < 64; ++i) m = max(m, finite(r[i]));
  m = row_max(m), m_pe = row_max(m_pe);
  // e = floor(log2(latent maximum)): the first term's scales are then at most 256 and the last term's still E4M3 normals
  // for groups 64 times smaller than the row; raised if the rope part (FP16, at most 2^15 after scaling) is more than 2^5
  // times larger
  int e = int(m >> 23) - 127, e_pe = int(m_pe >> 23) - 127;
  e = e > e_pe - 5 ? e : e_pe - 5;
  e = e < -100 ? -100 : e;
  const float up = __uint_as_float(uint32_t(9 - e + 127) << 23);  // 2^(9 - e), exact: the row maximum lands in [512, 1024)
#pragma unroll
  for (int i = 0; i < 64; ++i) {
    r[i] *= up;
    if (!(fabsf(r[i]) < INFINITY)) r[i] = 0.f;  // a non-finite query element has no meaningful result anyway; keep the rest of the row intact
  }
  {
    const bool ok = !dead && (!must_wait || ptx::mbar_wait(prev_done, prev_parity, &s.abort_flag));
    if (ptx::bar_red_or(2, 128, !ok)) return false;
    ptx::tc_fence_after_sync();
  }
  const uint32_t panel = uint32_t(sub) >> 2, c0 = 2 * (uint32_t(sub) & 3);
#pragma unroll 1  // (a term is some 700 instructions; unrolled, the routine is a third of the kernel's code and is fetched afresh at every request)
  for (int t = 0; t < kVtTerms; ++t) {
    uint32_t sc8[4];
    float scf[4], inv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t mt = 0;
#pragma unroll
      for (int i = 0; i < 16; ++i) mt = max(mt, __float_as_uint(r[16 * j + i]) & 0x7FFFFFFFu);
      mt = max(mt, __shfl_xor_sync(~0u, mt, 1));  // the other step of this 128-channel quarter
      sc8[j] = ptx::f32x2_to_e4m3x2(__uint_as_float(mt) * 0.25f, 0.f) & 0xFFu;  // E4M3 (positive), round to nearest
      scf[j] = __half2float(__ushort_as_half(uint16_t(ptx::e4m3x2_to_f16x2(uint16_t(sc8[j])) & 0xFFFFu)));
      inv[j] = scf[j] > 0.f ? __fdividef(1.f, scf[j]) : 0.f;  // (only steers the choice of codes: the residual is updated with what they decode to)
    }
    uint32_t cw[8];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      float y[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = r[8 * w + i] * inv[w >> 1];
      uint32_t h[4];
      cw[w] = ptx::f32x8_to_e2m1x8(y, h);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&h[i]));
        r[8 * w + 2 * i] = fmaf(-d.x, scf[w >> 1], r[8 * w + 2 * i]);
        r[8 * w + 2 * i + 1] = fmaf(-d.y, scf[w >> 1], r[8 * w + 2 * i + 1]);
      }
    }
    uint8_t* dst = s.q4[t >> 1][panel] + (16 * (t & 1) + n) * 128;  // (the swizzle term of row 16 + n is that of row n)
    *reinterpret_cast<uint4*>(dst + (((c0) ^ uint32_t(n & 7)) << 4)) = make_uint4(cw[0], cw[1], cw[2], cw[3]);
    *reinterpret_cast<uint4*>(dst + (((c0 + 1) ^ uint32_t(n & 7)) << 4)) = make_uint4(cw[4], cw[5], cw[6], cw[7]);
    if ((sub & 1) == 0) s.sfb[t][sub >> 1][n] = sc8[0] | (sc8[1] << 8) | (sc8[2] << 16) | (sc8[3] << 24);  // byte j = block j of the step
  }
  {
    uint32_t h[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = ptx::f32x2_to_f16x2(pe[2 * j] * up, pe[2 * j + 1] * up);
    *reinterpret_cast<uint4*>(s.qrope + n * 128 + (uint32_t(sub ^ (n & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
  }
  if (sub == 0) s.qa[par][n] = P.sm_scale_log2 * P.ckv_scale * __uint_as_float(uint32_t(e - 9 + 127) << 23);
  ptx::fence_proxy_async_smem();
  ptx::bar_sync(2, 128);
  // scale factors of B: pass p multiplies K with B rows [terms 2p | 2p + 1] x 16 heads; the scale word of row i for the
  // steps of quarter qd goes to lane i of every lane quadrant, column 16 p + 4 qd
  uint32_t w[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) w[i] = 0u;
#pragma unroll
  for (int pp = 0; pp < kVtPasses; ++pp)
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) w[16 * pp + 4 * qd] = s.sfb[2 * pp + (lane >> 4)][qd][lane & 15];
  ptx::tmem_st32(s.tmem_base + (uint32_t(quad * 32) << 16) + VtCols::SFB, w);
  ptx::tmem_wait_st();
  return true;
}

// One tile of a K thread. Returns false if a wait gave up.
__device__ __forceinline__ bool vt_k_step(VtSmem& s, const DecodeParams& P, const Seg& seg, int t, uint32_t it, int lane, int quad) {
  const int r = quad * 32 + lane;
  const uint32_t tm_lane = s.tmem_base + (uint32_t(quad * 32) << 16);
  const int slot = it % kVtRawSlots;
  const uint32_t raw = ptx::smem_u32(s.raw[slot]);
  const uint32_t buf = it & 1;
  if (!__all_sync(~0u, ptx::mbar_wait(&s.raw_full[slot], (it / kVtRawSlots) & 1, &s.abort_flag))) return false;
  const bool valid = seg.tok0 + t * TILE + r < seg.tok_end;
  // tests of the barriers needed further down, issued before the work that precedes them
  const uint32_t pr_kfree = ptx::mbar_probe(&s.k_free[buf], ((it >> 1) & 1) ^ 1), pr_rope = ptx::mbar_probe(&s.rope_free, (it & 1) ^ 1);

  // The two 32-register payloads (rope, scale factors) are built and stored one after the other, so that only one of
  // them is live at a time.
  // ---- rope: 64 E4M3 bytes -> 32 columns of FP16 pairs; the rope MMAs of tile it - 1 must be done with rope K
  {
    uint32_t h[32];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 v = ptx::lds128(raw + kVtRawKpe + r * 64 + (uint32_t(c) << 4));
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        h[8 * c + 2 * j] = ptx::e4m3x2_to_f16x2(uint16_t(w[j] & 0xFFFF));
        h[8 * c + 2 * j + 1] = ptx::e4m3x2_to_f16x2(uint16_t(w[j] >> 16));
      }
    }
    const bool ok = ptx::mbar_wait_probed(pr_rope, &s.rope_free, (it & 1) ^ 1, &s.abort_flag);
    ptx::tc_fence_after_sync();
    if (!__all_sync(~0u, ok)) return false;
    ptx::tmem_st32(tm_lane + VtCols::KROPE, h);
  }
  // ---- scale factors of A: lane l of this quadrant holds, for K step a, columns 4a + j = the scale word a of token
  // 32 j + l; QK^T of tile it - 2 must have finished with this scale-factor buffer
  {
    uint32_t f[32];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int tk = 32 * j + lane;
      const uint4 a = ptx::lds128(raw + kVtRawSf + tk * 32), b = ptx::lds128(raw + kVtRawSf + tk * 32 + 16);
      f[j] = a.x, f[4 + j] = a.y, f[8 + j] = a.z, f[12 + j] = a.w, f[16 + j] = b.x, f[20 + j] = b.y, f[24 + j] = b.z, f[28 + j] = b.w;
    }
    const bool ok = ptx::mbar_wait_probed(pr_kfree, &s.k_free[buf], ((it >> 1) & 1) ^ 1, &s.abort_flag);
    ptx::tc_fence_after_sync();
    if (!__all_sync(~0u, ok)) return false;
    ptx::tmem_st32(tm_lane + VtCols::sfa(buf), f);
  }
  ptx::tmem_wait_st();
  ptx::tc_fence_before_sync();
  __syncwarp();
  ptx::mbar_arrive_if(&s.k_full[buf], lane == 0);
  // ---- block scales of this token for the V warps, as FP16 pairs (s, s) ready to be multiplied with a converted byte; 0
  // beyond the request's end. Written last: the V warps are the furthest behind of all readers of the tile, and the wait
  // for a free table must not hold up QK^T.
  {
    const uint32_t x = 0;
    const uint4 a = ptx::lds128(raw + kVtRawSf + r * 32 + ((0u ^ x) << 4));
    const uint4 b = ptx::lds128(raw + kVtRawSf + r * 32 + ((1u ^ x) << 4));
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    const uint32_t qs = it % kVtScRing;  // the tile's table; this warp writes its quarter
    if (!__all_sync(~0u, ptx::mbar_wait(&s.sc_free[qs], ((it / kVtScRing) & 1) ^ 1, &s.abort_flag))) return false;
    // token lane = 16 h + 4 q + i of the quarter -> slot 8 q + 4 h + i
    const uint32_t dst = ptx::smem_u32(&s.sc[qs][quad][0][8 * ((lane >> 2) & 3) + 4 * (lane >> 4) + (lane & 3)]);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t wj = valid ? w[j] : 0u;
      const uint32_t lo = ptx::e4m3x2_to_f16x2(uint16_t(wj & 0xFFFF)), hi = ptx::e4m3x2_to_f16x2(uint16_t(wj >> 16));
      ptx::sts32(dst + (4 * j + 0) * 128, __byte_perm(lo, 0, 0x1010)), ptx::sts32(dst + (4 * j + 1) * 128, __byte_perm(lo, 0, 0x3232));
      ptx::sts32(dst + (4 * j + 2) * 128, __byte_perm(hi, 0, 0x1010)), ptx::sts32(dst + (4 * j + 3) * 128, __byte_perm(hi, 0, 0x3232));
    }
    __syncwarp();
    ptx::mbar_arrive_if(&s.sc_full[qs], lane == 0);
    ptx::mbar_arrive_if(&s.raw_empty[slot], lane == 0);  // every byte this warp needs from the raw tile is in a register or stored
  }
  return true;
}

// A warp whose wait gave up does not leave at once: the 128 K threads meet at a named barrier at the start of every
// segment, so it carries on (skipping the work) to the next such barrier, where the failure is OR-reduced and all
// four warps leave together.
__device__ __forceinline__ void vt_k_role(VtSmem& s, const DecodeParams& P, int n_segs, uint32_t& it, uint32_t& seg_count) {
  const int lane = ptx::lane_id();
  const int quad = (threadIdx.x >> 5) & 3;
  bool dead = false;
  for (int si = 0; si < n_segs; ++si) {
    const Seg seg = s.segs[si];
    if (seg.ntiles <= 0) continue;
    // the previous tile's QK^T must be done reading the query before the new one overwrites it (waited for inside,
    // after the rows have been fetched)
    if (!vt_load_query(s, P, seg, quad * 32 + lane, seg_count & 3, lane, quad, dead, it != 0, &s.k_free[(it - 1) & 1], ((it - 1) >> 1) & 1))
      return;
    ++seg_count;
    for (int t = 0; t < seg.ntiles; ++t, ++it) {
      if (!vt_k_step(s, P, seg, t, it, lane, quad)) {
        dead = true;
        break;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// role: V^T conversion (4 warps; warp % 4 = lane quadrant = channel pairs [32 quad, +32) of each 128-pair block)
// ---------------------------------------------------------------------------------------------------------------
// A unit of work is one transposing ldmatrix: 32 tokens x 16 channel pairs (two scale blocks), i.e. half of this
// warp's share of a V^T slot. A 32-token group is four units (2 blocks x 2 halves), a tile four groups. The scales come
// from the table as E4M3 byte pairs (b, b), which the conversion instruction turns into the FP16 pair (s, s) it is
// multiplied with. Every synchronisation costs this warp a shared-memory round trip during which it has nothing else
// to do, so there are few of them: the inputs are waited for once per tile, and V^T is handed to the PV warp in halves of
// 64 tokens (four ring slots). The loop over groups is software pipelined: the loads of a unit are issued before the
// arithmetic of the unit before it, barrier tests are issued ahead of the point that needs their answer, and a finished
// half is published only after the arithmetic of the following unit, when its tensor-memory stores have landed.
struct VtUnitRegs {
  uint32_t rw[4];
  uint4 sa[2], sb[2];  // (s, s) of the unit's two blocks: 8 tokens each (4q .. 4q + 3 of both 16-token halves)
};
__device__ __forceinline__ void vt_v_role(VtSmem& s, const DecodeParams& P, int n_segs, uint32_t& it, const uint32_t vw) {
  const int lane = ptx::lane_id();
  const int quad = (threadIdx.x >> 5) & 3;
  const int q = lane & 3;
  const int mrow = lane & 15, mat = lane >> 4;  // this lane addresses row `mrow` of ldmatrix matrix `mat`
  const uint32_t tm_q = s.tmem_base + (uint32_t(32 * quad) << 16);
  int total = 0;
  for (int si = 0; si < n_segs; ++si) total += s.segs[si].ntiles > 0 ? s.segs[si].ntiles : 0;
  // per-lane constants: byte offset of this lane's ldmatrix row inside a 32-token group, swizzle term
  const uint32_t row_off = uint32_t(16 * mat + mrow) * 128, swz = uint32_t(mrow & 7);
  uint32_t raw_base = 0, sc_base = 0;  // of the tile whose loads are being issued
  // unit (mb, ch) of group qt of the open tile: one ldmatrix and the scales of each of its 2 blocks x 8 tokens
  auto load_unit = [&](uint32_t qt, int mb, int ch, VtUnitRegs& R) {
    const uint32_t chunk = 2 * quad + ch;
    ptx::ldmatrix_x2_trans_b8(raw_base + qt * (32 * 128) + mb * kVtRawHi + ((chunk ^ swz) << 4), R.rw);
    const uint32_t a = sc_base + qt * 4096 + (16 * mb + 2 * chunk) * 128;  // block row of the table: [4 q][2 halves][4 tokens] words
    R.sa[0] = ptx::lds128(a), R.sa[1] = ptx::lds128(a + 16), R.sb[0] = ptx::lds128(a + 128), R.sb[1] = ptx::lds128(a + 144);
  };
  // arithmetic and store of unit (mb, ch) of group qt, whose loads are in R
  auto finish_unit = [&](uint32_t qt, int mb, int ch, const VtUnitRegs& R, uint32_t (&v)[16]) {
#pragma unroll
    for (int tg = 0; tg < 2; ++tg) {
      uint32_t ea[4], eb[4];
      ptx::e2m1x8_to_f16x8(R.rw[2 * tg], ea);      // channel pair g, tokens 16 tg + 4q + i
      ptx::e2m1x8_to_f16x8(R.rw[2 * tg + 1], eb);  // channel pair g + 8
      const uint32_t pa[4] = {R.sa[tg].x, R.sa[tg].y, R.sa[tg].z, R.sa[tg].w}, pb[4] = {R.sb[tg].x, R.sb[tg].y, R.sb[tg].z, R.sb[tg].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[8 * tg + 2 * i] = ptx::hmul2(ea[i], pa[i]);
        v[8 * tg + 2 * i + 1] = ptx::hmul2(eb[i], pb[i]);
      }
    }
  };
  auto store_unit = [&](uint32_t qt, int mb, int ch, const uint32_t (&v)[16]) {
    ptx::tmem_st_16x128b_x8(tm_q + (uint32_t(16 * ch) << 16) + VtCols::vt(2 * qt + mb), v);
  };
  VtUnitRegs ra, rb;  // ping-pong: neither set is ever copied
#pragma unroll 1
  for (int tl = 0; tl < total; ++tl) {
    const uint32_t tile = it + uint32_t(tl);
    const uint32_t slot = tile % kVtRawSlots, ts = tile % kVtScRing;
    {  // the tile's scale table and raw bytes
      bool ok = ptx::mbar_wait(&s.sc_full[ts], (tile / kVtScRing) & 1, &s.abort_flag);
      ok = ok && ptx::mbar_wait(&s.raw_full[slot], (tile / kVtRawSlots) & 1, &s.abort_flag);
      if (!__all_sync(~0u, ok)) return;
    }
    // PV must have released this half of the ring (the previous tile's): the test is issued now, its answer used after
    // the first unit's arithmetic
    const uint32_t probed = ptx::mbar_probe(&s.vt_free[vw], (tile & 1) ^ 1);
    raw_base = ptx::smem_u32(s.raw[slot]) + row_off;
    sc_base = ptx::smem_u32(&s.sc[ts][0][0][0]) + 32 * q;
    load_unit(2 * vw, 0, 0, ra);
#pragma unroll 1
    for (uint32_t gi = 0; gi < 2; ++gi) {
      const uint32_t qt = 2 * vw + gi;
      uint32_t v[16];
      load_unit(qt, 0, 1, rb);
      finish_unit(qt, 0, 0, ra, v);
      if (gi == 0) {
        const bool ok = ptx::mbar_wait_probed(probed, &s.vt_free[vw], (tile & 1) ^ 1, &s.abort_flag);
        ptx::tc_fence_after_sync();
        if (!__all_sync(~0u, ok)) return;
      }
      store_unit(qt, 0, 0, v);
      load_unit(qt, 1, 0, ra);
      finish_unit(qt, 0, 1, rb, v);
      store_unit(qt, 0, 1, v);
      load_unit(qt, 1, 1, rb);
      finish_unit(qt, 1, 0, ra, v);
      store_unit(qt, 1, 0, v);
      if (gi == 0) load_unit(qt + 1, 0, 0, ra);
      finish_unit(qt, 1, 1, rb, v);
      store_unit(qt, 1, 1, v);
    }
    // every input of the half is in a register or stored: release the table and this warp's share of the raw slot, then
    // hand the half to the PV warp once the stores have landed
    __syncwarp();
    ptx::mbar_arrive_if(&s.sc_free[ts], lane == 0);
    ptx::mbar_arrive_if(&s.raw_empty[slot], lane == 0);
    ptx::tmem_wait_st();
    ptx::tc_fence_before_sync();
    __syncwarp();
    ptx::mbar_arrive_if(&s.vt_full[vw], lane == 0);
  }
  it += uint32_t(total);
}

// ---------------------------------------------------------------------------------------------------------------
// roles: MMA issue. The whole warp runs the loop so that every operand is warp-uniform; one elected lane issues.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void vt_qk_role(VtSmem& s, const DecodeParams& P, int n_segs, uint32_t& it) {
  const bool leader = ptx::elect_one();
  const uint32_t tm = s.tmem_base;
  const uint32_t idesc16 = ptx::instr_desc(128, 16, ptx::FMT_F16, ptx::FMT_F16, false, false);
  const uint32_t idesc4 = ptx::instr_desc_mxf4nvf4(128, 32);
  const uint64_t qrope_desc = ptx::smem_desc_sw128(ptx::smem_u32(s.qrope), 16, 1024);
  const uint64_t q4_desc = ptx::smem_desc_sw128(ptx::smem_u32(s.q4[0][0]), 16, 1024);
  for (int si = 0; si < n_segs; ++si) {
    const int ntiles = s.segs[si].ntiles;
    for (int t = 0; t < ntiles; ++t, ++it) {
      const uint32_t buf = it & 1, slot = it % kVtRawSlots;
      // softmax of tile it - 2 must have read this S^T buffer; the packed bytes (this thread's MMAs read them through
      // the async proxy) and the K side in tensor memory must be there. The three tests are issued together.
      {
        const uint32_t p0 = ptx::mbar_probe(&s.s_free[buf], ((it >> 1) - 1) & 1), p1 = ptx::mbar_probe(&s.raw_full[slot], (it / kVtRawSlots) & 1),
                       p2 = ptx::mbar_probe(&s.k_full[buf], (it >> 1) & 1);
        bool ok = it < 2 || ptx::mbar_wait_probed(p0, &s.s_free[buf], ((it >> 1) - 1) & 1, &s.abort_flag);
        ok = ok && ptx::mbar_wait_probed(p1, &s.raw_full[slot], (it / kVtRawSlots) & 1, &s.abort_flag);
        ok = ok && ptx::mbar_wait_probed(p2, &s.k_full[buf], (it >> 1) & 1, &s.abort_flag);
        if (!__all_sync(~0u, ok)) return;
      }
      ptx::tc_fence_after_sync();
      if (leader) {
        const uint64_t k_desc = ptx::smem_desc_sw128(ptx::smem_u32(s.raw[slot]), 16, 1024);
        // K step a = channels [64 a, +64): panel a / 4, 32 bytes per step. B of pass pp = rows [term 2 pp | term 2 pp + 1].
        auto fp4 = [&](int pp, int a, uint32_t accum) {
          const uint32_t off = uint32_t(a >> 2) * kVtRawHi + uint32_t(a & 3) * 32;
          const uint32_t qoff = uint32_t(pp * 2 + (a >> 2)) * (32 * 128) + uint32_t(a & 3) * 32;
          ptx::mma_mxf4nvf4_ss(tm + VtCols::s(buf), k_desc + (off >> 4), q4_desc + (qoff >> 4), idesc4, tm + VtCols::sfa(buf) + 4 * a,
                               tm + VtCols::SFB + 16 * pp + 4 * (a >> 1), accum);
        };
        fp4(0, 0, 0);  // the first MMA of the tile overwrites all 32 columns of the accumulator
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)  // rope: 64 channels as FP16 from tensor memory, into the columns of the even terms
          ptx::mma_f16_ts(tm + VtCols::s(buf), tm + VtCols::KROPE + 8 * ks, qrope_desc + ((ks * 32) >> 4), idesc16, 1);
        ptx::mma_commit(&s.rope_free);
#pragma unroll 1
        // (rolled on purpose: unrolled, the 20 + 32 MMAs of the two issue warps with their descriptor arithmetic made the
        // whole kernel 15 % slower; the issue warps share schedulers and instruction caches with the working warps)
        for (int a = 1; a < 8 * kVtPasses; ++a) fp4(a >> 3, a & 7, 1);
        ptx::mma_commit(&s.k_free[buf]);
        ptx::mma_commit(&s.s_full[buf]);
        ptx::mma_commit(&s.raw_empty[slot]);
      }
    }
  }
}

__device__ __forceinline__ void vt_pv_role(VtSmem& s, const DecodeParams& P, int n_segs, uint32_t& it) {
  const bool leader = ptx::elect_one();
  const uint32_t tm = s.tmem_base;
  const uint32_t idesc = ptx::instr_desc(128, 32, ptx::FMT_F16, ptx::FMT_F16, false, false);
  for (int si = 0; si < n_segs; ++si) {
    const int ntiles = s.segs[si].ntiles;
    for (int t = 0; t < ntiles; ++t, ++it) {
      const uint32_t buf = it & 1;
      if (!__all_sync(~0u, ptx::mbar_wait(&s.p_full[buf], (it >> 1) & 1, &s.abort_flag))) return;
#pragma unroll 1
      for (int hf = 0; hf < 2; ++hf) {  // half of the ring = 64 tokens = slots 4 hf .. 4 hf + 3
        if (!__all_sync(~0u, ptx::mbar_wait(&s.vt_full[hf], it & 1, &s.abort_flag))) return;
        ptx::tc_fence_after_sync();
        if (leader) {
#pragma unroll 1
          for (int k = 0; k < 4; ++k) {  // slot = (32-token group sl / 2, channel-pair block sl % 2)
            const int sl = 4 * hf + k;
            const uint64_t p_desc = ptx::smem_desc_sw128(ptx::smem_u32(s.p[buf][sl >> 1]), 16, 1024);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              ptx::mma_f16_ts(tm + VtCols::o(sl & 1), tm + VtCols::vt(sl) + 8 * ks, p_desc + ((ks * 32) >> 4), idesc,
                              (t | (sl >> 1) | ks) != 0);
          }
          ptx::mma_commit(&s.vt_free[hf]);
          if (hf == 1) ptx::mma_commit(&s.p_free[buf]);
        }
      }
    }
  }
}


// ---------------------------------------------------------------------------------------------------------------
// role: softmax + epilogue (4 warps; thread r = token row of S^T and channel-pair row of O^T)
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void vt_softmax_role(VtSmem& s, const DecodeParams& P, int n_segs, uint32_t& it, uint32_t& seg_count) {
  constexpr int N = 16;
  const int lane = ptx::lane_id(), warp = threadIdx.x >> 5;
  const int r = threadIdx.x;  // 0..127
  const uint32_t tm_lane = s.tmem_base + (uint32_t(warp * 32) << 16);
  constexpr float kGrow = 8.f;  // rescale only when a score exceeds the running max by 2^8 (P stays <= 256)
  // P^T row n = 2h + parity (128 bytes = one 32-token group): token 16 tg + tl sits in column 16 tg + 4 (tl % 4) + tl / 4,
  // i.e. 16-byte chunk 4 tg + tl % 4, word tl / 4 of the chunk; the chunk index is swizzled by n % 8.
  const uint32_t tl = r & 15, tg = (r >> 4) & 1;
  const uint32_t p_chunk = 4 * tg + (tl & 3), p_off = 4 * (tl >> 2);
  for (int si = 0; si < n_segs; ++si) {
    const Seg seg = s.segs[si];
    if (seg.ntiles <= 0) continue;
    const int par_q = seg_count & 3;
    ++seg_count;
    // running maximum and sum per head. The maximum starts at a finite sentinel far below any score rather than at
    // -inf: x - m and m - m' then never meet inf - inf, and no special case is needed anywhere below.
    constexpr float kNoMax = -1e30f;
    float m[N], lsum[N];
#pragma unroll
    for (int h = 0; h < N; ++h) m[h] = kNoMax, lsum[h] = 0.f;

    for (int t = 0; t < seg.ntiles; ++t, ++it) {
      const uint32_t buf = it & 1;
      const bool ok = ptx::mbar_wait(&s.s_full[buf], (it >> 1) & 1, &s.abort_flag);
      ptx::tc_fence_after_sync();
      float x[N];
      float qa_r[N];  // per-head score scales, written by the K warps before the segment's first K side was published
      {
        const uint32_t qa_addr = ptx::smem_u32(&s.qa[par_q][0]);
#pragma unroll
        for (int j = 0; j < N / 4; ++j) {
          const uint4 v = ptx::lds128(qa_addr + 16 * j);
          qa_r[4 * j] = __uint_as_float(v.x), qa_r[4 * j + 1] = __uint_as_float(v.y), qa_r[4 * j + 2] = __uint_as_float(v.z), qa_r[4 * j + 3] = __uint_as_float(v.w);
        }
      }
      if (ok) {
        const bool valid = seg.tok0 + t * TILE + r < seg.tok_end;
        uint32_t sv[32];  // columns [0, 16): even terms + rope, [16, 32): odd terms
        ptx::tmem_ld32(tm_lane + VtCols::s(buf), sv);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int h = 0; h < N; ++h) x[h] = valid ? (__uint_as_float(sv[h]) + __uint_as_float(sv[16 + h])) * qa_r[h] : -INFINITY;
      } else {
#pragma unroll
        for (int h = 0; h < N; ++h) x[h] = -INFINITY;
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      ptx::mbar_arrive_if(&s.s_free[buf], lane == 0);  // QK^T of tile it + 2 may overwrite this S^T buffer
      // does any score exceed its running maximum by more than the slack? (one maximum over the differences: a chain of
      // sixteen predicate updates would be sixteen predicate latencies long; x = m = -inf gives NaN, which fmaxf drops)
      float dmax[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) dmax[j] = fmaxf(fmaxf(x[j] - m[j], x[4 + j] - m[4 + j]), fmaxf(x[8 + j] - m[8 + j], x[12 + j] - m[12 + j]));
      const bool need = !ok || fmaxf(fmaxf(dmax[0], dmax[1]), fmaxf(dmax[2], dmax[3])) > kGrow;
      if (ptx::bar_red_or(1, 128, need)) {
        if (ptx::bar_red_or(1, 128, s.abort_flag != 0)) return;  // uniform decision, whoever raised the flag
#pragma unroll
        for (int h = 0; h < N; ++h) {
          float v = x[h];
#pragma unroll
          for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(~0u, v, o));
          if (lane == 0) s.red[warp][h] = v;
        }
        ptx::bar_sync(1, 128);
        bool any_scale = false;
#pragma unroll
        for (int h = 0; h < N; ++h) {
          const float mx = fmaxf(fmaxf(s.red[0][h], s.red[1][h]), fmaxf(s.red[2][h], s.red[3][h]));
          const float mn = fmaxf(m[h], mx);
          const float c = ptx::ex2(m[h] - mn);  // 0 when the first real score replaces the sentinel, 1 when nothing changes
          any_scale |= c != 1.f;
          lsum[h] *= c;
          m[h] = mn;
          s.corr[h] = c;
        }
        // O^T *= corr per head: after the previous tile's PV has finished; this tile's PV is not issued before this
        // thread arrives on p_full.
        if (t > 0 && any_scale) {
          const bool okv = ptx::mbar_wait(&s.p_free[buf ^ 1], ((it - 1) >> 1) & 1, &s.abort_flag);  // PV of tile it - 1
          if (ptx::bar_red_or(1, 128, !okv)) return;
          ptx::tc_fence_after_sync();
#pragma unroll 1
          for (int c0 = 0; c0 < 64; c0 += 16) {
            uint32_t o[16];
            ptx::tmem_ld16(tm_lane + VtCols::O + c0, o);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * s.corr[((c0 & 31) + j) >> 1]);
            ptx::tmem_st16(tm_lane + VtCols::O + c0, o);
          }
          ptx::tmem_wait_st();
        }
      }
      // PV of tile it - 2 must have read this P^T buffer
      // (if this wait gives up the abort flag is raised and the next vote or the epilogue ends the role for all)
      if (it >= 2) ptx::mbar_wait(&s.p_free[buf], ((it >> 1) - 1) & 1, &s.abort_flag);
      const uint32_t p_base = ptx::smem_u32(s.p[buf][r >> 5]) + p_off;
      uint32_t p_row[8];  // row n of the panel: base + 128 n + the swizzled chunk, which depends on n % 8 only
#pragma unroll
      for (int c = 0; c < 8; ++c) p_row[c] = p_base + ((p_chunk ^ uint32_t(c)) << 4);
#pragma unroll
      for (int h = 0; h < N; ++h) {
        const float pv = ptx::ex2(x[h] - m[h]);  // x = -inf gives 0
        lsum[h] += pv;
        const uint32_t w = ptx::f32x2_to_f16x2(pv, 0.f);  // (p, 0): the even channel of the pair
        ptx::sts32(p_row[(2 * h) & 7] + (2 * h) * 128, w);
        ptx::sts32(p_row[(2 * h + 1) & 7] + (2 * h + 1) * 128, w << 16);
      }
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before_sync();
      __syncwarp();
      ptx::mbar_arrive_if(&s.p_full[buf], lane == 0);
    }

    // ---- segment epilogue: wait for the last PV, reduce the denominators, write the normalised partial
    const bool ok = ptx::mbar_wait(&s.p_free[(it - 1) & 1], ((it - 1) >> 1) & 1, &s.abort_flag);  // PV of the last tile
    if (ptx::bar_red_or(1, 128, !ok)) return;
    ptx::tc_fence_after_sync();
#pragma unroll
    for (int h = 0; h < N; ++h) {
      float v = lsum[h];
#pragma unroll
      for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(~0u, v, o);
      lsum[h] = v;
    }
    if (lane == 0) {
#pragma unroll
      for (int h = 0; h < N; ++h) s.red[warp][h] = lsum[h];
    }
    ptx::bar_sync(1, 128);
    float inv[N];
#pragma unroll
    for (int h = 0; h < N; ++h) {
      const float l = (s.red[0][h] + s.red[1][h]) + (s.red[2][h] + s.red[3][h]);
      inv[h] = l > 0.f ? __fdividef(P.ckv_scale, l) : 0.f;  // (2 ulp; the IEEE division is twenty instructions, sixteen times)
      lsum[h] = l;
    }
    const long long slot = (long long)seg.cta + seg.w;
    float* obase = P.o_part + slot * N * CKV;
#pragma unroll 1
    for (int mb = 0; mb < 2; ++mb) {
      uint32_t o[32];
      ptx::tmem_ld32(tm_lane + VtCols::o(mb), o);
      ptx::tmem_wait_ld();
      const int ch = 2 * (128 * mb + r);  // lane r of block mb holds channels 2 (128 mb + r) and the next one
#pragma unroll
      for (int h = 0; h < N; ++h)
        *reinterpret_cast<float2*>(obase + (long long)h * CKV + ch) =
            make_float2(__uint_as_float(o[2 * h]) * inv[h], __uint_as_float(o[2 * h + 1]) * inv[h]);
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
enum VtRole { kVtSoftmax, kVtK, kVtV, kVtQk, kVtProducer, kVtPv, kVtIdle };

template <int ROLE>
__device__ __forceinline__ void vt_run_role(VtSmem& s, const DecodeParams& P, const CUtensorMap* ckv_map, const CUtensorMap* sf_map,
                                            const CUtensorMap* kpe_map) {
  const int2 range = P.cta_range[blockIdx.x];
  uint32_t it = 0, seg_count = 0;  // every role advances its own copies identically
  for (int w0 = range.x; w0 < range.y; w0 += kSegBatch) {
    const int n_segs = range.y - w0 < kSegBatch ? range.y - w0 : kSegBatch;
    if (ROLE == kVtSoftmax && int(threadIdx.x) < n_segs) {
      Seg g = P.segs[(long long)blockIdx.x + w0 + threadIdx.x];
      if (g.cta != int(blockIdx.x) || g.w != w0 + int(threadIdx.x)) g.ntiles = 0;  // empty item or foreign slot
      s.segs[threadIdx.x] = g;
    }
    __syncthreads();
    if (ROLE == kVtSoftmax) vt_softmax_role(s, P, n_segs, it, seg_count);
    if (ROLE == kVtK) vt_k_role(s, P, n_segs, it, seg_count);
    if (ROLE == kVtV) vt_v_role(s, P, n_segs, it, (uint32_t(threadIdx.x) >> 7) - 2);
    if (ROLE == kVtQk) vt_qk_role(s, P, n_segs, it);
    if (ROLE == kVtProducer) vt_producer_role(s, P, ckv_map, sf_map, kpe_map, n_segs, it);
    if (ROLE == kVtPv) vt_pv_role(s, P, n_segs, it);
    __syncthreads();
    if (s.abort_flag) break;
  }
}

__global__ void __launch_bounds__(kVtThreads, 1)
mla_decode_vt_kernel(const __grid_constant__ CUtensorMap ckv_map, const __grid_constant__ CUtensorMap sf_map,
                     const __grid_constant__ CUtensorMap kpe_map, const DecodeParams P) {
  extern __shared__ uint8_t smem_raw[];
  VtSmem& s = *reinterpret_cast<VtSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kVtRawSlots; ++i) ptx::mbar_init(&s.raw_full[i], 1), ptx::mbar_init(&s.raw_empty[i], 13);  // 4 K + 8 V warps + QK^T
    for (int i = 0; i < 2; ++i) ptx::mbar_init(&s.vt_full[i], 4), ptx::mbar_init(&s.vt_free[i], 1);
    for (int i = 0; i < kVtScRing; ++i) ptx::mbar_init(&s.sc_full[i], 4), ptx::mbar_init(&s.sc_free[i], 8);
    ptx::mbar_init(&s.rope_free, 1);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&s.k_full[i], 4), ptx::mbar_init(&s.k_free[i], 1);
      ptx::mbar_init(&s.s_full[i], 1), ptx::mbar_init(&s.s_free[i], 4);
      ptx::mbar_init(&s.p_full[i], 4), ptx::mbar_init(&s.p_free[i], 1);
    }
    s.abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&ckv_map), ptx::prefetch_tensormap(&sf_map), ptx::prefetch_tensormap(&kpe_map);
  }
  if (warp == 16) {
    ptx::tmem_alloc(&s.tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  ptx::grid_dependency_wait();  // whatever precedes the call in the stream (the lengths' producer, the schedule kernel, the
                                // previous call's use of the workspace) is settled
  ptx::grid_launch_dependents();
  if (P.inline_sched) publish_own_schedule<kVtThreads>(reinterpret_cast<int*>(s.raw[0]), P, blockIdx.x);  // raw[0] is free until the first load

  // Register budgets per warp group (setmaxnreg); the pool is the launch allocation, 20 warps x 96, and the V warps keep
  // what they were launched with.
  constexpr int kSoftmaxRegs = 128, kKRegs = 112, kVRegs = 96, kMiscRegs = 48;
  static_assert(4 * kSoftmaxRegs + 4 * kKRegs + 8 * kVRegs + 4 * kMiscRegs <= 20 * 96, "register budgets exceed the CTA's allocation");
  if (warp < 4) {
    ptx::reg_alloc<kSoftmaxRegs>();
    vt_run_role<kVtSoftmax>(s, P, &ckv_map, &sf_map, &kpe_map);
  } else if (warp < 8) {
    ptx::reg_alloc<kKRegs>();
    vt_run_role<kVtK>(s, P, &ckv_map, &sf_map, &kpe_map);
  } else if (warp < 16) {
    vt_run_role<kVtV>(s, P, &ckv_map, &sf_map, &kpe_map);
  } else {
    ptx::reg_dealloc<kMiscRegs>();
    if (warp == 16) vt_run_role<kVtQk>(s, P, &ckv_map, &sf_map, &kpe_map);
    else if (warp == 17) vt_run_role<kVtProducer>(s, P, &ckv_map, &sf_map, &kpe_map);
    else if (warp == 18) vt_run_role<kVtPv>(s, P, &ckv_map, &sf_map, &kpe_map);
    else vt_run_role<kVtIdle>(s, P, &ckv_map, &sf_map, &kpe_map);
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 16) ptx::tmem_dealloc(s.tmem_base, kTmemCols);
  if (threadIdx.x == 0 && s.abort_flag) atomicExch(P.header, int(kWaitTimeout));
}

}  // namespace mla
