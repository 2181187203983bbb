// Weight-absorbed MLA decode, 16-bit mode, 16 heads per CTA: both MMAs take their A operand from TENSOR MEMORY.
//
//   HBM --TMA--> raw ring (smem) --K warps--> K  as FP16 in tensor memory, lanes = tokens        --QK^T--> S^T (TMEM)
//                               \--V warps--> V^T as FP16 in tensor memory, lanes = channel pairs --PV----> O^T (TMEM)
//
// No 16-bit copy of the tile ever touches shared memory: the packed bytes are dequantised twice, once per layout.
//   QK^T : S^T[token, head] = K[token, 576] . Q^T        A = K (lane = token, column j = channels 2j, 2j + 1),
//          B = Q^T from smem, rope rows of Q pre-multiplied by kpe_scale / ckv_scale so one accumulator holds the score
//   PV   : a byte of the cache holds one token's channels 2c and 2c + 1, and the conversion instruction turns it
//          into the FP16 pair (V[t, 2c], V[t, 2c + 1]). That pair is stored as ONE 32-bit column entry of lane c, i.e.
//          the contraction index is k = 2 t + parity, and the parity is sorted out on the B side:
//              O^T[c, 2h + e] = sum_{t, par} A[c, 2t + par] . B[2t + par, 2h + e],   B[2t + par, 2h + e] = P[t, h] (par == e)
//          so N = 32 (head, channel parity), M = 128 channel pairs per block (two blocks), and no value is ever
//          shuffled between registers: thread data from a transposing 8-bit ldmatrix goes straight through
//          convert-multiply into a 16-lane tcgen05.st. The softmax threads write P twice (as (p, 0) and (0, p)).
//   Tokens inside a 32-token group are stored in the column order the ldmatrix / tcgen05.st fragments give
//   (column 16 tg + 4 (t % 4) + (t % 16) / 4 for token 16 tg + t % 16); P^T uses the same order, and a contraction
//   does not care about the order of its index.
//
// Tensor memory (512 columns): K 288 | V^T ring 4 x 32 | S^T 2 x 16 | O^T 2 x 32.
//   K is single-buffered and released per chunk (rope, then four pairs of 64-channel panels), so the conversion of
//   the next tile follows QK^T of this one chunk by chunk. V^T is a ring of four slots of 32 tokens x 128 channel
//   pairs; a tile is eight slots. PV of tile j needs P(j), which exists about a tile after K(j) was converted, so the V
//   warps run about one tile behind the K warps; the raw ring (six slots of 64 tokens) holds the bytes meanwhile.
// The block scales as FP16 pairs (s, s) are computed once per tile by the K warps, which also park them in shared
// memory ([block][token], two tiles) for the V warps; rows beyond the request's end get scale 0 there, so V is 0 and
// finite wherever P is 0.
//
// Warp roles (512 threads): 0-3 softmax + epilogue, 4-7 K conversion (thread = token), 8-11 V^T conversion
// (warp % 4 = lane quadrant = 32 channel pairs of each block), 12 QK^T issue, 13 TMA producer, 14 PV issue.
// Every wait is bounded; a wait that gives up raises the CTA's abort flag and the kernel reports kWaitTimeout.
#pragma once
#include "mla_decode_sm100.cuh"

namespace mla {

constexpr int kVtRawSlots = 6;
constexpr int kVtRing = 4;

struct VtCols {
  static constexpr uint32_t K = 0, KROPE = 256, VT = 288, S = 416, O = 448;
  __host__ __device__ static constexpr uint32_t s(uint32_t buf) { return S + 16 * buf; }
  __host__ __device__ static constexpr uint32_t vt(uint32_t ring) { return VT + 32 * ring; }
  __host__ __device__ static constexpr uint32_t o(uint32_t mb) { return O + 32 * mb; }
  static_assert(O + 64 <= kTmemCols, "tensor memory overflow");
};

struct VtSmem {
  alignas(1024) uint8_t q[9][16 * 128];         // Q^T: 8 latent panels + rope, K-major, 128-byte swizzle
  alignas(1024) uint8_t p[2][4][32 * 128];      // P^T: [buffer][32-token group][row 2h + parity], 128-byte swizzle
  alignas(1024) uint8_t raw[kVtRawSlots][kRawSlotBytes];
  alignas(16) uint32_t sc[2][32][TILE];         // block scales as FP16 pairs (s, s): [tile parity][block][token]
  Seg segs[kSegBatch];
  float qa[4][16];                              // per-head score scale, ring indexed by segment count
  float red[4][16];
  float corr[16];
  alignas(8) uint64_t raw_full[kVtRawSlots];
  uint64_t raw_empty[kVtRawSlots];
  uint64_t k_full[5], k_free[5];                // K chunk written / read by QK^T: rope, panels {0,1}, {2,3}, {4,5}, {6,7}
  uint64_t s_full[2], s_free[2];
  uint64_t p_full[2], p_free[2];
  uint64_t vt_full[kVtRing], vt_free[kVtRing];
  uint64_t sc_full[2], sc_free[2];
  uint32_t tmem_base;
  int abort_flag;
};
constexpr size_t vt_smem_bytes() { return sizeof(VtSmem) + 1024; }

// ---------------------------------------------------------------------------------------------------------------
// role: K conversion (4 warps; thread = token row of the tile = tensor-memory lane)
// ---------------------------------------------------------------------------------------------------------------
// The query of a segment: 16 rows x (512 + 64) BF16, rope part times kpe_scale / ckv_scale, each row scaled by a power
// of two so that its largest magnitude lies in [2^14, 2^15), converted to FP16 and stored K-major with the 128-byte
// swizzle. Eight consecutive threads share a row, so the row maximum is three shuffles away.
__device__ __forceinline__ void vt_load_query(VtSmem& s, const DecodeParams& P, const Seg& seg, int kt, int par) {
  const int n = kt >> 3, sub = kt & 7;
  const long long row = (long long)seg.b * P.heads + (long long)seg.hg * 16 + n;
  uint4 qn[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) qn[k] = reinterpret_cast<const uint4*>(P.q_nope + row * CKV)[sub + 8 * k];
  const uint4 qp = reinterpret_cast<const uint4*>(P.q_pe + row * KPE)[sub];
  const float ratio = P.kpe_scale / P.ckv_scale;
  auto finite = [](uint32_t bits) { return bits < 0x7F800000u ? bits : 0u; };  // inf / nan do not set the scale
  uint32_t m = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t w[4] = {qn[k].x, qn[k].y, qn[k].z, qn[k].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) m = max(m, max(finite((w[j] << 16) & 0x7FFFFFFFu), finite(w[j] & 0x7FFF0000u)));
  }
  float pe[8];
  {
    const uint32_t w[4] = {qp.x, qp.y, qp.z, qp.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      pe[2 * j] = __uint_as_float(w[j] << 16) * ratio, pe[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u) * ratio;
      m = max(m, max(finite(__float_as_uint(pe[2 * j]) & 0x7FFFFFFFu), finite(__float_as_uint(pe[2 * j + 1]) & 0x7FFFFFFFu)));
    }
  }
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) m = max(m, __shfl_xor_sync(~0u, m, o));
  int e = int(m >> 23) - 127;  // floor(log2(amax)); -127 for 0 / subnormal rows
  e = e < -100 ? -100 : e;
  const float up = __uint_as_float(uint32_t(14 - e + 127) << 23);  // 2^(14 - e), exact
  const uint32_t swz = uint32_t(sub ^ (n & 7)) << 4;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t w[4] = {qn[k].x, qn[k].y, qn[k].z, qn[k].w};
    uint32_t h[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = ptx::f32x2_to_f16x2(__uint_as_float(w[j] << 16) * up, __uint_as_float(w[j] & 0xFFFF0000u) * up);
    *reinterpret_cast<uint4*>(s.q[k] + n * 128 + swz) = make_uint4(h[0], h[1], h[2], h[3]);
  }
  {
    uint32_t h[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = ptx::f32x2_to_f16x2(pe[2 * j] * up, pe[2 * j + 1] * up);
    *reinterpret_cast<uint4*>(s.q[8] + n * 128 + swz) = make_uint4(h[0], h[1], h[2], h[3]);
  }
  if (sub == 0) s.qa[par][n] = P.sm_scale_log2 * P.ckv_scale * __uint_as_float(uint32_t(e - 14 + 127) << 23);
  ptx::fence_proxy_async_smem();
}

// One tile of a K thread. Returns false if a wait gave up.
__device__ __forceinline__ bool vt_k_step(VtSmem& s, const DecodeParams& P, const Seg& seg, int t, uint32_t it, int lane, int quad) {
  const int r = quad * 32 + lane;
  const int half = quad >> 1, rr = r & 63;
  const uint32_t tm_lane = s.tmem_base + (uint32_t(quad * 32) << 16);
  const uint32_t hidx = 2 * it + half;
  const int slot = hidx % kVtRawSlots;
  const uint8_t* raw = s.raw[slot];
  const uint32_t kpar = it & 1;        // phase of the per-tile barriers completed by tile `it`
  const uint32_t buf = it & 1;         // scale table of this tile
  if (!__all_sync(~0u, ptx::mbar_wait(&s.raw_full[slot], (hidx / kVtRawSlots) & 1, &s.abort_flag))) return false;
  const bool valid = seg.tok0 + t * TILE + r < seg.tok_end;

  // ---- block scales: 32 E4M3 bytes -> 32 FP16 pairs (s, s); 0 for rows beyond the end of the request
  uint32_t sc[32];
  {
    const uint32_t x = (rr >> 2) & P.sf_swz_mask;
    const uint4 a = *reinterpret_cast<const uint4*>(raw + kRawSf + rr * 32 + ((0u ^ x) << 4));
    const uint4 b = *reinterpret_cast<const uint4*>(raw + kRawSf + rr * 32 + ((1u ^ x) << 4));
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t s01 = ptx::e4m3x2_to_f16x2(uint16_t(w[j] & 0xFFFF)), s23 = ptx::e4m3x2_to_f16x2(uint16_t(w[j] >> 16));
      sc[4 * j] = __byte_perm(s01, s01, 0x1010), sc[4 * j + 1] = __byte_perm(s01, s01, 0x3232);
      sc[4 * j + 2] = __byte_perm(s23, s23, 0x1010), sc[4 * j + 3] = __byte_perm(s23, s23, 0x3232);
    }
    if (!valid) {
#pragma unroll
      for (int j = 0; j < 32; ++j) sc[j] = 0u;
    }
  }
  auto publish = [&](int chunk) {
    ptx::tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(&s.k_full[chunk]);
  };
  // QK^T of the previous tile must have finished with the chunk's columns
  auto acquire = [&](int chunk) -> bool {
    const bool ok = ptx::mbar_wait(&s.k_free[chunk], kpar ^ 1, &s.abort_flag);
    ptx::tc_fence_after_sync();
    return __all_sync(~0u, ok);
  };

  // ---- rope chunk: 64 E4M3 bytes -> 32 columns
  {
    const uint32_t x = (rr >> 1) & P.kpe_swz_mask;
    uint32_t h[32];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 v = *reinterpret_cast<const uint4*>(raw + kRawKpe + rr * 64 + ((uint32_t(c) ^ x) << 4));
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        h[8 * c + 2 * j] = ptx::e4m3x2_to_f16x2(uint16_t(w[j] & 0xFFFF));
        h[8 * c + 2 * j + 1] = ptx::e4m3x2_to_f16x2(uint16_t(w[j] >> 16));
      }
    }
    if (!acquire(0)) return false;
    ptx::tmem_st32(tm_lane + VtCols::KROPE, h);
  }
  // ---- latent panels: 64 channels = 32 packed bytes -> 32 columns each. The publish of a chunk is deferred until the
  // next panel's values have been computed, so the latency of the tensor-memory store hides behind arithmetic.
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    const uint8_t* base = raw + (p >> 2) * kRawCkvHi + rr * 128;
    const uint32_t c0 = uint32_t(2 * (p & 3)), x = uint32_t(rr & 7);
    const uint4 n0 = *reinterpret_cast<const uint4*>(base + ((c0 ^ x) << 4));
    const uint4 n1 = *reinterpret_cast<const uint4*>(base + (((c0 + 1) ^ x) << 4));
    if (p == 7) {  // last read of the raw slot by this thread
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&s.raw_empty[slot]);
    }
    const uint32_t wds[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
    uint32_t h[32];
#pragma unroll
    for (int j = 0; j < 8; ++j) {  // word j = channels [8j, 8j + 8) of the panel, scale block 4p + j / 2
      uint32_t e[4];
      ptx::e2m1x8_to_f16x8(wds[j], e);
#pragma unroll
      for (int i = 0; i < 4; ++i) h[4 * j + i] = ptx::hmul2(e[i], sc[4 * p + (j >> 1)]);
    }
    if ((p & 1) == 0 && !acquire(1 + (p >> 1))) return false;
    ptx::tmem_wait_st();
    if (p == 0) publish(0);
    else if ((p & 1) == 0) publish(p >> 1);
    ptx::tmem_st32(tm_lane + VtCols::K + 32 * p, h);
    if (p == 1) {
      // park the scales for the V warps, once they have finished with the tile that used this table before
      if (!__all_sync(~0u, ptx::mbar_wait(&s.sc_free[buf], ((it >> 1) & 1) ^ 1, &s.abort_flag))) return false;
#pragma unroll
      for (int b = 0; b < 32; ++b) s.sc[buf][b][r] = sc[b];
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&s.sc_full[buf]);
    }
  }
  ptx::tmem_wait_st();
  publish(4);
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
    // the previous tile's QK^T must be done reading Q^T before the new query overwrites it
    const bool ok = !dead && ptx::mbar_wait(&s.k_free[4], (it & 1) ^ 1, &s.abort_flag);
    if (ptx::bar_red_or(2, 128, !ok)) return;
    vt_load_query(s, P, seg, quad * 32 + lane, seg_count & 3);
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
__device__ __forceinline__ void vt_v_role(VtSmem& s, const DecodeParams& P, int n_segs, uint32_t& it) {
  const int lane = ptx::lane_id();
  const int quad = (threadIdx.x >> 5) & 3;
  const int q = lane & 3;
  const int mrow = lane & 15, mat = lane >> 4;  // this lane addresses row `mrow` of ldmatrix matrix `mat`
  const uint32_t tm = s.tmem_base;
  for (int si = 0; si < n_segs; ++si) {
    const int ntiles = s.segs[si].ntiles;
    for (int t = 0; t < ntiles; ++t, ++it) {
      const uint32_t buf = it & 1;
      if (!__all_sync(~0u, ptx::mbar_wait(&s.sc_full[buf], (it >> 1) & 1, &s.abort_flag))) return;
#pragma unroll 1
      for (int qt = 0; qt < 4; ++qt) {   // 32-token group of the tile
        const uint32_t hidx = 2 * it + (qt >> 1);
        const int slot = hidx % kVtRawSlots;
        if (!__all_sync(~0u, ptx::mbar_wait(&s.raw_full[slot], (hidx / kVtRawSlots) & 1, &s.abort_flag))) return;
        const int rr = 32 * (qt & 1) + 16 * mat + mrow;  // token row inside the 64-token raw slot
        const uint32_t row_addr = ptx::smem_u32(s.raw[slot]) + rr * 128;
#pragma unroll
        for (int mb = 0; mb < 2; ++mb) {  // block of 128 channel pairs = 128-byte half of the packed row
          const uint32_t vs = 8 * it + 2 * qt + mb, ring = vs % kVtRing;
          const bool ok = ptx::mbar_wait(&s.vt_free[ring], ((vs / kVtRing) & 1) ^ 1, &s.abort_flag);
          ptx::tc_fence_after_sync();
          if (!__all_sync(~0u, ok)) return;
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {  // 16 channel pairs = two scale blocks
            const uint32_t chunk = 2 * quad + ch;
            uint32_t rw[4];
            ptx::ldmatrix_x2_trans_b8(row_addr + mb * kRawCkvHi + ((chunk ^ uint32_t(rr & 7)) << 4), rw);
            const uint32_t b0 = 16 * mb + 2 * chunk;
            const uint4 sa0 = *reinterpret_cast<const uint4*>(&s.sc[buf][b0][32 * qt + 4 * q]);
            const uint4 sb0 = *reinterpret_cast<const uint4*>(&s.sc[buf][b0 + 1][32 * qt + 4 * q]);
            const uint4 sa1 = *reinterpret_cast<const uint4*>(&s.sc[buf][b0][32 * qt + 16 + 4 * q]);
            const uint4 sb1 = *reinterpret_cast<const uint4*>(&s.sc[buf][b0 + 1][32 * qt + 16 + 4 * q]);
            const uint32_t sa[8] = {sa0.x, sa0.y, sa0.z, sa0.w, sa1.x, sa1.y, sa1.z, sa1.w};
            const uint32_t sb[8] = {sb0.x, sb0.y, sb0.z, sb0.w, sb1.x, sb1.y, sb1.z, sb1.w};
            uint32_t v[16];
#pragma unroll
            for (int tg = 0; tg < 2; ++tg) {
              uint32_t ea[4], eb[4];
              ptx::e2m1x8_to_f16x8(rw[2 * tg], ea);      // channel pair g, tokens 16 tg + 4q + i
              ptx::e2m1x8_to_f16x8(rw[2 * tg + 1], eb);  // channel pair g + 8
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                v[8 * tg + 2 * i] = ptx::hmul2(ea[i], sa[4 * tg + i]);
                v[8 * tg + 2 * i + 1] = ptx::hmul2(eb[i], sb[4 * tg + i]);
              }
            }
            ptx::tmem_st_16x128b_x8(tm + (uint32_t(32 * quad + 16 * ch) << 16) + VtCols::vt(ring), v);
          }
          ptx::tmem_wait_st();
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&s.vt_full[ring]);
        }
        if (qt & 1) {  // both 32-token groups of the raw slot have been read
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&s.raw_empty[slot]);
        }
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&s.sc_free[buf]);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// roles: MMA issue. The whole warp runs the loop so that every operand is warp-uniform; one elected lane issues.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void vt_qk_role(VtSmem& s, const DecodeParams& P, int n_segs, uint32_t& it) {
  const bool leader = ptx::elect_one();
  const uint32_t tm = s.tmem_base;
  const uint32_t idesc = ptx::instr_desc(128, 16, ptx::FMT_F16, ptx::FMT_F16, false, false);
  const uint64_t q_desc = ptx::smem_desc_sw128(ptx::smem_u32(s.q[0]), 16, 1024);
  for (int si = 0; si < n_segs; ++si) {
    const int ntiles = s.segs[si].ntiles;
    for (int t = 0; t < ntiles; ++t, ++it) {
      const uint32_t buf = it & 1;
      // softmax of tile it - 2 must have read this S^T buffer
      if (!__all_sync(~0u, it < 2 || ptx::mbar_wait(&s.s_free[buf], ((it >> 1) - 1) & 1, &s.abort_flag))) return;
#pragma unroll 1
      for (int c = 0; c < 5; ++c) {
        if (!__all_sync(~0u, ptx::mbar_wait(&s.k_full[c], it & 1, &s.abort_flag))) return;
        ptx::tc_fence_after_sync();
        if (leader) {
          if (c == 0) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              ptx::mma_f16_ts(tm + VtCols::s(buf), tm + VtCols::KROPE + 8 * ks, q_desc + ((8 * 16 * 128 + ks * 32) >> 4), idesc, ks > 0);
          } else {
#pragma unroll 1
            for (int p = 2 * (c - 1); p < 2 * c; ++p) {
#pragma unroll
              for (int ks = 0; ks < 4; ++ks)
                ptx::mma_f16_ts(tm + VtCols::s(buf), tm + VtCols::K + 32 * p + 8 * ks, q_desc + ((p * 16 * 128 + ks * 32) >> 4), idesc, 1);
            }
          }
          ptx::mma_commit(&s.k_free[c]);
          if (c == 4) ptx::mma_commit(&s.s_full[buf]);
        }
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
      for (int sl = 0; sl < 8; ++sl) {  // slot = (32-token group sl / 2, channel-pair block sl % 2)
        const uint32_t vs = 8 * it + sl, ring = vs % kVtRing;
        if (!__all_sync(~0u, ptx::mbar_wait(&s.vt_full[ring], (vs / kVtRing) & 1, &s.abort_flag))) return;
        ptx::tc_fence_after_sync();
        if (leader) {
          const uint64_t p_desc = ptx::smem_desc_sw128(ptx::smem_u32(s.p[buf][sl >> 1]), 16, 1024);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            ptx::mma_f16_ts(tm + VtCols::o(sl & 1), tm + VtCols::vt(ring) + 8 * ks, p_desc + ((ks * 32) >> 4), idesc,
                            (t | (sl >> 1) | ks) != 0);
          ptx::mma_commit(&s.vt_free[ring]);
          if (sl == 7) ptx::mma_commit(&s.p_free[buf]);
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
    float m[N], lsum[N];
#pragma unroll
    for (int h = 0; h < N; ++h) m[h] = -INFINITY, lsum[h] = 0.f;
    bool scales_loaded = false;
    float qa_r[N];

    for (int t = 0; t < seg.ntiles; ++t, ++it) {
      const uint32_t buf = it & 1;
      const bool ok = ptx::mbar_wait(&s.s_full[buf], (it >> 1) & 1, &s.abort_flag);
      ptx::tc_fence_after_sync();
      float x[N];
      if (!scales_loaded) {  // written by the K warps before the segment's first K chunk was published
#pragma unroll
        for (int h = 0; h < N; ++h) qa_r[h] = s.qa[par_q][h];
        scales_loaded = true;
      }
      if (ok) {
        const bool valid = seg.tok0 + t * TILE + r < seg.tok_end;
        uint32_t sv[16];
        ptx::tmem_ld16(tm_lane + VtCols::s(buf), sv);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int h = 0; h < N; ++h) x[h] = valid ? __uint_as_float(sv[h]) * qa_r[h] : -INFINITY;
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
          const float c = (m[h] == -INFINITY) ? 0.f : ptx::ex2(m[h] - mn);  // mn = -inf only if m = -inf
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
      uint8_t* const p_base = s.p[buf][r >> 5] + p_off;
#pragma unroll
      for (int h = 0; h < N; ++h) {
        const float pv = ptx::ex2(x[h] - (m[h] == -INFINITY ? 0.f : m[h]));  // x = -inf gives 0
        lsum[h] += pv;
        const uint32_t w = ptx::f32x2_to_f16x2(pv, 0.f);  // (p, 0): the even channel of the pair
        *reinterpret_cast<uint32_t*>(p_base + (2 * h) * 128 + ((p_chunk ^ uint32_t((2 * h) & 7)) << 4)) = w;
        *reinterpret_cast<uint32_t*>(p_base + (2 * h + 1) * 128 + ((p_chunk ^ uint32_t((2 * h + 1) & 7)) << 4)) = w << 16;
      }
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&s.p_full[buf]);
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
      inv[h] = l > 0.f ? P.ckv_scale / l : 0.f;
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
  uint32_t it = 0, seg_count = 0, hcount = 0;  // every role advances its own copies identically
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
    if (ROLE == kVtV) vt_v_role(s, P, n_segs, it);
    if (ROLE == kVtQk) vt_qk_role(s, P, n_segs, it);
    if (ROLE == kVtProducer) producer_role<kVtRawSlots>(s, P, ckv_map, sf_map, kpe_map, n_segs, hcount);
    if (ROLE == kVtPv) vt_pv_role(s, P, n_segs, it);
    __syncthreads();
    if (s.abort_flag) break;
  }
}

__global__ void __launch_bounds__(kDecodeThreads, 1)
mla_decode_vt_kernel(const __grid_constant__ CUtensorMap ckv_map, const __grid_constant__ CUtensorMap sf_map,
                     const __grid_constant__ CUtensorMap kpe_map, const DecodeParams P) {
  extern __shared__ uint8_t smem_raw[];
  VtSmem& s = *reinterpret_cast<VtSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kVtRawSlots; ++i) ptx::mbar_init(&s.raw_full[i], 1), ptx::mbar_init(&s.raw_empty[i], 6);  // 2 K + 4 V warps
    for (int i = 0; i < 5; ++i) ptx::mbar_init(&s.k_full[i], 4), ptx::mbar_init(&s.k_free[i], 1);
    for (int i = 0; i < kVtRing; ++i) ptx::mbar_init(&s.vt_full[i], 4), ptx::mbar_init(&s.vt_free[i], 1);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&s.s_full[i], 1), ptx::mbar_init(&s.s_free[i], 4);
      ptx::mbar_init(&s.p_full[i], 4), ptx::mbar_init(&s.p_free[i], 1);
      ptx::mbar_init(&s.sc_full[i], 4), ptx::mbar_init(&s.sc_free[i], 4);
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
  ptx::grid_dependency_wait();  // the schedule kernel's output (and the previous call's use of the workspace) is settled
  ptx::grid_launch_dependents();

  // Register budgets per warp group (setmaxnreg); the pool is the launch allocation, 16 warps x 128.
  constexpr int kSoftmaxRegs = 168, kKRegs = 152, kVRegs = 128;
  static_assert(4 * kSoftmaxRegs + 4 * kKRegs + 4 * kVRegs + 4 * 64 <= 16 * 128, "register budgets exceed the CTA's allocation");
  if (warp < 4) {
    ptx::reg_alloc<kSoftmaxRegs>();
    vt_run_role<kVtSoftmax>(s, P, &ckv_map, &sf_map, &kpe_map);
  } else if (warp < 8) {
    ptx::reg_alloc<kKRegs>();
    vt_run_role<kVtK>(s, P, &ckv_map, &sf_map, &kpe_map);
  } else if (warp < 12) {
    vt_run_role<kVtV>(s, P, &ckv_map, &sf_map, &kpe_map);
  } else {
    ptx::reg_dealloc<64>();
    if (warp == 12) vt_run_role<kVtQk>(s, P, &ckv_map, &sf_map, &kpe_map);
    else if (warp == 13) vt_run_role<kVtProducer>(s, P, &ckv_map, &sf_map, &kpe_map);
    else if (warp == 14) vt_run_role<kVtPv>(s, P, &ckv_map, &sf_map, &kpe_map);
    else vt_run_role<kVtIdle>(s, P, &ckv_map, &sf_map, &kpe_map);
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 12) ptx::tmem_dealloc(s.tmem_base, kTmemCols);
  if (threadIdx.x == 0 && s.abort_flag) atomicExch(P.header, int(kWaitTimeout));
}

}  // namespace mla
