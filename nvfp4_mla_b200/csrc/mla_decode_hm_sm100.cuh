// Weight-absorbed MLA decode for 128 heads per request, 8-bit mode, with the HEADS as the M dimension of both MMAs.
//
// With 128 heads the query block fills the 128 rows of a tcgen05 MMA, so one conversion of a token serves all of
// them (the tokens-as-M kernel in mla_decode_sm100.cuh converts a token once per 16 or 32 heads):
//
//   HBM --TMA--> raw ring (smem) --convert warps--> K/V tile in smem, E4M3, [token][channel], 128-byte swizzle
//   QK^T : S[head, token]  = Q[head, 576] . K^T     A = Q (E4M3) from TENSOR MEMORY (latent part) / smem (rope part),
//                                                   B = the K/V tile read K-major, N = 64 tokens
//   PV   : O[head, chan]  += P[head, token] . V     A = P (E4M3) from tensor memory, written there by the softmax threads,
//                                                   B = the same K/V tile read MN-major, N = 256 channels, K = 32 tokens
// One dequantised copy of a token in shared memory feeds both MMAs; nothing of K or V passes through tensor memory.
// O for 128 heads x 512 channels would need all 512 tensor-memory columns, so a PAIR of CTAs (a cluster of two) shares
// a request: both compute the full scores, CTA `cg` of the pair accumulates channels [256 cg, 256 cg + 256). The pair
// gets the same segments from the schedule (which is run over pairs) and writes one partial slot, so the combine
// kernel is unchanged. The conversion is shared: CTA `cg` loads and dequantises tokens [32 cg, 32 cg + 32) of every
// 64-token tile, writes them into its own K/V tile and sends the same bytes to its peer's tile with bulk copies through
// distributed shared memory, which count as transaction bytes on the peer's "tile converted" barrier. A tile buffer
// is reused when the PV of both CTAs has finished with it (a relay warp forwards the local completion to the peer).
//
// Tensor memory (512 columns): Q latent 0..127 | S: 128..191 | P buffers: 192..207, 208..223 | O: 256..511.
// One S buffer is enough: the softmax warps read a tile's scores into registers as their first step, so QK^T of tile
// j + 1 waits only for that read (not for PV of any tile, which sits behind later QK^T in the in-order tensor pipe) and
// runs while the softmax of tile j computes. P has two buffers of its own: PV of tile j reads one while the softmax of
// tile j + 1 fills the other.
// Softmax: thread = head (= tensor-memory lane), so the running max, the sum and the O rescale are thread-local; the
// tcgen05.ld/st of a rescale are warp-wide, so a warp rescales when any of its heads needs it.
// Numerics (8-bit mode): Q rows are E4M3 with one scale per row covering both parts (the rope part is pre-multiplied
// by kpe_scale / (8 ckv_scale) so that one accumulator holds the whole score), K/V bytes are
// E4M3((e2m1 x block scale) / 8) exactly as in the tokens-as-M kernel, P is E4M3 of 2^(x - m) <= 2^8.
//
// Warp roles (640 threads): 0-7 softmax + query load + epilogue, 8-15 dequantise, 16 QK^T issue, 17 TMA producer,
// 18 PV issue. Every wait is bounded (ptx::mbar_wait) as in the other kernel.
#pragma once
#include "mla_decode_sm100.cuh"

namespace mla {

constexpr int kHmThreads = 640;
constexpr int kHmHeads = 128;      // heads per CTA pair = MMA M
constexpr int kHmTile = HALF;      // tokens per tile = one staging slot
constexpr int kHmRows = kHmTile / 2;  // token rows one CTA of the pair loads and converts per tile
constexpr int kHmKvBufs = 4;
constexpr int kHmPanelBytes = kHmTile * 128;  // one 128-channel panel of the E4M3 K/V tile
// staging slot of kHmRows tokens: ckv low halves | ckv high halves | block scales | rope
constexpr int kHmRawCkvHi = kHmRows * 128, kHmRawSf = 2 * kHmRows * 128, kHmRawKpe = kHmRawSf + kHmRows * 32;
constexpr int kHmRawSlotBytes = kHmRows * TOKEN_BYTES;
constexpr uint32_t kHmPeerBytes = 8 * 2048 + 2 * 2048;  // what the peer sends per tile: 8 latent + 2 rope regions of 2 KB
static_assert(kHmRawSlotBytes % 1024 == 0 && kHmRawSf % 256 == 0 && kHmRawKpe % 512 == 0, "staging slot alignment");

template <int RAW_SLOTS>
struct HmSmem {
  alignas(1024) uint8_t kv[kHmKvBufs][5][kHmPanelBytes];  // panels 0..3: latent channels, panel 4: rope (64 of 128 bytes per row)
  alignas(1024) uint8_t qpe[kHmHeads * 128];              // rope part of Q, E4M3, row = head (64 of 128 bytes used)
  alignas(1024) uint8_t raw[RAW_SLOTS][kHmRawSlotBytes];
  Seg segs[kSegBatch];
  alignas(8) uint64_t raw_full[RAW_SLOTS];
  uint64_t raw_empty[RAW_SLOTS];
  uint64_t kv_full[kHmKvBufs];   // tile converted: 8 local convert warps + kHmPeerBytes from the peer CTA
  uint64_t kv_free[kHmKvBufs];   // PV of the tile (hence its QK^T too) has finished reading the buffer in BOTH CTAs (2 arrivals)
  uint64_t pv_local[kHmKvBufs];  // this CTA's PV of the tile is complete (relay warp forwards it to both kv_free)
  uint64_t s_full;               // QK^T of the tile complete (one phase per tile)
  uint64_t s_free;               // the softmax warps have read the tile's scores (8 arrivals, one phase per tile)
  uint64_t p_full[2];            // P written to tensor memory (8 softmax warps)
  uint64_t pv_done[2];           // PV of the tile complete: O may be rescaled, the P buffer reused
  uint64_t q_full;               // query of the segment in place (8 softmax warps)
  float xch[2][kHmHeads];        // softmax pairs: per-head maxima exchanged between a quadrant's two warps
  float xl[2][kHmHeads];         // softmax pairs: the two halves of a head's softmax sum (segment epilogue)
  uint32_t tmem_base;
  int abort_flag;
};
template <int RAW_SLOTS>
constexpr size_t hm_smem_bytes() { return sizeof(HmSmem<RAW_SLOTS>) + 1024; }

struct HmCols {
  static constexpr uint32_t QN = 0, S = 128, P0 = 192, O = 256;
  __host__ __device__ static constexpr uint32_t p(uint32_t buf) { return P0 + 16 * buf; }
};

// ---------------------------------------------------------------------------------------------------------------
// role: TMA producer: this CTA's kHmRows token rows of every tile
// ---------------------------------------------------------------------------------------------------------------
template <int RAW_SLOTS>
__device__ __forceinline__ void hm_producer_role(HmSmem<RAW_SLOTS>& s, const DecodeParams& P, const CUtensorMap* ckv_map,
                                                 const CUtensorMap* sf_map, const CUtensorMap* kpe_map, int n_segs, uint32_t& it, int cg) {
  const int lane = ptx::lane_id();
  const int ps = 1 << P.page_shift;
  for (int si = 0; si < n_segs; ++si) {
    const Seg seg = s.segs[si];
    if (seg.ntiles <= 0) continue;
    const int* pt = P.page_table + (long long)seg.b * P.pt_stride;
    // page ids of a window of 32 tiles, one per lane and load (see producer_role)
    constexpr int kAhead = 4;  // tiles between a load and its L2 prefetch
    int win0 = 0, win_page = 0;
    auto load_window = [&](int t0) {
      win0 = t0;
      const int tokl = seg.tok0 + (t0 + lane) * kHmTile + kHmRows * cg;
      win_page = tokl < seg.tok_end ? pt[tokl >> P.page_shift] : 0;
    };
    if (ps >= kHmRows) load_window(0);
    const int t_query = 2 * seg.ntiles > 6 ? 2 * seg.ntiles - 6 : 0;  // a few tiles before the end
    for (int t = 0; t < 2 * seg.ntiles; ++t, ++it) {
      if (t == t_query)  // the next segment's query rows (128 x 1152 bytes, contiguous per part) into L2: early enough to
        for (int sj = si + 1; sj < n_segs; ++sj) {  // be there when the softmax warps load them, late enough to still be
          const Seg nx = s.segs[sj];
          if (nx.ntiles <= 0) continue;
          const long long row0 = (long long)nx.b * P.heads + (long long)nx.hg * kHmHeads;
          for (int i = lane; i < kHmHeads * 9; i += 32)
            ptx::prefetch_l2(i < kHmHeads * 8 ? reinterpret_cast<const char*>(P.q_nope + row0 * CKV) + i * 128
                                              : reinterpret_cast<const char*>(P.q_pe + row0 * KPE) + (i - kHmHeads * 8) * 128);
          break;
        }
      const int slot = it % RAW_SLOTS;
      const uint32_t use = it / RAW_SLOTS;
      bool ok = ptx::mbar_wait(&s.raw_empty[slot], (use & 1) ^ 1, &s.abort_flag);
      if (!__all_sync(~0u, ok)) return;
      const int tok = seg.tok0 + t * kHmTile + kHmRows * cg;
      int nvalid = seg.tok_end - tok;
      nvalid = nvalid < 0 ? 0 : (nvalid > kHmRows ? kHmRows : nvalid);
      uint8_t* dst = s.raw[slot];
      uint64_t* bar = &s.raw_full[slot];
      if (nvalid == 0) {
        if (lane == 0) ptx::mbar_arrive(bar);
      } else if (ps >= kHmRows) {
        if (t + kAhead >= win0 + 32) load_window(t);
        const int page = __shfl_sync(~0u, win_page, t - win0);
        const int page2 = __shfl_sync(~0u, win_page, t + kAhead - win0);
        if (lane == 0) {
          // a stale or corrupt id is never dereferenced: boxes beyond the last row of the cache read as zeros (see producer_role)
          const bool bad = uint32_t(page) >= uint32_t(P.num_pages);
          if (bad) atomicExch(P.header, int(kBadPage));
          const int row = bad ? (P.num_pages << P.page_shift) : (page << P.page_shift) + (tok & (ps - 1));
          ptx::mbar_arrive_expect_tx(bar, kHmRows * TOKEN_BYTES);
          ptx::tma_load_2d(dst, ckv_map, 0, row, bar);
          ptx::tma_load_2d(dst + kHmRawCkvHi, ckv_map, 128, row, bar);
          ptx::tma_load_2d(dst + kHmRawSf, sf_map, 0, row, bar);
          ptx::tma_load_2d(dst + kHmRawKpe, kpe_map, 0, row, bar);
          const int tok_pf = tok + kAhead * kHmTile;  // L2 prefetch a few tiles ahead
          if (tok_pf < seg.tok_end && uint32_t(page2) < uint32_t(P.num_pages)) {
            const int row2 = (page2 << P.page_shift) + (tok_pf & (ps - 1));
            ptx::tma_prefetch_l2_2d(ckv_map, 0, row2);
            ptx::tma_prefetch_l2_2d(ckv_map, 128, row2);
            ptx::tma_prefetch_l2_2d(sf_map, 0, row2);
            ptx::tma_prefetch_l2_2d(kpe_map, 0, row2);
          }
        }
      } else {
        // small pages: one box per page that holds a valid token (at most 32 per slot), one lane per page; scales and
        // rope arrive unswizzled
        const int npages = (nvalid + ps - 1) >> P.page_shift;
        int page = lane < npages ? pt[(tok >> P.page_shift) + lane] : -1;
        const bool ok_page = lane < npages && uint32_t(page) < uint32_t(P.num_pages);
        if (lane < npages && !ok_page) atomicExch(P.header, int(kBadPage));
        const uint32_t good = __popc(__ballot_sync(~0u, ok_page));
        if (lane == 0) {
          if (good) ptx::mbar_arrive_expect_tx(bar, good * ps * TOKEN_BYTES);
          else ptx::mbar_arrive(bar);
        }
        __syncwarp();
        if (ok_page) {
          const int row = page << P.page_shift, r0 = lane << P.page_shift;
          ptx::tma_load_2d(dst + r0 * 128, ckv_map, 0, row, bar);
          ptx::tma_load_2d(dst + kHmRawCkvHi + r0 * 128, ckv_map, 128, row, bar);
          ptx::bulk_load(dst + kHmRawSf + r0 * 32, P.sf + (long long)row * 32, ps * 32, bar);
          ptx::bulk_load(dst + kHmRawKpe + r0 * 64, P.kpe + (long long)row * 64, ps * 64, bar);
        }
      }
      __syncwarp();
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// role: dequantise (8 warps) this CTA's 32 token rows of every tile, into its own tile and the peer's. Warp cw: panel
// cw % 4 (128 channels), rows 16 (cw / 4) .. + 15 of the CTA's 32; two threads per row (64 channels each). A warp's
// output is 16 consecutive 128-byte rows of one panel, 2 KB, which one bulk copy forwards to the peer. The warps of
// panel 0 also move their rows' rope bytes.
// ---------------------------------------------------------------------------------------------------------------
template <int RAW_SLOTS>
__device__ __forceinline__ void hm_convert_role(HmSmem<RAW_SLOTS>& s, const DecodeParams& P, int n_segs, uint32_t& it, int cg) {
  const int lane = ptx::lane_id();
  const int cw = (threadIdx.x >> 5) - 8, p = cw & 3, hh = lane & 1;
  const int r = (cw >> 2) * 16 + (lane >> 1);  // row in the staging slot
  const int R = kHmRows * cg + r;              // row in the tile
  const uint32_t swz = uint32_t(r & 7) << 4;   // = (R & 7) << 4
  const uint32_t peer = uint32_t(cg ^ 1);
  for (int si = 0; si < n_segs; ++si) {
    const Seg seg = s.segs[si];
    for (int t = 0; t < 2 * seg.ntiles; ++t, ++it) {
      const int slot = it % RAW_SLOTS, kb = it % kHmKvBufs;
      bool ok = ptx::mbar_wait(&s.raw_full[slot], (it / RAW_SLOTS) & 1, &s.abort_flag);
      if (!__all_sync(~0u, ok)) return;
      const uint8_t* raw = s.raw[slot];
      const bool valid = seg.tok0 + t * kHmTile + R < seg.tok_end;
      const bool full = seg.tok0 + (t + 1) * kHmTile <= seg.tok_end;  // warp-uniform: a live tile skips the masking
      // the 4 block scales of this thread's 64 channels, their 32 packed bytes, and (panel 0) 32 bytes of rope
      const uint32_t sf4 = *reinterpret_cast<const uint32_t*>(raw + kHmRawSf + r * 32 + ((uint32_t(p >> 1) ^ ((r >> 2) & P.sf_swz_mask)) << 4) +
                                                              (p & 1) * 8 + 4 * hh);
      const uint8_t* half_row = raw + (p >> 1) * kHmRawCkvHi + r * 128;
      uint4 w[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) w[i] = *reinterpret_cast<const uint4*>(half_row + ((uint32_t((p & 1) * 4 + 2 * hh + i) << 4) ^ swz));
      uint4 rope[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
      if (p == 0) {
        const uint32_t kswz = (r >> 1) & P.kpe_swz_mask;
#pragma unroll
        for (int i = 0; i < 2; ++i) rope[i] = *reinterpret_cast<const uint4*>(raw + kHmRawKpe + r * 64 + ((uint32_t(2 * hh + i) ^ kswz) << 4));
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&s.raw_empty[slot]);
      // the buffer's previous tile (it - kHmKvBufs) must have been consumed by the PV of both CTAs
      ok = it < kHmKvBufs || ptx::mbar_wait(&s.kv_free[kb], ((it / kHmKvBufs) - 1) & 1, &s.abort_flag);
      if (!__all_sync(~0u, ok)) return;
      uint8_t* out_row = s.kv[kb][p] + R * 128;
      const uint32_t words[8] = {w[0].x, w[0].y, w[0].z, w[0].w, w[1].x, w[1].y, w[1].z, w[1].w};
      const uint32_t vmask = valid ? 0xFFFFFFFFu : 0u;  // rows past the end of the request become zeros
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {  // two 16-byte chunks (= two scale blocks) per trip
        uint32_t s2 = ptx::e4m3x2_to_f16x2(uint16_t(sf4 >> (16 * c2)));  // (scale of chunk 2 c2, of chunk 2 c2 + 1)
        s2 = ptx::hmul2(s2, 0x30003000u);                                  // x 1/8, exact
        const uint32_t sc[2] = {__byte_perm(s2, s2, 0x1010), __byte_perm(s2, s2, 0x3232)};
#pragma unroll
        for (int k = 0; k < 2; ++k) {  // chunk c of this thread = channels [64 hh + 16 c, + 16) of the panel
          const int c = 2 * c2 + k;
          uint32_t o[4];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            uint32_t e[4];
            ptx::e2m1x8_to_f16x8(words[2 * c + j], e);
            o[2 * j] = ptx::f16x4_to_e4m3x4(ptx::hmul2(e[0], sc[k]), ptx::hmul2(e[1], sc[k]));
            o[2 * j + 1] = ptx::f16x4_to_e4m3x4(ptx::hmul2(e[2], sc[k]), ptx::hmul2(e[3], sc[k]));
          }
          if (!full) o[0] &= vmask, o[1] &= vmask, o[2] &= vmask, o[3] &= vmask;
          *reinterpret_cast<uint4*>(out_row + ((uint32_t(4 * hh + c) << 4) ^ swz)) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      if (p == 0) {  // rope bytes are E4M3 already: chunks 2 hh, 2 hh + 1 of the row's 64 bytes
#pragma unroll
        for (int i = 0; i < 2; ++i)
          *reinterpret_cast<uint4*>(s.kv[kb][4] + R * 128 + ((uint32_t(2 * hh + i) << 4) ^ swz)) = valid ? rope[i] : make_uint4(0, 0, 0, 0);
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        // the peer's tile gets the same bytes; they complete on its kv_full as transaction bytes
        const uint8_t* src = s.kv[kb][p] + (kHmRows * cg + (cw >> 2) * 16) * 128;
        const uint32_t peer_bar = ptx::map_to_cta(&s.kv_full[kb], peer);
        ptx::bulk_copy_to_cta(ptx::map_to_cta(src, peer), src, 2048, peer_bar);
        if (p == 0) {
          const uint8_t* rsrc = s.kv[kb][4] + (kHmRows * cg + (cw >> 2) * 16) * 128;
          ptx::bulk_copy_to_cta(ptx::map_to_cta(rsrc, peer), rsrc, 2048, peer_bar);
        }
        if (cw == 0) ptx::mbar_arrive_expect_tx(&s.kv_full[kb], kHmPeerBytes);  // what the peer will send for this tile
        else ptx::mbar_arrive(&s.kv_full[kb]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// role: relay (1 warp): when this CTA's PV of a tile is complete, release the tile buffer in both CTAs
// ---------------------------------------------------------------------------------------------------------------
template <int RAW_SLOTS>
__device__ __forceinline__ void hm_relay_role(HmSmem<RAW_SLOTS>& s, int n_segs, uint32_t& it, int cg) {
  const int lane = ptx::lane_id();
  for (int si = 0; si < n_segs; ++si) {
    const int ntiles = 2 * s.segs[si].ntiles;
    for (int t = 0; t < ntiles; ++t, ++it) {
      const uint32_t kb = it % kHmKvBufs;
      if (!__all_sync(~0u, ptx::mbar_wait(&s.pv_local[kb], (it / kHmKvBufs) & 1, &s.abort_flag))) return;
      if (lane == 0) {
        ptx::mbar_arrive(&s.kv_free[kb]);
        ptx::mbar_arrive_cta(ptx::map_to_cta(&s.kv_free[kb], uint32_t(cg ^ 1)));
      }
      __syncwarp();
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// roles: MMA issue
// ---------------------------------------------------------------------------------------------------------------
template <int RAW_SLOTS>
__device__ __forceinline__ void hm_qk_role(HmSmem<RAW_SLOTS>& s, const DecodeParams& P, int n_segs, uint32_t& it, uint32_t& seg_count) {
  const bool leader = ptx::elect_one();
  const uint32_t tm = s.tmem_base;
  const uint32_t idesc = ptx::instr_desc(kHmHeads, kHmTile, ptx::FMT_E4M3, ptx::FMT_E4M3, false, false);
  const uint64_t qpe_desc = ptx::smem_desc_sw128(ptx::smem_u32(s.qpe), 16, 1024);
  for (int si = 0; si < n_segs; ++si) {
    const int ntiles = 2 * s.segs[si].ntiles;
    if (ntiles <= 0) continue;
    if (!__all_sync(~0u, ptx::mbar_wait(&s.q_full, seg_count & 1, &s.abort_flag))) return;
    ++seg_count;
    for (int t = 0; t < ntiles; ++t, ++it) {
      const uint32_t kb = it % kHmKvBufs;
      // the softmax warps have read the scores of tile it - 1
      if (!__all_sync(~0u, it < 1 || ptx::mbar_wait(&s.s_free, (it - 1) & 1, &s.abort_flag))) return;
      if (!__all_sync(~0u, ptx::mbar_wait(&s.kv_full[kb], (it / kHmKvBufs) & 1, &s.abort_flag))) return;
      ptx::tc_fence_after_sync();
      if (leader) {
        const uint64_t k_desc = ptx::smem_desc_sw128(ptx::smem_u32(s.kv[kb][0]), 16, 1024);
#pragma unroll 1
        for (int p = 0; p < 4; ++p) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)  // 32 channels per MMA: 8 tensor-memory columns of Q, 32 bytes of the K rows
            ptx::mma_f8_ts(tm + HmCols::S, tm + HmCols::QN + 32 * p + 8 * ks, k_desc + ((p * kHmPanelBytes + ks * 32) >> 4), idesc,
                           (p | ks) != 0);
        }
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
          ptx::mma_f8_ss(tm + HmCols::S, qpe_desc + ((ks * 32) >> 4), k_desc + ((4 * kHmPanelBytes + ks * 32) >> 4), idesc, 1);
        ptx::mma_commit(&s.s_full);
      }
      __syncwarp();
    }
  }
}

template <int RAW_SLOTS>
__device__ __forceinline__ void hm_pv_role(HmSmem<RAW_SLOTS>& s, const DecodeParams& P, int n_segs, uint32_t& it, int cg) {
  const bool leader = ptx::elect_one();
  const uint32_t tm = s.tmem_base;
  // B = V read MN-major: N = 256 channels = two 128-byte runs (panels 2 cg, 2 cg + 1, one panel apart), K = 32 token rows
  const uint32_t idesc = ptx::instr_desc(kHmHeads, 256, ptx::FMT_E4M3, ptx::FMT_E4M3, false, true);
  for (int si = 0; si < n_segs; ++si) {
    const int ntiles = 2 * s.segs[si].ntiles;
    for (int t = 0; t < ntiles; ++t, ++it) {
      const uint32_t buf = it & 1, kb = it % kHmKvBufs;
      if (!__all_sync(~0u, ptx::mbar_wait(&s.p_full[buf], (it >> 1) & 1, &s.abort_flag))) return;
      ptx::tc_fence_after_sync();
      if (leader) {
        const uint64_t v_desc = ptx::smem_desc_sw128(ptx::smem_u32(s.kv[kb][2 * cg]), kHmPanelBytes, 1024);
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
          ptx::mma_f8_ts(tm + HmCols::O, tm + HmCols::p(buf) + 8 * ks, v_desc + ((ks * 32 * 128) >> 4), idesc, (t | ks) != 0);
        ptx::mma_commit(&s.pv_done[buf]);
        ptx::mma_commit(&s.pv_local[kb]);
      }
      __syncwarp();
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// role: softmax + query load + epilogue (8 warps). Warp w: tensor-memory quadrant w % 4 (heads 32 (w % 4) .. + 31),
// column half w / 4: the two warps of a quadrant share each head's tile (32 tokens each), its O row (128 columns each)
// and its query row (256 latent channels each; the upper half also takes the rope part). A head's running max must be
// the same in both, so the pair meets at a named barrier once per tile to vote (bar.red.or) and, only when some head
// of the quadrant outgrows its max, a second time to exchange the maxima through shared memory.
// ---------------------------------------------------------------------------------------------------------------
template <int RAW_SLOTS>
__device__ __forceinline__ void hm_softmax_role(HmSmem<RAW_SLOTS>& s, const DecodeParams& P, int n_segs, uint32_t& it, int cg) {
  const int lane = ptx::lane_id(), warp = threadIdx.x >> 5;
  const int quad = warp & 3, half = warp >> 2;
  const int h = quad * 32 + lane;  // head = tensor-memory lane
  const uint32_t tm_lane = s.tmem_base + (uint32_t(quad * 32) << 16);
  const uint32_t pair_bar = 1 + quad;  // named barrier of this quadrant's two warps
  constexpr float kGrow = 8.f;
  for (int si = 0; si < n_segs; ++si) {
    const Seg seg = s.segs[si];
    if (seg.ntiles <= 0) continue;
    // ---- query of (request seg.b, head group seg.hg), this head's row: channels [256 half, +256), rope with half 1.
    // Every MMA that read the previous segment's query has completed (both warps consumed the scores of its last tile).
    const long long row = (long long)seg.b * P.heads + (long long)seg.hg * kHmHeads + h;
    const uint4* qn = reinterpret_cast<const uint4*>(P.q_nope + row * CKV) + 32 * half;
    const uint4* qp = reinterpret_cast<const uint4*>(P.q_pe + row * KPE);
    const float ratio = P.kpe_scale / (8.f * P.ckv_scale);  // rope scores in units of the latent ones
    // This thread's part of the row is four 128-byte lines (+ one of rope): ask for all of them at once, so that the two
    // passes below pay at most one trip to memory instead of one per batch of loads (the producer warp has asked for the
    // rows of every segment but the first a few tiles ahead).
#pragma unroll
    for (int l = 0; l < 4; ++l) ptx::prefetch_l2(reinterpret_cast<const char*>(qn) + 128 * l);
    if (half) ptx::prefetch_l2(qp);
    auto amax8 = [](const uint4& v, float a) {
      const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = fabsf(__uint_as_float(wv[j] << 16)), hi = fabsf(__uint_as_float(wv[j] & 0xFFFF0000u));
        a = fmaxf(a, (lo < INFINITY ? lo : 0.f)), a = fmaxf(a, (hi < INFINITY ? hi : 0.f));  // ignore inf / nan for the scale
      }
      return a;
    };
    // largest magnitude of the row part: packed BF16 maxima (two values per instruction; a NaN operand is dropped by
    // the maximum); the element-wise pass that also ignores infinities runs only if one turned up
    auto amax_fast = [](const uint4* src, int n) {
      __nv_bfloat162 m2 = __float2bfloat162_rn(0.f);
#pragma unroll 1
      for (int c0 = 0; c0 < n; c0 += 8) {  // eight independent 16-byte loads in flight per trip
        uint4 v[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) v[c] = __ldg(src + c0 + c);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint32_t wv[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t a = wv[j] & 0x7FFF7FFFu;
            m2 = __hmax2(m2, *reinterpret_cast<const __nv_bfloat162*>(&a));
          }
        }
      }
      return fmaxf(__low2float(m2), __high2float(m2));
    };
    float a_loc = amax_fast(qn, 32), ap = half ? amax_fast(qp, KPE / 8) : 0.f;
    if (!(a_loc < INFINITY) || !(ap < INFINITY)) {
      a_loc = 0.f, ap = 0.f;
      for (int c = 0; c < 32; ++c) a_loc = amax8(qn[c], a_loc);
      if (half)
        for (int c = 0; c < KPE / 8; ++c) ap = amax8(qp[c], ap);
    }
    a_loc = fmaxf(a_loc, ap * ratio);
    s.xch[half][h] = a_loc;
    ptx::bar_sync(pair_bar, 64);
    const float amax = fmaxf(fmaxf(s.xch[0][h], s.xch[1][h]), 1e-30f);
    const float inv_n = 448.f / amax, inv_p = ratio * inv_n;
    const float qa = P.sm_scale_log2 * P.ckv_scale * 8.f * (amax / 448.f);  // score scale of this head, log2 units
    auto e4m3x8 = [](const uint4& v, float sc, uint32_t& o0, uint32_t& o1) {
      const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
      o0 = ptx::pack_e4m3x4(__uint_as_float(wv[0] << 16) * sc, __uint_as_float(wv[0] & 0xFFFF0000u) * sc,
                            __uint_as_float(wv[1] << 16) * sc, __uint_as_float(wv[1] & 0xFFFF0000u) * sc);
      o1 = ptx::pack_e4m3x4(__uint_as_float(wv[2] << 16) * sc, __uint_as_float(wv[2] & 0xFFFF0000u) * sc,
                            __uint_as_float(wv[3] << 16) * sc, __uint_as_float(wv[3] & 0xFFFF0000u) * sc);
    };
#pragma unroll 1
    for (int c0 = 0; c0 < 32; c0 += 8) {  // 64 channels = 64 bytes = 16 tensor-memory columns per trip
      uint32_t col[16];
      uint4 v[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) v[c] = __ldg(qn + c0 + c);
#pragma unroll
      for (int c = 0; c < 8; ++c) e4m3x8(v[c], inv_n, col[2 * c], col[2 * c + 1]);
      ptx::tmem_st16(tm_lane + HmCols::QN + 64 * half + 2 * c0, col);
    }
    if (half) {
#pragma unroll
      for (int c = 0; c < KPE / 8; c += 2) {  // 16 rope channels = one 16-byte chunk of the head's row in shared memory
        uint32_t o[4];
        e4m3x8(qp[c], inv_p, o[0], o[1]), e4m3x8(qp[c + 1], inv_p, o[2], o[3]);
        *reinterpret_cast<uint4*>(s.qpe + h * 128 + ((uint32_t(c >> 1) << 4) ^ (uint32_t(h & 7) << 4))) = make_uint4(o[0], o[1], o[2], o[3]);
      }
      ptx::fence_proxy_async_smem();
    }
    ptx::tmem_wait_st();
    ptx::tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(&s.q_full);

    float m = -INFINITY, l = 0.f;  // m is identical in the head's two threads; l is this thread's share of the sum
    const int ntiles = 2 * seg.ntiles;
    for (int t = 0; t < ntiles; ++t, ++it) {
      const uint32_t buf = it & 1;
      bool ok = ptx::mbar_wait(&s.s_full, it & 1, &s.abort_flag);
      // PV of tile it - 2 has read its P from the buffer this tile's P will overwrite (long done: it was issued two tiles ago)
      ok = ok && (it < 2 || ptx::mbar_wait(&s.pv_done[buf], ((it >> 1) - 1) & 1, &s.abort_flag));
      ptx::tc_fence_after_sync();
      const int nvalid = seg.tok_end - (seg.tok0 + t * kHmTile) - 32 * half;  // this warp's columns at or beyond it are masked
      // raw scores of this head for this warp's 32 tokens; the score scale qa > 0 is applied inside the exponent
      uint32_t sr[32];
      if (ok) {
        ptx::tmem_ld32(tm_lane + HmCols::S + 32 * half, sr);
        ptx::tmem_wait_ld();
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&s.s_free);  // QK^T of tile it + 1 may overwrite the scores
      if (!ok || nvalid < 32) {  // tail tile: masked tokens get the score -inf
#pragma unroll
        for (int j = 0; j < 32; ++j) sr[j] = (ok && j < nvalid) ? sr[j] : 0xFF800000u;
      }
      float mxs[4] = {__uint_as_float(sr[0]), __uint_as_float(sr[1]), __uint_as_float(sr[2]), __uint_as_float(sr[3])};
#pragma unroll
      for (int j = 4; j + 8 <= 32; j += 8)  // four chains of three-input maxima
#pragma unroll
        for (int k = 0; k < 4; ++k) mxs[k] = ptx::max3(mxs[k], __uint_as_float(sr[j + 2 * k]), __uint_as_float(sr[j + 2 * k + 1]));
#pragma unroll
      for (int k = 0; k < 4; ++k) mxs[k] = fmaxf(mxs[k], __uint_as_float(sr[28 + k]));
      const float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])) * qa;
      if (ptx::bar_red_or(pair_bar, 64, !ok || mx > m + kGrow)) {
        // some head of the quadrant outgrew its max (or a wait gave up): exchange the maxima, decide per head
        s.xch[half][h] = mx;
        if (ptx::bar_red_or(pair_bar, 64, s.abort_flag != 0)) return;  // uniform in the pair, whoever raised the flag
        const float mxp = fmaxf(s.xch[0][h], s.xch[1][h]);
        const bool need = mxp > m + kGrow;
        const float mn = need ? mxp : m;
        const float corr = need ? ((m == -INFINITY) ? 0.f : ptx::ex2(m - mn)) : 1.f;
        l *= corr, m = mn;
        if (t > 0) {  // O holds the segment's earlier tiles: wait for the PV of tile it - 1, then scale this head's half row
          const bool okv = ptx::mbar_wait(&s.pv_done[buf ^ 1], ((it - 1) >> 1) & 1, &s.abort_flag);
          if (ptx::bar_red_or(pair_bar, 64, !okv)) return;
          ptx::tc_fence_after_sync();
#pragma unroll 1
          for (int c0 = 0; c0 < 128; c0 += 32) {
            uint32_t o[32];
            ptx::tmem_ld32(tm_lane + HmCols::O + 128 * half + c0, o);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * corr);
            ptx::tmem_st32(tm_lane + HmCols::O + 128 * half + c0, o);
          }
          ptx::tmem_wait_st();
        }
      }
      // P = 2^(s qa - m) as E4M3 into this warp's 8 of the tile's 16 P columns
      const float neg_m = (m == -INFINITY) ? 0.f : -m;
      uint32_t pk[8];
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float p0 = ptx::ex2(fmaf(__uint_as_float(sr[4 * c]), qa, neg_m)), p1 = ptx::ex2(fmaf(__uint_as_float(sr[4 * c + 1]), qa, neg_m));
        const float p2 = ptx::ex2(fmaf(__uint_as_float(sr[4 * c + 2]), qa, neg_m)), p3 = ptx::ex2(fmaf(__uint_as_float(sr[4 * c + 3]), qa, neg_m));
        ls[0] += p0, ls[1] += p1, ls[2] += p2, ls[3] += p3;
        pk[c] = ptx::pack_e4m3x4(p0, p1, p2, p3);
      }
      l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      ptx::tmem_st8(tm_lane + HmCols::p(buf) + 8 * half, pk);
      ptx::tmem_wait_st();
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&s.p_full[buf]);
    }

    // ---- segment epilogue: wait for the last PV, add the two halves of the sum, write this warp's 128 of the head's
    // 256 channels of the normalised partial
    const bool ok = ptx::mbar_wait(&s.pv_done[(it - 1) & 1], ((it - 1) >> 1) & 1, &s.abort_flag);
    s.xl[half][h] = l;
    if (ptx::bar_red_or(pair_bar, 64, !ok)) return;
    ptx::tc_fence_after_sync();
    const float lt = s.xl[0][h] + s.xl[1][h];
    const float inv = lt > 0.f ? 8.f * P.ckv_scale / lt : 0.f;
    const long long slot = (long long)seg.cta + seg.w;
    float* orow = P.o_part + (slot * kHmHeads + h) * CKV + 256 * cg + 128 * half;
#pragma unroll 1
    for (int c0 = 0; c0 < 128; c0 += 32) {
      uint32_t o[32];
      ptx::tmem_ld32(tm_lane + HmCols::O + 128 * half + c0, o);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(orow + c0 + j) = make_float4(__uint_as_float(o[j]) * inv, __uint_as_float(o[j + 1]) * inv,
                                                                __uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
    }
    if (cg == 0 && half == 0) P.lse_part[slot * kHmHeads + h] = lt > 0.f ? m + log2f(lt) : -INFINITY;
    ptx::tc_fence_before_sync();
    ptx::bar_sync(pair_bar, 64);  // s.xl and s.xch are reused by the next segment
  }
}

// ---------------------------------------------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------------------------------------------
template <int RAW_SLOTS, int ROLE>
__device__ __forceinline__ void hm_run_role(HmSmem<RAW_SLOTS>& s, const DecodeParams& P, const CUtensorMap* ckv_map,
                                            const CUtensorMap* sf_map, const CUtensorMap* kpe_map) {
  const int pair = blockIdx.x >> 1, cg = blockIdx.x & 1;
  const int2 range = P.cta_range[pair];
  uint32_t it = 0, seg_count = 0;  // every role advances its own copies identically
  for (int w0 = range.x; w0 < range.y; w0 += kSegBatch) {
    const int n_segs = range.y - w0 < kSegBatch ? range.y - w0 : kSegBatch;
    if (ROLE == kRoleSoftmax && int(threadIdx.x) < n_segs) {
      Seg g = P.segs[(long long)pair + w0 + threadIdx.x];
      if (g.cta != pair || g.w != w0 + int(threadIdx.x)) g.ntiles = 0;  // empty item or foreign slot
      s.segs[threadIdx.x] = g;
    }
    __syncthreads();
    if (ROLE == kRoleSoftmax) hm_softmax_role<RAW_SLOTS>(s, P, n_segs, it, cg);
    if (ROLE == kRoleConvert) hm_convert_role<RAW_SLOTS>(s, P, n_segs, it, cg);
    if (ROLE == kRoleQk) hm_qk_role<RAW_SLOTS>(s, P, n_segs, it, seg_count);
    if (ROLE == kRoleProducer) hm_producer_role<RAW_SLOTS>(s, P, ckv_map, sf_map, kpe_map, n_segs, it, cg);
    if (ROLE == kRoleIdle) hm_relay_role<RAW_SLOTS>(s, n_segs, it, cg);
    if (ROLE == kRolePv) hm_pv_role<RAW_SLOTS>(s, P, n_segs, it, cg);
    __syncthreads();
    if (s.abort_flag) break;
  }
}

template <int RAW_SLOTS>
__global__ void __launch_bounds__(kHmThreads, 1)
mla_decode_hm_kernel(const __grid_constant__ CUtensorMap ckv_map, const __grid_constant__ CUtensorMap sf_map,
                     const __grid_constant__ CUtensorMap kpe_map, const DecodeParams P) {
  extern __shared__ uint8_t smem_raw[];
  using Smem = HmSmem<RAW_SLOTS>;
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    for (int i = 0; i < RAW_SLOTS; ++i) ptx::mbar_init(&s.raw_full[i], 1), ptx::mbar_init(&s.raw_empty[i], 8);
    for (int i = 0; i < kHmKvBufs; ++i)
      ptx::mbar_init(&s.kv_full[i], 8), ptx::mbar_init(&s.kv_free[i], 2), ptx::mbar_init(&s.pv_local[i], 1);
    ptx::mbar_init(&s.s_full, 1), ptx::mbar_init(&s.s_free, 8);
    for (int i = 0; i < 2; ++i) ptx::mbar_init(&s.p_full[i], 8), ptx::mbar_init(&s.pv_done[i], 1);
    ptx::mbar_init(&s.q_full, 8);
    s.abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&ckv_map), ptx::prefetch_tensormap(&sf_map), ptx::prefetch_tensormap(&kpe_map);
  }
  if (warp == 16) {
    ptx::tmem_alloc(&s.tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  ptx::cluster_sync();  // both CTAs' barriers are initialised before either signals the other's
  ptx::tc_fence_after_sync();
  ptx::grid_dependency_wait();
  ptx::grid_launch_dependents();  // after the wait: the combine kernel reads a schedule kernel's output as soon as it starts
  // the staging buffers are filled by this CTA's own loads only (the peer writes to kv), so the first one is free until then
  if (P.inline_sched) publish_own_schedule<kHmThreads>(reinterpret_cast<int*>(s.raw[0]), P, blockIdx.x >> 1);

  // 640 threads are launched with 96 registers each (65536 / 640 rounded down to a multiple of 8); that allocation is
  // the pool the role budgets must fit in, warp group by warp group (4 warps each): 2 softmax, 2 convert, 1 issue.
  constexpr int kLaunchRegs = 96, kSoftmaxRegs = 104, kConvertRegs = 112, kIssueRegs = 48;
  static_assert(8 * kSoftmaxRegs + 8 * kConvertRegs + 4 * kIssueRegs <= 20 * kLaunchRegs, "register budgets exceed the CTA's allocation");
  if (warp < 8) {
    ptx::reg_alloc<kSoftmaxRegs>();
    hm_run_role<RAW_SLOTS, kRoleSoftmax>(s, P, &ckv_map, &sf_map, &kpe_map);
  } else if (warp < 16) {
    ptx::reg_alloc<kConvertRegs>();
    hm_run_role<RAW_SLOTS, kRoleConvert>(s, P, &ckv_map, &sf_map, &kpe_map);
  } else {
    ptx::reg_dealloc<kIssueRegs>();
    if (warp == 16) hm_run_role<RAW_SLOTS, kRoleQk>(s, P, &ckv_map, &sf_map, &kpe_map);
    else if (warp == 17) hm_run_role<RAW_SLOTS, kRoleProducer>(s, P, &ckv_map, &sf_map, &kpe_map);
    else if (warp == 18) hm_run_role<RAW_SLOTS, kRolePv>(s, P, &ckv_map, &sf_map, &kpe_map);
    else hm_run_role<RAW_SLOTS, kRoleIdle>(s, P, &ckv_map, &sf_map, &kpe_map);
  }

  ptx::tc_fence_before_sync();
  ptx::cluster_sync();  // neither CTA leaves while the other may still write to its shared memory or signal its barriers
  if (warp == 16) ptx::tmem_dealloc(s.tmem_base, kTmemCols);
  if (threadIdx.x == 0 && s.abort_flag) atomicExch(P.header, int(kWaitTimeout));
}

}  // namespace mla
