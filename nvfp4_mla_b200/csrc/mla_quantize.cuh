// Cache writer: quantise new latent-KV rows to NVFP4 / E4M3 and append them to the paged cache.
//
//   per 16 latent channels: sf = e4m3_rn(amax / 6 / ckv_scale) (saturating at 448), stored as the block scale;
//   code = nearest E2M1 (ties to the even mantissa, magnitudes above 6 saturate) of x / (float(sf) * ckv_scale),
//   0 where the scale is 0; two codes per byte, low nibble = even channel;
//   rope: e4m3_rn(kpe / kpe_scale), saturating.
// Every step is defined as one fp32 IEEE operation in that order, so the bytes are reproducible on a CPU bit for bit.
// The 512 divisions per token would make the kernel instruction-bound, so the codes are first computed from
// x * (1 / scale): that product is within 2^-22 (relative) of the correctly rounded quotient, and the code is a
// monotone step function of the magnitude, so if the products shrunk and grown by 2^-21 get the same code, the
// quotient gets it too; a value that sits that close to a rounding boundary is settled on its own: an exact tie (which
// BF16 inputs hit in a few percent of the scale blocks) by one fused multiply-add, anything else by a real division.
//
// HBM-bound: 1152 bytes in, 352 bytes out per token. One warp per token per trip; lane l owns scale block l
// (channels 16l .. 16l+15: two 16-byte loads, one 8-byte store, the warp writes the token's 256 packed bytes as one
// contiguous run) and rope channels 2l, 2l+1.
#pragma once
#include <cuda_bf16.h>
#include "mla_common.cuh"
#include "mla_dequant.cuh"  // e4m3_value

namespace mla {

constexpr int kQuantThreads = 256;

__device__ __forceinline__ uint32_t f32x2_to_e4m3x2_sat(float lo, float hi) {  // lo -> low byte
  uint16_t d;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(d) : "f"(hi), "f"(lo));
  return d;
}
// eight floats -> eight E2M1 codes (round to nearest even, saturating), value 0 in the lowest nibble
__device__ __forceinline__ uint32_t e2m1x8(const float (&y)[8]) {
  uint32_t d;
  asm("{\n.reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\ncvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\ncvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3};\n}"
      : "=r"(d)
      : "f"(y[0]), "f"(y[1]), "f"(y[2]), "f"(y[3]), "f"(y[4]), "f"(y[5]), "f"(y[6]), "f"(y[7]));
  return d;
}
__device__ __forceinline__ uint32_t e2m1_code(float y) {
  // thresholds halfway between 0, .5, 1, 1.5, 2, 3, 4, 6; a tie goes to the code with the even mantissa bit
  const float a = fabsf(y);
  const uint32_t mag = uint32_t(a > 0.25f) + uint32_t(a >= 0.75f) + uint32_t(a > 1.25f) + uint32_t(a >= 1.75f) +
                       uint32_t(a > 2.5f) + uint32_t(a >= 3.5f) + uint32_t(a > 5.0f);
  return mag | ((__float_as_uint(y) >> 28) & 8u);
}

// status: optional device word, set to 1 if a token named a request, position or page outside the tables (the token
// is skipped, nothing is written for it).
__global__ void __launch_bounds__(kQuantThreads)
mla_quantize_append_kernel(const __nv_bfloat16* __restrict__ ckv, const __nv_bfloat16* __restrict__ kpe,
                           const int* __restrict__ batch_indices, const int* __restrict__ positions, long long nnz,
                           uint8_t* __restrict__ ckv_cache, uint8_t* __restrict__ sf_cache, uint8_t* __restrict__ kpe_cache,
                           long long num_pages, int page_shift, const int* __restrict__ kv_indices,
                           const int* __restrict__ kv_indptr, int batch, float ckv_scale, float kpe_scale, int* status) {
  const int lane = threadIdx.x & 31;
  constexpr float kDown = 1.f - 0x1p-21f, kUp = 1.f + 0x1p-21f;
  const long long warp0 = (long long)blockIdx.x * (kQuantThreads / 32) + (threadIdx.x >> 5);
  const long long stride = (long long)gridDim.x * (kQuantThreads / 32);
  for (long long t = warp0; t < nnz; t += stride) {
    const int b = batch_indices[t], pos = positions[t];
    bool ok = b >= 0 && b < batch && pos >= 0;
    long long row = 0;
    if (ok) {
      const int first = kv_indptr[b], npages = kv_indptr[b + 1] - first, pi = pos >> page_shift;
      ok = pi < npages;
      if (ok) {
        const int page = kv_indices[first + pi];
        ok = page >= 0 && page < num_pages;
        row = ((long long)page << page_shift) + (pos & ((1 << page_shift) - 1));
      }
    }
    if (!ok) {
      if (lane == 0 && status) *status = 1;
      continue;
    }
    // ---- latent block `lane`
    const uint4* src = reinterpret_cast<const uint4*>(ckv + t * CKV + 16 * lane);
    const uint4 w0 = src[0], w1 = src[1];
    const uint32_t w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    float x[16];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      x[2 * j] = __uint_as_float(w[j] << 16), x[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
      amax = fmaxf(amax, fmaxf(fabsf(x[2 * j]), fabsf(x[2 * j + 1])));
    }
    const uint32_t sf8 = f32x2_to_e4m3x2_sat(__fdiv_rn(__fdiv_rn(amax, 6.0f), ckv_scale), 0.f) & 0xFFu;
    const float sf = __fmul_rn(e4m3_value(uint8_t(sf8)), ckv_scale);
    uint32_t lo = 0, hi = 0;
    if (sf > 0.f) {
      const float r = __frcp_rn(sf), down = kDown, up = kUp;
      float yd[16], yu[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float q0 = x[j] * r;
        yd[j] = q0 * down, yu[j] = q0 * up;
      }
      lo = e2m1x8(reinterpret_cast<const float(&)[8]>(yd[0])), hi = e2m1x8(reinterpret_cast<const float(&)[8]>(yd[8]));
      const uint32_t dlo = lo ^ e2m1x8(reinterpret_cast<const float(&)[8]>(yu[0]));
      const uint32_t dhi = hi ^ e2m1x8(reinterpret_cast<const float(&)[8]>(yu[8]));
      // Some values are within 2^-21 of a rounding boundary: for those the defining computation decides. Nearly all of
      // them are exact ties (BF16 inputs over a scale of a few bits): every boundary has at most three significant
      // bits, so the candidate T is the product rounded to three bits, and T * sf == |x| (one fused multiply-add,
      // exact in sign and in zero) proves that x / sf is T itself; only the rest take the division. The loop visits
      // the flagged values alone (the value is read again from memory: the registers cannot be indexed).
      auto settle = [&](uint32_t codes, uint32_t diff, int base) {
        while (diff) {
          const int j = (__ffs(diff) - 1) >> 2;
          diff &= ~(15u << (4 * j));
          const float xv = __bfloat162float(ckv[t * CKV + 16 * lane + base + j]);
          const float tie = __uint_as_float((__float_as_uint(fabsf(xv) * r) + 0x00100000u) & 0xFFE00000u);
          const float q = __fmaf_rn(tie, sf, -fabsf(xv)) == 0.f ? copysignf(tie, xv) : __fdiv_rn(xv, sf);
          codes = (codes & ~(15u << (4 * j))) | (e2m1_code(q) << (4 * j));
        }
        return codes;
      };
      lo = settle(lo, dlo, 0), hi = settle(hi, dhi, 8);
    }
    *reinterpret_cast<uint2*>(ckv_cache + row * (CKV / 2) + 8 * lane) = make_uint2(lo, hi);
    sf_cache[row * (CKV / 16) + lane] = uint8_t(sf8);
    // ---- rope channels 2 lane, 2 lane + 1
    const uint32_t r = reinterpret_cast<const uint32_t*>(kpe + t * KPE)[lane];
    const uint32_t k8 = f32x2_to_e4m3x2_sat(__fdiv_rn(__uint_as_float(r << 16), kpe_scale),
                                            __fdiv_rn(__uint_as_float(r & 0xFFFF0000u), kpe_scale));
    reinterpret_cast<uint16_t*>(kpe_cache + row * KPE)[lane] = uint16_t(k8);
  }
}

}  // namespace mla
