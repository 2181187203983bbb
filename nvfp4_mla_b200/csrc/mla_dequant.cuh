// Whole-cache dequantisation: ckv = e2m1 * block_scale * ckv_scale, kpe = e4m3 * kpe_scale, to fp32 or bf16.
// The two multiplies are separate fp32 roundings in exactly that order (never fused), which makes the fp32 result
// bit-identical to the torch expression `lut[code] * sf.float() * ckv_scale`.
//
// HBM-bound: 352 bytes in, 2304 (fp32) or 1152 (bf16) bytes out per token. One warp per token per step; for fp32 lane l
// owns channels 4l .. 4l+3 of each 128-channel quarter, for bf16 channels 8l .. 8l+7 of each half, so every store
// instruction of the warp writes 512 contiguous bytes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include "mla_common.cuh"
#include "ptx_sm100.cuh"

namespace mla {

__device__ __forceinline__ float2 f16x2_to_f32x2(uint32_t h) {  // exact
  __half2 p;
  memcpy(&p, &h, sizeof p);
  return __half22float2(p);
}
__device__ __forceinline__ float e4m3_value(uint8_t x) {
  __nv_fp8_e4m3 f;
  f.__x = x;
  return float(f);
}

template <typename T> struct Store4;
template <> struct Store4<float> {
  static __device__ __forceinline__ void put(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
  }
  static __device__ __forceinline__ void put2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};
template <> struct Store4<__nv_bfloat16> {
  static __device__ __forceinline__ void put(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
  }
  static __device__ __forceinline__ void put2(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
  }
};

constexpr int kDequantThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kDequantThreads)
mla_dequant_kernel(const uint8_t* __restrict__ ckv, const uint8_t* __restrict__ sf, const uint8_t* __restrict__ kpe,
                   float ckv_scale, float kpe_scale, T* __restrict__ ckv_out, T* __restrict__ kpe_out, long long n_tok) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (kDequantThreads / 32) + (threadIdx.x >> 5);
  const long long stride = (long long)gridDim.x * (kDequantThreads / 32);
  for (long long tok = warp0; tok < n_tok; tok += stride) {
    const uint8_t* c = ckv + tok * (CKV / 2);
    const uint8_t* s = sf + tok * (CKV / 16);
    if constexpr (sizeof(T) == 2) {
      // 16-bit output: lane l owns channels 8l .. 8l+7 of each half of the row: one 4-byte load and one 16-byte store
      // per half, every instruction of the warp contiguous (128 / 512 bytes); the 32 block scales are loaded one per
      // lane and handed round by shuffle (block = channel / 16).
      const uint32_t sv = s[lane];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(c + 128 * j + 4 * lane);
        const float scale = e4m3_value(uint8_t(__shfl_sync(~0u, sv, 16 * j + (lane >> 1))));
        uint32_t o[4], e[4];
        ptx::e2m1x8_to_f16x8(w, e);  // the eight values as FP16 pairs (exact); FP16 -> fp32 is exact too
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 v = f16x2_to_f32x2(e[i]);
          const __nv_bfloat162 h = __floats2bfloat162_rn(__fmul_rn(__fmul_rn(v.x, scale), ckv_scale),
                                                         __fmul_rn(__fmul_rn(v.y, scale), ckv_scale));
          o[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(ckv_out + tok * CKV + 256 * j + 8 * lane) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    } else
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int ch = 128 * j + 4 * lane;  // first of this lane's 4 channels
      const uint32_t two = *reinterpret_cast<const uint16_t*>(c + ch / 2);
      const float scale = e4m3_value(s[ch / 16]);
      uint32_t e0, e1;  // this lane's four values as two FP16 pairs (exact)
      asm("{\n.reg .b8 b0, b1;\nmov.b16 {b0, b1}, %2;\ncvt.rn.f16x2.e2m1x2 %0, b0;\ncvt.rn.f16x2.e2m1x2 %1, b1;\n}"
          : "=r"(e0), "=r"(e1)
          : "h"(uint16_t(two)));
      const float2 v01 = f16x2_to_f32x2(e0);
      const float2 v23 = f16x2_to_f32x2(e1);
      const float v[4] = {__fmul_rn(__fmul_rn(v01.x, scale), ckv_scale), __fmul_rn(__fmul_rn(v01.y, scale), ckv_scale),
                          __fmul_rn(__fmul_rn(v23.x, scale), ckv_scale), __fmul_rn(__fmul_rn(v23.y, scale), ckv_scale)};
      Store4<T>::put(ckv_out + tok * CKV + ch, v[0], v[1], v[2], v[3]);
    }
    const uint32_t two = *reinterpret_cast<const uint16_t*>(kpe + tok * KPE + 2 * lane);
    Store4<T>::put2(kpe_out + tok * KPE + 2 * lane, __fmul_rn(e4m3_value(two & 255), kpe_scale),
                    __fmul_rn(e4m3_value(two >> 8), kpe_scale));
  }
}

}  // namespace mla
