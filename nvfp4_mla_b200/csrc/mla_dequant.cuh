// Whole-cache dequantisation: ckv = e2m1 * block_scale * ckv_scale, kpe = e4m3 * kpe_scale, to fp32 or bf16.
// The two multiplies are separate fp32 roundings in exactly that order (never fused), which makes the fp32 result
// bit-identical to the torch expression `lut[code] * sf.float() * ckv_scale`.
//
// HBM-bound: 352 bytes in, 2304 (fp32) or 1152 (bf16) bytes out per token. One warp per token per step; lane l owns
// channels 4l .. 4l+3 of each 128-channel quarter, so every store instruction of the warp writes 512 (fp32) or 256
// (bf16) contiguous bytes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include "mla_common.cuh"

namespace mla {

__device__ __forceinline__ float e2m1_value(uint32_t c) {
  // codes 0..7: 0, .5, 1, 1.5, 2, 3, 4, 6; bit 3 = sign. Built as fp32 bits: exponent field (c >> 1) + 126 for
  // normals, mantissa msb = c & 1; code 1 (the only subnormal) is 0.5.
  const uint32_t mag = c & 7;
  const float v = (mag & 6) ? __uint_as_float((((mag >> 1) + 126u) << 23) | ((mag & 1u) << 22)) : 0.5f * float(mag & 1);
  return (c & 8) ? -v : v;
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
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int ch = 128 * j + 4 * lane;  // first of this lane's 4 channels
      const uint32_t two = *reinterpret_cast<const uint16_t*>(c + ch / 2);
      const float scale = e4m3_value(s[ch / 16]);
      float v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = __fmul_rn(__fmul_rn(e2m1_value((two >> (4 * i)) & 15), scale), ckv_scale);
      Store4<T>::put(ckv_out + tok * CKV + ch, v[0], v[1], v[2], v[3]);
    }
    const uint32_t two = *reinterpret_cast<const uint16_t*>(kpe + tok * KPE + 2 * lane);
    Store4<T>::put2(kpe_out + tok * KPE + 2 * lane, __fmul_rn(e4m3_value(two & 255), kpe_scale),
                    __fmul_rn(e4m3_value(two >> 8), kpe_scale));
  }
}

}  // namespace mla
