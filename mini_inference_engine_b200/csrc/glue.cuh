// Helpers shared by the memory-bound glue kernels: 8 x bf16 <-> fp32 and the per-128-column e4m3 quantiser.
#pragma once

#include "common.cuh"

namespace mie {

__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(p[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return raw;
}

// Quantise 8 values held by each of 16 consecutive lanes (one 128-column group): this lane's eight e4m3
// bytes and the group's raw scale (amax / 448).
__device__ __forceinline__ void quantize_group(const float (&v)[8], uint32_t (&packed)[2], float& scale) {
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  scale = __fdiv_rn(amax, 448.0f);
  const float denom = fmaxf(scale, 1e-12f);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
        make_float2(__fdiv_rn(v[4 * h], denom), __fdiv_rn(v[4 * h + 1], denom)), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(
        make_float2(__fdiv_rn(v[4 * h + 2], denom), __fdiv_rn(v[4 * h + 3], denom)), __NV_SATFINITE, __NV_E4M3);
    packed[h] = (uint32_t)lo | ((uint32_t)hi << 16);
  }
}
__device__ __forceinline__ void quantize_group_store(const float (&v)[8], uint8_t* q_dst, float* scale_dst,
                                                     bool scale_writer) {
  uint32_t packed[2];
  float scale;
  quantize_group(v, packed, scale);
  if (q_dst != nullptr) *reinterpret_cast<uint2*>(q_dst) = make_uint2(packed[0], packed[1]);
  if (scale_writer && scale_dst != nullptr) *scale_dst = scale;
}

}  // namespace mie
