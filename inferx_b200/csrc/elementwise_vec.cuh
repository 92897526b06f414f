// 16-byte-vector forms of the row-wise kernels for bfloat16 activations.  Same
// arithmetic as the scalar kernels in elementwise.cu / rope_cache.cu (fp32 math,
// the same reduction helper); chosen when the row sizes allow 16-byte accesses.
#pragma once
#include "common.cuh"

__device__ __forceinline__ void bf8_to_f32(const uint4& r, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 f32_to_bf8(const float* f) {
  uint4 r;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return r;
}
