// Floating-point helpers whose results are defined bit for bit: they use only
// IEEE-754 binary32 add / multiply / fused multiply-add / divide / square root
// in a fixed order, so a CPU that evaluates the same sequence (compiled without
// contraction, with explicit fmaf) produces identical bits.  The routing
// weights are computed with these instead of the hardware approximations
// (__expf, rsqrtf) the reference uses (csrc/fabric/tiles/aux.cuh:358,371), which
// are not reproducible off the GPU.
#pragma once
#include <cuda_bf16.h>

namespace mf {

// exp(x) for any finite x: Cody-Waite reduction by ln2 (two constants), a
// degree-5 polynomial in Horner form on |r| <= ln2/2, exp(r) = 1 + r + r^2 P(r),
// and an exact two-step power-of-two scaling (so that results in the denormal
// range round exactly once).
__device__ __forceinline__ float det_expf(float x) {
  if (x < -103.0f) return 0.0f;
  x = fminf(x, 89.0f);
  const float n = rintf(__fmul_rn(x, 1.44269502162933349609375f));
  float r = __fmaf_rn(n, -0.693145751953125f, x);
  r = __fmaf_rn(n, -1.428606765330187045037746429443359375e-06f, r);
  float p = 1.9875691500e-4f;
  p = __fmaf_rn(p, r, 1.3981999507e-3f);
  p = __fmaf_rn(p, r, 8.3334519073e-3f);
  p = __fmaf_rn(p, r, 4.1665795894e-2f);
  p = __fmaf_rn(p, r, 1.6666665459e-1f);
  p = __fmaf_rn(p, r, 5.0000001201e-1f);
  const float rr = __fmul_rn(r, r);
  float y = __fmaf_rn(p, rr, r);
  y = __fadd_rn(y, 1.0f);
  const int ni = static_cast<int>(n);
  const int h = ni / 2;
  const float s1 = __int_as_float((h + 127) << 23);
  const float s2 = __int_as_float((ni - h + 127) << 23);
  return __fmul_rn(__fmul_rn(y, s1), s2);
}

__device__ __forceinline__ float det_sigmoidf(float x) {
  return __fdiv_rn(1.0f, __fadd_rn(1.0f, det_expf(-x)));
}

// 1 / sqrt(v) with correctly rounded square root and divide.
__device__ __forceinline__ float det_rsqrtf(float v) { return __fdiv_rn(1.0f, __fsqrt_rn(v)); }

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Butterfly sum over the warp: every lane ends with the same bits.
__device__ __forceinline__ float warp_sum_xor(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace mf
