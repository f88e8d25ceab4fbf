// Warp-level row routines shared by the stream-launched kernels and the fabric's
// row-wise tiles: routing of one token, and the RMSNorm of one row.  Their results
// are defined bit for bit (detmath.cuh), so the oracle can be compared exactly.
#pragma once
#include <cuda_bf16.h>

#include "detmath.cuh"
#include "types.h"

namespace mf {

__device__ __forceinline__ void unpack8(const uint4& u, float f[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ uint4 pack8(const float f[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// Routing of one token by one warp (csrc/fabric/tiles/aux.cuh:326-417): softmax
// or sigmoid (+ selection bias) over E <= 256 logits, K <= 16 rounds of arg-max with
// the lowest index winning ties, renormalisation in pick order, scale.  Lane k < K
// returns pick k in (my_id, my_w).  zero_logits: clear the row after reading it.
__device__ __forceinline__ void route_row(float* lg, const float* bias, int E, int K, int scoring, int renorm,
                                          float scale, int zero_logits, int& my_id, float& my_w_out) {
  constexpr int kMaxPer = kMaxExperts / 32;
  const int lane = threadIdx.x & 31;
  float p[kMaxPer], sel[kMaxPer];
#pragma unroll
  for (int i = 0; i < kMaxPer; ++i) {
    const int e = lane + 32 * i;
    p[i] = e < E ? lg[e] : -1e30f;
  }
  if (zero_logits) {
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i)
      if (lane + 32 * i < E) lg[lane + 32 * i] = 0.f;
  }
  if (scoring == 0) {
    float mx = -1e30f;
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i) mx = fmaxf(mx, p[i]);
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i) {
      p[i] = det_expf(__fsub_rn(p[i], mx));
      s = __fadd_rn(s, p[i]);
    }
    s = warp_sum_xor(s);
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i) {
      p[i] = __fdiv_rn(p[i], s);
      sel[i] = lane + 32 * i < E ? p[i] : -1e30f;
    }
  } else {
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i) {
      const int e = lane + 32 * i;
      p[i] = det_sigmoidf(p[i]);
      sel[i] = e < E ? __fadd_rn(p[i], bias ? bias[e] : 0.f) : -1e30f;
    }
  }
  my_id = 0;
  float my_w = 0.f, wsum = 0.f;
  for (int k = 0; k < K; ++k) {
    float bv = -1e30f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i) {
      const int e = lane + 32 * i;
      if (sel[i] > bv || (sel[i] == bv && e < bi)) {
        bv = sel[i];
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    float mine = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i) {
      if (i == (bi >> 5)) {
        mine = p[i];
        if (lane == (bi & 31)) sel[i] = -1e30f;
      }
    }
    const float w = __shfl_sync(0xffffffffu, mine, bi & 31);
    if (lane == k) {
      my_id = bi;
      my_w = w;
    }
    wsum = __fadd_rn(wsum, w);
  }
  my_w_out = __fmul_rn(renorm ? __fdiv_rn(my_w, wsum) : my_w, scale);
}

// RMSNorm of a bf16 row that this warp holds in `x` (H elements, lane l owns the
// 8-element groups l, l + 32, ...): out = bf16(bf16(x * inv) * w), inv = 1 / sqrt(ss / H + eps)
// with correctly rounded square root and divide (csrc/fabric/tiles/aux.cuh:60-122 uses
// rsqrtf).  ss is this lane's partial sum of squares, accumulated by the caller with
// one fmaf per element in storage order.  out2 optionally receives a copy.
__device__ __forceinline__ void norm_store_row(const uint4* x, float ss, const __nv_bfloat16* norm_w,
                                               __nv_bfloat16* out, __nv_bfloat16* out2, int H, float eps) {
  const int lane = threadIdx.x & 31, n16 = H / 8;
  ss = warp_sum_xor(ss);
  const float inv = det_rsqrtf(__fadd_rn(__fdiv_rn(ss, static_cast<float>(H)), eps));
  __syncwarp();
  const uint4* w4 = reinterpret_cast<const uint4*>(norm_w);
  uint4* o = reinterpret_cast<uint4*>(out);
  uint4* o2 = reinterpret_cast<uint4*>(out2);
  for (int c = lane; c < n16; c += 32) {
    float f[8], g[8];
    unpack8(x[c], f);
    unpack8(w4[c], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = __fmul_rn(round_bf16(__fmul_rn(f[j], inv)), g[j]);
    const uint4 v = pack8(f);
    o[c] = v;
    if (o2) o2[c] = v;
  }
}

}  // namespace mf
