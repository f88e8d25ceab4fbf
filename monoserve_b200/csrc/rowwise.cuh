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

// Routing of one token by one warp: what the reference's router tile computes
// (csrc/fabric/tiles/aux.cuh:326-417): scores = softmax of the E <= 256 logits, or their sigmoid with
// an optional selection bias; K <= 16 picks, each the best remaining selection score with the lowest
// expert id winning ties; weights = the picks' scores, renormalised by their sum taken in pick
// order, times `scale`.  Lane k < K returns pick k in (pick_id, pick_weight).  zero_logits: clear the
// row once read.
//
// Lane l holds experts l, l + 32, ... (slot i = expert l + 32 i).  The floating-point order is part
// of the result's definition (the oracle repeats it): row maximum (any order: max is exact), per lane
// the exponentials summed over its slots in slot order, the lanes' sums by the xor butterfly 16..1,
// one IEEE division per score.  The K arg-max rounds only compare, so they are done on integers:
// a score and its expert id become one 64-bit key whose order is (score ascending, id descending).
namespace route {

constexpr int kSlots = kMaxExperts / 32;
constexpr float kAbsent = -1e30f;   // stands in for experts past E

// 32-bit pattern whose unsigned order is the order of the (non-NaN) floats.
__device__ __forceinline__ unsigned int ordered_bits(float v) {
  const unsigned int u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long pick_key(float score, int expert) {
  return (static_cast<unsigned long long>(ordered_bits(score)) << 32) | (0xffffffffu - static_cast<unsigned int>(expert));
}
__device__ __forceinline__ int key_expert(unsigned long long key) { return static_cast<int>(0xffffffffu - static_cast<unsigned int>(key)); }

__device__ __forceinline__ unsigned long long warp_max_key(unsigned long long k) {
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, k, o);
    k = other > k ? other : k;
  }
  return k;
}

}  // namespace route

__device__ __forceinline__ void route_row(float* logits_row, const float* bias, int E, int K, int scoring, int renorm,
                                          float scale, int zero_logits, int& pick_id, float& pick_weight) {
  using namespace route;
  const int lane = threadIdx.x & 31;
  float score[kSlots];
#pragma unroll
  for (int i = 0; i < kSlots; ++i) {
    const int expert = lane + 32 * i;
    score[i] = expert < E ? logits_row[expert] : kAbsent;
    if (zero_logits && expert < E) logits_row[expert] = 0.f;
  }
  unsigned long long key[kSlots];   // selection key per slot; 0 once picked (below every real key)
  if (scoring == 0) {
    float top = kAbsent;
#pragma unroll
    for (int i = 0; i < kSlots; ++i) top = fmaxf(top, score[i]);
#pragma unroll
    for (int o = 16; o; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
    float lane_sum = 0.f;
#pragma unroll
    for (int i = 0; i < kSlots; ++i) {
      score[i] = det_expf(__fsub_rn(score[i], top));   // an absent expert gives exactly 0
      lane_sum = __fadd_rn(lane_sum, score[i]);
    }
    const float total = warp_sum_xor(lane_sum);
#pragma unroll
    for (int i = 0; i < kSlots; ++i) {
      score[i] = __fdiv_rn(score[i], total);
      key[i] = pick_key(lane + 32 * i < E ? score[i] : kAbsent, lane + 32 * i);
    }
  } else {
#pragma unroll
    for (int i = 0; i < kSlots; ++i) {
      const int expert = lane + 32 * i;
      score[i] = det_sigmoidf(score[i]);
      key[i] = pick_key(expert < E ? __fadd_rn(score[i], bias ? bias[expert] : 0.f) : kAbsent, expert);
    }
  }
  pick_id = 0;
  float mine = 0.f, picked_sum = 0.f;
  for (int k = 0; k < K; ++k) {
    unsigned long long best = 0;
#pragma unroll
    for (int i = 0; i < kSlots; ++i) best = key[i] > best ? key[i] : best;
    const int expert = key_expert(warp_max_key(best));
    // the lane that holds the pick takes it out of the running and hands its score round
    float held = 0.f;
#pragma unroll
    for (int i = 0; i < kSlots; ++i)
      if (lane + 32 * i == expert) {
        held = score[i];
        key[i] = 0;
      }
    const float weight = __shfl_sync(0xffffffffu, held, expert & 31);
    if (lane == k) {
      pick_id = expert;
      mine = weight;
    }
    picked_sum = __fadd_rn(picked_sum, weight);
  }
  pick_weight = __fmul_rn(renorm ? __fdiv_rn(mine, picked_sum) : mine, scale);
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
