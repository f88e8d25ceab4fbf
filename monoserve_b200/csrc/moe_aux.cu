// Routing, planning, packing and combining kernels of one MoE layer.  These
// are HBM/latency-bound integer and byte kernels built on warp primitives; no
// tensor cores.  Their results are defined exactly (see detmath.cuh) so that a
// CPU oracle can be compared bit for bit:
//
//   router_logits   logits[t][e] = sum_h x[t][h] * Wr[e][h]   fp32, fixed order
//   router_topk     softmax / sigmoid(+bias), K rounds of arg-max with the
//                   lowest index winning ties, renormalisation, scale
//                   (csrc/fabric/tiles/aux.cuh:326-417), plus the stable rank of
//                   every (token, pick) pair inside its 32-token chunk
//   plan            per-expert counts, exclusive prefix sums (aux.cuh:423-450),
//                   per-chunk bases, and the grouped-GEMM tile lists chosen
//                   through the layer's (region, slot) table (aux.cuh:453-616)
//   pack            expert-sorted activation rows and pair lists
//                   (aux.cuh:648-684).  The reference orders an expert's rows by
//                   atomic arrival; here the order is fixed: token ascending,
//                   then pick ascending.
//   combine         x[t] = bf16(x2[t] + sum_k w[t][k] * y[pos(t,k)]) in pick
//                   order, optionally followed by the next RMSNorm
//                   (aux.cuh:137-188; the reference sums with fp32 atomics).
#include <cuda_bf16.h>

#include "detmath.cuh"
#include "kernels.h"
#include "peer_sync.cuh"
#include "rowwise.cuh"

namespace mf {

// ------------------------------------------------------------ router logits
// One warp computes the logits of one token against kExpertsPerWarp experts.
// Lane l owns elements h = 256 j + 8 l + i (j outer, i = 0..7 inner) and
// accumulates them in that order with fused multiply-adds into one fp32
// partial; the 32 partials are summed by the xor butterfly 16, 8, 4, 2, 1.
constexpr int kExpertsPerWarp = 16;

template <int J>
__global__ void __launch_bounds__(256) router_logits_kernel(const bf16* __restrict__ x, const bf16* __restrict__ wr,
                                                            float* __restrict__ logits, int T, int H, int E) {
  chain_release();
  chain_wait();
  const int lane = threadIdx.x & 31;
  const int groups = (E + kExpertsPerWarp - 1) / kExpertsPerWarp;
  const long long unit = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= static_cast<long long>(T) * groups) return;
  const int t = static_cast<int>(unit / groups), eg = static_cast<int>(unit % groups);
  const int nj = J > 0 ? J : H / 256;
  const uint4* x4 = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H);
  float xr[J > 0 ? J : 1][8];
  if (J > 0) {
#pragma unroll
    for (int j = 0; j < J; ++j) unpack8(x4[32 * j + lane], xr[j]);
  }
  const int e_hi = min(E, (eg + 1) * kExpertsPerWarp);
  for (int e = eg * kExpertsPerWarp; e < e_hi; ++e) {
    const uint4* w4 = reinterpret_cast<const uint4*>(wr + static_cast<size_t>(e) * H);
    float acc = 0.f;
    if (J > 0) {
      uint4 wv[J > 0 ? J : 1];
#pragma unroll
      for (int j = 0; j < J; ++j) wv[j] = __ldg(w4 + 32 * j + lane);
#pragma unroll
      for (int j = 0; j < J; ++j) {
        float wf[8];
        unpack8(wv[j], wf);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc = __fmaf_rn(xr[j][i], wf[i], acc);
      }
    } else {
      for (int j = 0; j < nj; ++j) {
        float xf[8], wf[8];
        unpack8(x4[32 * j + lane], xf);
        unpack8(__ldg(w4 + 32 * j + lane), wf);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc = __fmaf_rn(xf[i], wf[i], acc);
      }
    }
    acc = warp_sum_xor(acc);
    if (lane == (e & 31)) logits[static_cast<size_t>(t) * E + e] = acc;
  }
}

// -------------------------------------------------------------- router top-k
// One block per chunk of 32 tokens, one warp per token.

__global__ void __launch_bounds__(1024) router_topk_kernel(const RouterParams A) {
  __shared__ int s_ids[kChunkTokens * kMaxTopK];
  __shared__ int s_hist[kMaxExperts];
  chain_release();
  chain_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int E = A.E, K = A.K;
  const int r = blockIdx.x * kChunkTokens + warp;
  if (threadIdx.x < kMaxExperts) s_hist[threadIdx.x] = 0;
  if (r < A.T) {
    int my_id;
    float my_w;
    route_row(A.logits + static_cast<size_t>(r) * E, A.bias, E, K, A.scoring, A.renorm, A.scale, A.zero_logits, my_id,
              my_w);
    if (lane < K) {
      A.topk_ids[static_cast<size_t>(r) * K + lane] = my_id;
      A.topk_w[static_cast<size_t>(r) * K + lane] = my_w;
      s_ids[warp * K + lane] = my_id;
    }
  }
  __syncthreads();
  const int rows = min(kChunkTokens, A.T - blockIdx.x * kChunkTokens);
  const int pairs = rows * K;
  if (static_cast<int>(threadIdx.x) < pairs) {
    const int me = s_ids[threadIdx.x];
    int rank = 0;
    for (int q = 0; q < static_cast<int>(threadIdx.x); ++q) rank += s_ids[q] == me;
    if (A.pair_rank) A.pair_rank[static_cast<size_t>(blockIdx.x) * kChunkTokens * K + threadIdx.x] = rank;
    atomicAdd(&s_hist[me], 1);
  }
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < E) {
    const int c = s_hist[threadIdx.x];
    if (A.chunk_counts) A.chunk_counts[static_cast<size_t>(blockIdx.x) * E + threadIdx.x] = c;
    if (A.counts && c) atomicAdd(A.counts + threadIdx.x, c);
  }
}

// ------------------------------------------------------------- chunk ranks
// The rank step of the stable pack on its own, for routing that was computed
// elsewhere: one block per chunk of 32 tokens; thread p = (token, pick) counts
// the earlier pairs of the chunk that chose the same expert, and the block
// writes the chunk's per-expert pair counts.
// A pair whose expert id lies outside [0, E) is dropped (rank -1, counted nowhere) and
// reported as kErrBadArgs when a status word is given.
__global__ void __launch_bounds__(kChunkTokens * kMaxTopK) chunk_rank_kernel(const int* __restrict__ topk_ids,
                                                                             int* __restrict__ pair_rank,
                                                                             int* __restrict__ chunk_counts,
                                                                             int T, int E, int K, int* status) {
  __shared__ int s_ids[kChunkTokens * kMaxTopK];
  __shared__ int s_hist[kMaxExperts];
  chain_release();
  chain_wait();
  const int rows = min(kChunkTokens, T - static_cast<int>(blockIdx.x) * kChunkTokens);
  const int pairs = rows * K;
  const int p = threadIdx.x;
  const size_t base = static_cast<size_t>(blockIdx.x) * kChunkTokens * K;
  if (p < kMaxExperts) s_hist[p] = 0;
  if (p < pairs) s_ids[p] = topk_ids[base + p];
  __syncthreads();
  if (p < pairs) {
    const int me = s_ids[p];
    if (me >= 0 && me < E) {
      int rank = 0;
      for (int q = 0; q < p; ++q) rank += s_ids[q] == me;
      pair_rank[base + p] = rank;
      atomicAdd(&s_hist[me], 1);
    } else {
      pair_rank[base + p] = -1;
      if (status) atomicOr(status, kErrBadArgs);
    }
  }
  __syncthreads();
  for (int e = p; e < E; e += blockDim.x) chunk_counts[static_cast<size_t>(blockIdx.x) * E + e] = s_hist[e];
}

// ---------------------------------------------------------------------- plan

// Exclusive scan of one int per thread over a 256-thread block; returns the
// exclusive prefix and writes the block total.
__device__ __forceinline__ int block_scan_256(int v, int* s_warp, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += y;
  }
  __syncthreads();
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  int base = 0;
  total = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    const int s = s_warp[w];
    if (w < warp) base += s;
    total += s;
  }
  return base + incl - v;
}

__global__ void __launch_bounds__(256) plan_kernel(const PlanParams A) {
  __shared__ int s_warp[8];
  const int e = threadIdx.x;
  const int E = A.E;
  int cnt = 0;
  bool bad = false;
  chain_release();
  chain_wait();
  if (A.wait_flags) {   // expert parallelism: the counts and the rows they describe come from peers
    if (e < A.wait_n && !wait_flag(A.wait_flags + e, A.wait_epoch)) atomicOr(A.status, kErrWaitTimeout);
    __syncthreads();
  }
  if (e < E && A.seg_counts) {
    const int tables = A.seg_tables > 0 ? A.seg_tables : 1;
    for (int i = 0; i < tables; ++i) {
      const int c = A.seg_counts[static_cast<size_t>(i) * A.seg_stride + e];
      bad |= c < 0;
      cnt += c;
    }
    if (bad) cnt = 0;
    A.counts[e] = cnt;
  } else if (e < E) {
    for (int c = 0; c < A.chunks; ++c) {
      int* cell = A.chunk_counts + static_cast<size_t>(c) * E + e;
      const int v = *cell;
      *cell = cnt;
      cnt += v;
    }
    A.counts[e] = cnt;
    if (A.hist) A.hist[e] += cnt;
  }
  int total;
  const int start = block_scan_256(cnt, s_warp, total);
  if (e < E) A.starts[e] = start;
  if (e == 0) A.starts[E] = total;

  if (!A.q) return;   // scan only: counts, starts and chunk prefixes
  int tier = kTierHot, z = 0, bh = 128, nb = 0;
  const int expert = (e < E && A.seg_expert) ? A.seg_expert[e] : e;
  // A segment of an expert the table does not hold, a negative count or more rows than the packed-row
  // buffers take: no tile is emitted and the layer reports a plan overflow.
  bad |= e < E && cnt > 0 && (expert < 0 || expert >= A.n_experts);
  const bool refuse = __syncthreads_or(bad) || total > A.rows_cap;
  if (e < E && cnt > 0 && !refuse) {
    tier = A.table[2 * expert] == 0 ? kTierHost : kTierHot;
    z = A.table[2 * expert + 1];
    if (tier == kTierHost) bh = A.form ? A.form : 256;
    nb = (cnt + bh - 1) / bh;
  }
  const int f13 = (A.I + 63) / 64, f2 = (A.H + 127) / 128;
  // per tier: [w13 tiles of every expert][w2 tiles of every expert]; row blocks numbered over all experts
  int first13[2], first2[2], total13[2], total2[2], blocks_total;
  const int block0 = block_scan_256(nb, s_warp, blocks_total);
  for (int tq = 0; tq < 2; ++tq) {
    const int mine = tier == tq ? nb : 0;
    first13[tq] = block_scan_256(mine * f13, s_warp, total13[tq]);
    first2[tq] = block_scan_256(mine * f2, s_warp, total2[tq]);
  }
  bool overflow = refuse || blocks_total > A.block_cap;
  for (int tq = 0; tq < 2; ++tq) overflow |= total13[tq] + total2[tq] > A.tile_cap;
  for (int b = e; b < blocks_total && !overflow; b += blockDim.x) A.done[b] = 0;
  if (e == 0) {
    for (int tq = 0; tq < 2; ++tq) {
      A.q->n_tiles[tq] = overflow ? 0 : total13[tq] + total2[tq];
      A.q->head[tq] = 0;
    }
    A.q->slots = 0;
    A.q->n_blocks = blocks_total;
    A.q->need = 4 * f13;   // four epilogue warps arrive per w13 tile
    if (overflow) atomicOr(A.status, kErrPlanOverflow);
  }
  // Every expert's tile list is written by a warp, a tile per lane (an expert at decode batch sizes has
  // 28 tiles; written from one thread per expert they were the longest serial stretch of the layer).
  __shared__ int s_job[kMaxExperts][8];   // nb, bh, rows, first row, slot, tier, first w13 tile, first w2 tile (+ block0 below)
  __shared__ int s_block0[kMaxExperts], s_expert[kMaxExperts];
  if (e < E) {
    s_job[e][0] = overflow ? 0 : nb;
    s_job[e][1] = bh;
    s_job[e][2] = cnt;
    s_job[e][3] = start;
    s_job[e][4] = z;
    s_job[e][5] = tier;
    s_job[e][6] = first13[tier];
    s_job[e][7] = total13[tier] + first2[tier];
    s_block0[e] = block0;
    s_expert[e] = expert;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_block = f13 + f2;
  for (int x = warp; x < E; x += static_cast<int>(blockDim.x >> 5)) {
    const int x_nb = s_job[x][0];
    if (x_nb == 0) continue;
    const int x_bh = s_job[x][1], x_cnt = s_job[x][2], x_start = s_job[x][3], x_tier = s_job[x][5];
    GemmTile* const list = A.tiles[x_tier];
    for (int j = lane; j < x_nb * per_block; j += 32) {
      const int b = j / per_block, f = j - b * per_block;
      const bool up = f >= f13;   // a w2 tile
      const int rows = min(x_bh, x_cnt - b * x_bh);
      int n = 16;
      while (n < rows) n <<= 1;
      GemmTile t;
      t.w_row0 = up ? (f - f13) * 128 : f * 64;
      t.act_row0 = x_start + b * x_bh;
      t.rows = rows;
      t.n = n;
      t.z = s_job[x][4];
      t.tier_phase = x_tier | (up ? 1 << 8 : 0);
      t.expert = s_expert[x];
      t.block = s_block0[x] + b;
      list[up ? s_job[x][7] + b * f2 + (f - f13) : s_job[x][6] + b * f13 + f] = t;
    }
  }
}

// ---------------------------------------------------------------------- pack

__global__ void __launch_bounds__(256) pack_kernel(const PackParams A) {
  chain_release();
  chain_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= A.T) return;
  const int K = A.K;
  int pos = -1;   // stays -1 for a pair whose expert id is outside [0, E): it is dropped
  if (lane < K) {
    const int e = A.topk_ids[static_cast<size_t>(t) * K + lane];
    if (e >= 0 && e < A.E) {
      pos = A.starts[e] + A.chunk_prefix[static_cast<size_t>(t / kChunkTokens) * A.E + e] +
            A.pair_rank[static_cast<size_t>(t) * K + lane];
      A.pair_token[pos] = t;
      A.pair_weight[pos] = A.topk_w[static_cast<size_t>(t) * K + lane];
    } else if (A.status) {
      atomicOr(A.status, kErrBadArgs);
    }
    A.pair_pos[static_cast<size_t>(t) * K + lane] = pos;
  }
  if (!A.src) return;   // pair lists only
  const uint4* src = reinterpret_cast<const uint4*>(A.src + static_cast<size_t>(t) * A.H);
  const int n16 = A.H / 8;
  for (int c0 = 0; c0 < n16; c0 += 32 * 8) {
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (c0 + 32 * i + lane < n16) v[i] = src[c0 + 32 * i + lane];
    for (int k = 0; k < K; ++k) {
      const int pk = __shfl_sync(0xffffffffu, pos, k);
      if (pk < 0) continue;
      uint4* dst = reinterpret_cast<uint4*>(A.dst + static_cast<size_t>(pk) * A.H);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (c0 + 32 * i + lane < n16) dst[c0 + 32 * i + lane] = v[i];
    }
  }
}

// ------------------------------------------------------------------- combine

constexpr int kCombineSplit = 4;   // warps per token when no row reduction follows

__global__ void __launch_bounds__(256) combine_kernel(const CombineParams A) {
  // Without the fused RMSNorm a row needs no reduction, so kCombineSplit warps share a token's columns:
  // a decode batch of a few hundred tokens otherwise leaves most of the machine idle.  Every column is
  // computed by the same instructions either way: the result does not depend on the split.
  const int lane = threadIdx.x & 31;
  chain_release();
  chain_wait();
  if (A.wait_flags) {   // expert parallelism: y is written by peers
    if (static_cast<int>(threadIdx.x) < A.wait_n && !wait_flag(A.wait_flags + threadIdx.x, A.wait_epoch))
      atomicOr(A.status, kErrWaitTimeout);
    __syncthreads();
  }
  const int split = A.norm_w ? 1 : kCombineSplit;
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int t = unit / split, part = unit - t * split;
  if (t >= A.T) return;
  const int K = A.K, H = A.H, n16 = H / 8;
  const int c_begin = part * n16 / split, c_end = (part + 1) * n16 / split;
  int pos = 0;
  float w = 0.f;
  if (lane < K) {
    pos = A.pair_pos[static_cast<size_t>(t) * K + lane];
    w = A.topk_w[static_cast<size_t>(t) * K + lane];
  }
  const uint4* x2 = A.x2 ? reinterpret_cast<const uint4*>(A.x2 + static_cast<size_t>(t) * H) : nullptr;
  uint4* xo = reinterpret_cast<uint4*>(A.x + static_cast<size_t>(t) * H);
  float ss = 0.f;
  // Same trip count in every lane: the shuffles inside need the whole warp.  A lane past the end of its
  // part goes through the motions on the part's last column and neither stores nor counts it.
  for (int c0 = c_begin; c0 < c_end; c0 += 32) {
    const int c = min(c0 + lane, c_end - 1);
    const bool on = c0 + lane < c_end;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = 0; k < K; ++k) {
      const int pk = __shfl_sync(0xffffffffu, pos, k);
      const float wk = __shfl_sync(0xffffffffu, w, k);
      if (pk < 0 || (A.y_rows && pk >= A.y_rows)) continue;   // a dropped pair adds nothing
      const float4* yr = reinterpret_cast<const float4*>(A.y + static_cast<size_t>(pk) * H) + 2 * c;
      const float4 a = __ldcs(yr), b = __ldcs(yr + 1);
      acc[0] = __fmaf_rn(wk, a.x, acc[0]);
      acc[1] = __fmaf_rn(wk, a.y, acc[1]);
      acc[2] = __fmaf_rn(wk, a.z, acc[2]);
      acc[3] = __fmaf_rn(wk, a.w, acc[3]);
      acc[4] = __fmaf_rn(wk, b.x, acc[4]);
      acc[5] = __fmaf_rn(wk, b.y, acc[5]);
      acc[6] = __fmaf_rn(wk, b.z, acc[6]);
      acc[7] = __fmaf_rn(wk, b.w, acc[7]);
    }
    float f[8];
    if (x2) {
      unpack8(x2[c], f);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      f[j] = round_bf16(__fadd_rn(f[j], acc[j]));
      if (on) ss = __fmaf_rn(f[j], f[j], ss);
    }
    if (on) xo[c] = pack8(f);
  }
  if (!A.norm_w) return;
  norm_store_row(xo, ss, A.norm_w, A.normed + static_cast<size_t>(t) * H, nullptr, H, A.eps);
}

// ------------------------------------------------------------------ launchers
cudaError_t launch_router_logits(const void* x, const void* wr, float* logits, int T, int H, int E,
                                 cudaStream_t stream) {
  if (T == 0) return cudaSuccess;
  const int groups = (E + kExpertsPerWarp - 1) / kExpertsPerWarp;
  const long long units = static_cast<long long>(T) * groups;
  const int blocks = static_cast<int>((units + 7) / 8);
  const bf16* xb = static_cast<const bf16*>(x);
  const bf16* wb = static_cast<const bf16*>(wr);
  switch (H / 256) {
    case 2: return launch_chained(router_logits_kernel<2>, blocks, 256, 0, stream, xb, wb, logits, T, H, E);
    case 4: return launch_chained(router_logits_kernel<4>, blocks, 256, 0, stream, xb, wb, logits, T, H, E);
    case 8: return launch_chained(router_logits_kernel<8>, blocks, 256, 0, stream, xb, wb, logits, T, H, E);
    case 16: return launch_chained(router_logits_kernel<16>, blocks, 256, 0, stream, xb, wb, logits, T, H, E);
    default: return launch_chained(router_logits_kernel<0>, blocks, 256, 0, stream, xb, wb, logits, T, H, E);
  }
}

cudaError_t launch_router_topk(const RouterParams& A, cudaStream_t stream) {
  if (A.T == 0) return cudaSuccess;
  return launch_chained(router_topk_kernel, (A.T + kChunkTokens - 1) / kChunkTokens, 1024, 0, stream, A);
}

cudaError_t launch_chunk_rank(const int* topk_ids, int* pair_rank, int* chunk_counts, int T, int E, int K,
                              int* status, cudaStream_t stream) {
  if (T == 0) return cudaSuccess;
  return launch_chained(chunk_rank_kernel, (T + kChunkTokens - 1) / kChunkTokens, kChunkTokens * kMaxTopK, 0, stream,
                        topk_ids, pair_rank, chunk_counts, T, E, K, status);
}

cudaError_t launch_plan(const PlanParams& A, cudaStream_t stream) {
  return launch_chained(plan_kernel, 1, 256, 0, stream, A);
}

cudaError_t launch_pack(const PackParams& A, cudaStream_t stream) {
  if (A.T == 0) return cudaSuccess;
  return launch_chained(pack_kernel, (A.T + 7) / 8, 256, 0, stream, A);
}

size_t pack_scratch_bytes(int T, int E, int K) {
  const size_t chunks = (static_cast<size_t>(T) + kChunkTokens - 1) / kChunkTokens;
  return chunks * E * sizeof(int) + static_cast<size_t>(T) * K * sizeof(int);
}

cudaError_t launch_pack_chain(const int* topk_ids, const float* topk_w, int T, int E, int K, int H, const bf16* src,
                              bf16* dst, int* counts, int* starts, int* pair_token, float* pair_weight,
                              int* pair_pos, void* scratch, int* status, cudaStream_t stream) {
  const int chunks = (T + kChunkTokens - 1) / kChunkTokens;
  int* chunk_counts = static_cast<int*>(scratch);
  int* pair_rank = chunk_counts + static_cast<size_t>(chunks) * E;
  cudaError_t err = launch_chunk_rank(topk_ids, pair_rank, chunk_counts, T, E, K, status, stream);
  if (err != cudaSuccess) return err;
  PlanParams pp{};
  pp.chunk_counts = chunk_counts;
  pp.counts = counts;
  pp.starts = starts;
  pp.chunks = chunks;
  pp.E = E;
  pp.n_experts = E;
  err = launch_plan(pp, stream);
  if (err != cudaSuccess) return err;
  PackParams kp{topk_ids, topk_w, pair_rank, chunk_counts, starts, src, dst, pair_token, pair_weight, pair_pos,
                T, E, K, H, status};
  return launch_pack(kp, stream);
}

cudaError_t launch_combine(const CombineParams& A, cudaStream_t stream) {
  if (A.T == 0) return cudaSuccess;
  const int units = A.T * (A.norm_w ? 1 : kCombineSplit);
  return launch_chained(combine_kernel, (units + 7) / 8, 256, 0, stream, A);
}

}  // namespace mf
