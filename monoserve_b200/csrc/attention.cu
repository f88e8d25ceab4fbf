// Paged-KV GQA attention for prefill and decode rows on tcgen05 / TMEM / TMA.
//
// What it computes is the reference's attention tiles (csrc/fabric/tiles/attention.cuh:
// 174-281 prefill, 286-371 decode; AttnArgs csrc/fabric/model_types.h:68-96): causal
// softmax(q k^T / sqrt(D)) v over a paged cache [pages][page][hkv][128] (K and V
// separately), head_dim 128, scores scaled in the exp2 domain, masked keys weight 0,
// P rounded to bf16 before P V, bf16 output.  How it computes it is different:
//
//   * one CTA handles one work item = (request, KV head, block of query tokens); the
//     MMA's 128 rows are (token, q head of the group) pairs, so the K/V tile is read
//     once for the whole GQA group (the reference re-reads it per q head in prefill and
//     uses `group` of 64 rows in decode);
//   * S = Q K^T lands in TMEM, double-buffered (2 x 128 columns); in the 32x32b TMEM
//     layout a thread owns one query row with all its columns, so the online softmax
//     needs no shuffles; P goes to shared memory (double-buffered) as a K-major bf16
//     operand;
//   * O = sum over tiles of P V accumulates in a third TMEM region across the whole item
//     (tcgen05.mma with accumulate); a row is rescaled in TMEM (tcgen05.ld / st) only in
//     a tile where its running maximum grows, which after the first tiles is rare, so the
//     softmax threads normally never wait for the P V product;
//   * V is used in place from the cache layout as an MN-major B operand (keys are the
//     contraction dimension), so no transposed copy of V exists anywhere;
//   * the page size is a parameter (16 and 64 are tested); pages of one 128-key tile
//     are fetched by parallel lanes of the producer warp.
//
// Warp roles (192 threads): warp 0 TMA producer, warp 1 TMEM owner + MMA issue,
// warps 2..5 softmax / output (TMEM lane quadrant = warp % 4).  Every wait is
// bounded; a timeout raises the status word and the CTA leaves, freeing its TMEM.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kernels.h"
#include "ptx.cuh"

namespace mf {

constexpr int kAttnThreads = 192;
constexpr int kHeadDim = 128;
constexpr int kKeysPerTile = 128;
constexpr int kHalfBytes = 128 * 128;            // 128 rows x 64 bf16: one swizzle atom column, 16 KB
constexpr int kTileBytes = 2 * kHalfBytes;       // 128 x 128 bf16
constexpr int kAttnSmemBytes = kTileBytes * 7 + 1024;   // Q, K x2, V x2, P x2
constexpr int kAttnTmemCols = 512;               // S x2 (256) + O (128), allocated as a power of two
constexpr unsigned long long kAttnWaitNs = 4000000000ull;

// Diagnostics: phase times of work item 0's softmax warp 2, lane 0 (cycles summed over the
// item's KV tiles): [0] wait for S, [1] max pass, [2] exp + P store, [3] rescale of O
// (tiles where a maximum grew), [4] final wait for O, [5] tiles, [6] total ns.  Written when AttnParams::pad is nonzero.
__device__ unsigned long long g_attn_trace[8];

struct AttnShared {
  uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], p_full[2], o_full[2];
  uint32_t tmem_base;
  int abort_flag;
};

// K-major SW128 descriptor of a 128-row tile with two 64-element column halves;
// step = one of the eight 16-element K steps.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_addr, int step) {
  return umma_desc_sw128(tile_addr + (step >> 2) * kHalfBytes + (step & 3) * 32);
}

// MN-major SW128 descriptor of V: rows are keys (the K dimension), 128 bytes = 64 d
// elements per row, eight-key groups 1024 bytes apart (SBO), the second d half one
// 16 KB half-tile further (LBO).  step = one of the eight 16-key K steps.
__device__ __forceinline__ uint64_t desc_v_mnmajor(uint32_t tile_addr, int step) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>(((tile_addr + step * 2048) & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(kHalfBytes >> 4) << 16;   // leading byte offset: next 64 d elements
  d |= static_cast<uint64_t>(1024u >> 4) << 32;        // stride byte offset: next 8 keys
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// 2^x by the special-function unit (one instruction; the scores are already scaled
// into the exp2 domain, as in the reference's tiles).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tma_load_4d(void* smem, const void* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d_plain(void* smem, const void* map, uint64_t* bar, int c0, int c1,
                                                  int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__global__ void __launch_bounds__(kAttnThreads, 1) paged_attention_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ AttnShared sh;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = base;
  uint8_t* sK = base + kTileBytes;          // two stages
  uint8_t* sV = base + 3 * kTileBytes;      // two stages
  uint8_t* sP = base + 5 * kTileBytes;      // two buffers
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sh.abort_flag;
  const AttnItem item = p.items[blockIdx.x];
  const int group = p.group;
  const int rows = item.q_tokens * group;
  // keys this block can see: up to the position of its last query token
  const int kv_end = min(item.kv_len, item.pos0 + item.q_tokens);
  const int n_tiles = (kv_end + kKeysPerTile - 1) / kKeysPerTile;

  if (threadIdx.x == 0) {
    mbar_init(&sh.q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh.k_full[i], 1);
      mbar_init(&sh.v_full[i], 1);
      mbar_init(&sh.k_empty[i], 1);
      mbar_init(&sh.v_empty[i], 1);
      mbar_init(&sh.s_full[i], 1);
      mbar_init(&sh.p_full[i], 128);
      mbar_init(&sh.o_full[i], 1);   // P V of tile j completes phase j / 2 of o_full[j % 2]
    }
    sh.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh.tmem_base, kAttnTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sh.tmem_base;
  const uint32_t tmem_o = tmem_base + 256;   // S buffers at columns 0 and 128

  if (warp == 0) {
    // --------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(&sh.q_full, 2u * p.q_box_rows * 128u);
      tma_load_3d_plain(sQ, &p.q_map, &sh.q_full, 0, item.kv_head * group, item.q_row0);
      tma_load_3d_plain(sQ + kHalfBytes, &p.q_map, &sh.q_full, 64, item.kv_head * group, item.q_row0);
    }
    const int pages_per_tile = kKeysPerTile / p.page;
    const int page_bytes = p.page * 128;   // one d half of one page
    const int last_page = (kv_end - 1) / p.page;
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j & 1;
      const uint32_t prev = ((j >> 1) - 1) & 1;
      if (j >= 2 && !mbar_wait_bounded(&sh.k_empty[s], prev, abort_flag, kAttnWaitNs)) break;
      if (lane == 0) mbar_arrive_expect_tx(&sh.k_full[s], kTileBytes);
      __syncwarp();
      int page_id = 0;
      if (lane < pages_per_tile) {
        // pages past the visible range repeat the last visible page; their keys are masked
        const int pg = min(j * pages_per_tile + lane, last_page);
        page_id = p.block_table[static_cast<size_t>(item.req) * p.bt_stride + pg];
        uint8_t* k = sK + s * kTileBytes + lane * page_bytes;
        tma_load_4d(k, &p.k_map, &sh.k_full[s], 0, item.kv_head, 0, page_id);
        tma_load_4d(k + kHalfBytes, &p.k_map, &sh.k_full[s], 64, item.kv_head, 0, page_id);
      }
      if (j >= 2 && !mbar_wait_bounded(&sh.v_empty[s], prev, abort_flag, kAttnWaitNs)) break;
      if (lane == 0) mbar_arrive_expect_tx(&sh.v_full[s], kTileBytes);
      __syncwarp();
      if (lane < pages_per_tile) {
        uint8_t* v = sV + s * kTileBytes + lane * page_bytes;
        tma_load_4d(v, &p.v_map, &sh.v_full[s], 0, item.kv_head, 0, page_id);
        tma_load_4d(v + kHalfBytes, &p.v_map, &sh.v_full[s], 64, item.kv_head, 0, page_id);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issue
    if (lane == 0) {
      // S = Q K^T: both K-major; O += P V: A K-major, B (V) MN-major
      const uint32_t idesc_s = umma_idesc_bf16(128, 128);
      const uint32_t idesc_o = umma_idesc_bf16(128, 128) | (1u << 16);
      const uint32_t q_addr = smem_u32(sQ);
      bool ok = mbar_wait_bounded(&sh.q_full, 0, abort_flag, kAttnWaitNs);
      auto mma_s = [&](int j) {
        const int s = j & 1;
        if (!mbar_wait_bounded(&sh.k_full[s], (j >> 1) & 1, abort_flag, kAttnWaitNs)) return false;
        // S[s] is free once the softmax threads have turned tile j - 2 into P
        if (j >= 2 && !mbar_wait_bounded(&sh.p_full[s], ((j >> 1) - 1) & 1, abort_flag, kAttnWaitNs)) return false;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(sK + s * kTileBytes);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          umma_bf16(tmem_base + s * 128, desc_kmajor(q_addr, i), desc_kmajor(k_addr, i), idesc_s, i != 0);
        umma_commit(&sh.s_full[s]);
        umma_commit(&sh.k_empty[s]);
        return true;
      };
      if (ok && n_tiles > 0) ok = mma_s(0);
      if (ok && n_tiles > 1) ok = mma_s(1);
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int s = j & 1;
        if (!mbar_wait_bounded(&sh.v_full[s], (j >> 1) & 1, abort_flag, kAttnWaitNs)) break;
        if (!mbar_wait_bounded(&sh.p_full[s], (j >> 1) & 1, abort_flag, kAttnWaitNs)) break;
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(sV + s * kTileBytes), p_addr = smem_u32(sP + s * kTileBytes);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          umma_bf16(tmem_o, desc_kmajor(p_addr, i), desc_v_mnmajor(v_addr, i), idesc_o, (j | i) != 0);
        umma_commit(&sh.o_full[s]);
        umma_commit(&sh.v_empty[s]);
        if (j + 2 < n_tiles && !mma_s(j + 2)) break;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------ softmax / output
    const int quad = warp & 3;
    const int r = quad * 32 + lane;              // query row = TMEM lane
    const bool row_ok = r < rows;
    const int token = r / group, head = item.kv_head * group + r % group;
    const int qpos = item.pos0 + token;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    float m = -1e30f, l = 0.f;
    bool ok = true;
    const bool tr = p.pad && blockIdx.x == 0 && warp == 2 && lane == 0;
    long long tc[5] = {0, 0, 0, 0, 0}, t_prev = clock64();
    const unsigned long long t_begin = globaltimer_ns();
    auto lap = [&](int i) {
      if (tr) {
        const long long now = clock64();
        tc[i] += now - t_prev;
        t_prev = now;
      }
    };
    for (int j = 0; ok && j < n_tiles; ++j) {
      const int s = j & 1;
      if (!mbar_wait_bounded(&sh.s_full[s], (j >> 1) & 1, abort_flag, kAttnWaitNs)) { ok = false; break; }
      tc_fence_after_sync();
      lap(0);
      const uint32_t tmem_s = tmem_base + s * 128 + lane_off;
      const int key0 = j * kKeysPerTile;
      // keys this row may attend to inside the tile: [0, lim)
      const int lim = row_ok ? min(min(item.kv_len, qpos + 1) - key0, kKeysPerTile) : 0;
      // pass 1: row maximum of the scaled scores
      float mx = m;
#pragma unroll
      for (int c0 = 0; c0 < kKeysPerTile; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_s + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (c0 + i < lim) mx = fmaxf(mx, __uint_as_float(v[i]) * p.scale_log2);
      }
      lap(1);
      // a row whose maximum grew rescales its part of O in TMEM, once the previous P V has landed
      if (j > 0 && __any_sync(0xffffffffu, mx > m)) {
        if (!mbar_wait_bounded(&sh.o_full[s ^ 1], ((j - 1) >> 1) & 1, abort_flag, kAttnWaitNs)) { ok = false; break; }
        tc_fence_after_sync();
        const float alpha = fast_exp2(m - mx);
#pragma unroll
        for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_o + lane_off + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x32(tmem_o + lane_off + c0, v);
        }
        tmem_st_wait();
        l *= alpha;
      } else if (j == 0) {
        l = 0.f;
      }
      m = mx;
      lap(3);
      // the P buffer is free once P V of tile j - 2 has completed
      if (j >= 2 && !mbar_wait_bounded(&sh.o_full[s], ((j >> 1) - 1) & 1, abort_flag, kAttnWaitNs)) { ok = false; break; }
      const float neg_mx = -mx;
      // pass 2: P = exp2(s - max) as bf16 into shared memory (K-major, 128-byte swizzle); row sum of the rounded P
      float sum = 0.f;
      uint8_t* p_tile = sP + s * kTileBytes;
#pragma unroll
      for (int c0 = 0; c0 < kKeysPerTile; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_s + c0, v);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = c0 + i < lim ? fast_exp2(fmaf(__uint_as_float(v[i]), p.scale_log2, neg_mx)) : 0.f;
          const float p1 = c0 + i + 1 < lim ? fast_exp2(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, neg_mx)) : 0.f;
          const __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
          sum += __bfloat162float(b.x) + __bfloat162float(b.y);
          packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&b);
        }
        // 32 keys = four 16-byte chunks of this row in key half c0 / 64
        uint8_t* row_base = p_tile + (c0 >> 6) * kHalfBytes + r * 128;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = ((c0 & 63) >> 3) + q;
          *reinterpret_cast<uint4*>(row_base + ((chunk ^ (r & 7)) << 4)) =
              make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        }
      }
      l += sum;
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(&sh.p_full[s]);
      lap(2);
    }
    if (ok && n_tiles > 0) ok = mbar_wait_bounded(&sh.o_full[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, abort_flag, kAttnWaitNs);
    tc_fence_after_sync();
    lap(4);
    if (tr) {
      for (int i = 0; i < 5; ++i) g_attn_trace[i] = tc[i];
      g_attn_trace[5] = n_tiles;
      g_attn_trace[6] = globaltimer_ns() - t_begin;
    }
    if (ok) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(item.q_row0 + token) * p.hq + head) * kHeadDim);
#pragma unroll
      for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
        uint32_t v[32];
        if (n_tiles > 0) {
          tmem_ld_32x32(tmem_o + lane_off + c0, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0;
        }
        if (row_ok) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            __nv_bfloat162 h[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
              h[i] = __floats2bfloat162_rn(__uint_as_float(v[8 * c + 2 * i]) * inv, __uint_as_float(v[8 * c + 2 * i + 1]) * inv);
            dst[(c0 >> 3) + c] = *reinterpret_cast<const uint4*>(h);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && sh.abort_flag) atomicOr(p.status, kErrWaitTimeout);
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kAttnTmemCols);
  }
}

cudaError_t read_attention_trace(unsigned long long out[8]) {
  return cudaMemcpyFromSymbol(out, g_attn_trace, sizeof(unsigned long long) * 8);
}

cudaError_t launch_attention(const AttnParams& p, cudaStream_t stream) {
  if (p.n_items == 0) return cudaSuccess;
  static bool attr = false;
  if (!attr) {
    const cudaError_t err =
        cudaFuncSetAttribute(paged_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmemBytes);
    if (err != cudaSuccess) return err;
    attr = true;
  }
  paged_attention_kernel<<<p.n_items, kAttnThreads, kAttnSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace mf
