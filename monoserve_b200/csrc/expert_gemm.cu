// Grouped SwiGLU expert GEMM for sm_100a: tcgen05.mma with TMEM accumulators,
// operands staged by TMA, one persistent CTA per SM.
//
// Operand roles follow the reference's GEMM tile (csrc/fabric/tiles/gemm.cuh:1-18,
// 133-346): the WEIGHT slice is the MMA's M operand (128 output features) and
// the expert's packed ACTIVATION rows are the N operand (16..128 tokens), so a
// decode batch of a few tokens per expert still fills a full-height MMA.  Both
// operands are K-major with the 128-byte swizzle; one K step is 64 elements.
//
// Two modes (csrc/fabric/model_types.h:29-35 epilogues kEpiSiluMul / kEpiWeightedAdd):
//   w13: two accumulators per tile, gate rows [f, f+128) and up rows
//        [I+f, I+f+128) of the same expert, sharing the activation operand;
//        epilogue h[m][f] = bf16(silu(g) * u).
//   w2 : one accumulator; the epilogue stores the fp32 rows y[m][n] of every
//        routed pair.  The weighted un-permute happens in the combine kernel in
//        pick order, which makes the layer output deterministic (the reference
//        adds with atomics in arrival order).
//
// Warp roles (192 threads): warp 0 = tile claim + TMA producer, warp 1 = TMEM
// owner + MMA issue, warps 2..5 = epilogue (TMEM lane quadrant = warp % 4).
// Accumulators are double-buffered in TMEM, so the epilogue of tile i overlaps
// the loads and MMAs of tile i+1.
//
// Link credits (csrc/fabric/runtime.cuh:415-423,451-485): tiles whose weights
// are in pinned host memory sit in a separate queue and are taken only by a
// CTA that holds one of `cap` slots; the other CTAs work on HBM tiles.
//
// Every wait is bounded: when one runs out the CTA raises kErrWaitTimeout in
// the status word and leaves through the common exit, freeing its TMEM.
#include <cuda_bf16.h>

#include "kernels.h"
#include "ptx.cuh"

namespace mf {

constexpr int kGemmThreads = 192;
constexpr int kBlockK = 64;                       // elements per K step (128 bytes of bf16)
constexpr int kSliceBytes = 128 * kBlockK * 2;    // one 128-row operand tile: 16 KB
constexpr int kMaxN = 128;
constexpr int kTmemCols = 512;
constexpr unsigned long long kWaitBudgetNs = 4000000000ull;   // 4 s

template <int MODE>
struct GemmCfg {
  static constexpr int kABytes = MODE == kGemmModeW13 ? 2 * kSliceBytes : kSliceBytes;
  static constexpr int kBBytes = kMaxN * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = MODE == kGemmModeW13 ? 4 : 6;
  static constexpr int kAccCols = MODE == kGemmModeW13 ? 256 : 128;   // TMEM columns per buffer
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;
};

struct GemmShared {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tile_ready[2];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  GemmTile tile[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ bool try_acquire_slot(int* slots, int cap) {
  int cur = *reinterpret_cast<volatile int*>(slots);
  while (cur < cap) {
    const int seen = atomicCAS(slots, cur, cur + 1);
    if (seen == cur) return true;
    cur = seen;
  }
  return false;
}

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.f + __expf(-g)) * u; }

template <int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1) expert_gemm_kernel(const __grid_constant__ GemmParams p) {
  using Cfg = GemmCfg<MODE>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ GemmShared sh;
  uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sh.abort_flag;

  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::kStages; ++i) {
      mbar_init(&sh.full[i], 1);
      mbar_init(&sh.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh.tile_ready[i], 1);
      mbar_init(&sh.acc_full[i], 1);
      mbar_init(&sh.acc_empty[i], 4);
    }
    sh.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sh.tmem_base;
  const int k_tiles = p.k_tiles;

  if (warp == 0) {
    // ------------------------------------------------ claim + TMA producer
    if (lane == 0) {
      prefetch_tensormap(&p.w_map[0]);
      prefetch_tensormap(&p.w_map[1]);
      GemmQueues* q = p.q;
      const int n_link = q->n_tiles[p.phase][0], n_hbm = q->n_tiles[p.phase][1];
      const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
      bool have_slot = false, link_left = n_link > 0, hbm_left = n_hbm > 0;
      int stage = 0;
      uint32_t phase = 0;
      for (int it = 0;; ++it) {
        const int buf = it & 1;
        if (!mbar_wait_bounded(&sh.acc_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag, kWaitBudgetNs)) break;
        const GemmTile* t = nullptr;
        if (link_left) {
          if (!have_slot) have_slot = try_acquire_slot(&q->slots[p.phase], p.cap);
          if (have_slot) {
            const int i = atomicAdd(&q->head[p.phase][0], 1);
            if (i < n_link) {
              t = p.tiles[0] + i;
            } else {
              link_left = false;
              atomicSub(&q->slots[p.phase], 1);
              have_slot = false;
            }
          }
        }
        if (!t && hbm_left) {
          const int i = atomicAdd(&q->head[p.phase][1], 1);
          if (i < n_hbm) t = p.tiles[1] + i; else hbm_left = false;
        }
        if (!t) {
          // Nothing this CTA may take: either both queues are drained, or the
          // remaining link tiles belong to the CTAs that hold the slots.
          sh.tile[buf].n = -1;
          mbar_arrive(&sh.tile_ready[buf]);
          break;
        }
        const GemmTile tile = *t;
        sh.tile[buf] = tile;
        mbar_arrive(&sh.tile_ready[buf]);
        int box = 0;
        while ((16 << box) < tile.n) ++box;
        const CUtensorMap* wmap = &p.w_map[tile.tier];
        const CUtensorMap* xmap = &p.act_map[box];
        const uint32_t bytes = Cfg::kABytes + tile.n * kBlockK * 2;
        bool ok = true;
        for (int kt = 0; kt < k_tiles; ++kt) {
          if (!mbar_wait_bounded(&sh.empty[stage], phase ^ 1, abort_flag, kWaitBudgetNs)) { ok = false; break; }
          uint8_t* a = stages + stage * Cfg::kStageBytes;
          uint8_t* b = a + Cfg::kABytes;
          mbar_arrive_expect_tx(&sh.full[stage], bytes);
          tma_load_3d(a, wmap, &sh.full[stage], kt * kBlockK, tile.w_row0, tile.z, pol_w);
          if (MODE == kGemmModeW13)
            tma_load_3d(a + kSliceBytes, wmap, &sh.full[stage], kt * kBlockK, p.up_offset + tile.w_row0,
                        tile.z, pol_w);
          tma_load_2d(b, xmap, &sh.full[stage], kt * kBlockK, tile.act_row0, pol_x);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
      }
      if (have_slot) atomicSub(&q->slots[p.phase], 1);
      if (*abort_flag) {
        // Let copies that are still in flight land before the block retires.
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 50000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issue
    int stage = 0;
    uint32_t phase = 0;
    for (int it = 0;; ++it) {
      const int buf = it & 1;
      const uint32_t use_parity = (it >> 1) & 1;
      if (!mbar_wait_bounded(&sh.tile_ready[buf], use_parity, abort_flag, kWaitBudgetNs)) break;
      const int n = sh.tile[buf].n;
      if (n < 0) break;
      if (!mbar_wait_bounded(&sh.acc_empty[buf], use_parity ^ 1, abort_flag, kWaitBudgetNs)) break;
      tc_fence_after_sync();
      const uint32_t idesc = umma_idesc_bf16(128, n);
      const uint32_t acc = tmem_base + buf * Cfg::kAccCols;
      bool ok = true;
      for (int kt = 0; kt < k_tiles; ++kt) {
        if (!mbar_wait_bounded(&sh.full[stage], phase, abort_flag, kWaitBudgetNs)) { ok = false; break; }
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t a = smem_u32(stages + stage * Cfg::kStageBytes);
          const uint32_t b = a + Cfg::kABytes;
          const uint64_t da = umma_desc_sw128(a), db = umma_desc_sw128(b);
          const uint64_t du = umma_desc_sw128(a + kSliceBytes);
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) {
            const uint32_t accum = (kt | k) != 0;
            umma_bf16(acc, da + 2 * k, db + 2 * k, idesc, accum);
            if (MODE == kGemmModeW13) umma_bf16(acc + kMaxN, du + 2 * k, db + 2 * k, idesc, accum);
          }
          umma_commit(&sh.empty[stage]);
        }
        __syncwarp();
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      if (lane == 0) umma_commit(&sh.acc_full[buf]);
      __syncwarp();
    }
  } else {
    // -------------------------------------------------------------- epilogue
    const int quad = warp & 3;
    for (int it = 0;; ++it) {
      const int buf = it & 1;
      const uint32_t use_parity = (it >> 1) & 1;
      if (!mbar_wait_bounded(&sh.tile_ready[buf], use_parity, abort_flag, kWaitBudgetNs)) break;
      const GemmTile tile = sh.tile[buf];
      if (tile.n < 0) break;
      if (!mbar_wait_bounded(&sh.acc_full[buf], use_parity, abort_flag, kWaitBudgetNs)) break;
      tc_fence_after_sync();
      const int f = tile.w_row0 + quad * 32 + lane;   // output feature of this thread
      const bool f_ok = f < p.n_limit;
      const uint32_t tacc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * Cfg::kAccCols;
      float sg = 1.f, su = 1.f;
      if (p.scale) {
        const float* sc = p.scale + static_cast<size_t>(tile.expert) * p.scale_ld;
        if (f_ok) {
          sg = sc[f];
          if (MODE == kGemmModeW13) su = sc[p.up_offset + f];
        }
      }
      for (int c0 = 0; c0 < tile.n; c0 += 32) {
        uint32_t g[32], u[32];
        if (tile.n - c0 >= 32) {
          tmem_ld_32x32(tacc + c0, g);
          if (MODE == kGemmModeW13) tmem_ld_32x32(tacc + kMaxN + c0, u);
        } else {
          uint32_t g16[16], u16[16];
          tmem_ld_32x16(tacc + c0, g16);
          if (MODE == kGemmModeW13) tmem_ld_32x16(tacc + kMaxN + c0, u16);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            g[j] = g16[j];
            if (MODE == kGemmModeW13) u[j] = u16[j];
            g[16 + j] = 0;
            u[16 + j] = 0;
          }
        }
        tmem_ld_wait();
        const int m_hi = min(32, tile.rows - c0);
        if (MODE == kGemmModeW13) {
          __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) +
                               static_cast<size_t>(tile.act_row0 + c0) * p.ld_out + f;
          if (f_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (j < m_hi) {
                const float h = silu_mul(__uint_as_float(g[j]) * sg, __uint_as_float(u[j]) * su);
                out[static_cast<size_t>(j) * p.ld_out] = __float2bfloat16(h);
              }
            }
          }
        } else {
          float* out = reinterpret_cast<float*>(p.out) + static_cast<size_t>(tile.act_row0 + c0) * p.ld_out + f;
          if (f_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < m_hi) out[static_cast<size_t>(j) * p.ld_out] = __uint_as_float(g[j]) * sg;
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.acc_empty[buf]);
    }
  }

  // ------------------------------------------------------------ common exit
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && sh.abort_flag) atomicOr(p.status, kErrWaitTimeout);
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

cudaError_t launch_expert_gemm(const GemmParams& p, int mode, int ctas, cudaStream_t stream) {
  cudaError_t err;
  if (mode == kGemmModeW13) {
    static bool attr13 = false;
    if (!attr13) {
      err = cudaFuncSetAttribute(expert_gemm_kernel<kGemmModeW13>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 GemmCfg<kGemmModeW13>::kSmemBytes);
      if (err != cudaSuccess) return err;
      attr13 = true;
    }
    expert_gemm_kernel<kGemmModeW13><<<ctas, kGemmThreads, GemmCfg<kGemmModeW13>::kSmemBytes, stream>>>(p);
  } else {
    static bool attr2 = false;
    if (!attr2) {
      err = cudaFuncSetAttribute(expert_gemm_kernel<kGemmModeW2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 GemmCfg<kGemmModeW2>::kSmemBytes);
      if (err != cudaSuccess) return err;
      attr2 = true;
    }
    expert_gemm_kernel<kGemmModeW2><<<ctas, kGemmThreads, GemmCfg<kGemmModeW2>::kSmemBytes, stream>>>(p);
  }
  return cudaGetLastError();
}

}  // namespace mf
