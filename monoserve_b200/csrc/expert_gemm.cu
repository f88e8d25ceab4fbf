// Grouped SwiGLU expert GEMM of one MoE layer as ONE persistent launch
// (1 CTA per SM) on the tile functions of gemm_core.cuh.
//
// Work comes from two queues the plan kernel filled, one per weight tier (host
// link / HBM); each holds the layer's w13 tiles followed by its w2 tiles.
//   w13 tile: 64 gate + 64 up rows of one expert x one row block, epilogue
//             h = bf16(silu(g) * u)                       (kEpiSiluMul)
//   w2 tile : 128 output rows x the same row block over h, epilogue stores the
//             fp32 rows y[pos][n] of every routed pair     (kEpiRowsF32)
// A w2 tile may start only when every w13 tile of its row block has stored h:
// the epilogue warps of w13 tiles count into done[block] (release), and the
// producer of a w2 tile waits (bounded) for the count before it issues the first
// load of h.  Tiles are claimed in queue order, so whatever a waiting CTA waits
// for has already been claimed by a CTA that is running: no deadlock.
//
// Warp roles (192 threads): warp 0 = tile claim + TMA producer, warp 1 = TMEM
// owner + MMA issue, warps 2..5 = epilogue.  Accumulators are double-buffered in
// TMEM so the epilogue of tile i overlaps the loads and MMAs of tile i+1, across
// tile and phase boundaries.
//
// Link credits (csrc/fabric/runtime.cuh:415-423,451-485): a CTA takes link
// tiles only while it holds one of `cap` slots; others work on the HBM queue and
// leave when it is drained.
//
// Every wait is bounded; on a timeout the CTA raises kErrWaitTimeout in the
// status word and leaves through the common exit, freeing its TMEM.
#include <cuda_bf16.h>

#include "gemm_core.cuh"
#include "kernels.h"

namespace mf {

constexpr int kGemmThreads = 192;

struct GemmShared {
  GemmBarriers bar;
  uint64_t tile_ready[2];
  GemmWork work[2];
  int block[2];        // row block of the tile in the slot (w13: to count; -1 otherwise)
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

__global__ void __launch_bounds__(kGemmThreads, 1) expert_gemm_kernel(const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ GemmShared sh;
  uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sh.abort_flag;

  if (threadIdx.x == 0) {
    gemm_barriers_init(sh.bar);
    mbar_init(&sh.tile_ready[0], 1);
    mbar_init(&sh.tile_ready[1], 1);
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

  if (warp == 0) {
    // ------------------------------------------------ claim + TMA producer
    if (lane == 0) {
      GemmQueues* q = p.q;
      const int n_link = q->n_tiles[0], n_hbm = q->n_tiles[1], need = q->need;
      const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
      bool have_slot = false, link_left = n_link > 0, hbm_left = n_hbm > 0;
      GemmPipe pipe;
      for (int it = 0;; ++it) {
        const int buf = it & 1;
        if (!mbar_wait_bounded(&sh.bar.acc_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag, kWaitBudgetNs)) break;
        const GemmTile* t = nullptr;
        if (link_left) {
          if (!have_slot) have_slot = try_acquire_slot(&q->slots, p.cap);
          if (have_slot) {
            const int i = atomicAdd(&q->head[0], 1);
            if (i < n_link) {
              t = p.tiles[0] + i;
            } else {
              link_left = false;
              atomicSub(&q->slots, 1);
              have_slot = false;
            }
          }
        }
        if (!t && hbm_left) {
          const int i = atomicAdd(&q->head[1], 1);
          if (i < n_hbm) t = p.tiles[1] + i; else hbm_left = false;
        }
        GemmWork& w = sh.work[buf];
        if (!t) {
          // Nothing this CTA may take: both queues are drained, or the remaining
          // link tiles belong to the CTAs that hold the slots.
          w.valid = 0;
          mbar_arrive(&sh.tile_ready[buf]);
          break;
        }
        const GemmTile tile = *t;
        const GemmPhaseParams& ph = p.ph[tile.phase];
        int box = 0;
        while ((16 << box) < tile.n) ++box;
        w.a_map = &ph.w_map[tile.tier];
        w.b_map = &ph.act_map[box];
        w.out = ph.out;
        w.scale = nullptr;
        w.bias = nullptr;
        w.residual = nullptr;
        w.a_row_lo = tile.w_row0;
        w.a_row_hi = ph.up_offset + tile.w_row0;
        w.a_z = tile.z;
        w.b_row0 = tile.act_row0;
        w.rows = tile.rows;
        w.n = tile.n;
        w.k0 = 0;
        w.k_tiles = ph.k_tiles;
        w.epi = ph.epi;
        w.ld_out = ph.ld_out;
        w.ld_res = 0;
        w.n_limit = ph.n_limit;
        w.valid = 1;
        sh.block[buf] = tile.phase == 0 ? tile.block : -1;
        mbar_arrive(&sh.tile_ready[buf]);
        if (tile.phase == 1) {
          // h of this row block must be complete before TMA reads it
          const int* flag = p.done + tile.block;
          if (ld_acquire_gpu(reinterpret_cast<const uint32_t*>(flag)) < static_cast<uint32_t>(need)) {
            const unsigned long long t0 = globaltimer_ns();
            bool ok = true;
            while (ld_acquire_gpu(reinterpret_cast<const uint32_t*>(flag)) < static_cast<uint32_t>(need)) {
              __nanosleep(64);
              if (*abort_flag || globaltimer_ns() - t0 > kWaitBudgetNs) {
                *abort_flag = 1;
                ok = false;
                break;
              }
            }
            if (!ok) break;
          }
          fence_proxy_async_all();
        }
        if (!gemm_produce(w, stages, sh.bar, pipe, abort_flag, pol_w, pol_x)) break;
      }
      if (have_slot) atomicSub(&q->slots, 1);
      if (*abort_flag) {
        // Let copies that are still in flight land before the block retires.
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 50000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issue
    GemmPipe pipe;
    for (int it = 0;; ++it) {
      const int buf = it & 1;
      const uint32_t parity = (it >> 1) & 1;
      if (!mbar_wait_bounded(&sh.tile_ready[buf], parity, abort_flag, kWaitBudgetNs)) break;
      if (!sh.work[buf].valid) break;
      if (!gemm_mma(sh.work[buf], stages, sh.bar, pipe, tmem_base, buf, parity, abort_flag)) break;
    }
  } else {
    // -------------------------------------------------------------- epilogue
    for (int it = 0;; ++it) {
      const int buf = it & 1;
      const uint32_t parity = (it >> 1) & 1;
      if (!mbar_wait_bounded(&sh.tile_ready[buf], parity, abort_flag, kWaitBudgetNs)) break;
      if (!sh.work[buf].valid) break;
      const int block = sh.block[buf];
      const GemmWork w = sh.work[buf];
      // the slot is released by acc_empty inside gemm_epilogue; publish h first
      if (block >= 0) {
        // run the epilogue body, then count this warp's part of the row block
        if (!gemm_epilogue_body(w, sh.bar, tmem_base, buf, parity, abort_flag)) break;
        __threadfence();
        fence_proxy_async_all();
        __syncwarp();
        if (lane == 0) {
          atomicAdd(p.done + block, 1);
          mbar_arrive(&sh.bar.acc_empty[buf]);
        }
      } else {
        if (!gemm_epilogue(w, sh.bar, tmem_base, buf, parity, abort_flag)) break;
      }
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

cudaError_t launch_expert_gemm(const GemmParams& p, int ctas, cudaStream_t stream) {
  static bool attr = false;
  if (!attr) {
    const cudaError_t err =
        cudaFuncSetAttribute(expert_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes);
    if (err != cudaSuccess) return err;
    attr = true;
  }
  expert_gemm_kernel<<<ctas, kGemmThreads, kGemmSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace mf
