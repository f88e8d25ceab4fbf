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
// scheduler waits (bounded) for the count before it hands a w2 tile to the
// producer.  Tiles are claimed in queue order, so whatever a waiting CTA waits
// for has already been claimed by a CTA that is running: no deadlock.
//
// Warp roles (224 threads):
//   warp 6  scheduler: claims tiles (link credits, queue heads), reads the tile
//           record, checks the row-block dependency, and fills a 4-deep ring of
//           work records, running ahead of the data path so that its global-memory
//           round trips never stall the copies;
//   warp 0  TMA producer;  warp 1  TMEM owner + MMA issue;  warps 2..5  epilogue.
// Accumulators are double-buffered in TMEM so the epilogue of tile i overlaps the
// loads and MMAs of tile i+1, across tile and phase boundaries.
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

constexpr int kGemmThreads = 224;
constexpr int kGemmThreadsFp8 = 352;   // + four converter warps (7..10)
constexpr int kWorkSlots = 4;

struct GemmShared {
  GemmBarriers bar;
  uint64_t work_full[kWorkSlots];    // scheduler -> producer, MMA, epilogue
  uint64_t work_empty[kWorkSlots];   // 6 arrivals: producer, MMA, four epilogue warps
  GemmWork work[kWorkSlots];
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

// Debug trace of CTA 0: slot [role][it][event] <- device time.
// role 0 scheduler, 1 producer, 2 MMA, 3 epilogue warp 2.
__device__ __forceinline__ void trace_ev(const GemmParams& p, int role, int it, int ev) {
  if (p.trace && blockIdx.x == 0 && it < 32 && (threadIdx.x & 31) == 0)
    p.trace[(role * 32 + it) * 4 + ev] = globaltimer_ns();
}

template <bool FP8>
__global__ void __launch_bounds__(FP8 ? kGemmThreadsFp8 : kGemmThreads, 1)
    expert_gemm_kernel(const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ GemmShared sh;
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sh.abort_flag;

  if (threadIdx.x == 0) {
    gemm_barriers_init(sh.bar);
    for (int i = 0; i < kWorkSlots; ++i) {
      mbar_init(&sh.work_full[i], 1);
      mbar_init(&sh.work_empty[i], FP8 ? 10 : 6);
    }
    sh.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  chain_release();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sh.tmem_base;
  chain_wait();   // the tile lists and the packed rows come from the kernels before this one

  if (warp == 6) {
    // ------------------------------------------------------------ scheduler
    if (lane == 0) {
      GemmQueues* q = p.q;
      const int n_link = q->n_tiles[0], n_hbm = q->n_tiles[1], need = q->need;
      bool have_slot = false, link_left = n_link > 0, hbm_left = n_hbm > 0;
      for (int it = 0;; ++it) {
        const int slot = it % kWorkSlots;
        trace_ev(p, 0, it, 0);
        if (!mbar_wait_bounded(&sh.work_empty[slot], ((it / kWorkSlots) & 1) ^ 1, abort_flag, kWaitBudgetNs)) break;
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
        GemmWork& w = sh.work[slot];
        if (!t) {
          // Nothing this CTA may take: both queues are drained, or the remaining
          // link tiles belong to the CTAs that hold the slots.
          w.valid = 0;
          mbar_arrive(&sh.work_full[slot]);
          break;
        }
        const GemmTile tile = *t;
        trace_ev(p, 0, it, 1);
        const int tier = tile.tier_phase & 0xff, phase = tile.tier_phase >> 8;
        const GemmPhaseParams& ph = p.ph[phase];
        int box = 0;
        while ((16 << box) < tile.n) ++box;
        const bool packed = phase == 0 && ph.packed[tier];
        w.a_map = (phase == 0 && !packed) ? &ph.w_map[tier] : &ph.w_map_big[tier];
        w.b_map = &ph.act_map[box];
        w.out = ph.out;
        w.scale = ph.scale ? ph.scale + static_cast<size_t>(tile.expert) * ph.scale_ld : nullptr;
        w.w_fp8 = ph.w_fp8;
        w.fetch = 0;
        w.bias = nullptr;
        w.residual = nullptr;
        w.pair_token = nullptr;
        w.pair_weight = nullptr;
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
        w.a_packed = packed;
        w.block = phase == 0 ? tile.block : -1;
        if (phase == 1) {
          // h of this row block must be complete before TMA reads it
          const uint32_t* flag = reinterpret_cast<const uint32_t*>(p.done + tile.block);
          bool ok = true;
          if (ld_acquire_gpu(flag) < static_cast<uint32_t>(need)) {
            const unsigned long long t0 = globaltimer_ns();
            while (ld_acquire_gpu(flag) < static_cast<uint32_t>(need)) {
              __nanosleep(64);
              if (*abort_flag || globaltimer_ns() - t0 > kWaitBudgetNs) {
                *abort_flag = 1;
                ok = false;
                break;
              }
            }
          }
          if (!ok) break;
          fence_proxy_async_all();
        }
        trace_ev(p, 0, it, 2);
        mbar_arrive(&sh.work_full[slot]);
      }
      if (have_slot) atomicSub(&q->slots, 1);
    }
  } else if (warp == 0) {
    // --------------------------------------------------------- TMA producer
    const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
    GemmPipe pipe;
    GemmInflight inflight;
    for (int it = 0;; ++it) {
      const int slot = it % kWorkSlots;
      if (!mbar_wait_bounded(&sh.work_full[slot], (it / kWorkSlots) & 1, abort_flag, kWaitBudgetNs)) break;
      if (!sh.work[slot].valid) break;
      trace_ev(p, 1, it, 0);
      if (!gemm_produce<false>(sh.work[slot], ring, sh.bar, pipe, inflight, abort_flag, pol_w, pol_x)) break;
      trace_ev(p, 1, it, 1);
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.work_empty[slot]);
    }
    if (lane == 0 && *abort_flag) {
      // Let copies that are still in flight land before the block retires.
      const unsigned long long t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 50000ull) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issue
    GemmPipe pipe;
    // with the trace on, every CTA also leaves a summary at trace[1024 + 8 * CTA]: entry, first and last
    // tile of the MMA warp (device time), tiles, w2 tiles, cycles spent waiting for operands / issuing
    unsigned long long* own = p.trace ? p.trace + 1024 + 8 * blockIdx.x : nullptr;
    long long sum_wait = 0, sum_issue = 0, sum_acc = 0, sum_work = 0;
    int n_w2 = 0;
    if (own && lane == 0) own[0] = globaltimer_ns();
    const long long c_begin = own ? clock64() : 0;
    for (int it = 0;; ++it) {
      const int slot = it % kWorkSlots, buf = it & 1;
      const long long tw = own ? clock64() : 0;
      if (!mbar_wait_bounded(&sh.work_full[slot], (it / kWorkSlots) & 1, abort_flag, kWaitBudgetNs)) break;
      if (own) sum_work += clock64() - tw;
      if (!sh.work[slot].valid) break;
      trace_ev(p, 2, it, 0);
      if (own && lane == 0 && it == 0) own[1] = globaltimer_ns();
      long long waited[3] = {0, 0, 0};
      if (!gemm_mma<false>(sh.work[slot], ring, sh.bar, pipe, tmem_base, buf, (it >> 1) & 1, abort_flag,
                           p.trace ? waited : nullptr))
        break;
      trace_ev(p, 2, it, 1);
      if (own && lane == 0) {
        sum_wait += waited[0];
        sum_issue += waited[1];
        sum_acc += waited[2];
        own[7] = sum_acc;
        n_w2 += sh.work[slot].block < 0;
        own[2] = globaltimer_ns();
        own[3] = it + 1;
        own[4] = static_cast<unsigned long long>(n_w2) | (static_cast<unsigned long long>(clock64() - c_begin) << 16);
        own[5] = sum_wait;
        own[6] = sum_issue + (static_cast<unsigned long long>(sum_work) << 32);
      }
      if (lane == 0) {
        mbar_arrive(&sh.work_empty[slot]);
        if (p.trace && blockIdx.x == 0 && it < 32) {
          p.trace[(2 * 32 + it) * 4 + 2] = sh.work[slot].n;
          p.trace[(2 * 32 + it) * 4 + 3] = waited[0];
          p.trace[(4 * 32 + it) * 4 + 0] = waited[1];
        }
      }
    }
  } else if (FP8 && warp >= 7) {
    // ------------------------------------------------- e4m3 -> bf16 converters
    GemmPipe pipe;
    const int row = threadIdx.x - 7 * 32;
    for (int it = 0;; ++it) {
      const int slot = it % kWorkSlots;
      if (!mbar_wait_bounded(&sh.work_full[slot], (it / kWorkSlots) & 1, abort_flag, kWaitBudgetNs)) break;
      if (!sh.work[slot].valid) break;
      if (!gemm_convert(sh.work[slot], ring, sh.bar, pipe, row, abort_flag)) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.work_empty[slot]);
    }
  } else {
    // -------------------------------------------------------------- epilogue
    for (int it = 0;; ++it) {
      const int slot = it % kWorkSlots, buf = it & 1;
      if (!mbar_wait_bounded(&sh.work_full[slot], (it / kWorkSlots) & 1, abort_flag, kWaitBudgetNs)) break;
      if (!sh.work[slot].valid) break;
      const GemmWork w = sh.work[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.work_empty[slot]);   // the record is copied: the slot may be refilled
      if (warp == 2) trace_ev(p, 3, it, 0);
      unsigned long long* seen =
          (p.trace && blockIdx.x == 0 && warp == 2 && it < 32) ? &p.trace[(3 * 32 + it) * 4 + 3] : nullptr;
      if (!gemm_epilogue<false>(w, sh.bar, tmem_base, buf, (it >> 1) & 1, abort_flag, seen)) break;
      if (warp == 2) trace_ev(p, 3, it, 1);
      if (w.block >= 0) {
        // publish this warp's part of h, then count it into the row block
        __threadfence();
        fence_proxy_async_all();
        __syncwarp();
        if (lane == 0) atomicAdd(p.done + w.block, 1);
      }
      if (warp == 2) trace_ev(p, 3, it, 2);
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

// Copy w13 stacks [n][2I][H] into the packed SwiGLU order: for every group of 16
// features, 16 gate rows then the 16 matching up rows, so that a tile of 64
// features is one contiguous block of 128 rows.  One warp per row.
__global__ void __launch_bounds__(256) pack_w13_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                       long long rows_total, int I, int row_vec) {
  const long long r = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows_total) return;
  const int lane = threadIdx.x & 31;
  const long long z = r / (2 * I);
  const int in_row = static_cast<int>(r % (2 * I));
  const int up = in_row >= I, f = up ? in_row - I : in_row;
  const long long out_row = z * 2 * I + 32LL * (f / 16) + 16 * up + (f % 16);
  const uint4* s = src + r * row_vec;
  uint4* d = dst + out_row * row_vec;
  for (int c = lane; c < row_vec; c += 32) d[c] = ld_nc_stream16(s + c);
}

cudaError_t launch_pack_w13(const void* src, void* dst, int n, int I, int H, int elt_bytes, cudaStream_t stream) {
  const long long rows = static_cast<long long>(n) * 2 * I;
  if (rows == 0) return cudaSuccess;
  const int row_vec = H * elt_bytes / 16;
  pack_w13_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, stream>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), rows, I, row_vec);
  return cudaGetLastError();
}

cudaError_t launch_expert_gemm(const GemmParams& p, int ctas, cudaStream_t stream) {
  static PerDeviceOnce once;
  const cudaError_t attr_err = once.run([] {
    cudaError_t err = cudaFuncSetAttribute(expert_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kGemmSmemBytes);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(expert_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kGemmSmemBytes);
    return err;
  });
  if (attr_err != cudaSuccess) return attr_err;
  if (p.ph[0].w_fp8) return launch_chained(expert_gemm_kernel<true>, ctas, kGemmThreadsFp8, kGemmSmemBytes, stream, p);
  return launch_chained(expert_gemm_kernel<false>, ctas, kGemmThreads, kGemmSmemBytes, stream, p);
}

}  // namespace mf
