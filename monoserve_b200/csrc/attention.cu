// Paged-KV GQA attention for prefill and decode rows on tcgen05 / TMEM / TMA.
//
// What it computes is the reference's attention tiles (csrc/fabric/tiles/attention.cuh:
// 174-281 prefill, 286-371 decode; AttnArgs csrc/fabric/model_types.h:68-96): causal
// softmax(q k^T / sqrt(D)) v over a paged cache [pages][page][hkv][128] (K and V
// separately), head_dim 128, scores scaled in the exp2 domain, masked keys weight 0,
// P rounded to bf16 before P V, bf16 output.  How it computes it is different:
//
//   * a work item is (request, KV head, block of query tokens); the MMA's 128 rows are
//     (token, q head of the group) pairs, so the K/V tile is read once for the whole GQA
//     group (the reference re-reads it per q head in prefill and uses `group` of 64 rows
//     in decode);
//   * the kernel is persistent: one CTA per SM claims items in list order (the host sorts
//     them longest first) and its producer warp already fetches the next item's Q, K and V
//     while the softmax warps finish the current one, so an item boundary costs neither a
//     CTA launch nor an empty operand ring;
//   * S = Q K^T lands in TMEM, double-buffered (2 x 128 columns); in the 32x32b TMEM
//     layout a thread owns one query row with all its columns, so the online softmax
//     needs no shuffles; P goes to shared memory (double-buffered) as a K-major bf16
//     operand;
//   * the two softmax groups of an item with more than 32 rows take alternate key tiles
//     (group g: tiles g, g + 2, ...), each with its own S buffer, P buffer, running
//     (max, sum) per row and accumulator O[g] = sum over its tiles of P V in TMEM
//     (tcgen05.mma with accumulate), so nothing passes between the groups inside the
//     tile loop and one group's exponentials overlap the other's; S[g] is released as
//     soon as its rows are in registers, and the S MMA of tile j + 2 is issued before
//     P V of tile j; at the end of the item the two threads of a row exchange (max, sum)
//     and each merges and stores half of the row's output from both accumulators;
//   * a row's part of O[g] is rescaled in TMEM (tcgen05.ld / st) only in a tile where
//     its running maximum grows past the reference point by more than 2^8, which after
//     the first tiles is rare, so the softmax threads normally never wait for P V;
//   * the producer requests K ahead of V (K of tile j + 1 or j + 2 before it waits for
//     the V stage of tile j, which only the P V product two tiles back releases);
//   * V is used in place from the cache layout as an MN-major B operand (keys are the
//     contraction dimension), so no transposed copy of V exists anywhere;
//   * the page size is a parameter (16 and 64 are tested); pages of one 128-key tile
//     are fetched by parallel lanes of the producer warp;
//   * an item with at most 32 rows (decode: one token x GQA group) loads its rows into
//     all four 32-lane quadrants of the MMA's M dimension; softmax warp w then handles
//     key columns [32 w, 32 w + 32) of every tile with its own running (max, sum) and
//     its own O rows, and the four partial results are merged once at the end of the
//     item.  That spreads a decode row's exponentials over four warps without any
//     cross-warp traffic inside the tile loop;
//   * an item may cover a key range [key_begin, key_end) only (split KV for load
//     balance, as the reference's KV chunks: csrc/fabric/tiles/attention.cuh:286-395);
//     it then leaves its unnormalised fp32 O rows and (max, sum) in a workspace and
//     attention_combine_kernel merges the parts in part order.
//
// Warp roles (320 threads): warp 0 TMA producer, warp 1 TMEM owner + MMA issue, warps 2..5 and
// 6..9 two softmax / output groups (TMEM lane quadrant = warp % 4) that take alternate key tiles
// of an item; a quad-replicated (decode) item is done by the first group alone.  One softmax
// warp per SM sub-partition is bound by instruction latency (max, ex2, bf16 packing per element);
// the second group doubles what is in flight.  Every wait is bounded; a timeout raises the status
// word and the CTA leaves, freeing its TMEM.
#include <algorithm>
#include <atomic>

#include "attention_core.cuh"

namespace mf {

// Diagnostics: phase times of work item 0's softmax lane of quadrant 2 (cycles summed over
// the item's KV tiles): [0] wait for S, [1] max pass, [2] exp + P store, [3] rescale of O
// (tiles where a maximum grew), [4] final wait for O, [5] tiles, [6] total ns.  Written when
// AttnParams::pad is nonzero.
__device__ unsigned long long g_attn_trace[8];

// The claim ring between the producer warp, which takes the CTA's next item from the launch's
// counter, and the MMA and softmax warps (1 + 4 * kAttnGroups readers per slot).
struct AttnClaims {
  uint64_t full[2], empty[2], q_empty, s_free[2];
  int item[2];
};
constexpr int kClaimSlots = 64;
// One counter per launch in flight (the launcher hands the slots out in turn).  A launch of n items on g
// CTAs makes exactly n + g claims, the last g of them failing, and the counter wraps to 0 with the last one,
// so nothing resets it between launches; a CTA that gives up early still makes its failing claim.  Limits:
// at most kClaimSlots launches of this kernel in flight on a device at a time, and a launch captured into a
// CUDA graph keeps the slot it was captured with (replays of one graph follow one another, but two graphs
// captured kClaimSlots launches apart must not run at the same time).
__device__ unsigned int g_attn_claim[kClaimSlots];

// A barrier of the CTA's softmax threads that also tells each of them whether any passed `flag`.
__device__ __forceinline__ bool softmax_threads_any(bool flag) {
  uint32_t any;
  asm volatile(
      "{\n\t"
      ".reg .pred P, Q;\n\t"
      "setp.ne.u32 Q, %1, 0;\n\t"
      "bar.red.or.pred P, 7, %2, Q;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(any)
      : "r"(static_cast<uint32_t>(flag)), "r"(128 * kAttnGroups)
      : "memory");
  return any != 0;
}

// Persistent: min(items, SMs) CTAs claim items in list order (longest first) until the list is exhausted.
// The roles of a CTA loop over its items independently; the producer runs ahead, so the next item's Q, K
// and V arrive while the softmax warps still merge and store the current one.
__global__ void __launch_bounds__(kAttnThreads, 1) paged_attention_kernel(const __grid_constant__ AttnParams p) {
  // The operand tiles need 1024-byte alignment (128-byte swizzle); static shared memory (under 3 KB) comes
  // first, so the seven tiles end exactly at the 227 KB a CTA may have.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ AttnShared sh;
  __shared__ AttnClaims cl;
  // (max, sum) pairs: the four column quarters of a quad-replicated item, or the two groups' halves of an item's rows;
  // every item ends with a barrier of all softmax threads after its last read
  __shared__ __align__(16) float2 xbuf[kAttnGroups * 128];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  AttnWork w;
  w.q_map = &p.q_map;
  w.q_map_small = &p.q_map_small;
  w.k_map = &p.k_map;
  w.v_map = &p.v_map;
  w.block_table = p.block_table;
  w.out = p.out;
  w.ws_o = p.ws_o;
  w.ws_ml = p.ws_ml;
  w.trace = nullptr;
  w.scale_log2 = p.scale_log2;
  w.bt_stride = p.bt_stride;
  w.hq = p.hq;
  w.group = p.group;
  w.page = p.page;
  w.q_box_rows = p.q_box_rows;
  w.rep_ok = p.rep_ok;
  AttnCtx c;
  c.sh = &sh;
  c.abort_flag = &sh.abort_flag;
  c.smem = smem_raw;
  if (smem_u32(smem_raw) & 1023u) {   // never seen; the tiles would not be where the descriptors say
    if (threadIdx.x == 0) {
      atomicOr(p.status, kErrBadArgs);
      // this CTA's share of the claims, so that the launch still leaves its counter at 0
      const unsigned int wrap = static_cast<unsigned int>(p.n_items) + gridDim.x - 1;
      while (atomicInc(&g_attn_claim[p.claim_slot], wrap) < static_cast<unsigned int>(p.n_items)) {
      }
    }
    return;
  }
  c.q_phase = 0;
  c.note = nullptr;
  c.xbuf = reinterpret_cast<float*>(xbuf);
  c.q_empty = &cl.q_empty;
  c.s_free = cl.s_free;
  c.base[0] = c.base[1] = 0;
  volatile int* abort_flag = &sh.abort_flag;

  if (threadIdx.x == 0) {
    sh.abort_flag = 0;
    sh.fail_site = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(&cl.full[i], 1);
      mbar_init(&cl.empty[i], 1 + 4 * kAttnGroups);
    }
    mbar_init(&cl.q_empty, 1);
    for (int i = 0; i < 2; ++i) mbar_init(&cl.s_free[i], 128);
    attn_barriers_init(sh, 128);   // P of a tile comes from one softmax group
  }
  if (warp == 1) {
    tmem_alloc(&sh.tmem_base, kAttnTmemCols);
    tmem_relinquish();
  }
  chain_release();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  c.tmem_base = sh.tmem_base;
  chain_wait();   // q and the caches may come from the kernel before this one

  const int n_items = p.n_items;
  if (warp == 0) {
    // ------------------------------------------------------ claims + TMA producer
    unsigned int* counter = &g_attn_claim[p.claim_slot];
    const unsigned int wrap = static_cast<unsigned int>(n_items) + gridDim.x - 1;
    bool list_ended = false;
    for (int it = 0;; ++it) {
      const int slot = it & 1;
      // the slot's previous record (item it - 2) has been read by every role
      if (it >= 2 && !warp_wait(&cl.empty[slot], ((it >> 1) - 1) & 1u, abort_flag, kAttnWaitNs)) break;
      int i = 0;
      if (lane == 0) {
        const unsigned int got = atomicInc(counter, wrap);
        i = got < static_cast<unsigned int>(n_items) ? static_cast<int>(got) : -1;
        cl.item[slot] = i;
        mbar_arrive(&cl.full[slot]);
      }
      i = __shfl_sync(0xffffffffu, i, 0);
      if (i < 0) {
        list_ended = true;
        break;
      }
      w.item = p.items[i];
      attn_derive(w, c);
      attn_produce<true>(w, c);
      attn_advance(c.n_tiles, c.q_phase, c.base);
      if (*abort_flag) break;
    }
    // a CTA that gives up still makes its failing claim, so that the counter ends at 0 for the slot's next launch
    if (!list_ended && lane == 0)
      while (atomicInc(counter, wrap) < static_cast<unsigned int>(n_items)) {
      }
  } else {
    for (int it = 0;; ++it) {
      const int slot = it & 1;
      const bool got = warp_wait(&cl.full[slot], (it >> 1) & 1u, abort_flag, kAttnWaitNs);
      const int i = got ? cl.item[slot] : -1;
      __syncwarp();
      if (got && lane == 0) mbar_arrive(&cl.empty[slot]);   // the record is read: the slot may be refilled
      // The softmax threads meet at named barriers inside an item, so they leave together or not at all: one
      // decision per item, taken by all of them at a barrier, on whether any of them has seen a wait give up.
      if (warp >= 2 ? softmax_threads_any(!got || *abort_flag != 0) : !got) break;
      if (i < 0) break;
      w.item = p.items[i];
      w.trace = (p.pad && blockIdx.x == 0 && it == 0) ? g_attn_trace : nullptr;
      attn_derive(w, c);
      if (warp == 1) {
        if (c.rep) attn_mma<2, true>(w, c);
        else attn_mma_alt<true>(w, c);
      } else if (c.rep) {
        softmax_role<true, 2, kAttnGroups, true, true>(w, c, (warp - 2) >> 2);
      } else {
        softmax_alt<true>(w, c, (warp - 2) >> 2, xbuf);
      }
      attn_advance(c.n_tiles, c.q_phase, c.base);
      if (warp == 1 && *abort_flag) break;   // the softmax threads decide at the top of the loop
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && sh.abort_flag) atomicOr(p.status, kErrWaitTimeout);
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(c.tmem_base, kAttnTmemCols);
  }
}

// Merge of split items: one warp per output row (token, q head); the parts are added in
// part order.  items: {first query token, query tokens, kv head, first workspace row,
// parts, workspace rows per part, 0, 0}.
__global__ void attention_combine_kernel(const int32_t* __restrict__ items, int n_items, const float* __restrict__ ws_o,
                                         const float2* __restrict__ ws_ml, __nv_bfloat16* __restrict__ out, int hq,
                                         int group) {
  chain_release();
  chain_wait();   // the parts come from the attention kernel launched just before
  const int32_t* it = items + static_cast<size_t>(blockIdx.x) * 8;
  attn_merge_rows(it[0], it[1], it[2], it[3], it[4], it[5], ws_o, ws_ml, out, hq, group, threadIdx.x >> 5, blockDim.x >> 5);
}

cudaError_t launch_attention_combine(const int32_t* items, int n_items, const float* ws_o, const float2* ws_ml,
                                     __nv_bfloat16* out, int hq, int group, cudaStream_t stream) {
  if (n_items == 0) return cudaSuccess;
  return launch_chained(attention_combine_kernel, n_items, 256, 0, stream, items, n_items, ws_o, ws_ml, out, hq, group);
}

cudaError_t read_attention_trace(unsigned long long out[8]) {
  return cudaMemcpyFromSymbol(out, g_attn_trace, sizeof(unsigned long long) * 8);
}

cudaError_t launch_attention(const AttnParams& params, cudaStream_t stream) {
  if (params.n_items == 0) return cudaSuccess;
  static PerDeviceOnce once;
  cudaError_t err = once.run([] {
    return cudaFuncSetAttribute(paged_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmemBytes);
  });
  if (err != cudaSuccess) return err;
  int device = 0, sms = 0;
  if ((err = cudaGetDevice(&device)) != cudaSuccess) return err;
  if ((err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return err;
  static std::atomic<unsigned int> ticket{0};
  AttnParams p = params;
  p.claim_slot = static_cast<int32_t>(ticket.fetch_add(1) % kClaimSlots);
  return launch_chained(paged_attention_kernel, std::min(p.n_items, sms), kAttnThreads, kAttnSmemBytes, stream, p);
}

}  // namespace mf
