// Device code of the paged-KV GQA attention work item (see attention.cu for the design):
// the TMA producer, MMA and softmax / output roles, shared by the stand-alone kernel and
// by the attention tiles of the persistent fabric kernel.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kernels.h"
#include "ptx.cuh"

namespace mf {

constexpr int kAttnGroups = 2;                   // softmax warp groups of the stand-alone kernel
constexpr int kAttnThreads = 64 + 128 * kAttnGroups;
constexpr int kHeadDim = 128;
constexpr int kKeysPerTile = 128;
constexpr int kHalfBytes = 128 * 128;            // 128 rows x 64 bf16: one swizzle atom column, 16 KB
constexpr int kTileBytes = 2 * kHalfBytes;       // 128 x 128 bf16
constexpr int kAttnSmemBytes = kTileBytes * 7;   // Q, K x2, V x2, P x2; the kernel declares the array 1024-byte aligned
constexpr int kAttnTmemCols = 512;               // S x2 (256) + O x2 (256: one accumulator per softmax group; the fabric worker uses one)
constexpr unsigned long long kAttnWaitNs = 4000000000ull;
constexpr float kMaxSlack = 8.f;   // how far a row maximum may exceed the reference point of its exponentials


struct AttnShared {
  uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], p_full[2], o_full[2];
  uint32_t tmem_base;
  int abort_flag;
  unsigned int fail_site;   // diagnostics: which wait gave up first (kAttnSite*), 0 = none
};
// Wait sites, for the diagnostics word.
enum : unsigned int {
  kAttnSiteProdK = 1, kAttnSiteProdV, kAttnSiteMmaQ, kAttnSiteMmaK, kAttnSiteMmaSFree, kAttnSiteMmaV, kAttnSiteMmaP,
  kAttnSiteSmaxS, kAttnSiteSmaxRescale, kAttnSiteSmaxPFree, kAttnSiteSmaxFinal, kAttnSiteMmaTail, kAttnSiteProdQ,
};
__device__ __forceinline__ bool attn_gave_up(AttnShared& sh, unsigned int site) {
  atomicCAS(&sh.fail_site, 0u, site);
  return false;
}
constexpr int kPartLd = 132;   // fp32 row stride of the merge scratch (conflict-free float4 access)
constexpr int kPartFloats = 4 * 32 * kPartLd;   // then float2 [4][32]: (max, sum) of the four column quarters

// One work item with everything its three roles need.
struct AttnWork {
  const CUtensorMap* q_map;         // dims (128, hq, T), box (64, group, tokens per block)
  const CUtensorMap* q_map_small;   // box (64, group, 32 / group), or unused when rep_ok is 0
  const CUtensorMap* k_map;         // dims (64, 8, 2 hkv, page / 8, pages), box (64, 8, 2, page / 8, 1)
  const CUtensorMap* v_map;
  const int32_t* block_table;
  __nv_bfloat16* out;               // [T][hq][128]
  float* ws_o;                      // split items: unnormalised O rows, fp32 [rows][128]
  float2* ws_ml;                    // and their (max, sum)
  unsigned long long* trace;        // phase trace of this item's first softmax lane, or NULL
  float scale_log2;
  int32_t bt_stride, hq, group, page, q_box_rows, rep_ok;
  AttnItem item;
};

// What the roles of one CTA share while they work on an item.
struct AttnCtx {
  AttnShared* sh;
  volatile int* abort_flag;
  uint8_t* smem;          // 1024-byte aligned, seven 32 KB tiles: Q, K x2, V x2, P x2
  uint32_t tmem_base;     // S x2 at columns 0 and 128, O at 256 (and a second O at 384 under alternating groups)
  int n_tiles, rows, kv_end;
  bool rep;
  // Phases the barriers have completed before this item: the barriers are armed once per
  // CTA and a CTA that works on many items (a fabric worker) carries the counts along.
  uint32_t q_phase;       // q_full
  uint32_t base[2];       // every per-tile barrier [s]: tiles of parity s so far
  volatile unsigned int* note;   // this role's wait note (tile << 8 | site), or NULL
  float* xbuf;            // several softmax groups: float [groups][128] for the exchange between the parts of a row
  uint64_t* q_empty;      // chained items only: completes once per item, when its last S MMA has read Q
  uint64_t* s_free;       // alternating softmax groups only: [2], S[s] of a tile has been read into registers
};

__device__ __forceinline__ void attn_note(const AttnCtx& c, int j, unsigned int site) {
  if (c.note) *c.note = (static_cast<unsigned int>(j) << 8) | site;
}

// Parity of the phase that tile j of the current item completes on a per-tile barrier [j & 1].
__device__ __forceinline__ uint32_t attn_parity(const AttnCtx& c, int j) { return (c.base[j & 1] + (j >> 1)) & 1u; }

// After an item of n_tiles tiles, every role advances its copy of the phase counts.
__device__ __forceinline__ void attn_advance(int n_tiles, uint32_t& q_phase, uint32_t (&base)[2]) {
  q_phase += 1;
  base[0] += (n_tiles + 1) >> 1;
  base[1] += n_tiles >> 1;
}

__device__ __forceinline__ void attn_derive(const AttnWork& w, AttnCtx& c) {
  const AttnItem& item = w.item;
  c.rows = item.q_tokens * w.group;
  // keys this item covers: from key_begin up to the position of its last query token
  // (and key_end, when the item is one part of a split)
  int kv_end = min(item.kv_len, item.pos0 + item.q_tokens);
  if (item.key_end > 0) kv_end = min(kv_end, item.key_end);
  c.kv_end = kv_end;
  c.n_tiles = max(0, (kv_end - item.key_begin + kKeysPerTile - 1) / kKeysPerTile);
  c.rep = w.rep_ok && c.rows <= 32;
}

// By one thread, once per CTA, before a CTA-wide barrier.
__device__ __forceinline__ void attn_barriers_init(AttnShared& sh, int softmax_threads = 128) {
  mbar_init(&sh.q_full, 1);
  for (int i = 0; i < 2; ++i) {
    mbar_init(&sh.k_full[i], 1);
    mbar_init(&sh.v_full[i], 1);
    mbar_init(&sh.k_empty[i], 1);
    mbar_init(&sh.v_empty[i], 1);
    mbar_init(&sh.s_full[i], 1);
    mbar_init(&sh.p_full[i], softmax_threads);
    mbar_init(&sh.o_full[i], 1);   // P V of tile j completes phase j / 2 of o_full[j % 2]
  }
  fence_barrier_init();
}

// K-major SW128 descriptor of the Q or P tile: 128 rows, two 64-element column halves 16 KB apart;
// step = one of the eight 16-element K steps.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_addr, int step) {
  return umma_desc_sw128(tile_addr + (step >> 2) * kHalfBytes + (step & 3) * 32);
}

// A K or V tile in shared memory: 128 keys in groups of eight; a group is 2 KB: its eight 128-byte rows of
// head-dim half 0, then those of half 1.  (One TMA box per page delivers both halves of the page's keys in
// this order: attention.cu, the cache maps.)  So the eight-key groups of one half are 2 KB apart and the
// other half lies 1 KB further.
constexpr uint32_t kKvGroupBytes = 2048, kKvHalfOffset = 1024;

// K as the K-major B operand of S = Q K^T (rows = keys, contraction over d): step = one of the eight
// 16-element d steps.
__device__ __forceinline__ uint64_t desc_k_tile(uint32_t tile_addr, int step) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>(((tile_addr + (step >> 2) * kKvHalfOffset + (step & 3) * 32) & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(kKvGroupBytes >> 4) << 32;   // stride byte offset: next 8 keys
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// V as the MN-major B operand of O += P V (rows are keys = the contraction dimension, 128 bytes = 64 d
// elements per row): step = one of the eight 16-key K steps.
__device__ __forceinline__ uint64_t desc_v_mnmajor(uint32_t tile_addr, int step) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>(((tile_addr + step * 2 * kKvGroupBytes) & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(kKvHalfOffset >> 4) << 16;   // leading byte offset: next 64 d elements
  d |= static_cast<uint64_t>(kKvGroupBytes >> 4) << 32;   // stride byte offset: next 8 keys
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

__device__ __forceinline__ void tma_load_5d(void* smem, const void* map, uint64_t* bar, int c0, int c1, int c2, int c3,
                                            int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      :
      : "r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3), "r"(c4)
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

// A bounded wait whose outcome is the same in every lane of the warp, so that the
// warp-wide TMEM instructions that follow are never reached by a part of a warp.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned long long budget_ns) {
  return __all_sync(0xffffffffu, mbar_wait_bounded(bar, parity, abort_flag, budget_ns));
}

// The TMA producer role: the whole warp calls it.
// kChain: the CTA works through a list of items with no barrier between them and the producer runs ahead of
// the other roles into the next item.  The first uses of a ring stage by an item then wait for the stage's
// last use by the item before (the barriers count uses across items: AttnCtx::base), and Q waits until the
// MMAs of the item before have read it.
template <bool kChain = false>
__device__ __forceinline__ void attn_produce(const AttnWork& p, const AttnCtx& c) {
  AttnShared& sh = *c.sh;
  volatile int* abort_flag = c.abort_flag;
  const AttnItem& item = p.item;
  const int lane = threadIdx.x & 31;
  const int group = p.group, n_tiles = c.n_tiles, kv_end = c.kv_end;
  const bool rep = c.rep;
  uint8_t* const sQ = c.smem;
  uint8_t* const sK = c.smem + kTileBytes;
  uint8_t* const sV = c.smem + 3 * kTileBytes;
  if (kChain && c.q_phase > 0 && !warp_wait(c.q_empty, (c.q_phase - 1) & 1u, abort_flag, kAttnWaitNs)) {
    attn_gave_up(sh, kAttnSiteProdQ);
    return;
  }
  if (lane == 0) {
    if (rep) {
      // the same 32 rows into every lane quadrant of the M dimension
      mbar_arrive_expect_tx(&sh.q_full, kTileBytes);
      for (int q = 0; q < 4; ++q) {
        tma_load_3d_plain(sQ + q * 4096, p.q_map_small, &sh.q_full, 0, item.kv_head * group, item.q_row0);
        tma_load_3d_plain(sQ + kHalfBytes + q * 4096, p.q_map_small, &sh.q_full, 64, item.kv_head * group,
                          item.q_row0);
      }
    } else {
      mbar_arrive_expect_tx(&sh.q_full, 2u * p.q_box_rows * 128u);
      tma_load_3d_plain(sQ, p.q_map, &sh.q_full, 0, item.kv_head * group, item.q_row0);
      tma_load_3d_plain(sQ + kHalfBytes, p.q_map, &sh.q_full, 64, item.kv_head * group, item.q_row0);
    }
  }
  const int pages_per_tile = kKeysPerTile / p.page;
  const int page_bytes = p.page * 256;   // one page's keys of this head, both d halves
  const int last_page = (kv_end - 1) / p.page;
  const int tile0 = item.key_begin / kKeysPerTile;
  // K runs ahead of V: K of tile j + lead is requested before the wait for V's stage of tile j, which is
  // released only by the P V product two tiles back, so that the next S never waits for a K tile that could
  // have been on its way.  One tile ahead where the tile loop is bound by the loads (a quad-replicated item,
  // and inside the fabric worker), two under the alternating softmax groups, whose S of tile j + 2 goes out
  // before P V of tile j.
  const int lead = (kChain && !rep) ? 2 : 1;
  auto page_of = [&](int j) {
    // pages past the visible range repeat the last visible page; their keys are masked
    const int pg = min((tile0 + j) * pages_per_tile + lane, last_page);
    return p.block_table[static_cast<size_t>(item.req) * p.bt_stride + pg];
  };
  for (int step = 0; step < n_tiles + lead; ++step) {
    if (step < n_tiles) {
      const int j = step, s = j & 1;
      const uint32_t uses = c.base[s] + (j >> 1);        // earlier uses of this stage, by this item and those before
      const bool reuse = kChain ? uses > 0 : j >= 2;
      const uint32_t prev = (uses - 1) & 1u;             // the stage's previous use (tile j - 2 of this item, if j >= 2)
      if (lane == 0) attn_note(c, j, kAttnSiteProdK);
      if (reuse && !warp_wait(&sh.k_empty[s], prev, abort_flag, kAttnWaitNs)) { attn_gave_up(sh, kAttnSiteProdK); break; }
      if (lane == 0) mbar_arrive_expect_tx(&sh.k_full[s], kTileBytes);
      __syncwarp();
      if (lane < pages_per_tile)
        tma_load_5d(sK + s * kTileBytes + lane * page_bytes, p.k_map, &sh.k_full[s], 0, 0, 2 * item.kv_head, 0, page_of(j));
    }
    if (step >= lead) {
      const int j = step - lead, s = j & 1;
      const uint32_t uses = c.base[s] + (j >> 1);
      const bool reuse = kChain ? uses > 0 : j >= 2;
      const uint32_t prev = (uses - 1) & 1u;
      if (lane == 0) attn_note(c, j, kAttnSiteProdV);
      if (reuse && !warp_wait(&sh.v_empty[s], prev, abort_flag, kAttnWaitNs)) { attn_gave_up(sh, kAttnSiteProdV); break; }
      if (lane == 0) mbar_arrive_expect_tx(&sh.v_full[s], kTileBytes);
      __syncwarp();
      if (lane < pages_per_tile)
        tma_load_5d(sV + s * kTileBytes + lane * page_bytes, p.v_map, &sh.v_full[s], 0, 0, 2 * item.kv_head, 0, page_of(j));
    }
  }
}

// The MMA role: the whole MMA warp calls it and runs the tile loop in step (every lane waits on the
// barriers itself); one elected lane issues the MMAs and commits.  The loop is convergent code, so the
// descriptors are warp-uniform values (in a single-lane branch the issue path was about twice as slow).
// PB = P buffers in shared memory (2: the stand-alone kernel; 1: inside the fabric
// worker, whose operand ring holds six 32 KB tiles).
template <int PB, bool kChain = false>
__device__ __forceinline__ void attn_mma(const AttnWork& p, const AttnCtx& c) {
  AttnShared& sh = *c.sh;
  volatile int* abort_flag = c.abort_flag;
  const int n_tiles = c.n_tiles;
  const bool leader = elect_one();
  const uint32_t tmem_base = c.tmem_base, tmem_o = c.tmem_base + 256;
  uint8_t* const sQ = c.smem;
  uint8_t* const sK = c.smem + kTileBytes;
  uint8_t* const sV = c.smem + 3 * kTileBytes;
  uint8_t* const sP = c.smem + 5 * kTileBytes;
  // S = Q K^T: both K-major; O += P V: A K-major, B (V) MN-major
  const uint32_t idesc_s = umma_idesc_bf16(128, 128);
  const uint32_t idesc_o = umma_idesc_bf16(128, 128) | (1u << 16);
  const uint32_t q_addr = smem_u32(sQ);
  if (leader) attn_note(c, 0, kAttnSiteMmaQ);
  bool ok = mbar_wait_bounded(&sh.q_full, c.q_phase & 1u, abort_flag, kAttnWaitNs) || attn_gave_up(sh, kAttnSiteMmaQ);
  auto mma_s = [&](int j) {
    const int s = j & 1;
    if (leader) attn_note(c, j, kAttnSiteMmaK);
    if (!mbar_wait_bounded(&sh.k_full[s], attn_parity(c, j), abort_flag, kAttnWaitNs)) return attn_gave_up(sh, kAttnSiteMmaK);
    if (leader) attn_note(c, j, kAttnSiteMmaSFree);
    // S[s] is free once the softmax threads have turned its previous tile (j - 2, or, in a chain of items,
    // the last one of the item before) into P
    const uint32_t uses = c.base[s] + (j >> 1);
    if ((kChain ? uses > 0 : j >= 2) && !mbar_wait_bounded(&sh.p_full[s], (uses - 1) & 1u, abort_flag, kAttnWaitNs))
      return attn_gave_up(sh, kAttnSiteMmaSFree);
    tc_fence_after_sync();
    const uint32_t k_addr = smem_u32(sK + s * kTileBytes);
    if (leader) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        umma_bf16(tmem_base + s * 128, desc_kmajor(q_addr, i), desc_k_tile(k_addr, i), idesc_s, i != 0);
      umma_commit(&sh.s_full[s]);
      umma_commit(&sh.k_empty[s]);
      if (kChain && j == n_tiles - 1) umma_commit(c.q_empty);   // Q has been read for the last time
    }
    return true;
  };
  if (kChain && ok && n_tiles == 0 && leader) mbar_arrive(c.q_empty);
  if (ok && n_tiles > 0) ok = mma_s(0);
  if (ok && n_tiles > 1) ok = mma_s(1);
  for (int j = 0; ok && j < n_tiles; ++j) {
    const int s = j & 1;
    if (leader) attn_note(c, j, kAttnSiteMmaV);
    if (!mbar_wait_bounded(&sh.v_full[s], attn_parity(c, j), abort_flag, kAttnWaitNs)) { attn_gave_up(sh, kAttnSiteMmaV); break; }
    if (leader) attn_note(c, j, kAttnSiteMmaP);
    if (!mbar_wait_bounded(&sh.p_full[s], attn_parity(c, j), abort_flag, kAttnWaitNs)) { attn_gave_up(sh, kAttnSiteMmaP); break; }
    tc_fence_after_sync();
    const uint32_t v_addr = smem_u32(sV + s * kTileBytes), p_addr = smem_u32(sP + (j % PB) * kTileBytes);
    if (leader) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        umma_bf16(tmem_o, desc_kmajor(p_addr, i), desc_v_mnmajor(v_addr, i), idesc_o, (j | i) != 0);
      umma_commit(&sh.o_full[s]);
      umma_commit(&sh.v_empty[s]);
    }
    if (j + 2 < n_tiles && !mma_s(j + 2)) break;
  }
  // Leave only after the last commits have arrived on their barriers: a caller that re-arms
  // the barriers for its next item must not see a late arrival from this one.
  for (int j = max(0, n_tiles - 2); ok && j < n_tiles; ++j) {
    if (leader) attn_note(c, j, kAttnSiteMmaTail);
    ok = (mbar_wait_bounded(&sh.k_empty[j & 1], attn_parity(c, j), abort_flag, kAttnWaitNs) ||
          attn_gave_up(sh, kAttnSiteMmaTail)) &&
         (mbar_wait_bounded(&sh.v_empty[j & 1], attn_parity(c, j), abort_flag, kAttnWaitNs) ||
          attn_gave_up(sh, kAttnSiteMmaTail + 16));
  }
  __syncwarp();
}

__device__ __forceinline__ void named_barrier_128(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }
__device__ __forceinline__ void named_barrier_64(int id) { asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory"); }
__device__ __forceinline__ void named_barrier_n(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// The softmax / output role.  WG = softmax warp groups of four warps (1 inside the fabric
// worker, kAttnGroups in the stand-alone kernel); `wg` is the caller's group.  A thread's row is
// its TMEM lane.  kRep (quad-replicated item, at most 32 rows): the thread's row is `lane`, its
// columns are quarter `quad` of the tile, and only group 0 works.  Otherwise the thread owns one
// of 128 query rows and, with WG groups, 1 / WG of the tile's key columns and of the row's output:
// the WG threads of a row agree on the row maximum through shared memory (`c.xbuf`) and a
// barrier per lane quadrant, which all warps of the quadrant pass exactly twice per tile
// whatever else happens, so that none can be left waiting.  (Two groups: with four, 576 threads
// leave 96 registers each and the spills cost more than the extra warps hide: decode 517 us
// against 226, prefill 301 us against 253 on the benchmark shapes.  The stand-alone kernel no longer splits
// columns between its groups: its items with more than 32 rows run softmax_alt below, 634 TFLOP/s against 542
// on the prefill benchmark.)
// kChain (a chain of items, see attn_produce): the K / V stages already receive the next item while this one
// ends, so the merge of a quad-replicated item uses the two P buffers (64 KB, rows XOR-swizzled by 16-byte
// chunk instead of padded) and `c.xbuf` for the (max, sum) pairs, and every softmax thread of the CTA, working
// or not, meets at one barrier when the merge has read them.
// kAlt: the kernel's other items run softmax_alt, whose barriers count one group (128 arrivals); a quad-replicated
// item is then done by group 0 alone, which also completes the s_free phases, and group 1 only joins the barrier
// at the end.
template <bool kRep, int PB, int WG, bool kChain = false, bool kAlt = false>
__device__ __forceinline__ void softmax_role(const AttnWork& p, const AttnCtx& c, int wg) {
  static_assert(!kChain || PB == 2, "the chained merge needs both P buffers");
  static_assert(!kAlt || (kRep && kChain), "kAlt: the quad-replicated items of the alternating kernel");
  if (kAlt && wg != 0) {
    named_barrier_n(6, 128 * WG);
    return;
  }
  constexpr int NC = kRep ? 32 : kKeysPerTile / WG;   // key columns of a tile this thread handles
  constexpr int ND = kRep ? kHeadDim : kHeadDim / WG; // output columns of its row it rescales and stores
  AttnShared& sh = *c.sh;
  volatile int* abort_flag = c.abort_flag;
  const AttnItem& item = p.item;
  uint8_t* const sP = c.smem + 5 * kTileBytes;
  // merge scratch over the K / V stages (over the P buffers in a chain), free once the last P V has completed
  float* const scratch = reinterpret_cast<float*>(kChain ? sP : c.smem + kTileBytes);
  float2(*const ml)[32] = reinterpret_cast<float2(*)[32]>(kChain ? c.xbuf : scratch + kPartFloats);
  constexpr int kLd = kChain ? kHeadDim : kPartLd;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad = warp & 3;
  const int r = quad * 32 + lane;                 // TMEM lane = row of S, P and O
  const int lr = kRep ? lane : r;                 // row of the item
  const bool row_ok = lr < c.rows;
  const bool works = kRep ? wg == 0 : quad * 32 < c.rows;   // warp-uniform: false = keep the barrier protocol only
  const bool pair = !kRep && WG > 1 && works;               // exchanges with the other warps of its quadrant
  const int group = p.group;
  const int token = lr / group, head = item.kv_head * group + lr % group;
  const int qpos = item.pos0 + token;
  const int c_lo = kRep ? quad * 32 : wg * NC;
  const int d_lo = kRep ? 0 : wg * ND;
  const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
  const uint32_t tmem_o = c.tmem_base + 256 + lane_off + d_lo;
  const int n_tiles = c.n_tiles;
  float m = -1e30f, l = 0.f;
  bool ok = true;
  const bool tr = p.trace != nullptr && quad == 2 && wg == 0 && lane == 0;
  long long tc[5] = {0, 0, 0, 0, 0}, t_prev = clock64();
  const unsigned long long t_begin = globaltimer_ns();
  auto lap = [&](int i) {
    if (tr) {
      const long long now = clock64();
      tc[i] += now - t_prev;
      t_prev = now;
    }
  };
  if (kRep && works) {
    // columns outside this thread's quarter stay zero in the P buffers
    for (int b = 0; b < PB; ++b)
      for (int h = 0; h < 2; ++h) {
        uint4* row = reinterpret_cast<uint4*>(sP + b * kTileBytes + h * kHalfBytes + r * 128);
#pragma unroll
        for (int i = 0; i < 8; ++i) row[i] = make_uint4(0, 0, 0, 0);
      }
  }
  for (int j = 0; j < n_tiles; ++j) {
    const int s = j & 1;
    if (ok) {
      if (lane == 0) attn_note(c, j, kAttnSiteSmaxS);
      if (!warp_wait(&sh.s_full[s], attn_parity(c, j), abort_flag, kAttnWaitNs)) ok = attn_gave_up(sh, kAttnSiteSmaxS);
      tc_fence_after_sync();
    }
    lap(0);
    if (!works) {   // no row of this warp exists, or the other group does the item: keep the barrier protocol only
      if (ok) mbar_arrive(&sh.p_full[s]);
      continue;
    }
    const uint32_t tmem_s = c.tmem_base + s * 128 + lane_off + c_lo;
    const int key0 = item.key_begin + j * kKeysPerTile + c_lo;
    // keys this thread may use among its NC columns: [0, lim)
    const int lim = row_ok ? min(min(c.kv_end, qpos + 1) - key0, NC) : 0;
    if (!ok) {   // after a wait gave up: only what the partner warp may still be waiting for
      if (pair) {
        named_barrier_n(2 + quad, 32 * WG);
        named_barrier_n(2 + quad, 32 * WG);
      }
      continue;
    }
    uint32_t v[NC];
    __syncwarp();
#pragma unroll
    for (int c0 = 0; c0 < NC; c0 += 32) tmem_ld_32x32(tmem_s + c0, *reinterpret_cast<uint32_t(*)[32]>(&v[c0]));
    tmem_ld_wait();
    // the scale is positive: the maximum of the scaled scores is the scaled maximum
    float mx = -1e30f;
    if (lim >= NC) {
#pragma unroll
      for (int i = 0; i < NC; ++i) mx = fmaxf(mx, __uint_as_float(v[i]));
    } else {
#pragma unroll
      for (int i = 0; i < NC; ++i)
        if (i < lim) mx = fmaxf(mx, __uint_as_float(v[i]));
    }
    mx = mx > -1e30f ? mx * p.scale_log2 : -1e30f;
    if (pair) {   // the row maximum over all parts of the tile
      c.xbuf[wg * 128 + r] = mx;
      named_barrier_n(2 + quad, 32 * WG);
#pragma unroll
      for (int g = 0; g < WG; ++g) mx = fmaxf(mx, c.xbuf[g * 128 + r]);
      named_barrier_n(2 + quad, 32 * WG);
    }
    mx = fmaxf(mx, m);
    lap(1);
    // The reference point of a row's exponentials moves only when the row's maximum has grown past
    // it by more than kMaxSlack (in the exp2 domain): P then stays below 2^kMaxSlack, exact in fp32
    // sums and within bf16's range, the result is the same quotient, and the rescale of the row's
    // part of O in TMEM (which waits for the previous P V) becomes rare instead of per tile.
    if (j > 0 && mx <= m + kMaxSlack) mx = m;
    if (j > 0 && __any_sync(0xffffffffu, mx > m)) {
      if (lane == 0) attn_note(c, j, kAttnSiteSmaxRescale);
      if (!warp_wait(&sh.o_full[s ^ 1], attn_parity(c, j - 1), abort_flag, kAttnWaitNs)) {
        ok = attn_gave_up(sh, kAttnSiteSmaxRescale);
        continue;
      }
      tc_fence_after_sync();
      const float alpha = fast_exp2(m - mx);
#pragma unroll
      for (int c0 = 0; c0 < ND; c0 += 32) {
        uint32_t o[32];
        __syncwarp();
        tmem_ld_32x32(tmem_o + c0, o);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st_32x32(tmem_o + c0, o);
      }
      tmem_st_wait();
      l *= alpha;
    }
    m = mx;
    lap(3);
    // the P buffer is free once P V of tile j - PB has completed
    if (lane == 0) attn_note(c, j, kAttnSiteSmaxPFree);
    if (j >= PB && !warp_wait(&sh.o_full[(j - PB) & 1], attn_parity(c, j - PB), abort_flag, kAttnWaitNs)) {
      ok = attn_gave_up(sh, kAttnSiteSmaxPFree);
      continue;
    }
    const float neg_mx = -mx;
    // P = exp2(s - max) as bf16 into shared memory (K-major, 128-byte swizzle); row sum of the rounded P
    float sum0 = 0.f, sum1 = 0.f;
    uint8_t* p_tile = sP + (j % PB) * kTileBytes;
#pragma unroll
    for (int c0 = 0; c0 < NC; c0 += 32) {
      uint32_t packed[16];
      if (c0 + 32 <= lim) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(v[c0 + i]), p.scale_log2, neg_mx));
          const float p1 = fast_exp2(fmaf(__uint_as_float(v[c0 + i + 1]), p.scale_log2, neg_mx));
          const __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
          const uint32_t u = *reinterpret_cast<const uint32_t*>(&b);
          sum0 += __uint_as_float(u << 16);
          sum1 += __uint_as_float(u & 0xffff0000u);
          packed[i >> 1] = u;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = c0 + i < lim ? fast_exp2(fmaf(__uint_as_float(v[c0 + i]), p.scale_log2, neg_mx)) : 0.f;
          const float p1 = c0 + i + 1 < lim ? fast_exp2(fmaf(__uint_as_float(v[c0 + i + 1]), p.scale_log2, neg_mx)) : 0.f;
          const __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
          const uint32_t u = *reinterpret_cast<const uint32_t*>(&b);
          sum0 += __uint_as_float(u << 16);
          sum1 += __uint_as_float(u & 0xffff0000u);
          packed[i >> 1] = u;
        }
      }
      // 32 keys = four 16-byte chunks of this row in key half col / 64
      const int col = c_lo + c0;
      uint8_t* row_base = p_tile + (col >> 6) * kHalfBytes + r * 128;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int chunk = ((col & 63) >> 3) + q;
        *reinterpret_cast<uint4*>(row_base + ((chunk ^ (r & 7)) << 4)) =
            make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
      }
    }
    l += sum0 + sum1;
    tc_fence_before_sync();
    fence_proxy_async_smem();
    mbar_arrive(&sh.p_full[s]);
    if (kAlt) mbar_arrive(&c.s_free[s]);
    lap(2);
  }
  if (lane == 0) attn_note(c, n_tiles, kAttnSiteSmaxFinal);
  if (ok && n_tiles > 0)
    ok = warp_wait(&sh.o_full[(n_tiles - 1) & 1], attn_parity(c, n_tiles - 1), abort_flag, kAttnWaitNs) ||
         attn_gave_up(sh, kAttnSiteSmaxFinal);
  tc_fence_after_sync();
  lap(4);
  if (tr) {
    for (int i = 0; i < 5; ++i) p.trace[i] = tc[i];
    p.trace[5] = n_tiles;
    p.trace[6] = globaltimer_ns() - t_begin;
  }
  const bool split = item.ws_row0 >= 0;
  if (!kRep) {
    if (pair) {   // the row sum over all parts, added in group order
      c.xbuf[wg * 128 + r] = l;
      named_barrier_n(2 + quad, 32 * WG);
      l = 0.f;
#pragma unroll
      for (int g = 0; g < WG; ++g) l += c.xbuf[g * 128 + r];
      if (kChain) named_barrier_n(2 + quad, 32 * WG);   // the next item's first exchange reuses the slots
    }
    // The TMEM loads are warp-wide (.sync.aligned): they sit in code every lane of the warp
    // runs, apart from anything that depends on the lane's row, and a warp barrier separates
    // them from the per-row stores so that the two cannot be merged into one divergent region.
    if (ok && works) {
      uint32_t o[ND];
      if (n_tiles > 0) {
#pragma unroll
        for (int c0 = 0; c0 < ND; c0 += 32) tmem_ld_32x32(tmem_o + c0, *reinterpret_cast<uint32_t(*)[32]>(&o[c0]));
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < ND; ++i) o[i] = 0;
      }
      __syncwarp();
      if (row_ok) {
        if (split) {
          float4* wdst = reinterpret_cast<float4*>(p.ws_o + static_cast<size_t>(item.ws_row0 + lr) * kHeadDim + d_lo);
          if (wg == 0) p.ws_ml[item.ws_row0 + lr] = make_float2(m, l);
#pragma unroll
          for (int i = 0; i < ND / 4; ++i)
            wdst[i] = make_float4(__uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]), __uint_as_float(o[4 * i + 2]),
                                  __uint_as_float(o[4 * i + 3]));
        } else {
          const float inv = l > 0.f ? 1.f / l : 0.f;
          uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(item.q_row0 + token) * p.hq + head) * kHeadDim +
                                                d_lo);
#pragma unroll
          for (int q = 0; q < ND / 8; ++q) {
            __nv_bfloat162 h[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
              h[i] = __floats2bfloat162_rn(__uint_as_float(o[8 * q + 2 * i]) * inv, __uint_as_float(o[8 * q + 2 * i + 1]) * inv);
            dst[q] = *reinterpret_cast<const uint4*>(h);
          }
        }
      }
      __syncwarp();
    }
    return;
  }
  if (!works) {   // the other softmax group merges the quad-replicated item
    if (kChain) named_barrier_n(6, 128 * WG);
    return;
  }
  // quad-replicated item: merge the four column quarters.  Every thread of the group takes part
  // in both barriers, also after a timeout, so that none of them can be left waiting.
  ml[quad][lane] = make_float2(m, l);
  named_barrier_128(1);
  float M = -1e30f;
#pragma unroll
  for (int q = 0; q < 4; ++q) M = fmaxf(M, ml[q][lane].x);
  float L = 0.f;
#pragma unroll
  for (int q = 0; q < 4; ++q) L += ml[q][lane].y * fast_exp2(ml[q][lane].x - M);
  {
    const float f = fast_exp2(m - M);
    float4* mine = reinterpret_cast<float4*>(scratch + (quad * 32 + lane) * kLd);
    const int sw = kChain ? lane : 0;   // chunk i of a row sits at i ^ lane: conflict-free without padding
#pragma unroll
    for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
      uint32_t o[32];
      __syncwarp();
      if (ok && n_tiles > 0) {
        tmem_ld_32x32(tmem_o + c0, o);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
        mine[((c0 >> 2) + i) ^ sw] = make_float4(__uint_as_float(o[4 * i]) * f, __uint_as_float(o[4 * i + 1]) * f,
                                                 __uint_as_float(o[4 * i + 2]) * f, __uint_as_float(o[4 * i + 3]) * f);
    }
  }
  named_barrier_128(1);
  if (ok && row_ok) {
    // this thread: row `lane`, output columns [32 quad, 32 quad + 32), quarters added in order
    float acc[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i] = 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4* src = reinterpret_cast<const float4*>(scratch + (q * 32 + lane) * kLd);
      const int sw = kChain ? lane : 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 t = src[(quad * 8 + i) ^ sw];
        acc[4 * i] += t.x;
        acc[4 * i + 1] += t.y;
        acc[4 * i + 2] += t.z;
        acc[4 * i + 3] += t.w;
      }
    }
    if (split) {
      float4* wdst = reinterpret_cast<float4*>(p.ws_o + static_cast<size_t>(item.ws_row0 + lr) * kHeadDim + quad * 32);
#pragma unroll
      for (int i = 0; i < 8; ++i) wdst[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
      if (quad == 0) p.ws_ml[item.ws_row0 + lr] = make_float2(M, L);
    } else {
      const float inv = L > 0.f ? 1.f / L : 0.f;
      uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(item.q_row0 + token) * p.hq + head) * kHeadDim +
                                            quad * 32);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        __nv_bfloat162 h[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(acc[8 * q + 2 * i] * inv, acc[8 * q + 2 * i + 1] * inv);
        dst[q] = *reinterpret_cast<const uint4*>(h);
      }
    }
  }
  // the scratch is the next item's P buffers and `ml` its exchange buffer: nobody goes on before all have read
  if (kChain) named_barrier_n(6, 128 * WG);
}

// ---------------------------------------------------------------------------------------------------------
// Alternating softmax groups (the stand-alone kernel's items with more than 32 rows).  Group g owns the tiles
// j = g, g + 2, ... of an item: S[g], P[g] and an accumulator O[g] of its own (TMEM columns 256 + 128 g), with its
// own running (max, sum) per row, so the two groups never talk inside the tile loop and one group's exponentials
// overlap the other's; at the end of the item the two threads of a row exchange (max, sum) and each merges and
// stores half of the row's output from both accumulators.  A thread reads its row of S in two passes of 64-column
// halves (maximum, then exponentials) and releases S[g] after the last load, before the exponentials, so that the
// next S MMA of the group does not wait for them.

// The MMA role of such an item (the whole warp, one elected lane issues).  S of tile j + 2 is issued before
// P V of tile j: it needs the S buffer (s_free), not P.
template <bool kChain>
__device__ __forceinline__ void attn_mma_alt(const AttnWork& p, const AttnCtx& c) {
  AttnShared& sh = *c.sh;
  volatile int* abort_flag = c.abort_flag;
  const int n_tiles = c.n_tiles;
  const bool leader = elect_one();
  const uint32_t tmem_base = c.tmem_base, tmem_o = c.tmem_base + 256;
  uint8_t* const sQ = c.smem;
  uint8_t* const sK = c.smem + kTileBytes;
  uint8_t* const sV = c.smem + 3 * kTileBytes;
  uint8_t* const sP = c.smem + 5 * kTileBytes;
  const uint32_t idesc_s = umma_idesc_bf16(128, 128);
  const uint32_t idesc_o = umma_idesc_bf16(128, 128) | (1u << 16);
  const uint32_t q_addr = smem_u32(sQ);
  if (leader) attn_note(c, 0, kAttnSiteMmaQ);
  bool ok = mbar_wait_bounded(&sh.q_full, c.q_phase & 1u, abort_flag, kAttnWaitNs) || attn_gave_up(sh, kAttnSiteMmaQ);
  auto mma_s = [&](int j) {
    const int s = j & 1;
    if (leader) attn_note(c, j, kAttnSiteMmaK);
    if (!mbar_wait_bounded(&sh.k_full[s], attn_parity(c, j), abort_flag, kAttnWaitNs)) return attn_gave_up(sh, kAttnSiteMmaK);
    if (leader) attn_note(c, j, kAttnSiteMmaSFree);
    const uint32_t uses = c.base[s] + (j >> 1);   // the buffer's previous tile has been read into registers
    if ((kChain ? uses > 0 : j >= 2) && !mbar_wait_bounded(&c.s_free[s], (uses - 1) & 1u, abort_flag, kAttnWaitNs))
      return attn_gave_up(sh, kAttnSiteMmaSFree);
    tc_fence_after_sync();
    const uint32_t k_addr = smem_u32(sK + s * kTileBytes);
    if (leader) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        umma_bf16(tmem_base + s * 128, desc_kmajor(q_addr, i), desc_k_tile(k_addr, i), idesc_s, i != 0);
      umma_commit(&sh.s_full[s]);
      umma_commit(&sh.k_empty[s]);
      if (kChain && j == n_tiles - 1) umma_commit(c.q_empty);
    }
    return true;
  };
  if (kChain && ok && n_tiles == 0 && leader) mbar_arrive(c.q_empty);
  if (ok && n_tiles > 0) ok = mma_s(0);
  if (ok && n_tiles > 1) ok = mma_s(1);
  for (int j = 0; ok && j < n_tiles; ++j) {
    const int s = j & 1;
    if (j + 2 < n_tiles && !mma_s(j + 2)) break;
    if (leader) attn_note(c, j, kAttnSiteMmaV);
    if (!mbar_wait_bounded(&sh.v_full[s], attn_parity(c, j), abort_flag, kAttnWaitNs)) { attn_gave_up(sh, kAttnSiteMmaV); break; }
    if (leader) attn_note(c, j, kAttnSiteMmaP);
    if (!mbar_wait_bounded(&sh.p_full[s], attn_parity(c, j), abort_flag, kAttnWaitNs)) { attn_gave_up(sh, kAttnSiteMmaP); break; }
    tc_fence_after_sync();
    const uint32_t v_addr = smem_u32(sV + s * kTileBytes), p_addr = smem_u32(sP + s * kTileBytes);
    if (leader) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        umma_bf16(tmem_o + s * 128, desc_kmajor(p_addr, i), desc_v_mnmajor(v_addr, i), idesc_o, ((j >> 1) | i) != 0);
      umma_commit(&sh.o_full[s]);
      umma_commit(&sh.v_empty[s]);
    }
  }
  for (int j = max(0, n_tiles - 2); ok && j < n_tiles; ++j) {
    if (leader) attn_note(c, j, kAttnSiteMmaTail);
    ok = (mbar_wait_bounded(&sh.k_empty[j & 1], attn_parity(c, j), abort_flag, kAttnWaitNs) ||
          attn_gave_up(sh, kAttnSiteMmaTail)) &&
         (mbar_wait_bounded(&sh.v_empty[j & 1], attn_parity(c, j), abort_flag, kAttnWaitNs) ||
          attn_gave_up(sh, kAttnSiteMmaTail + 16));
  }
  __syncwarp();
}

// The softmax / output role of such an item: group `wg` of two.  `ml`: float2 [2][128] for the (max, sum) exchange.
// Every thread passes the quadrant barrier once and the barrier of all softmax threads once per item, whatever
// else happens.
template <bool kChain>
__device__ __forceinline__ void softmax_alt(const AttnWork& p, const AttnCtx& c, int wg, float2* ml) {
  AttnShared& sh = *c.sh;
  volatile int* abort_flag = c.abort_flag;
  const AttnItem& item = p.item;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad = warp & 3;
  const int r = quad * 32 + lane;                 // TMEM lane = row of S, P and O = row of the item
  const bool row_ok = r < c.rows;
  const bool works = quad * 32 < c.rows;          // warp-uniform
  const int group = p.group;
  const int token = r / group, head = item.kv_head * group + r % group;
  const int qpos = item.pos0 + token;
  const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
  const uint32_t tmem_s = c.tmem_base + wg * 128 + lane_off;
  const uint32_t tmem_o = c.tmem_base + 256 + lane_off;   // O[0]; O[1] is 128 columns further
  const int n_tiles = c.n_tiles;
  const int s = wg;
  uint8_t* const p_tile = c.smem + (5 + wg) * kTileBytes;
  float m = -1e30f, l = 0.f;
  bool ok = true;
  const bool tr = p.trace != nullptr && quad == 2 && wg == 0 && lane == 0;
  long long tc[5] = {0, 0, 0, 0, 0}, t_prev = clock64();
  const unsigned long long t_begin = globaltimer_ns();
  auto lap = [&](int i) {
    if (tr) {
      const long long now = clock64();
      tc[i] += now - t_prev;
      t_prev = now;
    }
  };
  for (int j = wg; j < n_tiles; j += 2) {
    if (!ok) break;
    if (lane == 0) attn_note(c, j, kAttnSiteSmaxS);
    if (!warp_wait(&sh.s_full[s], attn_parity(c, j), abort_flag, kAttnWaitNs)) {
      ok = attn_gave_up(sh, kAttnSiteSmaxS);
      break;
    }
    tc_fence_after_sync();
    lap(0);
    if (!works) {
      // No row of this warp exists: keep the barrier protocol only.  S of this tile was issued when the buffer's
      // previous tile had been read, which is before that tile's P is complete: the arrival for this tile's P
      // must not land in that phase, so it waits, like a working warp, for the P V of the previous tile.
      mbar_arrive(&c.s_free[s]);
      if (j >= 2 && !warp_wait(&sh.o_full[s], attn_parity(c, j - 2), abort_flag, kAttnWaitNs)) {
        ok = attn_gave_up(sh, kAttnSiteSmaxPFree);
        break;
      }
      mbar_arrive(&sh.p_full[s]);
      continue;
    }
    const int key0 = item.key_begin + j * kKeysPerTile;
    const int lim = row_ok ? min(min(c.kv_end, qpos + 1) - key0, kKeysPerTile) : 0;   // keys [0, lim) of the tile count
    uint32_t v[64];
    // pass 1: the row maximum (the scale is positive: the maximum of the scaled scores is the scaled maximum)
    float mx0 = -1e30f, mx1 = -1e30f, mx2 = -1e30f, mx3 = -1e30f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      __syncwarp();
      tmem_ld_32x32(tmem_s + 64 * h, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
      tmem_ld_32x32(tmem_s + 64 * h + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
      tmem_ld_wait();
      const int lh = lim - 64 * h;
      if (lh >= 64) {
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
          mx0 = fmaxf(mx0, __uint_as_float(v[i]));
          mx1 = fmaxf(mx1, __uint_as_float(v[i + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(v[i + 2]));
          mx3 = fmaxf(mx3, __uint_as_float(v[i + 3]));
        }
      } else if (lh > 0) {
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
          mx0 = fmaxf(mx0, i < lh ? __uint_as_float(v[i]) : -1e30f);
          mx1 = fmaxf(mx1, i + 1 < lh ? __uint_as_float(v[i + 1]) : -1e30f);
          mx2 = fmaxf(mx2, i + 2 < lh ? __uint_as_float(v[i + 2]) : -1e30f);
          mx3 = fmaxf(mx3, i + 3 < lh ? __uint_as_float(v[i + 3]) : -1e30f);
        }
      }
    }
    float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
    mx = mx > -1e30f ? mx * p.scale_log2 : -1e30f;
    mx = fmaxf(mx, m);
    lap(1);
    // the reference point of the row's exponentials moves only when the maximum has grown past it by more than
    // kMaxSlack (see softmax_role); the group's accumulator is rescaled then, after its previous P V
    if (j >= 2 && mx <= m + kMaxSlack) mx = m;
    if (j >= 2 && __any_sync(0xffffffffu, mx > m)) {
      if (lane == 0) attn_note(c, j, kAttnSiteSmaxRescale);
      if (!warp_wait(&sh.o_full[s], attn_parity(c, j - 2), abort_flag, kAttnWaitNs)) {
        ok = attn_gave_up(sh, kAttnSiteSmaxRescale);
        break;
      }
      tc_fence_after_sync();
      const float alpha = fast_exp2(m - mx);
#pragma unroll
      for (int c0 = 0; c0 < kHeadDim; c0 += 32) {
        uint32_t o[32];
        __syncwarp();
        tmem_ld_32x32(tmem_o + s * 128 + c0, o);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st_32x32(tmem_o + s * 128 + c0, o);
      }
      tmem_st_wait();
      l *= alpha;
    }
    m = mx;
    lap(3);
    // the group's P buffer is free once P V of its previous tile has completed
    if (lane == 0) attn_note(c, j, kAttnSiteSmaxPFree);
    if (j >= 2 && !warp_wait(&sh.o_full[s], attn_parity(c, j - 2), abort_flag, kAttnWaitNs)) {
      ok = attn_gave_up(sh, kAttnSiteSmaxPFree);
      break;
    }
    const float neg_mx = -mx;
    float sum0 = 0.f, sum1 = 0.f;
    // pass 2: P = exp2(s - max) as bf16 into shared memory (K-major, 128-byte swizzle); row sum of the rounded P
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      __syncwarp();
      tmem_ld_32x32(tmem_s + 64 * h, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
      tmem_ld_32x32(tmem_s + 64 * h + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
      tmem_ld_wait();
      if (h == 1) {   // S has been read for the last time: the MMA warp may overwrite it
        tc_fence_before_sync();
        mbar_arrive(&c.s_free[s]);
      }
      const int lh = lim - 64 * h;
      uint8_t* row_base = p_tile + h * kHalfBytes + r * 128;
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t packed[16];
        if (c0 + 32 <= lh) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(v[c0 + i]), p.scale_log2, neg_mx));
            const float p1 = fast_exp2(fmaf(__uint_as_float(v[c0 + i + 1]), p.scale_log2, neg_mx));
            const __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
            const uint32_t u = *reinterpret_cast<const uint32_t*>(&b);
            sum0 += __uint_as_float(u << 16);
            sum1 += __uint_as_float(u & 0xffff0000u);
            packed[i >> 1] = u;
          }
        } else if (lh <= c0) {   // every key of the chunk is masked (half of a diagonal tile, on average)
#pragma unroll
          for (int i = 0; i < 16; ++i) packed[i] = 0;
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = c0 + i < lh ? fast_exp2(fmaf(__uint_as_float(v[c0 + i]), p.scale_log2, neg_mx)) : 0.f;
            const float p1 = c0 + i + 1 < lh ? fast_exp2(fmaf(__uint_as_float(v[c0 + i + 1]), p.scale_log2, neg_mx)) : 0.f;
            const __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
            const uint32_t u = *reinterpret_cast<const uint32_t*>(&b);
            sum0 += __uint_as_float(u << 16);
            sum1 += __uint_as_float(u & 0xffff0000u);
            packed[i >> 1] = u;
          }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = (c0 >> 3) + q;
          *reinterpret_cast<uint4*>(row_base + ((chunk ^ (r & 7)) << 4)) =
              make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        }
      }
    }
    l += sum0 + sum1;
    tc_fence_before_sync();
    fence_proxy_async_smem();
    mbar_arrive(&sh.p_full[s]);
    lap(2);
  }
  // both accumulators are complete once the last tile of each parity has been multiplied
  if (lane == 0) attn_note(c, n_tiles, kAttnSiteSmaxFinal);
  for (int j = max(0, n_tiles - 2); ok && j < n_tiles; ++j)
    ok = warp_wait(&sh.o_full[j & 1], attn_parity(c, j), abort_flag, kAttnWaitNs) || attn_gave_up(sh, kAttnSiteSmaxFinal);
  tc_fence_after_sync();
  lap(4);
  if (tr) {
    for (int i = 0; i < 5; ++i) p.trace[i] = tc[i];
    p.trace[5] = n_tiles;
    p.trace[6] = globaltimer_ns() - t_begin;
  }
  ml[wg * 128 + r] = make_float2(m, l);
  named_barrier_n(2 + quad, 64);
  const float2 a = ml[r], b = ml[128 + r];          // group 0's and group 1's (max, sum) of this row
  const float M = fmaxf(a.x, b.x);
  const float wa = fast_exp2(a.x - M), wb = fast_exp2(b.x - M);
  const float L = a.y * wa + b.y * wb;
  const int d_lo = wg * 64;                          // the half of the row's output this thread merges and stores
  uint32_t oa[64], ob[64];
  __syncwarp();
  if (ok && works && n_tiles > 0) {
    tmem_ld_32x32(tmem_o + d_lo, *reinterpret_cast<uint32_t(*)[32]>(&oa[0]));
    tmem_ld_32x32(tmem_o + d_lo + 32, *reinterpret_cast<uint32_t(*)[32]>(&oa[32]));
  } else {
#pragma unroll
    for (int i = 0; i < 64; ++i) oa[i] = 0;
  }
  if (ok && works && n_tiles > 1) {
    tmem_ld_32x32(tmem_o + 128 + d_lo, *reinterpret_cast<uint32_t(*)[32]>(&ob[0]));
    tmem_ld_32x32(tmem_o + 128 + d_lo + 32, *reinterpret_cast<uint32_t(*)[32]>(&ob[32]));
  } else {
#pragma unroll
    for (int i = 0; i < 64; ++i) ob[i] = 0;
  }
  tmem_ld_wait();
  tc_fence_before_sync();
  // nobody goes on to the next item (whose MMAs overwrite the accumulators, and whose exchange reuses `ml`)
  // before every thread has read both
  named_barrier_n(6, 256);
  if (ok && row_ok) {
    const bool split = item.ws_row0 >= 0;
    if (split) {
      float4* wdst = reinterpret_cast<float4*>(p.ws_o + static_cast<size_t>(item.ws_row0 + r) * kHeadDim + d_lo);
      if (wg == 0) p.ws_ml[item.ws_row0 + r] = make_float2(M, L);
#pragma unroll
      for (int i = 0; i < 16; ++i)
        wdst[i] = make_float4(__uint_as_float(oa[4 * i]) * wa + __uint_as_float(ob[4 * i]) * wb,
                              __uint_as_float(oa[4 * i + 1]) * wa + __uint_as_float(ob[4 * i + 1]) * wb,
                              __uint_as_float(oa[4 * i + 2]) * wa + __uint_as_float(ob[4 * i + 2]) * wb,
                              __uint_as_float(oa[4 * i + 3]) * wa + __uint_as_float(ob[4 * i + 3]) * wb);
    } else {
      const float inv = L > 0.f ? 1.f / L : 0.f;
      const float fa = wa * inv, fb = wb * inv;
      uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(item.q_row0 + token) * p.hq + head) * kHeadDim + d_lo);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        __nv_bfloat162 h[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          h[i] = __floats2bfloat162_rn(
              __uint_as_float(oa[8 * q + 2 * i]) * fa + __uint_as_float(ob[8 * q + 2 * i]) * fb,
              __uint_as_float(oa[8 * q + 2 * i + 1]) * fa + __uint_as_float(ob[8 * q + 2 * i + 1]) * fb);
        dst[q] = *reinterpret_cast<const uint4*>(h);
      }
    }
  }
}

// Merge of the parts of one split (request, block, KV head): one warp per output row
// (token, q head of the group), parts added in part order.  `warp` of `n_warps` warps.
__device__ __forceinline__ void attn_merge_rows(int q_row0, int q_tokens, int kv_head, int ws_row0, int parts, int stride,
                                                const float* __restrict__ ws_o, const float2* __restrict__ ws_ml,
                                                __nv_bfloat16* __restrict__ out, int hq, int group, int warp,
                                                int n_warps) {
  const int lane = threadIdx.x & 31;
  for (int row = warp; row < q_tokens * group; row += n_warps) {
    float M = -1e30f;
    for (int q = 0; q < parts; ++q) M = fmaxf(M, ws_ml[ws_row0 + q * stride + row].x);
    float L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int q = 0; q < parts; ++q) {
      const float2 ml = ws_ml[ws_row0 + q * stride + row];
      const float w = fast_exp2(ml.x - M);
      L += ml.y * w;
      const float4 t = reinterpret_cast<const float4*>(ws_o + static_cast<size_t>(ws_row0 + q * stride + row) * kHeadDim)[lane];
      acc.x += t.x * w;
      acc.y += t.y * w;
      acc.z += t.z * w;
      acc.w += t.w * w;
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    const int token = row / group, head = kv_head * group + row % group;
    __nv_bfloat162 h[2] = {__floats2bfloat162_rn(acc.x * inv, acc.y * inv), __floats2bfloat162_rn(acc.z * inv, acc.w * inv)};
    reinterpret_cast<uint2*>(out + (static_cast<size_t>(q_row0 + token) * hq + head) * kHeadDim)[lane] =
        *reinterpret_cast<const uint2*>(h);
  }
}

}  // namespace mf
