// The weight x activation GEMM tile on tcgen05 / TMEM / TMA, as three warp-role
// device functions shared by the stand-alone grouped expert GEMM kernel and by
// the persistent fabric worker.
//
// One tile (the reference's GEMM tile, csrc/fabric/tiles/gemm.cuh:1-18,133-346,
// csrc/fabric/model_types.h:37-49): 128 weight rows (output features) as the MMA
// M operand times up to 256 activation rows as the N operand, over a range of
// 64-element K steps; fp32 accumulation in TMEM.  Both operands are K-major with
// the 128-byte swizzle.  The weight slice is fetched as eight TMA boxes of 16
// rows, which lets a SwiGLU tile interleave 64 gate rows and 64 up rows in groups
// of 16: TMEM lane 32q+i (i < 16) then holds gate feature 16q+i and lane 32q+16+i
// the matching up feature, so the epilogue pairs them with a warp shuffle instead
// of a trip through shared memory.
//
// Roles: produce() runs in ONE thread (TMA issue), mma() in one warp (one lane
// issues tcgen05.mma / tcgen05.commit), epilogue() in the four warps whose
// warp index modulo 4 covers the four TMEM lane quadrants.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "ptx.cuh"
#include "types.h"

namespace mf {

constexpr int kBlockK = 64;                      // elements per K step (128 bytes of bf16)
constexpr int kATileBytes = 128 * kBlockK * 2;   // 16 KB
constexpr int kGemmMaxN = 256;
// Operand stages live in one byte ring: a stage takes 16 KB for the weight tile
// plus n * 128 bytes for the activation tile, so small-n (decode) tiles keep up
// to 12 stages in flight (about 200 KB per SM, which is what it takes to cover
// the loaded HBM latency) and n = 256 tiles still get four.
constexpr int kRingBytes = 216 * 1024;
constexpr int kGemmStages = 12;                  // most stages in flight (barrier pairs)
constexpr int kGemmSmemBytes = kRingBytes + 1024;
constexpr int kTmemCols = 512;
constexpr int kAccCols = 256;                    // TMEM columns per accumulator buffer (two buffers)
constexpr unsigned long long kWaitBudgetNs = 4000000000ull;   // 4 s of device time per wait

// Epilogues (csrc/fabric/model_types.h:29-35).
constexpr int kEpiStoreBf16 = 0;   // out[m][n] = bf16(acc (+ bias[n]) (+ residual[m][n]))
constexpr int kEpiSiluMul = 1;     // 64 gate + 64 up rows: out[m][f] = bf16(silu(g) * u)
constexpr int kEpiWeightedAdd = 2;  // out32[pair_token[m]][n] += pair_weight[m] * acc (fp32 atomics, arrival order)
constexpr int kEpiStoreF32 = 3;    // out32[m][n] = acc (+ bias[n])
constexpr int kEpiAtomicF32 = 4;   // out32[m][n] += acc : K-split partial sums
constexpr int kEpiRowsF32 = 5;     // out32[m][n] = acc : per-pair rows for the deterministic combine (not in the reference)

// Everything the three roles need to know about one tile; lives in shared memory.
struct GemmWork {
  const CUtensorMap* a_map;   // weights: dims (K, rows, Z); box (64, 16, 1) for SwiGLU tiles, else (64, 128, 1)
  const CUtensorMap* b_map;   // activations: dims (K, rows), box (64, n)
  void* out;
  const float* scale;         // fp32 per weight row (FP8 weights), or null
  const __nv_bfloat16* bias;      // per output feature, or null
  const __nv_bfloat16* residual;  // [rows][ld_res], or null
  const int32_t* pair_token;      // kEpiWeightedAdd: token of every activation row
  const float* pair_weight;       // kEpiWeightedAdd: routing weight of every activation row
  int32_t a_row_lo;           // first weight row
  int32_t a_row_hi;           // kEpiSiluMul: first up row; otherwise ignored
  int32_t a_z;
  int32_t b_row0;             // first activation row
  int32_t rows;               // valid activation rows (<= n)
  int32_t n;                  // MMA N: 16, 32, 64, 128 or 256
  int32_t k0, k_tiles;        // K steps [k0, k0 + k_tiles)
  int32_t epi;
  int32_t ld_out, ld_res;
  int32_t n_limit;            // valid output features
  int32_t valid;              // 0: no tile (the consumer roles stop or skip)
  int32_t a_packed;           // bit 0 (two slabs): the weight rows are already interleaved in memory (one 128-row box);
                              // bit 2: two slabs (64 rows at a_row_lo, 64 at a_row_hi) under kEpiAtomicF32, whose
                              // partial sums go to column = weight row (kEpiSiluMul always reads two slabs)
  int32_t block;              // row block whose counter the epilogue bumps, or -1
  int32_t w_fp8;              // the weight tensor holds e4m3 bytes: W8A16 (exact e4m3 -> bf16 in shared memory)
  // A fetch record moves fetch_bytes from fetch_src (host-resident weights) to `out` (an HBM staging
  // buffer) through the operand ring, in stages of kFetchStageBytes: no MMA, no accumulator.
  int32_t fetch;
  uint32_t fetch_bytes;
  const uint8_t* fetch_src;
};

struct GemmPipe {   // a role's cursor over the stage ring; producer and MMA warp replay the same sequence
  uint32_t vwr = 0;     // virtual write position in bytes (wraps modulo 2^32; only differences are used)
  uint32_t phys = 0;    // ring offset of the next stage
  uint32_t slot = 0;    // barrier pair of the next stage
  uint32_t parity = 0;  // parity of that pair's current use
  uint32_t i = 0;       // stages allocated so far
  // MMA role: one bit per barrier pair = parity of the pair's converter barrier.  That barrier
  // completes a phase only for stages with e4m3 weights, so when bf16 and e4m3 tiles share the
  // ring its parity is not a function of the stage's position, unlike full / empty.
  uint32_t conv_bits = 0;
  // Next stage of `size` bytes (a multiple of 1024): its offset in the ring, and
  // the virtual interval it covers (including a skipped tail when it wraps).
  __device__ __forceinline__ uint32_t alloc(uint32_t size, uint32_t& vbegin, uint32_t& vend) {
    vbegin = vwr;
    if (phys + size > kRingBytes) {
      vwr += kRingBytes - phys;
      phys = 0;
    }
    const uint32_t at = phys;
    phys += size;
    vwr += size;
    vend = vwr;
    return at;
  }
  __device__ __forceinline__ void advance() {
    ++i;
    if (++slot == kGemmStages) {
      slot = 0;
      parity ^= 1;
    }
  }
};

// Producer-only bookkeeping of the stages in flight.
struct GemmInflight {
  uint32_t vbegin[kGemmStages];
  uint32_t tail = 0;          // oldest stage not yet known to be consumed
  uint32_t tail_slot = 0;
  uint32_t tail_parity = 0;
};

// Bytes of one stage: weight tile (bf16), activation tile, and for FP8 weights the
// raw e4m3 tile the converter warps expand.
// K steps (of kBlockK elements) one stage holds.  A stage of e4m3 weights holds two: a row of the raw
// tile is then 128 bytes, which is what makes reads of host-resident weights over the link efficient
// (64-byte reads reach 42 GB/s, 128-byte reads 51 GB/s).
constexpr uint32_t kFetchStageBytes = 32 * 1024;
__device__ __forceinline__ int gemm_ksteps(const GemmWork& w) { return w.w_fp8 ? 2 : 1; }
// kFetch = false (a kernel that never sees fetch records) compiles their handling away.
template <bool kFetch = true>
__device__ __forceinline__ int gemm_stage_count(const GemmWork& w) {
  if (kFetch && w.fetch) return static_cast<int>((w.fetch_bytes + kFetchStageBytes - 1) / kFetchStageBytes);
  return w.w_fp8 ? (w.k_tiles + 1) >> 1 : w.k_tiles;
}
// Bytes of one stage: per K step the bf16 weight tile and the activation tile; layout: weight tiles,
// then activation tiles.  The raw e4m3 tile (128 rows of 128 bytes) lands in the second weight tile
// and is expanded in place: the 128-byte swizzle permutes 16-byte chunks inside a row, so row r of the
// second K step's bf16 tile covers exactly the bytes of raw row r, which one converter thread owns.
template <bool kFetch = true>
__device__ __forceinline__ uint32_t gemm_stage_bytes(const GemmWork& w) {
  if (kFetch && w.fetch) return kFetchStageBytes;
  return gemm_ksteps(w) * (kATileBytes + w.n * kBlockK * 2);
}

struct GemmBarriers {
  uint64_t full[kGemmStages];
  uint64_t conv[kGemmStages];    // FP8: converter warps -> MMA (4 arrivals)
  uint64_t empty[kGemmStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
};

__device__ __forceinline__ void gemm_barriers_init(GemmBarriers& b) {
  for (int i = 0; i < kGemmStages; ++i) {
    mbar_init(&b.full[i], 1);
    mbar_init(&b.conv[i], 4);
    mbar_init(&b.empty[i], 1);
  }
  for (int i = 0; i < 2; ++i) {
    mbar_init(&b.acc_full[i], 1);
    mbar_init(&b.acc_empty[i], 4);
  }
}

// TMA issue for one tile.  The WHOLE producer warp calls it: every lane keeps
// the same bookkeeping, lane 0 arms the barrier, and the copies of one stage go
// out as a single warp-wide instruction (lanes 0..7 the weight boxes, lane 8 the
// activation box), which costs one issue slot instead of nine.
// Returns false when a wait was abandoned.
template <bool kFetch = true>
__device__ __forceinline__ bool gemm_produce(const GemmWork& w, uint8_t* ring, GemmBarriers& bar, GemmPipe& pipe,
                                             GemmInflight& fl, volatile int* abort_flag, uint64_t pol_w,
                                             uint64_t pol_x) {
  const int lane = threadIdx.x & 31;
  const uint32_t size = gemm_stage_bytes<kFetch>(w);
  const uint32_t b_bytes = w.n * kBlockK * 2;
  const int ks = gemm_ksteps(w);
  // FP8 weights land as raw bytes in the second weight tile (128-byte rows = two K steps, no swizzle)
  const uint32_t a_off = w.w_fp8 ? kATileBytes : 0;
  const uint32_t a_box = 2048;   // bytes of one 16-row box: 128-byte rows either way
  const uint32_t b_off = ks * kATileBytes;
  const int n_stages = gemm_stage_count<kFetch>(w);
  // SwiGLU tiles of a tensor in the reference row order gather eight 16-row boxes;
  // every other tile is one 128-row box (a packed SwiGLU tensor stores gate/up
  // groups of 16 rows alternately, so its tile starts at row 2 * a_row_lo).
  const bool slab2 = w.epi == kEpiSiluMul || (w.a_packed & 4);
  const bool gather = slab2 && !(w.a_packed & 1);
  const int a_row = gather ? ((lane & 1) ? w.a_row_hi : w.a_row_lo) + 16 * ((lane & 7) >> 1)
                           : (slab2 ? 2 * w.a_row_lo : w.a_row_lo);
  const int n_a = gather ? 8 : 1;
  // read once: the record lives in shared memory and every copy below is a memory barrier to the compiler
  const bool fetch = kFetch && w.fetch != 0;
  const uint32_t fetch_bytes = kFetch ? w.fetch_bytes : 0;
  const uint8_t* const fetch_src = kFetch ? w.fetch_src : nullptr;
  const CUtensorMap* const a_map = w.a_map;
  const CUtensorMap* const b_map = w.b_map;
  const int a_z = w.a_z, b_row0 = w.b_row0, k0 = w.k0;
  const uint32_t tx_bytes = kATileBytes + ks * b_bytes;
  for (int st = 0; st < n_stages; ++st) {
    uint32_t vb, ve;
    const uint32_t phys = pipe.alloc(size, vb, ve);
    // room in the ring and a free barrier pair: retire the oldest stages as needed
    while (pipe.i - fl.tail >= kGemmStages || (pipe.i != fl.tail && ve - fl.vbegin[fl.tail_slot] > kRingBytes)) {
      if (!mbar_wait_bounded(&bar.empty[fl.tail_slot], fl.tail_parity, abort_flag, kWaitBudgetNs)) return false;
      ++fl.tail;
      if (++fl.tail_slot == kGemmStages) {
        fl.tail_slot = 0;
        fl.tail_parity ^= 1;
      }
    }
    const uint32_t slot = pipe.slot;
    fl.vbegin[slot] = vb;
    uint8_t* a = ring + phys;
    uint64_t* full = &bar.full[slot];
    if (fetch) {
      if (lane == 0) {
        const uint32_t at = st * kFetchStageBytes;
        const uint32_t bytes = min(kFetchStageBytes, fetch_bytes - at);
        mbar_arrive_expect_tx(full, bytes);
        bulk_load(a, fetch_src + at, bytes, full, pol_w);
      }
      __syncwarp();
      pipe.advance();
      continue;
    }
    // the second K step of an odd K range's last stage is loaded but not multiplied (gemm_mma)
    if (lane == 0) mbar_arrive_expect_tx(full, tx_bytes);
    __syncwarp();
    const int x = (k0 + st * ks) * kBlockK;
    if (lane < n_a) {
      tma_load_3d(a + a_off + lane * a_box, a_map, full, x, a_row, a_z, pol_w);
    } else if (lane >= 8 && lane < 8 + ks) {
      tma_load_2d(a + b_off + (lane - 8) * b_bytes, b_map, full, x + (lane - 8) * kBlockK, b_row0, pol_x);
    }
    pipe.advance();
  }
  return true;
}

// MMA issue for one tile into accumulator buffer `buf`.  The whole MMA warp runs the K loop in
// step (every lane waits for the stage itself, so the loop needs no warp barrier) and one elected
// lane issues the four tcgen05.mma and the commit of a stage.  Because the loop is convergent code,
// its descriptors and addresses are warp-uniform values; with the loop inside a single-lane branch
// the MMA warp spent twice as long issuing (measured: 67 -> 32 us of a 150 us launch), which is
// what bounds small-N tiles.
template <bool kFetch = true>
__device__ __forceinline__ bool gemm_mma(const GemmWork& w, uint8_t* ring, GemmBarriers& bar, GemmPipe& pipe,
                                         uint32_t tmem_base, int buf, uint32_t acc_parity, volatile int* abort_flag,
                                         long long* wait_cycles = nullptr) {
  int ok = 1;
  const bool leader = elect_one();
  {
    const long long ta = wait_cycles ? clock64() : 0;
    if (!mbar_wait_bounded(&bar.acc_empty[buf], acc_parity ^ 1, abort_flag, kWaitBudgetNs)) ok = 0;
    if (wait_cycles) wait_cycles[2] += clock64() - ta;
    tc_fence_after_sync();
    const uint32_t idesc = umma_idesc_bf16(128, w.n);
    const uint32_t acc = tmem_base + buf * kAccCols;
    const uint32_t size = gemm_stage_bytes<kFetch>(w);
    uint64_t* ready = w.w_fp8 ? bar.conv : bar.full;
    const uint32_t ring_addr = smem_u32(ring);
    const uint64_t desc0 = umma_desc_sw128(0);
    const int n_stages = gemm_stage_count<kFetch>(w);
    const uint32_t b_bytes = w.n * kBlockK * 2;
    // read once: the record lives in shared memory and every wait below is a memory barrier to the compiler
    const bool fp8 = w.w_fp8 != 0, fetch = kFetch && w.fetch != 0;
    const int k_steps = w.k_tiles;
    const uint32_t fetch_bytes = kFetch ? w.fetch_bytes : 0;
    uint8_t* const fetch_out = static_cast<uint8_t*>(w.out);
    for (int kt = 0; ok && kt < n_stages; ++kt) {
      uint32_t vb, ve;
      const uint32_t phys = pipe.alloc(size, vb, ve);
      const long long tw = wait_cycles ? clock64() : 0;
      const uint32_t ready_parity = fp8 ? (pipe.conv_bits >> pipe.slot) & 1u : pipe.parity;
      if (!mbar_wait_bounded(&ready[pipe.slot], ready_parity, abort_flag, kWaitBudgetNs)) {
        ok = 0;
        break;
      }
      if (fp8) pipe.conv_bits ^= 1u << pipe.slot;
      if (wait_cycles) wait_cycles[0] += clock64() - tw;
      if (fetch) {
        // the stage goes on to the staging buffer; its shared memory is free once the store has read it
        if (leader) {
          const uint32_t at = kt * kFetchStageBytes;
          bulk_store(fetch_out + at, ring + phys, min(kFetchStageBytes, fetch_bytes - at));
          bulk_commit();
          bulk_wait_read_all();
          mbar_arrive(&bar.empty[pipe.slot]);
        }
        pipe.advance();
        continue;
      }
      const long long ti = wait_cycles ? clock64() : 0;
      if (!leader) {
      } else if (!fp8) {   // one K step: weight tile, activation tile
        const uint64_t da = desc0 + ((ring_addr + phys) >> 4);
        const uint64_t db = da + (kATileBytes >> 4);
#pragma unroll
        for (int k = 0; k < kBlockK / 16; ++k) umma_bf16(acc, da + 2 * k, db + 2 * k, idesc, (kt | k) != 0);
      } else {      // two K steps: weight tiles 0 and 1, then activation tiles 0 and 1
        const uint64_t da = desc0 + ((ring_addr + phys) >> 4);
        const uint64_t db = da + (2 * kATileBytes >> 4);
#pragma unroll
        for (int k = 0; k < kBlockK / 16; ++k) umma_bf16(acc, da + 2 * k, db + 2 * k, idesc, (kt | k) != 0);
        // the last stage of an odd K range holds one K step of the range; its second half belongs to the
        // next range (a K split) or lies past the tensor, and is left out
        if (2 * kt + 1 < k_steps) {
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k)
            umma_bf16(acc, da + (kATileBytes >> 4) + 2 * k, db + (b_bytes >> 4) + 2 * k, idesc, true);
        }
      }
      if (leader) umma_commit(&bar.empty[pipe.slot]);
      if (wait_cycles) wait_cycles[1] += clock64() - ti;
      pipe.advance();
    }
    if (ok && fetch) {
      // the record counts as done when its bytes are in the staging buffer, for readers of either proxy
      if (leader) {
        bulk_wait_all();
        fence_proxy_async_all();
        __threadfence();
        mbar_arrive(&bar.acc_full[buf]);
      }
    } else if (ok && leader) {
      umma_commit(&bar.acc_full[buf]);
    }
  }
  return __all_sync(0xffffffffu, ok != 0);
}

// FP8 weights (W8A16, csrc/fabric/tiles/gemm.cuh:14-18,73-94): the four converter
// warps expand the raw e4m3 tile of every stage into the bf16 weight tile with the
// 128-byte swizzle.  Every e4m3 value is exactly a bf16 value, so the MMA sees the
// exact weights; the per-output-channel fp32 scale is applied in the epilogue.
// Thread t converts row t: per K step 64 bytes in, 128 bytes out in eight 16-byte chunks,
// chunk c of row r going to chunk c ^ (r & 7).
__device__ __forceinline__ bool gemm_convert(const GemmWork& w, uint8_t* ring, GemmBarriers& bar, GemmPipe& pipe,
                                             int row, volatile int* abort_flag) {
  const uint32_t size = gemm_stage_bytes(w);
  const int ks = gemm_ksteps(w), n_stages = gemm_stage_count(w);
  const uint32_t raw_off = kATileBytes;
  for (int kt = 0; kt < n_stages; ++kt) {
    uint32_t vb, ve;
    const uint32_t phys = pipe.alloc(size, vb, ve);
    if (!mbar_wait_bounded(&bar.full[pipe.slot], pipe.parity, abort_flag, kWaitBudgetNs)) return false;
    // The row's raw bytes [64 h, 64 h + 64) are K step h.  The thread reads its whole row before it
    // writes (the second K step's output overwrites the raw row), starting at 16-byte chunk t & 7 so
    // that the eight threads of a shared-memory phase read eight different bank groups.
    const uint4* src = reinterpret_cast<const uint4*>(ring + phys + raw_off + row * 128);
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = src[(i + row) & 7];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int q = (i + row) & 7, h = q >> 2, c = q & 3;
      uint8_t* dst = ring + phys + h * kATileBytes + row * 128;
      const uint32_t in[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
      uint32_t out[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(in[j] & 0xffffu), __NV_E4M3);
        const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(in[j] >> 16), __NV_E4M3);
        const float2 fl = __half22float2(*reinterpret_cast<const __half2*>(&lo));
        const float2 fh = __half22float2(*reinterpret_cast<const __half2*>(&hi));
        const __nv_bfloat162 bl = __floats2bfloat162_rn(fl.x, fl.y), bh = __floats2bfloat162_rn(fh.x, fh.y);
        out[2 * j] = *reinterpret_cast<const uint32_t*>(&bl);
        out[2 * j + 1] = *reinterpret_cast<const uint32_t*>(&bh);
      }
      // 16 input bytes -> 32 output bytes = chunks 2c and 2c + 1 of the row
      *reinterpret_cast<uint4*>(dst + (((2 * c) ^ (row & 7)) << 4)) = make_uint4(out[0], out[1], out[2], out[3]);
      *reinterpret_cast<uint4*>(dst + (((2 * c + 1) ^ (row & 7)) << 4)) = make_uint4(out[4], out[5], out[6], out[7]);
    }
    fence_proxy_async_smem();   // generic-proxy writes -> visible to the tensor core's operand reads
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(&bar.conv[pipe.slot]);
    pipe.advance();
  }
  return true;
}

__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }

// Epilogue of one tile from accumulator buffer `buf` (the four epilogue warps
// call): everything except handing the buffer back to the MMA warp.
template <bool kFetch = true>
__device__ __forceinline__ bool gemm_epilogue_body(const GemmWork& w, GemmBarriers& bar, uint32_t tmem_base, int buf,
                                                   uint32_t acc_parity, volatile int* abort_flag,
                                                   unsigned long long* acc_seen = nullptr) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, quad = warp & 3;
  if (!mbar_wait_bounded(&bar.acc_full[buf], acc_parity, abort_flag, kWaitBudgetNs)) return false;
  tc_fence_after_sync();
  if (acc_seen && lane == 0) *acc_seen = globaltimer_ns();
  if (kFetch && w.fetch) {   // nothing to drain: the MMA warp has already moved the bytes
    __syncwarp();
    return true;
  }
  const uint32_t tacc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * kAccCols;
  const bool silu = w.epi == kEpiSiluMul;
  // output feature of this lane, and the weight row its accumulator row came from
  int f, wrow;
  if (silu || (w.a_packed & 4)) {
    f = w.a_row_lo + 16 * quad + (lane & 15);
    wrow = (lane < 16 ? w.a_row_lo : w.a_row_hi) + 16 * quad + (lane & 15);
  } else {
    f = w.a_row_lo + 32 * quad + lane;
    wrow = f;
  }
  const bool f_ok = f < w.n_limit;
  const float sc = (w.scale && f_ok) ? w.scale[wrow] : 1.f;
  const float bias = (w.bias && f_ok && w.k0 == 0) ? __bfloat162float(w.bias[f]) : 0.f;
  for (int c0 = 0; c0 < w.n; c0 += 32) {
    uint32_t r[32];
    if (w.n - c0 >= 32) {
      tmem_ld_32x32(tacc + c0, r);
    } else {
      uint32_t r16[16];
      tmem_ld_32x16(tacc + c0, r16);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        r[j] = r16[j];
        r[16 + j] = 0;
      }
    }
    tmem_ld_wait();
    if (c0 >= w.rows) continue;
    if (silu) {
      // lanes < 16 own gate rows, lanes >= 16 the matching up rows; exchange halves
      const bool lo = lane < 16;
      const int t0 = c0 + (lo ? 0 : 16);
      unsigned short* out = reinterpret_cast<unsigned short*>(w.out) + static_cast<size_t>(w.b_row0 + t0) * w.ld_out + f;
      unsigned short hv[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float mine_keep = __uint_as_float(lo ? r[j] : r[16 + j]) * sc;
        const float send = __uint_as_float(lo ? r[16 + j] : r[j]) * sc;
        const float other = __shfl_xor_sync(0xffffffffu, send, 16);
        hv[j] = __bfloat16_as_ushort(__float2bfloat16(silu_mul(lo ? mine_keep : other, lo ? other : mine_keep)));
      }
      if (f_ok) {
        const int m_hi = w.rows - t0;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (j < m_hi) out[static_cast<size_t>(j) * w.ld_out] = hv[j];
      }
    } else if (w.epi == kEpiStoreBf16) {
      __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(w.out) + static_cast<size_t>(w.b_row0 + c0) * w.ld_out + f;
      const __nv_bfloat16* res =
          w.residual ? w.residual + static_cast<size_t>(w.b_row0 + c0) * w.ld_res + f : nullptr;
      if (f_ok) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (c0 + j < w.rows) {
            float v = __uint_as_float(r[j]) * sc + bias;
            if (res) v += __bfloat162float(res[static_cast<size_t>(j) * w.ld_res]);
            __stcs(reinterpret_cast<unsigned short*>(out + static_cast<size_t>(j) * w.ld_out),
                   __bfloat16_as_ushort(__float2bfloat16(v)));
          }
        }
      }
    } else if (w.epi == kEpiWeightedAdd) {
      float* out = reinterpret_cast<float*>(w.out) + f;
      if (f_ok) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (c0 + j < w.rows) {
            const int m = w.b_row0 + c0 + j;
            atomicAdd(out + static_cast<size_t>(w.pair_token[m]) * w.ld_out,
                      w.pair_weight[m] * (__uint_as_float(r[j]) * sc));
          }
        }
      }
    } else if (w.epi == kEpiAtomicF32) {
      // a two-slab tile (partial sums of a SwiGLU pair) adds into the column of its weight row
      float* out = reinterpret_cast<float*>(w.out) + static_cast<size_t>(w.b_row0 + c0) * w.ld_out + ((w.a_packed & 4) ? wrow : f);
      if (f_ok) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (c0 + j < w.rows) atomicAdd(out + static_cast<size_t>(j) * w.ld_out, __uint_as_float(r[j]) * sc + bias);
      }
    } else {
      // fp32 rows that are read once, later (per-pair expert outputs, logits): streaming stores
      float* out = reinterpret_cast<float*>(w.out) + static_cast<size_t>(w.b_row0 + c0) * w.ld_out + f;
      if (f_ok) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (c0 + j < w.rows) __stcs(out + static_cast<size_t>(j) * w.ld_out, __uint_as_float(r[j]) * sc + bias);
      }
    }
  }
  tc_fence_before_sync();
  __syncwarp();
  return true;
}

template <bool kFetch = true>
__device__ __forceinline__ bool gemm_epilogue(const GemmWork& w, GemmBarriers& bar, uint32_t tmem_base, int buf,
                                              uint32_t acc_parity, volatile int* abort_flag,
                                              unsigned long long* acc_seen = nullptr) {
  if (!gemm_epilogue_body<kFetch>(w, bar, tmem_base, buf, acc_parity, abort_flag, acc_seen)) return false;
  if ((threadIdx.x & 31) == 0) mbar_arrive(&bar.acc_empty[buf]);
  return true;
}

}  // namespace mf
