// The persistent fabric kernel: one worker (CTA) per SM runs tiles of the lanes'
// programs until the host asks it to leave.
//
// Scheduling protocol (the reference's, csrc/fabric/runtime.cuh:155-509, restated):
//   * a lane's program is a DAG of stages; an ACTIVE stage sits in one of the
//     lane's two rings (ungated / link) as tag << 20 | stage;
//   * a worker takes tiles of its own lane first, then of other lanes in the
//     published borrowing order; link stages only while it holds one of the
//     lane's `cap` link slots;
//   * a claim is one fetch-and-add on the stage's tag_next word for 1..8 tiles;
//   * the worker that completes a stage's last tile decrements the successors'
//     dependency counts and activates those that reach zero; the reset stage
//     ends an iteration: swap in a newer program, stop after N, or start again;
//   * the host publishes plans (worker->lane map, credits, order, programs) as
//     epochs through a double-buffered snapshot that workers re-read with a
//     seqlock-style double read.
// What differs from the reference, on purpose:
//   * a worker is warp-specialised: warp 0 schedules and runs AHEAD of the data
//     path through a four-deep ring of work records, so claims, descriptor loads
//     and epoch refreshes overlap the previous tile; warps 1..4 execute tiles and
//     are the epilogue of GEMM tiles; warp 5 issues the TMA copies and warp 6 owns
//     TMEM and issues tcgen05.mma (gemm_core.cuh), with accumulators double-buffered
//     across consecutive GEMM tiles; for FP8-e4m3 weights the exec warps are also the
//     converters of every operand stage (W8A16); an attention work item (attention_core.cuh) uses
//     the same three roles with the operand ring as its Q / K / V / P tiles, after the
//     worker's earlier tiles have drained;
//   * no wait is unbounded and nothing traps: a ring publication that waits too
//     long, a full worklist or an unknown tile kind raise an error bit that the
//     host reads from the mirror, and the kernel leaves by itself after
//     max_run_ns, so a fabric that owns every SM can always be stopped.
#include <cuda_runtime.h>

#include "attention_core.cuh"
#include "fabric_sched.cuh"
#include "fabric_types.h"
#include "gemm_core.cuh"
#include "operands.h"
#include "ptx.cuh"
#include "rowwise.cuh"

namespace mf {
namespace fab {

constexpr int kExecThreads = 128;
constexpr int kSlots = 4;   // work records the scheduler may run ahead of the exec warps
constexpr int kWorkerThreads = 32 + kExecThreads + 64;   // scheduler, exec/epilogue, TMA producer, MMA

__device__ __forceinline__ unsigned int smid() {
  unsigned int v;
  asm volatile("mov.u32 %0, %smid;" : "=r"(v));
  return v;
}

struct WorkSlot {
  TileDesc tile;
  GemmWork gemm;          // filled by the scheduler for GEMM tiles
  AttnWork attn;          // filled by the scheduler for attention work items
  const ProgramDesc* prog;
  uint32_t stage, tile_lane, link, index, cmd, worker_lane, is_gemm, is_attn;
  uint32_t counts, pad;   // counts: this record completes its tile (0 for all but the last row block of a kind-45 tile)
};

// A GEMM tile (kind 32) in the reference's operand convention
// (csrc/fabric/model_types.h:37-49): a[0] GemmArgs*, a[1] weight map record,
// a[2] activation map record, a[3] K range = first K tile | K tiles << 16 (0 = all),
// a[4] fp32 scale per weight row; i0 first weight row, i1 first activation row,
// i2 valid activation rows, i3 weight z (expert or slot).  A map record is four
// 128-byte slots (monofab_fabric_tensor_map): [0] the caller's box, [1] box
// (64, 16, 1), [2] box (64, 128, 1), [3] flags: word 0 = 1 when a w13 tensor is
// stored in the packed SwiGLU row order (monofab_pack_w13).
// A tile of kind 45 (csrc/fabric/model_types.h:47-49: one K range of the slice against all i2 rows of its
// expert) runs as one record per block of bm rows, `block` naming the record's block: the same symmetric tile
// with the K range a[3], rows [i1 + block * bm, ...).  Its epilogue adds (kEpiAtomicF32 / kEpiWeightedAdd), so
// the blocks and K ranges may complete in any order.  With up_offset set and kEpiAtomicF32 the slice is the
// 64 gate rows at i0 and the 64 up rows at up_offset + i0, and a partial sum goes to column = weight row (the
// layout the reduce tile, kind 46, reads).  The weights of the slice are re-read per row block (from L2 when
// they are in HBM); the staged form is this library's own answer to reading a host-resident expert once.
__device__ bool make_gemm_work(const TileDesc& t, GemmWork& w, uint32_t block = 0) {
  GemmArgs A;
  const uint4* src = reinterpret_cast<const uint4*>(t.a[0]);
  uint4* dst = reinterpret_cast<uint4*>(&A);
#pragma unroll
  for (int i = 0; i < 8; ++i) dst[i] = __ldcg(src + i);
  if (A.bm < 16 || A.bm > kGemmMaxN || (A.bm & (A.bm - 1))) return false;
  const CUtensorMap* wrec = reinterpret_cast<const CUtensorMap*>(t.a[1]);
  const CUtensorMap* xrec = reinterpret_cast<const CUtensorMap*>(t.a[2]);
  const bool silu = A.epi == kEpiSiluMul;
  const bool atomic_slabs = A.epi == kEpiAtomicF32 && A.up_offset != 0;
  const bool packed = silu && __ldcg(reinterpret_cast<const unsigned int*>(wrec + 3)) != 0;
  w.a_map = ((silu && !packed) || atomic_slabs) ? wrec + 1 : wrec + 2;
  w.b_map = xrec;
  w.out = reinterpret_cast<void*>(A.out);
  w.scale = reinterpret_cast<const float*>(t.a[4]);
  w.bias = reinterpret_cast<const __nv_bfloat16*>(A.bias);
  w.residual = reinterpret_cast<const __nv_bfloat16*>(A.residual);
  w.pair_token = reinterpret_cast<const int32_t*>(A.pair_token);
  w.pair_weight = reinterpret_cast<const float*>(A.pair_weight);
  w.a_row_lo = t.i0;
  w.a_row_hi = A.up_offset + t.i0;
  w.a_z = t.i3;
  const uint32_t row_off = block * A.bm;
  if (row_off >= t.i2 && t.i2 != 0) return false;
  w.b_row0 = t.i1 + row_off;
  w.rows = t.i2 - row_off < A.bm ? t.i2 - row_off : A.bm;
  w.n = A.bm;
  const uint32_t k0 = static_cast<uint32_t>(t.a[3] & 0xffff), kn = static_cast<uint32_t>((t.a[3] >> 16) & 0xffff);
  w.k0 = kn ? k0 : 0;
  w.k_tiles = kn ? kn : A.k_tiles;
  w.epi = A.epi;
  w.ld_out = A.ld_out;
  w.ld_res = A.ld_res;
  w.n_limit = A.n_limit;
  w.valid = 1;
  w.a_packed = (packed ? 1 : 0) | (atomic_slabs ? 4 : 0);
  w.block = -1;
  w.w_fp8 = A.w_fp8 != 0;   // e4m3 weights: the exec warps expand every stage to bf16 before its MMAs
  w.fetch = 0;
  return w.k_tiles > 0 && A.epi <= kEpiRowsF32;
}

// Fetch tile (kind 49): i0 bytes from a[0] (host-resident weights) to a[1] (an HBM staging buffer).
// It runs through the GEMM roles as a record without MMAs: the producer's bulk loads fill ring
// stages, the MMA warp stores each stage to the destination, the exec warps only keep step.
__device__ bool make_fetch_work(const TileDesc& t, GemmWork& w) {
  w.a_map = nullptr;
  w.b_map = nullptr;
  w.out = reinterpret_cast<void*>(t.a[1]);
  w.scale = nullptr;
  w.bias = nullptr;
  w.residual = nullptr;
  w.pair_token = nullptr;
  w.pair_weight = nullptr;
  w.a_row_lo = w.a_row_hi = w.a_z = w.b_row0 = w.rows = 0;
  w.n = 16;
  w.k0 = 0;
  w.k_tiles = 1;
  w.epi = kEpiStoreBf16;
  w.ld_out = w.ld_res = w.n_limit = 0;
  w.valid = 1;
  w.a_packed = 0;
  w.block = -1;
  w.w_fp8 = 0;
  w.fetch = 1;
  w.fetch_bytes = t.i0;
  w.fetch_src = reinterpret_cast<const uint8_t*>(t.a[0]);
  return t.i0 > 0 && ((t.i0 | t.a[0] | t.a[1]) & 15) == 0 && t.a[0] != 0 && t.a[1] != 0;
}

// ---------------------------------------------------------------- core tiles
__device__ __forceinline__ void exec_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kExecThreads) : "memory"); }
// Barrier of the exec threads that also tells each whether `v` held in all of them.
__device__ __forceinline__ bool exec_all(bool v) {
  int r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %1, 0;\n\tbar.red.and.pred p, 1, %2, q;\n\tselp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(static_cast<int>(v)), "n"(kExecThreads)
      : "memory");
  return r != 0;
}

__device__ void trace_tile(unsigned long long base, uint32_t idx, unsigned long long t0, unsigned long long t1,
                           uint32_t lane, uint32_t worker) {
  if (base == 0) return;
  TraceRec* r = reinterpret_cast<TraceRec*>(base) + idx;
  r->start_ns = t0;
  r->end_ns = t1;
  r->worker = worker;
  r->sm = smid();
  r->lane = lane;
  atomicAdd(&r->count, 1u);
}

// Scratch of the tile the exec warps are running; tiles run one at a time per worker,
// so they share one block instead of each holding static shared memory of its own.
constexpr int kExecScratchInts = 5 * (kMaxExperts + 1) + 16 + 64;
__shared__ __align__(16) int s_exec_scratch[kExecScratchInts];

}  // namespace fab
}  // namespace mf
#include "fabric_seq_tiles.cuh"
namespace mf {
namespace fab {

__device__ void tile_router(const TileDesc& t, int tid);
__device__ void tile_norm(const TileDesc& t, int tid, bool add);
__device__ void tile_router_logits(const TileDesc& t, int tid);
__device__ void tile_permute(const TileDesc& t, int tid);
__device__ void tile_combine(const TileDesc& t, int tid);
__device__ void tile_asym_reduce(const TileDesc& t, int tid);
__device__ void tile_norm_logits(const TileDesc& t, int tid);
__device__ void tile_expand(const TileDesc& t, const ProgramDesc* P, DeviceState& S, int tid);

// tid: index among the exec threads.
__device__ bool run_core_tile(DeviceState& S, const WorkSlot& w, int tid, uint32_t worker, unsigned long long* sh_t0) {
  const TileDesc& t = w.tile;
  switch (t.kind) {
    case kTileNop:
      return true;
    case kTileSpin:
      if (tid == 0) {
        const unsigned long long t0 = globaltimer_ns();
        const unsigned long long dur = t.a[0] < 1000000000ull ? t.a[0] : 1000000000ull;   // never spin for more than a second
        while (globaltimer_ns() - t0 < dur) {
        }
        trace_tile(t.a[1], t.i0, t0, globaltimer_ns(), t.i1, worker);
      }
      return true;
    case kTileRead: {
      if (tid == 0) *sh_t0 = globaltimer_ns();
      const uint4* p = reinterpret_cast<const uint4*>(t.a[0]);
      const size_t n = t.a[1] / 16;
      unsigned int acc = 0;
      for (size_t i = tid; i < n; i += kExecThreads) {
        const uint4 v = ld_nc_stream16(p + i);
        acc ^= v.x ^ v.y ^ v.z ^ v.w;
      }
      if (acc == 0x9e3779b9u && t.a[2] != 0) reinterpret_cast<unsigned int*>(t.a[2])[worker] = acc;
      exec_sync();
      if (tid == 0) trace_tile(t.a[3], t.i0, *sh_t0, globaltimer_ns(), t.i1, worker);
      return true;
    }
    case kTileProbe:
      if (tid == 0) {
        const volatile unsigned long long* base = reinterpret_cast<const volatile unsigned long long*>(t.a[0]);
        unsigned long long idx = 0;
        const unsigned long long t0 = globaltimer_ns();
        for (uint32_t i = 0; i < t.i0; ++i) idx = base[idx];
        const unsigned long long t1 = globaltimer_ns();
        unsigned long long* out = reinterpret_cast<unsigned long long*>(t.a[1]);
        out[t.i1] = (t1 - t0) * 1000ull / (t.i0 ? t.i0 : 1);   // picoseconds per load
        out[t.i1 + 1] = idx;
      }
      return true;
    case kTileZeroRuntime:
      for (uint32_t s = t.i0 + tid; s < t.i1; s += kExecThreads) {
        if (s == t.i2) continue;
        w.prog->runtime[s].done = 0;
        w.prog->runtime[s].deps = w.prog->stages[s].deps_init;
      }
      __threadfence();
      return true;
    case kTileRouter:
      tile_router(t, tid);
      return true;
    case kTileRouterLogits:
      tile_router_logits(t, tid);
      return true;
    case kTilePermute:
      tile_permute(t, tid);
      return true;
    case kTileCombine:
      tile_combine(t, tid);
      return true;
    case kTileAsymReduce:
      tile_asym_reduce(t, tid);
      return true;
    case kTileNormLogits:
      tile_norm_logits(t, tid);
      return true;
    case kTileExpand:
      tile_expand(t, w.prog, S, tid);
      return true;
    case kTileRmsNorm:
      tile_norm(t, tid, false);
      return true;
    case kTileAddNorm:
      tile_norm(t, tid, true);
      return true;
    case kTileAttnMerge:
      tile_attn_merge(t, tid);
      return true;
    case kTileQkRope:
      tile_qk_rope(t, tid);
      return true;
    case kTileEmbed:
      tile_embed(t, tid);
      return true;
    case kTileSample:
      tile_sample(t, tid);
      return true;
    case kTileAttnPlan:
      tile_attn_plan(t, w.prog, S, tid);
      return true;
    default:
      return false;
  }
}

// ----------------------------------------------------------- row-wise model tiles
// Row-wise tiles name rows [i0, i0 + i1); a[0] is the operand block.  One warp per
// row, the four exec warps striding over the rows.

// Reduce tile of the K-split w13 (kind 46, csrc/fabric/model_types.h:196-204, ReduceArgs) for rows
// [i0, i0 + i1): h[r][f] = bf16(silu(gate) * up) from the fp32 partial sums ws[r][f] and ws[r][I + f],
// whose row is then zeroed for the next layer.  One warp per row.
__device__ void tile_asym_reduce(const TileDesc& t, int tid) {
  ReduceArgs A;
  load_block(A, t.a[0]);
  const int warp = tid >> 5, lane = tid & 31;
  const uint32_t I = A.I;
  for (uint32_t r = t.i0 + warp; r < t.i0 + t.i1; r += kExecThreads / 32) {
    float* ws = reinterpret_cast<float*>(A.ws) + static_cast<size_t>(r) * A.ld_ws;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(A.out) + static_cast<size_t>(r) * A.ld_out;
    for (uint32_t f = lane; f < I; f += 32) {
      const float g = __ldcg(ws + f), u = __ldcg(ws + I + f);
      out[f] = __float2bfloat16(silu_mul(g, u));
      ws[f] = 0.f;
      ws[I + f] = 0.f;
    }
  }
}

// Router tile (kind 38, csrc/fabric/tiles/aux.cuh:326-417, RouterArgs): scores,
// top-K, renormalisation, per-expert counts; the logits row is zeroed once read.
// With chunk_counts set (a field this library adds) the tile counts every pick into
// chunk_counts[row / kFabChunk][expert] instead of counts[expert]: integer adds, so the
// result does not depend on the order in which tiles run; the expand tile turns these
// per-chunk counts into prefixes and the permute tiles into the stable pack order.
__device__ void tile_router(const TileDesc& t, int tid) {
  RouterArgs A;   // a copy in registers: the block lives in global memory
  load_block(A, t.a[0]);
  const int warp = tid >> 5, lane = tid & 31;
  const int E = static_cast<int>(A.E), K = static_cast<int>(A.K);
  if (E < 1 || E > kMaxExperts || K < 1 || K > kMaxTopK) return;
  int* chunk_counts = reinterpret_cast<int*>(A.chunk_counts);
  for (uint32_t r = t.i0 + warp; r < t.i0 + t.i1; r += kExecThreads / 32) {
    int id;
    float w;
    route_row(reinterpret_cast<float*>(A.logits) + static_cast<size_t>(r) * E, reinterpret_cast<const float*>(A.bias),
              E, K, static_cast<int>(A.scoring), static_cast<int>(A.renorm), A.scale, 1, id, w);
    if (lane < K) {
      reinterpret_cast<int*>(A.topk_ids)[static_cast<size_t>(r) * K + lane] = id;
      reinterpret_cast<float*>(A.topk_w)[static_cast<size_t>(r) * K + lane] = w;
      if (chunk_counts) atomicAdd(chunk_counts + static_cast<size_t>(r / kFabChunk) * E + id, 1);
      else if (A.counts) atomicAdd(reinterpret_cast<int*>(A.counts) + id, 1);
    }
  }
}

// Router projection tile (kind 48; not in the reference, whose router GEMM sums
// K-split partials with atomics): logits[t][e] for rows [i0, i0 + i1) and experts
// [i2, i2 + i3) (i3 = 0: all), lane l summing h = 256 j + 8 l + i in order with fmaf, then
// the xor butterfly: the same bits as the stream kernel and the oracle.  A warp keeps one
// expert's weight row in registers and walks the tile's rows, so the weights are read
// once per tile and the activation rows come from L1.
template <int J>
__device__ __forceinline__ void router_logits_rows(const __nv_bfloat16* x, const __nv_bfloat16* wr, float* logits, int H,
                                                   int E, int r0, int rows, int e_lo, int e_hi, int warp, int lane) {
  if constexpr (J > 0) {
    // two experts' weight rows in registers, two activation rows at a time: four independent
    // fmaf chains per lane, each in the defined order
    for (int e = e_lo + 2 * warp; e < e_hi; e += 2 * (kExecThreads / 32)) {
      const bool two_e = e + 1 < e_hi;
      const uint4* wa = reinterpret_cast<const uint4*>(wr + static_cast<size_t>(e) * H);
      const uint4* wb = reinterpret_cast<const uint4*>(wr + static_cast<size_t>(two_e ? e + 1 : e) * H);
      uint4 wva[J > 0 ? J : 1], wvb[J > 0 ? J : 1];
#pragma unroll
      for (int j = 0; j < J; ++j) {
        wva[j] = __ldg(wa + 32 * j + lane);
        wvb[j] = __ldg(wb + 32 * j + lane);
      }
      for (int r = r0; r < r0 + rows; r += 2) {
        const bool two_r = r + 1 < r0 + rows;
        const uint4* xa = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * H);
        const uint4* xb = reinterpret_cast<const uint4*>(x + static_cast<size_t>(two_r ? r + 1 : r) * H);
        float a00 = 0.f, a01 = 0.f, a10 = 0.f, a11 = 0.f;   // a[row][expert]
#pragma unroll
        for (int j = 0; j < J; ++j) {
          float x0[8], x1[8], w0[8], w1[8];
          unpack8(xa[32 * j + lane], x0);
          unpack8(xb[32 * j + lane], x1);
          unpack8(wva[j], w0);
          unpack8(wvb[j], w1);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            a00 = __fmaf_rn(x0[i], w0[i], a00);
            a01 = __fmaf_rn(x0[i], w1[i], a01);
            a10 = __fmaf_rn(x1[i], w0[i], a10);
            a11 = __fmaf_rn(x1[i], w1[i], a11);
          }
        }
        a00 = warp_sum_xor(a00);
        a01 = warp_sum_xor(a01);
        a10 = warp_sum_xor(a10);
        a11 = warp_sum_xor(a11);
        if (lane == (e & 31)) {
          logits[static_cast<size_t>(r) * E + e] = a00;
          if (two_r) logits[static_cast<size_t>(r + 1) * E + e] = a10;
        }
        if (two_e && lane == ((e + 1) & 31)) {
          logits[static_cast<size_t>(r) * E + e + 1] = a01;
          if (two_r) logits[static_cast<size_t>(r + 1) * E + e + 1] = a11;
        }
      }
    }
  } else {
    const int nj = H / 256;
    for (int e = e_lo + warp; e < e_hi; e += kExecThreads / 32) {
      const uint4* w4 = reinterpret_cast<const uint4*>(wr + static_cast<size_t>(e) * H);
      for (int r = r0; r < r0 + rows; ++r) {
        const uint4* x4 = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * H);
        float acc = 0.f;
        for (int j = 0; j < nj; ++j) {
          float xf[8], wf[8];
          unpack8(x4[32 * j + lane], xf);
          unpack8(__ldg(w4 + 32 * j + lane), wf);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc = __fmaf_rn(xf[i], wf[i], acc);
        }
        acc = warp_sum_xor(acc);
        if (lane == (e & 31)) logits[static_cast<size_t>(r) * E + e] = acc;
      }
    }
  }
}

__device__ void tile_router_logits(const TileDesc& t, int tid) {
  LogitsArgs A;   // a copy in registers: the block lives in global memory
  load_block(A, t.a[0]);
  const int warp = tid >> 5, lane = tid & 31;
  const int H = static_cast<int>(A.H), E = static_cast<int>(A.E);
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(A.x);
  const __nv_bfloat16* wr = reinterpret_cast<const __nv_bfloat16*>(A.wr);
  float* logits = reinterpret_cast<float*>(A.logits);
  const int e_lo = static_cast<int>(t.i2), e_hi = t.i3 ? min(E, e_lo + static_cast<int>(t.i3)) : E;
  const int r0 = static_cast<int>(t.i0), rows = static_cast<int>(t.i1);
  switch (H / 256) {
    case 2: router_logits_rows<2>(x, wr, logits, H, E, r0, rows, e_lo, e_hi, warp, lane); break;
    case 4: router_logits_rows<4>(x, wr, logits, H, E, r0, rows, e_lo, e_hi, warp, lane); break;
    case 8: router_logits_rows<8>(x, wr, logits, H, E, r0, rows, e_lo, e_hi, warp, lane); break;
    default: router_logits_rows<0>(x, wr, logits, H, E, r0, rows, e_lo, e_hi, warp, lane); break;
  }
}

// Permute tile (kind 40, csrc/fabric/tiles/aux.cuh:648-684, PermuteArgs) for rows
// [i0, i0 + i1) of ONE chunk of kFabChunk rows: pair lists and expert-sorted activation rows.
// With chunk_prefix set the position of pair (token, pick) is
//   starts[e] + pairs of e in earlier chunks + pairs of e earlier in this chunk
// (token ascending, pick ascending: the stable pack), the last term counted here from
// the chunk's ids; otherwise the reference's arrival order through atomicAdd(fill[e]).
// pair_pos (optional) receives the packed row of every pair.
__device__ void tile_permute(const TileDesc& t, int tid) {
  int* const s_ids = s_exec_scratch;   // ids of the chunk's rows up to the end of this tile
  PermuteArgs A;   // a copy in registers: the block lives in global memory
  load_block(A, t.a[0]);
  const int warp = tid >> 5, lane = tid & 31;
  const int K = static_cast<int>(A.K), H = static_cast<int>(A.H), E = static_cast<int>(A.E), n16 = H / 8;
  const int* ids = reinterpret_cast<const int*>(A.topk_ids);
  const float* tw = reinterpret_cast<const float*>(A.topk_w);
  const int* starts = reinterpret_cast<const int*>(A.starts);
  const bool stable = A.chunk_prefix != 0;
  const uint32_t chunk0 = (t.i0 / kFabChunk) * kFabChunk;
  if (stable) {
    const int n = static_cast<int>(t.i0 + t.i1 - chunk0) * K;
    for (int p = tid; p < n; p += kExecThreads) s_ids[p] = ids[static_cast<size_t>(chunk0) * K + p];
    exec_sync();
  }
  for (uint32_t r = t.i0 + warp; r < t.i0 + t.i1; r += kExecThreads / 32) {
    int pos = 0;
    if (lane < K) {
      const int e = ids[static_cast<size_t>(r) * K + lane];
      if (stable) {
        const int me = static_cast<int>(r - chunk0) * K + lane;
        int rank = 0;
        for (int q = 0; q < me; ++q) rank += s_ids[q] == e;
        pos = starts[e] + reinterpret_cast<const int*>(A.chunk_prefix)[static_cast<size_t>(r / kFabChunk) * E + e] + rank;
      } else {
        pos = starts[e] + atomicAdd(reinterpret_cast<int*>(A.fill) + e, 1);
      }
      reinterpret_cast<int*>(A.pair_token)[pos] = r;
      reinterpret_cast<float*>(A.pair_weight)[pos] = tw[static_cast<size_t>(r) * K + lane];
      if (A.pair_pos) reinterpret_cast<int*>(A.pair_pos)[static_cast<size_t>(r) * K + lane] = pos;
    }
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(A.src) + static_cast<size_t>(r) * H);
    for (int c = lane; c < n16; c += 32) {
      const uint4 v = src[c];
      for (int k = 0; k < K; ++k) {
        const int pk = __shfl_sync(0xffffffffu, pos, k);
        reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(A.dst) + static_cast<size_t>(pk) * H)[c] = v;
      }
    }
  }
}

// Combine tile (kind 47; not in the reference, which adds with fp32 atomics in the
// w2 epilogue and finishes in AddNorm): x[t] = bf16(x2[t] + sum_k w[t][k] * y[pos(t,k)])
// with the sum in pick order (plus, when `shared` is set, the fp32 row shared[t] of a shared
// expert: the GLM-style layer, tests/test_fabric_model_glm.py:57-67), then optionally
// out = rmsnorm(x) * w.
__device__ void tile_combine(const TileDesc& t, int tid) {
  CombineArgs A;   // a copy in registers: the block lives in global memory
  load_block(A, t.a[0]);
  const int warp = tid >> 5, lane = tid & 31;
  const int K = static_cast<int>(A.K), H = static_cast<int>(A.H), n16 = H / 8;
  const float* y = reinterpret_cast<const float*>(A.y);
  const float* shared = reinterpret_cast<const float*>(A.shared);
  // Without a following norm nothing ties a row to one warp: the four warps then share every
  // row, each taking a quarter of its 8-element column groups (the sums per element are the same).
  const bool split = A.w == 0;
  const int c_begin = split ? warp * 32 + lane : lane, c_step = split ? kExecThreads : 32;
  for (uint32_t r = t.i0 + (split ? 0 : warp); r < t.i0 + t.i1; r += split ? 1 : kExecThreads / 32) {
    int pos = 0;
    float w = 0.f;
    if (lane < K) {
      pos = reinterpret_cast<const int*>(A.pair_pos)[static_cast<size_t>(r) * K + lane];
      w = reinterpret_cast<const float*>(A.topk_w)[static_cast<size_t>(r) * K + lane];
    }
    const uint4* x2 = A.x2 ? reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(A.x2) + static_cast<size_t>(r) * H) : nullptr;
    uint4* xo = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(A.x) + static_cast<size_t>(r) * H);
    float ss = 0.f;
    for (int c = c_begin; c < n16; c += c_step) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int k = 0; k < K; ++k) {
        const int pk = __shfl_sync(0xffffffffu, pos, k);
        const float wk = __shfl_sync(0xffffffffu, w, k);
        const float4* yr = reinterpret_cast<const float4*>(y + static_cast<size_t>(pk) * H) + 2 * c;
        const float4 a = __ldcs(yr), b = __ldcs(yr + 1);
        const float yv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = __fmaf_rn(wk, yv[j], acc[j]);
      }
      if (shared) {   // a shared expert's fp32 output row, added after the routed experts
        const float4* sr = reinterpret_cast<const float4*>(shared + static_cast<size_t>(r) * H) + 2 * c;
        const float4 a = __ldcs(sr), b = __ldcs(sr + 1);
        const float sv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], sv[j]);
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
        ss = __fmaf_rn(f[j], f[j], ss);
      }
      xo[c] = pack8(f);
    }
    if (A.w)
      norm_store_row(xo, ss, reinterpret_cast<const __nv_bfloat16*>(A.w),
                     reinterpret_cast<__nv_bfloat16*>(A.out) + static_cast<size_t>(r) * H, nullptr, H, A.eps);
  }
}

// Expand tile (kind 39, csrc/fabric/tiles/aux.cuh:453-616, ExpandArgs), one per lane
// and MoE layer: per-expert counts -> exclusive prefix sums, then for every routed
// expert the GEMM tiles of its w13 and w2 stages, written into the program's dynamic
// region, with the stage records (first, count, link flag); unrouted experts are
// flagged kStageSkip and taken off the join stage's dependency count.  Differences
// from the reference: counts may come from the router tiles' chunk counts (then the
// per-chunk prefixes are produced too, for the stable pack); form 0 maps to 256-row
// blocks (one pass over the weights) instead of K-split tiles with a reduce stage, and,
// when the program has fetch stages (`staging` set), a host-resident expert with more than
// min_rows rows takes the staged form: fetch tiles copy its weights once into the HBM staging
// stack and its GEMM tiles read that copy, so the expert crosses the link once whatever its
// row count (what the reference's weight-stationary K-split form is for), without partial sums;
// an overflow of the dynamic region raises an error bit instead of trapping; red_stage0 =
// 0xffffffff says the program has no reduce stages (w2[e] follows w13[e] directly).
__device__ void tile_expand(const TileDesc& t, const ProgramDesc* P, DeviceState& S, int tid) {
  int* const s_cnt = s_exec_scratch;                              // [kMaxExperts]
  int* const s_start = s_cnt + kMaxExperts + 1;                   // [kMaxExperts + 1]
  int* const s_n = s_start + kMaxExperts + 1;                     // [kMaxExperts]
  int* const s_off = s_n + kMaxExperts + 1;                       // [kMaxExperts + 1]
  int& s_form = s_exec_scratch[4 * (kMaxExperts + 1)];
  int& s_active = s_exec_scratch[4 * (kMaxExperts + 1) + 1];
  int& s_skipped = s_exec_scratch[4 * (kMaxExperts + 1) + 2];
  int& s_overflow = s_exec_scratch[4 * (kMaxExperts + 1) + 3];
  int* const s_info = s_exec_scratch + 4 * (kMaxExperts + 1) + 16;   // [kMaxExperts]: slot << 12 | region << 4 | height class
  // [28] u64: GemmArgs and activation maps per height class (w13, w2), weight maps per region (w13, w2)
  unsigned long long* const s_tab = reinterpret_cast<unsigned long long*>(s_exec_scratch + 5 * (kMaxExperts + 1) + 16 + 1);
  ExpandArgs A;   // a copy in registers: the block lives in global memory
  load_block(A, t.a[0]);
  const int E = static_cast<int>(A.E);
  if (E < 1 || E > kMaxExperts) return;
  StagingArgs G{};
  if (A.staging) load_block(G, A.staging);
  const bool can_stage = A.staging != 0 && G.chunk_bytes >= 16 && (G.chunk_bytes & 15) == 0;
  // fetch tiles of a staged expert: its w13 block, then its w2 block, in chunks
  const int nf13 = can_stage ? static_cast<int>((G.w13_bytes + G.chunk_bytes - 1) / G.chunk_bytes) : 0;
  const int nf2 = can_stage ? static_cast<int>((G.w2_bytes + G.chunk_bytes - 1) / G.chunk_bytes) : 0;
  // the program's arrays, read once: the descriptor itself lives in global memory
  TileDesc* const p_tiles = P->tiles;
  StageStatic* const p_stages = P->stages;
  StageRuntime* const p_runtime = P->runtime;
  // diagnostics: with no reduce stages, red_args may name 8 u64 words for phase time stamps
  unsigned long long* stamps = (A.red_stage0 == 0xffffffffu && tid == 0) ? reinterpret_cast<unsigned long long*>(A.red_args) : nullptr;
  int n_stamp = 0;
  auto stamp = [&]() {
    if (stamps && n_stamp < 8) stamps[n_stamp++] = globaltimer_ns();
  };
  stamp();
  int* counts = reinterpret_cast<int*>(A.counts);
  int* starts = reinterpret_cast<int*>(A.starts);
  for (int e = tid; e < E; e += kExecThreads) {
    int cnt = 0;
    if (A.chunk_counts) {
      // exclusive prefix over the chunks into chunk_prefix (the same buffer when none is given);
      // the counts are cleared for the next iteration's router tiles
      int* cc = reinterpret_cast<int*>(A.chunk_counts);
      int* cp = A.chunk_prefix ? reinterpret_cast<int*>(A.chunk_prefix) : cc;
      for (uint32_t c0 = 0; c0 < A.chunks; c0 += 16) {
        int v[16];
        const uint32_t n = min(16u, A.chunks - c0);
#pragma unroll
        for (uint32_t i = 0; i < 16; ++i) v[i] = i < n ? cc[static_cast<size_t>(c0 + i) * E + e] : 0;
#pragma unroll
        for (uint32_t i = 0; i < 16; ++i) {
          if (i < n) {
            if (cp != cc) cc[static_cast<size_t>(c0 + i) * E + e] = 0;
            cp[static_cast<size_t>(c0 + i) * E + e] = cnt;
            cnt += v[i];
          }
        }
      }
    } else {
      cnt = counts[e];
    }
    s_cnt[e] = cnt;
  }
  if (tid == 0) {
    s_skipped = 0;
    s_overflow = 0;
    unsigned long long ep = ld_acq(&S.published);
    uint32_t f;
    for (;;) {
      f = ld_volatile(&S.snap[ep & 1].form[A.lane & 3]);
      const unsigned long long e2 = ld_acq(&S.published);
      if (e2 == ep) break;
      ep = e2;
    }
    s_form = (f == 0 || f == 16 || f == 32 || f == 64 || f == 128) ? static_cast<int>(f) : 64;
  }
  exec_sync();
  stamp();
  auto scan = [&](const int* v, int* out) {   // exclusive prefix sums by thread 0 (E <= 256)
    if (tid == 0) {
      int run = 0, act = 0;
      for (int e = 0; e < E; ++e) {
        out[e] = run;
        run += v[e];
        act += v[e] != 0;
      }
      out[E] = run;
      s_active = act;
    }
  };
  scan(s_cnt, s_start);
  exec_sync();
  stamp();
  const int active = s_active;
  for (int e = tid; e <= E; e += kExecThreads) starts[e] = s_start[e];
  const int* table = reinterpret_cast<const int*>(A.table);
  const int f13 = static_cast<int>(A.I) / 64, f2 = static_cast<int>(A.H) / 128;
  auto block_rows = [&](int M, bool link) {
    if (link) return s_form ? s_form : 256;
    return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
  };
  for (int e = tid; e < E; e += kExecThreads) {
    const int M = s_cnt[e];
    // One 8-byte read, once per layer: a host thread may move the expert between regions with a
    // single aligned 8-byte write while the kernel runs (staging by the copy engine).
    const unsigned long long entry = ld_volatile(reinterpret_cast<const unsigned long long*>(table) + e);
    const int region = static_cast<int>(entry & 0xffffffffu), slot = static_cast<int>(entry >> 32);
    const bool link = region == static_cast<int>(A.host_region);
    const bool staged = link && can_stage && s_form == 0 && M > static_cast<int>(G.min_rows);
    const int bm = block_rows(M, link);
    int cls = 0;
    while ((16 << cls) < bm) ++cls;   // 16, 32, 64, 128, 256 -> 0..4
    s_n[e] = M > 0 ? ((M + bm - 1) / bm) * (f13 + f2) + (staged ? nf13 + nf2 : 0) : 0;
    // a staged expert's GEMM tiles read region 3 (the lane's staging stack), slot = expert id
    s_info[e] = staged ? (e << 12) | (1 << 11) | (3 << 4) | cls : (slot << 12) | ((region & 0x7f) << 4) | cls;
  }
  if (tid < 5) {
    s_tab[tid] = reinterpret_cast<const unsigned long long*>(A.w13_args)[tid];
    s_tab[5 + tid] = reinterpret_cast<const unsigned long long*>(A.w2_args)[tid];
    s_tab[10 + tid] = reinterpret_cast<const unsigned long long*>(A.xp_maps)[tid];
    s_tab[15 + tid] = reinterpret_cast<const unsigned long long*>(A.h_maps)[tid];
  } else if (tid >= 32 && tid < 36) {   // weight maps of regions 0..3 (host, hot tier, two staging buffers)
    s_tab[20 + tid - 32] = reinterpret_cast<const unsigned long long*>(A.w13_maps)[tid - 32];
    s_tab[24 + tid - 32] = reinterpret_cast<const unsigned long long*>(A.w2_maps)[tid - 32];
  }
  exec_sync();
  stamp();
  scan(s_n, s_off);
  // close the expert stages' previous activation before their tiles and counts change
  const bool has_red = A.red_stage0 != 0xffffffffu;   // the reduce stages of the reference's chain are optional here
  for (int e = tid; e < E; e += kExecThreads) {
    atomicExch(&p_runtime[A.w13_stage0 + e].tag_next, 0ull);
    if (A.staging) atomicExch(&p_runtime[A.fetch_stage0 + e].tag_next, 0ull);
    if (has_red) atomicExch(&p_runtime[A.red_stage0 + e].tag_next, 0ull);
    atomicExch(&p_runtime[A.w2_stage0 + e].tag_next, 0ull);
  }
  __threadfence();
  exec_sync();
  stamp();
  if (s_off[E] > static_cast<int>(A.dyn_cap)) {
    if (tid == 0) raise_error(S, kFabErrDynOverflow);
    s_overflow = 1;   // every thread writes the same value
  }
  exec_sync();
  stamp();
  const unsigned long long* w13_maps = reinterpret_cast<const unsigned long long*>(A.w13_maps);
  const unsigned long long* w2_maps = reinterpret_cast<const unsigned long long*>(A.w2_maps);
  // The tiles of one expert are contiguous (blocks x (f13 + f2) descriptors of 64 bytes); a warp takes
  // one expert after the other.
  {
    const int warp = tid >> 5, lane = tid & 31;
    for (int e = warp; e < E; e += kExecThreads / 32) {
      const int M = s_overflow ? 0 : s_cnt[e];
      if (M == 0) continue;
      const int info = s_info[e];
      const int slot = info >> 12, region = (info >> 4) & 0x7f, cls = info & 0xf;
      const int nf = ((info >> 11) & 1) ? nf13 + nf2 : 0;
      const int bm = 16 << cls;
      const int blocks = (M + bm - 1) / bm;
      const int n13 = blocks * f13, total = nf + blocks * (f13 + f2);
      // One lane builds one whole 64-byte descriptor and stores it as four 16-byte pieces back to back.
      TileDesc* const out = p_tiles + A.dyn_first + s_off[e];
      const unsigned long long scale13 = A.w13_scale ? A.w13_scale + static_cast<unsigned long long>(e) * 2 * A.I * 4 : 0ull;
      const unsigned long long scale2 = A.w2_scale ? A.w2_scale + static_cast<unsigned long long>(e) * A.H * 4 : 0ull;
      const unsigned long long wmap13 = region < 4 ? s_tab[20 + region] : w13_maps[region];
      const unsigned long long wmap2 = region < 4 ? s_tab[24 + region] : w2_maps[region];
      const int row0 = s_start[e];
      for (int ti = lane; ti < total; ti += 32) {
        uint4 v0 = make_uint4(0u, 0u, 0u, 0u), v1 = v0, v2 = v0, v3 = v0;
        if (ti < nf) {   // a fetch tile: chunk ti of the expert's w13 block, then of its w2 block
          const bool f13b = ti < nf13;
          const unsigned long long bytes = f13b ? G.w13_bytes : G.w2_bytes;
          const unsigned long long at = static_cast<unsigned long long>(f13b ? ti : ti - nf13) * G.chunk_bytes;
          const unsigned long long off = static_cast<unsigned long long>(e) * bytes + at;
          const unsigned long long a0 = (f13b ? G.w13_src : G.w2_src) + off, a1 = (f13b ? G.w13_dst : G.w2_dst) + off;
          v0.x = kTileFetch;
          v0.z = static_cast<uint32_t>(min(static_cast<unsigned long long>(G.chunk_bytes), bytes - at));   // i0 bytes
          v1.z = static_cast<uint32_t>(a0);
          v1.w = static_cast<uint32_t>(a0 >> 32);
          v2.x = static_cast<uint32_t>(a1);
          v2.y = static_cast<uint32_t>(a1 >> 32);
        } else {
          const int g = ti - nf;
          const bool is13 = g < n13;
          const int local = is13 ? g : g - n13, per = is13 ? f13 : f2;
          const int blk = local / per, f = local - blk * per;
          const unsigned long long a0 = s_tab[(is13 ? 0 : 5) + cls], a1 = is13 ? wmap13 : wmap2;
          const unsigned long long a2 = s_tab[(is13 ? 10 : 15) + cls], a4 = is13 ? scale13 : scale2;
          v0.x = kTileGemm;                                          // kind | lane | flags; stage (unused)
          v0.z = static_cast<uint32_t>(is13 ? f * 64 : f * 128);     // i0 first weight row
          v0.w = static_cast<uint32_t>(row0 + blk * bm);             // i1 first activation row
          v1.x = static_cast<uint32_t>(min(bm, M - blk * bm));       // i2 rows
          v1.y = static_cast<uint32_t>(slot);                        // i3 weight slot
          v1.z = static_cast<uint32_t>(a0);                          // a[0] GemmArgs
          v1.w = static_cast<uint32_t>(a0 >> 32);
          v2 = make_uint4(static_cast<uint32_t>(a1), static_cast<uint32_t>(a1 >> 32),   // a[1] weight map
                          static_cast<uint32_t>(a2), static_cast<uint32_t>(a2 >> 32));  // a[2] activation map
          v3.z = static_cast<uint32_t>(a4);                          // a[3] K range (all); a[4] fp32 scale per weight row
          v3.w = static_cast<uint32_t>(a4 >> 32);
        }
        uint4* dst = reinterpret_cast<uint4*>(out + ti);
        dst[0] = v0;
        dst[1] = v1;
        dst[2] = v2;
        dst[3] = v3;
      }
    }
  }
  for (int e = tid; e < E; e += kExecThreads) {
    const int M = s_overflow ? 0 : s_cnt[e];
    const bool link = ((s_info[e] >> 4) & 0x7f) == static_cast<int>(A.host_region);   // the entry as read above
    const uint32_t base = A.dyn_first + s_off[e];
    StageStatic& s13 = p_stages[A.w13_stage0 + e];
    StageStatic& s2 = p_stages[A.w2_stage0 + e];
    const int bm = 16 << (s_info[e] & 0xf);   // the height chosen above
    const int blocks = M > 0 ? (M + bm - 1) / bm : 0;
    const int n13 = blocks * f13, n2 = blocks * f2;
    const bool staged = M > 0 && ((s_info[e] >> 11) & 1);
    const int nf = staged ? nf13 + nf2 : 0;
    const uint32_t gemm_flags = link ? kStageLink : 0u;   // staged (region 3): only the fetch tiles use the link
    const bool skip = M == 0 && active > 0;   // an unrouted expert: its chain is passed over
    if (A.staging) {
      StageStatic& sf = p_stages[A.fetch_stage0 + e];
      sf.first = base;
      sf.count = nf;
      sf.flags = skip ? kStageSkip : kStageLink;
    }
    s13.first = base + nf;
    s13.count = n13;
    s13.flags = gemm_flags;
    if (skip) {
      s13.flags = kStageSkip;
      atomicAdd(&s_skipped, 1);
    }
    if (has_red) {
      StageStatic& sr = p_stages[A.red_stage0 + e];
      sr.first = base + nf + n13;
      sr.count = 0;
      sr.flags = 0u;
    }
    s2.first = base + nf + n13;
    s2.count = n2;
    s2.flags = gemm_flags;
    if (A.hist && M > 0) atomicAdd(reinterpret_cast<int*>(A.hist) + e, M);
    counts[e] = 0;
    if (A.fill) reinterpret_cast<int*>(A.fill)[e] = 0;
  }
  __threadfence();
  exec_sync();
  stamp();
  const unsigned int skipped = static_cast<unsigned int>(s_skipped);   // the scratch is reused below
  exec_sync();
  if (A.permute_args) {
    // a small batch: the permute of every row, chunk by chunk, with the prefixes written above
    for (uint32_t r0 = 0; r0 < A.permute_rows; r0 += kFabChunk) {
      TileDesc pm = t;
      pm.a[0] = A.permute_args;
      pm.i0 = r0;
      pm.i1 = min(static_cast<uint32_t>(kFabChunk), A.permute_rows - r0);
      tile_permute(pm, tid);
      exec_sync();
    }
    __threadfence();
  }
  if (tid == 0 && skipped > 0) atomicSub(&p_runtime[A.join_stage].deps, skipped);
}

// Fused tile (kind 50): the norm of rows [i0, i0 + i1), then the router projection of those rows against the
// tile's expert range.  For a small batch this folds the norm stage into the projection's tiles: the tiles of a
// row group (one per expert range) all compute the same norm and write the same bytes, which costs a few
// microseconds each and saves a stage.  The norm must be one that can be repeated: plain (36), or add-norm (41)
// over slabs, which it only reads.
__device__ void tile_norm_logits(const TileDesc& t, int tid) {
  TileDesc part = t;
  const bool add = t.a[3] == kTileAddNorm;
  if (add) {   // an accumulator that is zeroed once read cannot be read by several tiles
    NormArgs A;
    load_block(A, t.a[0]);
    if (A.acc_parts <= 1) return;
  }
  tile_norm(part, tid, add);
  __threadfence_block();
  exec_sync();
  part.a[0] = t.a[1];
  tile_router_logits(part, tid);
}

// RMSNorm tile (kind 36) and AddNorm tile (kind 41), NormArgs
// (csrc/fabric/tiles/aux.cuh:124-188): AddNorm first forms x = bf16(x2 + acc), stores
// it, zeroes the fp32 accumulator rows, then normalises; gather >= 0 copies the
// normalised row to out2[gather].
__device__ void tile_norm(const TileDesc& t, int tid, bool add) {
  NormArgs A;   // a copy in registers: the block lives in global memory
  load_block(A, t.a[0]);
  const int warp = tid >> 5, lane = tid & 31;
  const int H = static_cast<int>(A.H), n16 = H / 8;
  for (uint32_t r = t.i0 + warp; r < t.i0 + t.i1; r += kExecThreads / 32) {
    const size_t o = static_cast<size_t>(r) * A.ld;
    uint4* x = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(A.x) + o);
    float ss = 0.f;
    if (add) {
      const uint4* x2 = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(A.x2) + o);
      float4* acc = reinterpret_cast<float4*>(reinterpret_cast<float*>(A.acc) + static_cast<size_t>(r) * H);
      const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
      const int parts = static_cast<int>(A.acc_parts);
      const size_t slab = static_cast<size_t>(A.acc_rows) * H / 4;   // float4 per slab
      for (int c = lane; c < n16; c += 32) {
        float f[8];
        unpack8(x2[c], f);
        float4 a0 = acc[2 * c], a1 = acc[2 * c + 1];
        if (parts > 1) {
          // the partial sums of a K-split GEMM, one slab per K range, added in slab order; four slabs' loads
          // are issued before the first of them is used
          for (int q0 = 1; q0 < parts; q0 += 4) {
            float4 b0[4], b1[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int q = min(q0 + i, parts - 1);
              b0[i] = acc[q * slab + 2 * c];
              b1[i] = acc[q * slab + 2 * c + 1];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              if (q0 + i < parts) {
                a0 = make_float4(__fadd_rn(a0.x, b0[i].x), __fadd_rn(a0.y, b0[i].y), __fadd_rn(a0.z, b0[i].z),
                                 __fadd_rn(a0.w, b0[i].w));
                a1 = make_float4(__fadd_rn(a1.x, b1[i].x), __fadd_rn(a1.y, b1[i].y), __fadd_rn(a1.z, b1[i].z),
                                 __fadd_rn(a1.w, b1[i].w));
              }
            }
          }
        } else {
          acc[2 * c] = zero;
          acc[2 * c + 1] = zero;
        }
        const float sv[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          f[j] = round_bf16(__fadd_rn(f[j], sv[j]));
          ss = __fmaf_rn(f[j], f[j], ss);
        }
        x[c] = pack8(f);
      }
    } else {
      for (int c = lane; c < n16; c += 32) {
        float f[8];
        unpack8(x[c], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = __fmaf_rn(f[j], f[j], ss);
      }
    }
    __nv_bfloat16* out2 = nullptr;
    if (A.gather) {
      const int gi = reinterpret_cast<const int*>(A.gather)[r];
      if (gi >= 0) out2 = reinterpret_cast<__nv_bfloat16*>(A.out2) + static_cast<size_t>(gi) * H;
    }
    norm_store_row(x, ss, reinterpret_cast<const __nv_bfloat16*>(A.w), reinterpret_cast<__nv_bfloat16*>(A.out) + o,
                   out2, H, A.eps);
  }
}

// Worker state word for hang diagnosis: running(63) | completing(62) | lane(56..61)
// | kind(44..55) | stage(24..43) | tile index(0..23).
__device__ void note_tile(DeviceState& S, uint32_t worker, const WorkSlot& w, unsigned long long state) {
  S.worker_tile[worker] = state | (static_cast<unsigned long long>(w.tile_lane & 0x3f) << 56) |
                          (static_cast<unsigned long long>(w.tile.kind & 0xfff) << 44) |
                          (static_cast<unsigned long long>(w.stage & kStageMask) << 24) | (w.index & 0xffffffull);
  if (state) S.worker_tile_ns[worker] = globaltimer_ns();
}

// Wait (whole warp or a single thread) until a counter in shared memory that another
// role of this worker advances has reached `target`; bounded like every other wait.
__device__ __forceinline__ bool wait_counter(const unsigned int* counter, unsigned int target, volatile int* abort_flag) {
  const volatile unsigned int* c = counter;
  if (static_cast<int>(*c - target) >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (uint32_t spins = 0;; ++spins) {
    if (static_cast<int>(*c - target) >= 0) return true;
    __nanosleep(32);
    if ((spins & 63u) == 63u) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > kAttnWaitNs) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

__device__ __forceinline__ unsigned long long role_ctx(uint32_t rec, uint32_t q_phase, const uint32_t (&base)[2]) {
  return (static_cast<unsigned long long>(rec & 0xffffu) << 48) | (static_cast<unsigned long long>(q_phase & 0xffu) << 40) |
         (static_cast<unsigned long long>(base[0] & 0xffu) << 32) | (static_cast<unsigned long long>(base[1] & 0xffu) << 24);
}

__device__ __forceinline__ AttnCtx attn_ctx(const AttnWork& w, AttnShared& sh, volatile int* abort_flag, uint8_t* ring,
                                            uint32_t tmem_base, uint32_t q_phase, const uint32_t (&base)[2],
                                            volatile unsigned int* note) {
  AttnCtx c;
  c.note = note;
  c.xbuf = nullptr;
  c.q_empty = nullptr;
  c.s_free = nullptr;
  c.q_phase = q_phase;
  c.base[0] = base[0];
  c.base[1] = base[1];
  c.sh = &sh;
  c.abort_flag = abort_flag;
  c.smem = ring;
  c.tmem_base = tmem_base;
  attn_derive(w, c);
  return c;
}

struct WorkerShared {
  uint64_t slot_full[kSlots], slot_empty[kSlots];
  GemmBarriers bar;
  Worklist wl;                  // completed stages the first exec warp still has to release
  SmallWorklist sched_wl;       // the same for the scheduler warp, when it starts a lane whose first stage is empty
  AttnShared attn;              // barriers of attention items, armed once; every role counts their phases
  unsigned int wait_note[3];    // producer, MMA, first exec warp: tile << 8 | site of the current wait
  unsigned long long wait_ctx[3];   // and the record / phase counts the role had then
  unsigned int tiles_done;      // work records the exec warps have finished
  unsigned int mma_done;        // work records the MMA warp has finished
  WorkSlot slot[kSlots];
  WorkerState ws;
  unsigned long long t0;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(kWorkerThreads, 1) fabric_kernel(DeviceState* Sp, uint32_t first_worker) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ WorkerShared sh;
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  DeviceState& S = *Sp;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t worker = first_worker + blockIdx.x;
  volatile int* abort_flag = &sh.abort_flag;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(&sh.slot_full[i], 1);
      mbar_init(&sh.slot_empty[i], 3);   // exec thread 0, producer, MMA
    }
    gemm_barriers_init(sh.bar);
    sh.abort_flag = 0;
    sh.attn.fail_site = 0;
    sh.wait_note[0] = sh.wait_note[1] = sh.wait_note[2] = 0;
    sh.wait_ctx[0] = sh.wait_ctx[1] = sh.wait_ctx[2] = 0;
    attn_barriers_init(sh.attn);
    sh.tiles_done = 0;
    sh.mma_done = 0;
    sh.ws.epoch = ~0ull;
    sh.ws.worker = worker;
    sh.ws.slot_lane = kNoLane;
    sh.ws.link_last = 0;
    sh.ws.done = &sh.tiles_done;
    sh.ws.idle_ns = 64;
    sh.ws.lane = kNoLane;
    sh.ws.n_lanes = 0;
    sh.ws.left = 0;
    sh.ws.row_block = 0;
    fence_barrier_init();
  }
  if (warp == 6) {
    tmem_alloc(&sh.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sh.tmem_base;
  constexpr unsigned long long kForever = ~0ull >> 1;   // the scheduler's exit record ends these waits

  if (warp == 0) {
    // ------------------------------------------------------------ scheduler
    // The whole warp schedules (fabric_sched.cuh); lane 0 owns the worker state and the work records.
    WorkerState& ws = sh.ws;
    unsigned long long t_start = 0;
    if (lane == 0) t_start = globaltimer_ns();
    // Lane 0: has the host asked the fabric to stop, or has the run-time limit passed?
    auto must_leave = [&](bool check_shutdown) {
      const unsigned long long limit = ld_volatile(&S.max_run_ns);
      const bool late = limit && globaltimer_ns() - t_start > limit;
      if (late && !check_shutdown) raise_error(S, kFabErrDeadline);
      return late || (check_shutdown && ld_acq(&S.shutdown) != 0);
    };
    for (uint32_t n = 0;; ++n) {
      const int s = n % kSlots;
      int go = 1;
      if (lane == 0) go = mbar_wait_bounded(&sh.slot_empty[s], ((n / kSlots) & 1) ^ 1, abort_flag, kForever);
      if (!__shfl_sync(kWarp, go, 0)) break;
      uint32_t cmd = kCmdRun;
      if (ws.left == 0) {
        for (;;) {
          cmd = schedule(S, ws, sh.sched_wl);
          if (cmd != kCmdIdle) break;
          int leave = 0;
          if (lane == 0 && must_leave(false)) {
            give_slot_back(S, ws);
            leave = 1;
          }
          if (__shfl_sync(kWarp, leave, 0)) {
            cmd = kCmdExit;
            break;
          }
        }
      } else {
        // mid-claim: on a stop the remaining tiles of the claim stay unexecuted (the fabric is stopping)
        int leave = 0;
        if (lane == 0 && must_leave(true)) {
          give_slot_back(S, ws);
          leave = 1;
        }
        if (__shfl_sync(kWarp, leave, 0)) cmd = kCmdExit;
      }
      WorkSlot& w = sh.slot[s];
      if (cmd == kCmdRun && lane < 4)   // the 64-byte descriptor, one 16-byte piece per lane
        reinterpret_cast<uint4*>(&w.tile)[lane] = __ldcg(reinterpret_cast<const uint4*>(&ws.prog->tiles[ws.next_index]) + lane);
      __syncwarp();
      if (lane == 0) {
        w.cmd = cmd;
        w.counts = 1;
        if (cmd == kCmdRun) {
          w.prog = ws.prog;
          w.stage = ws.stage;
          w.tile_lane = ws.tile_lane;
          w.link = ws.link;
          if (ws.link) ws.link_last = n + 1;
          w.index = ws.next_index;
          w.worker_lane = ws.lane;
          w.is_gemm = 0;
          w.is_attn = 0;
          if (w.tile.kind == kTileAttnPrefill || w.tile.kind == kTileAttnDecode) {
            if (make_attn_work(w.tile, w.attn)) {
              w.is_attn = 1;
            } else {
              raise_error(S, kFabErrBadTile);
              w.tile.kind = kTileNop;
            }
          } else if (w.tile.kind == kTileGemm || w.tile.kind == kTileFetch) {
            if (w.tile.kind == kTileGemm ? make_gemm_work(w.tile, w.gemm) : make_fetch_work(w.tile, w.gemm)) {
              w.is_gemm = 1;
            } else {
              raise_error(S, kFabErrBadTile);
              w.tile.kind = kTileNop;   // completes without running, so the program still ends
            }
          } else if (w.tile.kind == kTileGemmAsym) {
            // one record per row block; the tile is done with its last block's record
            if (make_gemm_work(w.tile, w.gemm, ws.row_block)) {
              w.is_gemm = 1;
              const uint32_t blocks = (w.tile.i2 + w.gemm.n - 1) / static_cast<uint32_t>(w.gemm.n);
              if (ws.row_block + 1 < blocks) {
                ++ws.row_block;
                w.counts = 0;
              }
            } else {
              raise_error(S, kFabErrBadTile);
              w.tile.kind = kTileNop;
            }
          }
          if (w.counts) {
            ws.row_block = 0;
            ++ws.next_index;
            --ws.left;
          }
        }
        mbar_arrive(&sh.slot_full[s]);
      }
      __syncwarp();
      if (cmd == kCmdExit) break;
    }
  } else if (warp == 5) {
    // --------------------------------------------------------- TMA producer
    const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
    GemmPipe pipe;
    GemmInflight inflight;
    bool prev_attn = false;
    uint32_t aq = 0, ab[2] = {0, 0};   // phases the attention barriers have completed
    for (uint32_t n = 0;; ++n) {
      const int s = n % kSlots;
      if (!mbar_wait_bounded(&sh.slot_full[s], (n / kSlots) & 1, abort_flag, kForever)) break;
      const WorkSlot& w = sh.slot[s];
      if (w.cmd == kCmdExit) break;
      bool ok = true;
      // An attention item uses the whole operand ring and TMEM outside the GEMM pipe's
      // bookkeeping: it starts once every earlier record of this worker is finished, and
      // the record after it waits for it in the same way.
      if ((w.is_attn || prev_attn) && lane == 0) {
        sh.wait_note[0] = 13;
        sh.wait_ctx[0] = role_ctx(n, aq, ab);
      }
      if (w.is_attn || prev_attn)
        ok = __all_sync(0xffffffffu, (wait_counter(&sh.tiles_done, n, abort_flag) || attn_gave_up(sh.attn, 13)) &&
                                         (wait_counter(&sh.mma_done, n, abort_flag) || attn_gave_up(sh.attn, 14)));
      prev_attn = w.is_attn != 0;
      if (ok && w.is_attn) {
        AttnCtx c = attn_ctx(w.attn, sh.attn, abort_flag, ring, tmem_base, aq, ab, &sh.wait_note[0]);
        attn_produce(w.attn, c);
        attn_advance(c.n_tiles, aq, ab);
      } else if (ok && w.is_gemm) {
        ok = gemm_produce(w.gemm, ring, sh.bar, pipe, inflight, abort_flag, pol_w, pol_x);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.slot_empty[s]);
      if (!ok) break;
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------ MMA issue
    GemmPipe pipe;
    uint32_t g = 0;   // GEMM tiles seen: accumulator buffer and parity
    uint32_t aq = 0, ab[2] = {0, 0};
    for (uint32_t n = 0;; ++n) {
      const int s = n % kSlots;
      if (!mbar_wait_bounded(&sh.slot_full[s], (n / kSlots) & 1, abort_flag, kForever)) break;
      const WorkSlot& w = sh.slot[s];
      if (w.cmd == kCmdExit) break;
      bool ok = true;
      if (w.is_attn) {
        // the item's loads are issued only after the worker's earlier records have drained,
        // so waiting for them is all the ordering this role needs
        AttnCtx c = attn_ctx(w.attn, sh.attn, abort_flag, ring, tmem_base, aq, ab, &sh.wait_note[1]);
        if (lane == 0) sh.wait_ctx[1] = role_ctx(n, aq, ab);
        attn_mma<1>(w.attn, c);
        attn_advance(c.n_tiles, aq, ab);
      } else if (w.is_gemm) {
        ok = gemm_mma(w.gemm, ring, sh.bar, pipe, tmem_base, g & 1, (g >> 1) & 1, abort_flag);
        ++g;
      }
      if (lane == 0) {
        *reinterpret_cast<volatile unsigned int*>(&sh.mma_done) = n + 1;
        mbar_arrive(&sh.slot_empty[s]);
      }
      if (!ok) break;
    }
  } else {
    // ------------------------------------------------------ exec / epilogue
    const int tid = threadIdx.x - 32;
    uint32_t g = 0;
    uint32_t aq = 0, ab[2] = {0, 0};
    GemmPipe conv_pipe;
    for (uint32_t n = 0;; ++n) {
      const int s = n % kSlots;
      if (!mbar_wait_bounded(&sh.slot_full[s], (n / kSlots) & 1, abort_flag, kForever)) break;
      const WorkSlot& w = sh.slot[s];
      if (w.cmd == kCmdExit) break;
      if (tid == 0) {
        if (w.link) {
          LaneState& L = S.lane[w.tile_lane];
          const unsigned int c = atomicAdd(&L.inflight, 1u) + 1;
          atomicMax(&L.inflight_max, c);
        }
        note_tile(S, worker, w, 1ull << 63);
      }
      if (w.is_attn) {
        AttnCtx c = attn_ctx(w.attn, sh.attn, abort_flag, ring, tmem_base, aq, ab, warp == 1 ? &sh.wait_note[2] : nullptr);
        if (tid == 0) sh.wait_ctx[2] = role_ctx(n, aq, ab);
        if (c.rep) softmax_role<true, 1, 1>(w.attn, c, 0);
        else softmax_role<false, 1, 1>(w.attn, c, 0);
        attn_advance(c.n_tiles, aq, ab);
      } else if (w.is_gemm) {
        // The exec warps follow the operand ring like the producer and the MMA warp do: for e4m3
        // weights they are the converters of every stage (then the tile's epilogue), for bf16
        // weights they only step their cursor over the tile's stages.
        bool ok = true;
        if (w.gemm.w_fp8) {
          ok = gemm_convert(w.gemm, ring, sh.bar, conv_pipe, tid, abort_flag);
        } else {
          const uint32_t size = gemm_stage_bytes(w.gemm);
          const int n_stages = gemm_stage_count(w.gemm);
          for (int kt = 0; kt < n_stages; ++kt) {
            uint32_t vb, ve;
            conv_pipe.alloc(size, vb, ve);
            conv_pipe.advance();
          }
        }
        ok = ok && gemm_epilogue(w.gemm, sh.bar, tmem_base, g & 1, (g >> 1) & 1, abort_flag);
        if (!ok && tid == 0) raise_error(S, kFabErrTileWait);
        ++g;
      } else if (!run_core_tile(S, w, tid, worker, &sh.t0) && tid == 0) {
        raise_error(S, kFabErrBadTile);
      }
      exec_sync();
      if (tid < 32) {   // the first exec warp does the completion bookkeeping
        if (tid == 0) {
          if (w.link) atomicSub(&S.lane[w.tile_lane].inflight, 1u);
          __threadfence();   // this worker's writes are visible device-wide before the tile counts as done
          note_tile(S, worker, w, 1ull << 62);
        }
        __syncwarp();
        if (w.counts) tiles_completed(S, w.tile_lane, w.prog, w.stage, 1, sh.wl);
        if (tid == 0) {
          note_tile(S, worker, w, 0);
          *reinterpret_cast<volatile unsigned int*>(&sh.tiles_done) = n + 1;
          mbar_arrive(&sh.slot_empty[s]);
        }
      }
    }
  }
  // a bounded wait that ran out inside a GEMM role is reported, and every role leaves
  tc_fence_before_sync();
  __syncthreads();
  // the wait that gave up first inside an attention item is reported in bits 32.. of the error word
  if (threadIdx.x == 0 && sh.abort_flag) {
    for (int i = 0; i < 3; ++i) S.worker_wait[worker][i] = sh.wait_ctx[i] | (sh.wait_note[i] & 0xffffffull);
    S.worker_wait[worker][3] = sh.tiles_done | (static_cast<unsigned long long>(sh.mma_done) << 32);
  }
  if (threadIdx.x == 0 && sh.abort_flag)
    raise_error(S, kFabErrTileWait | (static_cast<unsigned long long>(sh.attn.fail_site) << 32) |
                       (static_cast<unsigned long long>(sh.tiles_done & 0xffffu) << 48));
  if (warp == 6) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

cudaError_t launch_fabric(DeviceState* S, int workers, uint32_t first_worker, cudaStream_t stream) {
  static PerDeviceOnce once;
  const cudaError_t err = once.run([] {
    return cudaFuncSetAttribute(fabric_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes);
  });
  if (err != cudaSuccess) return err;
  fabric_kernel<<<workers, kWorkerThreads, kGemmSmemBytes, stream>>>(S, first_worker);
  return cudaGetLastError();
}

}  // namespace fab
}  // namespace mf
