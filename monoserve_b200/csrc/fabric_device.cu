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
//     path through a two-deep ring of work records, so claims, descriptor loads
//     and epoch refreshes overlap the previous tile; warps 1..4 execute tiles and
//     are the epilogue of GEMM tiles; warp 5 issues the TMA copies and warp 6 owns
//     TMEM and issues tcgen05.mma (gemm_core.cuh), with accumulators double-buffered
//     across consecutive GEMM tiles;
//   * no wait is unbounded and nothing traps: a ring publication that waits too
//     long, a full worklist or an unknown tile kind raise an error bit that the
//     host reads from the mirror, and the kernel leaves by itself after
//     max_run_ns, so a fabric that owns every SM can always be stopped.
#include <cuda_runtime.h>

#include "fabric_types.h"
#include "gemm_core.cuh"
#include "operands.h"
#include "ptx.cuh"
#include "rowwise.cuh"

namespace mf {
namespace fab {

constexpr uint32_t kStageBits = 20;
constexpr uint32_t kStageMask = (1u << kStageBits) - 1;
constexpr uint32_t kTagMask = 0xfffu;
constexpr int kScanDepth = 16;
constexpr int kWorklistCap = 512;
constexpr uint32_t kMaxBatch = 8;
constexpr uint32_t kBatchDivisor = 128;
constexpr int kExecThreads = 128;
constexpr int kWorkerThreads = 32 + kExecThreads + 64;   // scheduler, exec/epilogue, TMA producer, MMA
constexpr unsigned long long kRingWaitBudgetNs = 2000000000ull;

enum : uint32_t { kCmdRun = 0, kCmdIdle = 1, kCmdExit = 2 };

template <class T>
__device__ __forceinline__ T ld_volatile(const T* p) { return *reinterpret_cast<const volatile T*>(p); }

__device__ __forceinline__ unsigned int ld_acq(const unsigned int* p) { return ld_acquire_gpu(p); }
__device__ __forceinline__ unsigned long long ld_acq(const unsigned long long* p) { return ld_acquire_gpu64(p); }
__device__ __forceinline__ void st_rel(unsigned int* p, unsigned int v) { st_release_gpu(p, v); }
__device__ __forceinline__ void st_rel(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ unsigned int smid() {
  unsigned int v;
  asm volatile("mov.u32 %0, %smid;" : "=r"(v));
  return v;
}

__device__ void raise_error(DeviceState& S, unsigned long long bit) {
  const unsigned long long now = atomicOr(&S.error, bit) | bit;
  if (S.mirror) st_release_sys64(&S.mirror->error, now);   // pinned host memory
}

struct Worklist {
  uint32_t v[kWorklistCap];
  int n;
  bool overflow;
  __device__ void push(uint32_t s) {
    if (n < kWorklistCap) v[n++] = s; else overflow = true;
  }
  __device__ uint32_t pop() { return v[--n]; }
};

// Scheduling state of one worker (shared memory, touched by the scheduler thread
// and, for the lane statistics, by the completing exec thread).
struct WorkerState {
  unsigned long long epoch;
  uint32_t worker, lane, n_lanes, slot_lane, idle_ns;
  uint32_t cap[kMaxLanes], order[kMaxLanes], prog_gen[kMaxLanes];
  ProgramDesc* prog_snap[kMaxLanes];
  // the current claim
  const ProgramDesc* prog;
  uint32_t stage, tile_lane, link, next_index, left;
};

struct WorkSlot {
  TileDesc tile;
  GemmWork gemm;          // filled by the scheduler for GEMM tiles
  const ProgramDesc* prog;
  uint32_t stage, tile_lane, link, index, cmd, worker_lane, is_gemm, pad;
};

// A GEMM tile (kind 32) in the reference's operand convention
// (csrc/fabric/model_types.h:37-49): a[0] GemmArgs*, a[1] weight map record,
// a[2] activation map record, a[3] K range = first K tile | K tiles << 16 (0 = all),
// a[4] fp32 scale per weight row; i0 first weight row, i1 first activation row,
// i2 valid activation rows, i3 weight z (expert or slot).  A map record is three
// CUtensorMaps (monofab_fabric_tensor_map): [0] the caller's box, [1] box
// (64, 16, 1), [2] box (64, 128, 1).
__device__ bool make_gemm_work(const TileDesc& t, GemmWork& w) {
  GemmArgs A;
  const uint4* src = reinterpret_cast<const uint4*>(t.a[0]);
  uint4* dst = reinterpret_cast<uint4*>(&A);
#pragma unroll
  for (int i = 0; i < 8; ++i) dst[i] = __ldcg(src + i);
  if (A.w_fp8) return false;   // FP8 tiles need the converter warps of the stand-alone kernel
  if (A.bm < 16 || A.bm > kGemmMaxN || (A.bm & (A.bm - 1))) return false;
  const CUtensorMap* wrec = reinterpret_cast<const CUtensorMap*>(t.a[1]);
  const CUtensorMap* xrec = reinterpret_cast<const CUtensorMap*>(t.a[2]);
  const bool silu = A.epi == kEpiSiluMul;
  w.a_map = silu ? wrec + 1 : wrec + 2;
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
  w.b_row0 = t.i1;
  w.rows = t.i2 < A.bm ? t.i2 : A.bm;
  w.n = A.bm;
  const uint32_t k0 = static_cast<uint32_t>(t.a[3] & 0xffff), kn = static_cast<uint32_t>((t.a[3] >> 16) & 0xffff);
  w.k0 = kn ? k0 : 0;
  w.k_tiles = kn ? kn : A.k_tiles;
  w.epi = A.epi;
  w.ld_out = A.ld_out;
  w.ld_res = A.ld_res;
  w.n_limit = A.n_limit;
  w.valid = 1;
  w.a_packed = 0;
  w.block = -1;
  w.w_fp8 = 0;
  return w.k_tiles > 0 && A.epi <= kEpiAtomicF32;
}

__device__ void trace_stage(DeviceState& S, uint32_t lane, uint32_t s, uint32_t event, uint32_t tag) {
  const uint32_t cap = ld_volatile(&S.trace_cap);
  if (cap == 0) return;
  const uint32_t i = atomicAdd(&S.trace_n, 1u);
  if (i >= cap) return;
  unsigned long long* r = reinterpret_cast<unsigned long long*>(ld_volatile(&S.trace_ptr)) + 2ull * i;
  r[0] = static_cast<unsigned long long>(s) | (static_cast<unsigned long long>(lane) << 32) |
         (static_cast<unsigned long long>(event) << 40) | (static_cast<unsigned long long>(tag & kTagMask) << 48);
  r[1] = globaltimer_ns();
}

__device__ void mirror_lane(DeviceState& S, uint32_t lane, int what, unsigned long long v) {
  if (!S.mirror) return;
  LaneMirror& m = S.mirror->lane[lane];
  switch (what) {
    case 0: st_release_sys64(&m.iterations, v); break;
    case 1: st_release_sys64(&m.gen, v); break;
    case 2: st_release_sys64(&m.running, v); break;
    case 3:
      st_release_sys64(&m.mark_ns, globaltimer_ns());
      st_release_sys64(&m.mark, v);
      break;
  }
}

// ------------------------------------------------------------------- rings
// Append m entries with one reservation; publish them once every earlier
// reservation is published.  The wait for earlier producers is bounded.
__device__ void ring_push_n(DeviceState& S, LaneState& L, bool link, const uint32_t* entries, int m) {
  if (m == 0) return;
  Ring& R = L.ring[link ? 1 : 0];
  const unsigned long long pos = atomicAdd(&R.reserve, static_cast<unsigned long long>(m));
  for (int i = 0; i < m; ++i) R.ids[(pos + i) & (kRingCap - 1)] = entries[i];
  unsigned int ns = 32;
  const unsigned long long t0 = globaltimer_ns();
  while (ld_acq(&R.tail) != pos) {
    __nanosleep(ns);
    if (ns < 512) ns <<= 1;
    if (globaltimer_ns() - t0 > kRingWaitBudgetNs) {
      raise_error(S, kFabErrRingWait);
      return;
    }
  }
  st_rel(&R.tail, pos + m);
}

__device__ __forceinline__ uint32_t make_entry(uint32_t stage, uint32_t tag) {
  return ((tag & kTagMask) << kStageBits) | (stage & kStageMask);
}

// Take the next tiles of the stage an entry names: n tiles from `index`.  Valid
// only while the stage's runtime still carries the entry's tag.
__device__ bool claim(const ProgramDesc* P, uint32_t entry, uint32_t& stage, uint32_t& index, uint32_t& n) {
  const uint32_t s = entry & kStageMask, tag = entry >> kStageBits;
  if (s >= P->n_stages) return false;
  uint32_t count = ld_volatile(&P->stages[s].count);
  unsigned long long* tn = &P->runtime[s].tag_next;
  const unsigned long long v = ld_acq(tn);
  const uint32_t next = static_cast<uint32_t>(v);
  if ((static_cast<uint32_t>(v >> 32) & kTagMask) != tag || next >= count) return false;
  const uint32_t left = count - next;
  const uint32_t k = min(left, min(kMaxBatch, max(1u, left / kBatchDivisor)));
  const unsigned long long old = atomicAdd(tn, static_cast<unsigned long long>(k));
  const uint32_t ot = static_cast<uint32_t>(old >> 32) & kTagMask, on = static_cast<uint32_t>(old);
  if (ot == 0) return false;
  if (ot != tag) count = ld_volatile(&P->stages[s].count);
  if (on >= count) return false;
  stage = s;
  index = ld_volatile(&P->stages[s].first) + on;
  n = min(k, count - on);
  return true;
}

__device__ bool take_from(LaneState& L, bool link, const ProgramDesc* P, uint32_t& stage, uint32_t& index,
                          uint32_t& n) {
  Ring& R = L.ring[link ? 1 : 0];
  unsigned long long h = ld_acq(&R.head);
  const unsigned long long t = ld_acq(&R.tail);
  for (unsigned long long p = h; p < t && p < h + kScanDepth; ++p) {
    const uint32_t e = ld_volatile(&R.ids[p & (kRingCap - 1)]);
    if (claim(P, e, stage, index, n)) return true;
    if (p == h) {   // the head entry is stale or exhausted: step past it
      if (atomicCAS(&R.head, h, h + 1) == h) h = h + 1;
    }
  }
  return false;
}

// ---------------------------------------------- activation, completion, iterations
__device__ bool arm(DeviceState& S, uint32_t lane, const ProgramDesc* P, uint32_t s, uint32_t tag, Worklist& wl,
                    uint32_t& entry, bool& link) {
  trace_stage(S, lane, s, 0, tag);
  const uint32_t count = ld_volatile(&P->stages[s].count);
  if (count == 0) {   // nothing to run: completes at once
    wl.push(s);
    return false;
  }
  atomicExch(&P->runtime[s].tag_next, static_cast<unsigned long long>(tag & kTagMask) << 32);
  link = (ld_volatile(&P->stages[s].flags) & kStageLink) != 0;
  entry = make_entry(s, tag);
  return true;
}

__device__ void latest_program(DeviceState& S, uint32_t lane, ProgramDesc*& p, uint32_t& gen) {
  unsigned long long e = ld_acq(&S.published);
  for (;;) {
    const Snapshot& sn = S.snap[e & 1];
    p = ld_volatile(&sn.prog[lane]);
    gen = ld_volatile(&sn.prog_gen[lane]);
    const unsigned long long e2 = ld_acq(&S.published);
    if (e2 == e) return;
    e = e2;
  }
}

__device__ void begin_iteration(DeviceState& S, uint32_t lane, const ProgramDesc* P, uint32_t gen, bool fresh,
                                Worklist& wl) {
  LaneState& L = S.lane[lane];
  if (fresh) {   // every entry of the previous program is exhausted: drop them
    atomicExch(&L.ring[0].head, ld_acq(&L.ring[0].tail));
    atomicExch(&L.ring[1].head, ld_acq(&L.ring[1].tail));
    L.iter_in_prog = 0;
    st_rel(&L.prog, reinterpret_cast<unsigned long long>(P));
    st_rel(&L.gen, gen);
    mirror_lane(S, lane, 1, gen);
  }
  uint32_t t = ld_volatile(&L.tag) + 1;
  if ((t & kTagMask) == 0) ++t;   // tag 0 marks never-activated stages
  st_rel(&L.tag, t);
  uint32_t entry;
  bool link;
  if (arm(S, lane, P, P->first_stage, t & kTagMask, wl, entry, link)) ring_push_n(S, L, link, &entry, 1);
}

__device__ const ProgramDesc* end_iteration(DeviceState& S, uint32_t lane, const ProgramDesc* P, Worklist& wl) {
  LaneState& L = S.lane[lane];
  StageRuntime& rr = P->runtime[P->reset_stage];   // the reset tiles re-armed every other stage
  rr.done = 0;
  rr.deps = ld_volatile(&P->stages[P->reset_stage].deps_init);
  const uint32_t it = L.iter_in_prog + 1;
  L.iter_in_prog = it;
  if (S.mirror) {   // the end time is written before the count
    st_release_sys64(&S.mirror->lane[lane].iter_ns, globaltimer_ns());
    mirror_lane(S, lane, 0, ld_volatile(&S.mirror->lane[lane].iterations) + 1);
  }
  ProgramDesc* np;
  uint32_t ng;
  latest_program(S, lane, np, ng);
  if (np != nullptr && ng != ld_volatile(&L.gen)) {
    begin_iteration(S, lane, np, ng, true, wl);
    return np;
  }
  if (P->iterations != 0 && it >= P->iterations) {
    st_rel(&L.running, 0u);
    mirror_lane(S, lane, 2, 0);
    return P;
  }
  begin_iteration(S, lane, P, ld_volatile(&L.gen), false, wl);
  return P;
}

__device__ void drain(DeviceState& S, uint32_t lane, const ProgramDesc* P, Worklist& wl) {
  LaneState& L = S.lane[lane];
  constexpr int kPush = 64;
  while (wl.n > 0) {
    const uint32_t s = wl.pop();
    trace_stage(S, lane, s, 1, ld_volatile(&L.tag));
    const StageStatic& st = P->stages[s];
    const uint32_t flags = ld_volatile(&st.flags);
    if (flags & kStageMark) mirror_lane(S, lane, 3, ld_volatile(&st.mark));
    if (flags & kStageReset) {
      P = end_iteration(S, lane, P, wl);
      continue;
    }
    const uint32_t tag = ld_volatile(&L.tag) & kTagMask;
    const uint32_t sf = ld_volatile(&st.succ_first), sc = ld_volatile(&st.succ_count);
    uint32_t ring_e[kPush], link_e[kPush];
    int ring_n = 0, link_n = 0;
    for (uint32_t k = 0; k < sc; ++k) {
      const uint32_t j = P->succ[sf + k];
      if (ld_volatile(&P->stages[j].flags) & kStageSkip) continue;
      if (atomicSub(&P->runtime[j].deps, 1u) != 1u) continue;
      uint32_t entry;
      bool link;
      if (!arm(S, lane, P, j, tag, wl, entry, link)) continue;
      if (link) {
        link_e[link_n++] = entry;
        if (link_n == kPush) { ring_push_n(S, L, true, link_e, link_n); link_n = 0; }
      } else {
        ring_e[ring_n++] = entry;
        if (ring_n == kPush) { ring_push_n(S, L, false, ring_e, ring_n); ring_n = 0; }
      }
    }
    ring_push_n(S, L, false, ring_e, ring_n);
    ring_push_n(S, L, true, link_e, link_n);
  }
  if (wl.overflow) raise_error(S, kFabErrWorklist);
}

__device__ void complete_tile(DeviceState& S, uint32_t lane, const ProgramDesc* P, uint32_t s, uint32_t n) {
  const unsigned int d = atomicAdd(&P->runtime[s].done, n) + n;
  if (d == ld_volatile(&P->stages[s].count)) {
    __threadfence();   // acquire the other workers' tiles of the stage before releasing its successors
    Worklist wl;
    wl.n = 0;
    wl.overflow = false;
    wl.push(s);
    drain(S, lane, P, wl);
  }
}

// ---------------------------------------------------------------- scheduling
__device__ void refresh_epoch(DeviceState& S, WorkerState& ws) {
  unsigned long long e = ld_acq(&S.published);
  if (e == ws.epoch) return;
  for (;;) {
    const Snapshot& sn = S.snap[e & 1];
    ws.n_lanes = ld_volatile(&sn.n_lanes);
    ws.lane = ld_volatile(&sn.map[ws.worker]);
    for (int l = 0; l < kMaxLanes; ++l) {
      ws.cap[l] = ld_volatile(&sn.cap[l]);
      ws.order[l] = ld_volatile(&sn.order[l]);
      ws.prog_gen[l] = ld_volatile(&sn.prog_gen[l]);
      ws.prog_snap[l] = ld_volatile(&sn.prog[l]);
    }
    const unsigned long long e2 = ld_acq(&S.published);
    if (e2 == e) break;
    e = e2;
  }
  ws.epoch = e;
  if (S.mirror) {
    st_release_sys64(&S.mirror->worker_epoch_ns[ws.worker], globaltimer_ns());
    st_release_sys64(&S.mirror->worker_epoch[ws.worker], e);
  }
}

__device__ void start_idle_lanes(DeviceState& S, WorkerState& ws) {
  for (uint32_t l = 0; l < ws.n_lanes && l < kMaxLanes; ++l) {
    ProgramDesc* P = ws.prog_snap[l];
    if (P == nullptr) continue;
    LaneState& L = S.lane[l];
    if (ws.prog_gen[l] == ld_acq(&L.gen)) continue;
    if (ld_acq(&L.running) != 0) continue;   // a running lane switches at its own boundary
    if (atomicCAS(&L.running, 0u, 1u) != 0u) continue;
    mirror_lane(S, l, 2, 1);
    Worklist wl;
    wl.n = 0;
    wl.overflow = false;
    begin_iteration(S, l, P, ws.prog_gen[l], true, wl);
    drain(S, l, P, wl);
  }
}

__device__ bool acquire_slot(LaneState& L, uint32_t cap) {
  unsigned int s = ld_volatile(&L.slots);
  while (s < cap) {
    const unsigned int old = atomicCAS(&L.slots, s, s + 1);
    if (old == s) return true;
    s = old;
  }
  return false;
}

__device__ void release_slot(DeviceState& S, WorkerState& ws) {
  if (ws.slot_lane != kNoLane) {
    atomicSub(&S.lane[ws.slot_lane].slots, 1u);
    ws.slot_lane = kNoLane;
  }
}

__device__ void set_claim(WorkerState& ws, const ProgramDesc* P, uint32_t stage, uint32_t index, uint32_t lane,
                          uint32_t link, uint32_t n) {
  ws.prog = P;
  ws.stage = stage;
  ws.tile_lane = lane;
  ws.link = link;
  ws.next_index = index;
  ws.left = n;
}

__device__ bool try_lane(DeviceState& S, WorkerState& ws, uint32_t l) {
  if (l >= kMaxLanes) return false;
  LaneState& L = S.lane[l];
  if (ld_acq(&L.running) == 0) return false;
  const ProgramDesc* P = reinterpret_cast<const ProgramDesc*>(ld_acq(&L.prog));
  if (P == nullptr) return false;
  uint32_t s, idx, n;
  if (ld_acq(&L.ring[1].tail) > ld_volatile(&L.ring[1].head)) {
    bool held = ws.slot_lane == l;
    if (held && ld_volatile(&L.slots) > ws.cap[l]) {   // the grant shrank
      release_slot(S, ws);
      held = false;
    }
    if (!held) {
      release_slot(S, ws);
      if (acquire_slot(L, ws.cap[l])) {
        ws.slot_lane = l;
        held = true;
      }
    }
    if (held) {
      if (take_from(L, true, P, s, idx, n)) {
        set_claim(ws, P, s, idx, l, 1, n);
        return true;
      }
      release_slot(S, ws);
    }
  }
  if (take_from(L, false, P, s, idx, n)) {
    release_slot(S, ws);
    set_claim(ws, P, s, idx, l, 0, n);
    return true;
  }
  return false;
}

__device__ uint32_t schedule(DeviceState& S, WorkerState& ws) {
  refresh_epoch(S, ws);
  if (ld_acq(&S.shutdown) != 0) {
    release_slot(S, ws);
    return kCmdExit;
  }
  start_idle_lanes(S, ws);
  if (ws.lane < ws.n_lanes && try_lane(S, ws, ws.lane)) {
    ws.idle_ns = 64;
    return kCmdRun;
  }
  for (uint32_t i = 0; i < ws.n_lanes && i < kMaxLanes; ++i) {
    const uint32_t l = ws.order[i];
    if (l != ws.lane && try_lane(S, ws, l)) {
      ws.idle_ns = 64;
      return kCmdRun;
    }
  }
  release_slot(S, ws);
  __nanosleep(ws.idle_ns);
  ws.idle_ns = min(ws.idle_ns << 1, max(64u, ld_volatile(&S.idle_cap)));
  return kCmdIdle;
}

// ---------------------------------------------------------------- core tiles
__device__ __forceinline__ void exec_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kExecThreads) : "memory"); }

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

__device__ void tile_router(const TileDesc& t, int tid);
__device__ void tile_norm(const TileDesc& t, int tid, bool add);

// tid: index among the exec threads.
__device__ bool run_core_tile(const WorkSlot& w, int tid, uint32_t worker, unsigned long long* sh_t0) {
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
    case kTileRmsNorm:
      tile_norm(t, tid, false);
      return true;
    case kTileAddNorm:
      tile_norm(t, tid, true);
      return true;
    default:
      return false;
  }
}

// ----------------------------------------------------------- row-wise model tiles
// Row-wise tiles name rows [i0, i0 + i1); a[0] is the operand block.  One warp per
// row, the four exec warps striding over the rows.

// Router tile (kind 38, csrc/fabric/tiles/aux.cuh:326-417, RouterArgs): scores,
// top-K, renormalisation, per-expert counts; the logits row is zeroed once read.
__device__ void tile_router(const TileDesc& t, int tid) {
  const RouterArgs& A = *reinterpret_cast<const RouterArgs*>(t.a[0]);
  const int warp = tid >> 5, lane = tid & 31;
  const int E = static_cast<int>(A.E), K = static_cast<int>(A.K);
  if (E < 1 || E > kMaxExperts || K < 1 || K > kMaxTopK) return;
  for (uint32_t r = t.i0 + warp; r < t.i0 + t.i1; r += kExecThreads / 32) {
    int id;
    float w;
    route_row(reinterpret_cast<float*>(A.logits) + static_cast<size_t>(r) * E, reinterpret_cast<const float*>(A.bias),
              E, K, static_cast<int>(A.scoring), static_cast<int>(A.renorm), A.scale, 1, id, w);
    if (lane < K) {
      reinterpret_cast<int*>(A.topk_ids)[static_cast<size_t>(r) * K + lane] = id;
      reinterpret_cast<float*>(A.topk_w)[static_cast<size_t>(r) * K + lane] = w;
      atomicAdd(reinterpret_cast<int*>(A.counts) + id, 1);
    }
  }
}

// RMSNorm tile (kind 36) and AddNorm tile (kind 41), NormArgs
// (csrc/fabric/tiles/aux.cuh:124-188): AddNorm first forms x = bf16(x2 + acc), stores
// it, zeroes the fp32 accumulator rows, then normalises; gather >= 0 copies the
// normalised row to out2[gather].
__device__ void tile_norm(const TileDesc& t, int tid, bool add) {
  const NormArgs& A = *reinterpret_cast<const NormArgs*>(t.a[0]);
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
      for (int c = lane; c < n16; c += 32) {
        float f[8];
        unpack8(x2[c], f);
        const float4 a0 = acc[2 * c], a1 = acc[2 * c + 1];
        const float sv[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          f[j] = round_bf16(__fadd_rn(f[j], sv[j]));
          ss = __fmaf_rn(f[j], f[j], ss);
        }
        acc[2 * c] = zero;
        acc[2 * c + 1] = zero;
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

struct WorkerShared {
  uint64_t slot_full[2], slot_empty[2];
  GemmBarriers bar;
  WorkSlot slot[2];
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
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh.slot_full[i], 1);
      mbar_init(&sh.slot_empty[i], 3);   // exec thread 0, producer, MMA
    }
    gemm_barriers_init(sh.bar);
    sh.abort_flag = 0;
    sh.ws.epoch = ~0ull;
    sh.ws.worker = worker;
    sh.ws.slot_lane = kNoLane;
    sh.ws.idle_ns = 64;
    sh.ws.lane = kNoLane;
    sh.ws.n_lanes = 0;
    sh.ws.left = 0;
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
    if (lane == 0) {
      WorkerState& ws = sh.ws;
      const unsigned long long t_start = globaltimer_ns();
      for (uint32_t n = 0;; ++n) {
        const int s = n & 1;
        if (!mbar_wait_bounded(&sh.slot_empty[s], ((n >> 1) & 1) ^ 1, abort_flag, kForever)) break;
        uint32_t cmd = kCmdRun;
        if (ws.left == 0) {
          for (;;) {
            cmd = schedule(S, ws);
            if (cmd != kCmdIdle) break;
            const unsigned long long limit = ld_volatile(&S.max_run_ns);
            if (limit && globaltimer_ns() - t_start > limit) {
              raise_error(S, kFabErrDeadline);
              release_slot(S, ws);
              cmd = kCmdExit;
              break;
            }
          }
        } else {
          const unsigned long long limit = ld_volatile(&S.max_run_ns);
          if (ld_acq(&S.shutdown) != 0 || (limit && globaltimer_ns() - t_start > limit)) {
            // leave mid-claim: the remaining tiles of the claim stay unexecuted (the fabric is stopping)
            release_slot(S, ws);
            cmd = kCmdExit;
          }
        }
        WorkSlot& w = sh.slot[s];
        w.cmd = cmd;
        if (cmd == kCmdRun) {
          const uint4* src = reinterpret_cast<const uint4*>(&ws.prog->tiles[ws.next_index]);
          uint4* dst = reinterpret_cast<uint4*>(&w.tile);
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[i] = __ldcg(src + i);
          w.prog = ws.prog;
          w.stage = ws.stage;
          w.tile_lane = ws.tile_lane;
          w.link = ws.link;
          w.index = ws.next_index;
          w.worker_lane = ws.lane;
          w.is_gemm = 0;
          if (w.tile.kind == kTileGemm) {
            if (make_gemm_work(w.tile, w.gemm)) {
              w.is_gemm = 1;
            } else {
              raise_error(S, kFabErrBadTile);
              w.tile.kind = kTileNop;   // completes without running, so the program still ends
            }
          }
          ++ws.next_index;
          --ws.left;
        }
        mbar_arrive(&sh.slot_full[s]);
        if (cmd == kCmdExit) break;
      }
    }
  } else if (warp == 5) {
    // --------------------------------------------------------- TMA producer
    const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
    GemmPipe pipe;
    GemmInflight inflight;
    for (uint32_t n = 0;; ++n) {
      const int s = n & 1;
      if (!mbar_wait_bounded(&sh.slot_full[s], (n >> 1) & 1, abort_flag, kForever)) break;
      const WorkSlot& w = sh.slot[s];
      if (w.cmd == kCmdExit) break;
      bool ok = true;
      if (w.is_gemm) ok = gemm_produce(w.gemm, ring, sh.bar, pipe, inflight, abort_flag, pol_w, pol_x);
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.slot_empty[s]);
      if (!ok) break;
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------ MMA issue
    GemmPipe pipe;
    uint32_t g = 0;   // GEMM tiles seen: accumulator buffer and parity
    for (uint32_t n = 0;; ++n) {
      const int s = n & 1;
      if (!mbar_wait_bounded(&sh.slot_full[s], (n >> 1) & 1, abort_flag, kForever)) break;
      const WorkSlot& w = sh.slot[s];
      if (w.cmd == kCmdExit) break;
      bool ok = true;
      if (w.is_gemm) {
        ok = gemm_mma(w.gemm, ring, sh.bar, pipe, tmem_base, g & 1, (g >> 1) & 1, abort_flag);
        ++g;
      }
      if (lane == 0) mbar_arrive(&sh.slot_empty[s]);
      if (!ok) break;
    }
  } else {
    // ------------------------------------------------------ exec / epilogue
    const int tid = threadIdx.x - 32;
    uint32_t g = 0;
    for (uint32_t n = 0;; ++n) {
      const int s = n & 1;
      if (!mbar_wait_bounded(&sh.slot_full[s], (n >> 1) & 1, abort_flag, kForever)) break;
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
      if (w.is_gemm) {
        if (!gemm_epilogue(w.gemm, sh.bar, tmem_base, g & 1, (g >> 1) & 1, abort_flag) && tid == 0)
          raise_error(S, kFabErrTileWait);
        ++g;
      } else if (!run_core_tile(w, tid, worker, &sh.t0) && tid == 0) {
        raise_error(S, kFabErrBadTile);
      }
      exec_sync();
      if (tid == 0) {
        if (w.link) atomicSub(&S.lane[w.tile_lane].inflight, 1u);
        __threadfence();   // this worker's writes are visible device-wide before the tile counts as done
        note_tile(S, worker, w, 1ull << 62);
        complete_tile(S, w.tile_lane, w.prog, w.stage, 1);
        note_tile(S, worker, w, 0);
        mbar_arrive(&sh.slot_empty[s]);
      }
    }
  }
  // a bounded wait that ran out inside a GEMM role is reported, and every role leaves
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && sh.abort_flag) raise_error(S, kFabErrTileWait);
  if (warp == 6) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

cudaError_t launch_fabric(DeviceState* S, int workers, uint32_t first_worker, cudaStream_t stream) {
  static bool attr = false;
  if (!attr) {
    const cudaError_t err =
        cudaFuncSetAttribute(fabric_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes);
    if (err != cudaSuccess) return err;
    attr = true;
  }
  fabric_kernel<<<workers, kWorkerThreads, kGemmSmemBytes, stream>>>(S, first_worker);
  return cudaGetLastError();
}

}  // namespace fab
}  // namespace mf
