// Scheduling and DAG bookkeeping of the persistent fabric: how a worker finds its
// next tiles, and what happens when a stage's last tile completes.
//
// What is fixed by the wire protocol (the reference's, csrc/fabric/runtime.cuh:155-509,
// because its Python program builder, its state readers and its tests see it):
//   * a ring entry is tag << 20 | stage; tags are 12 bits, 0 = never activated;
//   * a ring has a reservation counter, a published tail and a consumer head;
//     entries become visible in reservation order;
//   * StageRuntime::tag_next = tag << 32 | next tile; a claim is ONE fetch-and-add on
//     it, valid only if the word still carried the entry's tag and tiles were left;
//   * a stage is armed (tag_next := tag << 32) before its entry is published;
//   * link stages are taken only under one of the lane's `cap` slots;
//   * the host mirror's write order (end time before count; running before gen).
// Everything else here is this library's own: the scheduler is a whole warp that
// probes up to 32 ring entries at once, drops a run of exhausted head entries with a
// single compare-and-swap, walks a visiting order computed once per epoch, and sizes
// claims for a 148-SM machine; completion releases a stage's successors 32 at a time.
#pragma once
#include "fabric_types.h"
#include "ptx.cuh"

namespace mf {
namespace fab {

constexpr uint32_t kStageBits = 20;
constexpr uint32_t kStageMask = (1u << kStageBits) - 1;
constexpr uint32_t kTagMask = 0xfffu;
constexpr int kWorklistCap = 448;   // bounded by the worker's shared memory; an overflow is reported, not fatal
// A claim takes about 1/256 of what is left of a stage, at least one tile and at most
// eight: with one worker per SM the first round over a large stage hands out eights,
// and the tail is shared out tile by tile so that the workers finish together.
constexpr uint32_t kClaimMax = 8;
constexpr uint32_t kClaimShareLog2 = 8;
constexpr unsigned long long kRingWaitBudgetNs = 2000000000ull;
constexpr unsigned kWarp = 0xffffffffu;

enum : uint32_t { kCmdRun = 0, kCmdIdle = 1, kCmdExit = 2 };

template <class T>
__device__ __forceinline__ T ld_volatile(const T* p) { return *reinterpret_cast<const volatile T*>(p); }
__device__ __forceinline__ unsigned int ld_acq(const unsigned int* p) { return ld_acquire_gpu(p); }
__device__ __forceinline__ unsigned long long ld_acq(const unsigned long long* p) { return ld_acquire_gpu64(p); }
__device__ __forceinline__ void st_rel(unsigned int* p, unsigned int v) { st_release_gpu(p, v); }
__device__ __forceinline__ void st_rel(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ void raise_error(DeviceState& S, unsigned long long bit) {
  const unsigned long long now = atomicOr(&S.error, bit) | bit;
  if (S.mirror) st_release_sys64(&S.mirror->error, now);   // pinned host memory
}

__device__ __forceinline__ void trace_stage(DeviceState& S, uint32_t lane, uint32_t s, uint32_t event, uint32_t tag) {
  const uint32_t cap = ld_volatile(&S.trace_cap);
  if (cap == 0) return;
  const uint32_t i = atomicAdd(&S.trace_n, 1u);
  if (i >= cap) return;
  unsigned long long* r = reinterpret_cast<unsigned long long*>(ld_volatile(&S.trace_ptr)) + 2ull * i;
  r[0] = static_cast<unsigned long long>(s) | (static_cast<unsigned long long>(lane) << 32) |
         (static_cast<unsigned long long>(event) << 40) | (static_cast<unsigned long long>(tag & kTagMask) << 48);
  r[1] = globaltimer_ns();
}

enum MirrorField { kMirrorIterations, kMirrorGen, kMirrorRunning, kMirrorMark };
__device__ __forceinline__ void mirror_lane(DeviceState& S, uint32_t lane, MirrorField what, unsigned long long v) {
  if (!S.mirror) return;
  LaneMirror& m = S.mirror->lane[lane];
  if (what == kMirrorIterations) st_release_sys64(&m.iterations, v);
  else if (what == kMirrorGen) st_release_sys64(&m.gen, v);
  else if (what == kMirrorRunning) st_release_sys64(&m.running, v);
  else {
    st_release_sys64(&m.mark_ns, globaltimer_ns());   // the time is there before the mark that announces it
    st_release_sys64(&m.mark, v);
  }
}

// ------------------------------------------------------------------ wire words
struct StageWord {   // decoded StageRuntime::tag_next
  uint32_t tag, next;
  __device__ explicit StageWord(unsigned long long w) : tag(static_cast<uint32_t>(w >> 32) & kTagMask), next(static_cast<uint32_t>(w)) {}
};
__device__ __forceinline__ uint32_t ring_word(uint32_t stage, uint32_t tag) {
  return ((tag & kTagMask) << kStageBits) | (stage & kStageMask);
}
__device__ __forceinline__ unsigned long long armed_word(uint32_t tag) {
  return static_cast<unsigned long long>(tag & kTagMask) << 32;
}

// Completed stages a releasing warp still has to process (shared memory; lane 0 owns it).
template <int kCap>
struct WorklistOf {
  uint32_t v[kCap];
  int n;
  bool overflow;
  __device__ void clear() { n = 0; overflow = false; }
  __device__ void push(uint32_t s) {
    if (n < kCap) v[n++] = s; else overflow = true;
  }
  __device__ uint32_t pop() { return v[--n]; }
};
using Worklist = WorklistOf<kWorklistCap>;
using SmallWorklist = WorklistOf<16>;   // the scheduler's: it only ever releases the empty stages at a program's start

// ---------------------------------------------------------------------- rings
// Producer side, any one thread: reserve m places, fill them, and move the published tail over
// them once every earlier reservation has been published.  The wait for earlier producers is
// bounded; if it runs out the entries stay unpublished and the host sees kFabErrRingWait.
__device__ __forceinline__ void ring_publish(DeviceState& S, Ring& R, const uint32_t* words, int m) {
  if (m <= 0) return;
  const unsigned long long at = atomicAdd(&R.reserve, static_cast<unsigned long long>(m));
  for (int i = 0; i < m; ++i) R.ids[(at + i) & (kRingCap - 1)] = words[i];
  const unsigned long long give_up = globaltimer_ns() + kRingWaitBudgetNs;
  for (unsigned int pause = 32; ld_acq(&R.tail) != at; pause = pause < 512 ? pause * 2 : pause) {
    __nanosleep(pause);
    if (globaltimer_ns() > give_up) {
      raise_error(S, kFabErrRingWait);
      return;
    }
  }
  st_rel(&R.tail, at + m);
}

// ---------------------------------------------------------------------- claims
struct Claim {
  uint32_t stage, first_tile, n;
};

// Tiles a ring entry can still give: 0 if its stage has moved on to another activation or
// has been handed out completely.  A read-only probe; the claim itself re-checks.
__device__ __forceinline__ uint32_t tiles_left(const ProgramDesc* P, uint32_t word) {
  const uint32_t s = word & kStageMask;
  if (s >= P->n_stages) return 0;
  const StageWord w(ld_acq(&P->runtime[s].tag_next));
  const uint32_t count = ld_volatile(&P->stages[s].count);
  return (w.tag == (word >> kStageBits) && w.next < count) ? count - w.next : 0;
}

// The fetch-and-add.  `left` is the probe's answer and only sizes the claim.
__device__ __forceinline__ bool claim_tiles(const ProgramDesc* P, uint32_t word, uint32_t left, Claim& c) {
  const uint32_t s = word & kStageMask;
  uint32_t want = left >> kClaimShareLog2;
  want = want < 1 ? 1 : (want > kClaimMax ? kClaimMax : want);
  const StageWord before(atomicAdd(&P->runtime[s].tag_next, static_cast<unsigned long long>(want)));
  // The add may land on a later activation of the stage (or on a stage that was closed, tag 0).
  // On a later activation it hands out that activation's tiles, which is as good; on a closed
  // stage, or past the end, it hands out nothing and the overshoot is harmless: `next` is only
  // ever compared with the count.
  if (before.tag == 0) return false;
  if (before.tag != (word >> kStageBits)) __threadfence();   // a later activation: its stage record may be newer than the probe saw
  const uint32_t count = ld_volatile(&P->stages[s].count);
  if (before.next >= count) return false;
  c.stage = s;
  c.first_tile = ld_volatile(&P->stages[s].first) + before.next;
  c.n = min(want, count - before.next);
  return true;
}

// Consumer side, the WHOLE warp: lane i probes entry head + i; a run of exhausted entries at the
// head is dropped with one compare-and-swap; the first entry that still has tiles is claimed.
__device__ __forceinline__ bool ring_take(Ring& R, const ProgramDesc* P, Claim& c) {
  const int lane = threadIdx.x & 31;
  // head and tail by two lanes at once (one round trip): a pair read out of step only looks empty, or
  // begins at entries that are exhausted and fail the compare-and-swap below
  unsigned long long word01 = 0;
  if (lane == 0) word01 = ld_acq(&R.head);
  else if (lane == 1) word01 = ld_acq(&R.tail);
  const unsigned long long head = __shfl_sync(kWarp, word01, 0), tail = __shfl_sync(kWarp, word01, 1);
  if (tail <= head) return false;
  const int n = static_cast<int>(min(tail - head, 32ull));
  uint32_t word = 0, left = 0;
  if (lane < n) {
    word = ld_volatile(&R.ids[(head + lane) & (kRingCap - 1)]);
    left = tiles_left(P, word);
  }
  unsigned live = __ballot_sync(kWarp, left != 0);
  const int spent = live ? __ffs(live) - 1 : n;   // exhausted entries in front of the first live one
  if (spent > 0 && lane == 0) atomicCAS(&R.head, head, head + spent);   // losing the race is fine: someone else dropped them
  while (live) {
    const int src = __ffs(live) - 1;
    live &= live - 1;
    int ok = 0;
    if (lane == src) ok = claim_tiles(P, word, left, c);
    ok = __shfl_sync(kWarp, ok, src);
    if (ok) {
      c.stage = __shfl_sync(kWarp, c.stage, src);
      c.first_tile = __shfl_sync(kWarp, c.first_tile, src);
      c.n = __shfl_sync(kWarp, c.n, src);
      return true;
    }
  }
  return false;
}

// -------------------------------------------------------- iterations of a lane
// The program a lane should be running according to the latest published plan.
__device__ __forceinline__ void planned_program(DeviceState& S, uint32_t lane, ProgramDesc*& prog, uint32_t& gen) {
  for (unsigned long long e = ld_acq(&S.published);;) {
    const Snapshot& sn = S.snap[e & 1];
    prog = ld_volatile(&sn.prog[lane]);
    gen = ld_volatile(&sn.prog_gen[lane]);
    const unsigned long long again = ld_acq(&S.published);   // the snapshot is double-buffered: re-read if a publish intervened
    if (again == e) return;
    e = again;
  }
}

// Arm stage s for activation `tag`.  Returns true if it has tiles (the caller publishes its ring
// word), false if it is empty and therefore complete at once (pushed on the worklist).
template <class WL>
__device__ __forceinline__ bool arm_stage(DeviceState& S, uint32_t lane, const ProgramDesc* P, uint32_t s, uint32_t tag,
                                          WL& wl) {
  trace_stage(S, lane, s, 0, tag);
  if (ld_volatile(&P->stages[s].count) == 0) {
    wl.push(s);
    return false;
  }
  atomicExch(&P->runtime[s].tag_next, armed_word(tag));
  return true;
}

// One thread.  Opens the next activation wave of a lane's program: a new tag (never 0) and the
// program's first stage.  `switched`: P is not the program the lane ran before.
template <class WL>
__device__ __forceinline__ void open_wave(DeviceState& S, uint32_t lane, const ProgramDesc* P, uint32_t gen, bool switched,
                                          WL& wl) {
  LaneState& L = S.lane[lane];
  if (switched) {
    for (Ring& R : L.ring) atomicExch(&R.head, ld_acq(&R.tail));   // what is left in the rings belongs to the old program
    L.iter_in_prog = 0;
    st_rel(&L.prog, reinterpret_cast<unsigned long long>(P));
    st_rel(&L.gen, gen);
    mirror_lane(S, lane, kMirrorGen, gen);
  }
  uint32_t tag = (ld_volatile(&L.tag) + 1) & kTagMask;
  if (tag == 0) tag = 1;
  st_rel(&L.tag, tag);
  const uint32_t s = P->first_stage;
  if (arm_stage(S, lane, P, s, tag, wl)) {
    const uint32_t word = ring_word(s, tag);
    ring_publish(S, L.ring[(ld_volatile(&P->stages[s].flags) & kStageLink) ? 1 : 0], &word, 1);
  }
}

// One thread.  The reset stage completed: count the iteration, then switch to a newer program,
// stop after the program's last iteration, or go round again.  Returns the program now current.
template <class WL>
__device__ __forceinline__ const ProgramDesc* close_iteration(DeviceState& S, uint32_t lane, const ProgramDesc* P, WL& wl) {
  LaneState& L = S.lane[lane];
  StageRuntime& reset = P->runtime[P->reset_stage];   // the reset tiles re-armed every stage but their own
  reset.done = 0;
  reset.deps = ld_volatile(&P->stages[P->reset_stage].deps_init);
  const uint32_t done_iterations = ++L.iter_in_prog;
  if (S.mirror) {
    st_release_sys64(&S.mirror->lane[lane].iter_ns, globaltimer_ns());
    mirror_lane(S, lane, kMirrorIterations, ld_volatile(&S.mirror->lane[lane].iterations) + 1);
  }
  ProgramDesc* wanted;
  uint32_t wanted_gen;
  planned_program(S, lane, wanted, wanted_gen);
  if (wanted != nullptr && wanted_gen != ld_volatile(&L.gen)) {
    open_wave(S, lane, wanted, wanted_gen, true, wl);
    return wanted;
  }
  if (P->iterations != 0 && done_iterations >= P->iterations) {
    st_rel(&L.running, 0u);
    mirror_lane(S, lane, kMirrorRunning, 0);
    return P;
  }
  open_wave(S, lane, P, ld_volatile(&L.gen), false, wl);
  return P;
}

// The WHOLE warp.  Processes the worklist: for every completed stage, lane 0 reports marks and
// handles the iteration boundary; the stage's successors are counted down and armed by the 32
// lanes side by side, and their ring words go out in two publications (ungated, link), so a
// stage with 128 successors releases them in a few microseconds.
template <class WL>
__device__ __forceinline__ void release_successors(DeviceState& S, uint32_t lane_id, const ProgramDesc* P, WL& wl) {
  const int lane = threadIdx.x & 31;
  LaneState& L = S.lane[lane_id];
  for (;;) {
    uint32_t first = 0, count = 0, tag = 0;
    int have = 0;
    if (lane == 0) {
      while (wl.n > 0 && !have) {
        const uint32_t s = wl.pop();
        trace_stage(S, lane_id, s, 1, ld_volatile(&L.tag));
        const StageStatic& st = P->stages[s];
        const uint32_t flags = ld_volatile(&st.flags);
        if (flags & kStageMark) mirror_lane(S, lane_id, kMirrorMark, ld_volatile(&st.mark));
        if (flags & kStageReset) {
          P = close_iteration(S, lane_id, P, wl);
        } else {
          tag = ld_volatile(&L.tag) & kTagMask;
          first = ld_volatile(&st.succ_first);
          count = ld_volatile(&st.succ_count);
          have = 1;
        }
      }
    }
    if (!__shfl_sync(kWarp, have, 0)) break;
    first = __shfl_sync(kWarp, first, 0);
    count = __shfl_sync(kWarp, count, 0);
    tag = __shfl_sync(kWarp, tag, 0);
    const ProgramDesc* Pw = reinterpret_cast<const ProgramDesc*>(__shfl_sync(kWarp, reinterpret_cast<unsigned long long>(P), 0));
    for (uint32_t base = 0; base < count; base += 32) {
      enum { kNone, kUngated, kLink, kEmpty };
      int fate = kNone;
      uint32_t word = 0, succ = 0;
      if (base + lane < count) {
        succ = Pw->succ[first + base + lane];
        const uint32_t flags = ld_volatile(&Pw->stages[succ].flags);
        if (!(flags & kStageSkip) && atomicSub(&Pw->runtime[succ].deps, 1u) == 1u) {
          trace_stage(S, lane_id, succ, 0, tag);
          if (ld_volatile(&Pw->stages[succ].count) == 0) {
            fate = kEmpty;
          } else {
            atomicExch(&Pw->runtime[succ].tag_next, armed_word(tag));
            __threadfence();   // armed before lane 0 publishes the word
            word = ring_word(succ, tag);
            fate = (flags & kStageLink) ? kLink : kUngated;
          }
        }
      }
      for (int want = kUngated; want <= kEmpty; ++want) {
        unsigned mask = __ballot_sync(kWarp, fate == want);
        uint32_t batch[32];
        int n = 0;
        for (; mask; mask &= mask - 1) {
          const uint32_t v = __shfl_sync(kWarp, want == kEmpty ? succ : word, __ffs(mask) - 1);
          if (lane == 0) {
            if (want == kEmpty) wl.push(v);
            else batch[n++] = v;
          }
        }
        if (lane == 0 && want != kEmpty) ring_publish(S, L.ring[want == kLink ? 1 : 0], batch, n);
      }
    }
  }
  if (lane == 0 && wl.overflow) raise_error(S, kFabErrWorklist);
}

// The WHOLE warp.  n tiles of stage s are done; the warp whose tiles complete the stage releases
// its successors.
__device__ __forceinline__ void tiles_completed(DeviceState& S, uint32_t lane_id, const ProgramDesc* P, uint32_t s, uint32_t n,
                                                Worklist& wl) {
  int last = 0;
  if ((threadIdx.x & 31) == 0) last = atomicAdd(&P->runtime[s].done, n) + n == ld_volatile(&P->stages[s].count);
  if (!__shfl_sync(kWarp, last, 0)) return;
  __threadfence();   // the other workers' tiles of the stage are visible before its successors start
  if ((threadIdx.x & 31) == 0) {
    wl.clear();
    wl.push(s);
  }
  __syncwarp();
  release_successors(S, lane_id, P, wl);
}

// ------------------------------------------------------------------ the worker
// Scheduling state of one worker (shared memory).  Written by lane 0 of the scheduler warp
// between warp barriers; the link accounting is also read by the completing exec thread.
struct WorkerState {
  unsigned long long epoch;
  uint32_t worker, lane, n_lanes, idle_ns;
  uint32_t cap[kMaxLanes], prog_gen[kMaxLanes];
  ProgramDesc* prog_snap[kMaxLanes];
  uint32_t visit[kMaxLanes];   // lanes in the order this worker looks for work: its own, then the borrowing order
  uint32_t n_visit;
  // the current claim
  const ProgramDesc* prog;
  uint32_t stage, tile_lane, link, next_index, left;
  uint32_t row_block;   // a kind-45 tile runs as one record per row block: the block of its next record
  // The link slot this worker holds (kNoLane = none).  The worker runs its records through a pipeline
  // behind the scheduler, so the slot goes back only when the exec warps have finished the last link
  // record issued under it.
  uint32_t slot_lane;
  uint32_t link_last;                  // records issued up to and including the last link record
  const volatile unsigned int* done;   // records the exec warps have finished
};

// Lane 0 of the scheduler warp.
__device__ __forceinline__ void give_slot_back(DeviceState& S, WorkerState& ws) {
  if (ws.slot_lane == kNoLane) return;
  if (ws.done) {   // bounded: after a second the slot goes back regardless (the fabric is stuck or stopping)
    const unsigned long long give_up = globaltimer_ns() + 1000000000ull;
    while (static_cast<int>(*ws.done - ws.link_last) < 0 && globaltimer_ns() < give_up) __nanosleep(64);
  }
  atomicSub(&S.lane[ws.slot_lane].slots, 1u);
  ws.slot_lane = kNoLane;
}

__device__ __forceinline__ bool take_slot(LaneState& L, uint32_t cap) {
  for (unsigned int held = ld_volatile(&L.slots); held < cap;) {
    const unsigned int seen = atomicCAS(&L.slots, held, held + 1);
    if (seen == held) return true;
    held = seen;
  }
  return false;
}

// The WHOLE scheduler warp.  Adopt a newer published plan: lane l < 4 reads lane l's share of the
// snapshot, lane 0 the rest; the read is repeated if a publish intervened.
__device__ __forceinline__ void adopt_epoch(DeviceState& S, WorkerState& ws) {
  const int lane = threadIdx.x & 31;
  unsigned long long e = 0;
  if (lane == 0) e = ld_acq(&S.published);
  e = __shfl_sync(kWarp, e, 0);
  if (e == ws.epoch) return;
  __shared__ uint32_t s_order[kMaxLanes];
  for (;;) {
    const Snapshot& sn = S.snap[e & 1];
    if (lane < kMaxLanes) {
      ws.cap[lane] = ld_volatile(&sn.cap[lane]);
      s_order[lane] = ld_volatile(&sn.order[lane]);
      ws.prog_gen[lane] = ld_volatile(&sn.prog_gen[lane]);
      ws.prog_snap[lane] = ld_volatile(&sn.prog[lane]);
    }
    if (lane == 0) {
      ws.n_lanes = min(ld_volatile(&sn.n_lanes), static_cast<uint32_t>(kMaxLanes));
      ws.lane = ld_volatile(&sn.map[ws.worker]);
    }
    unsigned long long again = 0;
    if (lane == 0) again = ld_acq(&S.published);
    again = __shfl_sync(kWarp, again, 0);
    if (again == e) break;
    e = again;
  }
  __syncwarp();
  if (lane == 0) {
    ws.n_visit = 0;
    if (ws.lane < ws.n_lanes) ws.visit[ws.n_visit++] = ws.lane;
    for (uint32_t i = 0; i < ws.n_lanes; ++i)
      if (s_order[i] != ws.lane && s_order[i] < kMaxLanes) ws.visit[ws.n_visit++] = s_order[i];
    ws.epoch = e;
    if (S.mirror) {
      st_release_sys64(&S.mirror->worker_epoch_ns[ws.worker], globaltimer_ns());
      st_release_sys64(&S.mirror->worker_epoch[ws.worker], e);
    }
  }
  __syncwarp();
}

// The WHOLE scheduler warp.  A lane whose planned program is not the one it runs, and that is not
// running, is started by whichever worker gets there first.
__device__ __forceinline__ void start_waiting_lanes(DeviceState& S, WorkerState& ws, SmallWorklist& wl) {
  const int lane = threadIdx.x & 31;
  for (uint32_t l = 0; l < ws.n_lanes; ++l) {
    int mine = 0;
    ProgramDesc* P = ws.prog_snap[l];
    if (lane == 0 && P != nullptr) {
      LaneState& L = S.lane[l];
      if (ws.prog_gen[l] != ld_acq(&L.gen) && ld_acq(&L.running) == 0 && atomicCAS(&L.running, 0u, 1u) == 0u) {
        mirror_lane(S, l, kMirrorRunning, 1);
        wl.clear();
        open_wave(S, l, P, ws.prog_gen[l], true, wl);
        mine = 1;
      }
    }
    if (__shfl_sync(kWarp, mine, 0)) release_successors(S, l, P, wl);   // an empty first stage completes at once
  }
}

// The WHOLE scheduler warp.  Look for tiles in lane l: link stages first, under a slot; then the
// ungated ring.  On success the claim is in ws (written by lane 0).
__device__ __forceinline__ bool look_in_lane(DeviceState& S, WorkerState& ws, uint32_t l) {
  const int lane = threadIdx.x & 31;
  LaneState& L = S.lane[l];
  // `running` and the link ring's ends by three lanes at once, then the program (which is read after
  // `running`, as before): two round trips instead of four
  unsigned long long v = 0;
  if (lane == 0) v = ld_acq(&L.running);
  else if (lane == 1) v = ld_acq(&L.ring[1].tail);
  else if (lane == 2) v = ld_volatile(&L.ring[1].head);
  const bool running = __shfl_sync(kWarp, v, 0) != 0;
  if (!running) return false;
  const bool link_waiting = __shfl_sync(kWarp, v, 1) > __shfl_sync(kWarp, v, 2);
  unsigned long long prog = 0;
  if (lane == 0) prog = ld_acq(&L.prog);
  const ProgramDesc* P = reinterpret_cast<const ProgramDesc*>(__shfl_sync(kWarp, prog, 0));
  if (P == nullptr) return false;
  Claim c;
  if (link_waiting) {
    int held = 0;
    if (lane == 0) {
      held = ws.slot_lane == l;
      if (held && ld_volatile(&L.slots) > ws.cap[l]) {   // the grant shrank under this worker
        give_slot_back(S, ws);
        held = 0;
      }
      if (!held) {
        give_slot_back(S, ws);   // a slot of another lane
        if (take_slot(L, ws.cap[l])) {
          ws.slot_lane = l;
          held = 1;
        }
      }
    }
    if (__shfl_sync(kWarp, held, 0)) {
      if (ring_take(L.ring[1], P, c)) {
        if (lane == 0) {
          ws.prog = P; ws.stage = c.stage; ws.tile_lane = l; ws.link = 1; ws.next_index = c.first_tile; ws.left = c.n;
        }
        return true;
      }
      if (lane == 0) give_slot_back(S, ws);
    }
  }
  if (!ring_take(L.ring[0], P, c)) return false;
  if (lane == 0) {
    give_slot_back(S, ws);
    ws.prog = P; ws.stage = c.stage; ws.tile_lane = l; ws.link = 0; ws.next_index = c.first_tile; ws.left = c.n;
  }
  return true;
}

// The WHOLE scheduler warp.  One scheduling round: kCmdRun with a claim in ws, kCmdExit when the
// host asked the fabric to stop, or kCmdIdle after a back-off that grows to the plan's idle cap.
__device__ __forceinline__ uint32_t schedule(DeviceState& S, WorkerState& ws, SmallWorklist& wl) {
  const int lane = threadIdx.x & 31;
  adopt_epoch(S, ws);
  int stop = 0;
  if (lane == 0) stop = ld_acq(&S.shutdown) != 0;
  if (__shfl_sync(kWarp, stop, 0)) {
    if (lane == 0) give_slot_back(S, ws);
    return kCmdExit;
  }
  start_waiting_lanes(S, ws, wl);
  __syncwarp();
  const uint32_t n_visit = ws.n_visit;
  for (uint32_t i = 0; i < n_visit; ++i) {
    if (look_in_lane(S, ws, ws.visit[i])) {
      if (lane == 0) ws.idle_ns = 64;
      __syncwarp();
      return kCmdRun;
    }
  }
  if (lane == 0) {
    give_slot_back(S, ws);
    __nanosleep(ws.idle_ns);
    const uint32_t cap = max(64u, ld_volatile(&S.idle_cap));
    ws.idle_ns = min(ws.idle_ns * 2, cap);
  }
  __syncwarp();
  return kCmdIdle;
}

}  // namespace fab
}  // namespace mf
