// The host loop behind the C ABI: a host thread that follows the lanes' marks in the
// fabric's pinned mirror and stages host-resident experts into a lane's HBM staging
// buffer with the copy engine, ahead of the layer that will use them.
//
// Counterpart of the reference's HostLoop (csrc/host/host_loop.h:1-90,
// csrc/host/host_loop.cpp:18-160, bound at csrc/bindings.cpp:306-330).  Behaviour kept:
//   * a lane's staging buffer has two halves of `slots` experts; half (layer & 1) holds
//     layer `layer`; experts are staged in the order the caller gives per layer;
//   * a lane's mark is (layer << 8) | phase with phase 1 = attention window, 2 = MoE
//     window, 3 = layer done; the layer staged next is the one the lane works on while
//     its MoE window has not begun, else the following one;
//   * one expert (its w13 block, then its w2 block) is in flight per lane at a time, on
//     the loop's own stream; when it has landed, the expert's entry in the lane's
//     (region, slot) table is switched by ONE aligned 8-byte copy on the same stream, so
//     the expander reads either the old or the new entry, never a mixture; a copy that
//     lands late is harmless, the expander then still finds the host entry;
//   * when a layer is done its half is given back: the entries return to
//     (host_region, expert) and the half is refilled for the layer after next; a new
//     program generation or an idle lane gives both halves back.
// Structure that differs: the decisions are taken by `poll_lane` from a plain snapshot of
// the three mirror words, and everything it does goes through `issue_copy`, `copy_landed` and
// `write_entry`, so the same code runs against the copy engine or, for a loop created without a fabric, against a log that
// a test reads (`monofab_host_loop_inject / _step / _log`): the policy is testable on a
// machine without a GPU.
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#include "../../include/monofab.h"
#include "release.h"
#include "fabric_types.h"

namespace mf {
int fail(int code, const char* fmt, ...);                            // api.cu
const fab::HostMirror* fabric_mirror(const monofab_fabric* f);      // fabric_host.cu
int fabric_device(const monofab_fabric* f);                         // fabric_host.cu
}  // namespace mf

using namespace mf;

namespace {

// Pinned 8-byte table entries that may be queued on the stream at once.  Entry copies queue behind at most
// one expert copy; in that time a lane gives back at most its two halves (2 x slots <= 2 x 256 entries) and
// switches one entry, so 4096 covers several lanes.
constexpr int kEntryRing = 4096;

struct Flip { int expert, slot; };

struct Half {
  int layer = -1;             // layer this half is reserved for, or -1
  int filled = 0;             // experts whose copy has been issued
  std::vector<Flip> flips;    // entries that point into this half
};

struct Snapshot { unsigned long long mark, gen, running; };

struct StagedLane {
  int lane = 0, region = 0, slots = 0;
  uint64_t w13_dst = 0, w2_dst = 0, tables = 0;
  std::vector<std::vector<int>> order;   // per layer, best first
  unsigned long long gen = 0;
  Half half[2];
  bool copying = false;
  int c_half = 0, c_expert = -1, c_slot = -1;
  cudaEvent_t landed = nullptr;
  Snapshot injected{0, 0, 0};   // dry mode
  bool dry_landed = false;      // dry mode: the copy in flight lands at the next poll
};

}  // namespace

struct monofab_host_loop {
  monofab_fabric* fab = nullptr;   // null: dry mode (no CUDA call is made)
  int layers = 0, experts = 0, host_region = 0, device = 0;
  size_t w13_bytes = 0, w2_bytes = 0;
  std::vector<uint64_t> host_w13, host_w2;   // host addresses of the per-layer stacks (0 = no experts)
  std::vector<StagedLane> lanes;
  cudaStream_t stream = nullptr;
  int* entry_ring = nullptr;   // pinned
  int entry_at = 0;
  std::thread thread;
  std::atomic<bool> run{false};
  std::mutex mu;               // lanes / log against the polling thread
  std::atomic<uint64_t> copies{0}, bytes{0}, flips{0}, restores{0}, polls{0};
  std::vector<int32_t> log;    // dry mode: records of 5 ints (kind, lane, layer, expert, slot)
  int error = 0;               // first CUDA error seen by the thread
};

namespace {

enum { kLogCopy = 0, kLogFlip = 1, kLogRestore = 2 };

void log_action(monofab_host_loop* h, int kind, int lane, int layer, int expert, int slot) {
  const int32_t rec[5] = {kind, lane, layer, expert, slot};
  h->log.insert(h->log.end(), rec, rec + 5);
}

bool cuda_ok(monofab_host_loop* h, cudaError_t e) {
  if (e != cudaSuccess && h->error == 0) h->error = static_cast<int>(e);
  return e == cudaSuccess;
}

// The expert's table entry becomes (region, slot): one 8-byte copy, ordered on the loop's
// stream after the expert's bytes.
void write_entry(monofab_host_loop* h, StagedLane& s, int layer, int expert, int region, int slot) {
  if (!h->fab) return;
  int* e = h->entry_ring + 2 * (h->entry_at++ % kEntryRing);
  e[0] = region;
  e[1] = slot;
  const uint64_t dst = s.tables + (static_cast<uint64_t>(layer) * h->experts + expert) * 8;
  cuda_ok(h, cudaMemcpyAsync(reinterpret_cast<void*>(dst), e, 8, cudaMemcpyHostToDevice, h->stream));
}

void give_back(monofab_host_loop* h, StagedLane& s, int which) {
  Half& half = s.half[which];
  if (half.layer >= 0) {
    for (const Flip& f : half.flips) {
      write_entry(h, s, half.layer, f.expert, h->host_region, f.expert);
      if (!h->fab) log_action(h, kLogRestore, s.lane, half.layer, f.expert, f.expert);
      ++h->restores;
    }
  }
  half.flips.clear();
  half.layer = -1;
  half.filled = 0;
}

bool copy_landed(monofab_host_loop* h, StagedLane& s) {
  if (!h->fab) {
    const bool landed = s.dry_landed;
    s.dry_landed = true;   // lands one poll after it was issued
    return landed;
  }
  return cudaEventQuery(s.landed) == cudaSuccess;
}

void issue_copy(monofab_host_loop* h, StagedLane& s, int layer, int expert, int slot) {
  if (h->fab) {
    const uint64_t src13 = h->host_w13[layer] + static_cast<uint64_t>(expert) * h->w13_bytes;
    const uint64_t src2 = h->host_w2[layer] + static_cast<uint64_t>(expert) * h->w2_bytes;
    cuda_ok(h, cudaMemcpyAsync(reinterpret_cast<void*>(s.w13_dst + static_cast<uint64_t>(slot) * h->w13_bytes),
                               reinterpret_cast<const void*>(src13), h->w13_bytes, cudaMemcpyHostToDevice, h->stream));
    cuda_ok(h, cudaMemcpyAsync(reinterpret_cast<void*>(s.w2_dst + static_cast<uint64_t>(slot) * h->w2_bytes),
                               reinterpret_cast<const void*>(src2), h->w2_bytes, cudaMemcpyHostToDevice, h->stream));
    cuda_ok(h, cudaEventRecord(s.landed, h->stream));
  } else {
    log_action(h, kLogCopy, s.lane, layer, expert, slot);
    s.dry_landed = false;
  }
  ++h->copies;
  h->bytes += h->w13_bytes + h->w2_bytes;
}

Snapshot read_mirror(monofab_host_loop* h, const StagedLane& s) {
  if (!h->fab) return s.injected;
  // the device publishes running, then gen, then marks; read in the opposite order
  const volatile fab::LaneMirror* m = &fabric_mirror(h->fab)->lane[s.lane];
  Snapshot v;
  v.mark = m->mark;
  std::atomic_thread_fence(std::memory_order_acquire);
  v.gen = m->gen;
  std::atomic_thread_fence(std::memory_order_acquire);
  v.running = m->running;
  return v;
}

void poll_lane(monofab_host_loop* h, StagedLane& s) {
  const Snapshot now = read_mirror(h, s);
  if (s.copying && copy_landed(h, s)) {   // publish the expert that has arrived
    s.copying = false;
    Half& half = s.half[s.c_half];
    if (half.layer >= 0) {
      write_entry(h, s, half.layer, s.c_expert, s.region, s.c_slot);
      if (!h->fab) log_action(h, kLogFlip, s.lane, half.layer, s.c_expert, s.c_slot);
      half.flips.push_back({s.c_expert, s.c_slot});
      ++h->flips;
    }
  }
  if (now.gen != s.gen || !now.running) {   // another program, or nothing runs: start over
    if (!s.copying) {
      give_back(h, s, 0);
      give_back(h, s, 1);
      s.gen = now.gen;
    }
    if (!now.running) return;
  }
  const int layer = static_cast<int>(now.mark >> 8), phase = static_cast<int>(now.mark & 0xff);
  const int working = phase == 3 ? layer + 1 : layer;   // the layer the lane is in
  for (int i = 0; i < 2; ++i)
    if (s.half[i].layer >= 0 && s.half[i].layer < working && !(s.copying && s.c_half == i)) give_back(h, s, i);
  if (s.copying) return;
  // once a layer's MoE window has begun its expander has read the table: stage for the next layer
  const int target = (phase == 2 && layer == working) ? working + 1 : working;
  if (target >= h->layers) return;
  Half& half = s.half[target & 1];
  if (half.layer != target) {
    if (half.layer >= 0) return;   // an earlier layer still uses this half
    half.layer = target;
    half.filled = 0;
  }
  const std::vector<int>& order = s.order[target];
  if (half.filled >= static_cast<int>(order.size()) || half.filled >= s.slots) return;
  if (h->fab && (h->host_w13[target] == 0 || h->host_w2[target] == 0)) return;   // a layer without experts
  const int expert = order[half.filled];
  const int slot = (target & 1) * s.slots + half.filled;
  ++half.filled;
  issue_copy(h, s, target, expert, slot);
  s.copying = true;
  s.c_half = target & 1;
  s.c_expert = expert;
  s.c_slot = slot;
}

void poll_all(monofab_host_loop* h) {
  std::lock_guard<std::mutex> lock(h->mu);
  for (StagedLane& s : h->lanes) poll_lane(h, s);
  ++h->polls;
}

void wind_down(monofab_host_loop* h) {
  std::lock_guard<std::mutex> lock(h->mu);
  for (StagedLane& s : h->lanes) {
    if (s.copying && h->fab) cudaEventSynchronize(s.landed);
    s.copying = false;
    give_back(h, s, 0);
    give_back(h, s, 1);
  }
  if (h->fab) cudaStreamSynchronize(h->stream);
}

void thread_main(monofab_host_loop* h, int poll_us) {
  cudaSetDevice(h->device);
  while (h->run.load(std::memory_order_acquire)) {
    poll_all(h);
    std::this_thread::sleep_for(std::chrono::microseconds(poll_us));
  }
  wind_down(h);
}

}  // namespace

extern "C" {

int monofab_host_loop_create(monofab_fabric* fab, int layers, int experts, size_t w13_bytes, size_t w2_bytes,
                             const uint64_t* host_w13, const uint64_t* host_w2, int host_region,
                             monofab_host_loop** out) {
  if (!out || layers < 1 || experts < 1) return fail(MONOFAB_EINVAL, "host loop: bad shape");
  if (fab && (!host_w13 || !host_w2 || w13_bytes == 0 || w2_bytes == 0))
    return fail(MONOFAB_EINVAL, "host loop: the per-layer host stacks and expert sizes are needed");
  auto* h = new monofab_host_loop;
  h->fab = fab;
  h->layers = layers;
  h->experts = experts;
  h->host_region = host_region;
  h->w13_bytes = w13_bytes;
  h->w2_bytes = w2_bytes;
  h->host_w13.assign(layers, 0);
  h->host_w2.assign(layers, 0);
  for (int l = 0; l < layers && host_w13 && host_w2; ++l) {
    h->host_w13[l] = host_w13[l];
    h->host_w2[l] = host_w2[l];
  }
  if (fab) {
    h->device = fabric_device(fab);
    cudaError_t e = cudaSetDevice(h->device);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void**>(&h->entry_ring), kEntryRing * 8, cudaHostAllocDefault);
    if (e != cudaSuccess) {
      delete h;
      return fail(MONOFAB_ECUDA, "host loop: %s", cudaGetErrorString(e));
    }
  }
  *out = h;
  return MONOFAB_OK;
}

int monofab_host_loop_add_lane(monofab_host_loop* h, int lane, int region, uint64_t w13_dst, uint64_t w2_dst,
                               int slots, uint64_t tables, const int32_t* order, const int32_t* order_offsets) {
  if (!h || !order_offsets || slots < 1 || lane < 0 || lane >= fab::kMaxLanes)
    return fail(MONOFAB_EINVAL, "host loop: bad lane");
  if (h->run.load()) return fail(MONOFAB_EINVAL, "host loop: add lanes before start");
  if (h->fab && (!w13_dst || !w2_dst || !tables)) return fail(MONOFAB_EINVAL, "host loop: staging buffers and tables are needed");
  StagedLane s;
  s.lane = lane;
  s.region = region;
  s.slots = slots;
  s.w13_dst = w13_dst;
  s.w2_dst = w2_dst;
  s.tables = tables;
  s.order.resize(h->layers);
  for (int l = 0; l < h->layers; ++l) {
    if (order_offsets[l + 1] < order_offsets[l]) return fail(MONOFAB_EINVAL, "host loop: order offsets decrease");
    for (int i = order_offsets[l]; i < order_offsets[l + 1]; ++i) {
      if (order[i] < 0 || order[i] >= h->experts) return fail(MONOFAB_EINVAL, "host loop: expert %d out of range", order[i]);
      s.order[l].push_back(order[i]);
    }
  }
  if (h->fab) {
    cudaError_t e = cudaSetDevice(h->device);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&s.landed, cudaEventDisableTiming);
    if (e != cudaSuccess) return fail(MONOFAB_ECUDA, "host loop: %s", cudaGetErrorString(e));
  }
  std::lock_guard<std::mutex> lock(h->mu);
  h->lanes.push_back(std::move(s));
  return MONOFAB_OK;
}

int monofab_host_loop_start(monofab_host_loop* h, int poll_us) {
  if (!h) return fail(MONOFAB_EINVAL, "host loop: null");
  if (!h->fab) return fail(MONOFAB_EINVAL, "host loop: a loop without a fabric is stepped by hand");
  if (h->run.exchange(true)) return MONOFAB_OK;
  h->thread = std::thread(thread_main, h, poll_us < 1 ? 1 : poll_us);
  return MONOFAB_OK;
}

int monofab_host_loop_stop(monofab_host_loop* h) {
  if (!h) return fail(MONOFAB_EINVAL, "host loop: null");
  if (h->run.exchange(false) && h->thread.joinable()) h->thread.join();
  if (h->error) return fail(MONOFAB_ECUDA, "host loop: %s", cudaGetErrorString(static_cast<cudaError_t>(h->error)));
  return MONOFAB_OK;
}

int monofab_host_loop_stats(monofab_host_loop* h, uint64_t out[5]) {
  if (!h || !out) return fail(MONOFAB_EINVAL, "host loop: null");
  out[0] = h->copies.load();
  out[1] = h->bytes.load();
  out[2] = h->flips.load();
  out[3] = h->restores.load();
  out[4] = h->polls.load();
  return MONOFAB_OK;
}

int monofab_host_loop_destroy(monofab_host_loop* h) {
  if (!h) return MONOFAB_OK;
  monofab_host_loop_stop(h);
  if (h->fab) {
    cudaSetDevice(h->device);
    // the fabric this loop served may still be resident: then these wait until it has stopped
    for (StagedLane& s : h->lanes) release_event(h->device, s.landed);
    release_stream(h->device, h->stream);
    release_host(h->device, h->entry_ring);
  }
  delete h;
  return MONOFAB_OK;
}

int monofab_host_loop_inject(monofab_host_loop* h, int lane_index, uint64_t mark, uint64_t gen, uint64_t running) {
  if (!h || h->fab) return fail(MONOFAB_EINVAL, "host loop: marks are injected only into a loop without a fabric");
  std::lock_guard<std::mutex> lock(h->mu);
  if (lane_index < 0 || lane_index >= static_cast<int>(h->lanes.size())) return fail(MONOFAB_EINVAL, "host loop: no such lane");
  h->lanes[lane_index].injected = Snapshot{mark, gen, running};
  return MONOFAB_OK;
}

int monofab_host_loop_step(monofab_host_loop* h) {
  if (!h || h->fab) return fail(MONOFAB_EINVAL, "host loop: only a loop without a fabric is stepped by hand");
  poll_all(h);
  return MONOFAB_OK;
}

int monofab_host_loop_log(monofab_host_loop* h, int32_t* out, int cap, int* n) {
  if (!h || !n) return fail(MONOFAB_EINVAL, "host loop: null");
  std::lock_guard<std::mutex> lock(h->mu);
  const int records = static_cast<int>(h->log.size() / 5);
  *n = records;
  if (out)
    for (int i = 0; i < records && i < cap; ++i) std::memcpy(out + 5 * i, h->log.data() + 5 * i, 5 * sizeof(int32_t));
  return MONOFAB_OK;
}

}  // extern "C"
