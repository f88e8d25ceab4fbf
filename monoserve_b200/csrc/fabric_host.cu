// Host side of the fabric behind the C ABI: device state, the program pool,
// pinned staging, upload / release / publish, safe reads and writes while the
// kernel runs, lane statistics, iteration timers, the tensor-map table.
//
// Mirrors the reference's Fabric class (csrc/host/fabric.h:31-168,
// csrc/host/fabric.cpp:61-475, bound at csrc/bindings.cpp:184-296): nothing is
// cudaMalloc'ed after construction, every copy to or from the device goes
// through pinned staging on a control stream that is independent of the stream
// the persistent kernel runs on, and one mutex serialises the host methods.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/monofab.h"
#include "release.h"
#include "fabric_types.h"

namespace mf {

int fail(int code, const char* fmt, ...);   // api.cu
int encode_map(CUtensorMap* map, int dtype, const void* base, int rank, const uint64_t* dims,
               const uint64_t* strides, const uint32_t* box, int swizzle);   // api.cu

namespace fab {
cudaError_t launch_fabric(DeviceState* S, int workers, uint32_t first_worker, cudaStream_t stream);
}

#define MF_CUDA(expr)                                                                          \
  do {                                                                                         \
    cudaError_t e_ = (expr);                                                                   \
    if (e_ != cudaSuccess) return fail(MONOFAB_ECUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

struct PoolBlock { size_t off, size; };

struct ProgramRecord {
  size_t blocks[5];       // offsets of tiles, stages, runtime, succ, desc in the pool
  size_t sizes[5];
  uint32_t gen, n_tiles, n_stages, first_stage, reset_stage, iterations;
};

}  // namespace mf

using namespace mf;
using namespace mf::fab;

struct monofab_fabric {
  std::mutex mu;
  int device = 0, num_sms = 0, num_workers = 0;
  bool running = false;
  cudaStream_t run_stream = nullptr, ctrl = nullptr;
  DeviceState* state = nullptr;          // device
  HostMirror* mirror = nullptr;          // pinned host, device-visible
  uint8_t* pool = nullptr;
  size_t pool_bytes = 0;
  std::vector<PoolBlock> free_list;      // sorted by offset
  uint8_t* staging = nullptr;            // pinned
  size_t staging_bytes = 16u << 20;
  unsigned long long epoch = 0;
  uint32_t next_gen = 1;
  std::map<uint64_t, ProgramRecord> programs;
  std::map<uint64_t, size_t> blobs;      // device address -> size
  CUtensorMap* map_table = nullptr;      // device: records of 4 slots each
  int map_count = 0, map_cap = 4096;
  uint64_t lane_handle[kMaxLanes] = {0, 0, 0, 0};
  std::vector<cudaStream_t> caller_streams;   // launches made by start_on, waited for by stop
};

namespace mf {
// for the host loop (host_loop.cu)
const fab::HostMirror* fabric_mirror(const monofab_fabric* f) { return f->mirror; }
int fabric_device(const monofab_fabric* f) { return f->device; }
}  // namespace mf

namespace mf {

static bool pool_alloc(monofab_fabric* f, size_t bytes, size_t align, size_t* off) {
  bytes = (bytes + 63) & ~size_t(63);
  for (size_t i = 0; i < f->free_list.size(); ++i) {
    PoolBlock& b = f->free_list[i];
    const size_t start = (b.off + align - 1) & ~(align - 1);
    if (start + bytes > b.off + b.size) continue;
    const size_t tail = b.off + b.size - (start + bytes);
    const size_t head = start - b.off;
    const PoolBlock old = b;
    f->free_list.erase(f->free_list.begin() + i);
    if (tail) f->free_list.insert(f->free_list.begin() + i, PoolBlock{start + bytes, tail});
    if (head) f->free_list.insert(f->free_list.begin() + i, PoolBlock{old.off, head});
    *off = start;
    return true;
  }
  return false;
}

static void pool_free(monofab_fabric* f, size_t off, size_t bytes) {
  bytes = (bytes + 63) & ~size_t(63);
  size_t i = 0;
  while (i < f->free_list.size() && f->free_list[i].off < off) ++i;
  f->free_list.insert(f->free_list.begin() + i, PoolBlock{off, bytes});
  // coalesce with neighbours
  if (i + 1 < f->free_list.size() && f->free_list[i].off + f->free_list[i].size == f->free_list[i + 1].off) {
    f->free_list[i].size += f->free_list[i + 1].size;
    f->free_list.erase(f->free_list.begin() + i + 1);
  }
  if (i > 0 && f->free_list[i - 1].off + f->free_list[i - 1].size == f->free_list[i].off) {
    f->free_list[i - 1].size += f->free_list[i].size;
    f->free_list.erase(f->free_list.begin() + i);
  }
}

// Copies through pinned staging on the control stream; safe while the kernel runs.
static int to_device(monofab_fabric* f, void* dst, const void* src, size_t bytes) {
  const uint8_t* s = static_cast<const uint8_t*>(src);
  uint8_t* d = static_cast<uint8_t*>(dst);
  while (bytes) {
    const size_t n = bytes < f->staging_bytes ? bytes : f->staging_bytes;
    std::memcpy(f->staging, s, n);
    MF_CUDA(cudaMemcpyAsync(d, f->staging, n, cudaMemcpyHostToDevice, f->ctrl));
    MF_CUDA(cudaStreamSynchronize(f->ctrl));
    s += n;
    d += n;
    bytes -= n;
  }
  return MONOFAB_OK;
}

static int from_device(monofab_fabric* f, void* dst, const void* src, size_t bytes) {
  uint8_t* d = static_cast<uint8_t*>(dst);
  const uint8_t* s = static_cast<const uint8_t*>(src);
  while (bytes) {
    const size_t n = bytes < f->staging_bytes ? bytes : f->staging_bytes;
    MF_CUDA(cudaMemcpyAsync(f->staging, s, n, cudaMemcpyDeviceToHost, f->ctrl));
    MF_CUDA(cudaStreamSynchronize(f->ctrl));
    std::memcpy(d, f->staging, n);
    s += n;
    d += n;
    bytes -= n;
  }
  return MONOFAB_OK;
}

static int stop_locked(monofab_fabric* f) {
  if (!f->running) return MONOFAB_OK;
  const unsigned int one = 1;
  if (int r = to_device(f, &f->state->shutdown, &one, 4)) return r;
  MF_CUDA(cudaStreamSynchronize(f->run_stream));
  for (cudaStream_t st : f->caller_streams) MF_CUDA(cudaStreamSynchronize(st));
  f->caller_streams.clear();
  f->running = false;
  fabric_stopped(f->device);   // carries out the releases that were queued while this kernel was resident
  return MONOFAB_OK;
}

}  // namespace mf

extern "C" {

int monofab_fabric_create(int num_workers, int device, size_t pool_bytes, monofab_fabric** out) {
  if (!out) return fail(MONOFAB_EINVAL, "fabric_create: NULL argument");
  if (num_workers < 0 || num_workers > kMaxWorkers) return fail(MONOFAB_EINVAL, "fabric_create: num_workers=%d outside [0, %d]", num_workers, kMaxWorkers);
  MF_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  MF_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) return fail(MONOFAB_ECUDA, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
  monofab_fabric* f = new monofab_fabric();
  f->device = device;
  f->num_sms = prop.multiProcessorCount;
  f->num_workers = num_workers > 0 ? (num_workers < f->num_sms ? num_workers : f->num_sms) : f->num_sms;
  f->pool_bytes = pool_bytes ? pool_bytes : (size_t(1) << 30);
  cudaError_t e = cudaStreamCreateWithFlags(&f->run_stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&f->ctrl, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&f->state), sizeof(DeviceState));
  if (e == cudaSuccess) e = cudaMemset(f->state, 0, sizeof(DeviceState));
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&f->pool), f->pool_bytes);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&f->map_table), sizeof(CUtensorMap) * 4 * f->map_cap);
  if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void**>(&f->mirror), sizeof(HostMirror), cudaHostAllocMapped | cudaHostAllocPortable);
  if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void**>(&f->staging), f->staging_bytes, cudaHostAllocDefault);
  if (e != cudaSuccess) {
    const int r = fail(MONOFAB_ECUDA, "fabric_create: %s", cudaGetErrorString(e));
    monofab_fabric_destroy(f);
    return r;
  }
  std::memset(f->mirror, 0, sizeof(HostMirror));
  f->free_list.push_back(PoolBlock{0, f->pool_bytes});
  void* mirror_dev = nullptr;
  cudaHostGetDevicePointer(&mirror_dev, f->mirror, 0);
  DeviceState init;
  std::memset(&init, 0, sizeof init);
  // only the scalar fields are copied; the rings are already zero
  const unsigned int idle_cap = 4096;
  const unsigned long long max_run = 120ull * 1000000000ull;
  cudaMemcpy(&f->state->idle_cap, &idle_cap, 4, cudaMemcpyHostToDevice);
  cudaMemcpy(&f->state->max_run_ns, &max_run, 8, cudaMemcpyHostToDevice);
  cudaMemcpy(&f->state->mirror, &mirror_dev, 8, cudaMemcpyHostToDevice);
  *out = f;
  return MONOFAB_OK;
}

int monofab_fabric_destroy(monofab_fabric* f) {
  if (!f) return MONOFAB_OK;
  {
    std::lock_guard<std::mutex> lock(f->mu);
    stop_locked(f);
  }
  // another fabric may still be resident on this device: its releases wait for it
  release_device(f->device, f->state);
  release_device(f->device, f->pool);
  release_device(f->device, f->map_table);
  release_host(f->device, f->mirror);
  release_host(f->device, f->staging);
  release_stream(f->device, f->run_stream);
  release_stream(f->device, f->ctrl);
  delete f;
  return MONOFAB_OK;
}

int monofab_fabric_info(monofab_fabric* f, int32_t* num_workers, int32_t* num_sms, int32_t* running, uint64_t* epoch) {
  if (!f) return fail(MONOFAB_EINVAL, "fabric_info: NULL handle");
  std::lock_guard<std::mutex> lock(f->mu);
  if (num_workers) *num_workers = f->num_workers;
  if (num_sms) *num_sms = f->num_sms;
  if (running) *running = f->running;
  if (epoch) *epoch = f->epoch;
  return MONOFAB_OK;
}

int monofab_fabric_start(monofab_fabric* f) {
  if (!f) return fail(MONOFAB_EINVAL, "fabric_start: NULL handle");
  std::lock_guard<std::mutex> lock(f->mu);
  if (f->running) return MONOFAB_OK;
  MF_CUDA(cudaSetDevice(f->device));
  const unsigned int zero = 0;
  if (int r = to_device(f, &f->state->shutdown, &zero, 4)) return r;
  MF_CUDA(launch_fabric(f->state, f->num_workers, 0, f->run_stream));
  f->running = true;
  fabric_started(f->device);
  return MONOFAB_OK;
}

int monofab_fabric_start_on(monofab_fabric* f, uint64_t stream, uint64_t context, int workers, int first_worker) {
  if (!f) return fail(MONOFAB_EINVAL, "fabric_start_on: NULL handle");
  std::lock_guard<std::mutex> lock(f->mu);
  if (workers <= 0 || first_worker < 0 || first_worker + workers > f->num_workers)
    return fail(MONOFAB_EINVAL, "fabric_start_on: workers [%d, %d) outside [0, %d)", first_worker, first_worker + workers,
                f->num_workers);
  MF_CUDA(cudaSetDevice(f->device));
  if (!f->running) {
    const unsigned int zero = 0;
    if (int r = to_device(f, &f->state->shutdown, &zero, 4)) return r;
  }
  // An optional driver context (a green context's) is made current around the launch.
  typedef CUresult (*PushFn)(CUcontext);
  typedef CUresult (*PopFn)(CUcontext*);
  PushFn push = nullptr;
  PopFn pop = nullptr;
  if (context) {
    void *a = nullptr, *b = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuCtxPushCurrent", &a, cudaEnableDefault, &q) != cudaSuccess ||
        cudaGetDriverEntryPoint("cuCtxPopCurrent", &b, cudaEnableDefault, &q) != cudaSuccess || !a || !b)
      return fail(MONOFAB_ECUDA, "fabric_start_on: the driver's context calls are not available");
    push = reinterpret_cast<PushFn>(a);
    pop = reinterpret_cast<PopFn>(b);
    if (push(reinterpret_cast<CUcontext>(context)) != CUDA_SUCCESS) return fail(MONOFAB_ECUDA, "fabric_start_on: context push failed");
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const cudaError_t e = launch_fabric(f->state, workers, static_cast<uint32_t>(first_worker), st);
  if (context) {
    CUcontext prev;
    pop(&prev);
  }
  if (e != cudaSuccess) return fail(MONOFAB_ECUDA, "fabric_start_on: launch: %s", cudaGetErrorString(e));
  f->caller_streams.push_back(st);
  if (!f->running) fabric_started(f->device);
  f->running = true;
  return MONOFAB_OK;
}

int monofab_fabric_lane_ring(monofab_fabric* f, int lane, int link, int max_entries, uint64_t counters[3],
                             uint32_t* entries, int* n_entries) {
  if (!f || !counters || !n_entries) return fail(MONOFAB_EINVAL, "fabric_lane_ring: NULL argument");
  if (lane < 0 || lane >= kMaxLanes) return fail(MONOFAB_EINVAL, "fabric_lane_ring: lane %d", lane);
  std::lock_guard<std::mutex> lock(f->mu);
  const Ring* ring = &f->state->lane[lane].ring[link ? 1 : 0];
  unsigned long long head = 0, tail = 0, reserve = 0;
  if (int r = from_device(f, &head, &ring->head, 8)) return r;
  if (int r = from_device(f, &tail, &ring->tail, 8)) return r;
  if (int r = from_device(f, &reserve, &ring->reserve, 8)) return r;
  counters[0] = head;
  counters[1] = tail;
  counters[2] = reserve;
  int n = 0;
  if (entries && tail > head && max_entries > 0) {
    std::vector<unsigned int> ids(kRingCap);
    if (int r = from_device(f, ids.data(), ring->ids, sizeof(unsigned int) * kRingCap)) return r;
    for (unsigned long long p = head; p < tail && n < max_entries; ++p) entries[n++] = ids[p & (kRingCap - 1)];
  }
  *n_entries = n;
  return MONOFAB_OK;
}

int monofab_fabric_wait_note_address(monofab_fabric* f, uint64_t* addr) {
  if (!f || !addr) return fail(MONOFAB_EINVAL, "fabric_wait_note_address: NULL argument");
  *addr = reinterpret_cast<uint64_t>(&f->state->worker_wait[0][0]);
  return MONOFAB_OK;
}

int monofab_fabric_stop(monofab_fabric* f) {
  if (!f) return fail(MONOFAB_EINVAL, "fabric_stop: NULL handle");
  std::lock_guard<std::mutex> lock(f->mu);
  return stop_locked(f);
}

int monofab_fabric_set_limits(monofab_fabric* f, uint32_t idle_cap_ns, uint64_t max_run_ns) {
  if (!f) return fail(MONOFAB_EINVAL, "fabric_set_limits: NULL handle");
  std::lock_guard<std::mutex> lock(f->mu);
  if (idle_cap_ns)
    if (int r = to_device(f, &f->state->idle_cap, &idle_cap_ns, 4)) return r;
  const unsigned long long v = max_run_ns;
  return to_device(f, &f->state->max_run_ns, &v, 8);
}

int monofab_fabric_upload(monofab_fabric* f, const int64_t* tiles, int n_tiles, const int32_t* stages, int n_stages,
                          const int32_t* succ, int n_succ, int first_stage, int reset_stage, int iterations,
                          uint64_t* handle) {
  if (!f || !handle || !stages || !succ) return fail(MONOFAB_EINVAL, "fabric_upload: NULL argument");
  if (n_tiles < 0 || n_stages < 1 || n_succ < 1) return fail(MONOFAB_EINVAL, "fabric_upload: empty program");
  if (n_tiles > 0 && !tiles) return fail(MONOFAB_EINVAL, "fabric_upload: NULL tiles");
  if (n_stages > (1 << 20)) return fail(MONOFAB_EINVAL, "fabric_upload: %d stages exceed the 20-bit stage id", n_stages);
  if (first_stage < 0 || first_stage >= n_stages || reset_stage < 0 || reset_stage >= n_stages)
    return fail(MONOFAB_EINVAL, "fabric_upload: first_stage=%d / reset_stage=%d outside [0, %d)", first_stage, reset_stage, n_stages);
  for (int s = 0; s < n_stages; ++s) {
    const int32_t* r = stages + 8 * s;
    if (r[0] < 0 || r[1] < 0 || r[0] + r[1] > n_tiles)
      return fail(MONOFAB_EINVAL, "fabric_upload: stage %d names tiles [%d, %d) of %d", s, r[0], r[0] + r[1], n_tiles);
    if (r[2] < 0 || r[3] < 0 || r[2] + r[3] > n_succ)
      return fail(MONOFAB_EINVAL, "fabric_upload: stage %d names successors [%d, %d) of %d", s, r[2], r[2] + r[3], n_succ);
  }
  for (int k = 0; k < n_succ; ++k)
    if (succ[k] < 0 || succ[k] >= n_stages) return fail(MONOFAB_EINVAL, "fabric_upload: successor %d is stage %d of %d", k, succ[k], n_stages);
  std::lock_guard<std::mutex> lock(f->mu);
  ProgramRecord rec{};
  const size_t sizes[5] = {size_t(n_tiles ? n_tiles : 1) * 64, size_t(n_stages) * 32, size_t(n_stages) * 16,
                           size_t(n_succ) * 4, sizeof(ProgramDesc)};
  int got = 0;
  for (; got < 5; ++got) {
    rec.sizes[got] = sizes[got];
    if (!pool_alloc(f, sizes[got], 64, &rec.blocks[got])) break;
  }
  if (got < 5) {
    for (int i = 0; i < got; ++i) pool_free(f, rec.blocks[i], rec.sizes[i]);
    return fail(MONOFAB_EINVAL, "fabric_upload: the program pool of %zu bytes is exhausted", f->pool_bytes);
  }
  uint8_t* base = f->pool;
  std::vector<StageRuntime> rt(n_stages);
  for (int s = 0; s < n_stages; ++s) rt[s] = StageRuntime{0ull, 0u, static_cast<unsigned int>(stages[8 * s + 4])};
  ProgramDesc d{};
  d.tiles = reinterpret_cast<TileDesc*>(base + rec.blocks[0]);
  d.stages = reinterpret_cast<StageStatic*>(base + rec.blocks[1]);
  d.runtime = reinterpret_cast<StageRuntime*>(base + rec.blocks[2]);
  d.succ = reinterpret_cast<uint32_t*>(base + rec.blocks[3]);
  d.n_tiles = n_tiles;
  d.n_stages = n_stages;
  d.first_stage = first_stage;
  d.reset_stage = reset_stage;
  d.iterations = iterations;
  d.gen = rec.gen = f->next_gen++;
  rec.n_tiles = n_tiles;
  rec.n_stages = n_stages;
  rec.first_stage = first_stage;
  rec.reset_stage = reset_stage;
  rec.iterations = iterations;
  int r = 0;
  if (n_tiles) r = to_device(f, d.tiles, tiles, size_t(n_tiles) * 64);
  if (!r) r = to_device(f, d.stages, stages, size_t(n_stages) * 32);
  if (!r) r = to_device(f, d.runtime, rt.data(), size_t(n_stages) * 16);
  if (!r) r = to_device(f, d.succ, succ, size_t(n_succ) * 4);
  if (!r) r = to_device(f, base + rec.blocks[4], &d, sizeof d);
  if (r) {
    for (int i = 0; i < 5; ++i) pool_free(f, rec.blocks[i], rec.sizes[i]);
    return r;
  }
  const uint64_t h = reinterpret_cast<uint64_t>(base + rec.blocks[4]);
  f->programs[h] = rec;
  *handle = h;
  return MONOFAB_OK;
}

int monofab_fabric_release(monofab_fabric* f, uint64_t handle) {
  if (!f) return fail(MONOFAB_EINVAL, "fabric_release: NULL handle");
  std::lock_guard<std::mutex> lock(f->mu);
  auto it = f->programs.find(handle);
  if (it == f->programs.end()) return fail(MONOFAB_EINVAL, "fabric_release: unknown program handle");
  for (int l = 0; l < kMaxLanes; ++l)
    if (f->lane_handle[l] == handle && f->running)
      return fail(MONOFAB_EINVAL, "fabric_release: the program is published on lane %d of a running fabric", l);
  for (int i = 0; i < 5; ++i) pool_free(f, it->second.blocks[i], it->second.sizes[i]);
  f->programs.erase(it);
  return MONOFAB_OK;
}

int monofab_fabric_program_info(monofab_fabric* f, uint64_t handle, uint32_t info[6]) {
  if (!f || !info) return fail(MONOFAB_EINVAL, "fabric_program_info: NULL argument");
  std::lock_guard<std::mutex> lock(f->mu);
  auto it = f->programs.find(handle);
  if (it == f->programs.end()) return fail(MONOFAB_EINVAL, "fabric_program_info: unknown program handle");
  const ProgramRecord& r = it->second;
  info[0] = r.gen; info[1] = r.n_tiles; info[2] = r.n_stages; info[3] = r.first_stage; info[4] = r.reset_stage;
  info[5] = r.iterations;
  return MONOFAB_OK;
}

int monofab_fabric_publish(monofab_fabric* f, const int32_t* map, int n_map, const uint32_t* caps, const int32_t* order,
                           const uint64_t* programs, int n_lanes, const uint32_t* forms, uint64_t* epoch_out) {
  if (!f || !map || !caps || !order || !programs) return fail(MONOFAB_EINVAL, "fabric_publish: NULL argument");
  if (n_lanes < 1 || n_lanes > kMaxLanes) return fail(MONOFAB_EINVAL, "fabric_publish: %d lanes outside [1, %d]", n_lanes, kMaxLanes);
  if (n_map < 0 || n_map > kMaxWorkers) return fail(MONOFAB_EINVAL, "fabric_publish: map of %d workers", n_map);
  std::lock_guard<std::mutex> lock(f->mu);
  Snapshot sn;
  std::memset(&sn, 0, sizeof sn);
  std::memset(sn.map, kNoLane, sizeof sn.map);
  for (int w = 0; w < n_map; ++w) {
    if (map[w] != static_cast<int>(kNoLane) && (map[w] < 0 || map[w] >= n_lanes))
      return fail(MONOFAB_EINVAL, "fabric_publish: worker %d is mapped to lane %d of %d", w, map[w], n_lanes);
    sn.map[w] = static_cast<uint8_t>(map[w]);
  }
  for (int l = 0; l < n_lanes; ++l) {
    if (order[l] < 0 || order[l] >= n_lanes) return fail(MONOFAB_EINVAL, "fabric_publish: order[%d]=%d", l, order[l]);
    sn.cap[l] = caps[l];
    sn.order[l] = order[l];
    const uint32_t fm = forms ? forms[l] : 64;
    if (fm != 0 && fm != 16 && fm != 32 && fm != 64 && fm != 128) return fail(MONOFAB_EINVAL, "fabric_publish: form %u", fm);
    sn.form[l] = fm;
    if (programs[l]) {
      auto it = f->programs.find(programs[l]);
      if (it == f->programs.end()) return fail(MONOFAB_EINVAL, "fabric_publish: lane %d names an unknown program", l);
      for (int k = 0; k < l; ++k)
        if (programs[k] == programs[l]) return fail(MONOFAB_EINVAL, "fabric_publish: one program on lanes %d and %d", k, l);
      sn.prog[l] = reinterpret_cast<ProgramDesc*>(programs[l]);
      sn.prog_gen[l] = it->second.gen;
    }
  }
  sn.n_workers = f->num_workers;
  sn.n_lanes = n_lanes;
  const unsigned long long e = f->epoch + 1;
  sn.epoch = e;
  if (int r = to_device(f, &f->state->snap[e & 1], &sn, sizeof sn)) return r;
  if (int r = to_device(f, &f->state->published, &e, 8)) return r;   // the epoch word goes last
  f->epoch = e;
  for (int l = 0; l < kMaxLanes; ++l) f->lane_handle[l] = l < n_lanes ? programs[l] : 0;
  if (epoch_out) *epoch_out = e;
  return MONOFAB_OK;
}

int monofab_fabric_progress(monofab_fabric* f, uint64_t lanes[4][5], uint64_t* worker_epoch, uint64_t* worker_epoch_ns,
                            uint64_t* error) {
  if (!f || !lanes) return fail(MONOFAB_EINVAL, "fabric_progress: NULL argument");
  // lock-free reads of the pinned mirror, in the opposite order of the device's writes
  const volatile HostMirror* m = f->mirror;
  for (int l = 0; l < kMaxLanes; ++l) {
    const unsigned long long running = m->lane[l].running;
    std::atomic_thread_fence(std::memory_order_acquire);
    const unsigned long long iterations = m->lane[l].iterations;
    std::atomic_thread_fence(std::memory_order_acquire);
    lanes[l][0] = iterations;
    lanes[l][1] = m->lane[l].gen;
    lanes[l][2] = running;
    lanes[l][3] = m->lane[l].mark;
    lanes[l][4] = m->lane[l].mark_ns;
  }
  for (int w = 0; w < kMaxWorkers; ++w) {
    if (worker_epoch) worker_epoch[w] = m->worker_epoch[w];
    if (worker_epoch_ns) worker_epoch_ns[w] = m->worker_epoch_ns[w];
  }
  if (error) *error = m->error;
  return MONOFAB_OK;
}

int monofab_fabric_lane_stats(monofab_fabric* f, int lane, uint32_t stats[7]) {
  if (!f || !stats) return fail(MONOFAB_EINVAL, "fabric_lane_stats: NULL argument");
  if (lane < 0 || lane >= kMaxLanes) return fail(MONOFAB_EINVAL, "fabric_lane_stats: lane %d", lane);
  std::lock_guard<std::mutex> lock(f->mu);
  unsigned int raw[8];
  if (int r = from_device(f, raw, &f->state->lane[lane].slots, sizeof raw)) return r;
  // slots, inflight, inflight_max, running, tag, iter_in_prog, gen
  for (int i = 0; i < 7; ++i) stats[i] = raw[i];
  return MONOFAB_OK;
}

int monofab_fabric_reset_inflight_max(monofab_fabric* f, int lane) {
  if (!f || lane < 0 || lane >= kMaxLanes) return fail(MONOFAB_EINVAL, "fabric_reset_inflight_max: bad argument");
  std::lock_guard<std::mutex> lock(f->mu);
  const unsigned int zero = 0;
  return to_device(f, &f->state->lane[lane].inflight_max, &zero, 4);
}

int monofab_fabric_read(monofab_fabric* f, uint64_t src, void* dst, size_t bytes) {
  if (!f || !dst || !src) return fail(MONOFAB_EINVAL, "fabric_read: NULL argument");
  std::lock_guard<std::mutex> lock(f->mu);
  return from_device(f, dst, reinterpret_cast<const void*>(src), bytes);
}

int monofab_fabric_write(monofab_fabric* f, uint64_t dst, const void* src, size_t bytes) {
  if (!f || !dst || !src) return fail(MONOFAB_EINVAL, "fabric_write: NULL argument");
  std::lock_guard<std::mutex> lock(f->mu);
  return to_device(f, reinterpret_cast<void*>(dst), src, bytes);
}

int monofab_fabric_blob_alloc(monofab_fabric* f, size_t bytes, uint64_t* addr) {
  if (!f || !addr || !bytes) return fail(MONOFAB_EINVAL, "fabric_blob_alloc: bad argument");
  std::lock_guard<std::mutex> lock(f->mu);
  size_t off;
  if (!pool_alloc(f, bytes, 256, &off)) return fail(MONOFAB_EINVAL, "fabric_blob_alloc: the pool of %zu bytes is exhausted", f->pool_bytes);
  *addr = reinterpret_cast<uint64_t>(f->pool + off);
  f->blobs[*addr] = bytes;
  return MONOFAB_OK;
}

int monofab_fabric_blob_free(monofab_fabric* f, uint64_t addr) {
  if (!f) return fail(MONOFAB_EINVAL, "fabric_blob_free: NULL handle");
  std::lock_guard<std::mutex> lock(f->mu);
  auto it = f->blobs.find(addr);
  if (it == f->blobs.end()) return fail(MONOFAB_EINVAL, "fabric_blob_free: unknown blob");
  pool_free(f, static_cast<size_t>(reinterpret_cast<uint8_t*>(addr) - f->pool), it->second);
  f->blobs.erase(it);
  return MONOFAB_OK;
}

int monofab_fabric_set_trace(monofab_fabric* f, uint64_t ptr, uint32_t capacity) {
  if (!f) return fail(MONOFAB_EINVAL, "fabric_set_trace: NULL handle");
  std::lock_guard<std::mutex> lock(f->mu);
  const unsigned int zero = 0;
  if (int r = to_device(f, &f->state->trace_cap, &zero, 4)) return r;   // off while the pointer changes
  if (int r = to_device(f, &f->state->trace_n, &zero, 4)) return r;
  const unsigned long long p = ptr;
  if (int r = to_device(f, &f->state->trace_ptr, &p, 8)) return r;
  return to_device(f, &f->state->trace_cap, &capacity, 4);
}

int monofab_fabric_trace_count(monofab_fabric* f, uint32_t* count) {
  if (!f || !count) return fail(MONOFAB_EINVAL, "fabric_trace_count: NULL argument");
  std::lock_guard<std::mutex> lock(f->mu);
  return from_device(f, count, &f->state->trace_n, 4);
}

int monofab_fabric_worker_tiles(monofab_fabric* f, uint64_t* words, uint64_t* since_ns) {
  if (!f || !words) return fail(MONOFAB_EINVAL, "fabric_worker_tiles: NULL argument");
  std::lock_guard<std::mutex> lock(f->mu);
  if (int r = from_device(f, words, f->state->worker_tile, sizeof(uint64_t) * kMaxWorkers)) return r;
  if (since_ns) return from_device(f, since_ns, f->state->worker_tile_ns, sizeof(uint64_t) * kMaxWorkers);
  return MONOFAB_OK;
}

int monofab_fabric_wait_notes(monofab_fabric* f, uint64_t* notes) {
  if (!f || !notes) return fail(MONOFAB_EINVAL, "fabric_wait_notes: NULL argument");
  std::lock_guard<std::mutex> lock(f->mu);
  return from_device(f, notes, f->state->worker_wait, sizeof(uint64_t) * kMaxWorkers * 4);
}

int monofab_fabric_iteration_times(monofab_fabric* f, int lane, uint64_t start, int count, double timeout_s,
                                   uint64_t* end_ns) {
  if (!f || !end_ns || lane < 0 || lane >= kMaxLanes || count < 1) return fail(MONOFAB_EINVAL, "fabric_iteration_times: bad argument");
  // Polls the mirror: the device writes iter_ns, then iterations.  Iterations that
  // complete between two polls are missed, so poll tightly.
  const volatile LaneMirror* m = &f->mirror->lane[lane];
  const auto t0 = std::chrono::steady_clock::now();
  int got = 0;
  unsigned long long last = ~0ull;
  while (got < count) {
    const unsigned long long it = m->iterations;
    std::atomic_thread_fence(std::memory_order_acquire);
    const unsigned long long ns = m->iter_ns;
    if (it != last && it > start) {
      if (it - start - 1 >= static_cast<unsigned long long>(got)) end_ns[got++] = ns;
      last = it;
    }
    if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout_s)
      return fail(MONOFAB_EINVAL, "fabric_iteration_times: timed out after %d of %d iterations", got, count);
  }
  return MONOFAB_OK;
}

int monofab_fabric_tensor_map(monofab_fabric* f, uint64_t base, const uint64_t* dims, const uint64_t* strides_bytes,
                              const uint32_t* box, int rank, int dtype, int swizzle, uint64_t* handle) {
  if (!f || !dims || !strides_bytes || !box || !handle) return fail(MONOFAB_EINVAL, "fabric_tensor_map: NULL argument");
  if (rank < 2 || rank > 5) return fail(MONOFAB_EINVAL, "fabric_tensor_map: rank %d outside [2, 5]", rank);
  std::lock_guard<std::mutex> lock(f->mu);
  if (f->map_count >= f->map_cap) return fail(MONOFAB_EINVAL, "fabric_tensor_map: the table of %d maps is full", f->map_cap);
  // Record = three encodings of the same tensor: [0] the caller's box; for rank-3
  // weight tensors (box of one z slice) also [1] box (64, 16, 1) and [2] box (64, 128, 1), which the
  // B200 GEMM tile uses instead of the 64-row box the reference's tile asks for.
  CUtensorMap rec[4];   // [3] holds flags (monofab_fabric_tensor_map_packed)
  std::memset(rec, 0, sizeof rec);
  if (int r = encode_map(&rec[0], dtype, reinterpret_cast<const void*>(base), rank, dims, strides_bytes, box, swizzle)) return r;
  if (rank == 3 && box[2] == 1) {
    // e4m3 weights: a stage of the GEMM holds two 64-element K steps, i.e. rows of 128 bytes, whatever
    // K extent the caller's box has (the reference's own maps ask for 64 x 64 bytes)
    const uint32_t kbox = dtype == 2 ? 128 : box[0];
    const uint32_t b16[3] = {kbox, 16, 1}, b128[3] = {kbox, 128, 1};
    if (int r = encode_map(&rec[1], dtype, reinterpret_cast<const void*>(base), rank, dims, strides_bytes, b16, swizzle)) return r;
    if (int r = encode_map(&rec[2], dtype, reinterpret_cast<const void*>(base), rank, dims, strides_bytes, b128, swizzle)) return r;
  }
  CUtensorMap* dst = f->map_table + 4 * f->map_count;
  if (int r = to_device(f, dst, rec, sizeof rec)) return r;
  ++f->map_count;
  *handle = reinterpret_cast<uint64_t>(dst);
  return MONOFAB_OK;
}

int monofab_fabric_tensor_map_packed(monofab_fabric* f, uint64_t handle, int packed) {
  if (!f) return fail(MONOFAB_EINVAL, "fabric_tensor_map_packed: NULL handle");
  std::lock_guard<std::mutex> lock(f->mu);
  const uint64_t lo = reinterpret_cast<uint64_t>(f->map_table), hi = reinterpret_cast<uint64_t>(f->map_table + 4 * f->map_count);
  if (handle < lo || handle >= hi || (handle - lo) % (4 * sizeof(CUtensorMap)))
    return fail(MONOFAB_EINVAL, "fabric_tensor_map_packed: not a map record of this fabric");
  const unsigned int flag = packed != 0;
  return to_device(f, reinterpret_cast<CUtensorMap*>(handle) + 3, &flag, 4);
}

}  // extern "C"
