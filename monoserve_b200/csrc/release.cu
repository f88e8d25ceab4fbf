// The deferred-release registry (see release.h) and its diagnostics entry point.
#include "release.h"

#include <mutex>
#include <vector>

#include "../../include/monofab.h"

namespace mf {

namespace {

constexpr int kDevices = 64;
struct Pending {
  ReleaseKind kind;
  void* handle;
};
std::mutex g_mu;
int g_running[kDevices] = {};
std::vector<Pending> g_queue[kDevices];
unsigned long long g_probes_done = 0;   // kReleaseProbe entries carried out (diagnostics)

void carry_out(const Pending& p) {
  switch (p.kind) {
    case kReleaseDevice: cudaFree(p.handle); break;
    case kReleaseHost: cudaFreeHost(p.handle); break;
    case kReleaseStream: cudaStreamDestroy(static_cast<cudaStream_t>(p.handle)); break;
    case kReleaseEvent: cudaEventDestroy(static_cast<cudaEvent_t>(p.handle)); break;
    case kReleaseProbe: ++g_probes_done; break;
  }
}

bool valid(int device) { return device >= 0 && device < kDevices; }

}  // namespace

void fabric_started(int device) {
  if (!valid(device)) return;
  std::lock_guard<std::mutex> lock(g_mu);
  ++g_running[device];
}

void fabric_stopped(int device) {
  if (!valid(device)) return;
  std::vector<Pending> todo;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_running[device] > 0) --g_running[device];
    if (g_running[device] == 0) todo.swap(g_queue[device]);
  }
  if (todo.empty()) return;
  bool cuda = false;
  for (const Pending& p : todo) cuda |= p.kind != kReleaseProbe;
  if (cuda) {   // the owners could not wait for their own work when they queued these
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(device);
    cudaDeviceSynchronize();
    for (const Pending& p : todo) carry_out(p);
    if (prev >= 0) cudaSetDevice(prev);
  } else {
    for (const Pending& p : todo) carry_out(p);
  }
}

int fabrics_running(int device) {
  if (!valid(device)) return 0;
  std::lock_guard<std::mutex> lock(g_mu);
  return g_running[device];
}

bool release(int device, ReleaseKind kind, void* handle) {
  if (valid(device)) {
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_running[device] > 0) {
      g_queue[device].push_back(Pending{kind, handle});
      return true;
    }
  }
  carry_out(Pending{kind, handle});
  return false;
}

}  // namespace mf

extern "C" int monofab_release_debug(int op, int device, uint64_t* out) {
  using namespace mf;
  if (!valid(device)) return MONOFAB_EINVAL;
  switch (op) {
    case 0: fabric_started(device); break;                       // as if a fabric kernel had been launched
    case 1: fabric_stopped(device); break;                       // as if it had left
    case 2: release(device, kReleaseProbe, nullptr); break;      // a release that only counts itself
    case 3: {                                                    // out[0] = queued, out[1] = probes carried out, out[2] = running
      if (!out) return MONOFAB_EINVAL;
      std::lock_guard<std::mutex> lock(g_mu);
      out[0] = g_queue[device].size();
      out[1] = g_probes_done;
      out[2] = static_cast<uint64_t>(g_running[device]);
      break;
    }
    default: return MONOFAB_EINVAL;
  }
  return MONOFAB_OK;
}
