// Flag words between GPUs: one rank's kernel stores data into a peer's memory,
// then raises a flag there; the peer's kernel waits for the flag before it reads
// the data.  Flags only grow (the value is the step number), so nothing is ever
// reset and a late reader cannot miss one.  Every wait is bounded: after
// kPeerWaitNs of device time it gives up and the caller records the error in the
// layer's status word instead of hanging the GPU.
#pragma once
#include <cstdint>

namespace mf {

constexpr unsigned long long kPeerWaitNs = 2000000000ull;   // two seconds

__device__ __forceinline__ unsigned long long peer_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// True once *flag >= epoch (wrap-safe compare); false if the wait ran out.
__device__ __forceinline__ bool wait_flag(const unsigned int* flag, unsigned int epoch) {
  if (static_cast<int>(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const unsigned long long t0 = peer_timer_ns();
  unsigned int spins = 0;
  while (static_cast<int>(ld_acquire_sys(flag) - epoch) < 0) {
    if ((++spins & 63u) == 0) {
      if (peer_timer_ns() - t0 > kPeerWaitNs) return false;
      __nanosleep(100);
    }
  }
  return true;
}

}  // namespace mf
