// Releases that must not run beside a resident fabric kernel.
//
// cudaFree, cudaFreeHost and the destruction of streams synchronise the whole
// device, so while a persistent fabric kernel is resident they block the calling
// host thread until that kernel leaves (up to its run-time limit, or for ever
// without one).  The reference defers such frees until no fabric kernel runs on
// the device (csrc/host/fabric.cpp:20-59,150-158).  Here every release in the
// library goes through this registry: with no fabric running on the device it
// happens at once; otherwise it is queued and carried out when the last running
// fabric of that device has stopped.
#pragma once
#include <cuda_runtime.h>

namespace mf {

enum ReleaseKind { kReleaseDevice = 0, kReleaseHost = 1, kReleaseStream = 2, kReleaseEvent = 3, kReleaseProbe = 4 };

// Called by the fabric around its kernel's lifetime.  fabric_stopped drains the
// device's queue when the count of running fabrics reaches zero (the caller has
// already waited for its kernel).
void fabric_started(int device);
void fabric_stopped(int device);
int fabrics_running(int device);

// Release now, or queue if a fabric runs on `device`.  Returns true if queued.
bool release(int device, ReleaseKind kind, void* handle);
inline bool release_device(int device, void* p) { return p ? release(device, kReleaseDevice, p) : false; }
inline bool release_host(int device, void* p) { return p ? release(device, kReleaseHost, p) : false; }
inline bool release_stream(int device, cudaStream_t s) { return s ? release(device, kReleaseStream, s) : false; }
inline bool release_event(int device, cudaEvent_t e) { return e ? release(device, kReleaseEvent, e) : false; }

}  // namespace mf
