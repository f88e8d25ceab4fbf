// monofab_pack_pairs_static: the stable pack for callers that must not allocate.
//
// Some users of this library cannot call cudaMalloc at the point where they
// need to pack: a serving process that has a persistent kernel resident on the
// device (cudaMalloc and cudaFree synchronise the whole device and so wait for
// a kernel that never ends), a component that was handed a fixed memory budget
// at start-up and owns no allocator, or code that runs on a latency path where
// an allocation's implicit synchronisation is not acceptable.  For them this
// entry point keeps the pack's scratch (per-chunk expert counts and per-pair
// ranks) in one fixed array that is part of the library image: every GPU that
// loads libmonofab holds kPackStaticBytes of it until the process exits.
//
// The price is a size limit and sharing: T <= kPackStaticMaxTokens, and all
// calls on one device use the same array, so two calls whose kernels overlap on
// the GPU (different streams, or different host threads) race.  Serialise them
// on one stream.  The array keeps the previous call's contents; the pack
// overwrites every cell it later reads, so nothing needs clearing.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "../../include/monofab.h"
#include "kernels.h"

namespace mf {

int fail(int code, const char* fmt, ...);   // api.cu: records the message for monofab_last_error

constexpr int kPackStaticMaxTokens = MONOFAB_PACK_STATIC_MAX_TOKENS;
constexpr size_t kPackStaticBytes =
    (static_cast<size_t>(kPackStaticMaxTokens) / kChunkTokens) * kMaxExperts * sizeof(int) +   // chunk counts
    static_cast<size_t>(kPackStaticMaxTokens) * kMaxTopK * sizeof(int);                        // pair ranks

// In host code this name is only a handle for the runtime's symbol table, not a
// device address; the address is looked up once per device below.
static __device__ __align__(256) unsigned char g_pack_scratch[kPackStaticBytes];

constexpr int kMaxDevices = 64;
static std::mutex g_setup_mu;
static void* g_scratch_addr[kMaxDevices] = {};

// Device address of the scratch array on the CURRENT device (looked up on the
// first call per device; that call must not happen inside a stream capture).
static int scratch_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(MONOFAB_ECUDA, "pack_pairs_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(MONOFAB_EINVAL, "pack_pairs_static: device index %d not supported", dev);
  std::lock_guard<std::mutex> lock(g_setup_mu);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_pack_scratch);
    if (e != cudaSuccess || !p)
      return fail(MONOFAB_ECUDA, "pack_pairs_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return MONOFAB_OK;
}

}  // namespace mf

using namespace mf;

extern "C" int monofab_pack_pairs_static(const int32_t* topk_ids, const float* topk_w, int T, int E, int K, int H,
                                         const void* src, void* dst, int32_t* counts, int32_t* starts,
                                         int32_t* pair_token, float* pair_weight, int32_t* pair_pos, void* stream) {
  if (!counts || !starts || (T > 0 && (!topk_ids || !topk_w || !pair_token || !pair_weight || !pair_pos)))
    return fail(MONOFAB_EINVAL, "pack_pairs_static: NULL argument");
  if (E < 1 || E > kMaxExperts) return fail(MONOFAB_EINVAL, "pack_pairs_static: E=%d outside [1, %d]", E, kMaxExperts);
  if (K < 1 || K > kMaxTopK) return fail(MONOFAB_EINVAL, "pack_pairs_static: K=%d outside [1, %d]", K, kMaxTopK);
  if (T < 0) return fail(MONOFAB_EINVAL, "pack_pairs_static: negative T");
  if (T > kPackStaticMaxTokens)
    return fail(MONOFAB_EINVAL, "pack_pairs_static: T=%d exceeds the built-in scratch (at most %d tokens); "
                "use monofab_pack_pairs with caller-provided scratch", T, kPackStaticMaxTokens);
  if ((src == nullptr) != (dst == nullptr)) return fail(MONOFAB_EINVAL, "pack_pairs_static: src and dst go together");
  if (src && (H <= 0 || H % 8)) return fail(MONOFAB_EINVAL, "pack_pairs_static: H=%d must be a positive multiple of 8", H);
  if (pack_scratch_bytes(T, E, K) > kPackStaticBytes)
    return fail(MONOFAB_EINVAL, "pack_pairs_static: internal scratch too small");
  void* scratch = nullptr;
  if (int r = scratch_address(&scratch)) return r;
  const cudaError_t e = launch_pack_chain(topk_ids, topk_w, T, E, K, H, static_cast<const bf16*>(src),
                                          static_cast<bf16*>(dst), counts, starts, pair_token, pair_weight, pair_pos,
                                          scratch, nullptr, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(MONOFAB_ECUDA, "pack_pairs_static: launch: %s", cudaGetErrorString(e));
  return MONOFAB_OK;
}
