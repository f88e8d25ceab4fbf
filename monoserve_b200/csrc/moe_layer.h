// The host-side record of one MoE layer and the helpers its entry points share
// (api.cu owns the definitions; ep_exchange.cu builds the expert-parallel layer on them).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <vector>

#include "../../include/monofab.h"
#include "kernels.h"

namespace mf {

int fail(int code, const char* fmt, ...);   // records the message for monofab_last_error

#define MF_CUDA(expr)                                                                          \
  do {                                                                                         \
    cudaError_t e_ = (expr);                                                                   \
    if (e_ != cudaSuccess) return mf::fail(MONOFAB_ECUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

constexpr int kNumTimes = 6;

}  // namespace mf

struct monofab_moe {
  monofab_moe_config cfg{};
  std::mutex mu;
  int device = 0, num_sms = 0;
  int ctas = 0, credits = 8, form = 64;
  // weights
  const void* router_w = nullptr;
  const float* router_bias = nullptr;
  const void* w13[2] = {nullptr, nullptr};   // device-visible addresses per region
  const void* w2[2] = {nullptr, nullptr};
  int slots[2] = {0, 0};
  int packed[2] = {0, 0};                    // w13 of the region is in the packed SwiGLU row order
  bool trace_on = false;
  const float* s13 = nullptr;
  const float* s2 = nullptr;
  // workspaces (device)
  float* logits = nullptr;
  int* topk_ids = nullptr;
  float* topk_w = nullptr;
  int* counts = nullptr;
  int* starts = nullptr;
  int* chunk_counts = nullptr;
  int* pair_rank = nullptr;
  int* pair_token = nullptr;
  float* pair_weight = nullptr;
  int* pair_pos = nullptr;
  int* table = nullptr;
  int* hist = nullptr;
  void* xp = nullptr;
  void* h = nullptr;
  float* y = nullptr;
  void* xin = nullptr;    // staging of the host-buffer entry point
  void* x2in = nullptr;
  void* xout = nullptr;
  mf::GemmTile* tiles[2] = {nullptr, nullptr};
  mf::GemmQueues* queues = nullptr;
  int* done = nullptr;
  unsigned long long* trace = nullptr;
  int block_cap = 0;
  int* status = nullptr;
  int* status_host = nullptr;
  int tile_cap = 0;
  size_t pairs_cap = 0;
  bool maps_dirty = true;
  mf::GemmParams gp{};
  bool profile = false;
  cudaEvent_t ev[mf::kNumTimes + 1] = {};
  float times[mf::kNumTimes] = {};
  bool times_valid = false;
  std::vector<void*> owned;
};

namespace mf {

int build_maps(monofab_moe* m);
// Plan + grouped GEMM over caller-described segments of the layer's packed rows.  `seg` gives
// seg_counts / seg_expert / E (= segments) and the optional stride and peer flags; the layer fills in
// the rest.  after_plan, if set, is recorded between the two launches.
int experts_locked(monofab_moe* m, const PlanParams& seg, cudaStream_t st, cudaEvent_t after_plan);

}  // namespace mf
