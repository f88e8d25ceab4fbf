// Expert parallelism for one MoE layer over peer memory: the experts are partitioned
// over the GPUs of one node, and token dispatch / return are done by this library's own
// kernels, which store rows straight into the destination GPU's buffers over NVLink and
// raise a flag there.  No collective library call and no host round trip sits on the
// per-layer path: split sizes never reach the host.
//
// The reference has no collective of its own (its only multi-GPU mode is stock vLLM
// expert parallelism, monoserve/baselines/serve_ep.py:24-28), so there is no reference
// kernel for this file; the per-layer stage chain it distributes is the one of
// monoserve/runtime/lane.py:340-380.
//
// Rank r owns experts [r * E/N, (r + 1) * E/N).  Routing, packing and combining are
// data-parallel over a rank's own tokens.  Per layer pass and rank (all on one stream):
//
//   router_logits, router_topk   local routing over all E experts (bit-exact, as on one GPU)
//   ep_counts_kernel             per-expert counts and exclusive starts of the local pairs;
//                                both are stored into EVERY rank's table, then flag "counts"
//   ep_dispatch_kernel           waits for all ranks' counts; every rank can now compute every
//                                destination's layout: the packed rows of destination d are
//                                ordered (local expert, source rank, source's packed order), so an
//                                expert's rows from all sources form ONE segment and share its
//                                weight tiles.  Copies each pair's activation row from xn straight
//                                into xp[dest row] of the owning rank, then flag "rows"
//   plan_kernel + expert GEMM    wait for all sources' "rows" flags, then the local grouped
//                                SwiGLU FFN over E/N segments (rows = the counts table summed over sources)
//   ep_return_kernel             pushes every fp32 output row into y_back[pos] of the rank it
//                                came from (pos = the pair's place in that rank's own packed
//                                order), then flag "y"
//   combine_kernel               waits for all "y" flags; weighted sum in pick order, as on one GPU
//
// Flags carry the pass number and only grow.  Buffer reuse needs no barrier between passes: a rank
// starts pass n + 1 only after its combine of pass n has seen every peer's "y" flag, which a peer
// raises after its GEMM of pass n has finished reading xp, and the counts table is double-buffered
// by pass parity.  Only plain peer loads and stores are used: no multicast, no TMA on peer memory.
// Every wait is bounded (peer_sync.cuh) and every remote index is range-checked, so a rank that
// never arrives shows up as MONOFAB_STATUS_WAIT_TIMEOUT in the status word, not as a hang or a fault.
#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <cstring>

#include "moe_layer.h"
#include "peer_sync.cuh"
#include "release.h"

namespace mf {

constexpr int kMaxRanks = MONOFAB_EP_MAX_RANKS;
constexpr int kFlagCounts = 0, kFlagRows = 1, kFlagY = 2;
// Layout of a rank's communication buffer (peer-visible):
//   [0, 4 KB)        flags: u32 [3 kinds][32]; word [kind][src] is written by rank src only
//   [4 KB, 68 KB)    tables: int32 [2 parities][2 (counts, starts)][kMaxRanks][kMaxExperts]
//   [128 KB, ...)    y_back: fp32 [max_tokens * K][H], filled by the peers' return kernels
constexpr size_t kCommTables = 4096;
constexpr size_t kCommYBack = 128 * 1024;
static_assert(kCommTables + 2 * 2 * kMaxRanks * kMaxExperts * sizeof(int) <= kCommYBack, "tables overlap y_back");

__host__ __device__ inline unsigned int* comm_flag(unsigned char* comm, int kind, int src) {
  return reinterpret_cast<unsigned int*>(comm) + kind * 32 + src;
}
// which = 0: counts[src][e]; 1: exclusive starts[src][e] of rank src's packed order
__host__ __device__ inline int* comm_table(unsigned char* comm, unsigned int epoch, int which) {
  return reinterpret_cast<int*>(comm + kCommTables) + ((epoch & 1u) * 2 + which) * kMaxRanks * kMaxExperts;
}
__host__ __device__ inline float* comm_yback(unsigned char* comm) { return reinterpret_cast<float*>(comm + kCommYBack); }

struct EpDev {
  int rank, world, E, El, K, H, T;
  unsigned int epoch;
  int rows_cap;    // rows a rank's packed-row buffer takes
  int pairs_cap;   // rows of a rank's y_back
  int* status;
  int* block_counter;   // [2]: dispatch, return
  unsigned char* comm[kMaxRanks];
  bf16* xp[kMaxRanks];
};

}  // namespace mf

// First row, in the packed-row buffer of the rank that owns expert e, of the rows that rank `src`
// sends for e: every rank's rows of the owner's lower experts, then the lower ranks' rows of e.
// counts_all is int32 [world][stride].  The dispatch kernel computes the same through shared memory.
extern "C" int monofab_ep_dest_base(const int32_t* counts_all, int stride, int world, int experts, int src, int e) {
  const int El = experts / world, lo = (e / El) * El;
  int base = 0;
  for (int x = lo; x < e; ++x)
    for (int s = 0; s < world; ++s) base += counts_all[s * stride + x];
  for (int s = 0; s < src; ++s) base += counts_all[s * stride + e];
  return base;
}

namespace mf {

// ------------------------------------------------------------------ counts
// One block.  counts[e] = sum of the chunk counts, starts = exclusive scan, chunk counts become
// exclusive prefixes over chunks (as the scan-only plan kernel); then both rows go to every rank.
__global__ void __launch_bounds__(256) ep_counts_kernel(const EpDev A, int* __restrict__ chunk_counts, int chunks,
                                                        int* __restrict__ counts, int* __restrict__ starts) {
  __shared__ int s_warp[8];
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
  int cnt = 0;
  chain_release();
  chain_wait();
  if (e < A.E) {
    for (int c = 0; c < chunks; ++c) {
      int* cell = chunk_counts + static_cast<size_t>(c) * A.E + e;
      const int v = *cell;
      *cell = cnt;
      cnt += v;
    }
    counts[e] = cnt;
  }
  int incl = cnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += y;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  int base = 0, total = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    const int s = s_warp[w];
    if (w < warp) base += s;
    total += s;
  }
  const int start = base + incl - cnt;
  if (e < A.E) starts[e] = start;
  if (e == 0) starts[A.E] = total;
  if (e < A.E) {
    for (int d = 0; d < A.world; ++d) {
      comm_table(A.comm[d], A.epoch, 0)[A.rank * kMaxExperts + e] = cnt;
      comm_table(A.comm[d], A.epoch, 1)[A.rank * kMaxExperts + e] = start;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (e < A.world) st_release_sys(comm_flag(A.comm[e], kFlagCounts, A.rank), A.epoch);
}

// Last block of a grid raises flag `kind` at every rank (after every block's stores are visible).
__device__ __forceinline__ void signal_all_when_grid_done(const EpDev& A, int counter, int kind) {
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(A.block_counter + counter, 1);
    s_last = prev == static_cast<int>(gridDim.x) - 1;
    if (s_last) A.block_counter[counter] = 0;
  }
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (static_cast<int>(threadIdx.x) < A.world) st_release_sys(comm_flag(A.comm[threadIdx.x], kind, A.rank), A.epoch);
  }
}

// ---------------------------------------------------------------- dispatch
constexpr int kRowSplit = 4;   // warps that share one row's columns

__global__ void __launch_bounds__(256) ep_dispatch_kernel(const EpDev A, const int* __restrict__ topk_ids,
                                                          const int* __restrict__ pair_rank,
                                                          const int* __restrict__ chunk_prefix,
                                                          const int* __restrict__ starts, const bf16* __restrict__ xn,
                                                          int* __restrict__ pair_pos) {
  __shared__ int s_total[kMaxExperts], s_base[kMaxExperts];
  const int tid = threadIdx.x, lane = tid & 31;
  unsigned char* mine = A.comm[A.rank];
  chain_release();
  chain_wait();
  if (tid < A.world && !wait_flag(comm_flag(mine, kFlagCounts, tid), A.epoch)) atomicOr(A.status, kErrWaitTimeout);
  __syncthreads();
  const int* call = comm_table(mine, A.epoch, 0);
  int below = 0;   // rows of expert `tid` that lower ranks send
  if (tid < A.E) {
    int total = 0;
    for (int s = 0; s < A.world; ++s) {
      const int c = call[s * kMaxExperts + tid];
      if (s < A.rank) below += c;
      total += c;
    }
    s_total[tid] = total;
  }
  __syncthreads();
  if (tid < A.E) {
    int base = below;
    for (int x = (tid / A.El) * A.El; x < tid; ++x) base += s_total[x];
    s_base[tid] = base;
  }
  if (blockIdx.x == 0 && tid < A.world) {   // rows that rank `tid` receives in total
    int total = 0;
    for (int j = 0; j < A.El; ++j) total += s_total[tid * A.El + j];
    if (total > A.rows_cap) atomicOr(A.status, kErrPlanOverflow);
  }
  __syncthreads();
  const int unit = blockIdx.x * (blockDim.x >> 5) + (tid >> 5);
  const int t = unit / kRowSplit, part = unit - t * kRowSplit;
  if (t < A.T) {
    const int K = A.K, E = A.E;
    int dst_rank = -1, dst_row = 0;
    if (lane < K) {
      const int e = topk_ids[static_cast<size_t>(t) * K + lane];
      const int within = chunk_prefix[static_cast<size_t>(t / kChunkTokens) * E + e] + pair_rank[static_cast<size_t>(t) * K + lane];
      dst_row = s_base[e] + within;
      if (dst_row >= 0 && dst_row < A.rows_cap) dst_rank = e / A.El;   // rows beyond the capacity are not sent
      if (part == 0) pair_pos[static_cast<size_t>(t) * K + lane] = starts[e] + within;
    }
    const int n16 = A.H / 8;
    const int c_begin = part * n16 / kRowSplit, c_end = (part + 1) * n16 / kRowSplit;
    const uint4* src = reinterpret_cast<const uint4*>(xn + static_cast<size_t>(t) * A.H);
    // The column loop has the same trip count in every lane (the shuffles below need the whole warp);
    // a lane past the end of its part only skips the load and the stores.
    for (int c0 = c_begin; c0 < c_end; c0 += 32) {
      const int c = c0 + lane;
      const bool on = c < c_end;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (on) v = src[c];
      for (int k = 0; k < K; ++k) {
        const int dk = __shfl_sync(0xffffffffu, dst_rank, k);
        const int rk = __shfl_sync(0xffffffffu, dst_row, k);
        if (on && dk >= 0) reinterpret_cast<uint4*>(A.xp[dk] + static_cast<size_t>(rk) * A.H)[c] = v;
      }
    }
  }
  signal_all_when_grid_done(A, 0, kFlagRows);
}

// ------------------------------------------------------------------ return
// seg_starts: the local plan's exclusive row offsets of the El local experts.
__global__ void __launch_bounds__(256) ep_return_kernel(const EpDev A, const int* __restrict__ seg_starts,
                                                        const float* __restrict__ y) {
  __shared__ int s_start[kMaxExperts + 1], s_cnt[kMaxExperts], s_src0[kMaxExperts];   // [source][local expert]
  const int tid = threadIdx.x, lane = tid & 31;
  const int El = A.El;
  chain_release();
  chain_wait();
  const int* counts_all = comm_table(A.comm[A.rank], A.epoch, 0);
  const int* starts_all = comm_table(A.comm[A.rank], A.epoch, 1);
  for (int i = tid; i <= El; i += blockDim.x) s_start[i] = seg_starts[i];
  for (int i = tid; i < A.world * El; i += blockDim.x) {
    const int at = (i / El) * kMaxExperts + A.rank * El + i % El;
    s_cnt[i] = counts_all[at];
    s_src0[i] = starts_all[at];
  }
  __syncthreads();
  const int rows = min(s_start[El], A.rows_cap);
  const int n4 = A.H / 4;
  const int warps = gridDim.x * (blockDim.x >> 5);
  for (int unit = blockIdx.x * (blockDim.x >> 5) + (tid >> 5); unit < rows * kRowSplit; unit += warps) {
    const int r = unit / kRowSplit, part = unit - r * kRowSplit;
    int lo = 0, hi = El;   // the expert holding row r: the last segment that starts at or before r
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_start[mid] <= r) lo = mid; else hi = mid;
    }
    int i = r - s_start[lo], src = 0;   // then the source rank inside the expert's segment
    while (src < A.world - 1 && i >= s_cnt[src * El + lo]) i -= s_cnt[src * El + lo], ++src;
    const int pos = s_src0[src * El + lo] + i;
    if (i < 0 || i >= s_cnt[src * El + lo] || pos < 0 || pos >= A.pairs_cap) continue;
    const float4* from = reinterpret_cast<const float4*>(y + static_cast<size_t>(r) * A.H);
    float4* to = reinterpret_cast<float4*>(comm_yback(A.comm[src]) + static_cast<size_t>(pos) * A.H);
    const int c_begin = part * n4 / kRowSplit, c_end = (part + 1) * n4 / kRowSplit;
    for (int c = c_begin + lane; c < c_end; c += 32) to[c] = __ldcs(from + c);
  }
  signal_all_when_grid_done(A, 1, kFlagY);
}

// A rank without tokens still has to see every peer's "y" flag before its next pass may write rows.
__global__ void ep_wait_kernel(const unsigned int* flags, unsigned int epoch, int n, int* status) {
  if (static_cast<int>(threadIdx.x) < n && !wait_flag(flags + threadIdx.x, epoch)) atomicOr(status, kErrWaitTimeout);
}

typedef CUresult (*AddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

static AddressRangeFn address_range_fn() {
  static AddressRangeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
    return reinterpret_cast<AddressRangeFn>(p);
  }();
  return fn;
}

// What one rank tells the others about its buffers (MONOFAB_EP_HANDLE_BYTES bytes).
struct EpHandle {
  uint64_t pid;
  int32_t device, rank;
  uint64_t comm_ptr, xp_ptr;       // addresses in the owner's process
  uint64_t comm_off, xp_off;       // offsets from the base of their allocations
  cudaIpcMemHandle_t comm_ipc, xp_ipc;
  unsigned char pad[MONOFAB_EP_HANDLE_BYTES - 48 - 2 * sizeof(cudaIpcMemHandle_t)];
};
static_assert(sizeof(EpHandle) == MONOFAB_EP_HANDLE_BYTES, "EpHandle size");

constexpr int kEpTimes = 8;

}  // namespace mf

using namespace mf;

struct monofab_ep {
  monofab_moe_config cfg{};   // the global layer: E experts, top-K, max_tokens per rank
  int rank = 0, world = 1, El = 0, rows_cap = 0, device = 0;
  monofab_moe* local = nullptr;
  std::mutex mu;
  const void* router_w = nullptr;
  const float* router_bias = nullptr;
  unsigned char* comm = nullptr;
  size_t comm_bytes = 0;
  float* logits = nullptr;
  int *topk_ids = nullptr, *counts = nullptr, *starts = nullptr, *chunk_counts = nullptr, *pair_rank = nullptr,
      *pair_pos = nullptr, *block_counter = nullptr;
  float* topk_w = nullptr;
  unsigned int epoch = 0;
  bool connected = false;
  unsigned char* peer_comm[kMaxRanks] = {};
  bf16* peer_xp[kMaxRanks] = {};
  void* ipc_open[2 * kMaxRanks] = {};   // bases returned by cudaIpcOpenMemHandle, to close
  int n_ipc = 0;
  bool profile = false, times_valid = false;
  cudaEvent_t ev[kEpTimes + 1] = {};
  std::vector<void*> owned;
};

namespace {

int ep_alloc(monofab_ep* ep, void** p, size_t bytes) {
  MF_CUDA(cudaMalloc(p, bytes ? bytes : 16));
  MF_CUDA(cudaMemset(*p, 0, bytes ? bytes : 16));
  ep->owned.push_back(*p);
  return MONOFAB_OK;
}

EpDev device_params(monofab_ep* ep, int T) {
  EpDev A{};
  A.rank = ep->rank;
  A.world = ep->world;
  A.E = ep->cfg.experts;
  A.El = ep->El;
  A.K = ep->cfg.top_k;
  A.H = ep->cfg.hidden;
  A.T = T;
  A.epoch = ep->epoch;
  A.rows_cap = ep->rows_cap;
  A.pairs_cap = ep->cfg.max_tokens * ep->cfg.top_k;
  A.status = ep->local->status;
  A.block_counter = ep->block_counter;
  for (int r = 0; r < ep->world; ++r) {
    A.comm[r] = ep->peer_comm[r];
    A.xp[r] = ep->peer_xp[r];
  }
  return A;
}

// The four phases of a pass.  A rank runs them back to back on one stream; a test that stands
// several ranks on ONE GPU runs phase p of every rank before phase p + 1 of any, so that no kernel
// ever waits for a kernel that has not been launched before it on the same stream.
int phase_locked(monofab_ep* ep, int phase, const void* xn, const void* x2, void* out, int T, cudaStream_t st) {
  const monofab_moe_config& c = ep->cfg;
  monofab_moe* m = ep->local;
  const int H = c.hidden, E = c.experts, K = c.top_k;
  const int chunks = (T + kChunkTokens - 1) / kChunkTokens;
  const bool prof = ep->profile;
  auto mark = [&](int i) -> cudaError_t { return prof ? cudaEventRecord(ep->ev[i], st) : cudaSuccess; };
  const EpDev A = device_params(ep, T);
  switch (phase) {
    case 0: {
      MF_CUDA(mark(0));
      MF_CUDA(launch_router_logits(xn, ep->router_w, ep->logits, T, H, E, st));
      MF_CUDA(mark(1));
      RouterParams rp{ep->logits, ep->router_bias, ep->topk_ids, ep->topk_w, nullptr, ep->chunk_counts, ep->pair_rank,
                      T, E, K, c.scoring, c.renorm, c.routed_scale, 0};
      MF_CUDA(launch_router_topk(rp, st));
      MF_CUDA(mark(2));
      MF_CUDA(launch_chained(ep_counts_kernel, 1, 256, 0, st, A, ep->chunk_counts, chunks, ep->counts, ep->starts));
      MF_CUDA(mark(3));
      return MONOFAB_OK;
    }
    case 1: {
      const int units = T * kRowSplit;
      const int blocks = units > 0 ? (units + 7) / 8 : 1;
      MF_CUDA(launch_chained(ep_dispatch_kernel, blocks, 256, 0, st, A, ep->topk_ids, ep->pair_rank, ep->chunk_counts,
                             ep->starts, static_cast<const bf16*>(xn), ep->pair_pos));
      MF_CUDA(mark(4));
      return MONOFAB_OK;
    }
    case 2: {
      PlanParams seg{};
      seg.seg_counts = comm_table(ep->comm, ep->epoch, 0) + ep->rank * ep->El;
      seg.seg_tables = ep->world;
      seg.seg_stride = kMaxExperts;
      seg.E = ep->El;
      seg.wait_flags = comm_flag(ep->comm, kFlagRows, 0);
      seg.wait_epoch = ep->epoch;
      seg.wait_n = ep->world;
      {
        std::lock_guard<std::mutex> lock(m->mu);
        if (int r = experts_locked(m, seg, st, prof ? ep->ev[5] : nullptr)) return r;
      }
      MF_CUDA(mark(6));
      MF_CUDA(launch_chained(ep_return_kernel, 2 * m->num_sms, 256, 0, st, A, m->starts, m->y));
      MF_CUDA(mark(7));
      return MONOFAB_OK;
    }
    case 3: {
      CombineParams cp{};
      cp.y = comm_yback(ep->comm);
      cp.pair_pos = ep->pair_pos;
      cp.topk_w = ep->topk_w;
      cp.x2 = static_cast<const bf16*>(x2);
      cp.x = static_cast<bf16*>(out);
      cp.T = T;
      cp.K = K;
      cp.H = H;
      cp.y_rows = c.max_tokens * K;
      cp.wait_flags = comm_flag(ep->comm, kFlagY, 0);
      cp.wait_epoch = ep->epoch;
      cp.wait_n = ep->world;
      cp.status = m->status;
      if (T == 0) {
        ep_wait_kernel<<<1, 32, 0, st>>>(cp.wait_flags, cp.wait_epoch, cp.wait_n, cp.status);
        MF_CUDA(cudaGetLastError());
      } else {
        MF_CUDA(launch_combine(cp, st));
      }
      MF_CUDA(mark(8));
      ep->times_valid = prof;
      return MONOFAB_OK;
    }
  }
  return fail(MONOFAB_EINVAL, "ep_phase: phase %d outside 0..3", phase);
}

int check_pass_args(monofab_ep* ep, const void* xn, void* out, int T) {
  if (!ep->connected) return fail(MONOFAB_EINVAL, "ep: not connected (monofab_ep_connect)");
  if (T < 0 || T > ep->cfg.max_tokens) return fail(MONOFAB_EINVAL, "ep: T=%d outside [0, max_tokens=%d]", T, ep->cfg.max_tokens);
  if (T > 0 && (!xn || !out)) return fail(MONOFAB_EINVAL, "ep: xn and out must not be NULL");
  if (!ep->router_w) return fail(MONOFAB_EINVAL, "ep: router weight not set (monofab_ep_set_router)");
  return MONOFAB_OK;
}

}  // namespace

extern "C" {

int monofab_ep_create(const monofab_moe_config* cfg, int rank, int world, int rows_cap, monofab_ep** out) {
  if (!cfg || !out) return fail(MONOFAB_EINVAL, "ep_create: NULL argument");
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return fail(MONOFAB_EINVAL, "ep_create: rank %d of %d (at most %d ranks)", rank, world, kMaxRanks);
  if (cfg->experts < 1 || cfg->experts > kMaxExperts || cfg->experts % world)
    return fail(MONOFAB_EINVAL, "ep_create: %d experts do not divide evenly over %d ranks", cfg->experts, world);
  if (cfg->top_k < 1 || cfg->top_k > kMaxTopK || cfg->top_k > cfg->experts || cfg->max_tokens < 1)
    return fail(MONOFAB_EINVAL, "ep_create: bad top_k=%d or max_tokens=%d", cfg->top_k, cfg->max_tokens);
  const long long worst = static_cast<long long>(cfg->max_tokens) * cfg->top_k * world;
  if (rows_cap <= 0) rows_cap = static_cast<int>(worst);   // every pair of every rank may land on one rank
  if (rows_cap > worst) rows_cap = static_cast<int>(worst);
  monofab_ep* ep = new monofab_ep();
  ep->cfg = *cfg;
  ep->rank = rank;
  ep->world = world;
  ep->El = cfg->experts / world;
  ep->rows_cap = rows_cap;
  int r = 0;
  if (cudaGetDevice(&ep->device) != cudaSuccess) r = fail(MONOFAB_ECUDA, "ep_create: cudaGetDevice failed");
  monofab_moe_config lc = *cfg;   // the local layer: this rank's experts, one pick per received row
  lc.experts = ep->El;
  lc.top_k = 1;
  lc.max_tokens = rows_cap;
  if (!r) r = monofab_moe_create(&lc, &ep->local);
  const size_t T = cfg->max_tokens, E = cfg->experts, K = cfg->top_k, H = cfg->hidden, P = T * K;
  const size_t chunks = (T + kChunkTokens - 1) / kChunkTokens;
  ep->comm_bytes = kCommYBack + P * H * sizeof(float);
  auto A = [&](auto** p, size_t bytes) { if (!r) r = ep_alloc(ep, reinterpret_cast<void**>(p), bytes); };
  A(&ep->comm, ep->comm_bytes);
  A(&ep->logits, T * E * 4);
  A(&ep->topk_ids, P * 4);
  A(&ep->topk_w, P * 4);
  A(&ep->counts, kMaxExperts * 4);
  A(&ep->starts, (kMaxExperts + 1) * 4);
  A(&ep->chunk_counts, chunks * E * 4);
  A(&ep->pair_rank, P * 4);
  A(&ep->pair_pos, P * 4);
  A(&ep->block_counter, 16);
  for (int i = 0; !r && i <= kEpTimes; ++i)
    if (cudaEventCreate(&ep->ev[i]) != cudaSuccess) r = fail(MONOFAB_ECUDA, "ep_create: cudaEventCreate failed");
  if (r) {
    monofab_ep_destroy(ep);
    return r;
  }
  *out = ep;
  return MONOFAB_OK;
}

monofab_moe* monofab_ep_local(monofab_ep* ep) { return ep ? ep->local : nullptr; }

int monofab_ep_export(monofab_ep* ep, void* handle) {
  if (!ep || !handle) return fail(MONOFAB_EINVAL, "ep_export: NULL argument");
  EpHandle h;
  std::memset(&h, 0, sizeof h);
  h.pid = static_cast<uint64_t>(getpid());
  h.device = ep->device;
  h.rank = ep->rank;
  h.comm_ptr = reinterpret_cast<uint64_t>(ep->comm);
  h.xp_ptr = reinterpret_cast<uint64_t>(ep->local->xp);
  AddressRangeFn range = address_range_fn();
  if (!range) return fail(MONOFAB_ECUDA, "ep_export: cuMemGetAddressRange is not available from this driver");
  CUdeviceptr base = 0;
  size_t size = 0;
  if (range(&base, &size, static_cast<CUdeviceptr>(h.comm_ptr)) != CUDA_SUCCESS) return fail(MONOFAB_ECUDA, "ep_export: address range of the communication buffer");
  h.comm_off = h.comm_ptr - base;
  MF_CUDA(cudaIpcGetMemHandle(&h.comm_ipc, reinterpret_cast<void*>(base)));
  if (range(&base, &size, static_cast<CUdeviceptr>(h.xp_ptr)) != CUDA_SUCCESS) return fail(MONOFAB_ECUDA, "ep_export: address range of the packed-row buffer");
  h.xp_off = h.xp_ptr - base;
  MF_CUDA(cudaIpcGetMemHandle(&h.xp_ipc, reinterpret_cast<void*>(base)));
  std::memcpy(handle, &h, sizeof h);
  return MONOFAB_OK;
}

int monofab_ep_connect(monofab_ep* ep, const void* handles) {
  if (!ep || !handles) return fail(MONOFAB_EINVAL, "ep_connect: NULL argument");
  std::lock_guard<std::mutex> lock(ep->mu);
  if (ep->connected) return fail(MONOFAB_EINVAL, "ep_connect: already connected");
  const EpHandle* hs = static_cast<const EpHandle*>(handles);
  const uint64_t me = static_cast<uint64_t>(getpid());
  for (int r = 0; r < ep->world; ++r) {
    EpHandle h;
    std::memcpy(&h, hs + r, sizeof h);
    if (h.rank != r) return fail(MONOFAB_EINVAL, "ep_connect: handle %d belongs to rank %d", r, h.rank);
    if (r == ep->rank) {
      ep->peer_comm[r] = ep->comm;
      ep->peer_xp[r] = static_cast<bf16*>(ep->local->xp);
    } else if (h.pid == me) {   // a rank of this process: its addresses are valid here
      if (h.device != ep->device) {
        int can = 0;
        MF_CUDA(cudaDeviceCanAccessPeer(&can, ep->device, h.device));
        if (!can) return fail(MONOFAB_ECUDA, "ep_connect: device %d cannot access device %d", ep->device, h.device);
        const cudaError_t e = cudaDeviceEnablePeerAccess(h.device, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
          return fail(MONOFAB_ECUDA, "ep_connect: cudaDeviceEnablePeerAccess: %s", cudaGetErrorString(e));
        cudaGetLastError();
      }
      ep->peer_comm[r] = reinterpret_cast<unsigned char*>(h.comm_ptr);
      ep->peer_xp[r] = reinterpret_cast<bf16*>(h.xp_ptr);
    } else {
      void *a = nullptr, *b = nullptr;
      MF_CUDA(cudaIpcOpenMemHandle(&a, h.comm_ipc, cudaIpcMemLazyEnablePeerAccess));
      ep->ipc_open[ep->n_ipc++] = a;
      MF_CUDA(cudaIpcOpenMemHandle(&b, h.xp_ipc, cudaIpcMemLazyEnablePeerAccess));
      ep->ipc_open[ep->n_ipc++] = b;
      ep->peer_comm[r] = static_cast<unsigned char*>(a) + h.comm_off;
      ep->peer_xp[r] = reinterpret_cast<bf16*>(static_cast<unsigned char*>(b) + h.xp_off);
    }
  }
  ep->connected = true;
  return MONOFAB_OK;
}

int monofab_ep_disconnect(monofab_ep* ep) {
  if (!ep) return MONOFAB_OK;
  std::lock_guard<std::mutex> lock(ep->mu);
  if (ep->n_ipc && !fabrics_running(ep->device)) cudaDeviceSynchronize();
  for (int i = 0; i < ep->n_ipc; ++i) cudaIpcCloseMemHandle(ep->ipc_open[i]);
  ep->n_ipc = 0;
  ep->connected = false;
  return MONOFAB_OK;
}

int monofab_ep_destroy(monofab_ep* ep) {
  if (!ep) return MONOFAB_OK;
  monofab_ep_disconnect(ep);
  if (!fabrics_running(ep->device)) cudaDeviceSynchronize();
  for (void* p : ep->owned) release_device(ep->device, p);
  for (cudaEvent_t e : ep->ev) release_event(ep->device, e);
  if (ep->local) monofab_moe_destroy(ep->local);
  delete ep;
  return MONOFAB_OK;
}

int monofab_ep_set_router(monofab_ep* ep, const void* wr_bf16, const float* bias) {
  if (!ep || !wr_bf16) return fail(MONOFAB_EINVAL, "ep_set_router: NULL argument");
  std::lock_guard<std::mutex> lock(ep->mu);
  ep->router_w = wr_bf16;
  ep->router_bias = bias;
  return MONOFAB_OK;
}

int monofab_ep_forward(monofab_ep* ep, const void* xn, const void* x2, void* out, int T, void* stream) {
  if (!ep) return fail(MONOFAB_EINVAL, "ep_forward: NULL handle");
  std::lock_guard<std::mutex> lock(ep->mu);
  if (int r = check_pass_args(ep, xn, out, T)) return r;
  ++ep->epoch;
  for (int phase = 0; phase < 4; ++phase)
    if (int r = phase_locked(ep, phase, xn, x2, out, T, static_cast<cudaStream_t>(stream))) return r;
  return MONOFAB_OK;
}

int monofab_ep_phase(monofab_ep* ep, int phase, const void* xn, const void* x2, void* out, int T, void* stream) {
  if (!ep) return fail(MONOFAB_EINVAL, "ep_phase: NULL handle");
  std::lock_guard<std::mutex> lock(ep->mu);
  if (int r = check_pass_args(ep, xn, out, T)) return r;
  if (phase == 0) ++ep->epoch;
  return phase_locked(ep, phase, xn, x2, out, T, static_cast<cudaStream_t>(stream));
}

int monofab_ep_workspace(monofab_ep* ep, const char* name, void** ptr, size_t* bytes) {
  if (!ep || !name || !ptr || !bytes) return fail(MONOFAB_EINVAL, "ep_workspace: NULL argument");
  const size_t P = static_cast<size_t>(ep->cfg.max_tokens) * ep->cfg.top_k, E = ep->cfg.experts;
  struct Entry { const char* name; void* p; size_t bytes; };
  const Entry entries[] = {
      {"logits", ep->logits, static_cast<size_t>(ep->cfg.max_tokens) * E * 4},
      {"topk_ids", ep->topk_ids, P * 4}, {"topk_w", ep->topk_w, P * 4}, {"pair_pos", ep->pair_pos, P * 4},
      {"counts", ep->counts, E * 4},     {"starts", ep->starts, (E + 1) * 4},
      {"y_back", comm_yback(ep->comm), P * ep->cfg.hidden * 4},
  };
  for (const Entry& e : entries)
    if (!std::strcmp(e.name, name)) {
      *ptr = e.p;
      *bytes = e.bytes;
      return MONOFAB_OK;
    }
  return fail(MONOFAB_EINVAL, "ep_workspace: unknown name '%s'", name);
}

int monofab_ep_set_profile(monofab_ep* ep, int on) {
  if (!ep) return fail(MONOFAB_EINVAL, "ep_set_profile: NULL handle");
  std::lock_guard<std::mutex> lock(ep->mu);
  ep->profile = on != 0;
  ep->times_valid = false;
  return MONOFAB_OK;
}

int monofab_ep_last_times(monofab_ep* ep, float ms[8]) {
  if (!ep || !ms) return fail(MONOFAB_EINVAL, "ep_last_times: NULL argument");
  std::lock_guard<std::mutex> lock(ep->mu);
  if (!ep->times_valid) return fail(MONOFAB_EINVAL, "ep_last_times: no profiled pass to report (monofab_ep_set_profile)");
  MF_CUDA(cudaEventSynchronize(ep->ev[kEpTimes]));
  for (int i = 0; i < kEpTimes; ++i) MF_CUDA(cudaEventElapsedTime(&ms[i], ep->ev[i], ep->ev[i + 1]));
  return MONOFAB_OK;
}

}  // extern "C"
