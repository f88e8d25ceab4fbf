// Parameter blocks and launchers of the layer's kernels, shared by the kernel
// files and the host entry points.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>

#include "types.h"

namespace mf {

using bf16 = __nv_bfloat16;

// Programmatic dependent launch: the kernels of one layer pass form a chain on one stream, each reading what
// the one before wrote.  Launched with launch_chained, a kernel may be scheduled while its predecessor is still
// draining: its blocks run their prologue (barrier set-up, TMEM allocation, operand-block loads that do not
// depend on the predecessor) and then stop in chain_wait() until the predecessor has completed and its writes
// are visible.  chain_release() lets the successor start being scheduled; it is called first thing, because
// every kernel here waits before it touches dependent data.  Without the launch attribute both are no-ops.
#if defined(__CUDACC__)
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <class... KArgs, class... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// A function attribute (dynamic shared memory above 48 KB) belongs to a device's context, so it is
// set once per DEVICE, not once per process: `configure` runs under a lock the first time the
// current device launches the kernel.
struct PerDeviceOnce {
  std::mutex mu;
  std::atomic<unsigned long long> done{0};
  template <class F>
  cudaError_t run(F configure) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    const unsigned long long bit = 1ull << (dev & 63);
    if (done.load(std::memory_order_acquire) & bit) return cudaSuccess;
    std::lock_guard<std::mutex> lock(mu);
    if (done.load(std::memory_order_relaxed) & bit) return cudaSuccess;
    err = configure();
    if (err == cudaSuccess) done.fetch_or(bit, std::memory_order_release);
    return err;
  }
};

struct RouterParams {
  float* logits;            // fp32 [T][E]; zeroed after reading when zero_logits is set
  const float* bias;        // fp32 [E] selection bias (sigmoid scoring) or null
  int* topk_ids;            // int32 [T][K]
  float* topk_w;            // fp32 [T][K]
  int* counts;              // int32 [E], accumulated with integer atomics, or null
  int* chunk_counts;        // int32 [chunks][E] pairs of each chunk per expert, or null
  int* pair_rank;           // int32 [T][K] stable rank inside (chunk, expert), or null
  int T, E, K;
  int scoring;              // 0 softmax, 1 sigmoid
  int renorm;
  float scale;
  int zero_logits;
};

struct PlanParams {
  const int* seg_counts;    // if set: rows per segment are given (no chunk sums); E is then the segment count
  const int* seg_expert;    // if set: expert id of every segment (table row, scale row); else identity
  int* chunk_counts;        // in: [chunks][E] counts; out: exclusive prefix over chunks per expert
  int* counts;              // out int32 [E]
  int* starts;              // out int32 [E + 1]
  const int* table;         // int32 [E][2] = (region, slot): region 0 host, 1 hot tier
  int* hist;                // int32 [E] activation histogram (+=), or null
  GemmTile* tiles[2];       // [0 = link, 1 = hbm]: w13 tiles, then w2 tiles; null q = scan only
  GemmQueues* q;
  int* done;                // int32 [block_cap] row-block counters (zeroed here)
  int* status;
  int chunks, E, H, I;
  int form;                 // row-block height of host-resident experts: 16..128; 0 = 256 (one pass up to 256 rows)
  int tile_cap;             // capacity of each tile list
  int block_cap;            // capacity of done[]
  int n_experts;            // rows of `table`: a segment's expert id must lie in [0, n_experts)
  int rows_cap;             // rows the packed-row buffers hold; a plan over more rows is refused
  // Segment counts may be the sum of several tables: segment s has
  // sum over i < seg_tables of seg_counts[i * seg_stride + s] rows (seg_tables 0 = one table).
  int seg_tables, seg_stride;
  // Peer flags to wait for before the counts are read (expert parallelism: every source rank's
  // rows have landed when wait_flags[0 .. wait_n) have reached wait_epoch); null = no wait.
  const unsigned int* wait_flags;
  unsigned int wait_epoch;
  int wait_n;
};

struct PackParams {
  const int* topk_ids;      // [T][K]
  const float* topk_w;      // [T][K]
  const int* pair_rank;     // [T][K]
  const int* chunk_prefix;  // [chunks][E]
  const int* starts;        // [E + 1]
  const bf16* src;          // [T][H]
  bf16* dst;                // [P][H]
  int* pair_token;          // [P]
  float* pair_weight;       // [P]
  int* pair_pos;            // [T][K] packed row of every (token, pick)
  int T, E, K, H;
  int* status;              // device error word: kErrBadArgs when an expert id lies outside [0, E); may be null
};

struct CombineParams {
  const float* y;           // fp32 [P][H] expert outputs of every pair
  const int* pair_pos;      // [T][K]
  const float* topk_w;      // [T][K]
  const bf16* x2;           // bf16 [T][H] residual, or null (treated as zero)
  bf16* x;                  // bf16 [T][H] out: bf16(x2 + moe)
  const bf16* norm_w;       // bf16 [H] weight of the following RMSNorm, or null
  bf16* normed;             // bf16 [T][H] out: rmsnorm(x) * norm_w (when norm_w is set)
  int T, K, H;
  float eps;
  int y_rows;               // rows of y: a pair_pos outside [0, y_rows) contributes nothing (0 = unchecked)
  // Peer flags to wait for before y is read (expert parallelism: every peer has returned its
  // rows when wait_flags[0 .. wait_n) have reached wait_epoch); null = no wait.
  const unsigned int* wait_flags;
  unsigned int wait_epoch;
  int wait_n;
  int* status;              // receives kErrWaitTimeout if the wait runs out
};

cudaError_t launch_router_logits(const void* x, const void* wr, float* logits, int T, int H, int E,
                                 cudaStream_t stream);
cudaError_t launch_router_topk(const RouterParams& A, cudaStream_t stream);
cudaError_t launch_chunk_rank(const int* topk_ids, int* pair_rank, int* chunk_counts, int T, int E, int K,
                              int* status, cudaStream_t stream);
cudaError_t launch_plan(const PlanParams& A, cudaStream_t stream);
cudaError_t launch_pack(const PackParams& A, cudaStream_t stream);
cudaError_t launch_combine(const CombineParams& A, cudaStream_t stream);
cudaError_t launch_expert_gemm(const GemmParams& p, int ctas, cudaStream_t stream);
cudaError_t launch_pack_w13(const void* src, void* dst, int n, int I, int H, int elt_bytes, cudaStream_t stream);

// Paged-KV attention (attention.cu).
struct AttnItem {
  int32_t req;        // row of the block table
  int32_t kv_head;
  int32_t q_row0;     // first query token (row of q / out)
  int32_t q_tokens;   // query tokens in this block (q_tokens * group <= 128)
  int32_t pos0;       // position of the first query token
  int32_t kv_len;     // keys visible to the request: positions 0 .. kv_len - 1
  int32_t key_begin;  // first key this item covers (a multiple of 128)
  int32_t key_end;    // one past the last key it covers; <= 0: no limit
  int32_t ws_row0;    // >= 0: the item is one part of a split and leaves fp32 rows there
  int32_t pad[3];
};
static_assert(sizeof(AttnItem) == 48, "AttnItem is twelve int32");

struct AttnParams {
  CUtensorMap q_map;    // dims (128, hq, T), box (64, group, tokens per block)
  CUtensorMap k_map;    // dims (64, 8, 2 hkv, page / 8, pages), box (64, 8, 2, page / 8, 1): see monofab_attention
  CUtensorMap v_map;
  CUtensorMap q_map_small;   // box (64, group, 32 / group): items of at most 32 rows
  const AttnItem* items;
  const int32_t* block_table;
  __nv_bfloat16* out;   // [T][hq][128]
  int* status;
  float scale_log2;     // softmax scale * log2(e)
  int32_t bt_stride, hq, hkv, group, page, n_items;
  int32_t q_box_rows;   // rows of the q box: group * tokens per block (the bytes one q copy delivers)
  int32_t pad;          // nonzero: record the phase trace of item 0
  float* ws_o;          // split items: unnormalised O rows, fp32 [rows][128]
  float2* ws_ml;        // and their (max, sum)
  int32_t rep_ok;       // q_map_small is valid (the group divides 32)
  int32_t claim_slot;   // which of the launch counters this launch claims its items from (set by launch_attention)
};

cudaError_t launch_attention(const AttnParams& p, cudaStream_t stream);
cudaError_t launch_attention_combine(const int32_t* items, int n_items, const float* ws_o, const float2* ws_ml,
                                     __nv_bfloat16* out, int hq, int group, cudaStream_t stream);
cudaError_t read_attention_trace(unsigned long long out[8]);

// The stable pack from given routing: ranks -> scan -> pair lists (and, when src
// is set, the packed rows).  `scratch` holds pack_scratch_bytes(T, E, K) bytes.
size_t pack_scratch_bytes(int T, int E, int K);
cudaError_t launch_pack_chain(const int* topk_ids, const float* topk_w, int T, int E, int K, int H, const bf16* src,
                              bf16* dst, int* counts, int* starts, int* pair_token, float* pair_weight,
                              int* pair_pos, void* scratch, int* status, cudaStream_t stream);

}  // namespace mf
