/* monofab.h — C ABI of the B200-native MonoFab MoE hot path.
 *
 * Every entry point is plain C: pointers, sizes and integer handles, no C++
 * or torch types.  Device pointers are ordinary `void*` values valid on the
 * current CUDA device; `stream` is a `cudaStream_t` passed as `void*` (NULL =
 * the legacy default stream).  All functions return 0 on success and a negative
 * MONOFAB_E* code on failure; `monofab_last_error()` then describes the failure
 * for the calling thread.  Nothing here falls back to the CPU: without a CUDA
 * device the compute entry points fail with MONOFAB_ECUDA.
 *
 * Each declaration cites the interface of the reference (MonoServe) that it
 * stands in for, by the file's path inside that project.
 */
#ifndef MONOFAB_H_
#define MONOFAB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MONOFAB_OK 0
#define MONOFAB_EINVAL (-1)   /* bad argument (the message names it) */
#define MONOFAB_ECUDA (-2)    /* a CUDA runtime / driver call failed */
#define MONOFAB_EDEVICE (-3)  /* a kernel reported an error in its status word */

/* Bits of a layer's device status word (monofab_moe_status). */
#define MONOFAB_STATUS_WAIT_TIMEOUT 1  /* a bounded in-kernel wait ran out */
#define MONOFAB_STATUS_PLAN_OVERFLOW 2 /* more rows or GEMM tiles than the buffers hold, or a bad segment */
#define MONOFAB_STATUS_BAD_ARGS 4      /* an expert id outside [0, E) reached a kernel */

/* Region ids of the expert indirection table (monoserve/runtime/kinds.py:16-18). */
#define MONOFAB_REGION_HOST 0
#define MONOFAB_REGION_HOT 1

int monofab_version(void);
const char* monofab_last_error(void);

/* Field layouts of the operand structs, as JSON
 * {"Name": [sizeof, {"field": [offset, "u64"|"u32"|"f32"]}]}.
 * Replaces _C.struct_layouts() (csrc/bindings.cpp:66-168). */
const char* monofab_struct_layouts_json(void);

/* Device alias of a pinned, mapped host address.
 * Replaces _C.host_device_pointer (csrc/bindings.cpp:173-178). */
int monofab_host_device_pointer(const void* host, uint64_t* device);

/* Pinned + mapped host memory for the host-resident expert stacks and for the
 * staging buffers of the host-buffer entry points
 * (monoserve/runtime/weights.py:57-58 `pin`, csrc/host/fabric.cpp:71-73). */
int monofab_host_alloc(size_t bytes, void** host);
int monofab_host_free(void* host);

/* ---- kernel-level entry points (device pointers) ------------------------ */

/* Router projection logits[t][e] = sum_h x[t][h] * wr[e][h] in fp32 with a
 * fixed summation order (H a multiple of 256).  Stands in for the router GEMM
 * stage of a lane program (monoserve/runtime/lane.py:340-342). */
int monofab_router_logits(const void* x_bf16, const void* wr_bf16, float* logits, int T, int H, int E,
                          void* stream);

/* Routing scores, top-K, renormalisation and per-expert counts: the router tile
 * (csrc/fabric/tiles/aux.cuh:326-417, RouterArgs csrc/fabric/model_types.h:147-159).
 * scoring 0 = softmax, 1 = sigmoid (+ selection bias).  `counts` (int32 [E]) is
 * accumulated; `chunk_counts` (int32 [ceil(T/32)][E]) and `pair_rank`
 * (int32 [T][K]) feed the stable pack and may be NULL.  E <= 256, K <= 16. */
int monofab_router_topk(float* logits, const float* bias, int32_t* topk_ids, float* topk_w, int32_t* counts,
                        int32_t* chunk_counts, int32_t* pair_rank, int T, int E, int K, int scoring, int renorm,
                        float scale, int zero_logits, void* stream);

/* Stable pack from given routing: per-expert counts, exclusive prefix sums
 * (starts[0..E]) and the expert-sorted pair lists; with src/dst also the packed
 * activation rows dst[pos] = src[token].  Inside an expert's segment the order is
 * token ascending, then pick ascending.  The expander's prefix sum and the
 * permute tile (csrc/fabric/tiles/aux.cuh:423-450, 648-684; PermuteArgs
 * csrc/fabric/model_types.h:207-216).  `scratch` is device memory of at least
 * monofab_pack_scratch_bytes(T, E, K) bytes that the call may overwrite. */
size_t monofab_pack_scratch_bytes(int T, int E, int K);
int monofab_pack_pairs(const int32_t* topk_ids, const float* topk_w, int T, int E, int K, int H,
                       const void* src_bf16, void* dst_bf16, int32_t* counts, int32_t* starts,
                       int32_t* pair_token, float* pair_weight, int32_t* pair_pos, void* scratch,
                       size_t scratch_bytes, void* stream);

/* The same pack with NO allocation anywhere: the scratch lives in a fixed array
 * inside the library image (about 384 KB per GPU, held until the process exits)
 * instead of being passed in.  It has no counterpart in the reference.  It is for
 * callers that cannot allocate device memory when they need to pack - a process
 * with a persistent kernel resident (cudaMalloc/cudaFree would wait for it), a
 * component with a fixed memory budget and no allocator, a latency path that
 * cannot afford an allocation's device-wide synchronisation.
 * Limits: T <= MONOFAB_PACK_STATIC_MAX_TOKENS, else MONOFAB_EINVAL.  All calls on
 * a device share the array: calls whose kernels overlap on the GPU race, so keep
 * them on one stream.  The first call on each device looks up the array's
 * address; make that call outside any stream capture. */
#define MONOFAB_PACK_STATIC_MAX_TOKENS 4096
int monofab_pack_pairs_static(const int32_t* topk_ids, const float* topk_w, int T, int E, int K, int H,
                              const void* src_bf16, void* dst_bf16, int32_t* counts, int32_t* starts,
                              int32_t* pair_token, float* pair_weight, int32_t* pair_pos, void* stream);

/* Un-permute + weighted combine (+ optional following RMSNorm): the AddNorm tile
 * together with the weighted-add GEMM epilogue (csrc/fabric/tiles/aux.cuh:137-188,
 * csrc/fabric/tiles/gemm.cuh:310-319).  y fp32 [P][H]; x2 / norm_w / normed may be NULL. */
int monofab_combine(const float* y, const int32_t* pair_pos, const float* topk_w, const void* x2_bf16,
                    void* x_bf16, const void* norm_w_bf16, void* normed_bf16, int T, int K, int H, float eps,
                    void* stream);

/* Paged-KV GQA attention for prefill and decode rows, head_dim 128: the attention
 * tiles (csrc/fabric/tiles/attention.cuh:174-395, AttnArgs csrc/fabric/model_types.h:68-96).
 * q / out bf16 [tokens][hq][128]; k_cache, v_cache bf16 [n_pages][page_size][hkv][128]
 * (monoserve/runtime/kv.py:8-11, with the page size a parameter: 8..128, dividing 128);
 * block_table int32 [requests][bt_stride]; scale_log2 = log2(e) / sqrt(128).
 * items int32 [n_items][12] on the device, one work item per (request, KV head, block of
 * query tokens, key range): {block-table row, kv head, first query token, query tokens
 * (<= 128 / (hq / hkv)), position of the first query token, keys visible to the
 * request, first key covered (a multiple of 128), one past the last key covered (<= 0:
 * no limit), first workspace row or -1, 0, 0, 0}; a decode row is an item with one
 * query token.  An item whose workspace row is -1 covers all keys and writes `out`
 * directly.  Items that split one (request, KV head, block) over key ranges (the
 * reference's KV chunks, csrc/fabric/tiles/attention.cuh:286-395) each leave
 * query tokens x (hq / hkv) unnormalised fp32 rows in `ws` from their workspace row on;
 * `ws` holds ws_rows x 130 floats (rows of 128, then (max, sum) pairs).  merge_items
 * int32 [n_merge][8]: {first query token, query tokens, kv head, workspace row of
 * part 0, parts, workspace rows from one part to the next, 0, 0}; the parts are merged
 * in part order after the main kernel, on the same stream.  ws / merge_items may be
 * NULL when no item is split.  `status` is a device int32 that receives
 * MONOFAB_STATUS_WAIT_TIMEOUT if a bounded wait ran out. */
int monofab_attention(const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* block_table,
                      int bt_stride, const int32_t* items, int n_items, int tokens, int hq, int hkv, int page_size,
                      int n_pages, float scale_log2, float* ws, int ws_rows, const int32_t* merge_items, int n_merge,
                      int32_t* status, void* stream);

/* Diagnostics of the attention kernel (no counterpart in the reference): enable or
 * disable the phase trace of work item 0, and read the last one (out may be NULL):
 * cycles waiting for S, in the max pass, in exp + P store, rescaling O (tiles where a
 * row maximum grew), in the final wait for P V; then the item's KV tiles and its total
 * nanoseconds.  Synchronises the device. */
int monofab_attention_trace(int enable, uint64_t out[8]);

/* ---- one MoE layer ------------------------------------------------------- */

typedef struct monofab_moe monofab_moe;

typedef struct monofab_moe_config {
  int32_t hidden;        /* H, multiple of 256 */
  int32_t intermediate;  /* I, multiple of 64 */
  int32_t experts;       /* E <= 256 */
  int32_t top_k;         /* K <= 16 */
  int32_t max_tokens;    /* workspace size */
  int32_t scoring;       /* 0 softmax, 1 sigmoid */
  int32_t renorm;        /* renormalise the selected weights */
  float routed_scale;    /* multiplies the routing weights */
  int32_t fp8;           /* expert weights are e4m3 bytes with fp32 per-row scales */
  int32_t reserved[7];
} monofab_moe_config;

/* Allocates every workspace of the layer; nothing is allocated afterwards
 * (csrc/host/fabric.h:134-137).  Uses the current CUDA device. */
int monofab_moe_create(const monofab_moe_config* cfg, monofab_moe** out);
int monofab_moe_destroy(monofab_moe* m);

/* Router weight bf16 [E][H] (device) and optional fp32 [E] selection bias. */
int monofab_moe_set_router(monofab_moe* m, const void* wr_bf16, const float* bias);

/* Expert weight stacks of one region: w13 [slots][2I][H], w2 [slots][H][I]
 * (bf16, or e4m3 bytes).  Region MONOFAB_REGION_HOST takes HOST addresses of
 * pinned mapped memory, read in place over the host link; MONOFAB_REGION_HOT
 * takes device addresses (monoserve/runtime/weights.py:100-143). */
int monofab_moe_set_region(monofab_moe* m, int region, const void* w13, const void* w2, int slots);

/* The HBM hot tier is this library's own copy of the hot experts, so it may store
 * w13 in the order the tensor core wants: for every 16 features, 16 gate rows then
 * the 16 matching up rows ("packed"), which makes a SwiGLU tile one contiguous
 * 128-row TMA box.  monofab_pack_w13 makes such a copy of n stacks [2I][H] (src may
 * be the device alias of pinned host memory: the copy is then the placement
 * transfer itself, monoserve/runtime/weights.py:112-113); monofab_moe_set_w13_packed
 * tells the layer which regions hold packed w13.  The host region normally keeps
 * the reference's row order (gate rows, then up rows) and is gathered on the fly. */
int monofab_pack_w13(const void* src, void* dst, int n, int intermediate, int hidden, int elt_bytes, void* stream);
int monofab_moe_set_w13_packed(monofab_moe* m, int region, int packed);

/* FP8 per-output-channel scales, fp32 [E][2I] and [E][H] on the device, indexed by
 * expert id wherever the expert's weights are (monoserve/runtime/weights.py:103-104). */
int monofab_moe_set_scales(monofab_moe* m, const float* s13, const float* s2);

/* Hot-tier placement: int32 [E][2] = (region, slot) per expert, host memory
 * (monoserve/runtime/weights.py:127-158 `set_location`).  Copied on `stream`. */
int monofab_moe_set_table(monofab_moe* m, const int32_t* table, void* stream);

/* The part of a published plan this layer consumes (csrc/bindings.cpp:211-232
 * `Fabric.publish`): `ctas` = SMs given to the lane (0 = all), `credits` = link
 * slots (CTAs that may read host memory at once), `form` = row-block height of
 * host-resident experts, 16/32/64/128, or 0 for the weight-stationary form (one
 * pass over the weights for up to 256 rows of an expert). */
int monofab_moe_set_plan(monofab_moe* m, int ctas, int credits, int form);

/* One layer pass on device buffers: xn bf16 [T][H] (normalised input), x2 bf16
 * [T][H] residual or NULL, out bf16 [T][H] = bf16(x2 + moe(xn)).  Asynchronous on
 * `stream`.  The per-layer chain router -> expand -> permute -> experts -> add
 * of monoserve/runtime/lane.py:340-380. */
int monofab_moe_forward(monofab_moe* m, const void* xn, const void* x2, void* out, int T, void* stream);

/* The expert FFN alone, over rows the caller placed in the layer's packed-row
 * workspace "xp" (for example the receive buffer of an all-to-all): segment s
 * holds seg_counts[s] consecutive rows (device int32 [n_seg]) that all belong to
 * expert seg_expert[s] (device int32 [n_seg], NULL = segment index), n_seg <= 256.
 * Results: fp32 rows in workspace "y", bf16 hidden rows in "h", segment offsets in
 * "starts".  The total must not exceed max_tokens * top_k rows.  This is the
 * per-expert w13 -> w2 stage chain of monoserve/runtime/lane.py:352-363 on its own,
 * which expert parallelism needs between dispatch and return. */
int monofab_moe_experts(monofab_moe* m, const int32_t* seg_counts, const int32_t* seg_expert, int n_seg,
                        void* stream);

/* The same pass from and to HOST buffers (pinned for full speed): copies xn and
 * x2 to the device, runs the layer, copies `out` back and waits for it. */
int monofab_moe_forward_host(monofab_moe* m, const void* xn_host, const void* x2_host, void* out_host, int T,
                             void* stream);

/* Reads and clears the device status word (synchronises `stream`). */
int monofab_moe_status(monofab_moe* m, int32_t* status, void* stream);

/* Device address and size of a named workspace, for inspection:
 * "logits" "topk_ids" "topk_w" "counts" "starts" "pair_token" "pair_weight"
 * "pair_pos" "xp" "h" "y" "queues" (monoserve/runtime/lane.py:101-122). */
int monofab_moe_workspace(monofab_moe* m, const char* name, void** ptr, size_t* bytes);

/* Per-kernel device times of the LAST forward, in milliseconds, measured with
 * CUDA events on the launching stream when profiling is on:
 * [0] router logits [1] router top-k [2] plan [3] pack [4] expert GEMMs (w13 + w2, one launch)
 * [5] combine. */
int monofab_moe_set_profile(monofab_moe* m, int on);   /* bit 0: event times; bit 1: in-kernel role trace */
int monofab_moe_last_times(monofab_moe* m, float ms[6]);

/* ---- one MoE layer, experts partitioned over the GPUs of a node ------------------
 * Expert parallelism with this library's own exchange: rank r of `world` owns experts
 * [r * E / world, (r + 1) * E / world); routing, packing and combining stay local to a
 * rank's tokens, and the rows travel by plain stores into the owning GPU's memory over
 * NVLink, signalled with flags (no collective library call and no host round trip per
 * layer).  The reference has no collective of its own: its only multi-GPU mode is stock
 * vLLM expert parallelism (monoserve/baselines/serve_ep.py:24-28); the stage chain that is
 * distributed here is monoserve/runtime/lane.py:340-380.
 *
 * Set-up, once: every rank creates its object on its own GPU, sets the weights of ITS experts
 * on monofab_ep_local() (monofab_moe_set_region / _set_table / _set_plan, experts numbered
 * 0 .. E / world - 1), exports a handle, gathers all ranks' handles by any means (they are plain
 * bytes) and connects.  Ranks may be separate processes (CUDA IPC) or objects of one process.
 * cfg describes the whole layer (E experts, top-K) and max_tokens per rank.  rows_cap = rows a
 * rank's receive buffer takes; 0 = the worst case max_tokens * top_k * world, with which nothing
 * can overflow.  With a smaller capacity, rows beyond it are not sent and every rank reports
 * MONOFAB_STATUS_PLAN_OVERFLOW for that pass.
 * A pass is collective: every rank must call it (T may differ per rank and may be 0).  A peer
 * that never arrives ends the bounded in-kernel waits with MONOFAB_STATUS_WAIT_TIMEOUT. */
#define MONOFAB_EP_MAX_RANKS 16
#define MONOFAB_EP_HANDLE_BYTES 256
typedef struct monofab_ep monofab_ep;
int monofab_ep_create(const monofab_moe_config* cfg, int rank, int world, int rows_cap, monofab_ep** out);
monofab_moe* monofab_ep_local(monofab_ep* ep);
int monofab_ep_export(monofab_ep* ep, void* handle /* MONOFAB_EP_HANDLE_BYTES */);
int monofab_ep_connect(monofab_ep* ep, const void* handles /* world x MONOFAB_EP_HANDLE_BYTES, by rank */);
/* Closes the mappings of the peers' buffers; call on every rank, then synchronise the ranks,
 * before any rank destroys its object. */
int monofab_ep_disconnect(monofab_ep* ep);
int monofab_ep_destroy(monofab_ep* ep);
int monofab_ep_set_router(monofab_ep* ep, const void* wr_bf16, const float* bias);
/* out bf16 [T][H] = bf16(x2 + moe(xn)) for this rank's T tokens.  Asynchronous on `stream`.
 * Read the status word with monofab_moe_status(monofab_ep_local(ep), ...). */
int monofab_ep_forward(monofab_ep* ep, const void* xn, const void* x2, void* out, int T, void* stream);
/* One of the four phases of a pass (0 route + post counts, 1 dispatch rows, 2 experts + return
 * rows, 3 combine); monofab_ep_forward runs them in order.  A process that holds several ranks on
 * ONE GPU (a test) must run phase p of every rank before phase p + 1 of any, on one stream, because
 * kernels of one GPU must not wait for one another. */
int monofab_ep_phase(monofab_ep* ep, int phase, const void* xn, const void* x2, void* out, int T, void* stream);
/* "logits" "topk_ids" "topk_w" "pair_pos" "counts" "starts" "y_back" */
int monofab_ep_workspace(monofab_ep* ep, const char* name, void** ptr, size_t* bytes);
/* Device times of the last pass in milliseconds (CUDA events on the launching stream):
 * [0] router logits [1] top-k [2] counts + post [3] wait counts + dispatch [4] wait rows + plan
 * [5] expert GEMMs [6] return [7] wait y + combine. */
int monofab_ep_set_profile(monofab_ep* ep, int on);
int monofab_ep_last_times(monofab_ep* ep, float ms[8]);
/* Host arithmetic of the exchange layout, for tests: first row, in the receive buffer of the rank
 * that owns expert e, of the rows rank `src` sends for e; counts_all int32 [world][stride]. */
int monofab_ep_dest_base(const int32_t* counts_all, int stride, int world, int experts, int src, int e);

/* ---- the persistent fabric ------------------------------------------------- */

/* Error bits a running fabric reports through its host mirror (monofab_fabric_progress). */
#define MONOFAB_FABRIC_ERR_RING_WAIT 1
#define MONOFAB_FABRIC_ERR_WORKLIST 2
#define MONOFAB_FABRIC_ERR_DEADLINE 4
#define MONOFAB_FABRIC_ERR_BAD_TILE 8
#define MONOFAB_FABRIC_ERR_TILE_WAIT 16

typedef struct monofab_fabric monofab_fabric;

/* The fabric on one GPU: device state, a program pool of pool_bytes (0 = 1 GiB),
 * pinned staging and a host mirror.  num_workers 0 = one worker per SM.  Nothing is
 * allocated after this call.  class Fabric of csrc/bindings.cpp:184-187,
 * csrc/host/fabric.h:31-62. */
int monofab_fabric_create(int num_workers, int device, size_t pool_bytes, monofab_fabric** out);
int monofab_fabric_destroy(monofab_fabric* f);
int monofab_fabric_info(monofab_fabric* f, int32_t* num_workers, int32_t* num_sms, int32_t* running, uint64_t* epoch);

/* Launch / stop the persistent kernel (Fabric.start / stop, csrc/bindings.cpp:188-191).
 * The device state survives a stop, so lanes resume at the next start. */
int monofab_fabric_start(monofab_fabric* f);
int monofab_fabric_stop(monofab_fabric* f);

/* Launch workers [first_worker, first_worker + workers) of the persistent kernel on the caller's
 * stream, optionally inside a driver context (a green context's CUcontext, 0 = none): the way a
 * fabric is started beside other work, or as several partitions (Fabric.start_on,
 * csrc/bindings.cpp:189-190, csrc/host/fabric.cpp:204-227).  monofab_fabric_stop waits for every
 * such launch. */
int monofab_fabric_start_on(monofab_fabric* f, uint64_t stream, uint64_t context, int workers, int first_worker);

/* Longest idle back-off of a worker (Fabric.set_idle_cap, csrc/host/fabric.h:50), and
 * the run-time limit after which the kernel leaves on its own with
 * MONOFAB_FABRIC_ERR_DEADLINE (default 120 s, 0 = no limit; no counterpart in the
 * reference, whose kernel can only be stopped by the host). */
int monofab_fabric_set_limits(monofab_fabric* f, uint32_t idle_cap_ns, uint64_t max_run_ns);

/* A packed program: tiles int64 [n_tiles][8], stages int32 [n_stages][8] =
 * (first, count, succ_first, succ_count, deps_init, flags, mark, 0), successors
 * int32 [n_succ]; host pointers.  Returns the device address of the program
 * descriptor.  Fabric.upload / release / program_info / generation,
 * csrc/bindings.cpp:199-210, csrc/host/fabric.cpp:252-315. */
int monofab_fabric_upload(monofab_fabric* f, const int64_t* tiles, int n_tiles, const int32_t* stages, int n_stages,
                          const int32_t* succ, int n_succ, int first_stage, int reset_stage, int iterations,
                          uint64_t* handle);
int monofab_fabric_release(monofab_fabric* f, uint64_t handle);
/* info = gen, n_tiles, n_stages, first_stage, reset_stage, iterations */
int monofab_fabric_program_info(monofab_fabric* f, uint64_t handle, uint32_t info[6]);

/* Publish a plan as a new epoch: map[w] = lane of worker w or 255; per lane the
 * link credits, the borrowing order, the program handle (0 = none) and the kernel
 * form of host-resident experts (NULL = 64 everywhere).
 * Fabric.publish, csrc/bindings.cpp:211-232, csrc/host/fabric.cpp:317-355. */
int monofab_fabric_publish(monofab_fabric* f, const int32_t* map, int n_map, const uint32_t* caps, const int32_t* order,
                           const uint64_t* programs, int n_lanes, const uint32_t* forms, uint64_t* epoch_out);

/* The host mirror: per lane (iterations, gen, running, mark, mark_ns); per worker
 * the last epoch seen and when (256 entries each, may be NULL); the device error
 * bits.  Fabric.progress, csrc/bindings.cpp:26-62. */
int monofab_fabric_progress(monofab_fabric* f, uint64_t lanes[4][5], uint64_t* worker_epoch, uint64_t* worker_epoch_ns,
                            uint64_t* error);
/* stats = slots, inflight, inflight_max, running, tag, iter_in_prog, gen
 * (Fabric.lane_stats / reset_inflight_max, csrc/host/fabric.cpp:357-378). */
int monofab_fabric_lane_stats(monofab_fabric* f, int lane, uint32_t stats[7]);
int monofab_fabric_reset_inflight_max(monofab_fabric* f, int lane);

/* Copies to and from device memory that are safe while the kernel runs, and small
 * allocations from the program pool (Fabric.read / write / blob_alloc / blob_free,
 * csrc/host/fabric.cpp:122-148,405-450). */
int monofab_fabric_read(monofab_fabric* f, uint64_t src, void* dst, size_t bytes);
int monofab_fabric_write(monofab_fabric* f, uint64_t dst, const void* src, size_t bytes);
int monofab_fabric_blob_alloc(monofab_fabric* f, size_t bytes, uint64_t* addr);
int monofab_fabric_blob_free(monofab_fabric* f, uint64_t addr);

/* Stage-event tracing into a caller-provided device buffer of capacity records of
 * two u64 (stage | lane << 32 | event << 40 | tag << 48, device time);
 * capacity 0 turns it off (Fabric.set_trace / trace_count, csrc/host/fabric.cpp:165-179). */
int monofab_fabric_set_trace(monofab_fabric* f, uint64_t ptr, uint32_t capacity);
int monofab_fabric_trace_count(monofab_fabric* f, uint32_t* count);

/* A lane's ring of activated stages (link != 0: the ring of its link-gated stages):
 * counters = head, tail, reserve; up to max_entries waiting entries, oldest first, each
 * tag << 20 | stage (Fabric.lane_ring, csrc/bindings.cpp:255-265, csrc/host/fabric.cpp:418-434). */
int monofab_fabric_lane_ring(monofab_fabric* f, int lane, int link, int max_entries, uint64_t counters[3],
                             uint32_t* entries, int* n_entries);

/* What every worker is doing, for hang diagnosis: 256 state words and the device
 * time each state began (Fabric.worker_tiles, csrc/bindings.cpp:266-281). */
int monofab_fabric_worker_tiles(monofab_fabric* f, uint64_t* words, uint64_t* since_ns);

/* Where each worker's roles were waiting when the worker left after a bounded wait ran
 * out: 256 x 4 words (zero for workers that never did): [0] TMA producer, [1] MMA, [2] first
 * exec warp, each record << 48 | q phases << 40 | phases[0] << 32 | phases[1] << 24 |
 * tile << 8 | wait site; [3] records finished by the exec warps | by the MMA warp << 32.
 * The counterpart of the reference's per-warp wait notes (wait_note_address,
 * csrc/bindings.cpp:182, csrc/fabric/runtime.cuh:511-555). */
int monofab_fabric_wait_notes(monofab_fabric* f, uint64_t* notes);
/* Device address of those 256 x 4 words (wait_note_address, csrc/bindings.cpp:182). */
int monofab_fabric_wait_note_address(monofab_fabric* f, uint64_t* addr);

/* Device end times of `count` iterations of a lane after iteration `start`, taken
 * from the in-kernel timer (Fabric.iteration_times, csrc/host/fabric.cpp:380-403). */
int monofab_fabric_iteration_times(monofab_fabric* f, int lane, uint64_t start, int count, double timeout_s,
                                   uint64_t* end_ns);

/* A TMA tensor map in the fabric's table; returns the device address of its
 * record.  dims / strides (bytes, rank - 1 of them) / box innermost first; dtype
 * 0 bf16, 1 f32, 2 u8; swizzle 0/32/64/128 (Fabric.tensor_map,
 * csrc/bindings.cpp:283-296, csrc/host/tensor_map.cpp:8-50). */
int monofab_fabric_tensor_map(monofab_fabric* f, uint64_t base, const uint64_t* dims, const uint64_t* strides_bytes,
                              const uint32_t* box, int rank, int dtype, int swizzle, uint64_t* handle);

/* Marks the weight tensor behind a map record as stored in the packed SwiGLU row
 * order (monofab_pack_w13), so its SwiGLU tiles load one 128-row box.  No
 * counterpart in the reference, whose weights have one row order. */
int monofab_fabric_tensor_map_packed(monofab_fabric* f, uint64_t handle, int packed);

/* ------------------------------------------------------------------ host loop
 * A host thread that follows the lanes' marks ((layer << 8) | phase: 1 attention
 * window, 2 MoE window, 3 layer done) in the fabric's pinned mirror and stages
 * host-resident experts into a lane's HBM staging buffer with the copy engine, one
 * expert at a time on its own stream, ahead of the layer that uses them; when an
 * expert has landed, its entry in the lane's (region, slot) table int32
 * [layers][experts][2] is switched with one aligned 8-byte copy, and switched back to
 * (host_region, expert) when the layer is done (class HostLoop,
 * csrc/host/host_loop.h:25-90, csrc/host/host_loop.cpp:18-160, bound at
 * csrc/bindings.cpp:306-330).
 *
 * host_w13 / host_w2: per layer, the HOST address of the pinned [experts][...] stack,
 * 0 for a layer without experts.  A loop created with fab = NULL makes no CUDA call:
 * its marks are injected, it is stepped by hand and its actions are read back as a log
 * (for tests of the staging policy on a machine without a GPU). */
typedef struct monofab_host_loop monofab_host_loop;
int monofab_host_loop_create(monofab_fabric* fab, int layers, int experts, size_t w13_bytes, size_t w2_bytes,
                             const uint64_t* host_w13, const uint64_t* host_w2, int host_region,
                             monofab_host_loop** out);
/* A lane to stage for (HostLoop::add_lane, csrc/host/host_loop.cpp:33-40;
 * StagingLaneConfig, csrc/host/host_loop.h:27-34): region = the region id of the lane's
 * staging buffer, w13_dst / w2_dst = its [2 * slots] expert slots (two halves of `slots`),
 * tables = device address of the lane's tables, order = experts to stage per layer, best
 * first, concatenated, layer l being order[order_offsets[l] .. order_offsets[l + 1]). */
int monofab_host_loop_add_lane(monofab_host_loop* h, int lane, int region, uint64_t w13_dst, uint64_t w2_dst,
                               int slots, uint64_t tables, const int32_t* order, const int32_t* order_offsets);
/* HostLoop::start / stop (csrc/host/host_loop.cpp:42-51); stop gives every half back. */
int monofab_host_loop_start(monofab_host_loop* h, int poll_us);
int monofab_host_loop_stop(monofab_host_loop* h);
/* copies, bytes, flips, restores, polls (HostLoopStats, csrc/host/host_loop.h:36-38). */
int monofab_host_loop_stats(monofab_host_loop* h, uint64_t out[5]);
int monofab_host_loop_destroy(monofab_host_loop* h);
/* Loops without a fabric only (no counterpart in the reference): set the mirror words of
 * the lane added `lane_index`-th, run one poll of every lane (a copy lands two polls after
 * it was issued), read the actions so far as records of five int32: kind (0 copy issued,
 * 1 entry switched to the staging buffer, 2 entry switched back), lane, layer, expert, slot. */
int monofab_host_loop_inject(monofab_host_loop* h, int lane_index, uint64_t mark, uint64_t gen, uint64_t running);
int monofab_host_loop_step(monofab_host_loop* h);
int monofab_host_loop_log(monofab_host_loop* h, int32_t* out, int cap, int* n);

/* ---- plans: the control plane's time estimator and plan search -------------------
 * What one lane's remaining work costs at a given SM share, link-credit grant and kernel
 * form (Estimator, csrc/control/estimator.h:108-145, estimator.cpp:200-258), and the
 * search for shares / grants / forms that keep every lane's deadline (PlanSearch,
 * csrc/control/search.h:46-88, search.cpp:184-334); bound in the reference as
 * monoserve._C.control (csrc/control/py_control.cpp:10-254).  Host code only: none of
 * these touches a GPU.  Structured arguments are flat arrays of doubles:
 *   model [MONOFAB_PLAN_MODEL_FIELDS]: hidden, intermediate, experts, top_k, layers, heads,
 *     kv_heads, head_dim, vocab, dense_layers, dense_intermediate, shared_intermediate,
 *     expert_weight_bytes, dense_weight_bytes
 *   curve: n, through_origin, x[n], y[n]     rates: flops curve, bytes curve, q_per_sm
 *   calibration: sms, R_H, R_C, q_max, link peak (bytes/s), reference form, layer overhead,
 *     tail overhead, one-pass rows, one-pass bytes per row (< 0: the reference's K-split
 *     formula); stretch curve; rates of dense, prefill attention, decode attention;
 *     n, (form, rates) x n; n, (form, link-rate curve) x n; n, (form, credits per tile) x n
 *   work: decode, first_layer, staging, deadline, samples; n, active[n]; n, miss[n];
 *     passes, per pass: seqs, (tokens, context) x seqs
 *   estimate [MONOFAB_PLAN_ESTIMATE_FIELDS]: total, attn, moe, staged, a_cmp, a_rd, m_cmp,
 *     m_rd, m_link
 *   plan: header [MONOFAB_PLAN_HEADER_FIELDS] = feasible, lanes, copy_rate, min_slack,
 *     total_time, evaluations, micros, 0; per lane [MONOFAB_PLAN_LANE_FIELDS] = sms,
 *     credits, form, cap, rate, slack, estimate
 * Form 0 is the one-pass (the reference's asymmetric) form. */
#define MONOFAB_PLAN_MODEL_FIELDS 14
#define MONOFAB_PLAN_ESTIMATE_FIELDS 9
#define MONOFAB_PLAN_HEADER_FIELDS 8
#define MONOFAB_PLAN_LANE_FIELDS 15
typedef struct monofab_plan_estimator monofab_plan_estimator;
typedef struct monofab_plan_load monofab_plan_load;
typedef struct monofab_plan_search monofab_plan_search;
double monofab_plan_curve_at(const double* x, const double* y, int n, int through_origin, double v);
int monofab_plan_estimator_create(const double* model, int n_model, const double* calibration, int n_calibration,
                                  int contention_aware, double ewma, monofab_plan_estimator** out);
int monofab_plan_estimator_destroy(monofab_plan_estimator* e);
/* out = Q^link (saturating credits), exposure bound, bytes of one expert, KV bytes per token */
int monofab_plan_estimator_info(monofab_plan_estimator* e, double out[4]);
double monofab_plan_gamma_ratio(monofab_plan_estimator* e, double own_exposure);
int monofab_plan_observe(monofab_plan_estimator* e, int decode, int moe, double ratio);
double monofab_plan_correction(monofab_plan_estimator* e, int decode, int moe);
int monofab_plan_load_create(monofab_plan_estimator* e, const double* work, int n_work, monofab_plan_load** out);
int monofab_plan_load_destroy(monofab_plan_load* l);
int monofab_plan_evaluate(monofab_plan_estimator* e, const monofab_plan_load* l, int share, double credits, int form,
                          double out[MONOFAB_PLAN_ESTIMATE_FIELDS]);
/* n_forms 0 / non-positive numbers / negative tolerance = the defaults (forms 16 32 64 128 0; 2; 8; 4; 0.01) */
int monofab_plan_search_create(monofab_plan_estimator* e, const int32_t* forms, int n_forms, int pour_quantum,
                               int pour_candidates, int decode_choices, double tolerance, monofab_plan_search** out);
int monofab_plan_search_destroy(monofab_plan_search* s);
/* smallest SM share that meets the lane's deadline; sms + 1 if none does */
int monofab_plan_deadline_floor(monofab_plan_search* s, const monofab_plan_load* l, double credits, int form, int* share);
/* lanes: at most one decode lane (first) and two prefill lanes; decode_key caches the decode lane's options (0: no cache) */
int monofab_plan_solve(monofab_plan_search* s, const monofab_plan_load* const* lanes, int n_lanes, uint64_t decode_key,
                       double* out, int out_cap);
int monofab_plan_clear_cache(monofab_plan_search* s);

/* Expected activated experts per layer for a number of routed rows, from per-layer activation shares
 * and the hot-tier mask (ProfileView, csrc/control/admission.h:26-49); out = activated, and of those
 * outside the hot tier. */
typedef struct monofab_plan_profile monofab_plan_profile;
int monofab_plan_profile_create(int layers, int experts, monofab_plan_profile** out);
int monofab_plan_profile_destroy(monofab_plan_profile* p);
int monofab_plan_profile_set(monofab_plan_profile* p, int decode, const double* shares, int n /* layers x experts */);
int monofab_plan_profile_set_hot(monofab_plan_profile* p, const uint8_t* hot, int n /* layers x experts */);
int monofab_plan_profile_expected(monofab_plan_profile* p, int decode, int layer, double pairs, double out[2]);

/* Admission (csrc/control/admission.h:51-161, admission.cpp:226-448): which requests join the decode
 * batch, which prompts are batched into a prefill lane, which are rejected, and the plan to publish,
 * decided at serving events.  config [MONOFAB_PLAN_ADMISSION_FIELDS] = max_prefill_lanes, token_budget,
 * max_batch_requests, max_decode, staging_experts, kv_capacity, kv_bytes_per_token, workspace_capacity,
 * lane_workspace, batch_trials, reject_checks.  Events:
 *   ARRIVE     id = request; args = prompt, max_output, arrival, ttft, tpot, now
 *   PASS_DONE  id = prefill lane (1, 2); args = now      FINISHED  id = request; args = now
 *   BEHIND     id = lane; args = now
 *   PROGRESS   id = lane; args = layers done (no decision)   GENERATED  id = request; args = tokens so far
 * A decision comes back as int64 words: publish, feasible, decode_changed, searches; then four counted
 * lists (the fabric lane of every plan lane; the decode batch; requests that joined it; requests
 * rejected); then the prefill passes to start: count, and per pass its lane, its request count and per
 * request (id, tokens, first position, 1 if the prompt ends in this pass).  The plan is laid out as by
 * monofab_plan_solve, with the decision's microseconds in header word 7. */
#define MONOFAB_PLAN_ADMISSION_FIELDS 11
#define MONOFAB_PLAN_EVENT_ARRIVE 0
#define MONOFAB_PLAN_EVENT_PASS_DONE 1
#define MONOFAB_PLAN_EVENT_FINISHED 2
#define MONOFAB_PLAN_EVENT_BEHIND 3
#define MONOFAB_PLAN_EVENT_PROGRESS 4
#define MONOFAB_PLAN_EVENT_GENERATED 5
typedef struct monofab_plan_admission monofab_plan_admission;
int monofab_plan_admission_create(monofab_plan_estimator* e, monofab_plan_search* s, monofab_plan_profile* p,
                                  const double* config, int n_config, monofab_plan_admission** out);
int monofab_plan_admission_destroy(monofab_plan_admission* a);
/* out = queued requests, requests waiting to join, open prefill lanes, KV bytes reserved */
int monofab_plan_admission_state(monofab_plan_admission* a, double out[4]);
int monofab_plan_admission_event(monofab_plan_admission* a, int kind, int64_t id, const double* args, int n_args,
                                 int64_t* out, int out_cap, int* out_n, double* plan, int plan_cap);

/* ---- deferred releases ---------------------------------------------------------
 * Freeing device or pinned memory and destroying streams synchronises the device, which
 * would wait for a resident fabric kernel.  Every release inside this library therefore
 * goes through one registry per device: at once when no fabric kernel runs there, else
 * queued until the last one has stopped (the reference's release_when_idle,
 * csrc/host/fabric.cpp:20-59,150-158).  This entry point drives and reads that registry
 * without a GPU, for tests: op 0 = as if a fabric had started on `device`, 1 = as if it
 * had stopped, 2 = hand in a release that only counts itself, 3 = out[0] queued
 * releases, out[1] counting releases carried out so far, out[2] fabrics running. */
int monofab_release_debug(int op, int device, uint64_t* out);

#ifdef __cplusplus
}
#endif
#endif /* MONOFAB_H_ */
