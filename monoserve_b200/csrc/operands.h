// Operand blocks of model tiles: the wire format between the Python program
// builders and the device tiles.  Field names, types and order are the ABI of
// the reference (csrc/fabric/model_types.h:50-235), because its Python side
// packs these blocks by the offsets the native library reports
// (monoserve/fabric/args.py:11-31).  Each block is declared once, as an
// X-macro list, from which both the C struct and the layout table are built.
#pragma once
#include <cstddef>
#include <cstdint>

namespace mf {

#define MF_GEMM_ARGS(U64, U32, F32) \
  U64(out) U64(pair_token) U64(pair_weight) U64(residual) U64(bias) \
  U32(ld_out) U32(ld_res) U32(k_tiles) U32(epi) U32(bm) U32(n_limit) U32(up_offset) U32(w_fp8)

#define MF_ATTN_ARGS(U64, U32, F32) \
  U64(q_map) U64(k_map) U64(v_map) U64(out) U64(ws_o) U64(ws_m) U64(ws_l) U64(block_table) U64(req_info) \
  F32(scale_log2) U32(bt_stride) U32(hq) U32(hkv) U32(group) U32(chunk_blocks) U32(max_chunks) \
  U32(page_size) U64(q_map_small)

/* acc_parts / acc_rows are not in the reference: with acc_parts > 1 the add-norm tile's `acc` is that many
 * fp32 slabs of acc_rows rows (the partial sums of a K-split GEMM, one slab per K range), added in slab order
 * and left as they are; otherwise it is one accumulator, zeroed once read. */
#define MF_NORM_ARGS(U64, U32, F32) \
  U64(x) U64(x2) U64(acc) U64(w) U64(out) U64(embed) U64(tokens) U64(gather) U64(out2) U64(step) \
  U32(H) U32(ld) F32(eps) U32(acc_parts) U32(acc_rows)

#define MF_STEP_ARGS(U64, U32, F32) \
  U64(row_req) U64(last_token) U64(seq_len) U64(block_table) U64(tok_pos) U64(tok_slot) U64(req_info) \
  U32(bt_stride) U32(page_size)

/* qkv_parts / qkv_rows are not in the reference: with qkv_parts > 1 `qkv` is that many fp32 slabs of qkv_rows
 * rows (the partial sums of a K-split projection, one slab per K range, the first with the bias); the tile adds
 * them in slab order and rounds the sum to bf16, which is the value a one-range projection would have stored. */
#define MF_QK_ARGS(U64, U32, F32) \
  U64(qkv) U64(q_out) U64(k_cache) U64(v_cache) U64(q_norm) U64(k_norm) U64(tok_pos) U64(tok_slot) \
  U64(cos_sin) U32(ld_qkv) U32(hq) U32(hkv) U32(rot_dim) F32(theta) F32(eps) U32(max_pos) U32(qkv_parts) \
  U32(qkv_rows)

#define MF_ROUTER_ARGS(U64, U32, F32) \
  U64(logits) U64(topk_ids) U64(topk_w) U64(counts) U64(bias) U32(E) U32(K) U32(scoring) U32(renorm) \
  F32(scale) U32(reserved0) U64(chunk_counts) U64(pair_rank)

#define MF_EXPAND_ARGS(U64, U32, F32) \
  U64(counts) U64(starts) U64(fill) U64(table) U64(w13_maps) U64(w2_maps) U64(xp_maps) U64(h_maps) \
  U64(w13_args) U64(w2_args) U64(hist) U64(w13_asym_args) U64(w2_asym_args) U64(red_args) \
  U64(w13_scale) U64(w2_scale) U32(E) U32(H) U32(I) U32(host_region) U32(w13_stage0) U32(w2_stage0) \
  U32(red_stage0) U32(dyn_first) U32(dyn_cap) U32(lane) U32(join_stage) U32(chunks) U64(chunk_counts) \
  U64(chunk_prefix) U64(staging) U32(fetch_stage0) U32(permute_rows) U64(permute_args)

/* ExpandArgs::permute_args / permute_rows are not in the reference: when set, the expand tile itself runs the
 * permute of rows [0, permute_rows) once its prefixes are written (the batch is small and a stage costs more than
 * the copy), and the program has no permute stage. */
/* Not in the reference: the staged form of a host-resident expert with many rows.  Its weights are
 * copied once into an HBM staging stack (slot = expert id) by fetch tiles, and its GEMM tiles read
 * that copy, so the expert crosses the host link once however many row blocks it has. */
#define MF_STAGING_ARGS(U64, U32, F32) \
  U64(w13_src) U64(w13_dst) U64(w13_bytes) U64(w2_src) U64(w2_dst) U64(w2_bytes) U32(chunk_bytes) U32(min_rows)

#define MF_REDUCE_ARGS(U64, U32, F32) U64(ws) U64(out) U32(I) U32(ld_ws) U32(ld_out)

#define MF_PERMUTE_ARGS(U64, U32, F32) \
  U64(topk_ids) U64(topk_w) U64(starts) U64(fill) U64(pair_token) U64(pair_weight) U64(src) U64(dst) \
  U32(K) U32(H) U64(pair_rank) U64(chunk_prefix) U64(pair_pos) U32(E)

#define MF_SAMPLE_ARGS(U64, U32, F32) \
  U64(logits) U64(temperature) U64(last_token) U64(steps) U64(host_tokens) U64(host_steps) U64(seed) \
  U32(V) U32(ring)

#define MF_ATTN_PLAN_ARGS(U64, U32, F32) \
  U64(attn) U64(req_info) U32(rows) U32(hkv) U32(chunk_keys) U32(stage_attn) U32(stage_comb) \
  U32(dyn_first) U32(dyn_cap) U32(workers) U32(reserved0) U64(row_req)

/* Not in the reference: the deterministic router projection and the deterministic
 * un-permute + weighted combine as fabric tiles. */
#define MF_LOGITS_ARGS(U64, U32, F32) U64(x) U64(wr) U64(logits) U32(T) U32(H) U32(E)

#define MF_COMBINE_ARGS(U64, U32, F32) \
  U64(y) U64(pair_pos) U64(topk_w) U64(x2) U64(x) U64(w) U64(out) U32(K) U32(H) F32(eps) U32(reserved0) \
  U64(shared)

#define MF_FIELD_U64(name) unsigned long long name;
#define MF_FIELD_U32(name) uint32_t name;
#define MF_FIELD_F32(name) float name;

#define MF_DECLARE(Name, LIST, SIZE)                                   \
  struct alignas(64) Name {                                            \
    LIST(MF_FIELD_U64, MF_FIELD_U32, MF_FIELD_F32)                     \
  };                                                                   \
  static_assert(sizeof(Name) == SIZE, #Name " has the wrong size");

MF_DECLARE(GemmArgs, MF_GEMM_ARGS, 128)
MF_DECLARE(AttnArgs, MF_ATTN_ARGS, 128)
MF_DECLARE(NormArgs, MF_NORM_ARGS, 128)
MF_DECLARE(StepArgs, MF_STEP_ARGS, 64)
MF_DECLARE(QkArgs, MF_QK_ARGS, 128)
MF_DECLARE(RouterArgs, MF_ROUTER_ARGS, 128)
MF_DECLARE(ExpandArgs, MF_EXPAND_ARGS, 256)
MF_DECLARE(StagingArgs, MF_STAGING_ARGS, 64)
MF_DECLARE(ReduceArgs, MF_REDUCE_ARGS, 64)
MF_DECLARE(PermuteArgs, MF_PERMUTE_ARGS, 128)
MF_DECLARE(SampleArgs, MF_SAMPLE_ARGS, 64)
MF_DECLARE(AttnPlanArgs, MF_ATTN_PLAN_ARGS, 64)
MF_DECLARE(LogitsArgs, MF_LOGITS_ARGS, 64)
MF_DECLARE(CombineArgs, MF_COMBINE_ARGS, 128)

}  // namespace mf
