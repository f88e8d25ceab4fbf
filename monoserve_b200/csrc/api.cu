// extern "C" entry points of libmonofab (see include/monofab.h) and the host
// side of one MoE layer: workspace ownership, tensor-map encoding, the launch
// chain, host-buffer staging and per-kernel event timing.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/monofab.h"
#include "kernels.h"
#include "moe_layer.h"
#include "release.h"
#include "operands.h"

namespace mf {


thread_local std::string g_error;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_error = std::string("monofab: ") + buf;
  return code;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point table, so the
// library needs no link-time dependency on libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// dims/strides innermost first; strides has rank-1 entries, in bytes.
int encode_map(CUtensorMap* map, int dtype, const void* base, int rank, const uint64_t* dims,
               const uint64_t* strides, const uint32_t* box, int swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(MONOFAB_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const CUtensorMapDataType dt = dtype == 0   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                              : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const CUtensorMapSwizzle sw = swizzle == 128  ? CU_TENSOR_MAP_SWIZZLE_128B
                                : swizzle == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                : swizzle == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                : CU_TENSOR_MAP_SWIZZLE_NONE;
  cuuint64_t d[5], s[4];
  cuuint32_t b[5], es[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) s[i] = strides[i];
  }
  const CUresult r = fn(map, dt, rank, const_cast<void*>(base), d, s, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MONOFAB_ECUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return MONOFAB_OK;
}

}  // namespace mf

using namespace mf;

namespace mf {

int dev_alloc(monofab_moe* m, void** p, size_t bytes) {
  MF_CUDA(cudaMalloc(p, bytes ? bytes : 16));
  MF_CUDA(cudaMemset(*p, 0, bytes ? bytes : 16));
  m->owned.push_back(*p);
  return MONOFAB_OK;
}

int build_maps(monofab_moe* m) {
  const monofab_moe_config& c = m->cfg;
  const int H = c.hidden, I = c.intermediate;
  const int esz = c.fp8 ? 1 : 2;
  GemmParams& gp = m->gp;
  std::memset(&gp, 0, sizeof gp);
  for (int phase = 0; phase < 2; ++phase) {
    GemmPhaseParams& ph = gp.ph[phase];
    const uint64_t K = phase == 0 ? H : I, rows = phase == 0 ? 2 * I : H;
    for (int region = 0; region < 2; ++region) {
      const void* base = phase == 0 ? m->w13[region] : m->w2[region];
      int slots = m->slots[region];
      if (!base) {   // region unused: encode a valid map over the other region
        base = phase == 0 ? m->w13[1 - region] : m->w2[1 - region];
        slots = m->slots[1 - region];
      }
      if (!base) return fail(MONOFAB_EINVAL, "no expert weights set (monofab_moe_set_region)");
      const uint64_t dims[3] = {K, rows, static_cast<uint64_t>(slots)};
      const uint64_t strides[2] = {K * esz, rows * K * esz};
      // 128 bytes of K per row: 64 bf16 elements (one K step), or 128 e4m3 bytes (the two K steps of a stage)
      const uint32_t kbox = c.fp8 ? 128 : 64;
      const uint32_t box[3] = {kbox, 16, 1};
      const uint32_t box_big[3] = {kbox, 128, 1};
      if (int r = encode_map(&ph.w_map[region], c.fp8 ? 2 : 0, base, 3, dims, strides, box, c.fp8 ? 0 : 128)) return r;
      if (int r = encode_map(&ph.w_map_big[region], c.fp8 ? 2 : 0, base, 3, dims, strides, box_big, c.fp8 ? 0 : 128))
        return r;
    }
    const void* act = phase == 0 ? m->xp : m->h;
    for (int i = 0; i < kActBoxes; ++i) {
      const uint64_t dims[2] = {K, m->pairs_cap};
      const uint64_t strides[1] = {K * 2};
      const uint32_t box[2] = {64, static_cast<uint32_t>(16 << i)};
      if (int r = encode_map(&ph.act_map[i], 0, act, 2, dims, strides, box, 128)) return r;
    }
    ph.scale = phase == 0 ? m->s13 : m->s2;
    ph.out = phase == 0 ? m->h : static_cast<void*>(m->y);
    ph.k_tiles = static_cast<int>(K / 64);
    ph.up_offset = I;
    ph.n_limit = phase == 0 ? I : H;
    ph.ld_out = phase == 0 ? I : H;
    ph.scale_ld = phase == 0 ? 2 * I : H;
    ph.epi = phase == 0 ? 1 : 5;   // kEpiSiluMul / kEpiRowsF32
    ph.packed[0] = m->packed[0];
    ph.packed[1] = m->packed[1];
    ph.w_fp8 = c.fp8;
  }
  gp.tiles[0] = m->tiles[0];
  gp.tiles[1] = m->tiles[1];
  gp.q = m->queues;
  gp.done = m->done;
  gp.status = m->status;
  m->maps_dirty = false;
  return MONOFAB_OK;
}

int forward_locked(monofab_moe* m, const void* xn, const void* x2, void* out, int T, cudaStream_t st) {
  const monofab_moe_config& c = m->cfg;
  if (T < 0 || T > c.max_tokens) return fail(MONOFAB_EINVAL, "T=%d outside [0, max_tokens=%d]", T, c.max_tokens);
  if (T == 0) return MONOFAB_OK;
  if (!xn || !out) return fail(MONOFAB_EINVAL, "xn and out must not be NULL");
  if (!m->router_w) return fail(MONOFAB_EINVAL, "router weight not set (monofab_moe_set_router)");
  if (c.fp8 && (!m->s13 || !m->s2)) return fail(MONOFAB_EINVAL, "FP8 experts need their scales (monofab_moe_set_scales)");
  if (m->maps_dirty)
    if (int r = build_maps(m)) return r;
  const int H = c.hidden, I = c.intermediate, E = c.experts, K = c.top_k;
  const int chunks = (T + kChunkTokens - 1) / kChunkTokens;
  const int ctas = m->ctas > 0 && m->ctas < m->num_sms ? m->ctas : m->num_sms;
  const bool prof = m->profile;
  int evi = 0;
  auto mark = [&]() -> cudaError_t { return prof ? cudaEventRecord(m->ev[evi++], st) : cudaSuccess; };

  MF_CUDA(mark());
  MF_CUDA(launch_router_logits(xn, m->router_w, m->logits, T, H, E, st));
  MF_CUDA(mark());
  RouterParams rp{m->logits, m->router_bias, m->topk_ids, m->topk_w, nullptr, m->chunk_counts, m->pair_rank,
                  T, E, K, c.scoring, c.renorm, c.routed_scale, 0};
  MF_CUDA(launch_router_topk(rp, st));
  MF_CUDA(mark());
  PlanParams pp{};
  pp.chunk_counts = m->chunk_counts;
  pp.counts = m->counts;
  pp.starts = m->starts;
  pp.table = m->table;
  pp.hist = m->hist;
  pp.tiles[0] = m->tiles[0];
  pp.tiles[1] = m->tiles[1];
  pp.done = m->done;
  pp.block_cap = m->block_cap;
  pp.q = m->queues;
  pp.status = m->status;
  pp.chunks = chunks;
  pp.E = E;
  pp.H = H;
  pp.I = I;
  pp.form = m->form;
  pp.tile_cap = m->tile_cap;
  pp.n_experts = E;
  pp.rows_cap = static_cast<int>(m->pairs_cap) - 256;
  MF_CUDA(launch_plan(pp, st));
  MF_CUDA(mark());
  PackParams kp{m->topk_ids, m->topk_w, m->pair_rank, m->chunk_counts, m->starts, static_cast<const bf16*>(xn),
                static_cast<bf16*>(m->xp), m->pair_token,
                m->pair_weight, m->pair_pos, T, E, K, H, m->status};
  MF_CUDA(launch_pack(kp, st));
  MF_CUDA(mark());
  m->gp.cap = m->credits;
  m->gp.trace = m->trace_on ? m->trace : nullptr;
  MF_CUDA(launch_expert_gemm(m->gp, ctas, st));
  MF_CUDA(mark());
  CombineParams cp{};
  cp.y = m->y;
  cp.pair_pos = m->pair_pos;
  cp.topk_w = m->topk_w;
  cp.x2 = static_cast<const bf16*>(x2);
  cp.x = static_cast<bf16*>(out);
  cp.T = T;
  cp.K = K;
  cp.H = H;
  MF_CUDA(launch_combine(cp, st));
  MF_CUDA(mark());
  m->times_valid = prof;
  return MONOFAB_OK;
}

// Expert FFN over caller-described segments of the layer's packed-row buffer.  `seg` carries the
// segment description (seg_counts, seg_expert, E = number of segments, optional stride and peer
// flags to wait for); the layer fills in its own buffers and limits.
int experts_locked(monofab_moe* m, const PlanParams& seg, cudaStream_t st, cudaEvent_t after_plan) {
  const monofab_moe_config& c = m->cfg;
  const int n_seg = seg.E;
  if (n_seg < 1 || n_seg > kMaxExperts) return fail(MONOFAB_EINVAL, "experts: n_seg=%d outside [1, %d]", n_seg, kMaxExperts);
  if (!seg.seg_counts) return fail(MONOFAB_EINVAL, "experts: seg_counts must not be NULL");
  if (c.fp8 && (!m->s13 || !m->s2)) return fail(MONOFAB_EINVAL, "FP8 experts need their scales (monofab_moe_set_scales)");
  if (m->maps_dirty)
    if (int r = build_maps(m)) return r;
  const int ctas = m->ctas > 0 && m->ctas < m->num_sms ? m->ctas : m->num_sms;
  PlanParams pp = seg;
  pp.counts = m->counts;
  pp.starts = m->starts;
  pp.table = m->table;
  pp.tiles[0] = m->tiles[0];
  pp.tiles[1] = m->tiles[1];
  pp.done = m->done;
  pp.block_cap = m->block_cap;
  pp.q = m->queues;
  pp.status = m->status;
  pp.H = c.hidden;
  pp.I = c.intermediate;
  pp.form = m->form;
  pp.tile_cap = m->tile_cap;
  pp.n_experts = c.experts;
  pp.rows_cap = static_cast<int>(m->pairs_cap) - 256;
  MF_CUDA(launch_plan(pp, st));
  if (after_plan) MF_CUDA(cudaEventRecord(after_plan, st));
  m->gp.cap = m->credits;
  m->gp.trace = nullptr;
  MF_CUDA(launch_expert_gemm(m->gp, ctas, st));
  return MONOFAB_OK;
}

template <class T>
void layout_field(std::string& s, const char* name, size_t off, const char* type, bool& first) {
  char buf[160];
  snprintf(buf, sizeof buf, "%s\"%s\": [%zu, \"%s\"]", first ? "" : ", ", name, off, type);
  s += buf;
  first = false;
}

#define MF_JSON_U64(name) layout_field<S>(s, #name, offsetof(S, name), "u64", first);
#define MF_JSON_U32(name) layout_field<S>(s, #name, offsetof(S, name), "u32", first);
#define MF_JSON_F32(name) layout_field<S>(s, #name, offsetof(S, name), "f32", first);
#define MF_JSON_STRUCT(Name, LIST)                                              \
  {                                                                             \
    using S = Name;                                                             \
    bool first = true;                                                          \
    char head[96];                                                              \
    snprintf(head, sizeof head, "%s\"%s\": [%zu, {", any ? ", " : "", #Name, sizeof(S)); \
    s += head;                                                                  \
    LIST(MF_JSON_U64, MF_JSON_U32, MF_JSON_F32)                                 \
    s += "}]";                                                                  \
    any = true;                                                                 \
  }

const std::string& layouts_json() {
  static const std::string json = [] {
    std::string s = "{";
    bool any = false;
    MF_JSON_STRUCT(GemmArgs, MF_GEMM_ARGS)
    MF_JSON_STRUCT(AttnArgs, MF_ATTN_ARGS)
    MF_JSON_STRUCT(NormArgs, MF_NORM_ARGS)
    MF_JSON_STRUCT(StepArgs, MF_STEP_ARGS)
    MF_JSON_STRUCT(QkArgs, MF_QK_ARGS)
    MF_JSON_STRUCT(RouterArgs, MF_ROUTER_ARGS)
    MF_JSON_STRUCT(ExpandArgs, MF_EXPAND_ARGS)
    MF_JSON_STRUCT(ReduceArgs, MF_REDUCE_ARGS)
    MF_JSON_STRUCT(PermuteArgs, MF_PERMUTE_ARGS)
    MF_JSON_STRUCT(SampleArgs, MF_SAMPLE_ARGS)
    MF_JSON_STRUCT(AttnPlanArgs, MF_ATTN_PLAN_ARGS)
    MF_JSON_STRUCT(LogitsArgs, MF_LOGITS_ARGS)
    MF_JSON_STRUCT(CombineArgs, MF_COMBINE_ARGS)
    MF_JSON_STRUCT(StagingArgs, MF_STAGING_ARGS)
    s += "}";
    return s;
  }();
  return json;
}

}  // namespace mf

extern "C" {

int monofab_version(void) { return 100; }

const char* monofab_last_error(void) { return g_error.c_str(); }

const char* monofab_struct_layouts_json(void) { return layouts_json().c_str(); }

int monofab_host_device_pointer(const void* host, uint64_t* device) {
  if (!host || !device) return fail(MONOFAB_EINVAL, "host_device_pointer: NULL argument");
  void* d = nullptr;
  MF_CUDA(cudaHostGetDevicePointer(&d, const_cast<void*>(host), 0));
  *device = reinterpret_cast<uint64_t>(d);
  return MONOFAB_OK;
}

int monofab_host_alloc(size_t bytes, void** host) {
  if (!host) return fail(MONOFAB_EINVAL, "host_alloc: NULL argument");
  MF_CUDA(cudaHostAlloc(host, bytes ? bytes : 16, cudaHostAllocMapped | cudaHostAllocPortable));
  return MONOFAB_OK;
}

int monofab_host_free(void* host) {
  if (host) MF_CUDA(cudaFreeHost(host));
  return MONOFAB_OK;
}

int monofab_router_logits(const void* x, const void* wr, float* logits, int T, int H, int E, void* stream) {
  if (!x || !wr || !logits) return fail(MONOFAB_EINVAL, "router_logits: NULL argument");
  if (T < 0 || E <= 0 || H <= 0 || H % 256) return fail(MONOFAB_EINVAL, "router_logits: H=%d must be a positive multiple of 256", H);
  MF_CUDA(launch_router_logits(x, wr, logits, T, H, E, static_cast<cudaStream_t>(stream)));
  return MONOFAB_OK;
}

int monofab_router_topk(float* logits, const float* bias, int32_t* topk_ids, float* topk_w, int32_t* counts,
                        int32_t* chunk_counts, int32_t* pair_rank, int T, int E, int K, int scoring, int renorm,
                        float scale, int zero_logits, void* stream) {
  if (!logits || !topk_ids || !topk_w) return fail(MONOFAB_EINVAL, "router_topk: NULL argument");
  if (E < 1 || E > kMaxExperts) return fail(MONOFAB_EINVAL, "router_topk: E=%d outside [1, %d]", E, kMaxExperts);
  if (K < 1 || K > kMaxTopK || K > E) return fail(MONOFAB_EINVAL, "router_topk: K=%d outside [1, min(E, %d)]", K, kMaxTopK);
  if (T < 0) return fail(MONOFAB_EINVAL, "router_topk: negative T");
  RouterParams rp{logits, bias, topk_ids, topk_w, counts, chunk_counts, pair_rank, T, E, K, scoring, renorm, scale,
                  zero_logits};
  MF_CUDA(launch_router_topk(rp, static_cast<cudaStream_t>(stream)));
  return MONOFAB_OK;
}

int monofab_combine(const float* y, const int32_t* pair_pos, const float* topk_w, const void* x2, void* x,
                    const void* norm_w, void* normed, int T, int K, int H, float eps, void* stream) {
  if (!y || !pair_pos || !topk_w || !x) return fail(MONOFAB_EINVAL, "combine: NULL argument");
  if (norm_w && !normed) return fail(MONOFAB_EINVAL, "combine: norm_w given without an output");
  if (K < 1 || K > 32 || H <= 0 || H % 8) return fail(MONOFAB_EINVAL, "combine: bad K=%d or H=%d", K, H);
  CombineParams cp{};
  cp.y = y;
  cp.pair_pos = pair_pos;
  cp.topk_w = topk_w;
  cp.x2 = static_cast<const bf16*>(x2);
  cp.x = static_cast<bf16*>(x);
  cp.norm_w = static_cast<const bf16*>(norm_w);
  cp.normed = static_cast<bf16*>(normed);
  cp.T = T;
  cp.K = K;
  cp.H = H;
  cp.eps = eps;
  MF_CUDA(launch_combine(cp, static_cast<cudaStream_t>(stream)));
  return MONOFAB_OK;
}

size_t monofab_pack_scratch_bytes(int T, int E, int K) {
  if (T < 0 || E < 1 || K < 1) return 0;
  return pack_scratch_bytes(T, E, K);
}

int monofab_pack_pairs(const int32_t* topk_ids, const float* topk_w, int T, int E, int K, int H, const void* src,
                       void* dst, int32_t* counts, int32_t* starts, int32_t* pair_token, float* pair_weight,
                       int32_t* pair_pos, void* scratch, size_t scratch_bytes, void* stream) {
  if (!counts || !starts || (T > 0 && (!topk_ids || !topk_w || !pair_token || !pair_weight || !pair_pos)))
    return fail(MONOFAB_EINVAL, "pack_pairs: NULL argument");
  if (E < 1 || E > kMaxExperts) return fail(MONOFAB_EINVAL, "pack_pairs: E=%d outside [1, %d]", E, kMaxExperts);
  if (K < 1 || K > kMaxTopK) return fail(MONOFAB_EINVAL, "pack_pairs: K=%d outside [1, %d]", K, kMaxTopK);
  if (T < 0) return fail(MONOFAB_EINVAL, "pack_pairs: negative T");
  if ((src == nullptr) != (dst == nullptr)) return fail(MONOFAB_EINVAL, "pack_pairs: src and dst go together");
  if (src && (H <= 0 || H % 8)) return fail(MONOFAB_EINVAL, "pack_pairs: H=%d must be a positive multiple of 8", H);
  if (!scratch || scratch_bytes < pack_scratch_bytes(T, E, K))
    return fail(MONOFAB_EINVAL, "pack_pairs: scratch of %zu bytes is smaller than the %zu needed", scratch_bytes,
                pack_scratch_bytes(T, E, K));
  if (reinterpret_cast<uintptr_t>(scratch) & 3) return fail(MONOFAB_EINVAL, "pack_pairs: scratch must be 4-byte aligned");
  MF_CUDA(launch_pack_chain(topk_ids, topk_w, T, E, K, H, static_cast<const bf16*>(src), static_cast<bf16*>(dst),
                            counts, starts, pair_token, pair_weight, pair_pos, scratch, nullptr,
                            static_cast<cudaStream_t>(stream)));
  return MONOFAB_OK;
}

static int g_attention_trace = 0;

int monofab_attention_trace(int enable, uint64_t out[8]) {
  g_attention_trace = enable != 0;
  if (out) {
    unsigned long long v[8];
    MF_CUDA(cudaDeviceSynchronize());
    MF_CUDA(read_attention_trace(v));
    for (int i = 0; i < 8; ++i) out[i] = v[i];
  }
  return MONOFAB_OK;
}

int monofab_attention(const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* block_table,
                      int bt_stride, const int32_t* items, int n_items, int tokens, int hq, int hkv, int page_size,
                      int n_pages, float scale_log2, float* ws, int ws_rows, const int32_t* merge_items, int n_merge,
                      int32_t* status, void* stream) {
  if (!q || !k_cache || !v_cache || !out || !block_table || !status || (n_items > 0 && !items))
    return fail(MONOFAB_EINVAL, "attention: NULL argument");
  if (ws_rows < 0 || n_merge < 0 || (n_merge > 0 && (!merge_items || !ws || ws_rows < 1)))
    return fail(MONOFAB_EINVAL, "attention: split items need a workspace and a merge list");
  if (hkv < 1 || hq < hkv || hq % hkv) return fail(MONOFAB_EINVAL, "attention: hq=%d must be a multiple of hkv=%d", hq, hkv);
  const int group = hq / hkv;
  if (group > 128) return fail(MONOFAB_EINVAL, "attention: GQA group %d exceeds 128 rows", group);
  if (page_size < 8 || page_size > 128 || 128 % page_size) return fail(MONOFAB_EINVAL, "attention: page_size=%d must be 8, 16, 32, 64 or 128", page_size);
  if (tokens < 1 || n_pages < 1 || n_items < 0 || bt_stride < 1) return fail(MONOFAB_EINVAL, "attention: bad sizes");
  AttnParams p;
  std::memset(&p, 0, sizeof p);
  const int tok_box = 128 / group;
  {
    const uint64_t dims[3] = {128, static_cast<uint64_t>(hq), static_cast<uint64_t>(tokens)};
    const uint64_t strides[2] = {256, static_cast<uint64_t>(hq) * 256};
    const uint32_t box[3] = {64, static_cast<uint32_t>(group), static_cast<uint32_t>(tok_box)};
    if (int r = encode_map(&p.q_map, 0, q, 3, dims, strides, box, 128)) return r;
    if (32 % group == 0) {
      const uint32_t small[3] = {64, static_cast<uint32_t>(group), static_cast<uint32_t>(32 / group)};
      if (int r = encode_map(&p.q_map_small, 0, q, 3, dims, strides, small, 128)) return r;
      p.rep_ok = 1;
    }
  }
  for (int i = 0; i < 2; ++i) {
    // One box = one page's keys of one KV head with both halves of the head dimension, delivered as groups of
    // eight keys: (64 d, 8 keys, the 2 halves, page / 8 groups).  The cache row of a key holds hkv heads of
    // 128 elements, i.e. 2 hkv halves of 128 bytes, so a head's halves are coordinates 2 h and 2 h + 1 of
    // the third dimension.
    const uint64_t row = static_cast<uint64_t>(hkv) * 256;
    const uint64_t dims[5] = {64, 8, 2 * static_cast<uint64_t>(hkv), static_cast<uint64_t>(page_size / 8),
                              static_cast<uint64_t>(n_pages)};
    const uint64_t strides[4] = {row, 128, 8 * row, static_cast<uint64_t>(page_size) * row};
    const uint32_t box[5] = {64, 8, 2, static_cast<uint32_t>(page_size / 8), 1};
    if (int r = encode_map(i == 0 ? &p.k_map : &p.v_map, 0, i == 0 ? k_cache : v_cache, 5, dims, strides, box, 128)) return r;
  }
  p.items = reinterpret_cast<const AttnItem*>(items);
  p.block_table = block_table;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.status = status;
  p.scale_log2 = scale_log2;
  p.bt_stride = bt_stride;
  p.hq = hq;
  p.hkv = hkv;
  p.group = group;
  p.page = page_size;
  p.n_items = n_items;
  p.q_box_rows = tok_box * group;
  p.pad = g_attention_trace;
  p.ws_o = ws;
  p.ws_ml = ws ? reinterpret_cast<float2*>(ws + static_cast<size_t>(ws_rows) * 128) : nullptr;
  MF_CUDA(launch_attention(p, static_cast<cudaStream_t>(stream)));
  MF_CUDA(launch_attention_combine(merge_items, n_merge, p.ws_o, p.ws_ml, p.out, hq, group,
                                   static_cast<cudaStream_t>(stream)));
  return MONOFAB_OK;
}

int monofab_moe_create(const monofab_moe_config* cfg, monofab_moe** out) {
  if (!cfg || !out) return fail(MONOFAB_EINVAL, "moe_create: NULL argument");
  const monofab_moe_config& c = *cfg;
  if (c.hidden <= 0 || c.hidden % 256) return fail(MONOFAB_EINVAL, "hidden=%d must be a positive multiple of 256", c.hidden);
  if (c.intermediate <= 0 || c.intermediate % 64) return fail(MONOFAB_EINVAL, "intermediate=%d must be a positive multiple of 64", c.intermediate);
  if (c.experts < 1 || c.experts > kMaxExperts) return fail(MONOFAB_EINVAL, "experts=%d outside [1, %d]", c.experts, kMaxExperts);
  if (c.top_k < 1 || c.top_k > kMaxTopK || c.top_k > c.experts) return fail(MONOFAB_EINVAL, "top_k=%d outside [1, min(E, %d)]", c.top_k, kMaxTopK);
  if (c.max_tokens < 1) return fail(MONOFAB_EINVAL, "max_tokens=%d must be positive", c.max_tokens);
  int dev = 0;
  MF_CUDA(cudaGetDevice(&dev));
  cudaDeviceProp prop;
  MF_CUDA(cudaGetDeviceProperties(&prop, dev));
  if (prop.major != 10) return fail(MONOFAB_ECUDA, "device %d is sm_%d%d; this library is built for sm_100a only", dev, prop.major, prop.minor);
  monofab_moe* m = new monofab_moe();
  m->cfg = c;
  m->device = dev;
  m->num_sms = prop.multiProcessorCount;
  const size_t T = c.max_tokens, H = c.hidden, I = c.intermediate, E = c.experts, K = c.top_k;
  const size_t P = T * K, chunks = (T + kChunkTokens - 1) / kChunkTokens;
  // Packed rows are addressed by TMA boxes of up to 256 rows; pad so a box that
  // starts at the last row stays inside the allocation.
  m->pairs_cap = P + 256;
  // Row blocks: at most P/16 + one ragged tail per segment (form 16; monofab_moe_experts takes up
  // to kMaxExperts segments whatever E is).
  const size_t blocks_max = P / 16 + kMaxExperts;
  m->block_cap = static_cast<int>(blocks_max);
  m->tile_cap = static_cast<int>(blocks_max * ((I + 63) / 64 + (H + 127) / 128));
  int r = 0;
  auto A = [&](auto** p, size_t bytes) { if (!r) r = dev_alloc(m, reinterpret_cast<void**>(p), bytes); };
  A(&m->logits, T * E * 4);
  A(&m->topk_ids, P * 4);
  A(&m->topk_w, P * 4);
  A(&m->counts, kMaxExperts * 4);            // also used per segment by monofab_moe_experts
  A(&m->starts, (kMaxExperts + 1) * 4);
  A(&m->chunk_counts, chunks * E * 4);
  A(&m->pair_rank, P * 4);
  A(&m->pair_token, m->pairs_cap * 4);
  A(&m->pair_weight, m->pairs_cap * 4);
  A(&m->pair_pos, P * 4);
  A(&m->table, E * 2 * 4);
  A(&m->hist, E * 4);
  A(&m->xp, m->pairs_cap * H * 2);
  A(&m->h, m->pairs_cap * I * 2);
  A(&m->y, m->pairs_cap * H * 4);
  A(&m->xin, T * H * 2);
  A(&m->x2in, T * H * 2);
  A(&m->xout, T * H * 2);
  for (int q = 0; q < 2; ++q) A(&m->tiles[q], static_cast<size_t>(m->tile_cap) * sizeof(GemmTile));
  A(&m->queues, sizeof(GemmQueues));
  A(&m->done, static_cast<size_t>(m->block_cap) * 4);
  A(&m->trace, 4096 * 8);
  A(&m->status, 4);
  if (!r && cudaHostAlloc(reinterpret_cast<void**>(&m->status_host), 64, cudaHostAllocDefault) != cudaSuccess)
    r = fail(MONOFAB_ECUDA, "cudaHostAlloc of the status mirror failed");
  for (int i = 0; !r && i <= kNumTimes; ++i)
    if (cudaEventCreate(&m->ev[i]) != cudaSuccess) r = fail(MONOFAB_ECUDA, "cudaEventCreate failed");
  if (r) {
    monofab_moe_destroy(m);
    return r;
  }
  // default placement: every expert in the hot tier, slot = expert id
  std::vector<int> table(2 * E);
  for (size_t e = 0; e < E; ++e) {
    table[2 * e] = MONOFAB_REGION_HOT;
    table[2 * e + 1] = static_cast<int>(e);
  }
  if (cudaMemcpy(m->table, table.data(), table.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess) {
    monofab_moe_destroy(m);
    return fail(MONOFAB_ECUDA, "copy of the default placement table failed");
  }
  *out = m;
  return MONOFAB_OK;
}

int monofab_moe_destroy(monofab_moe* m) {
  if (!m) return MONOFAB_OK;
  // With a fabric kernel resident on the device nothing here may synchronise it: the buffers are
  // handed to the release registry and freed when that kernel has left.  Otherwise wait for the
  // layer's own kernels first, then free.
  if (!fabrics_running(m->device)) cudaDeviceSynchronize();
  for (void* p : m->owned) release_device(m->device, p);
  release_host(m->device, m->status_host);
  for (cudaEvent_t e : m->ev) release_event(m->device, e);
  delete m;
  return MONOFAB_OK;
}

int monofab_moe_set_router(monofab_moe* m, const void* wr, const float* bias) {
  if (!m || !wr) return fail(MONOFAB_EINVAL, "set_router: NULL argument");
  std::lock_guard<std::mutex> lock(m->mu);
  m->router_w = wr;
  m->router_bias = bias;
  return MONOFAB_OK;
}

int monofab_moe_set_region(monofab_moe* m, int region, const void* w13, const void* w2, int slots) {
  if (!m) return fail(MONOFAB_EINVAL, "set_region: NULL handle");
  if (region != MONOFAB_REGION_HOST && region != MONOFAB_REGION_HOT)
    return fail(MONOFAB_EINVAL, "set_region: region %d is neither host (0) nor hot (1)", region);
  if (!w13 || !w2 || slots < 1) return fail(MONOFAB_EINVAL, "set_region: NULL weights or slots=%d < 1", slots);
  std::lock_guard<std::mutex> lock(m->mu);
  if (region == MONOFAB_REGION_HOST) {
    void *d13 = nullptr, *d2 = nullptr;
    MF_CUDA(cudaHostGetDevicePointer(&d13, const_cast<void*>(w13), 0));
    MF_CUDA(cudaHostGetDevicePointer(&d2, const_cast<void*>(w2), 0));
    w13 = d13;
    w2 = d2;
  }
  if ((reinterpret_cast<uintptr_t>(w13) | reinterpret_cast<uintptr_t>(w2)) & 15)
    return fail(MONOFAB_EINVAL, "set_region: weight stacks must be 16-byte aligned");
  m->w13[region] = w13;
  m->w2[region] = w2;
  m->slots[region] = slots;
  m->maps_dirty = true;
  return MONOFAB_OK;
}

int monofab_moe_set_w13_packed(monofab_moe* m, int region, int packed) {
  if (!m) return fail(MONOFAB_EINVAL, "set_w13_packed: NULL handle");
  if (region != MONOFAB_REGION_HOST && region != MONOFAB_REGION_HOT)
    return fail(MONOFAB_EINVAL, "set_w13_packed: region %d is neither host (0) nor hot (1)", region);
  std::lock_guard<std::mutex> lock(m->mu);
  m->packed[region] = packed != 0;
  m->maps_dirty = true;
  return MONOFAB_OK;
}

int monofab_pack_w13(const void* src, void* dst, int n, int intermediate, int hidden, int elt_bytes, void* stream) {
  if (!src || !dst) return fail(MONOFAB_EINVAL, "pack_w13: NULL argument");
  if (n < 0 || intermediate <= 0 || intermediate % 16) return fail(MONOFAB_EINVAL, "pack_w13: intermediate=%d must be a positive multiple of 16", intermediate);
  if ((elt_bytes != 1 && elt_bytes != 2) || hidden <= 0 || (hidden * elt_bytes) % 16)
    return fail(MONOFAB_EINVAL, "pack_w13: rows of %d x %d bytes are not a whole number of 16-byte vectors", hidden, elt_bytes);
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15)
    return fail(MONOFAB_EINVAL, "pack_w13: buffers must be 16-byte aligned");
  MF_CUDA(launch_pack_w13(src, dst, n, intermediate, hidden, elt_bytes, static_cast<cudaStream_t>(stream)));
  return MONOFAB_OK;
}

int monofab_moe_set_scales(monofab_moe* m, const float* s13, const float* s2) {
  if (!m) return fail(MONOFAB_EINVAL, "set_scales: NULL handle");
  std::lock_guard<std::mutex> lock(m->mu);
  m->s13 = s13;
  m->s2 = s2;
  m->maps_dirty = true;
  return MONOFAB_OK;
}

int monofab_moe_set_table(monofab_moe* m, const int32_t* table, void* stream) {
  if (!m || !table) return fail(MONOFAB_EINVAL, "set_table: NULL argument");
  std::lock_guard<std::mutex> lock(m->mu);
  const int E = m->cfg.experts;
  for (int e = 0; e < E; ++e) {
    const int region = table[2 * e], slot = table[2 * e + 1];
    if (region != MONOFAB_REGION_HOST && region != MONOFAB_REGION_HOT)
      return fail(MONOFAB_EINVAL, "set_table: expert %d has region %d (host 0 / hot 1 expected)", e, region);
    if (slot < 0 || slot >= m->slots[region])
      return fail(MONOFAB_EINVAL, "set_table: expert %d slot %d outside region %d (%d slots)", e, slot, region,
                  m->slots[region]);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MF_CUDA(cudaMemcpyAsync(m->table, table, static_cast<size_t>(E) * 8, cudaMemcpyHostToDevice, st));
  MF_CUDA(cudaStreamSynchronize(st));
  return MONOFAB_OK;
}

int monofab_moe_set_plan(monofab_moe* m, int ctas, int credits, int form) {
  if (!m) return fail(MONOFAB_EINVAL, "set_plan: NULL handle");
  if (ctas < 0) return fail(MONOFAB_EINVAL, "set_plan: ctas=%d is negative", ctas);
  if (credits < 0) return fail(MONOFAB_EINVAL, "set_plan: credits=%d is negative", credits);
  if (form != 0 && form != 16 && form != 32 && form != 64 && form != 128)
    return fail(MONOFAB_EINVAL, "set_plan: form=%d is not one of 0, 16, 32, 64, 128", form);
  std::lock_guard<std::mutex> lock(m->mu);
  m->ctas = ctas;
  m->credits = credits;
  m->form = form;
  return MONOFAB_OK;
}

int monofab_moe_forward(monofab_moe* m, const void* xn, const void* x2, void* out, int T, void* stream) {
  if (!m) return fail(MONOFAB_EINVAL, "forward: NULL handle");
  std::lock_guard<std::mutex> lock(m->mu);
  return forward_locked(m, xn, x2, out, T, static_cast<cudaStream_t>(stream));
}

int monofab_moe_experts(monofab_moe* m, const int32_t* seg_counts, const int32_t* seg_expert, int n_seg, void* stream) {
  if (!m) return fail(MONOFAB_EINVAL, "experts: NULL handle");
  std::lock_guard<std::mutex> lock(m->mu);
  PlanParams seg{};
  seg.seg_counts = seg_counts;
  seg.seg_expert = seg_expert;
  seg.E = n_seg;
  return experts_locked(m, seg, static_cast<cudaStream_t>(stream), nullptr);
}

int monofab_moe_forward_host(monofab_moe* m, const void* xn_host, const void* x2_host, void* out_host, int T,
                             void* stream) {
  if (!m) return fail(MONOFAB_EINVAL, "forward_host: NULL handle");
  if (!xn_host || !out_host) return fail(MONOFAB_EINVAL, "forward_host: NULL buffer");
  std::lock_guard<std::mutex> lock(m->mu);
  if (T < 0 || T > m->cfg.max_tokens) return fail(MONOFAB_EINVAL, "T=%d outside [0, max_tokens=%d]", T, m->cfg.max_tokens);
  if (T == 0) return MONOFAB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t bytes = static_cast<size_t>(T) * m->cfg.hidden * 2;
  MF_CUDA(cudaMemcpyAsync(m->xin, xn_host, bytes, cudaMemcpyHostToDevice, st));
  if (x2_host) MF_CUDA(cudaMemcpyAsync(m->x2in, x2_host, bytes, cudaMemcpyHostToDevice, st));
  if (int r = forward_locked(m, m->xin, x2_host ? m->x2in : nullptr, m->xout, T, st)) return r;
  MF_CUDA(cudaMemcpyAsync(out_host, m->xout, bytes, cudaMemcpyDeviceToHost, st));
  MF_CUDA(cudaStreamSynchronize(st));
  return MONOFAB_OK;
}

int monofab_moe_status(monofab_moe* m, int32_t* status, void* stream) {
  if (!m || !status) return fail(MONOFAB_EINVAL, "status: NULL argument");
  std::lock_guard<std::mutex> lock(m->mu);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MF_CUDA(cudaMemcpyAsync(m->status_host, m->status, 4, cudaMemcpyDeviceToHost, st));
  MF_CUDA(cudaMemsetAsync(m->status, 0, 4, st));
  MF_CUDA(cudaStreamSynchronize(st));
  *status = *m->status_host;
  if (*status) return fail(MONOFAB_EDEVICE, "device status 0x%x%s%s", *status,
                           (*status & MONOFAB_STATUS_WAIT_TIMEOUT) ? " (a bounded wait timed out)" : "",
                           (*status & MONOFAB_STATUS_PLAN_OVERFLOW) ? " (GEMM plan overflow)" : "");
  return MONOFAB_OK;
}

int monofab_moe_workspace(monofab_moe* m, const char* name, void** ptr, size_t* bytes) {
  if (!m || !name || !ptr || !bytes) return fail(MONOFAB_EINVAL, "workspace: NULL argument");
  const monofab_moe_config& c = m->cfg;
  const size_t T = c.max_tokens, H = c.hidden, I = c.intermediate, E = c.experts, K = c.top_k, P = T * K;
  struct Entry { const char* name; void* p; size_t bytes; };
  const Entry entries[] = {
      {"logits", m->logits, T * E * 4},        {"topk_ids", m->topk_ids, P * 4},
      {"topk_w", m->topk_w, P * 4},            {"counts", m->counts, E * 4},
      {"starts", m->starts, (E + 1) * 4},      {"pair_token", m->pair_token, P * 4},
      {"pair_weight", m->pair_weight, P * 4},  {"pair_pos", m->pair_pos, P * 4},
      {"xp", m->xp, P * H * 2},                {"h", m->h, P * I * 2},
      {"y", m->y, P * H * 4},                  {"queues", m->queues, sizeof(GemmQueues)},
      {"hist", m->hist, E * 4},                {"table", m->table, E * 8},
      {"trace", m->trace, 4096 * 8},
  };
  for (const Entry& e : entries)
    if (!std::strcmp(e.name, name)) {
      *ptr = e.p;
      *bytes = e.bytes;
      return MONOFAB_OK;
    }
  return fail(MONOFAB_EINVAL, "workspace: unknown name '%s'", name);
}

int monofab_moe_set_profile(monofab_moe* m, int on) {
  if (!m) return fail(MONOFAB_EINVAL, "set_profile: NULL handle");
  std::lock_guard<std::mutex> lock(m->mu);
  m->profile = (on & 1) != 0;
  m->trace_on = (on & 2) != 0;
  m->times_valid = false;
  return MONOFAB_OK;
}

int monofab_moe_last_times(monofab_moe* m, float ms[6]) {
  if (!m || !ms) return fail(MONOFAB_EINVAL, "last_times: NULL argument");
  std::lock_guard<std::mutex> lock(m->mu);
  if (!m->times_valid) return fail(MONOFAB_EINVAL, "last_times: no profiled forward to report (monofab_moe_set_profile)");
  MF_CUDA(cudaEventSynchronize(m->ev[kNumTimes]));
  for (int i = 0; i < kNumTimes; ++i) MF_CUDA(cudaEventElapsedTime(&ms[i], m->ev[i], m->ev[i + 1]));
  return MONOFAB_OK;
}

}  // extern "C"
