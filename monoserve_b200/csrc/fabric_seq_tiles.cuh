// Tiles of the transformer sequence path inside the persistent fabric kernel: token
// embedding with decode bookkeeping, per-head q/k norm + rotary embedding + KV append,
// attention work items, the merge of split attention items, the per-step plan of the
// decode attention items, and next-token selection.  Included by fabric_device.cu after
// its scheduling code (one translation unit); kinds and operand blocks are those of the
// reference (csrc/fabric/model_types.h:8-24,68-235), the fields this library adds are
// named in operands.h.
#pragma once

namespace mf {
namespace fab {

template <class T>
__device__ __forceinline__ void load_block(T& dst, unsigned long long addr) {
  static_assert(sizeof(T) % 16 == 0, "operand blocks are multiples of 16 bytes");
  const uint4* src = reinterpret_cast<const uint4*>(addr);
  uint4* d = reinterpret_cast<uint4*>(&dst);
#pragma unroll
  for (int i = 0; i < static_cast<int>(sizeof(T) / 16); ++i) d[i] = __ldcg(src + i);
}

// An attention work item (kinds 33 prefill / 34 decode, one code path):
//   a[0] AttnArgs*; i0 first query token (row of q / out); i1 = query tokens | kv head << 16;
//   i2 first key (a multiple of 128); i3 one past the last key (0: no limit);
//   a[1] = block-table row | (workspace row + 1) << 32 (0: the item writes `out`);
//   a[2] = position of the first query token | keys visible to the request << 32.
// The reference's tiles name (request, q head or KV head, q block, KV chunk) and read the
// positions from req_info (csrc/fabric/model_types.h:68-80); here the planner (host for
// prefill, the plan tile for decode) has resolved them.  AttnArgs::ws_m is used as the
// float2 (max, sum) array of the split workspace.
__device__ bool make_attn_work(const TileDesc& t, AttnWork& w) {
  AttnArgs A;
  load_block(A, t.a[0]);
  const int group = A.group ? static_cast<int>(A.group) : (A.hkv ? static_cast<int>(A.hq / A.hkv) : 0);
  const int page = A.page_size ? static_cast<int>(A.page_size) : 64;
  if (!A.q_map || !A.k_map || !A.v_map || !A.out || !A.block_table) return false;
  if (group < 1 || group > 128 || page < 8 || page > 128 || (128 % page)) return false;
  w.q_map = reinterpret_cast<const CUtensorMap*>(A.q_map);
  w.q_map_small = reinterpret_cast<const CUtensorMap*>(A.q_map_small);
  w.k_map = reinterpret_cast<const CUtensorMap*>(A.k_map);
  w.v_map = reinterpret_cast<const CUtensorMap*>(A.v_map);
  w.block_table = reinterpret_cast<const int32_t*>(A.block_table);
  w.out = reinterpret_cast<__nv_bfloat16*>(A.out);
  w.ws_o = reinterpret_cast<float*>(A.ws_o);
  w.ws_ml = reinterpret_cast<float2*>(A.ws_m);
  w.trace = nullptr;
  w.scale_log2 = A.scale_log2;
  w.bt_stride = static_cast<int32_t>(A.bt_stride);
  w.hq = static_cast<int32_t>(A.hq);
  w.group = group;
  w.page = page;
  w.q_box_rows = (128 / group) * group;
  w.rep_ok = A.q_map_small != 0 && (32 % group) == 0;
  AttnItem& it = w.item;
  it.req = static_cast<int32_t>(t.a[1] & 0xffffffffull);
  it.ws_row0 = static_cast<int32_t>(t.a[1] >> 32) - 1;
  it.kv_head = static_cast<int32_t>(t.i1 >> 16);
  it.q_tokens = static_cast<int32_t>(t.i1 & 0xffffu);
  it.q_row0 = static_cast<int32_t>(t.i0);
  it.pos0 = static_cast<int32_t>(t.a[2] & 0xffffffffull);
  it.kv_len = static_cast<int32_t>(t.a[2] >> 32);
  it.key_begin = static_cast<int32_t>(t.i2);
  it.key_end = static_cast<int32_t>(t.i3);
  if (it.q_tokens < 1 || it.q_tokens * group > 128 || (it.key_begin & 127)) return false;
  if (it.ws_row0 >= 0 && (!w.ws_o || !w.ws_ml)) return false;
  return true;
}

// Merge tile (kind 35): a[0] AttnArgs*; i0 first query token; i1 = query tokens |
// kv head << 16; i2 workspace row of part 0; i3 = parts | workspace rows per part << 16.
__device__ void tile_attn_merge(const TileDesc& t, int tid) {
  AttnArgs A;
  load_block(A, t.a[0]);
  const int group = A.group ? static_cast<int>(A.group) : static_cast<int>(A.hq / A.hkv);
  attn_merge_rows(static_cast<int>(t.i0), static_cast<int>(t.i1 & 0xffffu), static_cast<int>(t.i1 >> 16),
                  static_cast<int>(t.i2), static_cast<int>(t.i3 & 0xffffu), static_cast<int>(t.i3 >> 16),
                  reinterpret_cast<const float*>(A.ws_o), reinterpret_cast<const float2*>(A.ws_m),
                  reinterpret_cast<__nv_bfloat16*>(A.out), static_cast<int>(A.hq), group, tid >> 5, kExecThreads / 32);
}

// Plan tile of the decode attention (kind 44, csrc/fabric/tiles/aux.cuh:687-752,
// AttnPlanArgs), one per decode layer and step: for the lengths the embedding tiles have
// just advanced, write one work item per (request, KV head, key range) into the program's
// dynamic region as stage `stage_attn`, and one merge tile per split (request, KV head) as
// stage `stage_comb`.  The range length is chosen so that the items make about two even
// rounds over `workers` SMs (at least four 128-key tiles per range); chunk_keys > 0 fixes
// it instead; AttnArgs::max_chunks (when nonzero) caps the ranges per request, which is what
// the host sizes the split workspace for: max_chunks * rows * hq rows.  a[0] AttnPlanArgs*.
__device__ void tile_attn_plan(const TileDesc& t, const ProgramDesc* P, DeviceState& S, int tid) {
  constexpr int kMaxReq = 256;
  static_assert(3 * (kMaxReq + 1) + 2 <= kExecScratchInts, "plan scratch");
  int* const s_tiles = s_exec_scratch;                 // [kMaxReq]
  int* const s_item0 = s_tiles + kMaxReq + 1;          // [kMaxReq + 1]
  int* const s_merge0 = s_item0 + kMaxReq + 1;         // [kMaxReq + 1]
  int& s_part_tiles = s_exec_scratch[3 * (kMaxReq + 1)];
  int& s_bad = s_exec_scratch[3 * (kMaxReq + 1) + 1];
  AttnPlanArgs A;
  load_block(A, t.a[0]);
  AttnArgs At;
  load_block(At, A.attn);
  const int R = static_cast<int>(A.rows), hkv = static_cast<int>(A.hkv);
  const int group = At.group ? static_cast<int>(At.group) : static_cast<int>(At.hq / At.hkv);
  const int* req_info = reinterpret_cast<const int*>(A.req_info);
  const int* row_req = reinterpret_cast<const int*>(A.row_req);
  if (tid == 0) s_bad = (R < 0 || R > kMaxReq || hkv < 1);
  exec_sync();
  if (s_bad) {
    if (tid == 0) raise_error(S, kFabErrBadTile);
    return;
  }
  for (int r = tid; r < R; r += kExecThreads) {
    const int kv_len = req_info[4 * r + 3];
    s_tiles[r] = (max(kv_len, 0) + 127) / 128;
  }
  exec_sync();
  if (tid == 0) {
    long long total = 0;
    for (int r = 0; r < R; ++r) total += s_tiles[r];
    total *= hkv;
    int part = 4;
    if (A.chunk_keys) {
      part = max(1, static_cast<int>(A.chunk_keys) / 128);
    } else {
      const int workers = A.workers ? static_cast<int>(A.workers) : 148;
      part = max(4, static_cast<int>((total + 2 * workers - 1) / (2 * workers)));
      // A small step fits one round: the shortest parts (4 .. 16 tiles) that give every worker at most one
      // item.  An item costs about as much to start as six tiles take, so a second round of short items is
      // worse than one round of items twice as long.
      for (int cand = 4; cand <= 16; ++cand) {
        int items = 0;
        for (int r = 0; r < R; ++r) items += hkv * (s_tiles[r] >= 8 ? (s_tiles[r] + cand - 1) / cand : 1);
        if (items <= workers) {
          part = cand;
          break;
        }
      }
    }
    s_part_tiles = part;
    int items = 0, merges = 0;
    for (int r = 0; r < R; ++r) {
      const int tiles = s_tiles[r];
      int parts = tiles >= 8 ? (tiles + part - 1) / part : 1;
      if (At.max_chunks && parts > static_cast<int>(At.max_chunks)) parts = static_cast<int>(At.max_chunks);
      if (parts > 1) {
        const int per = (tiles + parts - 1) / parts;
        parts = (tiles + per - 1) / per;
      }
      s_item0[r] = items;
      s_merge0[r] = merges;
      items += parts * hkv;
      merges += parts > 1 ? hkv : 0;
    }
    s_item0[R] = items;
    s_merge0[R] = merges;
  }
  // close the two stages' previous activation before their tiles and counts change
  if (tid == 1) atomicExch(&P->runtime[A.stage_attn].tag_next, 0ull);
  if (tid == 2) atomicExch(&P->runtime[A.stage_comb].tag_next, 0ull);
  __threadfence();
  exec_sync();
  const int n_items = s_item0[R], n_merge = s_merge0[R];
  const bool overflow = n_items + n_merge > static_cast<int>(A.dyn_cap);
  if (overflow && tid == 0) raise_error(S, kFabErrDynOverflow);
  const int part = s_part_tiles;
  const uint32_t item_first = A.dyn_first, merge_first = A.dyn_first + n_items;
  for (int r = tid; r < R && !overflow; r += kExecThreads) {
    const int tiles = s_tiles[r];
    const int parts = (s_item0[r + 1] - s_item0[r]) / hkv;
    const int per = parts > 1 ? (tiles + parts - 1) / parts : tiles;
    const int row0 = req_info[4 * r], pos0 = req_info[4 * r + 1], kv_len = req_info[4 * r + 3];
    const int slot = row_req ? row_req[r] : r;
    (void)part;
    TileDesc d{};
    d.kind = 34;
    d.a[0] = A.attn;
    d.i0 = static_cast<uint32_t>(row0);
    d.a[2] = static_cast<unsigned long long>(static_cast<uint32_t>(pos0)) |
             (static_cast<unsigned long long>(static_cast<uint32_t>(kv_len)) << 32);
    for (int h = 0; h < hkv; ++h) {
      d.i1 = 1u | (static_cast<uint32_t>(h) << 16);
      // workspace rows: one block of `group` rows per (merge, part)
      const int ws_base = (s_merge0[r] + h) * group;
      for (int q = 0; q < parts; ++q) {
        d.i2 = static_cast<uint32_t>(q * per * 128);
        d.i3 = parts > 1 ? static_cast<uint32_t>(min(tiles, (q + 1) * per) * 128) : 0u;
        const unsigned long long ws = parts > 1 ? static_cast<unsigned long long>(ws_base + q * n_merge * group + 1) : 0ull;
        d.a[1] = static_cast<unsigned long long>(static_cast<uint32_t>(slot)) | (ws << 32);
        P->tiles[item_first + s_item0[r] + h * parts + q] = d;
      }
      if (parts > 1) {
        TileDesc m{};
        m.kind = 35;
        m.a[0] = A.attn;
        m.i0 = static_cast<uint32_t>(row0);
        m.i1 = 1u | (static_cast<uint32_t>(h) << 16);
        m.i2 = static_cast<uint32_t>(ws_base);
        m.i3 = static_cast<uint32_t>(parts) | (static_cast<uint32_t>(n_merge * group) << 16);
        P->tiles[merge_first + s_merge0[r] + h] = m;
      }
    }
  }
  if (tid == 0) {
    StageStatic& sa = P->stages[A.stage_attn];
    StageStatic& sc = P->stages[A.stage_comb];
    sa.first = item_first;
    sa.count = overflow ? 0u : static_cast<uint32_t>(n_items);
    sc.first = merge_first;
    sc.count = overflow ? 0u : static_cast<uint32_t>(n_merge);
  }
  __threadfence();
}

// Embedding tile (kind 42, csrc/fabric/tiles/aux.cuh:192-230, NormArgs + StepArgs): rows
// [i0, i0 + i1): x[row] = embed[token], out = rmsnorm(x) * w.  Prefill rows take the token
// from `tokens`; decode rows (step != 0) take the request's last token and do the step's
// bookkeeping: position = sequence length (clamped to the block table), length + 1, the
// cache slot of the new key, and the request's req_info row {row, position, 1, position + 1}.
// The page size is StepArgs::page_size (0 = 64, the reference's fixed size).
__device__ void tile_embed(const TileDesc& t, int tid) {
  NormArgs A;
  load_block(A, t.a[0]);
  const int warp = tid >> 5, lane = tid & 31;
  const int H = static_cast<int>(A.H), n16 = H / 8;
  StepArgs St{};
  if (A.step) load_block(St, A.step);
  const int page = St.page_size ? static_cast<int>(St.page_size) : 64;
  for (uint32_t r = t.i0 + warp; r < t.i0 + t.i1; r += kExecThreads / 32) {
    int token;
    if (A.step) {
      const int slot = reinterpret_cast<const int*>(St.row_req)[r];
      token = reinterpret_cast<const int*>(St.last_token)[slot];
      if (lane == 0) {
        int* seq_len = reinterpret_cast<int*>(St.seq_len);
        const int pos = min(seq_len[slot], static_cast<int>(St.bt_stride) * page - 1);
        seq_len[slot] = pos + 1;
        reinterpret_cast<int*>(St.tok_pos)[r] = pos;
        const int pg = reinterpret_cast<const int*>(St.block_table)[static_cast<size_t>(slot) * St.bt_stride + pos / page];
        reinterpret_cast<int*>(St.tok_slot)[r] = pg * page + pos % page;
        int4* info = reinterpret_cast<int4*>(St.req_info);
        info[r] = make_int4(static_cast<int>(r), pos, 1, pos + 1);
      }
    } else {
      token = reinterpret_cast<const int*>(A.tokens)[r];
    }
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(A.embed) + static_cast<size_t>(token) * H);
    const size_t o = static_cast<size_t>(r) * A.ld;
    uint4* x = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(A.x) + o);
    float ss = 0.f;
    for (int c = lane; c < n16; c += 32) {
      const uint4 v = src[c];
      float f[8];
      unpack8(v, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = __fmaf_rn(f[j], f[j], ss);
      x[c] = v;
    }
    norm_store_row(x, ss, reinterpret_cast<const __nv_bfloat16*>(A.w), reinterpret_cast<__nv_bfloat16*>(A.out) + o, nullptr,
                   H, A.eps);
  }
}

// q/k head norm + rotary embedding + KV append (kind 37, csrc/fabric/tiles/aux.cuh:232-320,
// QkArgs).  Items [i0, i0 + i1) are (row, head) pairs, item = row * (hq + 2 hkv) + head;
// heads 0 .. hq-1 are q heads (to q_out), then hkv k heads and hkv v heads (to the paged
// caches at the row's tok_slot = page * page_size + offset).  One warp per item, lane l
// holds dims 4l .. 4l+3 of the 128.  q / k: v = bf16(v * inv_rms) * w (fp32 product kept,
// norm skipped when the weight pointer is 0), then the neox rotation of the first rot_dim
// dims in fp32 with the host-made cos/sin table fp32 [max_pos][rot_dim / 2][2], one bf16
// rounding at the store.  v heads are copied.
__device__ void tile_qk_rope(const TileDesc& t, int tid) {
  QkArgs A;
  load_block(A, t.a[0]);
  const int warp = tid >> 5, lane = tid & 31;
  const int hq = static_cast<int>(A.hq), hkv = static_cast<int>(A.hkv), heads = hq + 2 * hkv;
  const int rot = static_cast<int>(A.rot_dim), half = rot / 2;
  const __nv_bfloat16* qkv = reinterpret_cast<const __nv_bfloat16*>(A.qkv);
  const int* tok_pos = reinterpret_cast<const int*>(A.tok_pos);
  const int* tok_slot = reinterpret_cast<const int*>(A.tok_slot);
  const float* cos_sin = reinterpret_cast<const float*>(A.cos_sin);
  for (uint32_t it = t.i0 + warp; it < t.i0 + t.i1; it += kExecThreads / 32) {
    const int row = static_cast<int>(it / heads), head = static_cast<int>(it % heads);
    uint2 raw;
    if (A.qkv_parts > 1) {
      const float* part = reinterpret_cast<const float*>(A.qkv) + static_cast<size_t>(row) * A.ld_qkv + head * 128 + 4 * lane;
      const size_t slab = static_cast<size_t>(A.qkv_rows) * A.ld_qkv;
      float4 a = *reinterpret_cast<const float4*>(part);
      for (uint32_t q = 1; q < A.qkv_parts; ++q) {
        const float4 b = *reinterpret_cast<const float4*>(part + q * slab);
        a = make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
      }
      const __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
      raw = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    } else {
      raw = *reinterpret_cast<const uint2*>(qkv + static_cast<size_t>(row) * A.ld_qkv + head * 128 + 4 * lane);
    }
    const bool is_q = head < hq, is_k = !is_q && head < hq + hkv;
    __nv_bfloat16* dst;
    if (is_q) {
      dst = reinterpret_cast<__nv_bfloat16*>(A.q_out) + (static_cast<size_t>(row) * hq + head) * 128;
    } else {
      const int kvh = is_k ? head - hq : head - hq - hkv;
      __nv_bfloat16* cache = reinterpret_cast<__nv_bfloat16*>(is_k ? A.k_cache : A.v_cache);
      dst = cache + (static_cast<size_t>(tok_slot[row]) * hkv + kvh) * 128;
    }
    if (!is_q && !is_k) {
      *reinterpret_cast<uint2*>(dst + 4 * lane) = raw;
      continue;
    }
    float v[4];
    {
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float2 a = __bfloat1622float2(h2[0]), b = __bfloat1622float2(h2[1]);
      v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
    const unsigned long long wp = is_q ? A.q_norm : A.k_norm;
    if (wp) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) ss = __fmaf_rn(v[j], v[j], ss);
      ss = warp_sum_xor(ss);
      const float inv = det_rsqrtf(__fadd_rn(__fdiv_rn(ss, 128.f), A.eps));
      const uint2 wr = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(wp) + 4 * lane);
      const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wr);
      const float2 wa = __bfloat1622float2(w2[0]), wb = __bfloat1622float2(w2[1]);
      const float wv[4] = {wa.x, wa.y, wb.x, wb.y};
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = __fmul_rn(round_bf16(__fmul_rn(v[j], inv)), wv[j]);
    }
    // neox pairs (d, d + half) for d < half: the partner dims live `half / 4` lanes away
    const int plane = half / 4;
    float other[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) other[j] = __shfl_xor_sync(0xffffffffu, v[j], plane);
    const int d0 = 4 * lane;
    if (d0 < rot) {
      const int pos = min(tok_pos[row], static_cast<int>(A.max_pos) - 1);
      const bool low = d0 < half;
      const float* cs = cos_sin + (static_cast<size_t>(pos) * half + (low ? d0 : d0 - half)) * 2;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float c = cs[2 * j], s = cs[2 * j + 1];
        // low half: x1 c - x2 s; high half: x2 c + x1 s
        v[j] = low ? __fsub_rn(__fmul_rn(v[j], c), __fmul_rn(other[j], s))
                   : __fadd_rn(__fmul_rn(v[j], c), __fmul_rn(other[j], s));
      }
    }
    __nv_bfloat162 o2[2] = {__floats2bfloat162_rn(v[0], v[1]), __floats2bfloat162_rn(v[2], v[3])};
    *reinterpret_cast<uint2*>(dst + 4 * lane) = *reinterpret_cast<const uint2*>(o2);
  }
}

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

// Next token of one request (kind 43, csrc/fabric/tiles/aux.cuh:763-827, SampleArgs):
// i0 row of the logits, i1 request slot.  Temperature 0: arg-max, lowest index on ties.
// Otherwise Gumbel-max over logits / temperature with u = (hash >> 40 + 0.5) / 2^24 from a
// splitmix64 hash of (seed, slot, step, index).  Writes last_token[slot], advances
// steps[slot], and publishes the token and the step count to pinned host memory.
__device__ void tile_sample(const TileDesc& t, int tid) {
  float* const s_v = reinterpret_cast<float*>(s_exec_scratch);   // [kExecThreads / 32]
  int* const s_i = s_exec_scratch + kExecThreads / 32;
  SampleArgs A;
  load_block(A, t.a[0]);
  const int row = static_cast<int>(t.i0), slot = static_cast<int>(t.i1);
  const int V = static_cast<int>(A.V);
  const float* lg = reinterpret_cast<const float*>(A.logits) + static_cast<size_t>(row) * V;
  const float temp = A.temperature ? reinterpret_cast<const float*>(A.temperature)[slot] : 0.f;
  int* steps = reinterpret_cast<int*>(A.steps);
  const int step = steps ? steps[slot] : 0;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  auto consider = [&](float v, int i) {
    if (temp > 0.f) {
      const unsigned long long h = splitmix64(A.seed ^ (static_cast<unsigned long long>(slot) << 40) ^
                                              (static_cast<unsigned long long>(step) << 20) ^ static_cast<unsigned long long>(i));
      const float u = (static_cast<float>(h >> 40) + 0.5f) * (1.f / 16777216.f);
      v = v / temp - logf(-logf(u));
    }
    if (v > bv || (v == bv && i < bi)) {
      bv = v;
      bi = i;
    }
  };
  if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(lg) & 15) == 0) {
    // four 16-byte loads in flight per thread: a row of 150 k logits is otherwise a chain of 1200 exposed loads
    const float4* lg4 = reinterpret_cast<const float4*>(lg);
    const int n4 = V >> 2;
    for (int i0 = tid; i0 < n4; i0 += 4 * kExecThreads) {
      float4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * kExecThreads;
        q[u] = i < n4 ? __ldcs(lg4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * kExecThreads;
        if (i < n4) {
          consider(q[u].x, 4 * i);
          consider(q[u].y, 4 * i + 1);
          consider(q[u].z, 4 * i + 2);
          consider(q[u].w, 4 * i + 3);
        }
      }
    }
  } else {
    for (int i = tid; i < V; i += kExecThreads) consider(__ldcs(lg + i), i);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) {
      bv = ov;
      bi = oi;
    }
  }
  if ((tid & 31) == 0) {
    s_v[tid >> 5] = bv;
    s_i[tid >> 5] = bi;
  }
  exec_sync();
  if (tid == 0) {
    for (int w = 1; w < kExecThreads / 32; ++w)
      if (s_v[w] > bv || (s_v[w] == bv && s_i[w] < bi)) {
        bv = s_v[w];
        bi = s_i[w];
      }
    if (bi == 0x7fffffff) bi = 0;   // a row of NaNs: every comparison failed
    if (A.last_token) reinterpret_cast<int*>(A.last_token)[slot] = bi;
    if (steps) steps[slot] = step + 1;
    if (A.host_tokens) {
      const uint32_t ring = A.ring ? A.ring : 1;
      reinterpret_cast<volatile int*>(A.host_tokens)[static_cast<size_t>(slot) * ring + step % ring] = bi;
      if (A.host_steps)
        st_release_sys64(reinterpret_cast<unsigned long long*>(A.host_steps) + slot, static_cast<unsigned long long>(step + 1));
    }
  }
}

}  // namespace fab
}  // namespace mf
