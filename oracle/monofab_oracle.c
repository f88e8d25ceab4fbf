/* CPU oracle of the MonoFab MoE hot path.  TEST INFRASTRUCTURE ONLY: it is
 * called by tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline
 * legs as the checker; the product (monoserve_b200/) never links or calls it.
 *
 * It restates, in plain C, the arithmetic of the reference (MonoServe):
 *   router      csrc/fabric/tiles/aux.cuh:326-417      (orc_router_topk)
 *   prefix sum  csrc/fabric/tiles/aux.cuh:423-450      (orc_scan)
 *   pack        csrc/fabric/tiles/aux.cuh:648-684      (orc_pack)
 *   expert FFN  tests/test_fabric_model.py:67-80, tests/test_fabric_gemm.py:155-164
 *                                                       (orc_expert_ffn)
 *   combine     csrc/fabric/tiles/aux.cuh:137-188 with the weighted-add epilogue
 *               csrc/fabric/tiles/gemm.cuh:310-319      (orc_combine)
 *   RMSNorm     csrc/fabric/tiles/aux.cuh:60-122, tests/test_fabric_model.py:30-32
 *
 * Parity pin: the reference stores no golden vectors for this path and its
 * native library cannot be built here (sm_90a-only, un-vendored CUTLASS and
 * ThunderKittens).  The floating-point restatement is pinned against the
 * reference's own torch oracle `reference_logits` (tests/test_fabric_model.py:
 * 46-82, tests/test_fabric_model_glm.py:34-68) run on the CPU, through the
 * fixtures in tests/golden/.  Routing ids / counts / pack lists: parity
 * unpinned in the reference (no reference test reads them); they are pinned
 * here against torch.topk on tie-free inputs and by their definition below.
 *
 * Where the reference leaves a result to the hardware (the order of its atomic
 * adds; __expf) this file fixes a definition that the CUDA kernels share:
 *   - exp is orc_expf: Cody-Waite reduction + degree-5 polynomial in fused
 *     multiply-adds, identical operation for operation to the device code;
 *   - an expert's packed rows are ordered by token, then by pick;
 *   - the combine adds a token's K expert outputs in pick order.
 * Build with -ffp-contract=off: every fused multiply-add here is an explicit
 * fmaf, and nothing else may be contracted.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_MAX_E 256
#define ORC_MAX_K 16

/* ------------------------------------------------------------- bf16 helpers */
static inline float bf16_to_f32(uint16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f32_to_bf16(float f) { /* round to nearest even */
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u); /* NaN */
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

static inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

static inline float bits_f32(int32_t i) {
  float f;
  memcpy(&f, &i, 4);
  return f;
}

/* ---------------------------------------------------------- exact-order math */
float orc_expf(float x) {
  if (x < -103.0f) return 0.0f;
  x = fminf(x, 89.0f);
  const float n = rintf(x * 1.44269502162933349609375f);
  float r = fmaf(n, -0.693145751953125f, x);
  r = fmaf(n, -1.428606765330187045037746429443359375e-06f, r);
  float p = 1.9875691500e-4f;
  p = fmaf(p, r, 1.3981999507e-3f);
  p = fmaf(p, r, 8.3334519073e-3f);
  p = fmaf(p, r, 4.1665795894e-2f);
  p = fmaf(p, r, 1.6666665459e-1f);
  p = fmaf(p, r, 5.0000001201e-1f);
  const float rr = r * r;
  float y = fmaf(p, rr, r);
  y = y + 1.0f;
  const int ni = (int)n;
  const int h = ni / 2;
  const float s1 = bits_f32((h + 127) << 23);
  const float s2 = bits_f32((ni - h + 127) << 23);
  return (y * s1) * s2;
}

float orc_sigmoidf(float x) { return 1.0f / (1.0f + orc_expf(-x)); }

static inline float orc_rsqrtf(float v) { return 1.0f / sqrtf(v); }

/* The xor butterfly 16, 8, 4, 2, 1 over 32 lane values; every lane ends with
 * the same sum, returned here. */
static float butterfly_sum(float v[32]) {
  float t[32];
  for (int o = 16; o; o >>= 1) {
    for (int l = 0; l < 32; ++l) t[l] = v[l] + v[l ^ o];
    memcpy(v, t, sizeof t);
  }
  return v[0];
}

/* ------------------------------------------------------------ router logits
 * logits[t][e] = sum_h x[t][h] * wr[e][h]; lane l accumulates h = 256 j + 8 l + i
 * (j outer, i inner) with fmaf, then the butterfly.  H % 256 == 0. */
void orc_router_logits(const uint16_t* x, const uint16_t* wr, float* logits, int T, int H, int E) {
  for (int t = 0; t < T; ++t)
    for (int e = 0; e < E; ++e) {
      float part[32];
      for (int l = 0; l < 32; ++l) {
        float acc = 0.f;
        for (int j = 0; j < H / 256; ++j)
          for (int i = 0; i < 8; ++i) {
            const int h = 256 * j + 8 * l + i;
            acc = fmaf(bf16_to_f32(x[(size_t)t * H + h]), bf16_to_f32(wr[(size_t)e * H + h]), acc);
          }
        part[l] = acc;
      }
      logits[(size_t)t * E + e] = butterfly_sum(part);
    }
}

/* -------------------------------------------------------------- router top-k
 * Expert e lives in lane e % 32, register e / 32 (8 registers per lane, the
 * unused ones hold -1e30).  Softmax: max; p = exp(l - max); per-lane sums over
 * the 8 registers in order, butterfly; p /= s.  Sigmoid: p = sigmoid(l), the
 * selection value is p + bias, the weight is p.  K rounds of arg-max, highest
 * value first and lowest expert index on ties; wsum accumulates the picked
 * weights in pick order; weight = (renorm ? w / wsum : w) * scale. */
int orc_router_topk(const float* logits, const float* bias, int32_t* topk_ids, float* topk_w,
                    int32_t* counts, int T, int E, int K, int scoring, int renorm, float scale) {
  if (E < 1 || E > ORC_MAX_E || K < 1 || K > ORC_MAX_K || K > E) return -1;
  for (int t = 0; t < T; ++t) {
    const float* lg = logits + (size_t)t * E;
    float p[ORC_MAX_E], sel[ORC_MAX_E];
    for (int e = 0; e < ORC_MAX_E; ++e) p[e] = e < E ? lg[e] : -1e30f;
    if (scoring == 0) {
      float mx = -1e30f;
      for (int e = 0; e < ORC_MAX_E; ++e) mx = fmaxf(mx, p[e]);
      float lane_sum[32];
      for (int l = 0; l < 32; ++l) {
        float s = 0.f;
        for (int i = 0; i < ORC_MAX_E / 32; ++i) {
          const int e = l + 32 * i;
          p[e] = orc_expf(p[e] - mx);
          s = s + p[e];
        }
        lane_sum[l] = s;
      }
      const float s = butterfly_sum(lane_sum);
      for (int e = 0; e < ORC_MAX_E; ++e) {
        p[e] = p[e] / s;
        sel[e] = e < E ? p[e] : -1e30f;
      }
    } else {
      for (int e = 0; e < ORC_MAX_E; ++e) {
        p[e] = orc_sigmoidf(p[e]);
        sel[e] = e < E ? p[e] + (bias ? bias[e] : 0.f) : -1e30f;
      }
    }
    float w[ORC_MAX_K], wsum = 0.f;
    int id[ORC_MAX_K];
    for (int k = 0; k < K; ++k) {
      float bv = -1e30f;
      int bi = 0x7fffffff;
      for (int e = 0; e < ORC_MAX_E; ++e)
        if (sel[e] > bv || (sel[e] == bv && e < bi)) {
          bv = sel[e];
          bi = e;
        }
      if (bi >= ORC_MAX_E) bi = 0; /* unreachable: E >= 1 */
      id[k] = bi;
      w[k] = p[bi];
      sel[bi] = -1e30f;
      wsum = wsum + w[k];
    }
    for (int k = 0; k < K; ++k) {
      topk_ids[(size_t)t * K + k] = id[k];
      topk_w[(size_t)t * K + k] = (renorm ? w[k] / wsum : w[k]) * scale;
      if (counts) counts[id[k]] += 1;
    }
  }
  return 0;
}

/* starts[0..E] = exclusive prefix sums of counts, starts[E] the total. */
void orc_scan(const int32_t* counts, int32_t* starts, int E) {
  int32_t run = 0;
  for (int e = 0; e < E; ++e) {
    starts[e] = run;
    run += counts[e];
  }
  starts[E] = run;
}

/* Expert-sorted pair lists; inside an expert's segment: token ascending, then
 * pick ascending.  pair_pos[t][k] is the packed row of pick k of token t. */
void orc_pack(const int32_t* topk_ids, const float* topk_w, const int32_t* starts, int T, int K, int E,
              int32_t* pair_token, float* pair_weight, int32_t* pair_pos) {
  int32_t* fill = (int32_t*)calloc((size_t)E, sizeof(int32_t));
  for (int t = 0; t < T; ++t)
    for (int k = 0; k < K; ++k) {
      const int e = topk_ids[(size_t)t * K + k];
      const int pos = starts[e] + fill[e]++;
      pair_token[pos] = t;
      pair_weight[pos] = topk_w[(size_t)t * K + k];
      pair_pos[(size_t)t * K + k] = pos;
    }
  free(fill);
}

/* xp[pos] = x[pair_token[pos]] (bf16 rows of H). */
void orc_permute_rows(const uint16_t* x, const int32_t* pair_token, int P, int H, uint16_t* xp) {
  for (int p = 0; p < P; ++p) memcpy(xp + (size_t)p * H, x + (size_t)pair_token[p] * H, (size_t)H * 2);
}

/* --------------------------------------------------------------- expert FFN
 * For every packed row m of expert e (rows starts[e] .. starts[e+1]):
 *   g = x . W13[e][f],  u = x . W13[e][I + f]      fp32 accumulate
 *   h[m][f] = bf16( silu(g) * u ),  silu(g) = g / (1 + exp(-g))
 *   y[m][n] = sum_f h[m][f] * W2[e][n][f]          fp32, NOT rounded
 * scale13 / scale2 (fp32 [E][2I] / [E][H]) multiply the accumulators of FP8
 * weights, which are then given as their exact bf16 images; NULL for bf16
 * weights.  Small cases only (plain loops). */
void orc_expert_ffn(const uint16_t* xp, const int32_t* starts, const uint16_t* w13, const uint16_t* w2,
                    const float* scale13, const float* scale2, int E, int H, int I, uint16_t* h, float* y) {
  float* xf = (float*)malloc(sizeof(float) * (size_t)H);
  float* hf = (float*)malloc(sizeof(float) * (size_t)I);
  for (int e = 0; e < E; ++e)
    for (int m = starts[e]; m < starts[e + 1]; ++m) {
      for (int k = 0; k < H; ++k) xf[k] = bf16_to_f32(xp[(size_t)m * H + k]);
      for (int f = 0; f < I; ++f) {
        const uint16_t* wg = w13 + ((size_t)e * 2 * I + f) * H;
        const uint16_t* wu = w13 + ((size_t)e * 2 * I + I + f) * H;
        float g = 0.f, u = 0.f;
        for (int k = 0; k < H; ++k) {
          g += xf[k] * bf16_to_f32(wg[k]);
          u += xf[k] * bf16_to_f32(wu[k]);
        }
        if (scale13) {
          g *= scale13[(size_t)e * 2 * I + f];
          u *= scale13[(size_t)e * 2 * I + I + f];
        }
        const float hv = g / (1.f + expf(-g)) * u;
        h[(size_t)m * I + f] = f32_to_bf16(hv);
        hf[f] = round_bf16(hv);
      }
      for (int n = 0; n < H; ++n) {
        const uint16_t* wr = w2 + ((size_t)e * H + n) * I;
        float acc = 0.f;
        for (int f = 0; f < I; ++f) acc += hf[f] * bf16_to_f32(wr[f]);
        if (scale2) acc *= scale2[(size_t)e * H + n];
        y[(size_t)m * H + n] = acc;
      }
    }
  free(xf);
  free(hf);
}

/* ------------------------------------------------------------------ combine
 * moe[t][c] = fma chain over k = 0..K-1 of w[t][k] * y[pos(t,k)][c] from 0;
 * x[t][c] = bf16(x2[t][c] + moe) (x2 NULL = 0).  With norm_w: the RMSNorm of
 * that row, out = bf16(x * inv) * w rounded to bf16, inv = 1 / sqrt(ss / H + eps),
 * where ss is accumulated as the device does: lane l owns the 8-element groups
 * c = l, l + 32, ... in order, ss = fmaf(v, v, ss) element by element, then the
 * butterfly over the 32 lanes. */
void orc_combine(const float* y, const int32_t* pair_pos, const float* topk_w, const uint16_t* x2, uint16_t* x,
                 const uint16_t* norm_w, uint16_t* normed, int T, int K, int H, float eps) {
  for (int t = 0; t < T; ++t) {
    float lane_ss[32];
    for (int l = 0; l < 32; ++l) lane_ss[l] = 0.f;
    for (int c = 0; c < H / 8; ++c) {
      const int l = c & 31;
      for (int j = 0; j < 8; ++j) {
        const int col = 8 * c + j;
        float acc = 0.f;
        for (int k = 0; k < K; ++k)
          acc = fmaf(topk_w[(size_t)t * K + k], y[(size_t)pair_pos[(size_t)t * K + k] * H + col], acc);
        const float base = x2 ? bf16_to_f32(x2[(size_t)t * H + col]) : 0.f;
        const float v = round_bf16(base + acc);
        lane_ss[l] = fmaf(v, v, lane_ss[l]);
        x[(size_t)t * H + col] = f32_to_bf16(v);
      }
    }
    if (!norm_w) continue;
    const float ss = butterfly_sum(lane_ss);
    const float inv = orc_rsqrtf(ss / (float)H + eps);
    for (int col = 0; col < H; ++col) {
      const float v = bf16_to_f32(x[(size_t)t * H + col]);
      normed[(size_t)t * H + col] = f32_to_bf16(round_bf16(v * inv) * bf16_to_f32(norm_w[col]));
    }
  }
}

/* Whole layer on small shapes: logits -> route -> pack -> FFN -> combine.
 * table-free (placement does not change arithmetic).  Work arrays are the
 * caller's: topk_ids/topk_w [T][K], counts [E], starts [E+1], pair_* [T*K],
 * pair_pos [T][K], xp [T*K][H], h [T*K][I], y [T*K][H], logits [T][E]. */
int orc_moe_layer(const uint16_t* xn, const uint16_t* x2, const uint16_t* wr, const float* bias,
                  const uint16_t* w13, const uint16_t* w2, int T, int H, int I, int E, int K, int scoring,
                  int renorm, float scale, float* logits, int32_t* topk_ids, float* topk_w, int32_t* counts,
                  int32_t* starts, int32_t* pair_token, float* pair_weight, int32_t* pair_pos, uint16_t* xp,
                  uint16_t* h, float* y, uint16_t* out) {
  orc_router_logits(xn, wr, logits, T, H, E);
  memset(counts, 0, sizeof(int32_t) * (size_t)E);
  if (orc_router_topk(logits, bias, topk_ids, topk_w, counts, T, E, K, scoring, renorm, scale)) return -1;
  orc_scan(counts, starts, E);
  orc_pack(topk_ids, topk_w, starts, T, K, E, pair_token, pair_weight, pair_pos);
  orc_permute_rows(xn, pair_token, T * K, H, xp);
  orc_expert_ffn(xp, starts, w13, w2, NULL, NULL, E, H, I, h, y);
  orc_combine(y, pair_pos, topk_w, x2, out, NULL, NULL, T, K, H, 0.f);
  return 0;
}
