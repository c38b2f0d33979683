/*
 * CPU oracle for the quantised mixture-of-experts FFN path.  TEST INFRASTRUCTURE ONLY: nothing the library ships
 * may call into this file; the tests, the smoke check and the bench's cpu_baseline leg use it as the checker.
 *
 * It restates, in plain C, the numerics of dsgx10's CPU references for this path:
 *   - router scores, top-k with ties to the lower expert id, fixed-order weight sum:
 *       altar1 engine/experts/formats.cuh:142-168 (route_sigmoid, route_sum8), tests/testdata.h:339-355 (route_ref),
 *       ds41f engine/kernels/common.cuh:266-315 (six-term sum), ds41f ref/inference/model.py:809-827 (Gate)
 *   - FP8 e4m3 128x128 block-scaled experts in the "W8A8-g128" recipe:
 *       ds41f ref/torchref/kernel.py:56-77 (act_quant), :105-108 (dequant_fp8_weight), :120-132 (fp8_gemm),
 *       ds41f ref/inference/model.py:841-851 (Expert), :889-904 (MoE)
 *   - INT4-g32 experts with bf16 activations:
 *       altar1 ref/glmref.py:108-121 (int4_dequant), :231-256 (linear, out_linear), :299-300 (silu_mul),
 *       :491-519 (bf16_mlp), :581-643 (moe); engine/experts/formats.cuh:102-119 (the dequant contract)
 *   - the engine weight layouts: altar1 engine/experts/layout.h:50-119 (pack_int4, pack_fp8)
 *
 * Pins: oracle/ref_shim.cu compiles the reference's own host functions (route_ref, the packers and readers, the
 * dequant contract) into oracle/_ref/, and tests/golden/ holds outputs of the reference's Python modules; the tests
 * check this file against both.  Group-limited expert selection, which neither engine runs, is checked against the
 * function altar1 docs/model.md:337-347 names as its definition (transformers' GlmMoeDsa route_tokens_to_experts; its
 * outputs on seeded logits are in tests/golden/group_route.npz).  Two rules have no reference test and are "parity
 * unpinned": ties between groups in that selection and the softmax score's summation order.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------------ scalar formats */

static inline float bits_f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

ORC_API float orc_bf16_to_f32(uint16_t b) { return bits_f((uint32_t)b << 16); }

/* round to nearest even; NaN kept quiet */
ORC_API uint16_t orc_f32_to_bf16(float f) {
  uint32_t u = f_bits(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static inline float bf16r(float f) { return orc_bf16_to_f32(orc_f32_to_bf16(f)); }

/* e4m3 ("fn": no infinity, 0x7f/0xff NaN, max 448): sign 1, exponent 4 (bias 7), mantissa 3 */
ORC_API float orc_e4m3_to_f32(uint8_t b) {
  const int s = b >> 7, e = (b >> 3) & 15, m = b & 7;
  float v;
  if (e == 15 && m == 7) return NAN;
  if (e == 0) v = ldexpf((float)m, -9);               /* subnormal: m * 2^-9 */
  else v = ldexpf((float)(8 + m), e - 10);            /* (1 + m/8) * 2^(e-7) */
  return s ? -v : v;
}

/* f32 -> e4m3, round to nearest even, saturating to +-448 (the conversion torch's .to(float8_e4m3fn) performs on
 * values already clamped to +-448, torchref/kernel.py:70-76, and cvt.rn.satfinite.e4m3x2.f32 on the device) */
ORC_API uint8_t orc_f32_to_e4m3(float f) {
  const uint32_t u = f_bits(f);
  const uint8_t sign = (uint8_t)((u >> 24) & 0x80);
  const float a = fabsf(f);
  if (a != a) return sign | 0x7f;
  if (a >= 448.f) return sign | 0x7e;
  if (a < 0x1p-10f) return sign;                      /* below half the smallest subnormal (2^-9): zero; tie -> even (0) */
  int e;
  (void)frexpf(a, &e);                                /* a = m * 2^e, m in [0.5, 1) */
  int ex = e - 1;                                     /* a in [2^ex, 2^(ex+1)) */
  if (ex < -6) ex = -6;                               /* subnormal range shares the exponent of 2^-6 */
  const float q = ldexpf(a, 3 - ex);                  /* in units of the ulp: [8, 16) normal, [0, 8) subnormal; exact */
  float r = nearbyintf(q);                            /* default rounding mode: to nearest even */
  int code;
  if (ex == -6 && r < 8.f) code = (int)r;             /* subnormal (or rounds up to the first normal at r == 8) */
  else {
    int ri = (int)r;
    if (ri == 16) { ri = 8; ex += 1; }
    code = ((ex + 7) << 3) | (ri - 8);
  }
  if (code > 0x7e) code = 0x7e;
  return sign | (uint8_t)code;
}

/* ------------------------------------------------------------------------------------------------------- router */

/* e^x from IEEE operations only, so a device build of the same steps returns the same bits:
 * n = rint(x log2 e), r = x - n ln2 by two fused steps, a degree-7 Taylor polynomial, then scaling by 2^n
 * (formats.cuh:142-160).  Valid for the router's range; callers clamp. */
static inline float exp_ieee(float x) {
  const float n = rintf(x * 1.44269504f);
  float r = fmaf(-n, 0.693145751953125f, x);
  r = fmaf(-n, 1.428606765330187e-06f, r);
  float p = 1.f / 5040;
  p = fmaf(p, r, 1.f / 720);
  p = fmaf(p, r, 1.f / 120);
  p = fmaf(p, r, 1.f / 24);
  p = fmaf(p, r, 1.f / 6);
  p = fmaf(p, r, 0.5f);
  p = fmaf(p, r, 1.f);
  p = fmaf(p, r, 1.f);
  return ldexpf(p, (int)n);
}

ORC_API float orc_route_sigmoid(float l) {
  const float x = -l;
  if (x > 88.f) return 0.f;
  if (x < -87.f) return 1.f;
  return 1.f / (1.f + exp_ieee(x));
}

/* ln(y) for y in [1, 2^31): IEEE operations only, so that a GPU repeats the bits.  y = 2^n m with m in [1/sqrt2, sqrt2),
 * s = (m - 1) / (m + 1), ln m = 2 s (1 + z/3 + z^2/5 + z^3/7 + z^4/9 + z^5/11), z = s^2 (Horner, fused steps);
 * ln y = n ln2_hi + (n ln2_lo + ln m). */
static inline float log_ieee(float y) {
  uint32_t u;
  memcpy(&u, &y, 4);
  int n = (int)(u >> 23) - 127;
  u = (u & 0x007FFFFFu) | 0x3F800000u;
  float m;
  memcpy(&m, &u, 4);
  if (m > 1.41421356f) m = m * 0.5f, n += 1;
  const float f = m - 1.f;
  const float sv = f / (2.f + f);
  const float z = sv * sv;
  float p = 1.f / 11;
  p = fmaf(p, z, 1.f / 9);
  p = fmaf(p, z, 1.f / 7);
  p = fmaf(p, z, 1.f / 5);
  p = fmaf(p, z, 1.f / 3);
  p = fmaf(p, z, 1.f);
  const float lm = (2.f * sv) * p;
  const float nf = (float)n;
  return fmaf(nf, 0.693145751953125f, fmaf(nf, 1.428606765330187e-06f, lm));
}
/* sqrt(softplus(l)) with torch's softplus (l > 20 ? l : log1p(exp(l)); ds41f engine/kernels/common.cuh:264-287,
 * ref/inference/model.py:818).  log1p(t) = ln(y) t / (y - 1) with y = fl(1 + t) (t itself when y == 1): a few ulp, and
 * every step is an IEEE operation. */
ORC_API float orc_route_sqrtsoftplus(float l) {
  float sp;
  if (l > 20.f) {
    sp = l;
  } else if (l < -87.f) {
    sp = 0.f;
  } else {
    const float t = exp_ieee(l);
    const float y = 1.f + t;
    const float d = y - 1.f;
    sp = d == 0.f ? t : (log_ieee(y) * t) / d;
  }
  return sqrtf(sp);
}

/* The sum of the picked scores p[0..k) (descending selection order): four running sums at stride 4, then
 * (t0 + t2) + (t1 + t3).  For k = 8 this is formats.cuh:166-168, for k = 6 common.cuh:307-310. */
static float route_sum(const float* p, int k) {
  float t[4] = {0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < 4 && j < k; ++j) t[j] = p[j];
  for (int i = 4; i < k; ++i) t[i & 3] = t[i & 3] + p[i];
  if (k <= 1) return t[0];
  if (k == 2) return t[0] + t[1];
  if (k == 3) return (t[0] + t[2]) + t[1];
  return (t[0] + t[2]) + (t[1] + t[3]);
}

/* A 32-lane butterfly sum (offsets 16, 8, 4, 2, 1), the order a warp's xor-shuffle reduction produces. */
static float butterfly32(float* p) {
  for (int o = 16; o > 0; o >>= 1) {
    float q[32];
    for (int j = 0; j < 32; ++j) q[j] = p[j] + p[j ^ o];
    memcpy(p, q, sizeof q);
  }
  return p[0];
}

/* logits[r][e] = sum_k f32(x[r][k]) * wr[e][k] in f32 (glmref.py:584, model.py:811) in the library's fixed order:
 * K is cut into slices of 1024 (the last may be shorter); in a slice lane j of 32 accumulates k = base + 128 i + 4 j + c
 * (i ascending, c = 0..3) with fused multiply-adds from zero, the 32 lane sums go through the butterfly, and the slice
 * sums are added in ascending order.  H must be a multiple of 128. */
ORC_API int orc_router_logits(const uint16_t* x, const float* wr, int R, int H, int E, float* logits) {
  if (H % 128) return -1;
#pragma omp parallel for schedule(static)
  for (int re = 0; re < R * E; ++re) {
    const int r = re / E, e = re % E;
    const uint16_t* xr = x + (size_t)r * H;
    const float* w = wr + (size_t)e * H;
    float total = 0.f;
    for (int base = 0; base < H; base += 1024) {
      const int len = H - base < 1024 ? H - base : 1024;
      float p[32];
      for (int j = 0; j < 32; ++j) {
        float a = 0.f;
        for (int i = 0; i < len / 128; ++i)
          for (int c = 0; c < 4; ++c) {
            const int k = base + 128 * i + 4 * j + c;
            a = fmaf(orc_bf16_to_f32(xr[k]), w[k], a);
          }
        p[j] = a;
      }
      const float s = butterfly32(p);
      total = base ? total + s : s;
    }
    logits[re] = total;
  }
  return 0;
}

/* RMSNorm of bf16 rows (ds41f ref/inference/model.py:281-293; altar1 ref/glmref.py:225-228 and its engine's
 * comm/glmcoll.cu:83-90): r = 1 / sqrt(mean(x^2) + eps), y = bf16(w * (x * r)) (mode 0, model.py: one rounding) or
 * y = bf16(w * bf16(x * r)) (mode 1, altar-1: the normalised value is rounded before the weight).  The mean's sum is
 * taken in the library's fixed order: the row in chunks of 8 values, chunk c to thread c mod 256 of 256, a thread adds
 * its chunks in ascending order by fused multiply-adds from zero, the 32 threads of a warp go through the butterfly, the
 * 8 warp sums are added in ascending order; then IEEE division, square root and reciprocal.  H a multiple of 8. */
static float rms_rstd_row(const uint16_t* x, int H, float eps) {
  float t[256];
  for (int j = 0; j < 256; ++j) {
    float a = 0.f;
    for (int c = j; c < H / 8; c += 256)
      for (int i = 0; i < 8; ++i) {
        const float v = orc_bf16_to_f32(x[8 * c + i]);
        a = fmaf(v, v, a);
      }
    t[j] = a;
  }
  float ss = 0.f;
  for (int w = 0; w < 8; ++w) {
    const float s = butterfly32(t + 32 * w);
    ss = w ? ss + s : s;
  }
  return 1.f / sqrtf(ss / (float)H + eps);
}
static inline uint16_t rms_out(uint16_t x, float r, uint16_t w, int mode) {
  const float xr = orc_bf16_to_f32(x) * r;
  return orc_f32_to_bf16(orc_bf16_to_f32(w) * (mode == 1 ? bf16r(xr) : xr));
}
ORC_API int orc_rmsnorm(const uint16_t* x, const uint16_t* w, int R, int H, float eps, int mode, uint16_t* y) {
  if (H % 8) return -1;
  for (int r = 0; r < R; ++r) {
    const float rs = rms_rstd_row(x + (size_t)r * H, H, eps);
    for (int k = 0; k < H; ++k) y[(size_t)r * H + k] = rms_out(x[(size_t)r * H + k], rs, w[k], mode);
  }
  return 0;
}
/* The step that follows the experts in both engines (altar1 engine/comm/glmcoll.cu:225-330 allreduce_add_norm; ds41f
 * model.py:  x = x + ffn(x), then the next norm): v = the layer's f32 sums (already reduced over ranks), out = bf16(v),
 * h = bf16(res + out) (add_f32 = 0) or bf16(res + v) (add_f32 = 1), normed = RMSNorm(h).  res may be null (h = out). */
ORC_API int orc_add_norm(const float* v, const uint16_t* res, const uint16_t* w, int R, int H, float eps, int mode,
                         int add_f32, uint16_t* out, uint16_t* h, uint16_t* normed) {
  if (H % 8) return -1;
  for (size_t i = 0; i < (size_t)R * H; ++i) {
    out[i] = orc_f32_to_bf16(v[i]);
    h[i] = res ? orc_f32_to_bf16(orc_bf16_to_f32(res[i]) + (add_f32 ? v[i] : orc_bf16_to_f32(out[i]))) : out[i];
  }
  return orc_rmsnorm(h, w, R, H, eps, mode, normed);
}

enum { ORC_SCORE_SIGMOID = 0, ORC_SCORE_SOFTMAX = 1, ORC_SCORE_SQRTSOFTPLUS = 2 };

/* Scores of one row.  softmax: t_e = exp(l_e - max), S = lane sums (lane j adds e = j, j + 32, ... ascending) through
 * the butterfly, s_e = t_e / S. */
static void row_scores(const float* l, int E, int score_fn, float* s) {
  if (score_fn == ORC_SCORE_SIGMOID) {
    for (int e = 0; e < E; ++e) s[e] = orc_route_sigmoid(l[e]);
  } else if (score_fn == ORC_SCORE_SOFTMAX) {
    float m = l[0];
    for (int e = 1; e < E; ++e) m = l[e] > m ? l[e] : m;
    float p[32];
    for (int j = 0; j < 32; ++j) p[j] = 0.f;
    for (int e = 0; e < E; ++e) {
      float d = l[e] - m;
      s[e] = d < -87.f ? 0.f : exp_ieee(d);
    }
    for (int j = 0; j < 32; ++j)
      for (int e = j; e < E; e += 32) p[j] = p[j] + s[e];
    const float S = butterfly32(p);
    for (int e = 0; e < E; ++e) s[e] = s[e] / S;
  } else {
    for (int e = 0; e < E; ++e) s[e] = orc_route_sqrtsoftplus(l[e]);
  }
}

/* idx [R][topk] (descending key, ties to the lower id), w [R][topk].
 * key = score + bias (bias may be NULL); with n_group > 1 only the topk_group groups with the largest
 * (sum of the group's two largest keys) stay eligible (ties to the lower group id): the rule of transformers' GlmMoeDsa
 * router, which altar1 docs/model.md:337-347 names as the definition (the engines run it with one group; the golden
 * fixture group_route.npz holds that function's outputs; the tie rule between groups is this file's own).  w = score / (sum + 1e-20) * route_scale when norm, else
 * score * route_scale (model.py:823-826). */
ORC_API int orc_route(const float* logits, const float* bias, int R, int E, int topk, int score_fn, int n_group,
                      int topk_group, int norm, float route_scale, int32_t* idx, float* w) {
  if (E < 1 || E > 4096 || topk < 1 || topk > 32 || topk > E) return -1;
  if (n_group < 1) n_group = 1;
  if (E % n_group || topk_group < 1 || topk_group > n_group) return -1;
  const int gs = E / n_group;
  if (n_group > 1 && (gs < 2 || topk > topk_group * gs)) return -1;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < R; ++r) {
    float* s = (float*)malloc(sizeof(float) * 2 * E);
    float* key = s + E;
    row_scores(logits + (size_t)r * E, E, score_fn, s);
    for (int e = 0; e < E; ++e) key[e] = s[e] + (bias ? bias[e] : 0.f);
    if (n_group > 1) {
      float gsc[256];
      char keep[256];
      for (int g = 0; g < n_group; ++g) {
        float a = -INFINITY, b = -INFINITY; /* largest, second largest */
        for (int e = g * gs; e < (g + 1) * gs; ++e) {
          const float v = key[e];
          if (v > a) b = a, a = v;
          else if (v > b) b = v;
        }
        gsc[g] = a + b;
        keep[g] = 0;
      }
      for (int t = 0; t < topk_group; ++t) {
        int best = -1;
        for (int g = 0; g < n_group; ++g)
          if (!keep[g] && (best < 0 || gsc[g] > gsc[best])) best = g;
        keep[best] = 1;
      }
      for (int e = 0; e < E; ++e)
        if (!keep[e / gs]) key[e] = -INFINITY;
    }
    float p[32];
    for (int k = 0; k < topk; ++k) {
      int b = -1;
      for (int e = 0; e < E; ++e)
        if (key[e] != -INFINITY && (b < 0 || key[e] > key[b])) b = e;
      if (b < 0) b = 0; /* cannot happen for finite keys */
      idx[(size_t)r * topk + k] = b;
      p[k] = s[b];
      key[b] = -INFINITY;
    }
    const float sum = route_sum(p, topk) + 1e-20f;
    for (int k = 0; k < topk; ++k) w[(size_t)r * topk + k] = norm ? p[k] / sum * route_scale : p[k] * route_scale;
    free(s);
  }
  return 0;
}

/* ---------------------------------------------------------------------------------------------------- sort/pack */

/* Stable token->expert sort.  Picks (t, j) ordered by (expert id, t) ascending.
 *   counts [E], offsets [E+1] (exclusive scan), perm_tok [P] (token of the pick at a position), perm_slot [P] (its j),
 *   pos_of [T][topk] (position of pick (t, j)), row_order [T][topk] (the row's j's in ascending expert id: the order
 *   the combine adds them, altar1 prefill.cu:136-149). */
ORC_API int orc_sort_pack(const int32_t* idx, int T, int topk, int E, int32_t* counts, int32_t* offsets,
                          int32_t* perm_tok, int32_t* perm_slot, int32_t* pos_of, int32_t* row_order) {
  memset(counts, 0, sizeof(int32_t) * E);
  for (size_t i = 0; i < (size_t)T * topk; ++i) {
    if (idx[i] < 0 || idx[i] >= E) return -1;
    counts[idx[i]]++;
  }
  offsets[0] = 0;
  for (int e = 0; e < E; ++e) offsets[e + 1] = offsets[e] + counts[e];
  int32_t* cur = (int32_t*)malloc(sizeof(int32_t) * E);
  memcpy(cur, offsets, sizeof(int32_t) * E);
  for (int t = 0; t < T; ++t)
    for (int j = 0; j < topk; ++j) {
      const int e = idx[(size_t)t * topk + j];
      const int pos = cur[e]++;
      perm_tok[pos] = t, perm_slot[pos] = j, pos_of[(size_t)t * topk + j] = pos;
    }
  free(cur);
  for (int t = 0; t < T; ++t) {
    int32_t* o = row_order + (size_t)t * topk;
    for (int j = 0; j < topk; ++j) o[j] = j;
    for (int a = 1; a < topk; ++a) { /* insertion sort by expert id */
      const int v = o[a];
      int b = a - 1;
      while (b >= 0 && idx[(size_t)t * topk + o[b]] > idx[(size_t)t * topk + v]) o[b + 1] = o[b], --b;
      o[b + 1] = v;
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------------------------ FP8 (W8A8-g128) FFN */

/* One row's activation quantisation per 128 values (kernel.py:64-77 with block 128 and f32 scales):
 * a = max(amax, 1e-4), s = a * (1/448), q = e4m3(clamp(v / s, +-448)).  n a multiple of 128. */
ORC_API void orc_act_quant(const float* v, int n, uint8_t* q, float* s) {
  const float inv448 = 1.0f / 448.0f;
  for (int b = 0; b < n / 128; ++b) {
    float a = 0.f;
    for (int i = 0; i < 128; ++i) a = fmaxf(a, fabsf(v[128 * b + i]));
    a = fmaxf(a, 1e-4f);
    const float sc = a * inv448;
    s[b] = sc;
    for (int i = 0; i < 128; ++i) {
      float t = v[128 * b + i] / sc;
      t = t > 448.f ? 448.f : t < -448.f ? -448.f : t;
      q[128 * b + i] = orc_f32_to_e4m3(t);
    }
  }
}

static float g_e4m3_lut[256];
static int g_lut_ready = 0;
static void lut_init(void) {
  if (g_lut_ready) return;
  for (int i = 0; i < 256; ++i) g_e4m3_lut[i] = orc_e4m3_to_f32((uint8_t)i);
  g_lut_ready = 1;
}

/* y[n] = bf16(sum_k (f32(qx[k]) sx[k/128]) * (f32(qw[n][k]) sw[n/128][k/128])) for n in [0, N): the dequantised
 * operands multiplied in f32 (kernel.py:105-132).  The reference's sum order is the BLAS's; here each 128-block is
 * summed in double and the block sums added in double, the centre of every f32 order.  out_f32: keep f32, no rounding. */
static void fp8_gemv(const uint8_t* qx, const float* sx, const uint8_t* qw, const float* sw, int N, int K, float* y,
                     int round_bf16) {
  const int KB = K / 128;
  float* xd = (float*)malloc(sizeof(float) * K);
  for (int k = 0; k < K; ++k) xd[k] = g_e4m3_lut[qx[k]] * sx[k / 128];
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const uint8_t* wr = qw + (size_t)n * K;
    const float* swr = sw + (size_t)(n / 128) * KB;
    double acc = 0.0;
    for (int kb = 0; kb < KB; ++kb) {
      const float s = swr[kb];
      double a = 0.0;
      for (int i = 0; i < 128; ++i) {
        const float wv = g_e4m3_lut[wr[128 * kb + i]] * s; /* f32 dequantised weight, as dequant_fp8_weight */
        a += (double)xd[128 * kb + i] * (double)wv;
      }
      acc += a;
    }
    y[n] = round_bf16 ? bf16r((float)acc) : (float)acc;
  }
  free(xd);
}

static inline float silu_f(float g) { return g / (1.f + expf(-g)); }

/* MXFP4 weights (ds41f ref/torchref/kernel.py:16, 111-118 dequant_fp4_weight): e2m1 nibbles [N][K/2], value k of row n in
 * byte k/2, the even k in the low nibble; one ue8m0 scale byte per 32 along K, W = value * 2^(byte - 127).
 * y[n] = bf16(sum_k (f32(qx[k]) sx[k/128]) * W[n][k]) (kernel.py:135-138 fp4_gemm over the fp8 activations of
 * model.py:187-196), summed in double like fp8_gemv. */
static const float g_e2m1[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};
static void mx4_gemv(const uint8_t* qx, const float* sx, const uint8_t* qw, const uint8_t* sw, int N, int K, float* y,
                     int round_bf16) {
  float* xd = (float*)malloc(sizeof(float) * K);
  for (int k = 0; k < K; ++k) xd[k] = g_e4m3_lut[qx[k]] * sx[k / 128];
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const uint8_t* wr = qw + (size_t)n * (K / 2);
    const uint8_t* swr = sw + (size_t)n * (K / 32);
    double acc = 0.0;
    for (int gq = 0; gq < K / 32; ++gq) {
      const float s = ldexpf(1.f, (int)swr[gq] - 127);
      double a = 0.0;
      for (int i = 0; i < 32; ++i) {
        const int k = 32 * gq + i;
        const float wv = g_e2m1[(wr[k / 2] >> (4 * (k & 1))) & 15] * s;
        a += (double)xd[k] * (double)wv;
      }
      acc += a;
    }
    y[n] = round_bf16 ? bf16r((float)acc) : (float)acc;
  }
  free(xd);
}
ORC_API void orc_mx4_dequant(const uint8_t* qw, const uint8_t* sw, int N, int K, float* out) {
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k)
      out[(size_t)n * K + k] = g_e2m1[(qw[(size_t)n * (K / 2) + k / 2] >> (4 * (k & 1))) & 15] *
                               ldexpf(1.f, (int)sw[(size_t)n * (K / 32) + k / 32] - 127);
}

/* One expert on one row (model.py:841-851): x bf16 [H] -> y [H] as bf16-rounded floats.  mx = 0: FP8 weights (e4m3
 * [N][K], f32 scales [N/128][K/128]); mx = 1: MXFP4 weights (nibbles, ue8m0 bytes); the activations, the roundings and
 * the SwiGLU are the same.
 * wroute: the routing weight applied to h in f32 before its rounding, or a negative number for "none" (shared expert).
 * limit > 0: the bf16 gate is clamped from above to limit and the bf16 up to +-limit before silu (model.py:845-847;
 * ds41f engine/kernels/prefill.cu:153-158 fixes limit = 10).  h_out (optional): the bf16-rounded h [I] as floats. */
static void expert_row(int mx, const uint16_t* x, int H, int I, const uint8_t* wg, const void* sg, const uint8_t* wu,
                       const void* su, const uint8_t* wd, const void* sd, float wroute, float limit, float* y, float* h_out) {
  lut_init();
  float* xf = (float*)malloc(sizeof(float) * (H > I ? H : I));
  uint8_t* q = (uint8_t*)malloc(H > I ? H : I);
  float* s = (float*)malloc(sizeof(float) * ((H > I ? H : I) / 128));
  float* g = (float*)malloc(sizeof(float) * I);
  float* u = (float*)malloc(sizeof(float) * I);
  for (int k = 0; k < H; ++k) xf[k] = orc_bf16_to_f32(x[k]);
  orc_act_quant(xf, H, q, s);
  if (mx) mx4_gemv(q, s, wg, (const uint8_t*)sg, I, H, g, 1), mx4_gemv(q, s, wu, (const uint8_t*)su, I, H, u, 1);
  else fp8_gemv(q, s, wg, (const float*)sg, I, H, g, 1), fp8_gemv(q, s, wu, (const float*)su, I, H, u, 1);
  for (int i = 0; i < I; ++i) {
    float gv = g[i], uv = u[i];
    if (limit > 0.f) {
      uv = uv > limit ? limit : uv < -limit ? -limit : uv;
      gv = gv > limit ? limit : gv;
    }
    float t = silu_f(gv) * uv;
    if (wroute >= 0.f) t = wroute * t;
    xf[i] = bf16r(t);
    if (h_out) h_out[i] = xf[i];
  }
  orc_act_quant(xf, I, q, s);
  if (mx) mx4_gemv(q, s, wd, (const uint8_t*)sd, H, I, y, 1);
  else fp8_gemv(q, s, wd, (const float*)sd, H, I, y, 1);
  free(xf), free(q), free(s), free(g), free(u);
}
ORC_API void orc_fp8_expert_row(const uint16_t* x, int H, int I, const uint8_t* wg, const float* sg, const uint8_t* wu,
                                const float* su, const uint8_t* wd, const float* sd, float wroute, float limit, float* y,
                                float* h_out) {
  expert_row(0, x, H, I, wg, sg, wu, su, wd, sd, wroute, limit, y, h_out);
}
ORC_API void orc_mx4_expert_row(const uint16_t* x, int H, int I, const uint8_t* wg, const uint8_t* sg, const uint8_t* wu,
                                const uint8_t* su, const uint8_t* wd, const uint8_t* sd, float wroute, float limit, float* y,
                                float* h_out) {
  expert_row(1, x, H, I, wg, sg, wu, su, wd, sd, wroute, limit, y, h_out);
}

/* A whole FP8 layer (model.py:889-904).  Expert e's canonical tensors: wg[e], wu[e] e4m3 [I][H] with scales
 * sg[e], su[e] f32 [I/128][H/128]; wd[e] [H][I], sd[e] [H/128][I/128].  Index E is the shared expert (pointers may be
 * NULL: no shared expert).  Only experts in [e_lo, e_hi) are computed (an expert-parallel rank's share); the shared
 * expert is added when with_shared.  acc [T][H] f32 (before the final rounding), out [T][H] bf16 (may be NULL).
 * limit: the SwiGLU clamp of orc_fp8_expert_row (0: none).  pickmax [T][H] (may be NULL): per element the largest
 * magnitude among the outputs that were added there (what one bf16 rounding flip of one of them can change). */
static int moe_layer(int mx, const uint16_t* x, const int32_t* idx, const float* w, int T, int H, int I, int E, int topk,
                     const uint8_t* const* wg, const void* const* sg, const uint8_t* const* wu, const void* const* su,
                     const uint8_t* const* wd, const void* const* sd, int e_lo, int e_hi, int with_shared, float limit,
                     float* acc, uint16_t* out, float* pickmax) {
  if (H % 128 || I % 128) return -1;
  lut_init();
  float* y = (float*)malloc(sizeof(float) * H);
  memset(acc, 0, sizeof(float) * (size_t)T * H);
  if (pickmax) memset(pickmax, 0, sizeof(float) * (size_t)T * H);
  for (int e = e_lo; e < e_hi; ++e) /* ascending expert id: each row's adds happen in that order */
    for (int t = 0; t < T; ++t)
      for (int j = 0; j < topk; ++j)
        if (idx[(size_t)t * topk + j] == e) {
          expert_row(mx, x + (size_t)t * H, H, I, wg[e], sg[e], wu[e], su[e], wd[e], sd[e], w[(size_t)t * topk + j], limit,
                     y, NULL);
          float* a = acc + (size_t)t * H;
          for (int n = 0; n < H; ++n) a[n] += y[n];
          if (pickmax)
            for (int n = 0; n < H; ++n) pickmax[(size_t)t * H + n] = fmaxf(pickmax[(size_t)t * H + n], fabsf(y[n]));
        }
  if (with_shared && wg[E])
    for (int t = 0; t < T; ++t) {
      expert_row(0, x + (size_t)t * H, H, I, wg[E], sg[E], wu[E], su[E], wd[E], sd[E], -1.f, limit, y, NULL); /* FP8 */
      float* a = acc + (size_t)t * H;
      for (int n = 0; n < H; ++n) a[n] += y[n];
      if (pickmax)
        for (int n = 0; n < H; ++n) pickmax[(size_t)t * H + n] = fmaxf(pickmax[(size_t)t * H + n], fabsf(y[n]));
    }
  if (out)
    for (size_t i = 0; i < (size_t)T * H; ++i) out[i] = orc_f32_to_bf16(acc[i]);
  free(y);
  return 0;
}

ORC_API int orc_moe_fp8_layer(const uint16_t* x, const int32_t* idx, const float* w, int T, int H, int I, int E,
                              int topk, const uint8_t* const* wg, const float* const* sg, const uint8_t* const* wu,
                              const float* const* su, const uint8_t* const* wd, const float* const* sd, int e_lo,
                              int e_hi, int with_shared, float limit, float* acc, uint16_t* out, float* pickmax) {
  return moe_layer(0, x, idx, w, T, H, I, E, topk, wg, (const void* const*)sg, wu, (const void* const*)su, wd,
                   (const void* const*)sd, e_lo, e_hi, with_shared, limit, acc, out, pickmax);
}
/* The same with MXFP4 routed experts (scale pointers: ue8m0 bytes) and an FP8 shared expert at index E (f32 scales): a
 * ds41f layer (model.py:872-887: routed experts in fp4, the shared expert in the default fp8). */
ORC_API int orc_moe_mx4_layer(const uint16_t* x, const int32_t* idx, const float* w, int T, int H, int I, int E,
                              int topk, const uint8_t* const* wg, const void* const* sg, const uint8_t* const* wu,
                              const void* const* su, const uint8_t* const* wd, const void* const* sd, int e_lo, int e_hi,
                              int with_shared, float limit, float* acc, uint16_t* out, float* pickmax) {
  return moe_layer(1, x, idx, w, T, H, I, E, topk, wg, sg, wu, su, wd, sd, e_lo, e_hi, with_shared, limit, acc, out, pickmax);
}

/* ------------------------------------------------------------------------------------------------- INT4-g32 FFN */

/* Canonical INT4 tensor (layout.h:24-31): wp bytes [N][K/2], value k of row n in byte k/2, low nibble = even k, the
 * stored nibble u = q + 8; s bf16 [N][K/32]; zp u32 [N/8][K/32], row n's zero-point nibble at bits 4 (n % 8), or NULL
 * for symmetric (u_z = 8).  W = bf16((u - u_z) * s), one rounding (formats.cuh:117-119; glmref.py:108-121). */
static inline float i4_value(const uint8_t* wp, const uint16_t* s, const uint32_t* zp, int K, int n, int k) {
  const int u = (wp[(size_t)n * (K / 2) + k / 2] >> (4 * (k & 1))) & 15;
  const int uz = zp ? (int)((zp[(size_t)(n / 8) * (K / 32) + k / 32] >> (4 * (n % 8))) & 15) : 8;
  return bf16r((float)(u - uz) * orc_bf16_to_f32(s[(size_t)n * (K / 32) + k / 32]));
}
ORC_API void orc_int4_dequant(const uint8_t* wp, const uint16_t* s, const uint32_t* zp, int N, int K, uint16_t* out) {
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) out[(size_t)n * K + k] = orc_f32_to_bf16(i4_value(wp, s, zp, K, n, k));
}

/* y[n] = sum_k x[k] W[n][k] over bf16 operands (exact f32 products), accumulated in double, rounded to f32 and, when
 * round_bf16, to bf16 (glmref.py:231-233 linear; :251-256 out_linear keeps f32). */
static void bf16w_gemv(const float* xf, const uint16_t* wb, int N, int K, float* y, int round_bf16) {
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const uint16_t* wr = wb + (size_t)n * K;
    double acc = 0.0;
    for (int k = 0; k < K; ++k) acc += (double)xf[k] * (double)orc_bf16_to_f32(wr[k]);
    y[n] = round_bf16 ? bf16r((float)acc) : (float)acc;
  }
}

/* One expert with bf16 weight values (an INT4 expert after orc_int4_dequant, or the bf16 shared expert) on one row:
 * g, u rounded to bf16; h = bf16(bf16(silu(g)) * u) (glmref.py:299-300 on bf16 tensors); y = f32 down (not rounded). */
ORC_API void orc_bf16w_expert_row(const uint16_t* x, int H, int I, const uint16_t* wg, const uint16_t* wu,
                                  const uint16_t* wd, float* y, float* h_out) {
  float* xf = (float*)malloc(sizeof(float) * (H > I ? H : I));
  float* g = (float*)malloc(sizeof(float) * I);
  float* u = (float*)malloc(sizeof(float) * I);
  for (int k = 0; k < H; ++k) xf[k] = orc_bf16_to_f32(x[k]);
  bf16w_gemv(xf, wg, I, H, g, 1);
  bf16w_gemv(xf, wu, I, H, u, 1);
  for (int i = 0; i < I; ++i) {
    xf[i] = bf16r(bf16r(silu_f(g[i])) * u[i]);
    if (h_out) h_out[i] = xf[i];
  }
  bf16w_gemv(xf, wd, H, I, y, 0);
  free(xf), free(g), free(u);
}

/* A whole INT4 layer (glmref.py:581-643): experts given dequantised (bf16 [I][H], [I][H], [H][I]); acc += y * w in
 * ascending expert id (:626-627), then the shared expert's f32 output (:633-634).  Pointers at index E: shared. */
ORC_API int orc_moe_bf16w_layer(const uint16_t* x, const int32_t* idx, const float* w, int T, int H, int I, int E,
                                int topk, const uint16_t* const* wg, const uint16_t* const* wu,
                                const uint16_t* const* wd, int e_lo, int e_hi, int with_shared, float* acc,
                                uint16_t* out) {
  float* y = (float*)malloc(sizeof(float) * H);
  memset(acc, 0, sizeof(float) * (size_t)T * H);
  for (int e = e_lo; e < e_hi; ++e)
    for (int t = 0; t < T; ++t)
      for (int j = 0; j < topk; ++j)
        if (idx[(size_t)t * topk + j] == e) {
          orc_bf16w_expert_row(x + (size_t)t * H, H, I, wg[e], wu[e], wd[e], y, NULL);
          const float we = w[(size_t)t * topk + j];
          float* a = acc + (size_t)t * H;
          for (int n = 0; n < H; ++n) a[n] += y[n] * we;
        }
  if (with_shared && wg[E])
    for (int t = 0; t < T; ++t) {
      orc_bf16w_expert_row(x + (size_t)t * H, H, I, wg[E], wu[E], wd[E], y, NULL);
      float* a = acc + (size_t)t * H;
      for (int n = 0; n < H; ++n) a[n] += y[n];
    }
  if (out)
    for (size_t i = 0; i < (size_t)T * H; ++i) out[i] = orc_f32_to_bf16(acc[i]);
  free(y);
  return 0;
}

/* ------------------------------------------------------------------------------------------------ engine layouts */

/* FP8 tile layout (layout.h:108-119): canonical e4m3 [N][K] -> [N/8][K/128][32 lanes][32 B]; lane l = 4 g + t holds
 * row 8 n8 + g, k = 128 j + 64 q + 16 t + i at byte 16 q + i. */
ORC_API void orc_pack_fp8_tile(const uint8_t* w, int N, int K, uint8_t* out) {
  const int J = K / 128;
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) {
      const int n8 = n >> 3, g = n & 7, j = k >> 7, q = (k >> 6) & 1, t = (k >> 4) & 3, i = k & 15;
      out[(((size_t)n8 * J + j) * 32 + 4 * g + t) * 32 + 16 * q + i] = w[(size_t)n * K + k];
    }
}
ORC_API void orc_unpack_fp8_tile(const uint8_t* m, int N, int K, uint8_t* out) {
  const int J = K / 128;
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) {
      const int n8 = n >> 3, g = n & 7, j = k >> 7, q = (k >> 6) & 1, t = (k >> 4) & 3, i = k & 15;
      out[(size_t)n * K + k] = m[(((size_t)n8 * J + j) * 32 + 4 * g + t) * 32 + 16 * q + i];
    }
}

/* INT4 block layout (layout.h:50-58, 78-95): blocks of 8 rows x 512 k, 2368 B, [N/8][K/512]:
 *   value bytes: unit jj (128 k) at 512 jj + 16 l, byte 8 q + i/2 = canonical byte of k0 = 512 b + 128 jj + 64 q + 16 t
 *   scale bf16 of group c = k0/32 at 2048 + 32 g + 16 (t>>1) + 2 (2 jj + q)
 *   zero-point nibble 2 jj + q of the u32 at 2304 + 8 g + 4 (t>>1) */
ORC_API void orc_pack_int4_block(const uint8_t* wp, const uint16_t* s, const uint32_t* zp, int N, int K, uint8_t* out) {
  const int B = K / 512;
  for (int n8 = 0; n8 < N / 8; ++n8)
    for (int b = 0; b < B; ++b) {
      uint8_t* blk = out + ((size_t)n8 * B + b) * 2368;
      memset(blk + 2304, 0, 64);
      for (int l = 0; l < 32; ++l) {
        const int g = l >> 2, t = l & 3, h = t >> 1, n = 8 * n8 + g;
        for (int jj = 0; jj < 4; ++jj)
          for (int q = 0; q < 2; ++q) {
            const int k0 = 512 * b + 128 * jj + 64 * q + 16 * t, c = k0 / 32, j = 2 * jj + q;
            memcpy(blk + 512 * jj + 16 * l + 8 * q, wp + (size_t)n * (K / 2) + k0 / 2, 8);
            memcpy(blk + 2048 + 32 * g + 16 * h + 2 * j, s + (size_t)n * (K / 32) + c, 2);
            if (t == 2 * h) {
              const int uz = zp ? (int)((zp[(size_t)(n / 8) * (K / 32) + c] >> (4 * (n % 8))) & 15) : 8;
              blk[2304 + 8 * g + 4 * h + j / 2] |= (uint8_t)(uz << (4 * (j & 1)));
            }
          }
      }
    }
}
/* the bf16 contract value of (n, k) read back from packed blocks */
ORC_API uint16_t orc_read_int4_block(const uint8_t* m, int K, int n, int k) {
  const int B = K / 512, n8 = n / 8, g = n % 8, b = k / 512, jj = (k / 128) % 4, q = (k / 64) % 2, t = (k / 16) % 4,
            i = k % 16, l = 4 * g + t, h = t >> 1, j = 2 * jj + q;
  const uint8_t* blk = m + ((size_t)n8 * B + b) * 2368;
  const int u = (blk[512 * jj + 16 * l + 8 * q + i / 2] >> (4 * (i & 1))) & 15;
  uint16_t s;
  memcpy(&s, blk + 2048 + 32 * g + 16 * h + 2 * j, 2);
  const int uz = (blk[2304 + 8 * g + 4 * h + j / 2] >> (4 * (j & 1))) & 15;
  return orc_f32_to_bf16((float)(u - uz) * orc_bf16_to_f32(s));
}
/* bf16 tile layout of the shared expert ([N/8][K/128] blocks of 2048 B; layout.h:96-107): the lane's 16 B at
 * 512 p + 16 l are k = 128 b + 64 (p >> 1) + 16 t + 8 (p & 1) + 0..7 */
ORC_API void orc_pack_bf16_tile(const uint16_t* w, int N, int K, uint8_t* out) {
  const int B = K / 128;
  for (int n8 = 0; n8 < N / 8; ++n8)
    for (int b = 0; b < B; ++b) {
      uint8_t* blk = out + ((size_t)n8 * B + b) * 2048;
      for (int l = 0; l < 32; ++l) {
        const int g = l >> 2, t = l & 3, n = 8 * n8 + g;
        for (int p = 0; p < 4; ++p)
          memcpy(blk + 512 * p + 16 * l, w + (size_t)n * K + 128 * b + 64 * (p >> 1) + 16 * t + 8 * (p & 1), 16);
      }
    }
}

/* the thread count of the parallel loops (a launcher may have exported OMP_NUM_THREADS=1) */
ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
