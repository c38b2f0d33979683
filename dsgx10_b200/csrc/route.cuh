// The routing function of one row by one warp, shared by the standalone route kernel and the decode step's fused
// route + union kernel: the same code, so the same bits.  IEEE operations only (explicit fmas, correctly rounded
// divisions), which a CPU reproduces exactly.
#pragma once
#include "common.cuh"
#include "kernels.h"

namespace dsgx {

// e^x: n = rint(x log2 e), r = x - n ln 2 in two fused steps, a degree-7 Taylor polynomial in Horner form, an exact
// scaling by 2^n (n in [-126, 127] for the callers' ranges).
DSGX_DEV float exp_ieee(float x) {
  const float n = rintf(__fmul_rn(x, 1.44269504f));
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
  return __fmul_rn(p, __int_as_float(((int)n + 127) << 23));
}
DSGX_DEV float route_sigmoid(float l) {
  const float x = -l;
  if (x > 88.f) return 0.f;
  if (x < -87.f) return 1.f;
  return __fdiv_rn(1.f, __fadd_rn(1.f, exp_ieee(x)));
}

// ln(y) for y in [1, 2^31) with IEEE operations only (a CPU repeats the bits): y = 2^n m, m in [1/sqrt2, sqrt2),
// s = (m - 1) / (m + 1), ln m = 2 s (1 + z/3 + z^2/5 + z^3/7 + z^4/9 + z^5/11), z = s^2; ln y = n ln2_hi + (n ln2_lo + ln m).
DSGX_DEV float log_ieee(float y) {
  uint32_t u = __float_as_uint(y);
  int n = (int)(u >> 23) - 127;
  float m = __uint_as_float((u & 0x007FFFFFu) | 0x3F800000u);
  if (m > 1.41421356f) m = __fmul_rn(m, 0.5f), n += 1;
  const float f = __fsub_rn(m, 1.f);
  const float sv = __fdiv_rn(f, __fadd_rn(2.f, f));
  const float z = __fmul_rn(sv, sv);
  float p = 1.f / 11;
  p = fmaf(p, z, 1.f / 9);
  p = fmaf(p, z, 1.f / 7);
  p = fmaf(p, z, 1.f / 5);
  p = fmaf(p, z, 1.f / 3);
  p = fmaf(p, z, 1.f);
  const float lm = __fmul_rn(__fmul_rn(2.f, sv), p);
  const float nf = (float)n;
  return fmaf(nf, 0.693145751953125f, fmaf(nf, 1.428606765330187e-06f, lm));
}
// sqrt(softplus(l)), torch's softplus (l > 20 ? l : log1p(exp(l))): the score of ds41f's router
// (engine/kernels/common.cuh:264-287).  log1p(t) = ln(y) t / (y - 1) with y = fl(1 + t), t itself when y == 1.
DSGX_DEV float route_sqrtsoftplus(float l) {
  float sp;
  if (l > 20.f) {
    sp = l;
  } else if (l < -87.f) {
    sp = 0.f;
  } else {
    const float t = exp_ieee(l);
    const float y = __fadd_rn(1.f, t);
    const float d = __fsub_rn(y, 1.f);
    sp = d == 0.f ? t : __fdiv_rn(__fmul_rn(log_ieee(y), t), d);
  }
  return __fsqrt_rn(sp);
}
DSGX_DEV float route_score1(int score_fn, float l) { return score_fn == DSGX_SCORE_SIGMOID ? route_sigmoid(l) : route_sqrtsoftplus(l); }

constexpr int kRJ = 16;  // experts a lane: E <= 512

// One row.  Expert e = lane + 32 j.  The row's logit of expert e is the sum, in ascending s, of nsplit partial sums
// l[s * split_stride + e] (nsplit = 1: plain logits).  Lane k < topk ends with pick k in (id_out, w_out); when
// logits_out is given, the summed logits are stored there.
DSGX_DEV void route_row(const RouteParams& p, const float* __restrict__ l, int nsplit, size_t split_stride,
                        const float* __restrict__ bias, int lane, int& id_out, float& w_out, float* logits_out) {
  float s[kRJ], key[kRJ];
  // every load before any math: one round trip (up to four slices of partial sums at a time, added in ascending order)
#pragma unroll
  for (int j = 0; j < kRJ; ++j) {
    const int e = lane + 32 * j;
    s[j] = e < p.E ? (nsplit ? __ldcg(l + e) : l[e]) : -INFINITY;  // (nsplit 0: summed logits behind a plain pointer)
    key[j] = e < p.E && bias ? __ldg(bias + e) : 0.f;
  }
  for (int sp0 = 1; sp0 < nsplit; sp0 += 3) {
    float part[3][kRJ];
#pragma unroll
    for (int q = 0; q < 3; ++q)
#pragma unroll
      for (int j = 0; j < kRJ; ++j) {
        const int e = lane + 32 * j;
        part[q][j] = sp0 + q < nsplit && e < p.E ? __ldcg(l + (sp0 + q) * split_stride + e) : 0.f;
      }
#pragma unroll
    for (int q = 0; q < 3; ++q)
      if (sp0 + q < nsplit) {
#pragma unroll
        for (int j = 0; j < kRJ; ++j)
          if (lane + 32 * j < p.E) s[j] = __fadd_rn(s[j], part[q][j]);
      }
  }
  if (logits_out) {
#pragma unroll
    for (int j = 0; j < kRJ; ++j)
      if (lane + 32 * j < p.E) logits_out[lane + 32 * j] = s[j];
  }
  if (p.score_fn != DSGX_SCORE_SOFTMAX) {
#pragma unroll
    for (int j = 0; j < kRJ; ++j) s[j] = lane + 32 * j < p.E ? route_score1(p.score_fn, s[j]) : 0.f;
  } else {  // softmax: t = exp(l - max), lane sums over j ascending, butterfly, one division each
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < kRJ; ++j) m = fmaxf(m, s[j]);
    m = warp_max(m);
    float ps = 0.f;
#pragma unroll
    for (int j = 0; j < kRJ; ++j) {
      if (lane + 32 * j < p.E) {
        const float d = __fsub_rn(s[j], m);
        s[j] = d < -87.f ? 0.f : exp_ieee(d);
        ps = __fadd_rn(ps, s[j]);
      } else {
        s[j] = 0.f;
      }
    }
    const float S = warp_sum(ps);
#pragma unroll
    for (int j = 0; j < kRJ; ++j) s[j] = __fdiv_rn(s[j], S);
  }
#pragma unroll
  for (int j = 0; j < kRJ; ++j) key[j] = lane + 32 * j < p.E ? __fadd_rn(s[j], key[j]) : -INFINITY;

  if (p.n_group > 1) {
    // group score = the sum of the group's two largest keys; keep the topk_group best groups (ties: lower id)
    const int gs = p.E / p.n_group;
    float mine = -INFINITY;  // lane g < n_group holds group g's score
    for (int g = 0; g < p.n_group; ++g) {
      float a = -INFINITY, b = -INFINITY;
#pragma unroll
      for (int j = 0; j < kRJ; ++j) {
        const int e = lane + 32 * j;
        if (e < p.E && e / gs == g) {
          const float v = key[j];
          if (v > a) b = a, a = v;
          else if (v > b) b = v;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, a, o), ob = __shfl_xor_sync(0xffffffffu, b, o);
        const float na = fmaxf(a, oa), nb = fmaxf(fminf(a, oa), fmaxf(b, ob));
        a = na, b = nb;
      }
      if (lane == g) mine = __fadd_rn(a, b);
    }
    uint32_t keep = 0;
    for (int t = 0; t < p.topk_group; ++t) {
      float bv = lane < p.n_group && !((keep >> lane) & 1) ? mine : -INFINITY;
      int bg = lane < p.n_group && !((keep >> lane) & 1) ? lane : 1 << 30;
      if (bv != bv) bv = -INFINITY;  // a NaN score never wins
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int og = __shfl_xor_sync(0xffffffffu, bg, o);
        if (og < (1 << 30) && (bg == (1 << 30) || ov > bv || (ov == bv && og < bg))) bv = ov, bg = og;
      }
      if (bg < 32) keep |= 1u << bg;
    }
#pragma unroll
    for (int j = 0; j < kRJ; ++j) {
      const int e = lane + 32 * j;
      if (e < p.E && !((keep >> (e / gs)) & 1)) key[j] = -INFINITY;
    }
  }

  // The picks.  The keys become order-preserving integers once (a NaN and a key that is out of the running rank as -inf,
  // -0 as +0); every round each lane offers its largest, the warp takes the maximum, then the lowest expert id among the
  // lanes that hold it (ties go to the lower id), and that expert leaves the running.
  constexpr uint32_t kGone = 0x007FFFFFu;  // ord(-inf)
  uint32_t ok[kRJ];
#pragma unroll
  for (int j = 0; j < kRJ; ++j) {
    const float f = __fadd_rn(key[j], 0.f);
    const uint32_t b = __float_as_uint(f);
    ok[j] = f != f ? kGone : (b & 0x80000000u) ? ~b : b | 0x80000000u;
  }
  float picked[8];
  int ids[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    picked[k] = 0.f, ids[k] = 0;
    if (k < p.topk) {
      uint32_t mine = kGone;
#pragma unroll
      for (int j = 0; j < kRJ; ++j) mine = max(mine, ok[j]);
      const uint32_t top = __reduce_max_sync(0xffffffffu, mine);
      int cand = 1 << 30;
#pragma unroll
      for (int j = kRJ - 1; j >= 0; --j)
        if (ok[j] == top) cand = lane + 32 * j;
      int e = top == kGone ? 0 : (int)__reduce_min_sync(0xffffffffu, (unsigned)cand);  // (nothing left: expert 0)
      ids[k] = e;
      float sv = 0.f;
#pragma unroll
      for (int j = 0; j < kRJ; ++j)
        if (lane + 32 * j == e) sv = s[j], ok[j] = kGone;
      picked[k] = __shfl_sync(0xffffffffu, sv, e & 31);
    }
  }
  // the sum of the picked scores: four running sums at stride 4, then (t0 + t2) + (t1 + t3)
  float t[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) t[j] = j < p.topk ? picked[j] : 0.f;
#pragma unroll
  for (int i = 4; i < 8; ++i)
    if (i < p.topk) t[i & 3] = __fadd_rn(t[i & 3], picked[i]);
  float sum;
  if (p.topk <= 1) sum = t[0];
  else if (p.topk == 2) sum = __fadd_rn(t[0], t[1]);
  else if (p.topk == 3) sum = __fadd_rn(__fadd_rn(t[0], t[2]), t[1]);
  else sum = __fadd_rn(__fadd_rn(t[0], t[2]), __fadd_rn(t[1], t[3]));
  sum = __fadd_rn(sum, 1e-20f);
  id_out = 0, w_out = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k)
    if (k < p.topk && lane == k) {
      id_out = ids[k];
      w_out = p.norm_topk ? __fmul_rn(__fdiv_rn(picked[k], sum), p.route_scale) : __fmul_rn(picked[k], p.route_scale);
    }
}

}  // namespace dsgx

namespace dsgx {

// ---- the same routing function by one whole CTA (blockDim.x = E rounded up to 32, at least 32) ------------------------
// For decode widths the routing is a chain of dependent steps, so the scores are computed one thread an expert (all
// slice loads in one round trip), and one warp then selects from shared memory with the keys in registers: no block-wide
// barrier inside the pick loop.  Comparisons are exact and every sum keeps the order of route_row: the same bits.
// float -> unsigned with the same order (and back); 0 is below every float
DSGX_DEV uint32_t ord_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
DSGX_DEV float ord_float(uint32_t u) { return __uint_as_float((u & 0x80000000u) ? (u ^ 0x80000000u) : ~u); }

struct __align__(16) RouteSmem {
  float key[512];
  float s[512];
  float red[16];
  float gsc[32];
  float S;
  uint32_t keep;
  uint32_t pad[2];
  uint32_t ck[128];  // the warps' best candidates: ordered keys ...
  int ci[128];       // ... and their expert ids (8 a warp)
};

// nsplit 0: l is this thread's summed logit itself (l points at it); cp: the threads that take part (threadIdx.x < cp.nt).
DSGX_DEV void route_row_cta(const RouteParams& p, const float* __restrict__ l, int nsplit, size_t split_stride,
                            const float* __restrict__ bias, RouteSmem& sm, float* logits_out, int* idx_out, float* w_out,
                            int* idx_copy = nullptr, float* w_copy = nullptr, CtaPart cp = CtaPart{0, 0}) {
  if (cp.nt == 0) cp = whole_cta();
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5, nW = cp.nt >> 5;
  const bool valid = e < p.E;
  float lg = -INFINITY, b = 0.f;
  if (valid && nsplit == 0) {
    lg = *l;
    if (bias) b = __ldg(bias + e);
    if (logits_out) logits_out[e] = lg;
  } else if (valid) {
    float part[8];
#pragma unroll
    for (int sp = 0; sp < 8; ++sp) part[sp] = sp < nsplit ? __ldcg(l + sp * split_stride + e) : 0.f;
    if (bias) b = __ldg(bias + e);
    lg = part[0];
#pragma unroll
    for (int sp = 1; sp < 8; ++sp)
      if (sp < nsplit) lg = __fadd_rn(lg, part[sp]);
    for (int sp = 8; sp < nsplit; ++sp) lg = __fadd_rn(lg, __ldcg(l + sp * split_stride + e));
    if (logits_out) logits_out[e] = lg;
  }
  float s;
  if (p.score_fn != DSGX_SCORE_SOFTMAX) {
    s = valid ? route_score1(p.score_fn, lg) : 0.f;
  } else {
    float m = warp_max(lg);
    if (lane == 0) sm.red[warp] = m;
    cp.sync();
    m = sm.red[0];
    for (int w = 1; w < nW; ++w) m = fmaxf(m, sm.red[w]);
    float t = 0.f;
    if (valid) {
      const float d = __fsub_rn(lg, m);
      t = d < -87.f ? 0.f : exp_ieee(d);
    }
    sm.key[e] = t;
    cp.sync();
    if (warp == 0) {  // lane sums over j ascending, then the butterfly
      float ps = 0.f;
      for (int ee = lane; ee < p.E; ee += 32) ps = __fadd_rn(ps, sm.key[ee]);
      ps = warp_sum(ps);
      if (lane == 0) sm.S = ps;
    }
    cp.sync();
    s = __fdiv_rn(t, sm.S);
    cp.sync();
  }
  // keys as order-preserving unsigned integers in shared memory (0 = not a candidate)
  uint32_t* ku = reinterpret_cast<uint32_t*>(sm.key);
  sm.s[e] = s;
  cp.sync();  // (softmax read sm.key above)
  ku[e] = valid ? ord_key(__fadd_rn(s, b)) : 0u;
  cp.sync();
  // ---- selection, all warps: group scores one warp a group, then every candidate ranks itself --------------------------
  float* picked = sm.red;  // [8] scores of the picks (sm.red is free by now)
  int* ids = reinterpret_cast<int*>(sm.red + 8);
  if (p.n_group > 1) {
    const int gs = p.E / p.n_group;
    uint32_t* gsc = reinterpret_cast<uint32_t*>(sm.gsc);
#pragma unroll 1
    for (int g = warp; g < p.n_group; g += nW) {  // the ordered sum of the group's two largest keys
      uint32_t lm = 0;
#pragma unroll 1
      for (int i = g * gs + lane; i < (g + 1) * gs; i += 32) lm = max(lm, ku[i]);
      const uint32_t m1 = __reduce_max_sync(0xffffffffu, lm);
      const uint32_t holder = __reduce_min_sync(0xffffffffu, lm == m1 ? (uint32_t)lane : 32u);
      uint32_t second = 0;  // the largest key left once one instance of m1 is taken out
      bool taken = lane != (int)holder;
#pragma unroll 1
      for (int i = g * gs + lane; i < (g + 1) * gs; i += 32) {
        const uint32_t v = ku[i];
        if (!taken && v == m1) taken = true;
        else second = max(second, v);
      }
      const uint32_t m2 = __reduce_max_sync(0xffffffffu, second);
      if (lane == 0) gsc[g] = ord_key(__fadd_rn(ord_float(m1), ord_float(m2)));
    }
    cp.sync();
    if (warp == 0) {  // keep the topk_group best groups, ties to the lower id
      const uint32_t mine = lane < p.n_group ? gsc[lane] : 0u;
      uint32_t keep = 0;
#pragma unroll 1
      for (int t = 0; t < p.topk_group; ++t) {
        const bool cand = lane < p.n_group && !((keep >> lane) & 1);
        const uint32_t m = __reduce_max_sync(0xffffffffu, cand ? mine : 0u);
        const uint32_t gsel = __reduce_min_sync(0xffffffffu, cand && mine == m ? (uint32_t)lane : 32u);
        if (gsel < 32) keep |= 1u << gsel;
      }
      if (lane == 0) sm.keep = keep;
    }
    cp.sync();
    if (valid && !((sm.keep >> (e / gs)) & 1)) ku[e] = 0u;
    cp.sync();
  }
  // The picks, in two levels.  Every warp takes the topk best of its 32 keys in order (a maximum over the warp, then the
  // lowest lane that holds it: ties go to the lower id), which contain every global pick; then each of those candidates
  // ranks itself among the candidates (keys above it + equal keys with a lower id): ranks 0 .. topk-1 are the picks in
  // order.  A few hundred instructions on the critical path instead of every candidate against every key.
  {
    uint32_t k = valid ? ku[e] : 0u;
    if (lane < 8) sm.ck[warp * 8 + lane] = 0u, sm.ci[warp * 8 + lane] = 0;
    __syncwarp();
#pragma unroll 1
    for (int r = 0; r < p.topk; ++r) {
      const uint32_t m = __reduce_max_sync(0xffffffffu, k);
      if (m == 0u) break;  // (no candidate left in this warp)
      const uint32_t holder = __reduce_min_sync(0xffffffffu, k == m ? (uint32_t)lane : 32u);
      if (lane == 0) sm.ck[warp * 8 + r] = m, sm.ci[warp * 8 + r] = warp * 32 + (int)holder;
      if ((uint32_t)lane == holder) k = 0u;
    }
  }
  cp.sync();
  const int nC = nW * 8;
  if (e < nC) {
    const uint32_t mine = sm.ck[e];
    if (mine) {
      const int myid = sm.ci[e];
      int rank = 0;
      const uint4* k4 = reinterpret_cast<const uint4*>(sm.ck);
      const int4* i4 = reinterpret_cast<const int4*>(sm.ci);
#pragma unroll 4
      for (int q = 0; q < (nC >> 2); ++q) {
        const uint4 v = k4[q];
        const int4 id = i4[q];
        rank += (v.x > mine) || (v.x == mine && id.x < myid);
        rank += (v.y > mine) || (v.y == mine && id.y < myid);
        rank += (v.z > mine) || (v.z == mine && id.z < myid);
        rank += (v.w > mine) || (v.w == mine && id.w < myid);
      }
      if (rank < p.topk) ids[rank] = myid, picked[rank] = sm.s[myid];
    }
  }
  cp.sync();
  if (warp != 0) return;
  // the sum of the picked scores: four running sums at stride 4, then (t0 + t2) + (t1 + t3)
  float t[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) t[j] = j < p.topk ? picked[j] : 0.f;
#pragma unroll 1
  for (int i = 4; i < p.topk; ++i) {
    const float v = picked[i];
    if ((i & 3) == 0) t[0] = __fadd_rn(t[0], v);
    else if ((i & 3) == 1) t[1] = __fadd_rn(t[1], v);
    else if ((i & 3) == 2) t[2] = __fadd_rn(t[2], v);
    else t[3] = __fadd_rn(t[3], v);
  }
  float sum;
  if (p.topk <= 1) sum = t[0];
  else if (p.topk == 2) sum = __fadd_rn(t[0], t[1]);
  else if (p.topk == 3) sum = __fadd_rn(__fadd_rn(t[0], t[2]), t[1]);
  else sum = __fadd_rn(__fadd_rn(t[0], t[2]), __fadd_rn(t[1], t[3]));
  sum = __fadd_rn(sum, 1e-20f);
  if (lane < p.topk) {
    const float pk = picked[lane];
    const float wv = p.norm_topk ? __fmul_rn(__fdiv_rn(pk, sum), p.route_scale) : __fmul_rn(pk, p.route_scale);
    idx_out[lane] = ids[lane];
    w_out[lane] = wv;
    if (idx_copy) idx_copy[lane] = ids[lane], w_copy[lane] = wv;  // (a copy in shared memory for the caller's next step)
  }
}

}  // namespace dsgx
