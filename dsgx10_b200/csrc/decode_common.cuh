// Pieces the decode kernels of every format share: the slot table (the sorted union of a step's picked experts, plus
// the shared expert) and the per-warp weight-streaming ring.
#pragma once
#include "common.cuh"
#include "kernels.h"

namespace dsgx {

// The slot table of a step, built once by one CTA and read by every CTA of the expert kernels.
// Slots 0 .. nslots-1: the picked experts this GPU owns, ascending id; slot nslots: the shared expert (if any).
// A row that did not pick a slot's expert has weight 0 there.  Size a multiple of 16 bytes (bulk-copied).
struct alignas(16) SlotEnt {
  const uint8_t *g, *u, *d;      // gate, up, down blocks
  const float *sg, *su, *sd;     // FP8: their f32 block scales
  float w[8];                    // the rows' routing weights
  int e;                         // expert id (-1: the shared expert)
  int pad[3];
};
struct alignas(16) SlotTab {
  int nslots;  // routed slots
  int ntot;    // + the shared expert's
  int bad;     // a dsgx_status when the picks or descriptors were refused (the routed work is then dropped)
  int bgu;     // 1: the bf16 shared expert's gate and up rows are interleaved in one matrix (ent.g; ent.u one tile on)
  SlotEnt ent[kMaxSlots + 1];
};
static_assert(sizeof(SlotEnt) == 96 && sizeof(SlotTab) % 16 == 0, "SlotTab is copied in 16-byte pieces");

// Builds the table in shared memory from the step's picks (idx, w: M x topk, shared or global memory), by one whole CTA.
// bm: 16 words of shared memory.
// The descriptor fields the table needs, of every expert, fetched into shared memory ahead of the selection (so that the
// table costs no dependent round trip to memory once the picks are known).
struct DescCache {
  uint64_t off[3][512];   // MatDesc.off
  uint64_t soff[3][512];  // FP8: the scales' offset
  uint32_t fmt[3][512];
};
struct DescRegs {
  uint4 a[3];
  uint2 b[3];
};
// thread e: its expert's three descriptors into registers (experts this GPU does not own are not read) ...
DSGX_DEV void desc_fetch(DescRegs& r, const dsgx_mat_desc* desc, int e, bool owned) {
#pragma unroll
  for (int m = 0; m < 3; ++m) {
    r.a[m] = make_uint4(0, 0, 0, 0), r.b[m] = make_uint2(0, 0);
    if (owned) {
      const uint8_t* d = reinterpret_cast<const uint8_t*>(desc + (size_t)e * 3 + m);
      r.a[m] = __ldg(reinterpret_cast<const uint4*>(d));
      r.b[m] = __ldg(reinterpret_cast<const uint2*>(d + 16));
    }
  }
}
// ... and from there into the cache
DSGX_DEV void desc_store(DescCache& dc, const DescRegs& r, int e) {
#pragma unroll
  for (int m = 0; m < 3; ++m) {
    dc.off[m][e] = (uint64_t)r.a[m].x | (uint64_t)r.a[m].y << 32;
    dc.fmt[m][e] = r.a[m].w;
    dc.soff[m][e] = (uint64_t)r.b[m].x | (uint64_t)r.b[m].y << 32;
  }
}

DSGX_DEV void build_slot_tab(SlotTab& tab, uint32_t* bm, const int* idx, const float* w, int M, int topk, int E, int e_lo,
                             int e_hi, const uint8_t* pool, const dsgx_mat_desc* desc, const dsgx_shared_w& sh,
                             uint32_t fmt, const DescCache* dc = nullptr, CtaPart cp = CtaPart{0, 0}) {
  if (cp.nt == 0) cp = whole_cta();
  const int tid = threadIdx.x, nt = cp.nt;
  if (tid < 16) bm[tid] = 0;
  if (tid == 0) tab.bad = 0, tab.bgu = 0;
  for (int i = tid; i < (kMaxSlots + 1) * 8; i += nt) tab.ent[i >> 3].w[i & 7] = 0.f;
  cp.sync();
  const int np = M * topk;
  for (int i = tid; i < np; i += nt) {
    const int e = idx[i];
    if (e < 0 || e >= E) tab.bad = DSGX_ERR_ARG;
    else if (e >= e_lo && e < e_hi) atomicOr(&bm[e >> 5], 1u << (e & 31));
  }
  cp.sync();
  auto rank_of = [&](int e) {
    int r = __popc(bm[e >> 5] & ((1u << (e & 31)) - 1u));
    for (int k = 0; k < (e >> 5); ++k) r += __popc(bm[k]);
    return r;
  };
  // one thread a pick: the pick's expert (a slot may be written by several rows' threads with the same values)
  for (int i = tid; i < np; i += nt) {
    const int e = idx[i];
    if (e < 0 || e >= E || e < e_lo || e >= e_hi) continue;
    const int s = rank_of(e);
    SlotEnt& en = tab.ent[s];
    en.w[i / topk] = w[i];
    const dsgx_mat_desc* d = desc + (size_t)e * 3;
    uint64_t o[3], so[3];
    bool fmt_ok = true;
#pragma unroll
    for (int m = 0; m < 3; ++m) {
      if (dc) {
        o[m] = dc->off[m][e], so[m] = dc->soff[m][e], fmt_ok = fmt_ok && dc->fmt[m][e] == fmt;
      } else {
        o[m] = d[m].off, so[m] = (uint64_t)d[m].rsv[0] | (uint64_t)d[m].rsv[1] << 32, fmt_ok = fmt_ok && d[m].fmt == fmt;
      }
    }
    if (!fmt_ok) tab.bad = DSGX_ERR_FORMAT;
    en.e = e;
    en.g = pool + o[0], en.u = pool + o[1], en.d = pool + o[2];
    if (fmt == DSGX_FMT_FP8) {  // (MXFP4 blocks carry their scales)
      en.sg = reinterpret_cast<const float*>(pool + so[0]);
      en.su = reinterpret_cast<const float*>(pool + so[1]);
      en.sd = reinterpret_cast<const float*>(pool + so[2]);
    } else {
      en.sg = en.su = en.sd = nullptr;
    }
  }
  cp.sync();
  if (tid == 0) {
    int n = 0;
    for (int k = 0; k < 16; ++k) n += __popc(bm[k]);
    if (tab.bad) n = 0;  // refuse the routed work, keep the kernels well-defined
    const bool has_sh = fmt_fp8_family(fmt) ? sh.g != nullptr : (sh.bg != nullptr || sh.bgu != nullptr);
    tab.nslots = n, tab.ntot = n + (has_sh ? 1 : 0);
    if (has_sh) {
      SlotEnt& en = tab.ent[n];
      en.e = -1;
#pragma unroll
      for (int r = 0; r < 8; ++r) en.w[r] = 0.f;
      if (fmt_fp8_family(fmt)) {
        en.g = sh.g, en.u = sh.u, en.d = sh.d, en.sg = sh.gs, en.su = sh.us, en.sd = sh.ds;
      } else {
        en.g = sh.bg ? sh.bg : sh.bgu, en.u = sh.bu, en.d = sh.bd, en.sg = en.su = en.sd = nullptr;
        tab.bgu = sh.bg ? 0 : 1;
      }
    }
  }
  cp.sync();
}

// The table from global memory into shared memory by one warp, in as few round trips as its size allows: the header
// and the first 15 slots together, the rest (wide steps only) after.
DSGX_DEV void load_slot_tab(SlotTab& dst, const SlotTab* src, int lane) {
  const uint4* s4 = reinterpret_cast<const uint4*>(src);
  uint4* d4 = reinterpret_cast<uint4*>(&dst);
  constexpr int kFirst = 1 + 15 * 6;  // header + 15 entries, 16-byte pieces (91: three per lane)
  uint4 v[3];
#pragma unroll
  for (int i = 0; i < 3; ++i) v[i] = lane + 32 * i < kFirst ? __ldcg(s4 + lane + 32 * i) : make_uint4(0, 0, 0, 0);
#pragma unroll
  for (int i = 0; i < 3; ++i)
    if (lane + 32 * i < kFirst) d4[lane + 32 * i] = v[i];
  __syncwarp();
  const int ntot = dst.ntot;
  if (ntot > 15) {
    const int total = 1 + ntot * 6;
    for (int i = kFirst + lane; i < total; i += 128) {
      uint4 u[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) u[k] = i + 32 * k < total ? __ldcg(s4 + i + 32 * k) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (i + 32 * k < total) d4[i + 32 * k] = u[k];
    }
  }
}

// order position -> slot: the shared expert's units come first (they are the same every step)
DSGX_DEV int ord_slot(const SlotTab& tab, int ord) {
  return tab.ntot > tab.nslots ? (ord == 0 ? tab.nslots : ord - 1) : ord;
}

DSGX_DEV uint4 lds128(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }

// ---- MXFP4 (e2m1 values, a ue8m0 scale per 32 k) ---------------------------------------------------------------------
DSGX_DEV uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
// Eight e2m1 values of one stored word -> the same values as e4m3 bytes (every e2m1 value is an e4m3 value): lo = values
// 0..3, hi = values 4..7.  Stored word: value j's magnitude code (0, .5, 1, 1.5, 2, 3, 4, 6) in bits 4 j .. 4 j + 2; the
// sign of value i < 4 in bit 8 i + 7, of value i >= 4 in bit 8 (i - 4) + 3 (the top bits of the odd and the even nibbles):
// where the e4m3 sign bits of lo lie, and four bits below those of hi.  Magnitudes by a byte table (prmt).
DSGX_DEV void e2m1x8_to_e4m3(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t m = w & 0x77777777u;
  lo = prmt(0x3C383000u, 0x4C484440u, m) | (w & 0x80808080u);
  hi = prmt(0x3C383000u, 0x4C484440u, m >> 16) | ((w << 4) & 0x80808080u);
}
// D = A B with a zero C operand (no accumulator to clear)
DSGX_DEV void mma_e4m3_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
// One 128-k block of two MXFP4 strips (A rows 0-7 from a, rows 8-15 from b) against an FP8 activation block: four MMAs of
// 32 k (one scale group each; k = 32 G + 8 t + 0..7 in lane (g, t)), each promoted with its rows' scales:
// d = ((d_0 s_0 + d_1 s_1) + d_2 s_2) + d_3 s_3 by fused multiply-adds from zero.  The scales are stored as bf16 (2^(e-127)
// exactly, e = 0 included), one shift or mask from a float.  (Measured on the way: the legacy mma.sync is the scarce
// resource here, a second MMA a group for the negative values cost more than the sign handling it saved.)
DSGX_DEV void block_mma_mx(float (&d)[4], const uint8_t* a, const uint8_t* b, const uint8_t* act, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const uint4 aw = lds128(a + 16 * lane), bw = lds128(b + 16 * lane);
  const uint2 sa = *reinterpret_cast<const uint2*>(a + 512 + 8 * g), sb = *reinterpret_cast<const uint2*>(b + 512 + 8 * g);
  // the activations of row g at k = 32 G + 8 t .. + 7: block position (k / 64, row, (k / 16) % 4, k % 16)
  const uint8_t* xr = act + (4 * g + (t >> 1)) * 16 + 8 * (t & 1);
  const uint2 x0 = *reinterpret_cast<const uint2*>(xr), x1 = *reinterpret_cast<const uint2*>(xr + 32);
  const uint2 x2 = *reinterpret_cast<const uint2*>(xr + 512), x3 = *reinterpret_cast<const uint2*>(xr + 544);
  d[0] = d[1] = d[2] = d[3] = 0.f;
  auto group = [&](uint32_t wa, uint32_t wb, const uint2& x, float fa, float fb) {
    uint32_t al, ah, bl, bh;
    e2m1x8_to_e4m3(wa, al, ah), e2m1x8_to_e4m3(wb, bl, bh);
    float e[4];
    mma_e4m3_zero(e, al, bl, ah, bh, x.x, x.y);
    d[0] = fmaf(e[0], fa, d[0]), d[1] = fmaf(e[1], fa, d[1]), d[2] = fmaf(e[2], fb, d[2]), d[3] = fmaf(e[3], fb, d[3]);
  };
  group(aw.x, bw.x, x0, __uint_as_float(sa.x << 16), __uint_as_float(sb.x << 16));
  group(aw.y, bw.y, x1, __uint_as_float(sa.x & 0xffff0000u), __uint_as_float(sb.x & 0xffff0000u));
  group(aw.z, bw.z, x2, __uint_as_float(sa.y << 16), __uint_as_float(sb.y << 16));
  group(aw.w, bw.w, x3, __uint_as_float(sa.y & 0xffff0000u), __uint_as_float(sb.y & 0xffff0000u));
}

// ---- the summation order of a unit's K, and its split over warps --------------------------------------------------
// A unit's sum over K is formed in pieces of kPB 128-k blocks: inside a piece the blocks' promoted partial sums are
// accumulated by fma from zero, ascending; the pieces are then added ascending, starting from the first piece's sum.
// That order is the same whether one warp runs all pieces of a unit or several warps (on different SMs) take
// consecutive runs of pieces and the last one to finish adds the piece sums it finds in the workspace: a row's bits do
// not depend on how a launch's pieces were dealt to the warps (the reference splits K over the warps of one CTA with one fixed
// split per format for the same reason: altar1 engine/experts/decode.cu:117-408, docs/experts.md:29-32).
// How many warps share a unit: the largest power of two that still leaves every run a warp of its own.
DSGX_DEV int pick_split(int units, int NP, int GW, int cap_units) {
  int s = 1;
  while (s * 2 <= NP && s * 2 <= kMaxPieces && units * s * 2 <= GW) s *= 2;
  return units > cap_units ? 1 : s;
}
DSGX_DEV bool piece_end(int kb, int KB) { return (kb % kPB) == kPB - 1 || kb == KB - 1; }
// folds a finished piece's sums into the totals (`first`: the unit's first piece) and clears them
DSGX_DEV void piece_fold(float (&tot)[4], float (&pc)[4], bool first) {
#pragma unroll
  for (int i = 0; i < 4; ++i) tot[i] = first ? pc[i] : __fadd_rn(tot[i], pc[i]), pc[i] = 0.f;
}

// ---- compact activation blocks (R = 1, 2, 4 or 8 rows), global-counter polls, the FP8 block product --------------------
// compact activation block of R rows x 128 k: [2 halves q][R rows][4 t][16 B] e4m3, then R f32 scales (padded to 16 B)
__host__ __device__ constexpr int cblk_bytes(int R) { return R * 128 + (R <= 4 ? 16 : 32); }

DSGX_DEV unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
DSGX_DEV int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// bounded poll until *p >= target
DSGX_DEV bool poll_ge(const int* p, int target) {
  if (ld_acquire(p) >= target) return true;
  const long long t0 = clock64();
  while (ld_acquire(p) < target) {
    __nanosleep(128);
    if (clock64() - t0 > kWaitCycles) return false;
  }
  return true;
}

// one row's 128 values (4 per lane) -> compact block
DSGX_DEV void cquant_row(uint8_t* blk, int R, int r, int lane, bool valid, float v0, float v1, float v2, float v3) {
  const int kl = 4 * lane, q = kl >> 6, t = (kl >> 4) & 3, i = kl & 15;
  uint32_t packed = 0;
  float sc = 0.f;
  if (valid) {
    sc = act_scale(warp_max(fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)))));
    packed = quant_e4m3(v0, sc) | quant_e4m3(v1, sc) << 8 | quant_e4m3(v2, sc) << 16 | quant_e4m3(v3, sc) << 24;
  }
  *reinterpret_cast<uint32_t*>(blk + ((q * R + r) * 4 + t) * 16 + i) = packed;
  if (lane == 0) reinterpret_cast<float*>(blk + R * 128)[r] = sc;
}

// One 128-k block: A rows 0-7 from strip a, rows 8-15 from strip b, B from a compact activation block.
DSGX_DEV void cblock_mma(float (&d)[4], const uint8_t* a, const uint8_t* b, const uint8_t* act, int R, int lane) {
  const uint4 a0 = lds128(a + 32 * lane), a1 = lds128(a + 32 * lane + 16);
  const uint4 b0 = lds128(b + 32 * lane), b1 = lds128(b + 32 * lane + 16);
  const int row = (lane >> 2) & (R - 1), t = lane & 3;
  const uint4 x0 = lds128(act + (row * 4 + t) * 16), x1 = lds128(act + ((R + row) * 4 + t) * 16);
  float e[4] = {0.f, 0.f, 0.f, 0.f};
  d[0] = d[1] = d[2] = d[3] = 0.f;
  mma_e4m3(d, a0.x, b0.x, a0.y, b0.y, x0.x, x0.y);
  mma_e4m3(e, a1.x, b1.x, a1.y, b1.y, x1.x, x1.y);
  mma_e4m3(d, a0.z, b0.z, a0.w, b0.w, x0.z, x0.w);
  mma_e4m3(e, a1.z, b1.z, a1.w, b1.w, x1.z, x1.w);
  d[0] += e[0], d[1] += e[1], d[2] += e[2], d[3] += e[3];
}

// quantises one row's 128 values (4 per lane, k = 4 lane ..) into an activation block
DSGX_DEV void quant_row_to_block(uint8_t* blk, int r, int lane, bool valid, float v0, float v1, float v2, float v3) {
  const int kl = 4 * lane, q = kl >> 6, t = (kl >> 4) & 3, i = kl & 15;
  uint32_t packed = 0;
  float sc = 0.f;
  if (valid) {
    sc = act_scale(warp_max(fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)))));
    packed = quant_e4m3(v0, sc) | quant_e4m3(v1, sc) << 8 | quant_e4m3(v2, sc) << 16 | quant_e4m3(v3, sc) << 24;
  }
  *reinterpret_cast<uint32_t*>(blk + (q * 32 + 4 * r + t) * 16 + i) = packed;
  if (lane == 0) reinterpret_cast<float*>(blk + 1024)[r] = sc;
}

// The RMSNorm in front of a layer step.  rstd: the rows' 1 / rms in shared memory (rms_rows_rstd); w null: no norm.
struct RowNorm {
  const __nv_bfloat16* w;
  const float* rstd;
  int mode;
};
constexpr int kRmsRed = 8 * kMaxRows + kMaxRows;  // floats of shared memory rms_rows_rstd wants
// Every row's 1 / rms into red[8 kMaxRows + r], by the first 256 threads of the CTA (all threads call; two CTA barriers).
// The sum of squares in a fixed order: the row in chunks of 8 values, chunk c to thread c mod 256, a thread adds its chunks
// in ascending order by fma from zero, the warps' butterflies, then the 8 warp sums in ascending order.
DSGX_DEV void rms_rows_rstd(const __nv_bfloat16* __restrict__ x, int M, int H, float eps, float* red) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < 256) {
    float ss[kMaxRows];
#pragma unroll
    for (int r = 0; r < kMaxRows; ++r) ss[r] = 0.f;
    for (int c = tid; c < H / 8; c += 256) {
      uint4 v[kMaxRows];
#pragma unroll
      for (int r = 0; r < kMaxRows; ++r)
        if (r < M) v[r] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)r * H + 8 * c));
#pragma unroll
      for (int r = 0; r < kMaxRows; ++r)
        if (r < M) {
          const uint32_t* vv = &v[r].x;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float lo = bf16_bits_to_f(vv[j] & 0xffffu), hi = bf16_bits_to_f(vv[j] >> 16);
            ss[r] = fmaf(lo, lo, ss[r]), ss[r] = fmaf(hi, hi, ss[r]);
          }
        }
    }
#pragma unroll
    for (int r = 0; r < kMaxRows; ++r)
      if (r < M) {
        const float s = warp_sum(ss[r]);
        if (lane == 0) red[warp * kMaxRows + r] = s;
      }
  }
  __syncthreads();
  if (tid < M) {
    float s = red[tid];
    for (int w = 1; w < 8; ++w) s = __fadd_rn(s, red[w * kMaxRows + tid]);
    red[8 * kMaxRows + tid] = rms_rstd(s, H, eps);
  }
  __syncthreads();
}
// four consecutive values of row r at column k (a multiple of 4), normalised
DSGX_DEV void norm4(const RowNorm& n, int r, int k, float& v0, float& v1, float& v2, float& v3) {
  if (!n.w) return;
  const uint2 wv = __ldg(reinterpret_cast<const uint2*>(n.w + k));
  const float rs = n.rstd[r];
  v0 = rms_apply(v0, rs, bf16_bits_to_f(wv.x & 0xffffu), n.mode), v1 = rms_apply(v1, rs, bf16_bits_to_f(wv.x >> 16), n.mode);
  v2 = rms_apply(v2, rs, bf16_bits_to_f(wv.y & 0xffffu), n.mode), v3 = rms_apply(v3, rs, bf16_bits_to_f(wv.y >> 16), n.mode);
}
DSGX_DEV uint2 pack_bf16x4(float v0, float v1, float v2, float v3) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v0, v1), hi = __floats2bfloat162_rn(v2, v3);
  return make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

DSGX_DEV void quant_x_block(const __nv_bfloat16* __restrict__ x, int M, int K, uint8_t* out, int j, int r, int lane,
                            const RowNorm& nrm = RowNorm{nullptr, nullptr, 0}, __nv_bfloat16* xn_out = nullptr) {
  float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
  if (r < M) {
    const uint2 xv = __ldg(reinterpret_cast<const uint2*>(x + (size_t)r * K + 128 * j + 4 * lane));
    v0 = bf16_bits_to_f(xv.x & 0xffffu), v1 = bf16_bits_to_f(xv.x >> 16);
    v2 = bf16_bits_to_f(xv.y & 0xffffu), v3 = bf16_bits_to_f(xv.y >> 16);
    norm4(nrm, r, 128 * j + 4 * lane, v0, v1, v2, v3);
    if (xn_out) *reinterpret_cast<uint2*>(xn_out + (size_t)r * K + 128 * j + 4 * lane) = pack_bf16x4(v0, v1, v2, v3);
  }
  quant_row_to_block(out + (size_t)j * kActBlk, r, lane, r < M, v0, v1, v2, v3);
}


// rows of a bf16 activation tile: M rounded up to 1, 2, 4 or 8
inline __host__ __device__ int rows_pow2(int M) { return M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8; }

// Position of value v (0..15) inside a 16-value group of a bf16 activation tile.  The INT4 kernels pair nibbles i and
// i + 4 of a 32-bit word into one bf16x2 register (one shift and one logic op per pair), so the activations of a group
// are stored in the order 0,4,1,5,2,6,3,7, 8,12,9,13,10,14,11,15.
DSGX_DEV int tile_pos(int v) { return (v & 8) | ((v & 3) << 1) | ((v >> 2) & 1); }

// x bf16 [M][K] -> tile [K/16 groups][R rows][16 values in tile_pos order]; rows M..R-1 are zero.  One thread a (group, row).
DSGX_DEV void tile_x_group(const __nv_bfloat16* __restrict__ x, int M, int K, int R, uint8_t* out, int kg, int r,
                           const RowNorm& nrm = RowNorm{nullptr, nullptr, 0}, __nv_bfloat16* xn_out = nullptr) {
  uint16_t v[16], o[16];
  if (r < M) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(x + (size_t)r * K + 16 * kg));
    const uint4 b = __ldg(reinterpret_cast<const uint4*>(x + (size_t)r * K + 16 * kg + 8));
    uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    if (nrm.w) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v0 = bf16_bits_to_f(w[2 * i] & 0xffffu), v1 = bf16_bits_to_f(w[2 * i] >> 16);
        float v2 = bf16_bits_to_f(w[2 * i + 1] & 0xffffu), v3 = bf16_bits_to_f(w[2 * i + 1] >> 16);
        norm4(nrm, r, 16 * kg + 4 * i, v0, v1, v2, v3);
        const uint2 pk = pack_bf16x4(v0, v1, v2, v3);
        w[2 * i] = pk.x, w[2 * i + 1] = pk.y;
      }
      if (xn_out) {
        uint4* d = reinterpret_cast<uint4*>(xn_out + (size_t)r * K + 16 * kg);
        d[0] = make_uint4(w[0], w[1], w[2], w[3]), d[1] = make_uint4(w[4], w[5], w[6], w[7]);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) v[2 * i] = (uint16_t)(w[i] & 0xffffu), v[2 * i + 1] = (uint16_t)(w[i] >> 16);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0;
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) o[(i & 8) | ((i & 3) << 1) | ((i >> 2) & 1)] = v[i];
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i] = o[2 * i] | (uint32_t)o[2 * i + 1] << 16;
  uint4* d = reinterpret_cast<uint4*>(out + ((size_t)kg * R + r) * 32);
  d[0] = make_uint4(w[0], w[1], w[2], w[3]);
  d[1] = make_uint4(w[4], w[5], w[6], w[7]);
}

// One (expert, 1024-k slice) of the router logits for every row, in the router's summation order: lane j accumulates
// k = base + 128 i + 4 j + c (i ascending, c = 0..3) by fma from zero, then the butterfly.  All weight loads go out first.
// The slice's router weights (they never change during a step: a kernel may fetch them before it waits for its inputs).
DSGX_DEV void logit_slice_weights(const float* __restrict__ wr, int H, int e, int sl, int lane, float4 (&wv)[8]) {
  const int base = sl * 1024, nit = min(1024, H - base) / 128;
#pragma unroll
  for (int i = 0; i < 8; ++i)
    wv[i] = i < nit ? __ldg(reinterpret_cast<const float4*>(wr + (size_t)e * H + base + 128 * i + 4 * lane))
                    : make_float4(0.f, 0.f, 0.f, 0.f);
}
DSGX_DEV void logit_slice_rows(const __nv_bfloat16* __restrict__ x, const float4 (&wv)[8], int M, int H, int E, int e, int sl,
                               float* __restrict__ lpart, int lane, const RowNorm& nrm = RowNorm{nullptr, nullptr, 0}) {
  const int base = sl * 1024, nit = min(1024, H - base) / 128;
  for (int r = 0; r < M; ++r) {
    uint2 xv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      xv[i] = i < nit ? __ldg(reinterpret_cast<const uint2*>(x + (size_t)r * H + base + 128 * i + 4 * lane)) : make_uint2(0, 0);
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < nit) {
        float v0 = bf16_bits_to_f(xv[i].x & 0xffffu), v1 = bf16_bits_to_f(xv[i].x >> 16);
        float v2 = bf16_bits_to_f(xv[i].y & 0xffffu), v3 = bf16_bits_to_f(xv[i].y >> 16);
        norm4(nrm, r, base + 128 * i + 4 * lane, v0, v1, v2, v3);
        a = fmaf(v0, wv[i].x, a);
        a = fmaf(v1, wv[i].y, a);
        a = fmaf(v2, wv[i].z, a);
        a = fmaf(v3, wv[i].w, a);
      }
    a = warp_sum(a);
    if (lane == 0) lpart[((size_t)sl * kMaxRows + r) * E + e] = a;
  }
}
DSGX_DEV void logit_slice_task(const __nv_bfloat16* __restrict__ x, const float* __restrict__ wr, int M, int H, int E, int e,
                               int sl, float* __restrict__ lpart, int lane, const RowNorm& nrm = RowNorm{nullptr, nullptr, 0}) {
  float4 wv[8];
  logit_slice_weights(wr, H, e, sl, lane, wv);
  logit_slice_rows(x, wv, M, H, E, e, sl, lpart, lane, nrm);
}

struct TabArgs {
  int M, topk, E, e_lo, e_hi;
  const uint8_t* pool;
  const dsgx_mat_desc* desc;
  dsgx_shared_w sh;
  uint32_t fmt;
};

}  // namespace dsgx
