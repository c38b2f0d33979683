// The front of a decode step, shared by every expert format: router logit slices, activation staging (FP8: quantised
// blocks; INT4 layers: bf16 tiles), routing of the rows and the slot table.
//
//   k_front:       (layer step) router logit partial sums, one warp per (expert, 1024-k slice), all loads in one
//                  round trip; the other CTAs stage x.
//   k_route_union: (layer step) one CTA a row, one thread an expert: sums the slices and routes the row (route.cuh);
//                  the last CTA to finish builds the slot table (a ticket, no waiting).
//   k_prep:        (moe_decode with the caller's idx / w) the slot table + the staging of x.
#include "common.cuh"
#include "decode_common.cuh"
#include "kernels.h"
#include "route.cuh"

namespace dsgx {

namespace {

// One CTA's share of staging x for the expert kernels.  FP8: one warp a (128-k block, row), quantised blocks.
// Other formats: one thread a (16-value group, row) of the bf16 tile.
DSGX_DEV void stage_x(const __nv_bfloat16* __restrict__ x, int M, int H, uint8_t* __restrict__ out, int fmt, int cta,
                      const RowNorm& nrm = RowNorm{nullptr, nullptr, 0}, __nv_bfloat16* xn_out = nullptr) {
  if (fmt_fp8_family((uint32_t)fmt)) {
    const int gw = cta * 8 + (threadIdx.x >> 5);
    const int j = gw >> 3, r = gw & 7;
    if (j < H / 128) quant_x_block(x, M, H, out, j, r, threadIdx.x & 31, nrm, xn_out);
  } else {
    const int R = rows_pow2(M);
    const int i = cta * 256 + threadIdx.x;
    if (i < H / 16 * R) tile_x_group(x, M, H, R, out, i / R, i % R, nrm, xn_out);
  }
}

// ----------------------------------------------------------------------------------------------------------- k_front
// CTAs [0, nlog): one warp per (expert, slice of 1024 k): the slice's partial logit of every row, in the router's
// summation order (lane j: k = base + 128 i + 4 j + c by fma, then the butterfly).  CTAs [nlog, ..): x -> blocks.
// kNorm: the rows are normalised first (a separate instantiation: the plain kernel keeps its registers and its start).
template <bool kNorm>
__global__ void __launch_bounds__(256) k_front(const __nv_bfloat16* __restrict__ x, const float* __restrict__ wr, int M,
                                               int H, int E, int nlog, float* __restrict__ lpart, uint8_t* __restrict__ xq,
                                               int fmt, FrontNorm fn) {
  __shared__ float red[kNorm ? kRmsRed : 1];
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const RowNorm nrm{kNorm ? fn.w : nullptr, red + (kNorm ? 8 * kMaxRows : 0), fn.mode};
  if ((int)blockIdx.x >= nlog) {
    pdl_wait();
    if (kNorm) rms_rows_rstd(x, M, H, fn.eps, red);
    stage_x(x, M, H, xq, fmt, (int)blockIdx.x - nlog, nrm, kNorm ? fn.xn_out : nullptr);
    return;
  }
  const int KS = (H + 1023) / 1024;
  const int gw = blockIdx.x * 8 + warp;
  const int e = gw / KS, sl = gw % KS;
  // the router weights are fetched while the kernels before this one still run; only x waits for them
  float4 wv[8];
  if (e < E) logit_slice_weights(wr, H, e, sl, lane, wv);
  pdl_wait();
  if (kNorm) rms_rows_rstd(x, M, H, fn.eps, red);  // (every CTA sums the rows itself: 8 KB a row out of L2, no launch in front)
  if (e >= E) return;
  logit_slice_rows(x, wv, M, H, E, e, sl, lpart, lane, nrm);
}

// ----------------------------------------------------------------------------------------------------- k_route_union
DSGX_DEV void store_tab(const SlotTab& tab, SlotTab* out) {
  const uint4* s = reinterpret_cast<const uint4*>(&tab);
  uint4* d = reinterpret_cast<uint4*>(out);
  for (int i = threadIdx.x; i < (int)(sizeof(SlotTab) / 16); i += blockDim.x) d[i] = s[i];
}

// One CTA a row, one thread an expert (route.cuh: route_row_cta); the last CTA to finish builds the slot table (a ticket).
__global__ void __launch_bounds__(512) k_route_union(RouteParams rp, TabArgs ta, const float* __restrict__ lpart, int nsplit,
                                                     const float* __restrict__ bias, float* __restrict__ logits,
                                                     int* __restrict__ idx, float* __restrict__ w, SlotTab* __restrict__ out,
                                                     int* __restrict__ status, int* __restrict__ cnt) {
  __shared__ SlotTab tab;
  __shared__ RouteSmem rs;
  __shared__ uint32_t bm[16];
  __shared__ int s_idx[kMaxRows * kMaxTopK];
  __shared__ float s_w[kMaxRows * kMaxTopK];
  __shared__ int s_ticket;
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  route_row_cta(rp, lpart + (size_t)row * rp.E, nsplit, (size_t)kMaxRows * rp.E, bias, rs,
                logits ? logits + (size_t)row * rp.E : nullptr, idx + row * rp.topk, w + row * rp.topk,
                ta.M == 1 ? s_idx : nullptr, s_w);
  if (ta.M > 1) {  // the last row to finish builds the slot table of the step (one row: its picks are in shared memory)
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_ticket = atomicAdd(cnt, 1);
    __syncthreads();
    if (s_ticket != ta.M - 1) return;
    __threadfence();
    for (int i = threadIdx.x; i < ta.M * ta.topk; i += blockDim.x) s_idx[i] = __ldcg(idx + i), s_w[i] = __ldcg(w + i);
    if (threadIdx.x == 0) *cnt = 0;
  }
  __syncthreads();
  build_slot_tab(tab, bm, s_idx, s_w, ta.M, ta.topk, ta.E, ta.e_lo, ta.e_hi, ta.pool, ta.desc, ta.sh, ta.fmt);
  if (threadIdx.x == 0 && tab.bad) atomicCAS(status, 0, tab.bad);
  store_tab(tab, out);
}

// ------------------------------------------------------------------------------------------------------------ k_prep
// CTA 0: the slot table from the caller's idx / w.  CTAs 1..: x -> blocks.
__global__ void __launch_bounds__(256) k_prep(TabArgs ta, const int* __restrict__ idx, const float* __restrict__ w,
                                              const __nv_bfloat16* __restrict__ x, int H, uint8_t* __restrict__ xq,
                                              SlotTab* __restrict__ out, int* __restrict__ status) {
  __shared__ SlotTab tab;
  __shared__ uint32_t bm[16];
  pdl_launch_dependents();
  pdl_wait();
  if (blockIdx.x == 0) {
    if (!idx) return;  // (the table comes from the routing kernel that follows: this launch only stages x)
    build_slot_tab(tab, bm, idx, w, ta.M, ta.topk, ta.E, ta.e_lo, ta.e_hi, ta.pool, ta.desc, ta.sh, ta.fmt);
    if (threadIdx.x == 0 && tab.bad) atomicCAS(status, 0, tab.bad);
    store_tab(tab, out);
    return;
  }
  stage_x(x, ta.M, H, xq, (int)ta.fmt, (int)blockIdx.x - 1);
}

// -------------------------------------------------------------------------------------------------------------- k_up

TabArgs tab_args(const DecodeParams& p, uint32_t fmt) {
  TabArgs ta;
  ta.M = p.M, ta.topk = p.topk, ta.E = p.E, ta.e_lo = p.e_lo, ta.e_hi = p.e_hi;
  ta.pool = p.pool, ta.desc = p.desc, ta.sh = p.sh, ta.fmt = fmt;
  return ta;
}

int stage_ctas(const DecodeParams& p, uint32_t fmt) {
  return fmt_fp8_family(fmt) ? (p.H / 128 * 8 + 7) / 8 : (p.H / 16 * rows_pow2(p.M) + 255) / 256;
}

}  // namespace

cudaError_t launch_prep(const DecodeParams& p, uint32_t fmt, const __nv_bfloat16* x, cudaStream_t st, bool pdl) {
  return launch_k(k_prep, dim3(1 + stage_ctas(p, fmt)), dim3(256), 0, st, pdl, tab_args(p, fmt), p.idx, p.w, x, p.H, p.ws.xq,
                  p.ws.tab, p.ws.status);
}

cudaError_t launch_front_route(const DecodeParams& p, uint32_t fmt, const RouteParams& rp, const __nv_bfloat16* x,
                               const float* wr, const float* bias, float* logits, int* idx, float* w, cudaStream_t st,
                               bool pdl) {
  const int KS = (p.H + 1023) / 1024;
  const int nlog = (p.E * KS + 7) / 8;
  cudaError_t e = launch_k(p.norm.w ? k_front<true> : k_front<false>, dim3(nlog + stage_ctas(p, fmt)), dim3(256), 0, st, pdl, x,
                           wr, p.M, p.H, p.E, nlog, p.ws.lpart, p.ws.xq, (int)fmt, p.norm);
  if (e != cudaSuccess) return e;
  return launch_k(k_route_union, dim3(p.M), dim3((p.E + 31) / 32 * 32), 0, st, pdl, rp, tab_args(p, fmt),
                  (const float*)p.ws.lpart, KS, bias, logits, idx, w, p.ws.tab, p.ws.status, p.ws.status + 16);
}

// The expert step on the caller's logits (the fused routing of the reference's DecodeCfg::logits): x staged, then the rows
// routed and the table built by the routing kernel; idx / w (the step's picks, an output here) go to the given buffers.
cudaError_t launch_stage_route(const DecodeParams& p, uint32_t fmt, const RouteParams& rp, const __nv_bfloat16* x,
                               const float* logits_in, const float* bias, int* idx, float* w, cudaStream_t st, bool pdl) {
  cudaError_t e = launch_k(k_prep, dim3(1 + stage_ctas(p, fmt)), dim3(256), 0, st, pdl, tab_args(p, fmt), (const int*)nullptr,
                           (const float*)nullptr, x, p.H, p.ws.xq, p.ws.tab, p.ws.status);
  if (e != cudaSuccess) return e;
  return launch_k(k_route_union, dim3(p.M), dim3((p.E + 31) / 32 * 32), 0, st, pdl, rp, tab_args(p, fmt), logits_in, 1, bias,
                  (float*)nullptr, idx, w, p.ws.tab, p.ws.status, p.ws.status + 16);
}

// the same without staging x (the one-kernel step stages x itself)
cudaError_t launch_front_route_only(const DecodeParams& p, const RouteParams& rp, const __nv_bfloat16* x, const float* wr,
                                    const float* bias, float* logits, int* idx, float* w, cudaStream_t st, bool pdl) {
  const int KS = (p.H + 1023) / 1024;
  const int nlog = (p.E * KS + 7) / 8;
  FrontNorm fn = p.norm;
  fn.xn_out = nullptr;  // (the one kernel that follows writes the copy)
  cudaError_t e = launch_k(fn.w ? k_front<true> : k_front<false>, dim3(nlog), dim3(256), 0, st, pdl, x, wr, p.M, p.H, p.E, nlog,
                           p.ws.lpart, p.ws.xq, (int)DSGX_FMT_FP8, fn);
  if (e != cudaSuccess) return e;
  return launch_k(k_route_union, dim3(p.M), dim3((p.E + 31) / 32 * 32), 0, st, pdl, rp, tab_args(p, DSGX_FMT_FP8),
                  (const float*)p.ws.lpart, KS, bias, logits, idx, w, p.ws.tab, p.ws.status, p.ws.status + 16);
}

}  // namespace dsgx
