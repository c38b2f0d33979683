// Pieces the decode kernels of every format share: the slot table (the sorted union of a step's picked experts, plus
// the shared expert) and the per-warp weight-streaming ring.
#pragma once
#include "common.cuh"
#include "kernels.h"

namespace dsgx {

// The slot table of a step, built once by one CTA and read by every CTA of the expert kernels.
// Slots 0 .. nslots-1: the picked experts this GPU owns, ascending id; slot nslots: the shared expert (if any).
// A row that did not pick a slot's expert has weight 0 there.  Size a multiple of 16 bytes (bulk-copied).
struct alignas(16) SlotTab {
  int nslots;  // routed slots
  int ntot;    // + the shared expert's
  int bad;     // a dsgx_status when the picks or descriptors were refused (the routed work is then dropped)
  int pad;
  int e[kMaxSlots + 3];
  float w[kMaxSlots][8];
  const uint8_t* g[kMaxSlots + 1];  // gate, up, down blocks
  const uint8_t* u[kMaxSlots + 1];
  const uint8_t* d[kMaxSlots + 1];
  const float* sg[kMaxSlots + 1];  // FP8: their f32 block scales
  const float* su[kMaxSlots + 1];
  const float* sd[kMaxSlots + 1];
};
static_assert(sizeof(SlotTab) % 16 == 0, "SlotTab is bulk-copied");

// Builds the table in shared memory from the step's picks (idx, w: M x topk, shared or global memory), by one whole CTA.
// scratch: 16 words of shared memory.
DSGX_DEV void build_slot_tab(SlotTab& tab, uint32_t* bm, const int* idx, const float* w, int M, int topk, int E, int e_lo,
                             int e_hi, const uint8_t* pool, const dsgx_mat_desc* desc, const dsgx_shared_w& sh,
                             uint32_t fmt) {
  const int tid = threadIdx.x, nt = blockDim.x;
  if (tid < 16) bm[tid] = 0;
  if (tid == 0) tab.bad = 0, tab.pad = 0;
  for (int i = tid; i < kMaxSlots * 8; i += nt) (&tab.w[0][0])[i] = 0.f;
  __syncthreads();
  const int np = M * topk;
  for (int i = tid; i < np; i += nt) {
    const int e = idx[i];
    if (e < 0 || e >= E) tab.bad = DSGX_ERR_ARG;
    else if (e >= e_lo && e < e_hi) atomicOr(&bm[e >> 5], 1u << (e & 31));
  }
  __syncthreads();
  auto rank_of = [&](int e) {
    int r = __popc(bm[e >> 5] & ((1u << (e & 31)) - 1u));
    for (int k = 0; k < (e >> 5); ++k) r += __popc(bm[k]);
    return r;
  };
  for (int e = tid; e < E; e += nt)
    if ((bm[e >> 5] >> (e & 31)) & 1) {
      const int s = rank_of(e);
      tab.e[s] = e;
      const dsgx_mat_desc* d = desc + (size_t)e * 3;
      if (d[0].fmt != fmt || d[1].fmt != fmt || d[2].fmt != fmt) tab.bad = DSGX_ERR_FORMAT;
      tab.g[s] = pool + d[0].off, tab.u[s] = pool + d[1].off, tab.d[s] = pool + d[2].off;
      if (fmt == DSGX_FMT_FP8) {
        tab.sg[s] = reinterpret_cast<const float*>(pool + ((uint64_t)d[0].rsv[0] | (uint64_t)d[0].rsv[1] << 32));
        tab.su[s] = reinterpret_cast<const float*>(pool + ((uint64_t)d[1].rsv[0] | (uint64_t)d[1].rsv[1] << 32));
        tab.sd[s] = reinterpret_cast<const float*>(pool + ((uint64_t)d[2].rsv[0] | (uint64_t)d[2].rsv[1] << 32));
      } else {
        tab.sg[s] = tab.su[s] = tab.sd[s] = nullptr;
      }
    }
  for (int i = tid; i < np; i += nt) {
    const int e = idx[i];
    if (e >= 0 && e < E && e >= e_lo && e < e_hi) tab.w[rank_of(e)][i / topk] = w[i];
  }
  __syncthreads();
  if (tid == 0) {
    int n = 0;
    for (int k = 0; k < 16; ++k) n += __popc(bm[k]);
    if (tab.bad) n = 0;  // refuse the routed work, keep the kernels well-defined
    const bool has_sh = fmt == DSGX_FMT_FP8 ? sh.g != nullptr : sh.bg != nullptr;
    tab.nslots = n, tab.ntot = n + (has_sh ? 1 : 0);
    if (has_sh) {
      tab.e[n] = -1;
      if (fmt == DSGX_FMT_FP8) {
        tab.g[n] = sh.g, tab.u[n] = sh.u, tab.d[n] = sh.d, tab.sg[n] = sh.gs, tab.su[n] = sh.us, tab.sd[n] = sh.ds;
      } else {
        tab.g[n] = sh.bg, tab.u[n] = sh.bu, tab.d[n] = sh.bd, tab.sg[n] = tab.su[n] = tab.sd[n] = nullptr;
      }
    }
  }
  __syncthreads();
}

// order position -> slot: the shared expert's units come first (they are the same every step)
DSGX_DEV int ord_slot(const SlotTab& tab, int ord) {
  return tab.ntot > tab.nslots ? (ord == 0 ? tab.nslots : ord - 1) : ord;
}

DSGX_DEV uint4 lds128(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }

}  // namespace dsgx
