// FP8 (e4m3, 128x128 block-scaled, W8A8-g128) expert step for 1..8 rows: an HBM-bound weight stream.
//
// Persistent kernels, one CTA a SM.  Every warp is its own producer and consumer: lane 0 issues bulk async copies
// (the untiled TMA path) of the next chunks of its unit's two weight strips into the warp's private ring in shared
// memory, an mbarrier per stage counts the bytes in, and the whole warp then feeds the chunk to m16n8k32 e4m3 MMAs with
// the weights as the A operand (16 output channels x 32 k) and the quantised activations as B (32 k x 8 rows).  One
// 128-k block is four MMAs into a fresh accumulator, promoted into the f32 sums with the product of the block's
// weight scale and the row's activation scale.
//
//   k_front:       (layer step) router logit partial sums, one warp per (expert, 1024-k slice), all loads in one
//                  round trip; the other CTAs quantise x per 128 values.
//   k_route_union: (layer step) one CTA: sums the slices, routes the rows (route.cuh), builds the slot table.
//   k_prep:        (moe_decode with the caller's idx / w) the slot table + the quantisation of x.
//   k_up:          unit = (slot, 8 intermediate channels): A rows 0-7 = gate, rows 8-15 = up, so a lane ends with gate
//                  and up of the same (channel, row) and applies SwiGLU in place.  The 16th unit to finish a
//                  128-group of h quantises the group for the down kernel (a ticket, no waiting).
//   k_down:        unit = (slot, 16 output channels); every pick's output is rounded to bf16, parked, and the last slot
//                  to finish an output tile adds the tile's picks in ascending expert id (a ticket again) and writes
//                  yr / ys (and, when asked, the rounded sum).
// The ticket of a finished unit is taken while the next unit already streams (fence and atomic are issued one chunk
// later, the answer is read another chunk later), so the stream never waits for a round trip to L2.
//
// Weight layout consumed as is: the reference's tile_fp8 ([N/8][K/128][32 lanes][32 B]; altar1
// engine/experts/layout.h:108-119), so an 8-row strip of a matrix is one contiguous run of 8 K bytes.
#include "common.cuh"
#include "decode_common.cuh"
#include "kernels.h"

namespace dsgx {

namespace {

// A kernel variant: warps a CTA, 128-k blocks a stage and strip, stages a warp.  Every variant computes the same bits
// (a unit's sums run over k in the same order whatever the chunking).
template <int W, int KCH, int NST>
struct Var {
  static constexpr int kWarps = W, kThreads = W * 32, kKCH = KCH, kNST = NST;
  static constexpr int kUpStage = 2 * KCH * 1024;
  static constexpr int kDownStage = 2 * KCH * 1024 + KCH * kActBlk;
};

constexpr int kTabSmem = (sizeof(SlotTab) + 127) & ~127;
static_assert(sizeof(SlotTab) <= kSlotTabBytes, "workspace room for the slot table");

// One 128-k block: A rows 0-7 from strip a, rows 8-15 from strip b, B from the activation block.
DSGX_DEV void block_mma(float (&d)[4], const uint8_t* a, const uint8_t* b, const uint8_t* act, int lane) {
  const uint4 a0 = lds128(a + 32 * lane), a1 = lds128(a + 32 * lane + 16);
  const uint4 b0 = lds128(b + 32 * lane), b1 = lds128(b + 32 * lane + 16);
  const uint4 x0 = lds128(act + 16 * lane), x1 = lds128(act + 512 + 16 * lane);
  float e[4] = {0.f, 0.f, 0.f, 0.f};
  d[0] = d[1] = d[2] = d[3] = 0.f;
  mma_e4m3(d, a0.x, b0.x, a0.y, b0.y, x0.x, x0.y);
  mma_e4m3(e, a1.x, b1.x, a1.y, b1.y, x1.x, x1.y);
  mma_e4m3(d, a0.z, b0.z, a0.w, b0.w, x0.z, x0.w);
  mma_e4m3(e, a1.z, b1.z, a1.w, b1.w, x1.z, x1.w);
  d[0] += e[0], d[1] += e[1], d[2] += e[2], d[3] += e[3];
}

template <class V>
__global__ void __launch_bounds__(V::kThreads, 1) k_up_fp8(const DecodeParams p) {
  constexpr int kWarps = V::kWarps, kKCH = V::kKCH, kNST = V::kNST, kUpStage = V::kUpStage;
  extern __shared__ __align__(128) uint8_t smem[];
  const int HB = p.H / 128, IB = p.I / 128;
  const int xq_bytes = (HB * kActBlk + 127) & ~127;
  uint8_t* xq = smem;
  SlotTab& tab = *reinterpret_cast<SlotTab*>(smem + xq_bytes);
  uint8_t* ring = smem + xq_bytes + kTabSmem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + kWarps * kNST * kUpStage);
  uint64_t* cbar = bars + kWarps * kNST;  // the CTA's barrier for the table and x
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* myring = ring + warp * kNST * kUpStage;
  uint64_t* mybar = bars + warp * kNST;

  pdl_launch_dependents();
  if (lane == 0)
    for (int s = 0; s < kNST; ++s) mbar_init(mybar + s, 1);
  if (threadIdx.x == 0) mbar_init(cbar, 1);
  mbar_fence_init();
  __syncthreads();
  pdl_wait();
  if (threadIdx.x == 0) {
    mbar_expect_tx(cbar, (uint32_t)(sizeof(SlotTab) + HB * kActBlk));
    bulk_g2s(&tab, p.ws.tab, sizeof(SlotTab), cbar);
    bulk_g2s(xq, p.ws.xq, HB * kActBlk, cbar);
  }
  bool dead = !mbar_wait(cbar, 0);

  const int upp = p.I / 8;  // units a slot
  const int total = dead ? 0 : tab.ntot * upp;
  const int GW = gridDim.x * kWarps, gw = blockIdx.x * kWarps + warp;
  const int cpu = HB / kKCH;  // chunks a unit
  const size_t strip = (size_t)8 * p.H;
  int pu = gw, pc = 0;  // lane 0's producer cursor
  uint32_t issued = 0, consumed = 0;
  const uint64_t pol = policy_evict_first();  // the weights are read once
  auto issue = [&]() {
    const int slot = ord_slot(tab, pu / upp), i8 = pu % upp;
    const size_t off = (size_t)i8 * strip + (size_t)pc * kKCH * 1024;
    uint8_t* st = myring + (issued % kNST) * kUpStage;
    uint64_t* bar = mybar + issued % kNST;
    mbar_expect_tx(bar, kUpStage);
    bulk_g2s_hint(st, tab.ent[slot].g + off, kKCH * 1024, bar, pol);
    bulk_g2s_hint(st + kKCH * 1024, tab.ent[slot].u + off, kKCH * 1024, bar, pol);
    ++issued;
    if (++pc == cpu) pc = 0, pu += GW;
  };
  if (lane == 0)
    for (int s = 0; s < kNST && pu < total; ++s) issue();

  const int g = lane >> 2, t = lane & 3;
  // the finished unit whose ticket is still to be taken (1), or whose ticket is in flight (2)
  int pend = 0, pend_slot = 0, pend_gi = 0, pend_ticket = 0;
  auto advance = [&]() {
    if (pend == 1) {
      __threadfence();
      __syncwarp();
      if (lane == 0) pend_ticket = atomicAdd(p.ws.cnt_h + pend_slot * IB + pend_gi, 1);
      pend = 2;
    } else if (pend == 2) {
      const int ticket = __shfl_sync(0xffffffffu, pend_ticket, 0);
      if (ticket == 15) {  // the 16th unit of a 128-group of h quantises it
        __threadfence();
        const __nv_bfloat16* hrow = p.ws.h + (size_t)pend_slot * 8 * p.I + 128 * pend_gi + 4 * lane;
        uint8_t* blk = p.ws.hq + ((size_t)pend_slot * IB + pend_gi) * kActBlk;
        uint2 hv[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
          hv[r] = r < p.M ? __ldcg(reinterpret_cast<const uint2*>(hrow + (size_t)r * p.I)) : make_uint2(0, 0);
#pragma unroll
        for (int r = 0; r < 8; ++r)
          quant_row_to_block(blk, r, lane, r < p.M, bf16_bits_to_f(hv[r].x & 0xffffu), bf16_bits_to_f(hv[r].x >> 16),
                             bf16_bits_to_f(hv[r].y & 0xffffu), bf16_bits_to_f(hv[r].y >> 16));
        if (lane == 0) p.ws.cnt_h[pend_slot * IB + pend_gi] = 0;
      }
      pend = 0;
    }
  };

  for (int unit = gw; unit < total && !dead; unit += GW) {
    const int slot = ord_slot(tab, unit / upp), i8 = unit % upp;
    const int srow = (i8 * 8) / 128;
    const float sgl = lane < HB ? __ldg(tab.ent[slot].sg + (size_t)srow * HB + lane) : 0.f;
    const float sul = lane < HB ? __ldg(tab.ent[slot].su + (size_t)srow * HB + lane) : 0.f;
    float ag0 = 0.f, ag1 = 0.f, au0 = 0.f, au1 = 0.f;
    for (int c = 0; c < cpu; ++c) {
      const uint32_t sidx = consumed % kNST;
      if (!mbar_wait(mybar + sidx, (consumed / kNST) & 1)) {
        dead = true;
        break;
      }
      const uint8_t* st = myring + sidx * kUpStage;
#pragma unroll
      for (int b = 0; b < kKCH; ++b) {
        const int kb = c * kKCH + b;
        const uint8_t* act = xq + kb * kActBlk;
        float d[4];
        block_mma(d, st + b * 1024, st + kKCH * 1024 + b * 1024, act, lane);
        const float2 xs = *reinterpret_cast<const float2*>(act + 1024 + 8 * t);
        const float sg = __shfl_sync(0xffffffffu, sgl, kb), su = __shfl_sync(0xffffffffu, sul, kb);
        ag0 = fmaf(d[0], sg * xs.x, ag0), ag1 = fmaf(d[1], sg * xs.y, ag1);
        au0 = fmaf(d[2], su * xs.x, au0), au1 = fmaf(d[3], su * xs.y, au1);
      }
      ++consumed;
      __syncwarp();
      if (lane == 0 && pu < total) issue();
      advance();
    }
    if (dead) break;
    while (pend) advance();
    // SwiGLU: g, u rounded to bf16; h = bf16(w_route * silu(g) * u) (no weight for the shared expert)
    const bool routed = slot < tab.nslots;
    const int ch = i8 * 8 + g, r0 = 2 * t, r1 = 2 * t + 1;
    float h0 = __fmul_rn(silu(bf16_round(ag0)), bf16_round(au0));
    float h1 = __fmul_rn(silu(bf16_round(ag1)), bf16_round(au1));
    if (routed) h0 = __fmul_rn(tab.ent[slot].w[r0], h0), h1 = __fmul_rn(tab.ent[slot].w[r1], h1);
    __nv_bfloat16* hrow = p.ws.h + (size_t)slot * 8 * p.I;
    if (r0 < p.M) hrow[(size_t)r0 * p.I + ch] = __float2bfloat16_rn(h0);
    if (r1 < p.M) hrow[(size_t)r1 * p.I + ch] = __float2bfloat16_rn(h1);
    pend = 1, pend_slot = slot, pend_gi = i8 / 16;
  }
  if (!dead)
    while (pend) advance();
  if (dead && lane == 0) atomicCAS(p.ws.status, 0, (int)DSGX_ERR_DEVICE_WAIT);
}

// ------------------------------------------------------------------------------------------------------------ k_down
template <class V>
__global__ void __launch_bounds__(V::kThreads, 1) k_down_fp8(const DecodeParams p) {
  constexpr int kWarps = V::kWarps, kThreads = V::kThreads, kKCH = V::kKCH, kNST = V::kNST, kDownStage = V::kDownStage;
  extern __shared__ __align__(128) uint8_t smem[];
  const int IB = p.I / 128, NT = p.H / 16;
  SlotTab& tab = *reinterpret_cast<SlotTab*>(smem);
  uint8_t* ring = smem + kTabSmem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + kWarps * kNST * kDownStage);
  uint64_t* cbar = bars + kWarps * kNST;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* myring = ring + warp * kNST * kDownStage;
  uint64_t* mybar = bars + warp * kNST;

  pdl_launch_dependents();
  if (lane == 0)
    for (int s = 0; s < kNST; ++s) mbar_init(mybar + s, 1);
  if (threadIdx.x == 0) mbar_init(cbar, 1);
  mbar_fence_init();
  __syncthreads();
  pdl_wait();
  if (threadIdx.x == 0) {
    mbar_expect_tx(cbar, (uint32_t)sizeof(SlotTab));
    bulk_g2s(&tab, p.ws.tab, sizeof(SlotTab), cbar);
  }
  bool dead = !mbar_wait(cbar, 0);

  const int GW = gridDim.x * kWarps, gw = blockIdx.x * kWarps + warp;
  if (!dead && tab.ntot == 0) {  // nothing to add on this GPU: the partial sum is zero
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < (size_t)p.M * p.H; i += (size_t)gridDim.x * kThreads) {
      p.yr[i] = 0.f;
      if (p.out) p.out[i] = __float2bfloat16_rn(0.f);
    }
    return;
  }
  const int total = dead ? 0 : tab.ntot * NT;
  const int cpu = IB / kKCH;
  const size_t strip = (size_t)8 * p.I;
  int pu = gw, pc = 0;
  uint32_t issued = 0, consumed = 0;
  const uint64_t pol = policy_evict_first();
  auto issue = [&]() {
    const int slot = ord_slot(tab, pu / NT), n16 = pu % NT;
    const size_t off = (size_t)(2 * n16) * strip + (size_t)pc * kKCH * 1024;
    uint8_t* st = myring + (issued % kNST) * kDownStage;
    uint64_t* bar = mybar + issued % kNST;
    mbar_expect_tx(bar, kDownStage);
    bulk_g2s_hint(st, tab.ent[slot].d + off, kKCH * 1024, bar, pol);
    bulk_g2s_hint(st + kKCH * 1024, tab.ent[slot].d + off + strip, kKCH * 1024, bar, pol);
    bulk_g2s(st + 2 * kKCH * 1024, p.ws.hq + ((size_t)slot * IB + (size_t)pc * kKCH) * kActBlk, kKCH * kActBlk, bar);
    ++issued;
    if (++pc == cpu) pc = 0, pu += GW;
  };
  if (lane == 0)
    for (int s = 0; s < kNST && pu < total; ++s) issue();

  const int g = lane >> 2, t = lane & 3;
  int pend = 0, pend_n16 = 0, pend_ticket = 0;
  auto advance = [&]() {
    if (pend == 1) {
      __threadfence();
      __syncwarp();
      if (lane == 0) pend_ticket = atomicAdd(p.ws.cnt_y + pend_n16, 1);
      pend = 2;
    } else if (pend == 2) {
      const int ticket = __shfl_sync(0xffffffffu, pend_ticket, 0);
      if (ticket == tab.ntot - 1) {  // the tile's last slot: add its picks in ascending expert id, the shared expert last
        __threadfence();
        const int n16 = pend_n16, ch = lane >> 1, r0 = 4 * (lane & 1);
        const float* yt = p.ws.ypick + (size_t)n16 * 128 + ch * 8 + r0;
        const bool sh = tab.ntot > tab.nslots;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        int s = 0;
        for (; s + 4 <= tab.nslots; s += 4) {  // four loads in flight, added in order
          float4 v[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) v[j] = __ldcg(reinterpret_cast<const float4*>(yt + (size_t)(s + j) * NT * 128));
#pragma unroll
          for (int j = 0; j < 4; ++j)
            a.x = __fadd_rn(a.x, v[j].x), a.y = __fadd_rn(a.y, v[j].y), a.z = __fadd_rn(a.z, v[j].z), a.w = __fadd_rn(a.w, v[j].w);
        }
        for (; s < tab.nslots; ++s) {
          const float4 v = __ldcg(reinterpret_cast<const float4*>(yt + (size_t)s * NT * 128));
          a.x = __fadd_rn(a.x, v.x), a.y = __fadd_rn(a.y, v.y), a.z = __fadd_rn(a.z, v.z), a.w = __fadd_rn(a.w, v.w);
        }
        float4 sv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (sh) sv = __ldcg(reinterpret_cast<const float4*>(yt + (size_t)tab.nslots * NT * 128));
        const float av[4] = {a.x, a.y, a.z, a.w}, svv[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (r0 + c < p.M) {
            const size_t o = (size_t)(r0 + c) * p.H + n16 * 16 + ch;
            const float both = __fadd_rn(av[c], svv[c]);
            p.yr[o] = p.ysum && sh ? both : av[c];
            if (sh && p.ys) p.ys[o] = svv[c];
            if (p.out) p.out[o] = __float2bfloat16_rn(both);
          }
        if (lane == 0) p.ws.cnt_y[n16] = 0;
      }
      pend = 0;
    }
  };

  for (int unit = gw; unit < total && !dead; unit += GW) {
    const int slot = ord_slot(tab, unit / NT), n16 = unit % NT;
    const int srow = (n16 * 16) / 128;
    const float sdl = lane < IB ? __ldg(tab.ent[slot].sd + (size_t)srow * IB + lane) : 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = 0; c < cpu; ++c) {
      const uint32_t sidx = consumed % kNST;
      if (!mbar_wait(mybar + sidx, (consumed / kNST) & 1)) {
        dead = true;
        break;
      }
      const uint8_t* st = myring + sidx * kDownStage;
#pragma unroll
      for (int b = 0; b < kKCH; ++b) {
        const int kb = c * kKCH + b;
        const uint8_t* act = st + 2 * kKCH * 1024 + b * kActBlk;
        float d[4];
        block_mma(d, st + b * 1024, st + kKCH * 1024 + b * 1024, act, lane);
        const float2 hs = *reinterpret_cast<const float2*>(act + 1024 + 8 * t);
        const float sd = __shfl_sync(0xffffffffu, sdl, kb);
        acc[0] = fmaf(d[0], sd * hs.x, acc[0]), acc[1] = fmaf(d[1], sd * hs.y, acc[1]);
        acc[2] = fmaf(d[2], sd * hs.x, acc[2]), acc[3] = fmaf(d[3], sd * hs.y, acc[3]);
      }
      ++consumed;
      __syncwarp();
      if (lane == 0 && pu < total) issue();
      advance();
    }
    if (dead) break;
    while (pend) advance();
    // every pick's output is rounded to bf16 before the f32 adds
    float* yt = p.ws.ypick + ((size_t)slot * NT + n16) * 128;
    *reinterpret_cast<float2*>(yt + g * 8 + 2 * t) = make_float2(bf16_round(acc[0]), bf16_round(acc[1]));
    *reinterpret_cast<float2*>(yt + (g + 8) * 8 + 2 * t) = make_float2(bf16_round(acc[2]), bf16_round(acc[3]));
    pend = 1, pend_n16 = n16;
  }
  if (!dead)
    while (pend) advance();
  if (dead && lane == 0) atomicCAS(p.ws.status, 0, (int)DSGX_ERR_DEVICE_WAIT);
}

template <class V>
size_t up_smem(int H) {
  return (size_t)(((H / 128) * kActBlk + 127) & ~127) + kTabSmem + (size_t)V::kWarps * V::kNST * V::kUpStage +
         (V::kWarps * V::kNST + 1) * 8 + 16;
}
template <class V>
size_t down_smem() {
  return kTabSmem + (size_t)V::kWarps * V::kNST * V::kDownStage + (V::kWarps * V::kNST + 1) * 8 + 16;
}

template <class V>
cudaError_t launch_up(const DecodeParams& p, cudaStream_t st, bool pdl) {
  static bool done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!done[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(k_up_fp8<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)up_smem<V>(4096));
    if (e != cudaSuccess) return e;
    done[dev & 63] = true;
  }
  return launch_k(k_up_fp8<V>, dim3(sm_count()), dim3(V::kThreads), up_smem<V>(p.H), st, pdl, p);
}
template <class V>
cudaError_t launch_down(const DecodeParams& p, cudaStream_t st, bool pdl) {
  static bool done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!done[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(k_down_fp8<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)down_smem<V>());
    if (e != cudaSuccess) return e;
    done[dev & 63] = true;
  }
  return launch_k(k_down_fp8<V>, dim3(sm_count()), dim3(V::kThreads), down_smem<V>(), st, pdl, p);
}

}  // namespace

int decode_fp8_up_variants() { return 7; }
int decode_fp8_down_variants() { return 5; }

static cudaError_t launch_up_down(const DecodeParams& p, cudaStream_t st, bool pdl, int parts) {
  cudaError_t e = cudaSuccess;
  if (parts & 1) {
    switch (p.up) {
      case 1: e = launch_up<Var<8, 4, 2>>(p, st, pdl); break;
      case 2: e = launch_up<Var<8, 2, 5>>(p, st, pdl); break;
      case 3: e = launch_up<Var<4, 8, 2>>(p, st, pdl); break;
      case 4: e = launch_up<Var<8, 2, 3>>(p, st, pdl); break;
      case 5: e = launch_up<Var<16, 1, 5>>(p, st, pdl); break;
      case 6: e = launch_up<Var<12, 2, 3>>(p, st, pdl); break;
      default: e = launch_up<Var<16, 2, 2>>(p, st, pdl); break;
    }
    if (e != cudaSuccess) return e;
  }
  if (parts & 2) {
    switch (p.down) {
      case 1: e = launch_down<Var<8, 4, 2>>(p, st, pdl); break;
      case 2: e = launch_down<Var<4, 8, 2>>(p, st, pdl); break;
      case 3: e = launch_down<Var<16, 1, 4>>(p, st, pdl); break;
      case 4: e = launch_down<Var<8, 2, 3>>(p, st, pdl); break;
      default: e = launch_down<Var<16, 2, 2>>(p, st, pdl); break;
    }
  }
  return e;
}

// The expert step on the caller's idx / w: k_prep, k_up, k_down.
cudaError_t launch_decode_fp8(const DecodeParams& p, const __nv_bfloat16* x, cudaStream_t st, bool pdl, int parts) {
  if ((parts & 1) && !(parts & 4)) {  // (bit 2: the table and the quantised rows of an earlier call are still in ws)
    cudaError_t e = launch_prep(p, DSGX_FMT_FP8, x, st, pdl);
    if (e != cudaSuccess) return e;
  }
  return launch_up_down(p, st, pdl, parts & 3);
}

// The whole layer step: k_front, k_route_union, k_up, k_down (idx / w / logits are outputs of the routing).
cudaError_t launch_layer_fp8(const DecodeParams& p, const RouteParams& rp, const __nv_bfloat16* x, const float* wr,
                             const float* bias, float* logits, int* idx, float* w, cudaStream_t st, bool pdl) {
  cudaError_t e = launch_front_route(p, DSGX_FMT_FP8, rp, x, wr, bias, logits, idx, w, st, pdl);
  if (e != cudaSuccess) return e;
  return launch_up_down(p, st, pdl, 3);
}

}  // namespace dsgx
