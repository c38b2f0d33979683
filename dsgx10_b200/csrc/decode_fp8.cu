// FP8 (e4m3, 128x128 block-scaled, W8A8-g128) expert step for 1..8 rows: an HBM-bound weight stream.
//
// Persistent kernels, one CTA a SM.  Every warp is its own producer and consumer: lane 0 issues bulk async copies
// (the untiled TMA path) of the next chunks of its item's two weight strips into the warp's private ring in shared
// memory, an mbarrier per stage counts the bytes in, and the whole warp then feeds the chunk to m16n8k32 e4m3 MMAs with
// the weights as the A operand (16 output channels x 32 k) and the quantised activations as B (32 k x 8 rows).  One
// 128-k block is four MMAs into a fresh accumulator, promoted into the f32 sums with the product of the block's
// weight scale and the row's activation scale.
//
//   k_up:   unit = (slot, 8 intermediate channels): A rows 0-7 = gate, rows 8-15 = up, so a lane ends with gate and up
//           of the same (channel, row) and applies SwiGLU in place.  The 16th unit to finish a 128-group of h quantises
//           the group for the down kernel (a ticket, no waiting).
//   k_down: unit = (slot, 16 output channels); every pick's output is rounded to bf16, parked, and the last slot
//           to finish an output tile adds the tile's picks in ascending expert id (a ticket again) and writes
//           yr / ys (and, when asked, the rounded sum).
//
// Work is dealt to the warps CTA-interleaved (consecutive items go to different SMs: one SM draws only a fraction of the
// memory's rate, so a launch with few items must not sit on a few SMs), and when a launch has fewer units than warps
// the K of a unit is split over 2, 4 or 8 warps in runs of whole pieces (decode_common.cuh: the summation order does not
// depend on the split), the piece sums meeting in the workspace: split-K across SMs.
// The ticket of a finished unit is taken while the next item already streams (fence and atomic are issued one chunk
// later, the answer is read another chunk later), so the stream never waits for a round trip to L2.
//
// Weight layout consumed as is: the reference's tile_fp8 ([N/8][K/128][32 lanes][32 B]; altar1
// engine/experts/layout.h:108-119), so an 8-row strip of a matrix is one contiguous run of 8 K bytes.
#include <atomic>

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
constexpr int kShSlot = kMaxSlots - 1;  // where the shared expert's h, hq and outputs live in the workspace
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

// kMx: the routed experts are MXFP4 (a separate instantiation: an FP8 layer's kernels carry none of that code)
template <class V, bool kMx>
__global__ void __launch_bounds__(V::kThreads, 1) k_up_fp8(const DecodeParams p) {
  constexpr int kWarps = V::kWarps, kKCH = V::kKCH, kNST = V::kNST, kUpStage = V::kUpStage;
  extern __shared__ __align__(128) uint8_t smem[];
  const int HB = p.H / 128, IB = p.I / 128, NP = (HB + kPB - 1) / kPB;
  const int xq_bytes = (HB * kActBlk + 127) & ~127;
  uint8_t* xq = smem;
  SlotTab& tab = *reinterpret_cast<SlotTab*>(smem + xq_bytes);
  uint8_t* ring = smem + xq_bytes + kTabSmem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + kWarps * kNST * kUpStage);
  uint64_t* tabbar = bars + kWarps * kNST;
  uint64_t* xbar = tabbar + 1;  // the quantised rows: needed at the first MMA, not to request the first weights
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int GW = gridDim.x * kWarps, gw = warp * gridDim.x + blockIdx.x;
  uint8_t* myring = ring + warp * kNST * kUpStage;
  uint64_t* mybar = bars + warp * kNST;

  if (lane == 0)
    for (int s = 0; s < kNST; ++s) mbar_init(mybar + s, 1);
  if (threadIdx.x == 0) mbar_init(tabbar, 1), mbar_init(xbar, 1);
  mbar_fence_init();
  __syncthreads();
  pdl_wait();
  // (after the wait: the down kernel, launched on this trigger, reads the slot table before its own wait, and by now the
  // kernel that wrote the table is complete)
  pdl_launch_dependents();
  if (threadIdx.x == 0) {  // the slot table and the quantised rows, made by the kernel ahead
    mbar_expect_tx(tabbar, (uint32_t)sizeof(SlotTab));
    bulk_g2s(&tab, p.ws.tab, sizeof(SlotTab), tabbar);
    mbar_expect_tx(xbar, (uint32_t)(HB * kActBlk));
    bulk_g2s(xq, p.ws.xq, HB * kActBlk, xbar);
  }

  const int upp = p.I / 8;  // units a slot
  const uint64_t pol = policy_evict_first();  // the weights are read once
  uint32_t issued = 0, consumed = 0;
  bool dead = false;

  // ---- what a finished run still owes: 1 its ticket among the unit's runs, 2 that ticket's answer (the last run adds
  // the pieces and applies SwiGLU), 3 the unit's ticket among the 16 units of its 128-group of h, 4 that answer (the
  // 16th quantises the group)
  int pend = 0, pend_uidx = 0, pend_split = 0, pend_wslot = 0, pend_tslot = -1, pend_i8 = 0, pend_ticket = 0;
  auto write_h = [&](const float (&a)[4]) {  // a = gate r0, gate r1, up r0, up r1 of channel 8 i8 + g
    const int ch = pend_i8 * 8 + g, r0 = 2 * t, r1 = 2 * t + 1;
    float g0 = bf16_round(a[0]), g1 = bf16_round(a[1]), u0 = bf16_round(a[2]), u1 = bf16_round(a[3]);
    swiglu_clamp(g0, u0, p.limit), swiglu_clamp(g1, u1, p.limit);
    float h0 = __fmul_rn(silu(g0), u0), h1 = __fmul_rn(silu(g1), u1);
    if (pend_tslot >= 0) h0 = __fmul_rn(tab.ent[pend_tslot].w[r0], h0), h1 = __fmul_rn(tab.ent[pend_tslot].w[r1], h1);
    __nv_bfloat16* hrow = p.ws.h + (size_t)pend_wslot * 8 * p.I;
    if (r0 < p.M) hrow[(size_t)r0 * p.I + ch] = __float2bfloat16_rn(h0);
    if (r1 < p.M) hrow[(size_t)r1 * p.I + ch] = __float2bfloat16_rn(h1);
  };
  auto advance = [&]() {
    if (pend == 1) {
      __threadfence();
      __syncwarp();
      if (lane == 0) pend_ticket = atomicAdd(p.ws.cnt_u + pend_uidx, 1);
      pend = 2;
    } else if (pend == 2) {
      const int ticket = __shfl_sync(0xffffffffu, pend_ticket, 0);
      if (ticket == pend_split - 1) {  // the unit's last run: the pieces in ascending order
        __threadfence();
        const float* pp = p.ws.part + (size_t)pend_uidx * kMaxPieces * 128 + lane * 4;
        float4 v[kMaxPieces];
#pragma unroll
        for (int j = 0; j < kMaxPieces; ++j)
          v[j] = j < NP ? __ldcg(reinterpret_cast<const float4*>(pp + j * 128)) : make_float4(0.f, 0.f, 0.f, 0.f);
        float a[4] = {v[0].x, v[0].y, v[0].z, v[0].w};
#pragma unroll
        for (int j = 1; j < kMaxPieces; ++j)
          if (j < NP)
            a[0] = __fadd_rn(a[0], v[j].x), a[1] = __fadd_rn(a[1], v[j].y), a[2] = __fadd_rn(a[2], v[j].z), a[3] = __fadd_rn(a[3], v[j].w);
        if (lane == 0) p.ws.cnt_u[pend_uidx] = 0;
        write_h(a);
        pend = 3;
      } else {
        pend = 0;
      }
    } else if (pend == 3) {
      __threadfence();
      __syncwarp();
      if (lane == 0) pend_ticket = atomicAdd(p.ws.cnt_h + pend_wslot * IB + pend_i8 / 16, 1);
      pend = 4;
    } else if (pend == 4) {
      const int ticket = __shfl_sync(0xffffffffu, pend_ticket, 0);
      if (ticket == 15) {  // the 16th unit of a 128-group of h quantises it
        __threadfence();
        const int gi = pend_i8 / 16;
        const __nv_bfloat16* hrow = p.ws.h + (size_t)pend_wslot * 8 * p.I + 128 * gi + 4 * lane;
        uint8_t* blk = p.ws.hq + ((size_t)pend_wslot * IB + gi) * kActBlk;
        uint2 hv[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
          hv[r] = r < p.M ? __ldcg(reinterpret_cast<const uint2*>(hrow + (size_t)r * p.I)) : make_uint2(0, 0);
#pragma unroll
        for (int r = 0; r < 8; ++r)
          quant_row_to_block(blk, r, lane, r < p.M, bf16_bits_to_f(hv[r].x & 0xffffu), bf16_bits_to_f(hv[r].x >> 16),
                             bf16_bits_to_f(hv[r].y & 0xffffu), bf16_bits_to_f(hv[r].y >> 16));
        if (lane == 0) p.ws.cnt_h[pend_wslot * IB + gi] = 0;
      }
      pend = 0;
    }
  };

  // ---- this warp's items first, first + GW, .. < end.  Item i = run i % split of unit i / split; run r covers the pieces
  // [r rp, (r + 1) rp) of the unit (rp = ceil(NP / split); a run past the last piece streams nothing and only reports).
  auto stream = [&](int first, int end, int split, int sh_units, int u0) {
    const int rp = (NP + split - 1) / split;
    int pi = first, pc = 0, pnc = -1, pblk = 1024;  // the producer (lane 0): its item, chunks issued of it, chunks it has
    const uint8_t *pg = nullptr, *pu = nullptr;
    auto issue = [&]() {
      while (pi < end) {
        if (pnc < 0) {
          const int unit = pi / split, r = pi % split;
          const int b0 = r * rp * kPB, b1 = min(HB, (r + 1) * rp * kPB);
          const bool shared = unit < sh_units;
          const int slot = shared ? 0 : (unit - sh_units) / upp, i8 = shared ? u0 + unit : (unit - sh_units) % upp;
          pblk = kMx && !shared ? kMxBlk : 1024;  // bytes of a (strip, 128-k block)
          const size_t off = ((size_t)i8 * HB + b0) * pblk;
          pg = (shared ? p.sh.g : tab.ent[slot].g) + off, pu = (shared ? p.sh.u : tab.ent[slot].u) + off;
          pnc = b1 > b0 ? (b1 - b0) / kKCH : 0, pc = 0;
        }
        if (pc < pnc) {
          uint8_t* st = myring + (issued % kNST) * kUpStage;
          uint64_t* bar = mybar + issued % kNST;
          mbar_expect_tx(bar, 2 * kKCH * pblk);
          bulk_g2s_hint(st, pg, kKCH * pblk, bar, pol);
          bulk_g2s_hint(st + kKCH * 1024, pu, kKCH * pblk, bar, pol);
          pg += kKCH * pblk, pu += kKCH * pblk;
          ++issued;
          if (++pc == pnc) pi += GW, pnc = -1;
          return;
        }
        pi += GW, pnc = -1;
      }
    };
    if (lane == 0)
      while (pi < end && issued - consumed < (uint32_t)kNST) issue();
    if (!mbar_wait(xbar, 0)) dead = true;  // (the first weights are on their way)
    for (int it = first; it < end && !dead; it += GW) {
      const int unit = it / split, r = it % split;
      const int b0 = r * rp * kPB, b1 = min(HB, (r + 1) * rp * kPB);
      const bool shared = unit < sh_units;
      const int slot = shared ? 0 : (unit - sh_units) / upp, i8 = shared ? u0 + unit : (unit - sh_units) % upp;
      const int uidx = unit;
      float tot[4] = {0.f, 0.f, 0.f, 0.f}, pc4[4] = {0.f, 0.f, 0.f, 0.f};  // gate r0, gate r1, up r0, up r1
      if (b1 > b0) {
        const bool mx = kMx && !shared;
        const int srow = (i8 * 8) / 128, blk = mx ? kMxBlk : 1024;
        const float* sgp = shared ? p.sh.gs : tab.ent[slot].sg;
        const float* sup = shared ? p.sh.us : tab.ent[slot].su;
        const float sgl = mx ? 1.f : lane < HB ? __ldg(sgp + (size_t)srow * HB + lane) : 0.f;  // (MXFP4: scales in the block)
        const float sul = mx ? 1.f : lane < HB ? __ldg(sup + (size_t)srow * HB + lane) : 0.f;
        const int nc = (b1 - b0) / kKCH;
        for (int c = 0; c < nc; ++c) {
          const uint32_t sidx = consumed % kNST;
          if (!mbar_wait(mybar + sidx, (consumed / kNST) & 1)) {
            dead = true;
            break;
          }
          const uint8_t* st = myring + sidx * kUpStage;
#pragma unroll
          for (int b = 0; b < kKCH; ++b) {
            const int kb = b0 + c * kKCH + b;
            const uint8_t* act = xq + kb * kActBlk;
            float d[4];
            if (mx) block_mma_mx(d, st + b * blk, st + kKCH * 1024 + b * blk, act, lane);
            else block_mma(d, st + b * 1024, st + kKCH * 1024 + b * 1024, act, lane);
            const float2 xs = *reinterpret_cast<const float2*>(act + 1024 + 8 * t);
            const float sg = __shfl_sync(0xffffffffu, sgl, kb), su = __shfl_sync(0xffffffffu, sul, kb);
            pc4[0] = fmaf(d[0], sg * xs.x, pc4[0]), pc4[1] = fmaf(d[1], sg * xs.y, pc4[1]);
            pc4[2] = fmaf(d[2], su * xs.x, pc4[2]), pc4[3] = fmaf(d[3], su * xs.y, pc4[3]);
            if (piece_end(kb, HB)) {
              if (split == 1) {
                piece_fold(tot, pc4, kb < kPB);
              } else {
                *reinterpret_cast<float4*>(p.ws.part + ((size_t)uidx * kMaxPieces + kb / kPB) * 128 + lane * 4) =
                    make_float4(pc4[0], pc4[1], pc4[2], pc4[3]);
                pc4[0] = pc4[1] = pc4[2] = pc4[3] = 0.f;
              }
            }
          }
          ++consumed;
          __syncwarp();
          if (lane == 0) issue();
          advance();
        }
      }
      if (dead) break;
      while (pend) advance();
      pend_uidx = uidx, pend_split = split, pend_wslot = shared ? kShSlot : slot, pend_tslot = shared ? -1 : slot, pend_i8 = i8;
      if (split == 1) {
        write_h(tot);
        pend = 3;
      } else {
        pend = 1;
      }
    }
  };

  // ---- the shared expert's units first (they are the same every step), then the routed slots' ----------------------------
  if (!mbar_wait(tabbar, 0)) dead = true;
  if (!dead) {
    const int sh_units = tab.ntot > tab.nslots ? (p.sh_hi - p.sh_lo) / 8 : 0;
    const int units = sh_units + tab.nslots * upp;
    const int split = pick_split(units, NP, GW, kPartUnits);
    stream(gw, units * split, split, sh_units, p.sh_lo / 8);
  }
  if (!dead)
    while (pend) advance();
  if (dead && lane == 0) atomicCAS(p.ws.status, 0, (int)DSGX_ERR_DEVICE_WAIT);
}

// ------------------------------------------------------------------------------------------------------------ k_down
template <class V, bool kMx>
__global__ void __launch_bounds__(V::kThreads, 1) k_down_fp8(const DecodeParams p) {
  constexpr int kWarps = V::kWarps, kThreads = V::kThreads, kKCH = V::kKCH, kNST = V::kNST, kDownStage = V::kDownStage;
  extern __shared__ __align__(128) uint8_t smem[];
  const int IB = p.I / 128, NT = p.H / 16, NP = (IB + kPB - 1) / kPB;
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
  // The slot table is older than the gate/up kernel (which needed it too, and triggered this launch only after its own
  // wait): it is read, and the first stages' down weights are requested, BEFORE the wait for the gate/up kernel, whose
  // last CTAs are still finishing then; only the quantised h, that kernel's output, is requested after the wait.
  if (threadIdx.x == 0) {
    mbar_expect_tx(cbar, (uint32_t)sizeof(SlotTab));
    bulk_g2s(&tab, p.ws.tab, sizeof(SlotTab), cbar);
  }
  bool dead = !mbar_wait(cbar, 0);

  const int GW = gridDim.x * kWarps, gw = warp * gridDim.x + blockIdx.x;
  if (!dead && tab.ntot == 0) {  // nothing to add on this GPU: the partial sum is zero
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < (size_t)p.M * p.H; i += (size_t)gridDim.x * kThreads) {
      p.yr[i] = 0.f;
      if (p.out) p.out[i] = __float2bfloat16_rn(0.f);
    }
    return;
  }
  const int units = dead ? 0 : tab.ntot * NT;
  const int split = pick_split(units, NP, GW, kPartUnits);
  const int rp = (NP + split - 1) / split;
  const int end = units * split;
  const bool sh_any = tab.ntot > tab.nslots;
  const int sh_b0 = p.sh_lo / 128, sh_b1 = p.sh_hi / 128;  // the shared expert's K blocks on this GPU
  uint32_t issued = 0, consumed = 0;
  const uint64_t pol = policy_evict_first();

  // item -> its unit's slot (in the table and in the workspace), its tile, its K blocks [b0, b1)
  auto decode = [&](int it, int& tslot, int& wslot, int& n16, int& b0, int& b1) {
    const int unit = it / split, r = it % split;
    tslot = ord_slot(tab, unit / NT), n16 = unit % NT;
    const bool sh = tslot >= tab.nslots;
    wslot = sh ? kShSlot : tslot;
    b0 = max(r * rp * kPB, sh ? sh_b0 : 0), b1 = min(min(IB, (r + 1) * rp * kPB), sh ? sh_b1 : IB);
  };
  int pi = gw, pc = 0, pnc = -1, pwslot = 0, pb = 0, pblk = 1024;
  const uint8_t* pd = nullptr;
  bool early = true;  // before the wait: the h blocks of the stages issued now are requested after it
  const uint8_t* late_src[kNST];
  auto issue = [&]() {
    while (pi < end) {
      if (pnc < 0) {
        int tslot, n16, b0, b1;
        decode(pi, tslot, pwslot, n16, b0, b1);
        pblk = kMx && tslot < tab.nslots ? kMxBlk : 1024;  // bytes of a (strip, 128-k block)
        pd = tab.ent[tslot].d + ((size_t)(2 * n16) * IB + b0) * pblk;
        pb = b0, pnc = b1 > b0 ? (b1 - b0) / kKCH : 0, pc = 0;
      }
      if (pc < pnc) {
        uint8_t* st = myring + (issued % kNST) * kDownStage;
        uint64_t* bar = mybar + issued % kNST;
        mbar_expect_tx(bar, 2 * kKCH * pblk + kKCH * kActBlk);
        bulk_g2s_hint(st, pd, kKCH * pblk, bar, pol);
        bulk_g2s_hint(st + kKCH * 1024, pd + (size_t)IB * pblk, kKCH * pblk, bar, pol);
        const uint8_t* hsrc = p.ws.hq + ((size_t)pwslot * IB + pb) * kActBlk;
        if (early) late_src[issued % kNST] = hsrc;
        else bulk_g2s(st + 2 * kKCH * 1024, hsrc, kKCH * kActBlk, bar);
        pd += kKCH * pblk, pb += kKCH;
        ++issued;
        if (++pc == pnc) pi += GW, pnc = -1;
        return;
      }
      pi += GW, pnc = -1;
    }
  };
  if (lane == 0)
    while (pi < end && issued - consumed < (uint32_t)kNST) issue();
  pdl_wait();
  if (lane == 0)
    for (uint32_t n = 0; n < issued; ++n)
      bulk_g2s(myring + n * kDownStage + 2 * kKCH * 1024, late_src[n], kKCH * kActBlk, mybar + n);
  early = false;

  const int g = lane >> 2, t = lane & 3;
  // what a finished run still owes: 1, 2 its ticket among the unit's runs (the last adds the pieces and parks the pick's
  // rounded output), 3, 4 the unit's ticket among the slots of its output tile (the last adds the tile's picks)
  int pend = 0, pend_uidx = 0, pend_wslot = 0, pend_n16 = 0, pend_p0 = 0, pend_p1 = 0, pend_ticket = 0;
  // every pick's output is rounded to bf16 before the f32 adds; a GPU that holds only a part of the shared expert's
  // intermediate channels keeps its part of that output in f32: it is rounded once all parts are added (across the GPUs)
  const bool sh_part = p.sh_lo != 0 || p.sh_hi != p.I;
  auto park = [&](const float (&acc)[4]) {
    float* yt = p.ws.ypick + ((size_t)pend_wslot * NT + pend_n16) * 128;
    const bool keep = sh_part && pend_wslot == kShSlot;
    *reinterpret_cast<float2*>(yt + g * 8 + 2 * t) =
        keep ? make_float2(acc[0], acc[1]) : make_float2(bf16_round(acc[0]), bf16_round(acc[1]));
    *reinterpret_cast<float2*>(yt + (g + 8) * 8 + 2 * t) =
        keep ? make_float2(acc[2], acc[3]) : make_float2(bf16_round(acc[2]), bf16_round(acc[3]));
  };
  auto advance = [&]() {
    if (pend == 1) {
      __threadfence();
      __syncwarp();
      if (lane == 0) pend_ticket = atomicAdd(p.ws.cnt_u + pend_uidx, 1);
      pend = 2;
    } else if (pend == 2) {
      const int ticket = __shfl_sync(0xffffffffu, pend_ticket, 0);
      if (ticket == split - 1) {  // the unit's last run: its pieces [p0, p1) in ascending order
        __threadfence();
        const float* pp = p.ws.part + (size_t)pend_uidx * kMaxPieces * 128 + lane * 4;
        float4 v[kMaxPieces];
#pragma unroll
        for (int j = 0; j < kMaxPieces; ++j)
          v[j] = j >= pend_p0 && j < pend_p1 ? __ldcg(reinterpret_cast<const float4*>(pp + j * 128)) : make_float4(0.f, 0.f, 0.f, 0.f);
        float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < kMaxPieces; ++j)
          if (j == pend_p0) a[0] = v[j].x, a[1] = v[j].y, a[2] = v[j].z, a[3] = v[j].w;
          else if (j > pend_p0 && j < pend_p1)
            a[0] = __fadd_rn(a[0], v[j].x), a[1] = __fadd_rn(a[1], v[j].y), a[2] = __fadd_rn(a[2], v[j].z), a[3] = __fadd_rn(a[3], v[j].w);
        if (lane == 0) p.ws.cnt_u[pend_uidx] = 0;
        park(a);
        pend = 3;
      } else {
        pend = 0;
      }
    } else if (pend == 3) {
      __threadfence();
      __syncwarp();
      if (lane == 0) pend_ticket = atomicAdd(p.ws.cnt_y + pend_n16, 1);
      pend = 4;
    } else if (pend == 4) {
      const int ticket = __shfl_sync(0xffffffffu, pend_ticket, 0);
      if (ticket == tab.ntot - 1) {  // the tile's last slot: add its picks in ascending expert id, the shared expert last
        __threadfence();
        const int n16 = pend_n16, ch = lane >> 1, r0 = 4 * (lane & 1);
        const float* yt = p.ws.ypick + (size_t)n16 * 128 + ch * 8 + r0;
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
        if (sh_any) sv = __ldcg(reinterpret_cast<const float4*>(yt + (size_t)kShSlot * NT * 128));
        const float av[4] = {a.x, a.y, a.z, a.w}, svv[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (r0 + c < p.M) {
            const size_t o = (size_t)(r0 + c) * p.H + n16 * 16 + ch;
            const float both = __fadd_rn(av[c], svv[c]);
            p.yr[o] = p.ysum && sh_any ? both : av[c];
            if (sh_any && p.ys) p.ys[o] = svv[c];
            if (p.out) p.out[o] = __float2bfloat16_rn(both);
          }
        if (lane == 0) p.ws.cnt_y[n16] = 0;
      }
      pend = 0;
    }
  };

  for (int it = gw; it < end && !dead; it += GW) {
    int tslot, wslot, n16, b0, b1;
    decode(it, tslot, wslot, n16, b0, b1);
    const bool sh = tslot >= tab.nslots;
    const int p0 = (sh ? sh_b0 : 0) / kPB, p1 = ((sh ? sh_b1 : IB) + kPB - 1) / kPB;  // the unit's pieces
    const int uidx = it / split;
    float tot[4] = {0.f, 0.f, 0.f, 0.f}, pc4[4] = {0.f, 0.f, 0.f, 0.f};
    if (b1 > b0) {
      const bool mx = kMx && !sh;
      const int srow = (n16 * 16) / 128, blk = mx ? kMxBlk : 1024;
      const float sdl = mx ? 1.f : lane < IB ? __ldg(tab.ent[tslot].sd + (size_t)srow * IB + lane) : 0.f;
      const int nc = (b1 - b0) / kKCH, kend = sh ? sh_b1 : IB;
      for (int c = 0; c < nc; ++c) {
        const uint32_t sidx = consumed % kNST;
        if (!mbar_wait(mybar + sidx, (consumed / kNST) & 1)) {
          dead = true;
          break;
        }
        const uint8_t* st = myring + sidx * kDownStage;
#pragma unroll
        for (int b = 0; b < kKCH; ++b) {
          const int kb = b0 + c * kKCH + b;
          const uint8_t* act = st + 2 * kKCH * 1024 + b * kActBlk;
          float d[4];
          if (mx) block_mma_mx(d, st + b * blk, st + kKCH * 1024 + b * blk, act, lane);
          else block_mma(d, st + b * 1024, st + kKCH * 1024 + b * 1024, act, lane);
          const float2 hs = *reinterpret_cast<const float2*>(act + 1024 + 8 * t);
          const float sd = __shfl_sync(0xffffffffu, sdl, kb);
          pc4[0] = fmaf(d[0], sd * hs.x, pc4[0]), pc4[1] = fmaf(d[1], sd * hs.y, pc4[1]);
          pc4[2] = fmaf(d[2], sd * hs.x, pc4[2]), pc4[3] = fmaf(d[3], sd * hs.y, pc4[3]);
          if (piece_end(kb, kend)) {
            if (split == 1) {
              piece_fold(tot, pc4, kb / kPB == p0);
            } else {
              *reinterpret_cast<float4*>(p.ws.part + ((size_t)uidx * kMaxPieces + kb / kPB) * 128 + lane * 4) =
                  make_float4(pc4[0], pc4[1], pc4[2], pc4[3]);
              pc4[0] = pc4[1] = pc4[2] = pc4[3] = 0.f;
            }
          }
        }
        ++consumed;
        __syncwarp();
        if (lane == 0) issue();
        advance();
      }
    }
    if (dead) break;
    while (pend) advance();
    pend_uidx = uidx, pend_wslot = wslot, pend_n16 = n16, pend_p0 = p0, pend_p1 = p1;
    if (split == 1) {
      park(tot);
      pend = 3;
    } else {
      pend = 1;
    }
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

template <class V, bool kMx>
cudaError_t launch_up_f(const DecodeParams& p, cudaStream_t st, bool pdl) {
  static std::atomic<bool> done[64];  // (per device; two host threads may both set the attribute: harmless)
  int dev = 0;
  cudaGetDevice(&dev);
  if (!done[dev & 63].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(k_up_fp8<V, kMx>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    done[dev & 63].store(true, std::memory_order_release);
  }
  const size_t smem = up_smem<V>(p.H);
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  return launch_k(k_up_fp8<V, kMx>, dim3(sm_count()), dim3(V::kThreads), smem, st, pdl, p);
}
template <class V>
cudaError_t launch_up(const DecodeParams& p, cudaStream_t st, bool pdl) {
  return p.mx ? launch_up_f<V, true>(p, st, pdl) : launch_up_f<V, false>(p, st, pdl);
}
template <class V, bool kMx>
cudaError_t launch_down_f(const DecodeParams& p, cudaStream_t st, bool pdl) {
  static std::atomic<bool> done[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (!done[dev & 63].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(k_down_fp8<V, kMx>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)down_smem<V>());
    if (e != cudaSuccess) return e;
    done[dev & 63].store(true, std::memory_order_release);
  }
  return launch_k(k_down_fp8<V, kMx>, dim3(sm_count()), dim3(V::kThreads), down_smem<V>(), st, pdl, p);
}
template <class V>
cudaError_t launch_down(const DecodeParams& p, cudaStream_t st, bool pdl) {
  return p.mx ? launch_down_f<V, true>(p, st, pdl) : launch_down_f<V, false>(p, st, pdl);
}

}  // namespace

// Variants (warps a CTA, 128-k blocks a chunk, ring stages): same bits, different occupancy of the memory system.
static const char* const kUpNames[] = {"w16 k2 s2", "w8 k4 s2", "w8 k2 s5", "w16 k4 s1", "w8 k2 s3", "w16 k1 s5", "w12 k2 s3"};
static const char* const kDownNames[] = {"w16 k2 s2", "w8 k4 s2", "w16 k4 s1", "w16 k1 s4", "w8 k2 s3"};
int decode_fp8_up_variants() { return 7; }
int decode_fp8_down_variants() { return 5; }
const char* decode_fp8_variant_name(int down, int i) {
  if (i < 0 || i >= (down ? 5 : 7)) return nullptr;
  return down ? kDownNames[i] : kUpNames[i];
}

static cudaError_t launch_up_down(const DecodeParams& p, cudaStream_t st, bool pdl, int parts) {
  cudaError_t e = cudaSuccess;
  // a chunk of four blocks needs K to be whole pieces of four blocks
  const int up = (p.H / 128) % 4 && (p.up == 1 || p.up == 3) ? 0 : p.up;
  const int down = (p.I / 128) % 4 && (p.down == 1 || p.down == 2) ? 0 : p.down;
  if (parts & 1) {
    switch (up) {
      case 1: e = launch_up<Var<8, 4, 2>>(p, st, pdl); break;
      case 2: e = launch_up<Var<8, 2, 5>>(p, st, pdl); break;
      case 3: e = launch_up<Var<16, 4, 1>>(p, st, pdl); break;
      case 4: e = launch_up<Var<8, 2, 3>>(p, st, pdl); break;
      case 5: e = launch_up<Var<16, 1, 5>>(p, st, pdl); break;
      case 6: e = launch_up<Var<12, 2, 3>>(p, st, pdl); break;
      default: e = launch_up<Var<16, 2, 2>>(p, st, pdl); break;
    }
    if (e != cudaSuccess) return e;
  }
  if (parts & 2) {
    switch (down) {
      case 1: e = launch_down<Var<8, 4, 2>>(p, st, pdl); break;
      case 2: e = launch_down<Var<16, 4, 1>>(p, st, pdl); break;
      case 3: e = launch_down<Var<16, 1, 4>>(p, st, pdl); break;
      case 4: e = launch_down<Var<8, 2, 3>>(p, st, pdl); break;
      default: e = launch_down<Var<16, 2, 2>>(p, st, pdl); break;
    }
  }
  return e;
}

// The expert step on the caller's idx / w: k_prep (slot table, quantised rows), k_up, k_down.
cudaError_t launch_decode_fp8(const DecodeParams& p, const __nv_bfloat16* x, cudaStream_t st, bool pdl, int parts,
                              const RouteParams* rp, const float* logits, const float* bias) {
  if ((parts & 1) && !(parts & 4)) {  // (bit 2: the table and the quantised rows of an earlier call are still in ws)
    cudaError_t e = rp ? launch_stage_route(p, p.mx ? DSGX_FMT_MXFP4 : DSGX_FMT_FP8, *rp, x, logits, bias, const_cast<int*>(p.idx), const_cast<float*>(p.w), st, pdl)
                       : launch_prep(p, p.mx ? DSGX_FMT_MXFP4 : DSGX_FMT_FP8, x, st, pdl);
    if (e != cudaSuccess) return e;
  }
  return launch_up_down(p, st, pdl, parts & 3);
}

// The whole layer step: k_front (logits, quantised rows, routing, slot table), k_up, k_down (idx / w / logits are outputs of
// the routing).
cudaError_t launch_layer_fp8(const DecodeParams& p, const RouteParams& rp, const __nv_bfloat16* x, const float* wr,
                             const float* bias, float* logits, int* idx, float* w, cudaStream_t st, bool pdl) {
  cudaError_t e = launch_front_route(p, p.mx ? DSGX_FMT_MXFP4 : DSGX_FMT_FP8, rp, x, wr, bias, logits, idx, w, st, pdl);
  if (e != cudaSuccess) return e;
  return launch_up_down(p, st, pdl, 3);
}

}  // namespace dsgx
