// The whole FP8 decode layer step as ONE persistent kernel: router logits, routing, slot table, gate/up with SwiGLU and
// requantisation, down, ordered combine and the final rounding.  One CTA a SM, sixteen warps a CTA, launched once a step.
//
// Why one kernel: at one row the step streams ~231 MB in ~35 us, so every kernel boundary (launch, prologue, pipeline
// fill, tail) costs several per cent.  Here the phases overlap instead:
//   - every CTA quantises x into its own shared memory (no global round trip);
//   - the router's logit slices (one warp per expert and 1024-k slice) and the shared expert's gate/up units (which need
//     no routing) start at once on disjoint warps;
//   - the last M CTAs wait for the logit slices, route one row each (route.cuh: a CTA a row) and the last of them
//     builds the slot table and raises a flag;
//   - every warp then takes its routed gate/up units, and after them its down units; a down unit's weight copies are
//     issued before its slot's h is ready (the weights do not depend on h), only the copy of h waits for the slot's
//     quantisation counter, so the rings keep HBM busy across the gate/up -> down dependency.
// Waits between CTAs (logit slices done, table ready, h of a slot ready) are polls of global counters; every poll is
// bounded (common.cuh kWaitCycles) and a run-out is recorded in the workspace status word.  The grid is at most one CTA
// a SM, so all CTAs become resident together; no CTA waits for work that itself waits for that CTA.
// The last CTA to leave resets every counter, so the workspace is ready for the next launch.
//
// The per-unit arithmetic (block order, scale promotion, rounding points) is that of the separate kernels
// (decode_fp8.cu), so both paths give the same bits.  Activation blocks here hold R = 1, 2, 4 or 8 rows (M rounded up).
#include <atomic>

#include "common.cuh"
#include "decode_common.cuh"
#include "kernels.h"
#include "route.cuh"

namespace dsgx {

namespace {

constexpr int kFW = 16, kFThreads = kFW * 32;
constexpr int kTabSmem = (sizeof(SlotTab) + 127) & ~127;

template <int KCH, int NST>
__global__ void __launch_bounds__(kFThreads, 1) k_step_fp8(const StepParams sp) {
  const DecodeParams& p = sp.d;
  extern __shared__ __align__(128) uint8_t smem[];
  const int R = sp.R, CB = cblk_bytes(R);
  const int HB = p.H / 128, IB = p.I / 128, NT = p.H / 16, upp = p.I / 8;
  const int stage = 2 * KCH * 1024 + ((KCH * CB + 127) & ~127);
  const int xq_bytes = (HB * CB + 127) & ~127;
  uint8_t* xq = smem;
  SlotTab& tab = *reinterpret_cast<SlotTab*>(smem + xq_bytes);
  uint8_t* ringbase = smem + xq_bytes + kTabSmem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ringbase + (size_t)kFW * NST * stage);
  uint64_t* tabbar = bars + kFW * NST;
  int* s_int = reinterpret_cast<int*>(tabbar + 1);  // [0] table loader elected, [1] logit warps done, [2] ticket / poll result
  RouteSmem& rs = *reinterpret_cast<RouteSmem*>(((uintptr_t)(s_int + 4) + 15) & ~(uintptr_t)15);  // 16-byte aligned: vector loads
  int* s_idx = reinterpret_cast<int*>(&rs + 1);
  float* s_w = reinterpret_cast<float*>(s_idx + kMaxRows * kMaxTopK);
  uint32_t* s_bm = reinterpret_cast<uint32_t*>(s_w + kMaxRows * kMaxTopK);
  float* s_red = reinterpret_cast<float*>(s_bm + 16);  // the rows' 1 / rms when the step normalises its input

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  // Work is dealt to warps CTA-interleaved (consecutive work items go to different SMs): one SM pulls at most ~50 GB/s,
  // so a small phase must not sit on a few SMs.
  const int GW = gridDim.x * kFW, gw = warp * gridDim.x + blockIdx.x;
  StepSync* sy = sp.sync;
  uint8_t* myring = ringbase + (size_t)warp * NST * stage;
  uint64_t* mybar = bars + warp * NST;
  uint32_t issued = 0, consumed = 0;
  bool dead = false;

  unsigned long long* stamp = sp.stamps ? sp.stamps + (size_t)(blockIdx.x * kFW + warp) * 8 : nullptr;  // phase timestamps
  if (stamp && lane == 0) stamp[0] = gtime();
  if (lane == 0)
    for (int s = 0; s < NST; ++s) mbar_init(mybar + s, 1);
  if (threadIdx.x == 0) {
    mbar_init(tabbar, 1);
    s_int[0] = 0, s_int[1] = 0, s_int[2] = 0, s_int[3] = 0;
  }
  mbar_fence_init();
  __syncthreads();
  const uint64_t pol = policy_evict_first();
  const int KS = (p.H + 1023) / 1024, ntask = p.E * KS;
  const int nroute = sp.pre_routed ? 0 : p.M;  // the last nroute CTAs route one row each (none when earlier kernels routed)
  const bool router_cta = (int)blockIdx.x >= (int)gridDim.x - nroute;
  const int nrc = (int)gridDim.x - nroute;       // CTAs that do not route
  const int GWn = nrc * kFW;                     // their warps take the logit slices and the shared expert's units
  const int gwn = warp * nrc + blockIdx.x;       // this warp's index among them (valid when !router_cta)
  const int sh_units = sp.has_sh ? upp : 0, sh_down = sp.has_sh ? NT : 0;

  // the RMSNorm in front of the step: every CTA sums the rows' squares itself (it quantises all of x anyway)
  const RowNorm nrm{p.norm.w, s_red + 8 * kMaxRows, p.norm.mode};
  if (p.norm.w) rms_rows_rstd(sp.x, p.M, p.H, p.norm.eps, s_red);

  // ---- the router's logit slices first: they head the longest chain of the step -------------------------------------------
  if (!router_cta && !sp.pre_routed) {
    int mine = 0;
    for (int task = gwn; task < ntask; task += GWn) {
      logit_slice_task(sp.x, sp.wr, p.M, p.H, p.E, task / KS, task % KS, p.ws.lpart, lane, nrm);
      ++mine;
    }
    if (mine) {  // one global add a CTA: its last logit warp reports all of the CTA's slices
      __threadfence();
      __syncwarp();
      if (lane == 0) {
        int nw = 0, nt = 0;  // this CTA's logit warps and slices
        for (int w2 = 0; w2 < kFW; ++w2) {
          const int f = w2 * nrc + (int)blockIdx.x;
          for (int task = f; task < ntask; task += GWn) ++nt, nw += task == f;
        }
        if (atomicAdd(&s_int[1], 1) == nw - 1) atomicAdd(&sy->cnt_lp, nt);
      }
    }
  }
  // ---- every CTA quantises x into its own shared memory (warps take (block, row) tasks as they become free) ---------------
  for (;;) {
    int task = 0;
    if (lane == 0) task = atomicAdd(&s_int[3], 1);
    task = __shfl_sync(0xffffffffu, task, 0);
    if (task >= HB * R) break;
    const int j = task / R, r = task % R;
    float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
    if (r < p.M) {
      const uint2 xv = __ldg(reinterpret_cast<const uint2*>(sp.x + (size_t)r * p.H + 128 * j + 4 * lane));
      v0 = bf16_bits_to_f(xv.x & 0xffffu), v1 = bf16_bits_to_f(xv.x >> 16);
      v2 = bf16_bits_to_f(xv.y & 0xffffu), v3 = bf16_bits_to_f(xv.y >> 16);
      norm4(nrm, r, 128 * j + 4 * lane, v0, v1, v2, v3);
      if (p.norm.w && p.norm.xn_out && blockIdx.x == 0)
        *reinterpret_cast<uint2*>(p.norm.xn_out + (size_t)r * p.H + 128 * j + 4 * lane) = pack_bf16x4(v0, v1, v2, v3);
    }
    cquant_row(xq + j * CB, R, r, lane, r < p.M, v0, v1, v2, v3);
  }
  __syncthreads();
  if (stamp && lane == 0) stamp[1] = gtime();

  // ---- the outstanding ticket of the unit a warp finished last --------------------------------------------------------
  int pend = 0, pend_kind = 0, pend_a = 0, pend_b = 0, pend_ticket = 0;  // kind 1: h group (slot a, group b); 2: tile a
  bool tab_loaded = false;
  auto advance = [&]() {
    if (pend == 1) {
      __threadfence();
      __syncwarp();
      if (lane == 0)
        pend_ticket = pend_kind == 1 ? atomicAdd(p.ws.cnt_h + pend_a * IB + pend_b, 1) : atomicAdd(p.ws.cnt_y + pend_a, 1);
      pend = 2;
    } else if (pend == 2) {
      if (pend_kind == 2 && !tab_loaded) return;  // the tile's slot count is in the table: look again later
      const int ticket = __shfl_sync(0xffffffffu, pend_ticket, 0);
      if (pend_kind == 1 && ticket == 15) {  // the 16th unit of a 128-group of h quantises it and reports the group
        __threadfence();
        const int slot = pend_a, gi = pend_b;
        const __nv_bfloat16* hrow = p.ws.h + (size_t)slot * 8 * p.I + 128 * gi + 4 * lane;
        uint8_t* blk = p.ws.hq + ((size_t)slot * IB + gi) * CB;
        uint2 hv[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
          hv[r] = r < p.M ? __ldcg(reinterpret_cast<const uint2*>(hrow + (size_t)r * p.I)) : make_uint2(0, 0);
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (r < R)
            cquant_row(blk, R, r, lane, r < p.M, bf16_bits_to_f(hv[r].x & 0xffffu), bf16_bits_to_f(hv[r].x >> 16),
                       bf16_bits_to_f(hv[r].y & 0xffffu), bf16_bits_to_f(hv[r].y >> 16));
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          p.ws.cnt_h[slot * IB + gi] = 0;
          atomicAdd(&sy->cnt_hq[slot], 1);
        }
      } else if (pend_kind == 2 && ticket == tab.ntot - 1) {  // the tile's last slot adds its picks in ascending expert id
        __threadfence();
        const int n16 = pend_a, ch = lane >> 1, r0 = 4 * (lane & 1);
        const float* yt = p.ws.ypick + (size_t)n16 * 128 + ch * 8 + r0;
        const bool sh = tab.ntot > tab.nslots;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        int s = 0;
        for (; s + 4 <= tab.nslots; s += 4) {
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
        if (sh) sv = __ldcg(reinterpret_cast<const float4*>(yt + (size_t)sp.sh_slot * NT * 128));
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

  // ---- a warp's sequence of units: static (first, first + stride, ..) or claimed one by one from a global queue ----------
  // (dynamic: a warp that is late takes fewer units; the claim of the unit after next is in flight while a unit streams)
  auto claim = [&](int* q, int prev, int stride) {
    if (!q) return prev + stride;
    int v = 0;
    if (lane == 0) v = atomicAdd(q, 1);
    return v;  // lane 0 only
  };

  // ---- gate/up units.  routed: unit u = slot u / upp, strip u % upp; shared: the shared expert's strips ------------------
  auto up_units = [&](int first, int stride, int total, bool shared, int* q) {
    const int cpu = HB / KCH;
    const size_t strip = (size_t)8 * p.H;
    int u_cur = q ? __shfl_sync(0xffffffffu, claim(q, 0, 0), 0) : first;
    int u_next = q ? 0 : u_cur + stride;   // dynamic: claimed by lane 0 when its producer gets there, not earlier (a
                                           // claim held in reserve is a unit another warp could be streaming)
    int p_on = 0, pc = 0;                  // producer (lane 0): on u_cur (0), on u_next (1), waiting for the consumer (2)
    const uint8_t *pgp = nullptr, *pup = nullptr;
    uint32_t pst = issued % NST;
    auto can_issue = [&]() { return p_on < 2 && (p_on ? u_next : u_cur) < total && issued - consumed < (uint32_t)NST; };
    auto issue = [&]() {
      if (pc == 0) {
        const int u = p_on ? u_next : u_cur;
        const int s = shared ? -1 : u / upp, i8 = u % upp;
        pgp = (shared ? p.sh.g : tab.ent[s].g) + (size_t)i8 * strip;
        pup = (shared ? p.sh.u : tab.ent[s].u) + (size_t)i8 * strip;
      }
      uint8_t* st = myring + (size_t)pst * stage;
      uint64_t* bar = mybar + pst;
      mbar_expect_tx(bar, 2 * KCH * 1024);
      bulk_g2s_hint(st, pgp, KCH * 1024, bar, pol);
      bulk_g2s_hint(st + KCH * 1024, pup, KCH * 1024, bar, pol);
      pgp += KCH * 1024, pup += KCH * 1024;
      ++issued;
      if (++pst == NST) pst = 0;
      if (++pc == cpu) {
        pc = 0;
        if (++p_on == 1 && q) u_next = atomicAdd(q, 1);
      }
    };
    if (lane == 0)
      while (can_issue()) issue();
    while (u_cur < total && !dead) {
      const int s = shared ? -1 : u_cur / upp, i8 = u_cur % upp;
      const int wslot = shared ? sp.sh_slot : s;  // where this unit's h lives in the workspace
      const int srow = (i8 * 8) / 128;
      const float* sgp = shared ? p.sh.gs : tab.ent[s].sg;
      const float* sup = shared ? p.sh.us : tab.ent[s].su;
      const float sgl = lane < HB ? __ldg(sgp + (size_t)srow * HB + lane) : 0.f;
      const float sul = lane < HB ? __ldg(sup + (size_t)srow * HB + lane) : 0.f;
      float tot[4] = {0.f, 0.f, 0.f, 0.f}, pc4[4] = {0.f, 0.f, 0.f, 0.f};  // gate r0, gate r1, up r0, up r1
      for (int c = 0; c < cpu; ++c) {
        const uint32_t sidx = consumed % NST;
        if (!mbar_wait(mybar + sidx, (consumed / NST) & 1)) {
          dead = true;
          break;
        }
        const uint8_t* st = myring + (size_t)sidx * stage;
#pragma unroll
        for (int b = 0; b < KCH; ++b) {
          const int kb = c * KCH + b;
          const uint8_t* act = xq + kb * CB;
          float d[4];
          cblock_mma(d, st + b * 1024, st + KCH * 1024 + b * 1024, act, R, lane);
          const float* xs = reinterpret_cast<const float*>(act + R * 128);
          const float x0 = xs[(2 * t) & (R - 1)], x1 = xs[(2 * t + 1) & (R - 1)];
          const float sg = __shfl_sync(0xffffffffu, sgl, kb), su = __shfl_sync(0xffffffffu, sul, kb);
          pc4[0] = fmaf(d[0], sg * x0, pc4[0]), pc4[1] = fmaf(d[1], sg * x1, pc4[1]);
          pc4[2] = fmaf(d[2], su * x0, pc4[2]), pc4[3] = fmaf(d[3], su * x1, pc4[3]);
          if (piece_end(kb, HB)) piece_fold(tot, pc4, kb < kPB);  // the pieces' order of decode_common.cuh
        }
        ++consumed;
        __syncwarp();
        if (lane == 0 && can_issue()) issue();
        advance();
      }
      if (dead) break;
      while (pend) advance();
      const int ch = i8 * 8 + g, r0 = 2 * t, r1 = 2 * t + 1;
      float g0 = bf16_round(tot[0]), g1 = bf16_round(tot[1]), u0 = bf16_round(tot[2]), u1 = bf16_round(tot[3]);
      swiglu_clamp(g0, u0, p.limit), swiglu_clamp(g1, u1, p.limit);
      float h0 = __fmul_rn(silu(g0), u0), h1 = __fmul_rn(silu(g1), u1);
      if (!shared) h0 = __fmul_rn(tab.ent[s].w[r0], h0), h1 = __fmul_rn(tab.ent[s].w[r1], h1);
      __nv_bfloat16* hrow = p.ws.h + (size_t)wslot * 8 * p.I;
      if (r0 < p.M) hrow[(size_t)r0 * p.I + ch] = __float2bfloat16_rn(h0);
      if (r1 < p.M) hrow[(size_t)r1 * p.I + ch] = __float2bfloat16_rn(h1);
      pend = 1, pend_kind = 1, pend_a = wslot, pend_b = i8 / 16;
      // on to the next unit of the sequence
      u_cur = q ? __shfl_sync(0xffffffffu, u_next, 0) : u_next;
      if (!q) u_next = u_cur + stride;
      if (lane == 0) {
        if (--p_on == 1 && q) u_next = atomicAdd(q, 1);  // the producer had finished the new current unit too
        while (can_issue()) issue();
      }
    }
    if (!dead)
      while (pend) advance();
  };

  // ---- down units (slot, 16 output channels).  Unit v < sh_down: the shared expert's tile v; else routed slot
  // (v - sh_down) / NT.  A unit's weight copies go out first; the copy of h waits for the slot's 128-groups. ---------------
  auto down_units = [&](int first, int stride, int total, int* q) {
    const int cpu = IB / KCH;
    const size_t strip = (size_t)8 * p.I;
    const uint32_t stage_bytes = 2 * KCH * 1024 + KCH * CB;
    int u_cur = q ? __shfl_sync(0xffffffffu, claim(q, 0, 0), 0) : first;
    int u_next = q ? 0 : u_cur + stride;
    int p_on = 0, pc = 0, ready_slot = -1, pslot = 0;
    bool poll_failed = false;
    const uint8_t *pdp = nullptr, *php = nullptr;
    uint32_t pst = issued % NST;
    auto can_issue = [&]() { return p_on < 2 && (p_on ? u_next : u_cur) < total && issued - consumed < (uint32_t)NST; };
    auto issue = [&]() {
      if (pc == 0) {
        const int v = p_on ? u_next : u_cur;
        const bool sh = v < sh_down;
        pslot = sh ? sp.sh_slot : (v - sh_down) / NT;  // the slot's index in the workspace
        const int n16 = sh ? v : (v - sh_down) % NT;
        pdp = (sh ? p.sh.d : tab.ent[pslot].d) + (size_t)(2 * n16) * strip;
        php = p.ws.hq + (size_t)pslot * IB * CB;
      }
      uint8_t* st = myring + (size_t)pst * stage;
      uint64_t* bar = mybar + pst;
      mbar_expect_tx(bar, stage_bytes);
      bulk_g2s_hint(st, pdp, KCH * 1024, bar, pol);
      bulk_g2s_hint(st + KCH * 1024, pdp + strip, KCH * 1024, bar, pol);
      if (ready_slot != pslot && !poll_failed) {
        if (poll_ge(&sy->cnt_hq[pslot], IB)) ready_slot = pslot;
        else poll_failed = true;
        asm volatile("fence.proxy.async;" ::: "memory");  // the bulk copy below reads what other SMs' stores wrote
      }
      if (!poll_failed) bulk_g2s(st + 2 * KCH * 1024, php, KCH * CB, bar);
      pdp += KCH * 1024, php += KCH * CB;
      ++issued;
      if (++pst == NST) pst = 0;
      if (++pc == cpu) {
        pc = 0;
        if (++p_on == 1 && q) u_next = atomicAdd(q, 1);
      }
    };
    if (lane == 0)
      while (can_issue()) issue();
    while (u_cur < total && !dead) {
      const bool sh = u_cur < sh_down;
      const int slot = sh ? sp.sh_slot : (u_cur - sh_down) / NT, n16 = sh ? u_cur : (u_cur - sh_down) % NT;
      const int srow = (n16 * 16) / 128;
      const float* sdp = sh ? p.sh.ds : tab.ent[slot].sd;
      const float sdl = lane < IB ? __ldg(sdp + (size_t)srow * IB + lane) : 0.f;
      float acc[4] = {0.f, 0.f, 0.f, 0.f}, pc4[4] = {0.f, 0.f, 0.f, 0.f};
      for (int c = 0; c < cpu; ++c) {
        const uint32_t sidx = consumed % NST;
        if (!mbar_wait(mybar + sidx, (consumed / NST) & 1)) {
          dead = true;
          break;
        }
        const uint8_t* st = myring + (size_t)sidx * stage;
#pragma unroll
        for (int b = 0; b < KCH; ++b) {
          const int kb = c * KCH + b;
          const uint8_t* act = st + 2 * KCH * 1024 + b * CB;
          float d[4];
          cblock_mma(d, st + b * 1024, st + KCH * 1024 + b * 1024, act, R, lane);
          const float* hs = reinterpret_cast<const float*>(act + R * 128);
          const float h0 = hs[(2 * t) & (R - 1)], h1 = hs[(2 * t + 1) & (R - 1)];
          const float sd = __shfl_sync(0xffffffffu, sdl, kb);
          pc4[0] = fmaf(d[0], sd * h0, pc4[0]), pc4[1] = fmaf(d[1], sd * h1, pc4[1]);
          pc4[2] = fmaf(d[2], sd * h0, pc4[2]), pc4[3] = fmaf(d[3], sd * h1, pc4[3]);
          if (piece_end(kb, IB)) piece_fold(acc, pc4, kb < kPB);
        }
        ++consumed;
        __syncwarp();
        if (lane == 0 && can_issue()) issue();
        advance();
      }
      if (dead) break;
      while (pend) advance();
      float* yt = p.ws.ypick + ((size_t)slot * NT + n16) * 128;
      *reinterpret_cast<float2*>(yt + g * 8 + 2 * t) = make_float2(bf16_round(acc[0]), bf16_round(acc[1]));
      *reinterpret_cast<float2*>(yt + (g + 8) * 8 + 2 * t) = make_float2(bf16_round(acc[2]), bf16_round(acc[3]));
      pend = 1, pend_kind = 2, pend_a = n16;
      u_cur = q ? __shfl_sync(0xffffffffu, u_next, 0) : u_next;
      if (!q) u_next = u_cur + stride;
      if (lane == 0) {
        if (--p_on == 1 && q) u_next = atomicAdd(q, 1);  // the producer had finished the new current unit too
        while (can_issue()) issue();
      }
    }
    if (!dead)
      while (pend) advance();
  };

  // ---- phase 1: logit slices and the shared expert's gate/up units, on disjoint warps -------------------------------------
  if (!router_cta) {
    if (sh_units) {  // shared unit u -> warp (ntask + u) mod GWn
      const int first = ((gwn - ntask % GWn) % GWn + GWn) % GWn;
      up_units(first, GWn, sh_units, true, nullptr);
    }
  } else {
    // ---- phase 2 (router CTAs): wait for the slices, route a row, the last one builds the slot table -------------------
    const int row = (int)blockIdx.x - ((int)gridDim.x - nroute);
    if (threadIdx.x == 0) s_int[2] = poll_ge(&sy->cnt_lp, ntask) ? 1 : 0;
    __syncthreads();
    const bool ok = s_int[2] != 0;
    __syncthreads();
    if (stamp && lane == 0) stamp[6] = gtime();
    if (ok) {
      route_row_cta(sp.rp, p.ws.lpart + (size_t)row * p.E, KS, (size_t)kMaxRows * p.E, sp.bias, rs,
                    sp.logits ? sp.logits + (size_t)row * p.E : nullptr, sp.idx + row * p.topk, sp.w + row * p.topk);
      if (stamp && lane == 0) stamp[7] = gtime();
      bool last = true;
      if (p.M > 1) {  // the last row to be routed builds the table
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) s_int[2] = atomicAdd(&sy->cnt_rt, 1);
        __syncthreads();
        last = s_int[2] == p.M - 1;
        if (last) {
          __threadfence();
          for (int i = threadIdx.x; i < p.M * p.topk; i += kFThreads) s_idx[i] = __ldcg(sp.idx + i), s_w[i] = __ldcg(sp.w + i);
        }
      } else if ((int)threadIdx.x < p.topk) {  // one row: the threads that wrote the picks hand them over
        s_idx[threadIdx.x] = sp.idx[threadIdx.x], s_w[threadIdx.x] = sp.w[threadIdx.x];
      }
      __syncthreads();
      if (last) {
        build_slot_tab(tab, s_bm, s_idx, s_w, p.M, p.topk, p.E, p.e_lo, p.e_hi, p.pool, p.desc, p.sh, DSGX_FMT_FP8);
        if (threadIdx.x == 0 && tab.bad) atomicCAS(p.ws.status, 0, tab.bad);
        {
          const uint4* s4 = reinterpret_cast<const uint4*>(&tab);
          uint4* d4 = reinterpret_cast<uint4*>(p.ws.tab);
          for (int i = threadIdx.x; i < 1 + tab.ntot * 6; i += kFThreads) d4[i] = s4[i];
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0 && !sp.test_no_table) atomicExch(&sy->tab_ready, 1);
      }
    } else {
      dead = true;
    }
    __syncthreads();
  }

  if (stamp && lane == 0) stamp[2] = gtime();
  // ---- phase 3: the slot table into shared memory (the first warp to get here loads it for the CTA) --------------------
  {
    int winner = 0;
    if (lane == 0) winner = atomicCAS(&s_int[0], 0, 1) == 0;
    winner = __shfl_sync(0xffffffffu, winner, 0);
    if (winner) {
      int ok = 0;
      if (lane == 0) ok = !dead && (sp.pre_routed || poll_ge(&sy->tab_ready, 1));
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (ok) {
        load_slot_tab(tab, p.ws.tab, lane);
        __threadfence_block();
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(tabbar)) : "memory");
      }
    }
    if (!mbar_wait(tabbar, 0, 256)) dead = true;
    tab_loaded = !dead;
  }

  if (stamp && lane == 0) stamp[3] = gtime();
  // ---- phase 4: routed gate/up units, continuing the round-robin after the first phase's work ------------------------------
  if (!dead) {
    if (p.M > 2) {
      up_units(0, 0, tab.nslots * upp, false, &sy->q_up);  // claimed from a queue: late warps take fewer
    } else {
      // few units a warp: a fixed deal over the warps that had no shared-expert unit (those are still busy with it)
      const int first = router_cta ? 0 : ((gwn - ntask % GWn) % GWn + GWn) % GWn;
      const int wn = GW - sh_units;  // warps in the deal
      const int pos = router_cta ? (GWn - sh_units) + ((int)blockIdx.x - nrc) * kFW + warp : first - sh_units;
      if (pos >= 0) up_units(pos, wn, tab.nslots * upp, false, nullptr);
    }
  }

  if (stamp && lane == 0) stamp[4] = gtime();
  // ---- phase 5: the routed slots' down units ------------------------------------------------------------------------------
  if (!dead && tab.ntot == 0) {
    for (size_t i = (size_t)blockIdx.x * kFThreads + threadIdx.x; i < (size_t)p.M * p.H; i += (size_t)gridDim.x * kFThreads) {
      p.yr[i] = 0.f;
      if (p.out) p.out[i] = __float2bfloat16_rn(0.f);
    }
  } else if (!dead) {
    if (p.M > 2) down_units(0, 0, sh_down + tab.nslots * NT, &sy->q_down);
    else down_units(gw, GW, sh_down + tab.nslots * NT, nullptr);
  }
  if (dead && lane == 0) atomicCAS(p.ws.status, 0, (int)DSGX_ERR_DEVICE_WAIT);
  if (stamp && lane == 0) stamp[5] = gtime();

  // ---- the last CTA to leave resets the step's counters -------------------------------------------------------------------
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_int[2] = atomicAdd(&sy->cnt_exit, 1);
  __syncthreads();
  if (s_int[2] == (int)gridDim.x - 1) {
    for (int i = threadIdx.x; i < kMaxSlots + 1; i += kFThreads) sy->cnt_hq[i] = 0;
    if (threadIdx.x == 0) sy->cnt_lp = 0, sy->cnt_rt = 0, sy->tab_ready = 0, sy->cnt_exit = 0, sy->q_up = 0, sy->q_down = 0;
  }
}

template <int KCH, int NST>
size_t step_smem(int H, int R) {
  const int CB = cblk_bytes(R);
  const size_t stage = 2 * KCH * 1024 + ((KCH * CB + 127) & ~127);
  return (size_t)(((H / 128) * CB + 127) & ~127) + kTabSmem + (size_t)kFW * NST * stage + (kFW * NST + 1) * 8 + 16 +
         sizeof(RouteSmem) + kMaxRows * kMaxTopK * 8 + 64 + kRmsRed * 4 + 128;
}

template <int KCH, int NST>
cudaError_t launch_step(const StepParams& sp, cudaStream_t st) {
  static std::atomic<bool> done[64];  // (per device; two host threads may both set the attribute: harmless)
  int dev = 0;
  cudaGetDevice(&dev);
  const size_t smem = step_smem<KCH, NST>(sp.d.H, sp.R);
  if (smem > 227 * 1024) return cudaErrorInvalidValue;
  if (!done[dev & 63].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(k_step_fp8<KCH, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    done[dev & 63].store(true, std::memory_order_release);
  }
  k_step_fp8<KCH, NST><<<sm_count(), kFThreads, smem, st>>>(sp);
  return cudaGetLastError();
}

}  // namespace

bool step_fp8_fits(int H, int I, int E, int M) {
  const int KS = (H + 1023) / 1024;
  // the first phase's work must fit the non-routing warps once, and the routing CTAs need a thread per expert
  return E <= kFThreads && M <= kMaxRows && sm_count() > M + 1 && H <= 4096 && I <= 4096 && KS >= 1;
}

cudaError_t launch_step_fp8(StepParams sp, cudaStream_t st) {
  sp.R = rows_pow2(sp.d.M);
  sp.sh_slot = kMaxSlots - 1;
  sp.has_sh = sp.d.sh.g != nullptr;
  if (sp.R == 1) return launch_step<2, 3>(sp, st);
  if (sp.R <= 4) return launch_step<2, 2>(sp, st);
  return launch_step<1, 3>(sp, st);
}

}  // namespace dsgx
