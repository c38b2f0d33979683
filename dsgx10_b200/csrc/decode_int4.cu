// INT4-g32 expert step for 1..8 rows (bf16 activations; the shared expert in bf16): an HBM-bound weight stream with
// in-register dequantisation.
//
// Same structure as the FP8 step (decode_fp8.cu): persistent kernels, one CTA a SM, every warp streams its unit's two
// weight strips through a private ring of bulk async copies and feeds m16n8k16 bf16 MMAs with the weights as the A
// operand (rows 0-7: strip a, rows 8-15: strip b) and the activations as B (16 k x 8 rows).
//
// Weight layouts consumed as they are (the reference's: altar1 engine/experts/layout.h:50-58, 78-107):
//   INT4 block  8 rows x 512 k, 2368 B: 4 units of [32 lanes][16 B] stored nibbles (lane 4 g + t, unit jj: row g,
//               k = 128 jj + 64 q + 16 t + i at byte 8 q + i / 2), bf16 scales at 2048 + 32 g + 16 (t >> 1) + 2 (2 jj + q),
//               zero-point nibble 2 jj + q of the word at 2304 + 8 g + 4 (t >> 1).
//   BF16 block  8 rows x 128 k, 2048 B: the lane's 16 B at 512 p + 16 l are k = 64 (p >> 1) + 16 t + 8 (p & 1) + 0..7.
// The dequantisation contract, W = bf16((u - u_z) * s) with one rounding (formats.cuh:102-119): 0x4300 | u is the bf16
// 128 + u, the subtraction of 128 + u_z is exact, one bf16 multiply rounds the product.  Nibbles i and i + 4 of a word
// are taken together ((w >> 4 i) & 0x000F000F), so a 16-value group reaches the MMAs in the order
// 0,4,1,5,2,6,3,7,8,12,9,13,10,14,11,15; the activation tiles are stored in that order (decode_common.cuh: tile_pos),
// and the bf16 shared expert's words are permuted to it.  A sum over k does not depend on the order the MMA meets the k.
//
//   k_up:   unit = (slot, 8 intermediate channels); g, u rounded to bf16, h = bf16(bf16(silu(g)) * u), stored straight
//           into the bf16 tile the down kernel reads (no quantisation, so no tickets).
//   k_down: unit = (slot, 16 output channels); each pick's f32 output is parked, the tile's last slot adds
//           w_route * y in ascending expert id (a ticket) and the shared expert's output after them.
#include <atomic>

#include "common.cuh"
#include "decode_common.cuh"
#include "kernels.h"

namespace dsgx {

namespace {

constexpr int kI4Blk = 2368, kB16Blk = 2048;
constexpr int kStageW = 2 * kI4Blk;                 // two strips' INT4 block (a bf16 chunk, 2 x 2048 B, fits)
constexpr int kUpStage = (kStageW + 127) & ~127;    // 4864
constexpr int kTabSmem = (sizeof(SlotTab) + 127) & ~127;

template <int W, int NST>
struct VarI {
  static constexpr int kWarps = W, kThreads = W * 32, kNST = NST;
};

DSGX_DEV uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
DSGX_DEV uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
// nibbles i and i + 4 of a word -> the two weights as bf16x2 (zz = 128 + u_z, ss = the group's scale, both halves)
DSGX_DEV uint32_t deq_pair(uint32_t w, int i, uint32_t zz, uint32_t ss) {
  return bf16x2_mul(bf16x2_sub(((w >> (4 * i)) & 0x000F000Fu) | 0x43004300u, zz), ss);
}

struct I4Raw {
  uint4 v[4];  // unit jj's 16 bytes
  uint4 s;     // the lane's eight group scales (bf16), group 2 jj + q at half 2 jj + q
  uint32_t z;  // its eight zero-point nibbles
};
DSGX_DEV void i4_load(I4Raw& r, const uint8_t* blk, int lane) {
#pragma unroll
  for (int jj = 0; jj < 4; ++jj) r.v[jj] = lds128(blk + 512 * jj + 16 * lane);
  const int g = lane >> 2, h = (lane >> 1) & 1;
  r.s = lds128(blk + 2048 + 32 * g + 16 * h);
  r.z = *reinterpret_cast<const uint32_t*>(blk + 2304 + 8 * g + 4 * h);
}
DSGX_DEV uint32_t sel4(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// One INT4 block pair (8 + 8 rows x 512 k) against the activation tile: acc += A B.
// act: the tile's groups of this block, [32 groups][R rows][32 B]; lane (g', t) reads row g' % R.
DSGX_DEV void i4_block_mma(float (&acc)[4], const uint8_t* a, const uint8_t* b, const uint8_t* act, int R, int lane) {
  I4Raw ra, rb;
  i4_load(ra, a, lane);
  i4_load(rb, b, lane);
  const int t = lane & 3, row = (lane >> 2) & (R - 1);
  // the eight zero-point nibbles of each strip as bytes (even groups, odd groups): 128 + u_z in both halves of a word is
  // then one byte permutation a group
  const uint32_t zae = ra.z & 0x0F0F0F0Fu, zao = (ra.z >> 4) & 0x0F0F0F0Fu;
  const uint32_t zbe = rb.z & 0x0F0F0F0Fu, zbo = (rb.z >> 4) & 0x0F0F0F0Fu;
#pragma unroll
  for (int jj = 0; jj < 4; ++jj) {
    const uint32_t sa = sel4(ra.s, jj), sb = sel4(rb.s, jj);
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const uint32_t ssa = __byte_perm(sa, 0, q ? 0x3232 : 0x1010), ssb = __byte_perm(sb, 0, q ? 0x3232 : 0x1010);
      const uint32_t zsel = 0x4040u + 0x0101u * jj;  // bytes (nibble byte jj, 0x43, nibble byte jj, 0x43)
      const uint32_t zza = __byte_perm(q ? zao : zae, 0x43434343u, zsel);
      const uint32_t zzb = __byte_perm(q ? zbo : zbe, 0x43434343u, zsel);
      const uint8_t* xp = act + ((size_t)(8 * jj + 4 * q + t) * R + row) * 32;
      const uint4 x0 = lds128(xp), x1 = lds128(xp + 16);
      const uint32_t alo = sel4(ra.v[jj], 2 * q), ahi = sel4(ra.v[jj], 2 * q + 1);
      const uint32_t blo = sel4(rb.v[jj], 2 * q), bhi = sel4(rb.v[jj], 2 * q + 1);
      mma_bf16(acc, deq_pair(alo, 0, zza, ssa), deq_pair(blo, 0, zzb, ssb), deq_pair(alo, 1, zza, ssa),
               deq_pair(blo, 1, zzb, ssb), x0.x, x0.y);
      mma_bf16(acc, deq_pair(alo, 2, zza, ssa), deq_pair(blo, 2, zzb, ssb), deq_pair(alo, 3, zza, ssa),
               deq_pair(blo, 3, zzb, ssb), x0.z, x0.w);
      mma_bf16(acc, deq_pair(ahi, 0, zza, ssa), deq_pair(bhi, 0, zzb, ssb), deq_pair(ahi, 1, zza, ssa),
               deq_pair(bhi, 1, zzb, ssb), x1.x, x1.y);
      mma_bf16(acc, deq_pair(ahi, 2, zza, ssa), deq_pair(bhi, 2, zzb, ssb), deq_pair(ahi, 3, zza, ssa),
               deq_pair(bhi, 3, zzb, ssb), x1.z, x1.w);
    }
  }
}

// One BF16 block pair (8 + 8 rows x 128 k).  act: [8 groups][R][32 B].
DSGX_DEV void b16_block_mma(float (&acc)[4], const uint8_t* a, const uint8_t* b, const uint8_t* act, int R, int lane) {
  const int t = lane & 3, row = (lane >> 2) & (R - 1);
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const uint4 a0 = lds128(a + 512 * (2 * q) + 16 * lane), a1 = lds128(a + 512 * (2 * q + 1) + 16 * lane);
    const uint4 b0 = lds128(b + 512 * (2 * q) + 16 * lane), b1 = lds128(b + 512 * (2 * q + 1) + 16 * lane);
    const uint8_t* xp = act + ((size_t)(4 * q + t) * R + row) * 32;
    const uint4 x0 = lds128(xp), x1 = lds128(xp + 16);
    // words (v0 v1)(v2 v3)(v4 v5)(v6 v7) -> pairs (v0 v4)(v1 v5)(v2 v6)(v3 v7)
    mma_bf16(acc, __byte_perm(a0.x, a0.z, 0x5410), __byte_perm(b0.x, b0.z, 0x5410), __byte_perm(a0.x, a0.z, 0x7632),
             __byte_perm(b0.x, b0.z, 0x7632), x0.x, x0.y);
    mma_bf16(acc, __byte_perm(a0.y, a0.w, 0x5410), __byte_perm(b0.y, b0.w, 0x5410), __byte_perm(a0.y, a0.w, 0x7632),
             __byte_perm(b0.y, b0.w, 0x7632), x0.z, x0.w);
    mma_bf16(acc, __byte_perm(a1.x, a1.z, 0x5410), __byte_perm(b1.x, b1.z, 0x5410), __byte_perm(a1.x, a1.z, 0x7632),
             __byte_perm(b1.x, b1.z, 0x7632), x1.x, x1.y);
    mma_bf16(acc, __byte_perm(a1.y, a1.w, 0x5410), __byte_perm(b1.y, b1.w, 0x5410), __byte_perm(a1.y, a1.w, 0x7632),
             __byte_perm(b1.y, b1.w, 0x7632), x1.z, x1.w);
  }
}

// Pieces of a shared-expert unit (its K cut in kShSplit): a piece parks its four sums in the workspace and takes a ticket;
// the piece that arrives last adds the parked sums in piece order (the same bits whichever piece that is) and goes on
// with the unit's epilogue (returns true); the others are done (false).
constexpr int kShSplit = 4;
DSGX_DEV bool piece_join(float (&acc)[4], float* part, int* cnt, int unit, int piece, int S, int lane) {
  float* pp = part + (size_t)unit * kMaxPieces * 128 + lane * 4;
  *reinterpret_cast<float4*>(pp + piece * 128) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  __threadfence();
  __syncwarp();
  int ticket = 0;
  if (lane == 0) ticket = atomicAdd(cnt + unit, 1);
  ticket = __shfl_sync(0xffffffffu, ticket, 0);
  if (ticket != S - 1) return false;
  __threadfence();
  float4 v[kShSplit];
#pragma unroll
  for (int j = 0; j < kShSplit; ++j) v[j] = j < S ? __ldcg(reinterpret_cast<const float4*>(pp + j * 128)) : make_float4(0.f, 0.f, 0.f, 0.f);
  acc[0] = v[0].x, acc[1] = v[0].y, acc[2] = v[0].z, acc[3] = v[0].w;
#pragma unroll
  for (int j = 1; j < kShSplit; ++j)
    if (j < S) acc[0] = __fadd_rn(acc[0], v[j].x), acc[1] = __fadd_rn(acc[1], v[j].y), acc[2] = __fadd_rn(acc[2], v[j].z), acc[3] = __fadd_rn(acc[3], v[j].w);
  if (lane == 0) cnt[unit] = 0;
  return true;
}

// -------------------------------------------------------------------------------------------------------------- k_up
template <class V>
__global__ void __launch_bounds__(V::kThreads, 1) k_up_i4(const DecodeParams p) {
  constexpr int kWarps = V::kWarps, kNST = V::kNST;
  extern __shared__ __align__(128) uint8_t smem[];
  const int R = rows_pow2(p.M);
  const int xt_bytes = p.H / 16 * R * 32;
  uint8_t* xt = smem;
  SlotTab& tab = *reinterpret_cast<SlotTab*>(smem + xt_bytes);
  uint8_t* ring = smem + xt_bytes + kTabSmem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + kWarps * kNST * kUpStage);
  uint64_t* cbar = bars + kWarps * kNST;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* myring = ring + warp * kNST * kUpStage;
  uint64_t* mybar = bars + warp * kNST;

  if (lane == 0)
    for (int s = 0; s < kNST; ++s) mbar_init(mybar + s, 1);
  if (threadIdx.x == 0) mbar_init(cbar, 1);
  mbar_fence_init();
  __syncthreads();
  pdl_wait();
  pdl_launch_dependents();  // (after the wait: the down kernel reads the slot table before its own wait)
  if (threadIdx.x == 0) {
    mbar_expect_tx(cbar, (uint32_t)(sizeof(SlotTab) + xt_bytes));
    bulk_g2s(&tab, p.ws.tab, sizeof(SlotTab), cbar);
    bulk_g2s(xt, p.ws.xq, xt_bytes, cbar);
  }
  bool dead = !mbar_wait(cbar, 0);

  const int upp = p.I / 8;
  const int GW = gridDim.x * kWarps, gw = warp * gridDim.x + blockIdx.x;  // consecutive items on different SMs
  const int cpu4 = p.H / 512, cpub = p.H / 128;  // chunks a unit: INT4 blocks, BF16 blocks
  // Items.  A unit of the bf16 shared expert is 3.5 times the bytes of an INT4 unit, and a warp streams at the rate its
  // two ring stages allow: left whole, the 256 warps that hold a shared unit would set the kernel's time.  So the shared
  // expert's units are cut into kShSplit pieces of their K (items 0 .. nshu S - 1, piece-major inside a unit), each summed
  // by its own warp, the piece sums parked in the workspace and added in piece order by the piece that arrives last (a
  // ticket); then the routed units, one item each.  A BF16 layer's units are all alike: no split.
  const bool sh_any = !dead && tab.ntot > tab.nslots;
  const int S = sh_any && !p.b16 && cpub % kShSplit == 0 ? kShSplit : 1;
  const int nshi = sh_any ? upp * S : 0;
  const int total = dead ? 0 : nshi + tab.nslots * upp;
  auto decode = [&](int it, int& slot, int& i8, int& c0, int& c1, int& piece) {
    if (it < nshi) {
      slot = tab.nslots, i8 = it / S, piece = it % S;
      c0 = piece * (cpub / S), c1 = c0 + cpub / S;
    } else {
      const int u = it - nshi;
      slot = u / upp, i8 = u % upp, piece = 0, c0 = 0, c1 = p.b16 ? cpub : cpu4;
    }
  };
  int pu = gw, pc = -1, pc1 = 0, pslot = 0, pi8 = 0;
  uint32_t issued = 0, consumed = 0;
  const uint64_t pol = policy_evict_first();
  auto issue = [&]() {
    if (pc < 0) {
      int piece;
      decode(pu, pslot, pi8, pc, pc1, piece);
    }
    const int slot = pslot, i8 = pi8;
    const bool sh = slot >= tab.nslots, b16 = sh || p.b16;  // (a BF16 layer's routed experts: the shared expert's block format)
    const uint32_t blk = b16 ? kB16Blk : kI4Blk;
    const int cpu = b16 ? cpub : cpu4;
    const size_t off = ((size_t)i8 * cpu + pc) * blk;
    uint8_t* st = myring + (issued % kNST) * kUpStage;
    uint64_t* bar = mybar + issued % kNST;
    mbar_expect_tx(bar, 2 * blk);
    if (sh && tab.bgu) {  // interleaved gate/up rows: the unit's 16 rows are two consecutive 8-row tiles of one matrix
      const uint8_t* gu = tab.ent[slot].g + ((size_t)(2 * i8) * cpu + pc) * blk;
      bulk_g2s_hint(st, gu, blk, bar, pol);
      bulk_g2s_hint(st + kI4Blk, gu + (size_t)cpu * blk, blk, bar, pol);
    } else {
      bulk_g2s_hint(st, tab.ent[slot].g + off, blk, bar, pol);
      bulk_g2s_hint(st + kI4Blk, tab.ent[slot].u + off, blk, bar, pol);
    }
    ++issued;
    if (++pc == pc1) pc = -1, pu += GW;
  };
  if (lane == 0)
    for (int s = 0; s < kNST && pu < total; ++s) issue();

  const int g = lane >> 2, t = lane & 3;
  for (int it = gw; it < total && !dead; it += GW) {
    int slot, i8, c0, c1, piece;
    decode(it, slot, i8, c0, c1, piece);
    const bool sh = slot >= tab.nslots, b16 = sh || p.b16;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = c0; c < c1; ++c) {
      const uint32_t sidx = consumed % kNST;
      if (!mbar_wait(mybar + sidx, (consumed / kNST) & 1)) {
        dead = true;
        break;
      }
      const uint8_t* st = myring + sidx * kUpStage;
      if (b16) b16_block_mma(acc, st, st + kI4Blk, xt + (size_t)c * 8 * R * 32, R, lane);
      else i4_block_mma(acc, st, st + kI4Blk, xt + (size_t)c * 32 * R * 32, R, lane);
      ++consumed;
      __syncwarp();
      if (lane == 0 && pu < total) issue();
    }
    if (dead) break;
    if (sh && S > 1 && !piece_join(acc, p.ws.part, p.ws.cnt_u, i8, piece, S, lane)) continue;  // (not the unit's last piece)
    if (dead) break;
    if (sh && tab.bgu) {
      // interleaved rows: A row 2 j is gate and 2 j + 1 up of the unit's channel j (rows 0-7: channels 0-3, rows 8-15:
      // channels 4-7), so the lanes of an odd row group hand their sums to the even group below them and the even groups
      // end with (gate, up) of channel g / 2 and of channel 4 + g / 2
      float o[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) o[c] = __shfl_down_sync(0xffffffffu, acc[c], 4);
      if (!(g & 1)) {
#pragma unroll
        for (int hi = 0; hi < 2; ++hi) {
          const int ch = i8 * 8 + 4 * hi + (g >> 1);
          uint8_t* hgrp = reinterpret_cast<uint8_t*>(p.ws.h) + ((size_t)slot * (p.I / 16) + ch / 16) * R * 32 + 2 * tile_pos(ch & 15);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int r = 2 * t + c;
            if (r < R) {
              const float h = __fmul_rn(bf16_round(silu(bf16_round(acc[2 * hi + c]))), bf16_round(o[2 * hi + c]));
              *reinterpret_cast<__nv_bfloat16*>(hgrp + (size_t)r * 32) = __float2bfloat16_rn(h);
            }
          }
        }
      }
      continue;
    }
    // g, u rounded to bf16; h = bf16(bf16(silu(g)) * u), into the down kernel's tile
    const int ch = i8 * 8 + g;
    uint8_t* hgrp = reinterpret_cast<uint8_t*>(p.ws.h) + ((size_t)slot * (p.I / 16) + ch / 16) * R * 32 + 2 * tile_pos(ch & 15);
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int r = 2 * t + c;
      if (r < R) {
        const float h = __fmul_rn(bf16_round(silu(bf16_round(acc[c]))), bf16_round(acc[2 + c]));
        *reinterpret_cast<__nv_bfloat16*>(hgrp + (size_t)r * 32) = __float2bfloat16_rn(h);
      }
    }
  }
  if (dead && lane == 0) atomicCAS(p.ws.status, 0, (int)DSGX_ERR_DEVICE_WAIT);
}

// ------------------------------------------------------------------------------------------------------------ k_down
template <class V>
__global__ void __launch_bounds__(V::kThreads, 1) k_down_i4(const DecodeParams p) {
  constexpr int kWarps = V::kWarps, kThreads = V::kThreads, kNST = V::kNST;
  extern __shared__ __align__(128) uint8_t smem[];
  const int R = rows_pow2(p.M), NT = p.H / 16;
  const int stage = (kStageW + R * 1024 + 127) & ~127;
  SlotTab& tab = *reinterpret_cast<SlotTab*>(smem);
  uint8_t* ring = smem + kTabSmem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (size_t)kWarps * kNST * stage);
  uint64_t* cbar = bars + kWarps * kNST;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* myring = ring + (size_t)warp * kNST * stage;
  uint64_t* mybar = bars + warp * kNST;

  pdl_launch_dependents();
  if (lane == 0)
    for (int s = 0; s < kNST; ++s) mbar_init(mybar + s, 1);
  if (threadIdx.x == 0) mbar_init(cbar, 1);
  mbar_fence_init();
  __syncthreads();
  // the slot table is older than the gate/up kernel: it is read, and the first stages' down weights are requested, before
  // the wait for that kernel; only h, its output, is requested after the wait (as in the FP8 down kernel)
  if (threadIdx.x == 0) {
    mbar_expect_tx(cbar, (uint32_t)sizeof(SlotTab));
    bulk_g2s(&tab, p.ws.tab, sizeof(SlotTab), cbar);
  }
  bool dead = !mbar_wait(cbar, 0);

  const int GW = gridDim.x * kWarps, gw = warp * gridDim.x + blockIdx.x;  // consecutive units on different SMs
  if (!dead && tab.ntot == 0) {
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < (size_t)p.M * p.H; i += (size_t)gridDim.x * kThreads) {
      p.yr[i] = 0.f;
      if (p.out) p.out[i] = __float2bfloat16_rn(0.f);
    }
    return;
  }
  const int cpu4 = p.I / 512, cpub = p.I / 128;
  // items as in the gate/up kernel: the shared expert's tiles cut into kShSplit pieces of their K first, then the routed
  // slots' tiles
  const bool sh_any = !dead && tab.ntot > tab.nslots;
  const int S = sh_any && !p.b16 && cpub % kShSplit == 0 ? kShSplit : 1;
  const int nshi = sh_any ? NT * S : 0;
  const int total = dead ? 0 : nshi + tab.nslots * NT;
  auto decode = [&](int it, int& slot, int& n16, int& c0, int& c1, int& piece) {
    if (it < nshi) {
      slot = tab.nslots, n16 = it / S, piece = it % S;
      c0 = piece * (cpub / S), c1 = c0 + cpub / S;
    } else {
      const int u = it - nshi;
      slot = u / NT, n16 = u % NT, piece = 0, c0 = 0, c1 = p.b16 ? cpub : cpu4;
    }
  };
  int pu = gw, pc = -1, pc1 = 0, pslot = 0, pn16 = 0;
  uint32_t issued = 0, consumed = 0;
  const uint64_t pol = policy_evict_first();
  bool early = true;  // before the wait: the h groups of the stages issued now are requested after it
  const uint8_t* late_src[kNST];
  uint32_t late_bytes[kNST];
  auto issue = [&]() {
    if (pc < 0) {
      int piece;
      decode(pu, pslot, pn16, pc, pc1, piece);
    }
    const int slot = pslot, n16 = pn16;
    const bool b16 = slot >= tab.nslots || p.b16;
    const uint32_t blk = b16 ? kB16Blk : kI4Blk;
    const int cpu = b16 ? cpub : cpu4;
    const uint32_t hb = (b16 ? 8 : 32) * R * 32;  // the chunk's h groups
    const size_t off = ((size_t)(2 * n16) * cpu + pc) * blk;
    uint8_t* st = myring + (size_t)(issued % kNST) * stage;
    uint64_t* bar = mybar + issued % kNST;
    mbar_expect_tx(bar, 2 * blk + hb);
    bulk_g2s_hint(st, tab.ent[slot].d + off, blk, bar, pol);
    bulk_g2s_hint(st + kI4Blk, tab.ent[slot].d + off + (size_t)cpu * blk, blk, bar, pol);
    const uint8_t* hsrc = reinterpret_cast<const uint8_t*>(p.ws.h) + ((size_t)slot * (p.I / 16) + (size_t)pc * (b16 ? 8 : 32)) * R * 32;
    if (early) late_src[issued % kNST] = hsrc, late_bytes[issued % kNST] = hb;
    else bulk_g2s(st + kStageW, hsrc, hb, bar);
    ++issued;
    if (++pc == pc1) pc = -1, pu += GW;
  };
  if (lane == 0)
    for (int s = 0; s < kNST && pu < total; ++s) issue();
  pdl_wait();
  if (lane == 0)
    for (uint32_t n = 0; n < issued; ++n) bulk_g2s(myring + (size_t)n * stage + kStageW, late_src[n], late_bytes[n], mybar + n);
  early = false;

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
      if (ticket == tab.ntot - 1) {  // the tile's last slot: yr += w_route * y in ascending expert id, then the shared expert
        __threadfence();
        const int n16 = pend_n16, ch = lane >> 1, r0 = 4 * (lane & 1);
        const float* yt = p.ws.ypick + (size_t)n16 * 128 + ch * 8 + r0;
        const bool sh = tab.ntot > tab.nslots;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < tab.nslots; ++s) {
          const float4 v = __ldcg(reinterpret_cast<const float4*>(yt + (size_t)s * NT * 128));
          const float4 wv = *reinterpret_cast<const float4*>(&tab.ent[s].w[r0]);
          a.x = __fadd_rn(a.x, __fmul_rn(v.x, wv.x)), a.y = __fadd_rn(a.y, __fmul_rn(v.y, wv.y));
          a.z = __fadd_rn(a.z, __fmul_rn(v.z, wv.z)), a.w = __fadd_rn(a.w, __fmul_rn(v.w, wv.w));
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

  for (int it = gw; it < total && !dead; it += GW) {
    int slot, n16, c0, c1, piece;
    decode(it, slot, n16, c0, c1, piece);
    const bool sh = slot >= tab.nslots, b16 = sh || p.b16;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = c0; c < c1; ++c) {
      const uint32_t sidx = consumed % kNST;
      if (!mbar_wait(mybar + sidx, (consumed / kNST) & 1)) {
        dead = true;
        break;
      }
      const uint8_t* st = myring + (size_t)sidx * stage;
      if (b16) b16_block_mma(acc, st, st + kI4Blk, st + kStageW, R, lane);
      else i4_block_mma(acc, st, st + kI4Blk, st + kStageW, R, lane);
      ++consumed;
      __syncwarp();
      if (lane == 0 && pu < total) issue();
      advance();
    }
    if (dead) break;
    while (pend) advance();
    if (sh && S > 1 && !piece_join(acc, p.ws.part, p.ws.cnt_u, n16, piece, S, lane)) continue;  // (not the tile's last piece)
    // the pick's f32 output (not rounded: the contract's down product stays f32)
    float* yt = p.ws.ypick + ((size_t)slot * NT + n16) * 128;
    *reinterpret_cast<float2*>(yt + g * 8 + 2 * t) = make_float2(acc[0], acc[1]);
    *reinterpret_cast<float2*>(yt + (g + 8) * 8 + 2 * t) = make_float2(acc[2], acc[3]);
    pend = 1, pend_n16 = n16;
  }
  if (!dead)
    while (pend) advance();
  if (dead && lane == 0) atomicCAS(p.ws.status, 0, (int)DSGX_ERR_DEVICE_WAIT);
}

template <class V>
size_t up_smem(int H, int R) {
  return (size_t)H / 16 * R * 32 + kTabSmem + (size_t)V::kWarps * V::kNST * kUpStage + (V::kWarps * V::kNST + 1) * 8 + 128;
}
template <class V>
size_t down_smem(int R) {
  const size_t stage = (kStageW + R * 1024 + 127) & ~127;
  return kTabSmem + (size_t)V::kWarps * V::kNST * stage + (V::kWarps * V::kNST + 1) * 8 + 128;
}
constexpr size_t kSmemMax = 227 * 1024;

template <class V>
cudaError_t launch_up(const DecodeParams& p, cudaStream_t st, bool pdl) {
  static std::atomic<bool> done[64];  // (per device; two host threads may both set the attribute: harmless)
  int dev = 0;
  cudaGetDevice(&dev);
  if (!done[dev & 63].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(k_up_i4<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMax);
    if (e != cudaSuccess) return e;
    done[dev & 63].store(true, std::memory_order_release);
  }
  return launch_k(k_up_i4<V>, dim3(sm_count()), dim3(V::kThreads), up_smem<V>(p.H, rows_pow2(p.M)), st, pdl, p);
}
template <class V>
cudaError_t launch_down(const DecodeParams& p, cudaStream_t st, bool pdl) {
  static std::atomic<bool> done[64];  // (per device; two host threads may both set the attribute: harmless)
  int dev = 0;
  cudaGetDevice(&dev);
  if (!done[dev & 63].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(k_down_i4<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemMax);
    if (e != cudaSuccess) return e;
    done[dev & 63].store(true, std::memory_order_release);
  }
  return launch_k(k_down_i4<V>, dim3(sm_count()), dim3(V::kThreads), down_smem<V>(rows_pow2(p.M)), st, pdl, p);
}

}  // namespace

// The widest variant whose shared memory fits (the activation tile grows with the row count and with H).
static cudaError_t launch_up_down(const DecodeParams& p, cudaStream_t st, bool pdl, int parts) {
  const int R = rows_pow2(p.M);
  cudaError_t e = cudaSuccess;
  if (parts & 1) {
    if (up_smem<VarI<16, 2>>(p.H, R) <= kSmemMax) e = launch_up<VarI<16, 2>>(p, st, pdl);
    else if (up_smem<VarI<12, 2>>(p.H, R) <= kSmemMax) e = launch_up<VarI<12, 2>>(p, st, pdl);
    else if (up_smem<VarI<8, 2>>(p.H, R) <= kSmemMax) e = launch_up<VarI<8, 2>>(p, st, pdl);
    else return cudaErrorInvalidValue;
    if (e != cudaSuccess) return e;
  }
  if (parts & 2) {
    if (down_smem<VarI<16, 2>>(R) <= kSmemMax) e = launch_down<VarI<16, 2>>(p, st, pdl);
    else if (down_smem<VarI<12, 2>>(R) <= kSmemMax) e = launch_down<VarI<12, 2>>(p, st, pdl);
    else e = launch_down<VarI<8, 2>>(p, st, pdl);
  }
  return e;
}

bool decode_int4_fits(int H, int M) { return up_smem<VarI<8, 2>>(H, rows_pow2(M)) <= kSmemMax; }

cudaError_t launch_decode_int4(const DecodeParams& p, const __nv_bfloat16* x, cudaStream_t st, bool pdl, int parts,
                               const RouteParams* rp, const float* logits, const float* bias) {
  if (parts & 1) {
    cudaError_t e = rp ? launch_stage_route(p, p.b16 ? DSGX_FMT_BF16 : DSGX_FMT_INT4, *rp, x, logits, bias, const_cast<int*>(p.idx), const_cast<float*>(p.w), st, pdl)
                       : launch_prep(p, p.b16 ? DSGX_FMT_BF16 : DSGX_FMT_INT4, x, st, pdl);
    if (e != cudaSuccess) return e;
  }
  return launch_up_down(p, st, pdl, parts);
}

cudaError_t launch_layer_int4(const DecodeParams& p, const RouteParams& rp, const __nv_bfloat16* x, const float* wr,
                              const float* bias, float* logits, int* idx, float* w, cudaStream_t st, bool pdl) {
  cudaError_t e = launch_front_route(p, p.b16 ? DSGX_FMT_BF16 : DSGX_FMT_INT4, rp, x, wr, bias, logits, idx, w, st, pdl);
  if (e != cudaSuccess) return e;
  return launch_up_down(p, st, pdl, 3);
}

}  // namespace dsgx
