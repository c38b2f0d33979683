// Prefill / verify path of the FP8 (W8A8-g128) layer: the experts as grouped GEMMs over token-sorted ragged segments
// on the 5th-generation tensor cores.
//
//   k_quant_scatter  x bf16 [T][H] -> e4m3 [T][H] + f32 scales [T][H/128] (once per token), written to the token's row
//                    and to its picks' rows in the (expert id, token) order of the sort, with the routing weights
//   k_tile_offsets prefix of the 128-row tiles per expert segment
//   k_gemm_fp8     C = A B^T per 256-row tile on a pair of CTAs (a cluster of two, tcgen05 cta_group::2): each CTA stages its
//                  128 rows of A and half of B by TMA (128-byte swizzle) through a 5-stage ring, so every byte of B
//                  crosses into shared memory once for 256 rows; tcgen05.mma kind::f8f6f4 M 256 x N 256 x K 32 issued
//                  by one thread of the pair's first CTA, accumulators in both CTAs' TMEM (two buffers of 256 columns);
//                  after every 128-k block each CTA's eight epilogue warps read the block's partial sums of their 128
//                  rows with tcgen05.ld and promote them into f32 registers with the product of the row's activation
//                  scale and the weight block's scale, while the next block's MMAs fill the other TMEM buffer.  The
//                  scales of a tile are copied into shared memory a tile ahead (template parameter kSS); the launches
//                  of a pass are programmatic dependents of one another.
//                  UP:   B = 128 gate + 128 up channels; epilogue: bf16 rounding, SwiGLU, routing weight, bf16 h,
//                        quantisation of the 128 channels (one scale group) to e4m3.
//                  DOWN: B = 256 output channels; epilogue: every pick's output rounded to bf16.
//   k_combine      per token: the picks' outputs added in f32 in ascending expert id, then the shared expert's.
//
// The weights are read from a K-major row-major copy ([expert][N][K] e4m3, scales [expert][N/128][K/128]) made once at
// load time by k_retile_fp8 from the engine's tile_fp8 blocks (the reference re-tiles its checkpoints the same way:
// ds41f engine/kernels/moe.cu:1187-1265, 1332-1336), because a TMA box wants whole rows.
// No multicast load anywhere: every CTA fetches its own tiles (L2 serves the reuse between pairs); the only multicast is
// the MMA thread's tcgen05.commit, which signals the barriers of both CTAs of its pair.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "kernels.h"

namespace dsgx {

namespace {

// ---- tcgen05 / TMA wrappers ------------------------------------------------------------------------------------------
DSGX_DEV void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                   smem_u32(dst)),
               "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
               : "memory");
}
// the load of one CTA of a pair: the completion may be signalled on the barrier of the pair's other CTA
// (a shared::cluster address)
DSGX_DEV void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}
// shared -> global store of one box (bulk group of the issuing thread)
DSGX_DEV void tma_store_2d(const CUtensorMap* map, int c0, int c1, const void* src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(smem_u32(src)),
               "r"(c0), "r"(c1)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// the issuing thread's earlier stores have read their shared-memory source
DSGX_DEV void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
DSGX_DEV void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
DSGX_DEV void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
DSGX_DEV void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
DSGX_DEV uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the shared::cluster address of a shared-memory object of the cluster's CTA `rank`
DSGX_DEV uint32_t map_to_rank(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
DSGX_DEV void mbar_arrive_cluster(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
DSGX_DEV void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
DSGX_DEV void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
DSGX_DEV void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// arrives on the barrier at this offset in both CTAs of the pair once the MMAs issued so far are complete
DSGX_DEV void tc_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"((uint16_t)3)
               : "memory");
}
DSGX_DEV void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
      "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
DSGX_DEV void cp_async16(void* dst_smem, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
DSGX_DEV void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
DSGX_DEV void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
DSGX_DEV void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile with 128-byte rows and the 128-byte swizzle: rows 128 B apart, 8-row groups 1024 B apart
DSGX_DEV uint64_t umma_desc_sw128(const void* smem) {
  uint64_t d = (uint64_t)((smem_u32(smem) >> 4) & 0x3FFFu);
  d |= (uint64_t)1 << 16;            // leading byte offset (unused for swizzled K-major), 16 B
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset: 8 rows
  d |= (uint64_t)1 << 46;            // descriptor version of this architecture
  d |= (uint64_t)2 << 61;            // SWIZZLE_128B
  return d;
}
// instruction descriptor: f32 accumulate, e4m3 x e4m3, both K-major, M 256 (128 rows in each CTA of the pair), N 256
constexpr uint32_t kIdesc = (1u << 4) | ((256u >> 3) << 17) | ((256u >> 4) << 24);

// warps 0..3: the producer group (warp 0 TMA, warp 1 MMA + TMEM, two spare), warps 4..11: epilogue.  After the set-up the
// producer group gives registers back (40 a thread) and the epilogue warps take them (232 a thread): 384 x 168 in all.
constexpr int kGThreads = 384;
constexpr int kProdRegs = 40, kEpiRegs = 232;
constexpr int kGStages = 5;
constexpr int kATile = 128 * 128, kGStage = 2 * kATile;  // a stage of one CTA: 128 rows of A, 128 of the 256 rows of B

// ---- small kernels -------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_retile_fp8(const uint8_t* __restrict__ tiled, int N, int K, uint8_t* __restrict__ out) {
  // one thread a 16-byte piece: tile_fp8 [N/8][K/128][32 lanes][32 B], lane 4 g + t: row 8 n8 + g, k = 128 j + 64 q + 16 t + i
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)N * K / 16) return;
  const size_t blk = i >> 6;
  const int within = (int)(i & 63), lane = within >> 1, q = within & 1, g = lane >> 2, t = lane & 3;
  const int J = K / 128;
  const int n8 = (int)(blk / J), j = (int)(blk % J);
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(tiled) + i);
  *reinterpret_cast<uint4*>(out + (size_t)(8 * n8 + g) * K + 128 * j + 64 * q + 16 * t) = v;
}

// A quarter warp a (token, 128-k block), a warp four blocks of one token: the block quantised once (e4m3 + its f32
// scale; 16 values a lane) and written to the token's row (the shared expert's operand) and to the row of each of the
// token's picks in the (expert id, token) order of the sort (pos_of), together with the picks' scales and routing
// weights: the routed GEMM's operand without a second pass over the quantised rows.  16-byte loads and stores.
__global__ void __launch_bounds__(256) k_quant_scatter(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                                       const int* __restrict__ pos_of, int T, int K, int topk,
                                                       uint8_t* __restrict__ q, float* __restrict__ s,
                                                       uint8_t* __restrict__ qs, float* __restrict__ ss, float* __restrict__ ws) {
  const int lane = threadIdx.x & 31, l8 = lane & 7;
  const size_t gw = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int KB = K / 128, groups = (KB + 3) / 4;
  if (gw >= (size_t)T * groups) return;
  const size_t r = gw / groups;
  const int j = 4 * (int)(gw % groups) + (lane >> 3);
  const bool on = j < KB;
  const int mypos = lane < topk ? __ldg(pos_of + r * topk + lane) : -1;  // (-1: a pick the sort refused)
  uint4 xa = make_uint4(0, 0, 0, 0), xb = xa;
  if (on) {
    const uint4* src = reinterpret_cast<const uint4*>(x + r * K + 128 * j + 16 * l8);
    xa = __ldg(src), xb = __ldg(src + 1);
  }
  const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
  float v[16];
  float am = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = bf16_bits_to_f(xw[i] & 0xffffu), v[2 * i + 1] = bf16_bits_to_f(xw[i] >> 16);
    am = fmaxf(am, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
  }
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
  const float sc = act_scale(am);
  uint32_t wd[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    wd[i] = quant_e4m3(v[4 * i], sc) | quant_e4m3(v[4 * i + 1], sc) << 8 | quant_e4m3(v[4 * i + 2], sc) << 16 |
            quant_e4m3(v[4 * i + 3], sc) << 24;
  const uint4 word = make_uint4(wd[0], wd[1], wd[2], wd[3]);
  if (on) {
    *reinterpret_cast<uint4*>(q + r * K + 128 * j + 16 * l8) = word;
    if (l8 == 0) s[r * KB + j] = sc;
  }
  for (int jj = 0; jj < topk; ++jj) {
    const int pos = __shfl_sync(0xffffffffu, mypos, jj);
    if (on && pos >= 0) *reinterpret_cast<uint4*>(qs + (size_t)pos * K + 128 * j + 16 * l8) = word;
    if (on && pos >= 0 && l8 == (jj & 7)) ss[(size_t)pos * KB + j] = sc;
  }
  if (lane < topk && mypos >= 0 && gw % groups == 0) ws[mypos] = __ldg(w + r * topk + lane);
}

// The 256-row tiles (128 rows for each CTA of a pair) of the ragged segments: tile_off [E + 1] the prefix of the tiles per
// expert (only this GPU's experts [e_lo, e_hi) get tiles) and, per tile, tile_info = {expert, first row, end of the
// segment's rows, 0}.
__global__ void __launch_bounds__(512) k_tile_offsets(const int* __restrict__ counts, const int* __restrict__ offsets, int E,
                                                      int e_lo, int e_hi, int* __restrict__ tile_off,
                                                      int4* __restrict__ tile_info) {
  __shared__ int pre[513];
  const int e = threadIdx.x;
  const int mine = e < E && e >= e_lo && e < e_hi ? (counts[e] + 255) >> 8 : 0;
  pre[e] = mine;
  __syncthreads();
  if (e == 0) {
    int acc = 0;
    for (int i = 0; i < E; ++i) {
      const int c = pre[i];
      pre[i] = acc, acc += c;
    }
    pre[E] = acc;
  }
  __syncthreads();
  if (e < E) tile_off[e] = pre[e];
  if (e == 0) tile_off[E] = pre[E];  // (E may equal the thread count: no thread has e == E then)
  if (e < E)
    for (int t = 0; t < mine; ++t) tile_info[pre[e] + t] = make_int4(e, offsets[e] + t * 256, offsets[e + 1], 0);
}

// ---- the grouped GEMM ---------------------------------------------------------------------------------------------
struct GemmArgs {
  int mode;            // 0 UP, 1 DOWN
  int K;               // H (UP) or I (DOWN)
  int N;               // I (UP: channels) or H (DOWN)
  int E;               // segments (1 for the shared expert's dense pass)
  int rows_total;      // rows of A
  int wrow0;           // first weight row block: expert e's rows start at (wrow0 + e) * N in the weight tensors
  const int* tile_off;   // [E + 1] 256-row tile prefix of the ragged segments (null: one segment [0, rows_total))
  const int4* tile_info; // per tile {segment, first row, row end, 0} (null with tile_off null)
  const float* sa;     // [rows_total][K / 128] activation scales
  const float* sb0;    // UP: gate scales, DOWN: down scales; [.. experts][N / 128][K / 128]
  const float* sb1;    // UP: up scales
  const float* wrow;   // UP: routing weight of every row (null: none)
  float limit;         // UP: the SwiGLU clamp (0: none)
  uint8_t* hq;         // UP out: e4m3 [rows][N]
  float* hs;           // UP out: [rows][N / 128]
  __nv_bfloat16* y;    // DOWN out: [rows][N]
  int* status;
};

// acc[c] += part[c] * s for 32 columns, two a packed f32 instruction
DSGX_DEV void promote32(float2* acc, const uint32_t (&part)[32], float2 s) {
#pragma unroll
  for (int c = 0; c < 16; ++c)
    acc[c] = __ffma2_rn(make_float2(__uint_as_float(part[2 * c]), __uint_as_float(part[2 * c + 1])), s, acc[c]);
}
// v / s for the quantisation of a group whose scale s is shared: with y = RN(1 / s), q0 = v y and the exact remainder
// v - q0 s, RN(q0 + rem y) is the IEEE quotient (for every bf16 v and every scale this library forms, except quotients
// below 2^-60, which are zero in e4m3 either way).  Two values -> two e4m3 bytes, saturating.
DSGX_DEV uint32_t quant2_e4m3(float v0, float v1, float s, float y) {
  const float q0 = __fmul_rn(v0, y), q1 = __fmul_rn(v1, y);
  const float d0 = __fmaf_rn(__fmaf_rn(-q0, s, v0), y, q0), d1 = __fmaf_rn(__fmaf_rn(-q1, s, v1), y, q1);
  return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(d0, d1), __NV_SATFINITE, __NV_E4M3);
}
// silu with the fast exponential and division (2 ulp each): the result is rounded to bf16 two operations later
DSGX_DEV float silu_fast(float g) { return __fdividef(g, 1.f + __expf(-g)); }
// two floats rounded to bf16 (the values, as floats)
DSGX_DEV float2 bf16_round2(float2 v) { return __bfloat1622float2(__float22bfloat162_rn(v)); }
// acc[c] = part[c] * s: the first block of a tile
DSGX_DEV void promote32_first(float2* acc, const uint32_t (&part)[32], float2 s) {
#pragma unroll
  for (int c = 0; c < 16; ++c)
    acc[c] = __fmul2_rn(make_float2(__uint_as_float(part[2 * c]), __uint_as_float(part[2 * c + 1])), s);
}
// The four MMAs of one 128-k block (K 32 each: the start address moves by 2 x 16 B along the swizzled row), the first
// overwriting the accumulator.  Descriptors as (low word, high word); one asm statement, so that nothing is scheduled
// between the issues.
// cta_group::2: the pair's 256 x 256 tile; A and the accumulator split by rows, B by rows of N, between the two CTAs.
DSGX_DEV void tc_mma_block(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t d_hi, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t.reg .b64 da, db;\n\t.reg .b32 al, bl;\n\t"
      "setp.ne.b32 p0, 0, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], da, db, %4, p0;\n\t"
      "add.u32 al, %1, 2;\n\tadd.u32 bl, %2, 2;\n\tmov.b64 da, {al, %3};\n\tmov.b64 db, {bl, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], da, db, %4, p1;\n\t"
      "add.u32 al, %1, 4;\n\tadd.u32 bl, %2, 4;\n\tmov.b64 da, {al, %3};\n\tmov.b64 db, {bl, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], da, db, %4, p1;\n\t"
      "add.u32 al, %1, 6;\n\tadd.u32 bl, %2, 6;\n\tmov.b64 da, {al, %3};\n\tmov.b64 db, {bl, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], da, db, %4, p1;\n\t}" ::"r"(tmem_d),
      "r"(a_lo), "r"(b_lo), "r"(d_hi), "r"(idesc)
      : "memory");
}

// Shared memory behind the operand ring: barriers, the TMEM address, and the epilogue warps' staging (UP: 2 KB a warp for
// the e4m3 rows, then the row maxima of the two column halves; DOWN: two buffers of 4 KB a warp for the bf16 rows of the
// two column halves).  The staging is laid out as the TMA swizzles want it (64-byte rows: SWIZZLE_64B, 128-byte rows:
// SWIZZLE_128B), which is also free of bank conflicts for a row a lane.
constexpr int kGCtl = 1024;
constexpr int kGStageOut = 8 * 8192;

// kSS: the tile's scales (its rows' activation scales and the two weight-scale rows) are brought into shared memory one
// tile ahead by the epilogue warps' own asynchronous 16-byte copies, so that a block reads them with three shared-memory
// loads; without it every block fetches them from global memory a block ahead, and the epilogue warps (two a scheduler,
// nothing to hide a global load behind) wait for them: 10 % of the gate/up launch.
template <int MODE, bool kSS>
__global__ void __launch_bounds__(kGThreads, 1) k_gemm_fp8(const __grid_constant__ CUtensorMap mapA,
                                                          const __grid_constant__ CUtensorMap mapB0,
                                                          const __grid_constant__ CUtensorMap mapB1,
                                                          const __grid_constant__ CUtensorMap mapOut, const GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kGStages * kGStage);
  uint64_t* empty = full + kGStages;
  uint64_t* tfull = empty + kGStages;
  uint64_t* tempty = tfull + 2;
  uint64_t* xbar = tempty + 2;  // the epilogue warps' exchange of row maxima
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xbar + 1);
  uint8_t* outst = smem + kGStages * kGStage + kGCtl;          // per-warp output staging
  float* amax_x = reinterpret_cast<float*>(outst + 8 * 2048);  // UP: [2 buffers][2 halves][128 rows]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the down launch's staging fills its 64 KB: with the scales in shared memory its ring is one stage shorter and the
  // scales take that stage's place
  constexpr int kRing = MODE == 1 && kSS ? kGStages - 1 : kGStages;

  // The pair: CTA 0 (the leader) issues the MMAs of both; its `full` and `tempty` barriers collect the loads and the
  // epilogue warps of both CTAs; `empty`, `tfull` exist in both CTAs and are signalled by the leader's commits.
  const uint32_t rank = cluster_rank();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kGStages; ++s) mbar_init(full + s, 1), mbar_init(empty + s, 1);
    for (int b = 0; b < 2; ++b) mbar_init(tfull + b, 1), mbar_init(tempty + b, 16);
    mbar_init(xbar, 8);
    mbar_fence_init();
  }
  if (warp == 1) {  // 512 TMEM columns in each CTA: two accumulator buffers of 256
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the other CTA's barriers are initialised before anything is signalled there
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // Launched as a programmatic dependent of the launch before it: the set-up above ran while that launch's last tiles
  // finished; its results (the operands and the tile table read below) are complete from here on.  The launch after
  // this one may set up in the same way as this one's CTAs leave.
  pdl_wait();
  pdl_launch_dependents();

  const int KB = a.K / 128;
  const int ntn = MODE == 0 ? a.N / 128 : a.N / 256;  // n-tiles
  const int mtiles = a.tile_off ? __ldg(a.tile_off + a.E) : (a.rows_total + 255) / 256;
  const int items = mtiles * ntn;
  const int first = blockIdx.x >> 1, stride = gridDim.x >> 1;  // items go round the pairs
  bool dead = false;

  // item -> {segment, first row, row end, n-tile}: one load
  auto locate = [&](int item) -> int4 {
    const int mt = item / ntn;
    int4 r = make_int4(0, mt * 256, a.rows_total, 0);
    if (a.tile_info)  // (a volatile asm: the load is issued here, not where its result is first used)
      asm volatile("ld.global.nc.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(a.tile_info + mt));
    r.w = item - mt * ntn;
    return r;
  };

  if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kProdRegs));
  if (warp == 0) {
    // ---------------------------------------------------------------------------------------------- TMA producer
    // Each CTA loads its 128 rows of A and its half of B (UP: the leader the gate rows, the other CTA the up rows; DOWN:
    // 128 of the 256 output channels each); every load signals the leader's barrier, which expects both CTAs' bytes.
    if (lane == 0) {
      const uint32_t full_leader = map_to_rank(full, 0);
      const CUtensorMap* mapB = MODE == 0 && rank ? &mapB1 : &mapB0;
      uint32_t it = 0;
      for (int item = first; item < items && !dead; item += stride) {
        const int4 ti = locate(item);
        const int arow = ti.y + (int)rank * 128;
        const int brow = (a.wrow0 + ti.x) * a.N + ti.w * (MODE == 0 ? 128 : 256) + (MODE == 0 ? 0 : (int)rank * 128);
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const uint32_t s = it % kRing;
          if (it >= kRing && !mbar_wait(empty + s, ((it / kRing) - 1) & 1)) {
            dead = true;
            break;
          }
          uint8_t* st = smem + s * kGStage;
          if (rank == 0) mbar_expect_tx(full + s, 2 * kGStage);
          tma_load_2d_pair(st, &mapA, kb * 128, arow, full_leader + s * 8);
          tma_load_2d_pair(st + kATile, mapB, kb * 128, brow, full_leader + s * 8);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------------------------------ MMA issuer
    // One thread; the tensor pipe takes an MMA only when the one before has gone in, so whatever this thread does
    // between two blocks is time the pipe may idle: the loop is kept to two barrier waits, one asm statement of four
    // MMAs and two commits.
    if (lane == 0 && rank == 0) {
      const uint64_t d0 = umma_desc_sw128(smem);
      const uint32_t d_hi = (uint32_t)(d0 >> 32), a_lo0 = (uint32_t)d0, b_lo0 = a_lo0 + (kATile >> 4);
      int nblk = 0;
      for (int item = first; item < items; item += stride) nblk += KB;
      for (int it = 0; it < nblk; ++it) {
        const uint32_t s = it % kRing, b = it & 1;
        if (!mbar_wait(full + s, (it / kRing) & 1) || (it >= 2 && !mbar_wait(tempty + b, ((it >> 1) - 1) & 1))) {
          dead = true;
          break;
        }
        tc_fence_after();
        tc_mma_block(tmem + b * 256, a_lo0 + s * (kGStage >> 4), b_lo0 + s * (kGStage >> 4), d_hi, kIdesc);
        tc_commit_pair(empty + s);   // the stage is free (in both CTAs) when these MMAs have read it
        tc_commit_pair(tfull + b);   // and the block's partial sums are in both CTAs' TMEM
      }
    }
  } else if (warp >= 4) {
    // -------------------------------------------------------------------------------------------------- epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kEpiRegs));
    const int ew = warp - 4, quarter = warp & 3, half = ew >> 2;
    const int trow = quarter * 32 + lane;  // the row of this CTA's 128 (TMEM lane) of this thread
    const int crow = (int)rank * 128;      // this CTA's first row in the pair's tile
    const uint32_t tempty_leader = map_to_rank(tempty, 0);
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    uint8_t* stg = outst + ew * (MODE == 0 ? 2048 : 8192);
    uint32_t it = 0, xn = 0;
    int item = first;
    int4 ti = item < items ? locate(item) : make_int4(0, 0, 0, 0);
    // the scales of a block are fetched two blocks ahead of their use; those of a tile's first two blocks before the
    // tail of the tile before
    float pa[2], p0[2], p1[2];
    // kSS: [2 buffers by tile parity][128 rows x (KB + 4) activation scales (the padding spreads the rows over the
    // banks), then the KB + KB weight scales].  Rows are written by the two warps that own them and the weight scales by
    // all eight, each warp all of what it reads: the copies of different warps carry the same bytes.  A warp requests tile
    // i + 1's scales after block 2 of tile i, when every warp of the CTA is past tile i - 1 (the MMAs of block 2 waited for
    // all their arrivals on block 0), whose buffer this is.
    float* const scl = reinterpret_cast<float*>(MODE == 0 ? outst + 8 * 2048 + 2048 : smem + (kGStages - 1) * kGStage);
    const int sstride = KB + 4, sbuf = 128 * sstride + 2 * KB;
    uint32_t tcount = 0;
    auto scale_ptrs = [&](const int4& t, const float*& sap, const float*& sb0p, const float*& sb1p) {
      const int row = t.y + crow + trow;
      sap = a.sa + (size_t)(row < t.z ? row : t.y) * KB;  // (a safe row for the rows past the segment's end)
      const size_t sbase = (size_t)(a.wrow0 + t.x) * (a.N / 128) * KB;
      sb0p = MODE == 0 ? a.sb0 + sbase + (size_t)t.w * KB : a.sb0 + sbase + (size_t)(2 * t.w) * KB;
      sb1p = MODE == 0 ? a.sb1 + sbase + (size_t)t.w * KB : a.sb0 + sbase + (size_t)(2 * t.w + 1) * KB;
    };
    auto first_scales = [&](const int4& t) {
      const float *sap, *sb0p, *sb1p;
      scale_ptrs(t, sap, sb0p, sb1p);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int k = j < KB ? j : 0;
        pa[j] = __ldg(sap + k), p0[j] = __ldg(sb0p + k), p1[j] = __ldg(sb1p + k);
      }
    };
    auto stage_scales = [&](const int4& t, uint32_t buf) {
      const float *sap, *sb0p, *sb1p;
      scale_ptrs(t, sap, sb0p, sb1p);
      float* dst = scl + buf * sbuf;
      for (int c = 0; c < KB / 4; ++c) cp_async16(dst + trow * sstride + 4 * c, sap + 4 * c);
      if (lane < KB / 2) {
        const int which = lane >= KB / 4, c = lane - which * (KB / 4);
        cp_async16(dst + 128 * sstride + which * KB + 4 * c, (which ? sb1p : sb0p) + 4 * c);
      }
      cp_async_commit();
    };
    if (item < items) {
      if constexpr (kSS) stage_scales(ti, 0);
      else first_scales(ti);
    }
    while (item < items && !dead) {
      const int next = item + stride;
      int4 tn = make_int4(0, 0, 0, 0);
      if (next < items) tn = locate(next);  // in flight during this tile's blocks
      const int row0 = ti.y + crow, rend = ti.z, nt = ti.w;
      const int row = row0 + trow;
      const bool live = row < rend;
      const int srow = live ? row : ti.y;
      const float *sap = nullptr, *sb0p = nullptr, *sb1p = nullptr;
      if constexpr (!kSS) scale_ptrs(ti, sap, sb0p, sb1p);
      const float* const scur = scl + (tcount & 1) * sbuf;
      if constexpr (kSS) {  // this tile's scales, requested a tile ago, are there (this warp's copies; the others' are the same)
        cp_async_wait_all();
        __syncwarp();
      }
      float2 acc0[32], acc1[32];  // columns [64 half, 64 half + 64) of the first and of the second 128, in pairs
      // one 128-k block; the tile's first block writes the accumulators (no zeroing pass)
      auto block = [&](auto first_tag, int kb) {
        constexpr bool kFirst = decltype(first_tag)::value;
        const uint32_t b = it & 1;
        float s0, s1;
        if constexpr (kSS) {
          const float sa_k = scur[trow * sstride + kb];
          s0 = sa_k * scur[128 * sstride + kb], s1 = sa_k * scur[128 * sstride + KB + kb];
        } else {
          s0 = pa[0] * p0[0], s1 = pa[0] * p1[0];
          pa[0] = pa[1], p0[0] = p0[1], p1[0] = p1[1];
          if (kb + 2 < KB) pa[1] = __ldg(sap + kb + 2), p0[1] = __ldg(sb0p + kb + 2), p1[1] = __ldg(sb1p + kb + 2);
        }
        if (!mbar_wait(tfull + b, (it >> 1) & 1)) {
          dead = true;
          return;
        }
        tc_fence_after();
        const uint32_t t0 = tmem + lane_addr + b * 256 + half * 64;
        const float2 s02 = make_float2(s0, s0), s12 = make_float2(s1, s1);
        uint32_t r[32], q[32];  // two loads in flight
        tc_ld32(t0, r);
        tc_ld32(t0 + 32, q);
        tc_wait_ld();
        if (kFirst) promote32_first(acc0, r, s02);
        else promote32(acc0, r, s02);
        tc_ld32(t0 + 128, r);
        if (kFirst) promote32_first(acc0 + 16, q, s02);
        else promote32(acc0 + 16, q, s02);
        tc_ld32(t0 + 160, q);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tempty_leader + b * 8);  // the buffer is free for the MMAs of the block after next
        if (kFirst) promote32_first(acc1, r, s12), promote32_first(acc1 + 16, q, s12);
        else promote32(acc1, r, s12), promote32(acc1 + 16, q, s12);
        ++it;
      };
      block(std::true_type{}, 0);
      for (int kb = 1; kb < KB && !dead; ++kb) {
        block(std::false_type{}, kb);
        if constexpr (kSS)
          if (kb == 2 && next < items) stage_scales(tn, (tcount + 1) & 1);
      }
      if (dead) break;
      if constexpr (!kSS)
        if (next < items) first_scales(tn);  // in flight during the tail
      ++tcount;
      const bool warp_live = row0 + quarter * 32 + 31 < rend;  // all 32 rows of this warp: one TMA store; else row by row
      if (lane == 0) tma_store_wait_read();  // the staging is free of the stores of the tile before
      __syncwarp();
      if (MODE == 0) {
        // g, u rounded to bf16; h = bf16(w_route * silu(g) * u); the tile's 128 channels are one quantisation group
        const float wr = a.wrow ? __ldg(a.wrow + srow) : 1.f;
        float am = 0.f;
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          float2 g = bf16_round2(acc0[c]), u = bf16_round2(acc1[c]);
          swiglu_clamp(g.x, u.x, a.limit), swiglu_clamp(g.y, u.y, a.limit);
          float2 h = make_float2(__fmul_rn(silu_fast(g.x), u.x), __fmul_rn(silu_fast(g.y), u.y));
          if (a.wrow) h = make_float2(__fmul_rn(wr, h.x), __fmul_rn(wr, h.y));
          h = bf16_round2(h);
          acc0[c] = h;
          am = fmaxf(am, fmaxf(fabsf(h.x), fabsf(h.y)));
        }
        // the other half's maximum: through shared memory, two buffers by item parity, one bounded barrier an item
        float* ax = amax_x + (xn & 1) * 256;
        ax[half * 128 + trow] = am;
        __syncwarp();
        if (lane == 0) mbar_arrive(xbar);
        if (!mbar_wait(xbar, xn & 1)) {
          dead = true;
          break;
        }
        ++xn;
        const float sc = act_scale(fmaxf(ax[trow], ax[128 + trow]));
        const float rsc = __frcp_rn(sc);
        if (live && half == 0) a.hs[(size_t)row * (a.N / 128) + nt] = sc;
        // the row's 64 bytes into the warp's staging (16-byte units, the 64-byte swizzle)
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint32_t wd[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int c = 8 * v + 2 * k;
            wd[k] = quant2_e4m3(acc0[c].x, acc0[c].y, sc, rsc) | quant2_e4m3(acc0[c + 1].x, acc0[c + 1].y, sc, rsc) << 16;
          }
          *reinterpret_cast<uint4*>(stg + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
        }
        fence_async_smem();
        __syncwarp();
        if (warp_live) {
          if (lane == 0) tma_store_2d(&mapOut, nt * 128 + half * 64, row0 + quarter * 32, stg);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {  // whole 64-byte row pieces a quarter warp: 8 rows a store instruction
            const int rr = 8 * i + (lane >> 2), u = lane & 3;
            const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 64 + ((u ^ ((rr >> 1) & 3)) << 4));
            const int grow = row0 + quarter * 32 + rr;
            if (grow < rend) *reinterpret_cast<uint4*>(a.hq + (size_t)grow * a.N + nt * 128 + half * 64 + u * 16) = v;
          }
          __syncwarp();
        }
      } else {
        // every pick's output rounded to bf16; the row's 128 bytes of each column half into the warp's staging (16-byte
        // units, the 128-byte swizzle), one buffer a half
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint8_t* sb = stg + hh * 4096;
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            uint32_t wd[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 f = hh ? acc1[4 * v + k] : acc0[4 * v + k];
              const __nv_bfloat162 t = __float22bfloat162_rn(f);
              wd[k] = *reinterpret_cast<const uint32_t*>(&t);
            }
            *reinterpret_cast<uint4*>(sb + lane * 128 + ((v ^ (lane & 7)) << 4)) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
          }
          fence_async_smem();
          __syncwarp();
          if (warp_live) {
            if (lane == 0) tma_store_2d(&mapOut, nt * 256 + hh * 128 + half * 64, row0 + quarter * 32, sb);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {  // whole 128-byte lines: 4 rows a store instruction
              const int rr = 4 * i + (lane >> 3), u = lane & 7;
              const uint4 v = *reinterpret_cast<const uint4*>(sb + rr * 128 + ((u ^ (rr & 7)) << 4));
              const int grow = row0 + quarter * 32 + rr;
              if (grow < rend)
                *reinterpret_cast<uint4*>(a.y + (size_t)grow * a.N + nt * 256 + hh * 128 + half * 64 + u * 8) = v;
            }
            __syncwarp();
          }
        }
      }
      ti = tn, item = next;
    }
    if (lane == 0) tma_store_wait_all();
  }
  if (dead && lane == 0) atomicCAS(a.status, 0, (int)DSGX_ERR_DEVICE_WAIT);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still read its shared memory or signal its barriers
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
}

// ---- combine ------------------------------------------------------------------------------------------------------
// (A plain launch: as a programmatic dependent of the last GEMM the pass was 37 us slower.)
// One thread 8 columns of one token: the picks' bf16 outputs added in f32 in ascending expert id, then the shared one.
__global__ void __launch_bounds__(256) k_combine(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ ysh,
                                                 const int* __restrict__ idx, int e_lo, int e_hi,
                                                 const int* __restrict__ pos_of, const int* __restrict__ row_order, int T, int H,
                                                 int topk, float* __restrict__ yr, float* __restrict__ ys,
                                                 __nv_bfloat16* __restrict__ out, int ysum) {
  const int per = H / 8;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)T * per) return;
  const size_t t = i / per;
  const int c = (int)(i % per) * 8;
  // all the picks' rows are fetched before the first add, so that the loads overlap; the adds keep their order
  uint4 v[kMaxTopK];
  bool on[kMaxTopK];
#pragma unroll
  for (int j = 0; j < kMaxTopK; ++j) {
    on[j] = false;
    if (j < topk) {
      const int jj = row_order[t * topk + j];
      const int e = idx[t * topk + jj];
      on[j] = e >= e_lo && e < e_hi;  // else another GPU's expert
      if (on[j]) v[j] = __ldg(reinterpret_cast<const uint4*>(y + (size_t)pos_of[t * topk + jj] * H + c));
    }
  }
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < kMaxTopK; ++j) {
    if (!on[j]) continue;
    const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      acc[2 * k] = __fadd_rn(acc[2 * k], bf16_bits_to_f(w[k] & 0xffffu));
      acc[2 * k + 1] = __fadd_rn(acc[2 * k + 1], bf16_bits_to_f(w[k] >> 16));
    }
  }
  float sh[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (ysh) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(ysh + t * H + c));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) sh[2 * k] = bf16_bits_to_f(w[k] & 0xffffu), sh[2 * k + 1] = bf16_bits_to_f(w[k] >> 16);
  }
  float both[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) both[k] = __fadd_rn(acc[k], sh[k]);
  const bool sum = ysum && ysh;
  if (yr) {  // (a caller that only wants the rounded rows gives no yr: a third of this kernel's traffic)
    float4* yr4 = reinterpret_cast<float4*>(yr + t * H + c);
    yr4[0] = sum ? make_float4(both[0], both[1], both[2], both[3]) : make_float4(acc[0], acc[1], acc[2], acc[3]);
    yr4[1] = sum ? make_float4(both[4], both[5], both[6], both[7]) : make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  if (ys && ysh) {
    float4* ys4 = reinterpret_cast<float4*>(ys + t * H + c);
    ys4[0] = make_float4(sh[0], sh[1], sh[2], sh[3]);
    ys4[1] = make_float4(sh[4], sh[5], sh[6], sh[7]);
  }
  if (out) {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) w[k] = f_to_bf16_bits(both[2 * k]) | f_to_bf16_bits(both[2 * k + 1]) << 16;
    *reinterpret_cast<uint4*>(out + t * H + c) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// ---- host side -------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  }
  return fn;
}

// a [rows][K] e4m3 row-major tensor, boxes of 128 rows x 128 bytes, 128-byte swizzle
bool make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t K) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {K, rows};
  const cuuint64_t strides[1] = {K};
  const cuuint32_t box[2] = {128, 128};
  const cuuint32_t es[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// the epilogue's output boxes of 32 rows: e4m3 h (64 bytes a row, SWIZZLE_64B) or bf16 y (64 values = 128 bytes a row,
// SWIZZLE_128B)
bool make_map_out(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, bool bf16) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * (bf16 ? 2 : 1)};
  const cuuint32_t box[2] = {64, 32};
  const cuuint32_t es[2] = {1, 1};
  return fn(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides,
            box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, bf16 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

constexpr size_t kGemmSmem = (size_t)kGStages * kGStage + 1024 + kGCtl + kGStageOut;  // (UP uses 16 KB + 2 KB of the 64 KB)

// CTA pairs (clusters of two), one pair for two SMs: as many pairs as the device keeps resident at once.
template <int MODE, bool kSS>
cudaError_t launch_gemm_ss(const CUtensorMap& mA, const CUtensorMap& mB0, const CUtensorMap& mB1, const CUtensorMap& mOut,
                           const GemmArgs& a, cudaStream_t st) {
  static int pairs[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2, at[0].val.clusterDim.y = 1, at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.blockDim = dim3(kGThreads), cfg.dynamicSmemBytes = kGemmSmem, cfg.stream = st, cfg.attrs = at, cfg.numAttrs = 1;
  if (!pairs[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(k_gemm_fp8<MODE, kSS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmem);
    if (e != cudaSuccess) return e;
    int n = 0;
    cfg.gridDim = dim3(sm_count() / 2 * 2);
    e = cudaOccupancyMaxActiveClusters(&n, k_gemm_fp8<MODE, kSS>, &cfg);
    if (e != cudaSuccess) return e;
    if (n < 1) return cudaErrorLaunchOutOfResources;
    pairs[dev & 63] = n < sm_count() / 2 ? n : sm_count() / 2;
  }
  cfg.gridDim = dim3(2 * pairs[dev & 63]);
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, k_gemm_fp8<MODE, kSS>, mA, mB0, mB1, mOut, a);
}
// The scales in shared memory: launches whose K is a multiple of 512 (16-byte pieces of the scale rows) and whose two
// buffers fit behind the 18 KB that the gate/up mode uses of the output staging, or in the ring stage the down mode gives up.
template <int MODE>
cudaError_t launch_gemm(const CUtensorMap& mA, const CUtensorMap& mB0, const CUtensorMap& mB1, const CUtensorMap& mOut,
                        const GemmArgs& a, cudaStream_t st) {
  const int KB = a.K / 128;
  const size_t need = 2 * (size_t)(128 * (KB + 4) + 2 * KB) * sizeof(float);
  const size_t room = MODE == 0 ? (size_t)kGStageOut - 8 * 2048 - 2048 : (size_t)kGStage;
  if (KB % 4 == 0 && KB <= 64 && need <= room) return launch_gemm_ss<MODE, true>(mA, mB0, mB1, mOut, a, st);
  return launch_gemm_ss<MODE, false>(mA, mB0, mB1, mOut, a, st);
}

size_t al256(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace

// ---- weights prepared for the prefill path ----------------------------------------------------------------------------
// [E + 1 experts] (index E: the shared expert, absent: E only): gate [I][H], up [I][H], down [H][I] row-major e4m3, then
// the f32 scales in the same order.
size_t prefill_weights_bytes(int H, int I, int E) {
  const size_t n = (size_t)E + 1;
  return 3 * al256(n * I * H) + 3 * al256(n * (I / 128) * (H / 128) * 4);
}
PrefillWeights prefill_weights_carve(void* buf, int H, int I, int E) {
  const size_t n = (size_t)E + 1;
  char* p = reinterpret_cast<char*>(buf);
  PrefillWeights w;
  w.g = reinterpret_cast<uint8_t*>(p), p += al256(n * I * H);
  w.u = reinterpret_cast<uint8_t*>(p), p += al256(n * I * H);
  w.d = reinterpret_cast<uint8_t*>(p), p += al256(n * I * H);
  w.sg = reinterpret_cast<float*>(p), p += al256(n * (I / 128) * (H / 128) * 4);
  w.su = reinterpret_cast<float*>(p), p += al256(n * (I / 128) * (H / 128) * 4);
  w.sd = reinterpret_cast<float*>(p);
  return w;
}

cudaError_t retile_matrix(const uint8_t* tiled, const float* scales, int N, int K, uint8_t* out, float* sout, cudaStream_t st) {
  const size_t pieces = (size_t)N * K / 16;
  k_retile_fp8<<<(unsigned)((pieces + 255) / 256), 256, 0, st>>>(tiled, N, K, out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  return cudaMemcpyAsync(sout, scales, (size_t)(N / 128) * (K / 128) * 4, cudaMemcpyDeviceToDevice, st);
}

// An MXFP4 matrix (576-byte blocks of 8 rows x 128 k: kernels.h, dsgx_moe.h) as the FP8 operand the grouped GEMM reads:
// K-major e4m3 values and one f32 scale per 128 x 128 block, W unchanged.  Every e2m1 value times a power of two is an
// e4m3 value as long as the exponent stays in range: with S = 2^(emax - 6) for the block's largest scale exponent emax, a
// group with exponent e holds v 2^(e - emax + 6), exact for emax - e <= 14 (6 x 2^6 = 384 <= 448; 0.5 x 2^-8 = 2^-9 and
// 1.5 x 2^-8 = 3 x 2^-9 are e4m3 subnormals).  A block whose scales spread wider is reported in *flag and its small groups
// are flushed; the caller refuses the layer.  One CTA a 128 x 128 block.
__global__ void __launch_bounds__(256) k_mx4_to_fp8(const uint8_t* __restrict__ blocks, int N, int K, uint8_t* __restrict__ out,
                                                    float* __restrict__ sout, int* __restrict__ flag) {
  __shared__ int s_max, s_min;
  const int KB = K / 128, nb = blockIdx.x / KB, kb = blockIdx.x % KB;
  if (threadIdx.x == 0) s_max = 0, s_min = 255;
  __syncthreads();
  auto scale_exp = [&](int strip, int g, int G) {  // the group's ue8m0 byte back from its bf16 form
    const uint8_t* b = blocks + ((size_t)(nb * 16 + strip) * KB + kb) * kMxBlk;
    const uint32_t h = *reinterpret_cast<const uint16_t*>(b + 512 + 8 * g + 2 * G);
    return h == 0x40u ? 0 : (int)(h >> 7);
  };
  for (int i = threadIdx.x; i < 512; i += 256) {  // 16 strips x 8 rows x 4 groups
    const int e = scale_exp(i >> 5, (i >> 2) & 7, i & 3);
    atomicMax(&s_max, e), atomicMin(&s_min, e);
  }
  __syncthreads();
  const int emax = s_max;
  if (threadIdx.x == 0) {
    sout[(size_t)nb * KB + kb] = ldexpf(1.f, emax - 127 - 6);
    if (emax - s_min > 14) atomicExch(flag, 1);
  }
  const float mags[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  for (int i = threadIdx.x; i < 2048; i += 256) {  // 16 strips x 32 lanes x 4 groups: one word of 8 values each
    const int strip = i >> 7, lane = (i >> 2) & 31, G = i & 3, g = lane >> 2, t = lane & 3;
    const uint8_t* b = blocks + ((size_t)(nb * 16 + strip) * KB + kb) * kMxBlk;
    const uint32_t w = *reinterpret_cast<const uint32_t*>(b + 16 * lane + 4 * G);
    const float f = ldexpf(1.f, scale_exp(strip, g, G) - emax + 6);
    uint32_t q[2] = {0, 0};
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      const bool neg = (w >> (v < 4 ? 8 * v + 7 : 8 * (v - 4) + 3)) & 1;
      const float val = mags[(w >> (4 * v)) & 7] * f;
      const uint32_t byte = (uint32_t)__nv_cvt_float_to_fp8(neg ? -val : val, __NV_SATFINITE, __NV_E4M3);
      q[v >> 2] |= byte << (8 * (v & 3));
    }
    *reinterpret_cast<uint2*>(out + (size_t)(nb * 128 + strip * 8 + g) * K + kb * 128 + 32 * G + 8 * t) = make_uint2(q[0], q[1]);
  }
}

cudaError_t convert_mx4_matrix(const uint8_t* blocks, int N, int K, uint8_t* out, float* sout, int* flag, cudaStream_t st) {
  k_mx4_to_fp8<<<(unsigned)((N / 128) * (K / 128)), 256, 0, st>>>(blocks, N, K, out, sout, flag);
  return cudaGetLastError();
}

// ---- workspace ---------------------------------------------------------------------------------------------------------
size_t prefill_ws_bytes(int T, int H, int I, int E, int topk) {
  const size_t P = (size_t)T * topk, HB = H / 128, IB = I / 128;
  size_t n = 256;
  n += al256((size_t)T * H) + al256((size_t)T * HB * 4);                           // xq, xs
  n += al256(P * H) + al256(P * HB * 4) + al256(P * 4);                            // sorted xq, xs, w
  n += al256(P * I) + al256(P * IB * 4);                                           // hq, hs (routed)
  n += al256((size_t)T * I) + al256((size_t)T * IB * 4);                           // hq, hs (shared)
  n += al256(P * H * 2) + al256((size_t)T * H * 2);                                // y (routed), y (shared)
  n += 6 * al256(P * 4) + 2 * al256((size_t)(E + 1) * 4) + al256((size_t)(E + 1) * 4);  // sort outputs + tile offsets
  n += al256((P / 128 + E + 1) * 16);                                              // tile table
  n += al256(sort_ws_bytes(T, topk, E));
  return n;
}

PrefillWs prefill_ws_carve(void* ws, int T, int H, int I, int E, int topk) {
  const size_t P = (size_t)T * topk, HB = H / 128, IB = I / 128;
  char* p = reinterpret_cast<char*>(ws);
  PrefillWs w;
  w.status = reinterpret_cast<int*>(p), p += 256;
  w.xq = reinterpret_cast<uint8_t*>(p), p += al256((size_t)T * H);
  w.xs = reinterpret_cast<float*>(p), p += al256((size_t)T * HB * 4);
  w.xq_s = reinterpret_cast<uint8_t*>(p), p += al256(P * H);
  w.xs_s = reinterpret_cast<float*>(p), p += al256(P * HB * 4);
  w.w_s = reinterpret_cast<float*>(p), p += al256(P * 4);
  w.hq = reinterpret_cast<uint8_t*>(p), p += al256(P * I);
  w.hs = reinterpret_cast<float*>(p), p += al256(P * IB * 4);
  w.hq_sh = reinterpret_cast<uint8_t*>(p), p += al256((size_t)T * I);
  w.hs_sh = reinterpret_cast<float*>(p), p += al256((size_t)T * IB * 4);
  w.y = reinterpret_cast<__nv_bfloat16*>(p), p += al256(P * H * 2);
  w.y_sh = reinterpret_cast<__nv_bfloat16*>(p), p += al256((size_t)T * H * 2);
  w.perm_tok = reinterpret_cast<int*>(p), p += al256(P * 4);
  w.perm_slot = reinterpret_cast<int*>(p), p += al256(P * 4);
  w.pos_of = reinterpret_cast<int*>(p), p += al256(P * 4);
  w.row_order = reinterpret_cast<int*>(p), p += 3 * al256(P * 4);
  w.counts = reinterpret_cast<int*>(p), p += al256((size_t)(E + 1) * 4);
  w.offsets = reinterpret_cast<int*>(p), p += al256((size_t)(E + 1) * 4);
  w.tile_off = reinterpret_cast<int*>(p), p += al256((size_t)(E + 1) * 4);
  w.tile_info = reinterpret_cast<int4*>(p), p += al256((P / 128 + E + 1) * 16);
  w.sort_ws = p;
  return w;
}

// ---- the whole prefill expert pass -----------------------------------------------------------------------------------
cudaError_t launch_prefill_fp8(const PrefillParams& q, cudaStream_t st) {
  const int T = q.T, H = q.H, I = q.I, E = q.E, topk = q.topk, P = T * topk;
  const PrefillWs& w = q.ws;
  const PrefillWeights& pw = q.pw;
  CUtensorMap mX, mXs, mHq, mHsh, mG, mU, mD, oHq, oHsh, oY, oYsh;
  const uint64_t nexp = (uint64_t)E + 1;
  if (!make_map(&mX, w.xq, T, H) || !make_map(&mXs, w.xq_s, P, H) || !make_map(&mHq, w.hq, P, I) ||
      !make_map(&mHsh, w.hq_sh, T, I) || !make_map(&mG, pw.g, nexp * I, H) || !make_map(&mU, pw.u, nexp * I, H) ||
      !make_map(&mD, pw.d, nexp * H, I) || !make_map_out(&oHq, w.hq, P, I, false) ||
      !make_map_out(&oHsh, w.hq_sh, T, I, false) || !make_map_out(&oY, w.y, P, H, true) ||
      !make_map_out(&oYsh, w.y_sh, T, H, true))
    return cudaErrorInvalidValue;
  cudaError_t e = cudaSuccess;
  GemmArgs a;
  a.limit = q.limit;
  a.status = w.status;
  const int ph = q.phases;
  if (ph & DSGX_PH_BUCKET) {  // (without it the workspace holds the order and the operands of an earlier call)
  // order, quantise, gather
  e = launch_sort_pack(q.idx, T, topk, E, w.counts, w.offsets, w.perm_tok, w.perm_slot, w.pos_of, w.row_order, w.sort_ws, st);
  if (e != cudaSuccess) return e;
  k_tile_offsets<<<1, 512, 0, st>>>(w.counts, w.offsets, E, q.e_lo, q.e_hi, w.tile_off, w.tile_info);
  {
    const size_t warps = (size_t)T * ((H / 128 + 3) / 4);
    k_quant_scatter<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>(q.x, q.w, w.pos_of, T, H, topk, w.xq, w.xs, w.xq_s,
                                                                          w.xs_s, w.w_s);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  }
  // routed gate/up
  a.mode = 0, a.K = H, a.N = I, a.E = E, a.rows_total = P, a.wrow0 = 0, a.tile_off = w.tile_off, a.tile_info = w.tile_info;
  a.sa = w.xs_s, a.sb0 = pw.sg, a.sb1 = pw.su, a.wrow = w.w_s, a.hq = w.hq, a.hs = w.hs, a.y = nullptr;
  if (ph & DSGX_PH_UP) e = launch_gemm<0>(mXs, mG, mU, oHq, a, st);
  if (e != cudaSuccess) return e;
  // routed down
  a.mode = 1, a.K = I, a.N = H, a.sa = w.hs, a.sb0 = pw.sd, a.sb1 = nullptr, a.wrow = nullptr, a.hq = nullptr, a.hs = nullptr;
  a.y = w.y;
  if (ph & DSGX_PH_DOWN) e = launch_gemm<1>(mHq, mD, mD, oY, a, st);
  if (e != cudaSuccess) return e;
  if (q.has_shared && (ph & DSGX_PH_SHARED)) {
    a.mode = 0, a.K = H, a.N = I, a.E = 1, a.rows_total = T, a.wrow0 = E, a.tile_off = nullptr, a.tile_info = nullptr;
    a.sa = w.xs, a.sb0 = pw.sg, a.sb1 = pw.su, a.wrow = nullptr, a.hq = w.hq_sh, a.hs = w.hs_sh, a.y = nullptr;
    e = launch_gemm<0>(mX, mG, mU, oHsh, a, st);
    if (e != cudaSuccess) return e;
    a.mode = 1, a.K = I, a.N = H, a.sa = w.hs_sh, a.sb0 = pw.sd, a.hq = nullptr, a.hs = nullptr, a.y = w.y_sh;
    e = launch_gemm<1>(mHsh, mD, mD, oYsh, a, st);
    if (e != cudaSuccess) return e;
  }
  if (!(ph & DSGX_PH_COMBINE)) return cudaSuccess;
  const size_t n = (size_t)T * (H / 8);
  k_combine<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(w.y, q.has_shared ? w.y_sh : nullptr, q.idx, q.e_lo, q.e_hi, w.pos_of,
                                                         w.row_order, T, H,
                                                         topk, q.yr, q.ys, q.out, q.ysum);
  return cudaGetLastError();
}

}  // namespace dsgx
