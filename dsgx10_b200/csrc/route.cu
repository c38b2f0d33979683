// Router and token-order kernels: logits GEMV with a fixed summation order, score + top-k selection (sigmoid or
// softmax, optional group-limited selection), the stable token -> expert sort, activation quantisation and the final
// rounding.  Integer / f32 CUDA-core work, bound by latency (decode) or by HBM and issue rate (prefill); no tensor
// cores on purpose: the selection must be reproducible bit for bit on a CPU.
#include <atomic>

#include "common.cuh"
#include "kernels.h"
#include "route.cuh"

namespace dsgx {

// ---------------------------------------------------------------------------------------------------- router logits
// One warp computes rows [r0, r0 + 8) x experts [e0, e0 + ET).  Order of every sum (what the CPU oracle restates): K in
// slices of 1024; in a slice lane j accumulates k = base + 128 i + 4 j + c (i ascending, c = 0..3) by fma from zero;
// the 32 lane sums are combined by the xor butterfly; slice sums are added in ascending order.
// The running total of output o = r * ET + j lives in lane o % 32 only (register o / 32), so a wide tile costs two
// registers of totals, not 8 * ET.
template <int ET>
__global__ void __launch_bounds__(256) k_router_logits(const __nv_bfloat16* __restrict__ x, const float* __restrict__ wr,
                                                       int M, int H, int E, float* __restrict__ logits) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int ntE = (E + ET - 1) / ET;
  const int rt = gw / ntE, et = gw % ntE;
  const int r0 = rt * 8, e0 = et * ET;
  if (r0 >= M) return;
  const int nr = min(8, M - r0);
  constexpr int NO = 8 * ET, NTOT = (NO + 31) / 32;
  float total[NTOT];
#pragma unroll
  for (int i = 0; i < NTOT; ++i) total[i] = 0.f;
  for (int base = 0; base < H; base += 1024) {
    const int nit = min(1024, H - base) / 128;
    float acc[8][ET];
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
      for (int j = 0; j < ET; ++j) acc[r][j] = 0.f;
#pragma unroll 1
    for (int i = 0; i < nit; ++i) {
      const int k = base + 128 * i + 4 * lane;
      float4 wv[ET];
#pragma unroll
      for (int j = 0; j < ET; ++j)
        wv[j] = e0 + j < E ? __ldg(reinterpret_cast<const float4*>(wr + (size_t)(e0 + j) * H + k)) : make_float4(0, 0, 0, 0);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < nr) {
          const uint2 xv = __ldg(reinterpret_cast<const uint2*>(x + (size_t)(r0 + r) * H + k));
          const float x0 = bf16_bits_to_f(xv.x & 0xffffu), x1 = bf16_bits_to_f(xv.x >> 16);
          const float x2 = bf16_bits_to_f(xv.y & 0xffffu), x3 = bf16_bits_to_f(xv.y >> 16);
#pragma unroll
          for (int j = 0; j < ET; ++j) {
            float a = acc[r][j];
            a = fmaf(x0, wv[j].x, a);
            a = fmaf(x1, wv[j].y, a);
            a = fmaf(x2, wv[j].z, a);
            a = fmaf(x3, wv[j].w, a);
            acc[r][j] = a;
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
      for (int j = 0; j < ET; ++j) {
        const float s = warp_sum(acc[r][j]);
        constexpr int dummy = 0;
        (void)dummy;
        const int o = r * ET + j;
        if (lane == (o & 31)) total[o >> 5] = base ? __fadd_rn(total[o >> 5], s) : s;
      }
  }
#pragma unroll
  for (int r = 0; r < 8; ++r)
#pragma unroll
    for (int j = 0; j < ET; ++j) {
      const int o = r * ET + j;
      if (lane == (o & 31) && r < nr && e0 + j < E) logits[(size_t)(r0 + r) * E + e0 + j] = total[o >> 5];
    }
}

cudaError_t launch_router_logits(const __nv_bfloat16* x, const float* wr, int M, int H, int E, float* logits,
                                 cudaStream_t st, bool pdl) {
  const int rts = (M + 7) / 8;
  if (M <= 64) {  // decode widths: one expert a warp, as many warps as possible
    const int warps = rts * E;
    return launch_k(k_router_logits<1>, dim3((warps + 7) / 8), dim3(256), 0, st, pdl, x, wr, M, H, E, logits);
  }
  const int warps = rts * ((E + 7) / 8);
  return launch_k(k_router_logits<8>, dim3((warps + 7) / 8), dim3(256), 0, st, pdl, x, wr, M, H, E, logits);
}

// ------------------------------------------------------------------------------------------------------------ route
// One row by one warp (route.cuh).
__global__ void __launch_bounds__(128) k_route(RouteParams p, const float* __restrict__ logits,
                                               const float* __restrict__ bias, int M, int* __restrict__ idx,
                                               float* __restrict__ wout) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= M) return;
  int id;
  float w;
  route_row(p, logits + (size_t)row * p.E, 1, 0, bias, lane, id, w, nullptr);
  if (lane < p.topk) idx[(size_t)row * p.topk + lane] = id, wout[(size_t)row * p.topk + lane] = w;
}

// decode widths: one CTA a row, one thread an expert
__global__ void __launch_bounds__(512) k_route_cta(RouteParams p, const float* __restrict__ logits,
                                                   const float* __restrict__ bias, int* __restrict__ idx,
                                                   float* __restrict__ wout) {
  __shared__ RouteSmem rs;
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  route_row_cta(p, logits + (size_t)row * p.E, 1, 0, bias, rs, nullptr, idx + (size_t)row * p.topk, wout + (size_t)row * p.topk);
}

cudaError_t launch_route(const RouteParams& p, const float* logits, const float* bias, int M, int* idx, float* w,
                         cudaStream_t st, bool pdl) {
  if (M <= 16) return launch_k(k_route_cta, dim3(M), dim3((p.E + 31) / 32 * 32), 0, st, pdl, p, logits, bias, idx, w);
  return launch_k(k_route, dim3((M + 3) / 4), dim3(128), 0, st, pdl, p, logits, bias, M, idx, w);
}

// ------------------------------------------------------------------------------------------------------- sort / pack
// Stable order of the picks by (expert id, token): chunks of kSortTok tokens; per-chunk histograms, an exclusive scan
// expert-major / chunk-minor, then each chunk ranks its own picks with per-expert token bitmaps.  Counts and bitmaps are
// built with shared-memory atomics whose results do not depend on their order, so every output is deterministic.
constexpr int kSortTok = 256;

__global__ void __launch_bounds__(kSortTok) k_sort_count(const int* __restrict__ idx, int T, int topk, int E,
                                                         int* __restrict__ hist, int* __restrict__ err) {
  extern __shared__ int sh[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) sh[e] = 0;
  __syncthreads();
  const int t = blockIdx.x * kSortTok + threadIdx.x;
  if (t < T)
    for (int j = 0; j < topk; ++j) {
      const int e = idx[(size_t)t * topk + j];
      if (e < 0 || e >= E) atomicOr(err, 1);
      else atomicAdd(&sh[e], 1);
    }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[(size_t)blockIdx.x * E + e] = sh[e];
}

// one block: counts, offsets and every (expert, chunk) base
__global__ void __launch_bounds__(512) k_sort_scan(const int* __restrict__ hist, int nchunk, int E, int* __restrict__ counts,
                                                   int* __restrict__ offsets, int* __restrict__ base) {
  __shared__ int tot[512];
  __shared__ int off[513];
  const int e = threadIdx.x;
  int c = 0;
  if (e < E)
    for (int k = 0; k < nchunk; ++k) c += hist[(size_t)k * E + e];
  tot[e] = e < E ? c : 0;
  __syncthreads();
  if (e == 0) {
    int a = 0;
    for (int i = 0; i < E; ++i) off[i] = a, a += tot[i];
    off[E] = a;
  }
  __syncthreads();
  if (e < E) {
    counts[e] = tot[e], offsets[e] = off[e];
    int a = off[e];
    for (int k = 0; k < nchunk; ++k) base[(size_t)k * E + e] = a, a += hist[(size_t)k * E + e];
  }
  if (e == 0) offsets[E] = off[E];
}

__global__ void __launch_bounds__(kSortTok) k_sort_scatter(const int* __restrict__ idx, int T, int topk, int E,
                                                           const int* __restrict__ base, int* __restrict__ perm_tok,
                                                           int* __restrict__ perm_slot, int* __restrict__ pos_of,
                                                           int* __restrict__ row_order) {
  extern __shared__ int sh[];  // [E][kSortTok / 32] token bitmaps
  constexpr int W = kSortTok / 32;
  uint32_t* mask = reinterpret_cast<uint32_t*>(sh);
  for (int i = threadIdx.x; i < E * W; i += blockDim.x) mask[i] = 0;
  __syncthreads();
  const int lt = threadIdx.x, t = blockIdx.x * kSortTok + lt;
  int ex[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    ex[j] = -1;
    if (t < T && j < topk) {
      const int e = idx[(size_t)t * topk + j];
      if (e >= 0 && e < E) ex[j] = e, atomicOr(&mask[e * W + (lt >> 5)], 1u << (lt & 31));
    }
  }
  __syncthreads();
  if (t >= T) return;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    if (ex[j] >= 0) {
      const uint32_t* m = mask + ex[j] * W;
      int rank = __popc(m[lt >> 5] & ((1u << (lt & 31)) - 1u));
      for (int w = 0; w < (lt >> 5); ++w) rank += __popc(m[w]);
      const int pos = base[(size_t)blockIdx.x * E + ex[j]] + rank;
      perm_tok[pos] = t, perm_slot[pos] = j, pos_of[(size_t)t * topk + j] = pos;
    } else if (j < topk) {
      pos_of[(size_t)t * topk + j] = -1;  // (an id outside [0, E): the pick has no place in the order)
    }
  // the row's picks in ascending expert id (insertion sort of at most 8)
  int o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = j;
#pragma unroll
  for (int a = 1; a < 8; ++a)
    if (a < topk) {
      const int v = o[a], ev = ex[v];
      int b = a - 1;
      while (b >= 0 && ex[o[b]] > ev) o[b + 1] = o[b], --b;
      o[b + 1] = v;
    }
  for (int j = 0; j < topk; ++j) row_order[(size_t)t * topk + j] = o[j];
}

size_t sort_ws_bytes(int T, int topk, int E) {
  (void)topk;
  const size_t nchunk = (size_t)(T + kSortTok - 1) / kSortTok;
  return 256 + 2 * nchunk * E * sizeof(int);
}

cudaError_t launch_sort_pack(const int* idx, int T, int topk, int E, int* counts, int* offsets, int* perm_tok,
                             int* perm_slot, int* pos_of, int* row_order, void* ws, cudaStream_t st) {
  const int nchunk = (T + kSortTok - 1) / kSortTok;
  int* err = reinterpret_cast<int*>(ws);
  int* hist = reinterpret_cast<int*>(reinterpret_cast<char*>(ws) + 256);
  int* base = hist + (size_t)nchunk * E;
  cudaError_t e = cudaMemsetAsync(err, 0, 4, st);
  if (e != cudaSuccess) return e;
  k_sort_count<<<nchunk, kSortTok, E * sizeof(int), st>>>(idx, T, topk, E, hist, err);
  k_sort_scan<<<1, 512, 0, st>>>(hist, nchunk, E, counts, offsets, base);
  k_sort_scatter<<<nchunk, kSortTok, (size_t)E * (kSortTok / 32) * sizeof(int), st>>>(idx, T, topk, E, base, perm_tok,
                                                                                      perm_slot, pos_of, row_order);
  return cudaGetLastError();
}

// The same sort with its scratch in a fixed array of this module instead of a caller's workspace: for callers that have
// no device allocator to ask (see dsgx_sort_pack_static).  The array is shared by every call on the device: it keeps
// the last call's histograms (every word a call reads it writes first; only the error word must be zero and is cleared
// by the call), and two calls that overlap on the device race on it.
static __device__ __align__(256) unsigned char g_sort_scratch[kSortStaticBytes];

// set-up, once per device: the array's device address (this may load the module, so the first call is not the one to
// time, and it belongs before any stream capture).  The cache is per device; two host threads that make the first call
// together both look the address up and store the same value.
static cudaError_t sort_scratch_addr(void** out) {
  static std::atomic<void*> addr[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  void* p = dev >= 0 && dev < 64 ? addr[dev].load(std::memory_order_acquire) : nullptr;
  if (!p) {
    e = cudaGetSymbolAddress(&p, g_sort_scratch);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) addr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return cudaSuccess;
}

cudaError_t launch_sort_pack_static(const int* idx, int T, int topk, int E, int* counts, int* offsets, int* perm_tok,
                                    int* perm_slot, int* pos_of, int* row_order, cudaStream_t st) {
  void* p = nullptr;
  cudaError_t e = sort_scratch_addr(&p);
  if (e != cudaSuccess) return e;
  return launch_sort_pack(idx, T, topk, E, counts, offsets, perm_tok, perm_slot, pos_of, row_order, p, st);
}

// the error word of the last static sort on this device (synchronous)
cudaError_t sort_static_status(int* word) {
  void* p = nullptr;
  cudaError_t e = sort_scratch_addr(&p);
  if (e != cudaSuccess) return e;
  return cudaMemcpy(word, p, sizeof(int), cudaMemcpyDeviceToHost);
}

// ------------------------------------------------------------------------------------------ activation quantisation
// x bf16 [M][K] -> blocks of 1056 B, one per 128 k: [2 halves q][32 lanes][16 B] e4m3 codes in the operand order of the
// decode MMAs (lane 4 r + t of half q holds row r, k = 128 j + 64 q + 16 t + 0..15) followed by the 8 rows' f32 scales.
// Rows M..7 are zero.  One warp a (block, row).
__global__ void __launch_bounds__(256) k_act_quant_tiled(const __nv_bfloat16* __restrict__ x, int M, int K,
                                                         uint8_t* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int j = gw >> 3, r = gw & 7;
  if (j >= K / 128) return;
  uint8_t* blk = out + (size_t)j * kActBlk;
  const int kl = 4 * lane, q = kl >> 6, t = (kl >> 4) & 3, i = kl & 15;
  uint32_t packed = 0;
  float sc = 0.f;
  if (r < M) {
    const uint2 xv = __ldg(reinterpret_cast<const uint2*>(x + (size_t)r * K + 128 * j + kl));
    const float v0 = bf16_bits_to_f(xv.x & 0xffffu), v1 = bf16_bits_to_f(xv.x >> 16);
    const float v2 = bf16_bits_to_f(xv.y & 0xffffu), v3 = bf16_bits_to_f(xv.y >> 16);
    const float amax = warp_max(fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3))));
    sc = act_scale(amax);
    packed = quant_e4m3(v0, sc) | quant_e4m3(v1, sc) << 8 | quant_e4m3(v2, sc) << 16 | quant_e4m3(v3, sc) << 24;
  }
  *reinterpret_cast<uint32_t*>(blk + (q * 32 + 4 * r + t) * 16 + i) = packed;
  if (lane == 0) reinterpret_cast<float*>(blk + 1024)[r] = sc;
}

cudaError_t launch_act_quant_tiled(const __nv_bfloat16* x, int M, int K, uint8_t* out, cudaStream_t st, bool pdl) {
  const int warps = (K / 128) * 8;
  return launch_k(k_act_quant_tiled, dim3((warps + 7) / 8), dim3(256), 0, st, pdl, x, M, K, out);
}

// ----------------------------------------------------------------------------------------------------------- finalize
__global__ void __launch_bounds__(256) k_finalize(const float* __restrict__ R, const float* __restrict__ S, size_t n,
                                                  __nv_bfloat16* __restrict__ out, int mode) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float r = R[i], s = S ? S[i] : 0.f;
  out[i] = mode == 1 ? __float2bfloat16_rn(__fadd_rn(bf16_round(r), bf16_round(s))) : __float2bfloat16_rn(__fadd_rn(r, s));
}
// a few KB from mapped host memory into device memory, 16 bytes a thread
__global__ void __launch_bounds__(256) k_copy_in(const uint4* __restrict__ src, uint4* __restrict__ dst, int n) {
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = src[i];
}
cudaError_t launch_copy_in(const void* src, void* dst, size_t bytes, cudaStream_t st) {
  const int n = (int)(bytes / 16);
  return launch_k(k_copy_in, dim3((n + 255) / 256), dim3(256), 0, st, false, reinterpret_cast<const uint4*>(src),
                  reinterpret_cast<uint4*>(dst), n);
}
cudaError_t launch_finalize(const float* R, const float* S, int M, int H, __nv_bfloat16* out, int mode, cudaStream_t st,
                            bool pdl) {
  const size_t n = (size_t)M * H;
  return launch_k(k_finalize, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, pdl, R, S, n, out, mode);
}

}  // namespace dsgx
