// Device helpers shared by the kernels: PTX wrappers (mbarrier, bulk async copies, programmatic dependent launch,
// FP8 / BF16 warp MMAs), scalar format conversions and the bounded-wait rule.  sm_100a only.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "dsgx_moe.h"

namespace dsgx {

// Every device wait in this library is bounded: after kWaitCycles clock ticks (about a second) the waiting warp
// records DSGX_ERR_DEVICE_WAIT in the workspace's status word and stops consuming; the host reads the word.
constexpr long long kWaitCycles = 2000000000ll;

#define DSGX_DEV __device__ __forceinline__

// ---- shared-memory addresses, mbarriers, bulk copies ------------------------------------------------------------
DSGX_DEV uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

DSGX_DEV void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
DSGX_DEV void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
DSGX_DEV void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
DSGX_DEV bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// the non-blocking test of a phase
DSGX_DEV bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait on a phase; false when the limit ran out.  sleep_ns > 0: back off between tries (for waits that are
// expected to be long, so that the waiting warps leave the issue slots to the warps that work).  A phase that is already
// complete is seen by the non-blocking test, which costs a fraction of a try_wait.
DSGX_DEV bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned sleep_ns = 0) {
  if (mbar_test_wait(bar, parity)) return true;
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (sleep_ns) __nanosleep(sleep_ns);
    if (clock64() - t0 > kWaitCycles) return false;
  }
  return true;
}
// global -> shared bulk copy (the untiled TMA path): both addresses 16-byte aligned, bytes a multiple of 16.
DSGX_DEV void bulk_g2s(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
DSGX_DEV uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
DSGX_DEV void bulk_g2s_hint(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          smem_u32(dst_smem)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// ---- a part of a CTA that works together: the first nt threads (a multiple of 32), with a barrier of their own -----------
// (the whole CTA: nt = blockDim.x, barrier 0 = __syncthreads)
struct CtaPart {
  int nt, bar;
  DSGX_DEV void sync() const {
    if (bar == 0) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(bar), "r"(nt) : "memory");
  }
};
DSGX_DEV CtaPart whole_cta() { return CtaPart{(int)blockDim.x, 0}; }

// ---- programmatic dependent launch ----------------------------------------------------------------------------------
DSGX_DEV void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
DSGX_DEV void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- warp MMAs ------------------------------------------------------------------------------------------------------
// D[16x8] += A[16x32] B[32x8], e4m3 operands, f32 accumulate.  Lane l = 4 g + t: a0 = A[g][4t..4t+3],
// a1 = A[g+8][4t..], a2 = A[g][16+4t..], a3 = A[g+8][16+4t..]; b0 = B[4t..4t+3][g], b1 = B[16+4t..][g];
// d0, d1 = D[g][2t, 2t+1], d2, d3 = D[g+8][2t, 2t+1].
DSGX_DEV void mma_e4m3(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D[16x8] += A[16x16] B[16x8], bf16 operands, f32 accumulate.  a0 = A[g][2t, 2t+1], a1 = A[g+8][2t..],
// a2 = A[g][8+2t..], a3 = A[g+8][8+2t..]; b0 = B[2t, 2t+1][g], b1 = B[8+2t..][g].
DSGX_DEV void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- scalar formats -------------------------------------------------------------------------------------------------
DSGX_DEV float bf16_bits_to_f(uint32_t b) { return __uint_as_float(b << 16); }
DSGX_DEV uint32_t f_to_bf16_bits(float f) {  // round to nearest even
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}
DSGX_DEV float bf16_round(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
DSGX_DEV uint32_t f_to_e4m3(float f) {  // round to nearest even, saturating at +-448
  return (uint32_t)__nv_cvt_float_to_fp8(f, __NV_SATFINITE, __NV_E4M3);
}
// The activation quantisation of the W8A8-g128 contract, one value: q = e4m3(clamp(v / s, +-448)) with an IEEE division.
DSGX_DEV uint32_t quant_e4m3(float v, float s) {
  float t = __fdiv_rn(v, s);
  t = fminf(fmaxf(t, -448.f), 448.f);
  return f_to_e4m3(t);
}
// scale of a block of 128 values from its absolute maximum: max(amax, 1e-4) * (1/448)
DSGX_DEV float act_scale(float amax) { return __fmul_rn(fmaxf(amax, 1e-4f), 1.0f / 448.0f); }
DSGX_DEV float silu(float g) { return __fdiv_rn(g, 1.f + expf(-g)); }
// The SwiGLU clamp on the bf16 gate and up values (ds41f ref/inference/model.py:845-847): up to +-lim, gate from above; lim 0: none.
DSGX_DEV void swiglu_clamp(float& g, float& u, float lim) {
  if (lim > 0.f) u = fminf(fmaxf(u, -lim), lim), g = fminf(g, lim);
}

DSGX_DEV float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// the 32-lane butterfly sum (offsets 16, 8, 4, 2, 1): every lane ends with the same bits
DSGX_DEV float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- RMSNorm pieces (IEEE operations only, so the CPU oracle repeats them bit for bit) ---------------------------------
DSGX_DEV float rms_rstd(float ss, int H, float eps) {
  return __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)H), eps)));
}
// mode 0: bf16(w (x r)); mode 1: bf16(w bf16(x r))
DSGX_DEV float rms_apply(float x, float r, float w, int mode) {
  float xr = __fmul_rn(x, r);
  if (mode == 1) xr = bf16_round(xr);
  return bf16_round(__fmul_rn(w, xr));
}

// ---- host-side launch helper ----------------------------------------------------------------------------------------
#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                            Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = at, cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

}  // namespace dsgx
