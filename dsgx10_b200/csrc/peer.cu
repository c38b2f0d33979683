// Expert parallelism inside one box: the reduction of the ranks' partial sums and the rounding in one kernel over peer
// memory (NVLink through NVSwitch, plain peer loads and stores).  It stands in for the all-reduce the reference issues
// after its expert step (ds41f ref/inference/model.py:901-902, altar1 engine/model/model.cu: the ring reduce before
// gx::finalize) followed by the rounding: every rank ends with out = bf16((sum over ranks, in rank order, of yr) + ys of
// the rank that holds the shared expert).
//
// Protocol, one launch a step on every rank (exactly one of these kernels runs on a GPU at a time; the kernels of one
// step on the different GPUs wait for one another, each wait bounded):
//   1. the step number e is this rank's counter + 1 (the counter lives in the rank's own memory and is bumped by the
//      last CTA of the launch, so every CTA of a launch reads the same value);
//   2. CTA 0 stores e into its word of every rank's flag array (system-scope release: the partial sums of the step, which
//      the kernels before this one on the stream wrote, are visible to whoever sees the flag);
//   3. every CTA waits until all ranks' words in its own flag array have reached e (a rank can be one step ahead, never
//      more: it needs this rank's flag of step e + 1 to finish that step), then adds the ranks' partial sums, read through
//      the peer pointers, and rounds;
//   4. the partial sums are double-buffered by the parity of e: a rank that is one step ahead writes the other half.
#include "common.cuh"
#include "kernels.h"

namespace dsgx {

namespace {

DSGX_DEV uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
DSGX_DEV void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// a load that does not use a line an earlier step may have left in this SM's L1
DSGX_DEV float4 ld_peer4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(256) k_finalize_peers(PeerParams p) {
  __shared__ int ok;
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(p.state) + 1;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < p.world) {
    __threadfence_system();
    st_release_sys(p.flags[threadIdx.x] + p.rank, e);
  }
  if (threadIdx.x < p.world) {
    const uint32_t* f = p.flags[p.rank] + threadIdx.x;
    const long long t0 = clock64();
    while ((int)(ld_acquire_sys(f) - e) < 0) {
      __nanosleep(64);
      if (clock64() - t0 > kWaitCycles) {
        ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (ok && p.outs) {
    // sliced form: this rank's rows only, eight columns a thread, the rounded rows stored into every rank's buffer
    const size_t half = (size_t)2 * p.rows_cap * p.H;
    const size_t off = (size_t)(e & 1) * half;
    const int per = p.H / 8;
    const int lo = (int)((long long)p.rank * p.M / p.world), hi = (int)((long long)(p.rank + 1) * p.M / p.world);
    for (long long i = (long long)lo * per + blockIdx.x * blockDim.x + threadIdx.x; i < (long long)hi * per;
         i += (long long)gridDim.x * blockDim.x) {
      const int r = (int)(i / per), c = (int)(i - (long long)r * per) * 8;
      float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0, s0 = a0, s1 = a0;
      if (p.shared_rank >= 0) {
        const float* sp = p.parts[p.shared_rank] + off + (size_t)(p.rows_cap + r) * p.H + c;
        s0 = ld_peer4(sp), s1 = ld_peer4(sp + 4);
      }
      for (int q0 = 0; q0 < p.world; q0 += 8) {
        float4 v0[8], v1[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (q0 + j < p.world) {
            const float* pp = p.parts[q0 + j] + off + (size_t)r * p.H + c;
            v0[j] = ld_peer4(pp), v1[j] = ld_peer4(pp + 4);
          }
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (q0 + j < p.world) {
            const bool first = q0 + j == 0;
            a0.x = first ? v0[j].x : __fadd_rn(a0.x, v0[j].x), a0.y = first ? v0[j].y : __fadd_rn(a0.y, v0[j].y);
            a0.z = first ? v0[j].z : __fadd_rn(a0.z, v0[j].z), a0.w = first ? v0[j].w : __fadd_rn(a0.w, v0[j].w);
            a1.x = first ? v1[j].x : __fadd_rn(a1.x, v1[j].x), a1.y = first ? v1[j].y : __fadd_rn(a1.y, v1[j].y);
            a1.z = first ? v1[j].z : __fadd_rn(a1.z, v1[j].z), a1.w = first ? v1[j].w : __fadd_rn(a1.w, v1[j].w);
          }
      }
      if (p.shared_rank >= 0) {
        a0.x = __fadd_rn(a0.x, s0.x), a0.y = __fadd_rn(a0.y, s0.y), a0.z = __fadd_rn(a0.z, s0.z), a0.w = __fadd_rn(a0.w, s0.w);
        a1.x = __fadd_rn(a1.x, s1.x), a1.y = __fadd_rn(a1.y, s1.y), a1.z = __fadd_rn(a1.z, s1.z), a1.w = __fadd_rn(a1.w, s1.w);
      }
      const __nv_bfloat162 b0 = __floats2bfloat162_rn(a0.x, a0.y), b1 = __floats2bfloat162_rn(a0.z, a0.w);
      const __nv_bfloat162 b2 = __floats2bfloat162_rn(a1.x, a1.y), b3 = __floats2bfloat162_rn(a1.z, a1.w);
      uint4 o;
      o.x = *reinterpret_cast<const uint32_t*>(&b0), o.y = *reinterpret_cast<const uint32_t*>(&b1);
      o.z = *reinterpret_cast<const uint32_t*>(&b2), o.w = *reinterpret_cast<const uint32_t*>(&b3);
      for (int q = 0; q < p.world; ++q) *reinterpret_cast<uint4*>(p.outs[q] + (size_t)r * p.H + c) = o;
    }
  } else if (ok) {
    const size_t half = (size_t)2 * p.rows_cap * p.H;  // floats of one parity: yr then ys
    const size_t off = (size_t)(e & 1) * half;
    const int per = p.H / 4;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < p.M * per; i += gridDim.x * blockDim.x) {
      const int r = i / per, c = (i - r * per) * 4;
      // every rank's piece is requested before the first add (the loads cross NVLink: one round trip, not one a rank);
      // the adds keep the rank order, the same on every rank
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f), sv = make_float4(0.f, 0.f, 0.f, 0.f);
      if (p.shared_rank >= 0) sv = ld_peer4(p.parts[p.shared_rank] + off + (size_t)(p.rows_cap + r) * p.H + c);
      for (int q0 = 0; q0 < p.world; q0 += 8) {
        float4 v[8], u[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (q0 + j < p.world) {
            v[j] = ld_peer4(p.parts[q0 + j] + off + (size_t)r * p.H + c);
            if (p.shared_rank == -2) u[j] = ld_peer4(p.parts[q0 + j] + off + (size_t)(p.rows_cap + r) * p.H + c);
          }
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (q0 + j < p.world) {
            const bool first = q0 + j == 0;
            a.x = first ? v[j].x : __fadd_rn(a.x, v[j].x), a.y = first ? v[j].y : __fadd_rn(a.y, v[j].y);
            a.z = first ? v[j].z : __fadd_rn(a.z, v[j].z), a.w = first ? v[j].w : __fadd_rn(a.w, v[j].w);
            if (p.shared_rank == -2) {  // every rank holds a part of the shared expert's output: added in rank order
              sv.x = first ? u[j].x : __fadd_rn(sv.x, u[j].x), sv.y = first ? u[j].y : __fadd_rn(sv.y, u[j].y);
              sv.z = first ? u[j].z : __fadd_rn(sv.z, u[j].z), sv.w = first ? u[j].w : __fadd_rn(sv.w, u[j].w);
            }
          }
      }
      if (p.shared_rank == -2)  // ... and rounded to bf16 once, as a whole expert's output is
        sv = make_float4(bf16_round(sv.x), bf16_round(sv.y), bf16_round(sv.z), bf16_round(sv.w));
      if (p.shared_rank >= 0 || p.shared_rank == -2)
        a.x = __fadd_rn(a.x, sv.x), a.y = __fadd_rn(a.y, sv.y), a.z = __fadd_rn(a.z, sv.z), a.w = __fadd_rn(a.w, sv.w);
      const __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
      uint2 o;
      o.x = *reinterpret_cast<const uint32_t*>(&lo), o.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(p.out + (size_t)r * p.H + c) = o;
    }
  } else if (threadIdx.x == 0) {
    atomicCAS(p.status, 0, (int)DSGX_ERR_DEVICE_WAIT);
  }
  // the last CTA of the launch closes the step
  __syncthreads();
  if (threadIdx.x == 0) {
    if (p.outs) __threadfence_system();
    else __threadfence();
    if (atomicAdd(p.state + 1, 1u) == gridDim.x - 1) {
      // every CTA's stores to the peers are fenced (system scope) before its ticket.  If a CTA of this launch gave up its
      // wait (the status word is set before that CTA's ticket), the slice is incomplete: nothing is published, so that the
      // peers' own bounded waits run out and report, instead of reading rows that never arrived.
      if (p.outs && *reinterpret_cast<volatile int*>(p.status) == 0) {
        __threadfence_system();
        for (int q = 0; q < p.world; ++q) st_release_sys(p.done[q] + p.rank, e);
      }
      p.state[1] = 0;
      __threadfence();
      p.state[0] = e;
    }
  }
}

// sliced form, second kernel: every rank's slice of step e (the counter the first kernel just closed) is in this rank's
// output rows
__global__ void __launch_bounds__(32) k_wait_peers(PeerParams p) {
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(p.state);
  if (threadIdx.x < p.world) {
    const uint32_t* f = p.done[p.rank] + threadIdx.x;
    const long long t0 = clock64();
    while ((int)(ld_acquire_sys(f) - e) < 0) {
      __nanosleep(64);
      if (clock64() - t0 > kWaitCycles) {
        atomicCAS(p.status, 0, (int)DSGX_ERR_DEVICE_WAIT);
        break;
      }
    }
  }
}

}  // namespace

cudaError_t launch_finalize_peers(const PeerParams& p, cudaStream_t st) {
  const int n = p.M * (p.H / 4);
  int grid = (n + 255) / 256;
  const int cap = n > (1 << 16) ? 4 * sm_count() : 32;  // decode widths: a few CTAs; a prefill's rows: the whole GPU
  if (grid > cap) grid = cap;
  k_finalize_peers<<<grid, 256, 0, st>>>(p);
  if (p.outs) k_wait_peers<<<1, 32, 0, st>>>(p);
  return cudaGetLastError();
}

}  // namespace dsgx
