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
#include "decode_common.cuh"
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

// Steps 1-3 of the protocol for one CTA: returns the step number; ok (shared memory) is 0 when a wait ran out.
DSGX_DEV uint32_t peers_arrive_wait(const PeerParams& p, int& ok) {
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
  return e;
}
// The last CTA of the launch closes the step.
DSGX_DEV void peers_close(const PeerParams& p, uint32_t e) {
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

__global__ void __launch_bounds__(256) k_finalize_peers(PeerParams p) {
  __shared__ int ok;
  // (a plain launch: as a programmatic dependent of the down kernel the step was 3.4 us slower on four GPUs, measured)
  const uint32_t e = peers_arrive_wait(p, ok);
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
  peers_close(p, e);
}

// ---------------------------------------------------------------------------------------------- reduce + add + RMSNorm
// What follows the experts in both engines, in the same kernel as the reduction (altar1 engine/comm/glmcoll.cu:225-330,
// allreduce_add_norm: the all-reduce's consumer adds the residual and normalises for the next block; ds41f
// ref/inference/model.py: x = x + ffn(x), then the next block's norm): for every row
//   v = the ranks' partial sums added in rank order (+ the shared expert's, as k_finalize_peers), out = bf16(v),
//   h = bf16(res + out)   (add_f32: bf16(res + v)),   normed = RMSNorm(h) with the row's sum of squares in the order of
//   rms_rows_rstd (chunks of 8 columns, chunk c to thread c mod 256).
// One CTA a row, eight columns a thread and chunk, the row's h kept in registers between the two passes.
// kPeers = false: one GPU, v = R + S from this GPU's own buffers (fin_mode as dsgx_finalize), no protocol.
constexpr int kNormChunks = 4;  // H <= 8192
DSGX_DEV float4 add4(const float4& a, const float4& b) {
  return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}
DSGX_DEV float4 round4(const float4& a) { return make_float4(bf16_round(a.x), bf16_round(a.y), bf16_round(a.z), bf16_round(a.w)); }

// the reduced f32 sums of eight columns of one row (v0: columns c..c+3, v1: c+4..c+7)
DSGX_DEV void peers_sum8(const PeerParams& p, size_t off, int r, int c, float4& v0, float4& v1) {
  float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0;
  if (p.shared_rank >= 0) {
    const float* sp = p.parts[p.shared_rank] + off + (size_t)(p.rows_cap + r) * p.H + c;
    s0 = ld_peer4(sp), s1 = ld_peer4(sp + 4);
  }
  for (int q0 = 0; q0 < p.world; q0 += 4) {
    float4 a0[4], a1[4], u0[4], u1[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (q0 + j < p.world) {
        const float* pp = p.parts[q0 + j] + off + (size_t)r * p.H + c;
        a0[j] = ld_peer4(pp), a1[j] = ld_peer4(pp + 4);
        if (p.shared_rank == -2) {
          const float* up = p.parts[q0 + j] + off + (size_t)(p.rows_cap + r) * p.H + c;
          u0[j] = ld_peer4(up), u1[j] = ld_peer4(up + 4);
        }
      }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (q0 + j < p.world) {
        const bool first = q0 + j == 0;
        v0 = first ? a0[j] : add4(v0, a0[j]), v1 = first ? a1[j] : add4(v1, a1[j]);
        if (p.shared_rank == -2) s0 = first ? u0[j] : add4(s0, u0[j]), s1 = first ? u1[j] : add4(s1, u1[j]);
      }
  }
  if (p.shared_rank == -2) s0 = round4(s0), s1 = round4(s1);
  if (p.shared_rank >= 0 || p.shared_rank == -2) v0 = add4(v0, s0), v1 = add4(v1, s1);
}

template <bool kPeers>
__global__ void __launch_bounds__(256) k_add_norm(PeerParams p, AddNormParams an) {
  __shared__ int ok;
  __shared__ float red[16];
  uint32_t e = 0;
  if (kPeers) {
    e = peers_arrive_wait(p, ok);
  } else {
    pdl_launch_dependents();
    pdl_wait();
  }
  if (!kPeers || ok) {
    const size_t off = kPeers ? (size_t)(e & 1) * 2 * p.rows_cap * p.H : 0;
    const int nch = p.H / 8, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int r = blockIdx.x; r < p.M; r += gridDim.x) {
      float h[kNormChunks][8];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < kNormChunks; ++i) {
        const int c = 8 * (tid + 256 * i);
        if (tid + 256 * i < nch) {
          float4 v0, v1;
          if (kPeers) {
            peers_sum8(p, off, r, c, v0, v1);
          } else {
            const float* rp = an.R + (size_t)r * p.H + c;
            v0 = *reinterpret_cast<const float4*>(rp), v1 = *reinterpret_cast<const float4*>(rp + 4);
            if (an.S) {
              const float* sp = an.S + (size_t)r * p.H + c;
              float4 s0 = *reinterpret_cast<const float4*>(sp), s1 = *reinterpret_cast<const float4*>(sp + 4);
              if (an.fin_mode == 1) v0 = round4(v0), v1 = round4(v1), s0 = round4(s0), s1 = round4(s1);
              v0 = add4(v0, s0), v1 = add4(v1, s1);
            }
          }
          const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = bf16_round(v[j]);
          if (p.out) {
            const uint2 a = pack_bf16x4(o[0], o[1], o[2], o[3]), b = pack_bf16x4(o[4], o[5], o[6], o[7]);
            *reinterpret_cast<uint4*>(p.out + (size_t)r * p.H + c) = make_uint4(a.x, a.y, b.x, b.y);
          }
          if (an.res) {
            const uint4 rv = *reinterpret_cast<const uint4*>(an.res + (size_t)r * p.H + c);
            const uint32_t* rw = &rv.x;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              h[i][2 * j] = bf16_round(__fadd_rn(bf16_bits_to_f(rw[j] & 0xffffu), an.add_f32 ? v[2 * j] : o[2 * j]));
              h[i][2 * j + 1] = bf16_round(__fadd_rn(bf16_bits_to_f(rw[j] >> 16), an.add_f32 ? v[2 * j + 1] : o[2 * j + 1]));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) h[i][j] = o[j];
          }
          if (an.res_out) {
            const uint2 a = pack_bf16x4(h[i][0], h[i][1], h[i][2], h[i][3]), b = pack_bf16x4(h[i][4], h[i][5], h[i][6], h[i][7]);
            *reinterpret_cast<uint4*>(an.res_out + (size_t)r * p.H + c) = make_uint4(a.x, a.y, b.x, b.y);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) ss = fmaf(h[i][j], h[i][j], ss);
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      if (tid == 0) {
        float s = red[0];
        for (int w = 1; w < 8; ++w) s = __fadd_rn(s, red[w]);
        red[8] = rms_rstd(s, p.H, an.eps);
      }
      __syncthreads();
      const float rs = red[8];
      if (an.normed) {
#pragma unroll
        for (int i = 0; i < kNormChunks; ++i) {
          const int c = 8 * (tid + 256 * i);
          if (tid + 256 * i < nch) {
            const uint4 wv = __ldg(reinterpret_cast<const uint4*>(an.w + c));
            const uint32_t* ww = &wv.x;
            float y[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              y[2 * j] = rms_apply(h[i][2 * j], rs, bf16_bits_to_f(ww[j] & 0xffffu), an.mode);
              y[2 * j + 1] = rms_apply(h[i][2 * j + 1], rs, bf16_bits_to_f(ww[j] >> 16), an.mode);
            }
            const uint2 a = pack_bf16x4(y[0], y[1], y[2], y[3]), b = pack_bf16x4(y[4], y[5], y[6], y[7]);
            *reinterpret_cast<uint4*>(an.normed + (size_t)r * p.H + c) = make_uint4(a.x, a.y, b.x, b.y);
          }
        }
      }
      __syncthreads();
    }
  } else if (threadIdx.x == 0) {
    atomicCAS(p.status, 0, (int)DSGX_ERR_DEVICE_WAIT);
  }
  if (kPeers) peers_close(p, e);
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

cudaError_t launch_add_norm(const PeerParams& p, const AddNormParams& an, bool peers, cudaStream_t st, bool pdl) {
  const int grid = p.M < 4 * sm_count() ? p.M : 4 * sm_count();
  if (peers) {
    k_add_norm<true><<<grid, 256, 0, st>>>(p, an);
    return cudaGetLastError();
  }
  return launch_k(k_add_norm<false>, dim3(grid), dim3(256), 0, st, pdl, p, an);
}

}  // namespace dsgx
