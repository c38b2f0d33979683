// Header-only C++ mirror of the engines' MoE operator interface (altar1 engine/experts/experts.h:99-193) over the C ABI
// of libdsgx_moe.so (include/dsgx_moe.h).  Same function names, argument order and meaning as the reference's `gx::`
// functions; the compile-time shape constants of the reference (experts.h:18-26) become a `MoeShape` the caller
// passes, and a failed call throws gx::Error(status) where the reference aborts the process (common/check.h).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "dsgx_moe.h"

namespace gx {

using MoeShape = dsgx_moe_shape;
using MatDesc = dsgx_mat_desc;   // experts.h:58-64
using SharedW = dsgx_shared_w;   // experts.h:66-87
using LayerW = dsgx_layer_w;     // experts.h:92-97
using DecodeCfg = dsgx_decode_cfg;

struct Error : std::runtime_error {
  int status;
  Error(int s, const char* where) : std::runtime_error(std::string(where) + ": " + dsgx_status_name(s)), status(s) {}
};
inline void check(int status, const char* where) {
  if (status != DSGX_OK) throw Error(status, where);
}

// logits f32 [M][E] -> idx [M][topk] (descending selection score, ties to the lower id), w [M][topk].  experts.h:99-102
inline void route(const MoeShape& s, const float* logits, const float* bias, int M, int* idx, float* w, cudaStream_t st) {
  check(dsgx_route(&s, logits, bias, M, idx, w, st), "gx::route");
}
// the runner's router GEMV (engine/model/model.cu:309-311)
inline void router_logits(const __nv_bfloat16* x, const float* wr, int M, int H, int E, float* logits, cudaStream_t st) {
  check(dsgx_router_logits(x, wr, M, H, E, logits, st), "gx::router_logits");
}
// the prefill path's bucket step on its own (experts.h: prefill.cu:94-150), deterministic
inline size_t sort_ws_bytes(int T, int topk, int E) { return dsgx_sort_ws_bytes(T, topk, E); }
inline void sort_pack(const int* idx, int T, int topk, int E, int* counts, int* offsets, int* perm_tok, int* perm_slot,
                      int* pos_of, int* row_order, void* ws, cudaStream_t st) {
  check(dsgx_sort_pack(idx, T, topk, E, counts, offsets, perm_tok, perm_slot, pos_of, row_order, ws, st), "gx::sort_pack");
}
// experts.h:139-145
inline size_t decode_ws_bytes(const MoeShape& s) { return dsgx_decode_ws_bytes(&s); }
inline int decode_up_variants() { return dsgx_decode_up_variants(); }
inline int decode_down_variants() { return dsgx_decode_down_variants(); }
inline const char* decode_up_name(int v) { return dsgx_decode_up_name(v); }
inline const char* decode_down_name(int v) { return dsgx_decode_down_name(v); }
inline void moe_decode(const MoeShape& s, const LayerW& L, const __nv_bfloat16* x, const int* idx, const float* w, int M,
                       void* ws, float* yr, float* ys, cudaStream_t st, const DecodeCfg& cfg = DecodeCfg{0, 1, 0, 0, 0, {0, 0, 0}, nullptr, nullptr}) {
  check(dsgx_moe_decode(&s, &L, x, idx, w, M, ws, yr, ys, st, &cfg), "gx::moe_decode");
}
// experts.h:146-147 (mode 1 is the reference's bf16(bf16(R) + bf16(S)); mode 0 rounds the f32 sum once)
inline void finalize(const float* R, const float* S, int M, int H, __nv_bfloat16* out, cudaStream_t st, int mode = 0) {
  check(dsgx_finalize(R, S, M, H, out, mode, st), "gx::finalize");
}
// experts.h:180-182; wbuf: the K-major weight copy made once by prefill_prepare
inline size_t prefill_weights_bytes(const MoeShape& s) { return dsgx_prefill_weights_bytes(&s); }
inline void prefill_prepare(const MoeShape& s, const LayerW& L, void* wbuf, cudaStream_t st) {
  check(dsgx_prefill_prepare(&s, &L, wbuf, st), "gx::prefill_prepare");
}
inline size_t prefill_ws_bytes(const MoeShape& s, int T) { return dsgx_prefill_ws_bytes(&s, T); }
inline void moe_prefill(const MoeShape& s, const LayerW& L, const void* wbuf, const __nv_bfloat16* x, const int* idx,
                        const float* w, int T, void* ws, float* yr, float* ys, cudaStream_t st, __nv_bfloat16* out = nullptr,
                        bool ysum = false) {
  check(dsgx_moe_prefill(&s, &L, wbuf, x, idx, w, T, ws, yr, ys, out, ysum ? 1 : 0, st), "gx::moe_prefill");
}

// experts.h:185-193: the pass in separate calls, and the workspace's intermediates
enum PrefillPhase { kPhBucket = DSGX_PH_BUCKET, kPhUp = DSGX_PH_UP, kPhDown = DSGX_PH_DOWN, kPhCombine = DSGX_PH_COMBINE,
                    kPhShared = DSGX_PH_SHARED, kPhAll = DSGX_PH_ALL };
constexpr int kPrefillAll = DSGX_PH_ALL;
inline void moe_prefill_phases(const MoeShape& s, const LayerW& L, const void* wbuf, const __nv_bfloat16* x, const int* idx,
                               const float* w, int T, void* ws, float* yr, float* ys, cudaStream_t st, int phases,
                               __nv_bfloat16* out = nullptr, bool ysum = false) {
  check(dsgx_moe_prefill_phases(&s, &L, wbuf, x, idx, w, T, ws, yr, ys, out, ysum ? 1 : 0, phases, st), "gx::moe_prefill_phases");
}
using PrefillView = dsgx_prefill_view;
inline PrefillView prefill_view(const MoeShape& s, void* ws, int T) {
  PrefillView v{};
  check(dsgx_prefill_view_of(&s, ws, T, &v), "gx::prefill_view");
  return v;
}

// the all-reduce after the expert step and the rounding in one call over peer-mapped buffers (ds41f
// ref/inference/model.py:901-902; altar1's ring reduce before gx::finalize)
using PeerSet = dsgx_peer_set;
inline void finalize_peers(const PeerSet& ps, int M, int H, __nv_bfloat16* out, int* status_word, cudaStream_t st) {
  check(dsgx_finalize_peers(&ps, M, H, out, status_word, st), "gx::finalize_peers");
}
// the same with the residual add and the next block's RMSNorm fused in (altar1 engine/comm/glmcoll.cu:225-330
// comm::glm::allreduce_add_norm), over peer memory or on one GPU
using AddNorm = dsgx_add_norm;
inline void finalize_peers_norm(const PeerSet& ps, int M, int H, __nv_bfloat16* out, const AddNorm& an, int* status_word,
                                cudaStream_t st) {
  check(dsgx_finalize_peers_norm(&ps, M, H, out, &an, status_word, st), "gx::finalize_peers_norm");
}
inline void finalize_add_norm(const float* R, const float* S, int M, int H, __nv_bfloat16* out, const AddNorm& an,
                              cudaStream_t st, int mode = 0) {
  check(dsgx_finalize_add_norm(R, S, M, H, mode, out, &an, st), "gx::finalize_add_norm");
}
// one layer step, router to rounded rows (the sequence of engine/model/model.cu:308-352)
using LayerStep = dsgx_layer_step;
inline void layer_decode(const MoeShape& s, const LayerW& L, const __nv_bfloat16* x, int M, const LayerStep& step,
                         cudaStream_t st, bool finalize = true) {
  check(dsgx_moe_layer_decode(&s, &L, x, M, &step, finalize ? 1 : 0, st), "gx::layer_decode");
}

}  // namespace gx
