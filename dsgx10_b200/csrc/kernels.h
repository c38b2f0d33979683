// Internal interface between the C-ABI layer (api.cu) and the kernel files.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "dsgx_moe.h"

namespace dsgx {

// A quantised activation block: 128 k of up to 8 rows as e4m3 in MMA operand order (1024 B) + the rows' f32 scales.
constexpr int kActBlk = 1024 + 32;
constexpr int kMaxRows = DSGX_MAX_ROWS;
constexpr int kMxBlk = 576;  // bytes of an MXFP4 block: 8 rows x 128 k of e2m1 + 8 x 4 scales as bf16
// FP8 activations and FP8 shared expert: the FP8 kernels serve the layer
inline __host__ __device__ bool fmt_fp8_family(uint32_t fmt) { return fmt == DSGX_FMT_FP8 || fmt == DSGX_FMT_MXFP4; }
constexpr int kMaxTopK = 8;
constexpr int kMaxSlots = kMaxRows * kMaxTopK + 1;  // the union of a step's picks + the shared expert

struct RouteParams {
  int E, topk, n_group, topk_group, score_fn, norm_topk;
  float route_scale;
};

cudaError_t launch_router_logits(const __nv_bfloat16* x, const float* wr, int M, int H, int E, float* logits,
                                 cudaStream_t st, bool pdl);
cudaError_t launch_route(const RouteParams& p, const float* logits, const float* bias, int M, int* idx, float* w,
                         cudaStream_t st, bool pdl);
size_t sort_ws_bytes(int T, int topk, int E);
constexpr size_t kSortStaticBytes = DSGX_SORT_STATIC_MAX_BYTES;  // the fixed scratch of launch_sort_pack_static
cudaError_t launch_sort_pack_static(const int* idx, int T, int topk, int E, int* counts, int* offsets, int* perm_tok,
                                    int* perm_slot, int* pos_of, int* row_order, cudaStream_t st);
cudaError_t sort_static_status(int* word);
cudaError_t launch_sort_pack(const int* idx, int T, int topk, int E, int* counts, int* offsets, int* perm_tok,
                             int* perm_slot, int* pos_of, int* row_order, void* ws, cudaStream_t st);
cudaError_t launch_act_quant_tiled(const __nv_bfloat16* x, int M, int K, uint8_t* out, cudaStream_t st, bool pdl);
cudaError_t launch_finalize(const float* R, const float* S, int M, int H, __nv_bfloat16* out, int mode, cudaStream_t st,
                            bool pdl);

// ---- decode ---------------------------------------------------------------------------------------------------------
// Workspace of a decode step (all offsets multiples of 256; the first 256 bytes hold the status word and the counters'
// base).  Zeroed once by the caller; the kernels leave every counter at zero.
struct DecodeWs {
  int* status;      // [0]: a dsgx_status recorded by a kernel, 0 if none
  uint8_t* xq;      // FP8: [H/128] activation blocks of x; INT4 layers: the bf16 tile of x [H/16][R][32 B]
  __nv_bfloat16* h; // FP8: [kMaxSlots][8][I] bf16 h before quantisation; INT4 layers: the bf16 tiles of h [slot][I/16][R][32 B]
  uint8_t* hq;      // [kMaxSlots][I/128] activation blocks of h
  float* ypick;     // [kMaxSlots][H/16][16][8] every pick's down output (bf16-rounded values kept as f32)
  int* cnt_h;       // [kMaxSlots][I/128] arrivals of the 16 gate/up units of a 128-group of h
  int* cnt_y;       // [H/16] arrivals of the slots of an output tile
  struct StepSync* sync;  // counters of the one-kernel step (decode_fused.cu)
  struct SlotTab* tab;  // the step's slot table (decode_common.cuh)
  float* lpart;     // [H/1024 slices][8][E] partial router logits of the layer step
  float* part;      // [kPartUnits][kMaxPieces][32 lanes][4] piece sums of the units whose K is split over several warps
  int* cnt_u;       // [kPartUnits] arrivals of a split unit's runs
  int* r_idx;       // [kMaxRows][kMaxTopK] the picks of a step that routes on the caller's logits
  float* r_w;
};
// A unit's K is summed in pieces of kPB 128-k blocks (decode_common.cuh); when a launch has fewer units than warps, the
// pieces of a unit go to several warps (of different SMs) and meet in `part`, indexed by the unit's number in the launch.
constexpr int kPB = 4;
constexpr int kMaxPieces = 8;          // H, I <= 4096
constexpr int kPartUnits = 2048;
constexpr size_t kSlotTabBytes = 8192;  // room reserved for a SlotTab
size_t decode_ws_bytes(int H, int I);
DecodeWs decode_ws_carve(void* ws, int H, int I);

// RMSNorm of the step's input rows in front of the router (layer-step calls): x is the residual stream, the router and the
// experts see xn = RMSNorm(x) (ds41f engine/kernels/dsk.h:130-135 gemv_bf16_norm; mode 0: bf16(w (x r)), the order of
// ref/inference/model.py:288-293; mode 1: bf16(w bf16(x r)), altar-1's ref/glmref.py:225-228).  w null: x is used as is.
struct FrontNorm {
  const __nv_bfloat16* w;
  __nv_bfloat16* xn_out;  // optional copy of the normalised rows [M][H]
  float eps;
  int mode;
};
struct DecodeParams {
  int H, I, E, topk, M, e_lo, e_hi;
  const uint8_t* pool;
  const dsgx_mat_desc* desc;
  dsgx_shared_w sh;
  const int* idx;
  const float* w;
  DecodeWs ws;
  float* yr;
  float* ys;
  __nv_bfloat16* out;  // when set, k_down also writes bf16(yr + ys)
  int ysum;
  int up, down;  // kernel variants (same bits)
  float limit;     // the SwiGLU clamp (0: none)
  int sh_lo, sh_hi;  // the shared expert's intermediate channels this GPU computes (multiples of 512; the whole: 0, I)
  FrontNorm norm;
  int b16;  // 1: the routed experts are DSGX_FMT_BF16 (the INT4 kernels stream them as they stream the bf16 shared expert)
  int mx;  // 1: the routed experts are DSGX_FMT_MXFP4 (the shared expert, the activations and the sums as FP8's)
};
cudaError_t launch_layer_fp8(const DecodeParams& p, const RouteParams& rp, const __nv_bfloat16* x, const float* wr,
                             const float* bias, float* logits, int* idx, float* w, cudaStream_t st, bool pdl);
int decode_fp8_up_variants();
int decode_fp8_down_variants();
const char* decode_fp8_variant_name(int down, int i);
// parts: 1 = activation quantisation + gate/up, 2 = down + combine, 3 = both
// rp: when not null, the step routes on the caller's logits (p.idx / p.w are outputs then)
cudaError_t launch_decode_fp8(const DecodeParams& p, const __nv_bfloat16* x, cudaStream_t st, bool pdl, int parts,
                              const RouteParams* rp = nullptr, const float* logits = nullptr, const float* bias = nullptr);

// the one-kernel FP8 layer step (decode_fused.cu)
struct StepSync {
  int cnt_lp;     // router logit slices done
  int cnt_rt;     // rows routed
  int tab_ready;  // the slot table is in the workspace
  int cnt_exit;   // CTAs that left
  int q_up, q_down;  // next unclaimed gate/up unit, down unit
  int cnt_hq[kMaxSlots + 1];  // quantised 128-groups of a slot's h
};
struct StepParams {
  DecodeParams d;
  RouteParams rp;
  const __nv_bfloat16* x;
  const float* wr;
  const float* bias;
  float* logits;
  int* idx;
  float* w;
  StepSync* sync;
  unsigned long long* stamps;  // optional [warps][8] phase timestamps (profiling aid), or null
  int R, sh_slot, has_sh;
  int pre_routed;  // 1: earlier kernels routed the rows and built the slot table; the step starts at the experts
  int test_no_table;  // test hook: the table is never announced, so every wait for it runs out (bounded) and is reported
};
bool step_fp8_fits(int H, int I, int E, int M);
cudaError_t launch_step_fp8(StepParams sp, cudaStream_t st);
cudaError_t launch_front_route_only(const DecodeParams& p, const RouteParams& rp, const __nv_bfloat16* x, const float* wr,
                                    const float* bias, float* logits, int* idx, float* w, cudaStream_t st, bool pdl);

cudaError_t launch_decode_int4(const DecodeParams& p, const __nv_bfloat16* x, cudaStream_t st, bool pdl, int parts,
                               const RouteParams* rp = nullptr, const float* logits = nullptr, const float* bias = nullptr);
cudaError_t launch_layer_int4(const DecodeParams& p, const RouteParams& rp, const __nv_bfloat16* x, const float* wr,
                              const float* bias, float* logits, int* idx, float* w, cudaStream_t st, bool pdl);
bool decode_int4_fits(int H, int M);

// the front of a decode step (decode_front.cu); fmt selects how x is staged for the expert kernels
cudaError_t launch_prep(const DecodeParams& p, uint32_t fmt, const __nv_bfloat16* x, cudaStream_t st, bool pdl);
cudaError_t launch_stage_route(const DecodeParams& p, uint32_t fmt, const RouteParams& rp, const __nv_bfloat16* x,
                               const float* logits_in, const float* bias, int* idx, float* w, cudaStream_t st, bool pdl);
cudaError_t launch_front_route(const DecodeParams& p, uint32_t fmt, const RouteParams& rp, const __nv_bfloat16* x,
                               const float* wr, const float* bias, float* logits, int* idx, float* w, cudaStream_t st,
                               bool pdl);

// ---- prefill (FP8) ----------------------------------------------------------------------------------------------------
struct PrefillWeights {  // K-major row-major copies of the layer's matrices, [E + 1 experts] each (index E: shared)
  uint8_t *g, *u, *d;
  float *sg, *su, *sd;
};
size_t prefill_weights_bytes(int H, int I, int E);
PrefillWeights prefill_weights_carve(void* buf, int H, int I, int E);
cudaError_t retile_matrix(const uint8_t* tiled, const float* scales, int N, int K, uint8_t* out, float* sout, cudaStream_t st);
// an MXFP4 matrix as the grouped GEMM's FP8 operand, W unchanged; *flag (device) is set when a 128 x 128 block's scales
// spread over more than 14 octaves (not representable)
cudaError_t convert_mx4_matrix(const uint8_t* blocks, int N, int K, uint8_t* out, float* sout, int* flag, cudaStream_t st);

struct PrefillWs {
  int* status;
  uint8_t* xq;   float* xs;                  // per token
  uint8_t* xq_s; float* xs_s; float* w_s;    // per sorted pick
  uint8_t* hq;   float* hs;                  // routed h
  uint8_t* hq_sh; float* hs_sh;              // shared h
  __nv_bfloat16* y; __nv_bfloat16* y_sh;
  int *perm_tok, *perm_slot, *pos_of, *row_order, *counts, *offsets, *tile_off;
  int4* tile_info;
  void* sort_ws;
};
size_t prefill_ws_bytes(int T, int H, int I, int E, int topk);
PrefillWs prefill_ws_carve(void* ws, int T, int H, int I, int E, int topk);

struct PrefillParams {
  int T, H, I, E, topk, has_shared, ysum, e_lo, e_hi;
  float limit;  // the SwiGLU clamp (0: none)
  int phases;  // DSGX_PH_* bits: the parts of the pass to run
  const __nv_bfloat16* x;
  const int* idx;
  const float* w;
  PrefillWeights pw;
  PrefillWs ws;
  float* yr;
  float* ys;
  __nv_bfloat16* out;
};
cudaError_t launch_prefill_fp8(const PrefillParams& q, cudaStream_t st);

int sm_count();
cudaError_t launch_copy_in(const void* src, void* dst, size_t bytes, cudaStream_t st);

// ---- reduction over peer memory (peer.cu)
struct PeerParams {
  const float* const* parts;  // device array [world]: rank r's partial sums, f32 [2 parities][yr, ys][rows_cap][H]
  uint32_t* const* flags;     // device array [world]: rank r's flag words, u32 [world]
  uint32_t* state;            // this rank's {step counter, CTA ticket}
  int rank, world, rows_cap, shared_rank, M, H;
  __nv_bfloat16* out;
  int* status;
  __nv_bfloat16* const* outs;  // sliced form: every rank's output rows (null: the plain form)
  uint32_t* const* done;       // sliced form: rank r's "slices landed" words, u32 [world]
};
cudaError_t launch_finalize_peers(const PeerParams& p, cudaStream_t st);
// the reduction followed by the residual add and the RMSNorm for the next block, one kernel (peers: over peer memory;
// else one GPU's own R / S)
struct AddNormParams {
  const __nv_bfloat16* res;  // residual stream in (null: h = out)
  __nv_bfloat16* res_out;    // h (may alias res), or null
  const __nv_bfloat16* w;    // norm weights [H]
  __nv_bfloat16* normed;     // RMSNorm(h), or null
  float eps;
  int mode, add_f32;
  const float* R;            // one GPU: the sums; S may be null
  const float* S;
  int fin_mode;
};
cudaError_t launch_add_norm(const PeerParams& p, const AddNormParams& an, bool peers, cudaStream_t st, bool pdl);

}  // namespace dsgx
