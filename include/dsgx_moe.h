/*
 * dsgx_moe.h - C ABI of the B200 (sm_100a) quantised mixture-of-experts FFN operator.
 *
 * A drop-in for the MoE operator of dsgx10's engines: every entry point names the reference interface it stands in
 * for (paths inside the reference project).  Plain pointers and sizes only; every pointer is caller-owned DEVICE memory
 * unless a comment says "host".  `stream` is a cudaStream_t passed as void*.  Every call is asynchronous on `stream`
 * and returns a dsgx_status; nothing aborts the process and no kernel traps (the reference's die()/__trap() become
 * status codes: altar1 engine/experts/decode.cu:708-730, prefill.cu:784-794).
 *
 * Numerics contracts (selected by dsgx_moe_shape.fmt):
 *   DSGX_FMT_FP8  "W8A8-g128": activations quantised per 128 values to e4m3 with an f32 scale amax/448, weights e4m3
 *                 with one f32 scale per 128x128 block, gate/up rounded to bf16, h = bf16(w_route * silu(g) * u),
 *                 h quantised again per 128, every pick's down output rounded to bf16 and added in f32 in ascending
 *                 expert id (ds41f ref/inference/model.py:841-851, 889-904; ref/torchref/kernel.py:56-132).
 *   DSGX_FMT_INT4 bf16 activations, W = bf16((u - u_z) * s) per group of 32 along K, gate/up rounded to bf16,
 *                 h = bf16(bf16(silu(g)) * u), f32 down, yr += w_route * y in ascending expert id
 *                 (altar1 ref/glmref.py:108-121, 581-643; engine/experts/formats.cuh:102-119).
 */
#ifndef DSGX_MOE_H_
#define DSGX_MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum dsgx_status {
  DSGX_OK = 0,
  DSGX_ERR_ARG = 1,         /* null pointer, row count out of range, misaligned pointer */
  DSGX_ERR_FORMAT = 2,      /* unknown or refused format tag (0 = NVFP4 and the retired tag 1 are refused) */
  DSGX_ERR_SHAPE = 3,       /* H, I, E, topk, groups not supported by the kernels */
  DSGX_ERR_CUDA = 4,        /* a CUDA runtime call failed; dsgx_last_cuda_error() has the code */
  DSGX_ERR_DEVICE_WAIT = 5, /* a bounded device-side wait ran out (read from the workspace's status word) */
  DSGX_ERR_UNSUPPORTED = 6,
  DSGX_ERR_LIMIT = 7        /* the request is beyond a fixed built-in size (dsgx_sort_pack_static) */
} dsgx_status;

/* Expert formats.  Tags 2 and 3 are the reference's (altar1 engine/experts/experts.h:39): INT4-g32 blocks of 8 rows x 512 k
 * (2368 B) and BF16 blocks of 8 rows x 128 k (2048 B), both consumed as the reference lays them out (layout.h:50-107); a
 * BF16 layer's routed experts (decode only) run under the INT4 layers' contract with W given directly.  Tag 4 is this
 * library's routed FP8 format: the reference's "tile_fp8" lane order (experts.h:66-70, layout.h:108-119) for the e4m3 values and
 * f32 scales [N/128][K/128] row-major. */
enum { DSGX_FMT_NVFP4 = 0, DSGX_FMT_RETIRED = 1, DSGX_FMT_INT4 = 2, DSGX_FMT_BF16 = 3, DSGX_FMT_FP8 = 4, DSGX_FMT_MXFP4 = 5 };
/* Tag 5, DSGX_FMT_MXFP4: ds41f's routed expert format (ref/inference/model.py expert_dtype "fp4" over
 * ref/torchref/kernel.py:111-138: e2m1 values with one ue8m0 scale per 32 along K; engine/kernels/dsk.h:176-210), "W4A8":
 * the activations are quantised as for DSGX_FMT_FP8 (e4m3 per 128 with an f32 scale), W = e2m1 * 2^(scale - 127), the
 * rest of the contract is DSGX_FMT_FP8's; the layer's shared expert is FP8 (dsgx_shared_w.g/u/d), as ds41f's.  The
 * decode kernels stream the format as it is; the prefill pass reads a copy dsgx_prefill_prepare makes: the same weights as
 * e4m3 values with a power-of-two scale per 128 x 128 block (every e2m1 value times a power of two is an e4m3 value while
 * a block's scale bytes differ by at most 14; a layer with a wider block is refused with DSGX_ERR_UNSUPPORTED), twice the
 * MXFP4 bytes.  Layout of a matrix [N][K] (N a multiple of 8, K of 128), made by dsgx10_b200/weights.py pack_mx4:
 *   [N/8 strips][K/128 blocks] of 576 bytes: [32 lanes (g = lane / 4, t = lane % 4)][4 groups G][one 32-bit word] = the
 *   8 values v0..v7 of row 8 strip + g at k = 128 block + 32 G + 8 t + 0..7: v_j's magnitude code (its e2m1 nibble
 *   without the sign) in bits 4 j .. 4 j + 2, the sign of v_i in bit 8 i + 7 for i < 4 and in bit 8 (i - 4) + 3 for
 *   i >= 4; then [8 rows g][4 groups G] the scales 2^(byte - 127) as bf16 (byte << 7; 0x0040 for byte 0).  A lossless
 *   re-tiling of the checkpoint's nibbles and scale bytes.  rsv is zero. */
/* scores of the router: sigmoid and softmax (altar1 engine/experts/formats.cuh:142-163; ds41f ref/inference/model.py:812-818),
 * sqrt(softplus(l)) (ds41f engine/kernels/common.cuh:264-287, the only score dsk::router_topk has) */
enum { DSGX_SCORE_SIGMOID = 0, DSGX_SCORE_SOFTMAX = 1, DSGX_SCORE_SQRTSOFTPLUS = 2 };

enum { DSGX_MAX_ROWS = 8 };  /* decode rows one launch sequence of the expert kernels takes */
/* Rows a decode call takes (the reference's kMaxRows, altar1 engine/experts/experts.h:24).  9..16 rows run as two launch
 * sequences of at most 8 rows on the same stream and workspace (rows 0..7, then 8..M-1): every row's result is the one a
 * smaller step gives it (the kernels are batch-invariant); an expert that both halves picked is streamed twice. */
enum { DSGX_MAX_STEP_ROWS = 16 };

/* One routed matrix of one expert: stands in for gx::MatDesc (altar1 engine/experts/experts.h:58-64), 64 bytes.
 *   off: byte offset of the matrix's blocks in the layer's pool, a multiple of 256
 *   s2:  per-tensor scale, exactly 1.0 for INT4, BF16 and FP8
 *   fmt: the layer's format tag
 *   rsv: zero, except for DSGX_FMT_FP8 where rsv[0] | rsv[1] << 32 is the byte offset in the pool of the matrix's f32
 *        block scales [N/128][K/128] (a multiple of 16) */
typedef struct dsgx_mat_desc {
  uint64_t off;
  float s2;
  uint32_t fmt;
  uint32_t rsv[12];
} dsgx_mat_desc;

/* The shared expert: stands in for gx::SharedW (experts.h:66-87).  FP8: g, u [I][H] and d [H][I] in the tile_fp8
 * layout with f32 block scales gs, us, ds.  BF16 (INT4 layers), in the bf16 tile layout (layout.h:96-107), either as
 * the reference's engine holds it: bgu, the interleaved gate/up [2 I][H] (row 2 i gate, 2 i + 1 up of channel i), and bd
 * [H][I]; or as three matrices bg, bu [I][H] and bd.  The two forms give the same bits.  All null: the layer has no fused
 * shared expert. */
typedef struct dsgx_shared_w {
  const uint8_t *g, *u, *d;
  const float *gs, *us, *ds;
  const uint8_t *bg, *bu, *bd;
  const uint8_t* bgu;
} dsgx_shared_w;

/* One layer's weights on one GPU: stands in for gx::LayerW (experts.h:92-97).  desc is [E][3] (gate, up, down) in
 * device memory; descriptors of experts outside [e_lo, e_hi) are never read. */
typedef struct dsgx_layer_w {
  const uint8_t* pool;
  const dsgx_mat_desc* desc;
  dsgx_shared_w sh;
  uint32_t fmt;
} dsgx_layer_w;

/* The reference fixes its shapes at compile time (experts.h:18-26); here they are run-time parameters. */
typedef struct dsgx_moe_shape {
  int32_t H;            /* hidden: K of gate/up, N of down; FP8: a multiple of 256, at most 4096; INT4: a multiple of 512 */
  int32_t I;            /* intermediate: N of gate/up, K of down; the same limits */
  int32_t E;            /* routed experts of the layer, <= 512 */
  int32_t topk;         /* picks a row, <= 8 */
  int32_t n_group;      /* expert groups for group-limited selection (1: none) */
  int32_t topk_group;   /* groups kept */
  int32_t score_fn;     /* DSGX_SCORE_* */
  int32_t norm_topk;    /* 1: weights = s / (sum + 1e-20) * route_scale; 0: s * route_scale */
  float route_scale;
  uint32_t fmt;         /* DSGX_FMT_FP8, DSGX_FMT_INT4, DSGX_FMT_BF16 or DSGX_FMT_MXFP4 */
  int32_t e_lo, e_hi;   /* this GPU's experts [e_lo, e_hi) (expert parallelism: ds41f ref/inference/model.py:863-870) */
  int32_t sh_lo, sh_hi; /* FP8 decode: the shared expert's intermediate channels [sh_lo, sh_hi) this GPU computes
                           (multiples of 512; both 0: all of them).  The ranks of an expert-parallel step split the shared
                           expert this way instead of leaving it to one of them: a rank reads rows [sh_lo, sh_hi) of its
                           gate and up matrices and those K columns of its down matrix (the pointers still address the
                           whole matrices), and its ys is an unrounded f32 partial sum: the parts are added across the
                           ranks and rounded to bf16 once (dsgx_finalize_peers with shared_rank = -2) */
  float swiglu_limit;   /* > 0: gate is clamped from above to this and up to +- this before silu, on their bf16 values
                           (ds41f ref/inference/model.py:845-847; engine/kernels/prefill.cu:153-158 fixes 10); 0: no clamp */
  int32_t reserved;
} dsgx_moe_shape;

int dsgx_last_cuda_error(void);
const char* dsgx_status_name(int status);

/* ---- router ---------------------------------------------------------------------------------------------------
 * logits[r][e] = sum_k f32(x[r][k]) * wr[e][k] in f32 with a fixed summation order, the same for every M, so that the
 * selection is reproducible bit for bit on a CPU: stands in for the engines' router GEMV
 * (altar1 engine/model/model.cu:309-311; ds41f engine/model/model.cu:607).  x bf16 [M][H], wr f32 [E][H]. */
int dsgx_router_logits(const void* x_bf16, const float* wr, int M, int H, int E, float* logits, void* stream);

/* idx [M][topk] (descending selection key, ties to the lower expert id) and w [M][topk]: stands in for gx::route
 * (altar1 engine/experts/experts.h:99-102) and dsk::router_topk (ds41f engine/kernels/dsk.h:164-175).  bias may be null. */
int dsgx_route(const dsgx_moe_shape* shape, const float* logits, const float* bias, int M, int32_t* idx, float* w,
               void* stream);

/* ---- token -> expert sort / pack ---------------------------------------------------------------------------------
 * The stable (expert id, token) order of the T * topk picks: stands in for the bucket kernels of the prefill path
 * (altar1 engine/experts/prefill.cu:94-150; ds41f engine/kernels/prefill.cu:673-781), but deterministic.
 * counts [E], offsets [E+1], perm_tok [T*topk], perm_slot [T*topk], pos_of [T][topk], row_order [T][topk];
 * ws: dsgx_sort_ws_bytes(T, topk, E) bytes of scratch.  A pick whose id is outside [0, E) is left out of the order (its
 * pos_of is -1) and recorded in the status word of ws. */
size_t dsgx_sort_ws_bytes(int T, int topk, int E);
int dsgx_sort_pack(const int32_t* idx, int T, int topk, int E, int32_t* counts, int32_t* offsets, int32_t* perm_tok,
                   int32_t* perm_slot, int32_t* pos_of, int32_t* row_order, void* ws, void* stream);

/* dsgx_sort_pack without a workspace argument and without any allocation: the scratch is a fixed array inside the
 * library's device module.  It has no counterpart in the reference, whose callers always bring a workspace.  It is for
 * callers that cannot get device memory at the moment of the call: an engine that gave all device memory to its own pools
 * at start-up and has no spare block to hand out, or a thin foreign-function binding (cgo, JNI) that passes pointers
 * through but owns no device allocator.
 *   Limit: dsgx_sort_ws_bytes(T, topk, E) <= DSGX_SORT_STATIC_MAX_BYTES (for instance 8192 rows x 512 experts or
 *   16384 rows x 256 experts); beyond it the call does nothing and returns DSGX_ERR_LIMIT.
 *   The first call on a device looks up the array's address (and may load the module): make it once at start-up, before
 *   any stream capture begins; later calls only launch.
 *   The array is shared: it keeps what the last call left (each call clears the one word that must be zero), and calls
 *   that overlap on the device, on any streams, race on it: serialise them.
 * Same outputs, bit for bit, as dsgx_sort_pack. */
#define DSGX_SORT_STATIC_MAX_BYTES 131328 /* 256 + 2 x 32 chunks x 512 experts x 4 bytes */
int dsgx_sort_pack_static(const int32_t* idx, int T, int topk, int E, int32_t* counts, int32_t* offsets, int32_t* perm_tok,
                          int32_t* perm_slot, int32_t* pos_of, int32_t* row_order, void* stream);
/* A pick whose expert id lies outside [0, E) is left out of the order (counts and offsets describe the picks that are in)
 * and recorded: after dsgx_sort_pack, dsgx_ws_status(ws) gives DSGX_ERR_ARG instead of DSGX_OK; after
 * dsgx_sort_pack_static, this call does, for the last static sort on the current device (it copies one word back and so
 * waits for that sort; the cached address of the array does not survive a cudaDeviceReset). */
int dsgx_sort_static_status(void);

/* ---- decode (1..DSGX_MAX_STEP_ROWS rows) ------------------------------------------------------------------------------
 * Stands in for gx::decode_ws_bytes / gx::moe_decode (altar1 engine/experts/experts.h:104-141) and dsk::moe_routed
 * (ds41f engine/kernels/dsk.h:212-236).  x bf16 [M][H]; idx, w from dsgx_route; ws: dsgx_decode_ws_bytes(shape) bytes,
 * zeroed once before the first call (its counters reset themselves).  Writes this GPU's f32 partial sums
 * yr [M][H] (the routed experts in [e_lo, e_hi), added in ascending expert id) and ys [M][H] (the shared expert, when the
 * layer has one; ys may be null when it has none).  Calls that share a workspace must not overlap on the device. */
typedef struct dsgx_decode_cfg {
  int32_t ysum;        /* 1: ys is added into yr after the routed experts and yr is the only output (experts.h:132-137) */
  int32_t pdl;         /* 1: launch with programmatic dependent launch (experts.h:120) */
  int32_t parts;       /* bench hook (experts.h:121): 0 or 3 the whole step, 1 gate/up only, 2 down only; FP8 layers: 5 the
                          gate/up kernel alone, over the slot table and quantised rows an earlier call left in ws */
  int32_t up, down;    /* kernel variants (experts.h:114-118): 0 the default; every variant gives the same bits */
  int32_t reserved[3];
  /* Fused routing (experts.h:123-127): with logits (the router GEMV's f32 [M][E]) set, the step routes the rows itself
   * (dsgx_route's code, the same bits) and the idx / w arguments are not read (may be null): no dsgx_route launch between
   * the router GEMV and the experts.  bias: the selection bias f32 [E], or null. */
  const float* logits;
  const float* bias;
} dsgx_decode_cfg;
size_t dsgx_decode_ws_bytes(const dsgx_moe_shape* shape);
/* The kernel variants dsgx_decode_cfg.up / .down select (FP8 layers), and their names: stands in for
 * gx::decode_up_variants / decode_down_variants / decode_up_name / decode_down_name (experts.h:142-145).  A name is a
 * static string ("w16 k2 s2": warps a CTA, 128-k blocks a chunk, ring stages), null beyond the count. */
int dsgx_decode_up_variants(void);
int dsgx_decode_down_variants(void);
const char* dsgx_decode_up_name(int v);
const char* dsgx_decode_down_name(int v);
int dsgx_moe_decode(const dsgx_moe_shape* shape, const dsgx_layer_w* L, const void* x_bf16, const int32_t* idx,
                    const float* w, int M, void* ws, float* yr, float* ys, void* stream, const dsgx_decode_cfg* cfg);

/* out = bf16(R + S) (S may be null): the single rounding after the partial sums are reduced; stands in for
 * gx::finalize (experts.h:146-147), whose bf16(bf16(R) + bf16(S)) order is mode 1. */
int dsgx_finalize(const float* R, const float* S, int M, int H, void* out_bf16, int mode, void* stream);

/* The reduction across the GPUs of one box and the rounding in one kernel over peer memory: stands in for the all-reduce
 * the reference issues after its expert step (ds41f ref/inference/model.py:901-902; altar1 engine/model/model.cu, the ring
 * reduce before gx::finalize) followed by dsgx_finalize(mode 0).  Every rank calls it once a step, after the kernels that
 * wrote its partial sums, on buffers every rank can address (peer-mapped or symmetric memory, NVLink):
 *   parts[r]  rank r's partial sums, f32 [2][2][rows_cap][H]: [parity of the step][yr, ys][row][column]; the caller's
 *             expert step of step number e (1, 2, ...) writes the half (e & 1)
 *   flags[r]  rank r's flag words, u32 [world], zeroed once before the first step
 *   state     this rank's own u32 [2] {step counter, ticket}, zeroed once
 *   parts, flags: device arrays of `world` pointers.
 * out (this rank's memory) = bf16((yr of rank 0 + yr of rank 1 + ...) + ys of rank `shared_rank`); shared_rank = -1: no
 * shared expert; shared_rank = -2: every rank holds a part of the shared expert (dsgx_moe_shape.sh_lo / sh_hi) and
 * out = bf16(sum of yr + bf16(ys of rank 0 + ys of rank 1 + ...)).  The same bits on every rank.  The kernels of one step on the different GPUs wait for one another (each
 * wait bounded; on a run-out the status word, this rank's memory, gets DSGX_ERR_DEVICE_WAIT): launch nothing else that
 * waits across GPUs at the same time, and one step at a time. */
typedef struct dsgx_peer_set {
  const float* const* parts;
  uint32_t* const* flags;
  uint32_t* state;
  int32_t rank, world, rows_cap, shared_rank;
  /* Sliced form (for many rows, a prefill's pass), when outs is not null: rank r reduces and rounds only rows
   * [r M / world, (r + 1) M / world) and stores them into every rank's outs[q] (bf16 [rows_cap][H], peer-mapped), then a
   * second small kernel waits until every rank's slice has landed here (done[r]: u32 [world], zeroed once).  The
   * out_bf16 argument is ignored: the rows are in outs[rank].  A rank then reads 1/world of the partial sums of the
   * others instead of all of them. */
  void* const* outs;
  uint32_t* const* done;
} dsgx_peer_set;
int dsgx_finalize_peers(const dsgx_peer_set* peers, int M, int H, void* out_bf16, int32_t* status_word, void* stream);

/* What follows the experts in both engines, fused into the reduction: the residual add and the RMSNorm that feeds the next
 * block.  Stands in for altar1's comm::glm::allreduce_add_norm (engine/comm/glmcoll.cu:225-330: the all-reduce's consumer
 * adds the residual and normalises) and for ds41f's x = x + ffn(x) followed by the next norm (ref/inference/model.py).
 * Per row: v = the reduced f32 sums (as dsgx_finalize_peers / dsgx_finalize), out = bf16(v),
 *   h = bf16(res + out)  (add_f32 != 0: bf16(res + v), altar-1's f32 combine),  normed = RMSNorm(h; norm_w, eps):
 *   r = 1 / sqrt(mean(h^2) + eps) in IEEE operations with the sum in a fixed order,
 *   norm_mode 0: bf16(w (h r)) (model.py:288-293);  1: bf16(w bf16(h r)) (altar-1, glmref.py:225-228, glmcoll.cu:83-90).
 * res (bf16 [M][H]) may be null (h = out); res_out (may alias res), normed and out_bf16 may each be null.  H a multiple of
 * 8, at most 8192.  One CTA a row.  The peer form follows dsgx_finalize_peers' protocol (plain form only: outs null). */
typedef struct dsgx_add_norm {
  const void* res;
  void* res_out;
  const void* norm_w; /* bf16 [H] */
  void* normed;
  float eps;
  int32_t norm_mode;
  int32_t add_f32;
  int32_t reserved;
} dsgx_add_norm;
int dsgx_finalize_peers_norm(const dsgx_peer_set* peers, int M, int H, void* out_bf16, const dsgx_add_norm* an,
                             int32_t* status_word, void* stream);
/* one GPU: v = R + S (mode as dsgx_finalize; S may be null) */
int dsgx_finalize_add_norm(const float* R, const float* S, int M, int H, int mode, void* out_bf16, const dsgx_add_norm* an,
                           void* stream);

/* ---- one layer step, router to rounded output --------------------------------------------------------------------
 * The sequence the engines' layer runners issue around the operator (altar1 engine/model/model.cu:308-352: router
 * GEMV, route, moe_decode, then the reduction and the rounding): logits = x wr^T, route, the expert step, and
 * out = bf16(yr + ys).  Every buffer is caller-owned device memory sized for the rows of the call (up to
 * DSGX_MAX_STEP_ROWS): logits [M][E] f32, idx [M][topk] i32, w [M][topk] f32, yr, ys [M][H] f32, out [M][H] bf16,
 * x_stage [M][H] bf16.
 * With n_ranks > 1 the caller reduces yr across GPUs between dsgx_moe_layer_decode(..., finalize = 0) and dsgx_finalize. */
typedef struct dsgx_layer_step {
  const float* wr;    /* router weights f32 [E][H] */
  const float* bias;  /* selection bias f32 [E] or null */
  float* logits;
  int32_t* idx;
  float* w;
  void* ws;           /* dsgx_decode_ws_bytes(shape), zeroed once */
  float* yr;
  float* ys;
  void* out_bf16;
  void* x_stage;      /* device staging for dsgx_moe_layer_decode_host */
  int32_t flags;      /* FP8 layers run the step as four kernels (front, route, gate/up, down) at one or two rows and as
                         one persistent kernel from three rows up (the measured crossover); bit 0: always the four
                         kernels; bit 2: always the one kernel; bit 3: two small routing kernels, then the experts in the
                         one kernel; every path gives the same bits.
                         The one kernel's CTAs (one a SM) wait for one another through counters in ws, so all of them must
                         be resident together: it wants the GPU to itself while it runs.  If other work holds SMs (another
                         stream's kernels, another process), its bounded waits run out after about a second, the status
                         word of ws gets DSGX_ERR_DEVICE_WAIT and the outputs are not written; the counters in ws are
                         reset either way, so the next call on the workspace is clean once the status word is cleared.
                         Callers that overlap the step with other kernels set bit 0.
                         bit 4: a test of exactly that: the table is never announced inside the one kernel, every wait
                         for it runs out and the step ends with the status word set */
  int32_t reserved;
  void* reserved_ptr; /* with flags bit 1: device memory for [warps][8] u64 phase timestamps of the one-kernel step
                         (a profiling aid; warps = 16 x SM count) */
  /* RMSNorm in front of the router, fused into the step's first kernel (ds41f engine/kernels/dsk.h:130-135 gemv_bf16_norm,
     engine/model/model.cu:606-608: ffn_norm + the router's logits + the experts' quantised input in one launch): when
     norm_w (bf16 [H]) is not null, x is the un-normalised residual stream and the router and the experts see
     xn = RMSNorm(x; norm_w, norm_eps), norm_mode as dsgx_add_norm.norm_mode; xn_out (bf16 [8][H], optional) gets a copy. */
  const void* norm_w;
  void* xn_out;
  float norm_eps;
  int32_t norm_mode;
} dsgx_layer_step;
int dsgx_moe_layer_decode(const dsgx_moe_shape* shape, const dsgx_layer_w* L, const void* x_bf16, int M,
                          const dsgx_layer_step* step, int finalize, void* stream);
/* The same with HOST buffers: x_host bf16 [M][H] is brought to the device, the step runs, and out_host bf16 [M][H]
 * receives the result; all in stream order, the caller synchronises.  Pinned (mapped) buffers are used in place: a small
 * kernel reads x_host over PCIe and the step's last kernel writes out_host directly; other host memory goes through
 * cudaMemcpyAsync.  out_host null: the step stops at the f32 partial sums yr / ys (an expert-parallel rank, whose rows
 * are rounded after the reduction: dsgx_finalize_peers may write its out_bf16 straight into mapped host memory). */
int dsgx_moe_layer_decode_host(const dsgx_moe_shape* shape, const dsgx_layer_w* L, const void* x_host, int M,
                               const dsgx_layer_step* step, void* out_host, void* stream);

/* ---- prefill / verify (any number of rows; FP8 layers) --------------------------------------------------------------
 * Stands in for gx::prefill_ws_bytes / gx::moe_prefill (altar1 engine/experts/experts.h:149-182) and dsk::moe_prefill
 * (ds41f engine/kernels/dsk.h:238-293): the rows' picks ordered by (expert id, token), the experts as grouped GEMMs on
 * the tensor cores, every pick's output added per row in ascending expert id.  x bf16 [T][H], idx / w from dsgx_route;
 * yr, ys f32 [T][H] as dsgx_moe_decode; out_bf16 (may be null) receives bf16(yr + ys); with out_bf16 given, yr and ys may
 * be null (one GPU: only the rounded rows are wanted, and the f32 sums are a third of the combine's traffic).
 *
 * The tensor-core path reads the weights K-major: dsgx_prefill_prepare re-tiles a layer's tile_fp8 blocks once at load
 * time into wbuf (dsgx_prefill_weights_bytes(shape) bytes of device memory), as the reference re-tiles its checkpoints
 * (ds41f engine/kernels/moe.cu:1332-1336); it reads the descriptors back to the host and synchronises, so it is a
 * load-time call.  Only the experts in [e_lo, e_hi) (and the shared expert, when the layer has one) are prepared and run.
 * ws: dsgx_prefill_ws_bytes(shape, T) bytes, T <= the value given there; no zeroing needed.
 * ysum: as dsgx_decode_cfg.ysum.
 * dsgx_prefill_prepare allocates host memory (and, for MXFP4 layers, one device word), reads the descriptors back and
 * synchronises: a load-time call.  The other calls of this header allocate nothing and do not synchronise (dsgx_ws_status and dsgx_sort_static_status copy one word
 * back and so wait for the stream's work).  The first dsgx_moe_prefill of a process sets the grouped GEMM kernels'
 * attributes and asks for their occupancy: make it before any stream capture; later calls only launch (clusters of two
 * CTAs, chained as programmatic dependents) and can be captured into a CUDA graph. */
size_t dsgx_prefill_weights_bytes(const dsgx_moe_shape* shape);
int dsgx_prefill_prepare(const dsgx_moe_shape* shape, const dsgx_layer_w* L, void* wbuf, void* stream);
size_t dsgx_prefill_ws_bytes(const dsgx_moe_shape* shape, int T);
int dsgx_moe_prefill(const dsgx_moe_shape* shape, const dsgx_layer_w* L, const void* wbuf, const void* x_bf16,
                     const int32_t* idx, const float* w, int T, void* ws, float* yr, float* ys, void* out_bf16, int ysum,
                     void* stream);

/* The same work in separate calls on one workspace, for per-phase timing: stands in for gx::moe_prefill_phases and its
 * PrefillPhase bits (altar1 engine/experts/experts.h:191-193).  A phase reads what the phases before it left in ws. */
enum {
  DSGX_PH_BUCKET = 1,   /* the sort, the tile table, the quantisation of x and the gather of the sorted rows */
  DSGX_PH_UP = 2,       /* the routed gate/up grouped GEMM (SwiGLU, h quantised) */
  DSGX_PH_DOWN = 4,     /* the routed down grouped GEMM */
  DSGX_PH_COMBINE = 8,  /* the per-row ordered sum, the shared expert's output added, the rounding */
  DSGX_PH_SHARED = 16,  /* the shared expert's two dense GEMMs */
  DSGX_PH_ALL = 31
};
int dsgx_moe_prefill_phases(const dsgx_moe_shape* shape, const dsgx_layer_w* L, const void* wbuf, const void* x_bf16,
                            const int32_t* idx, const float* w, int T, void* ws, float* yr, float* ys, void* out_bf16,
                            int ysum, int phases, void* stream);

/* The workspace's intermediates after a pass, for tests: stands in for gx::prefill_view (experts.h:185-190); the fields
 * are this library's (h is kept quantised).  P = T * topk sorted picks. */
typedef struct dsgx_prefill_view {
  const int32_t *counts, *offsets;       /* [E], [E + 1]: picks an expert, their first sorted position */
  const int32_t *perm_tok, *perm_slot;   /* [P]: the row and the pick number at a sorted position */
  const int32_t *pos_of, *row_order;     /* [T][topk]: the sorted position of a pick; a row's picks in ascending expert id */
  const uint8_t* hq;                     /* [P][I] e4m3: h of every sorted pick */
  const float* hs;                       /* [P][I / 128]: its scales */
  const uint8_t* hq_shared;              /* [T][I] e4m3, [T][I / 128]: the shared expert's h */
  const float* hs_shared;
} dsgx_prefill_view;
int dsgx_prefill_view_of(const dsgx_moe_shape* shape, void* ws, int T, dsgx_prefill_view* view);

/* Reads (synchronously) the device status word of a workspace: DSGX_OK or DSGX_ERR_DEVICE_WAIT. */
int dsgx_ws_status(const void* ws);

#ifdef __cplusplus
}
#endif
#endif
