// The C ABI (include/dsgx_moe.h): argument checks, workspace carving, kernel launches.  No allocation on the hot
// calls; every failure is a status code.
#include <atomic>
#include <cstdio>
#include <cstring>

#include "common.cuh"
#include "kernels.h"

namespace dsgx {

static std::atomic<int> g_last_cuda{0};
static int cuda_fail(cudaError_t e) {
  g_last_cuda.store((int)e);
  return DSGX_ERR_CUDA;
}

int sm_count() {
  static int n[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!n[dev]) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    n[dev] = v;
  }
  return n[dev];
}

static size_t al256(size_t v) { return (v + 255) & ~(size_t)255; }

size_t decode_ws_bytes(int H, int I) {
  const size_t HB = H / 128, IB = I / 128;
  size_t n = 256;
  n += al256(HB * kActBlk > (size_t)H * 16 ? HB * kActBlk : (size_t)H * 16);
  n += al256((size_t)kMaxSlots * 8 * I * 2);
  n += al256((size_t)kMaxSlots * IB * kActBlk);
  n += al256((size_t)kMaxSlots * (H / 16) * 128 * 4);
  n += al256((size_t)kMaxSlots * IB * 4);
  n += al256((size_t)(H / 16) * 4);
  n += kSlotTabBytes;
  n += al256((size_t)((H + 1023) / 1024) * kMaxRows * 512 * 4);
  n += al256(sizeof(StepSync));
  n += al256((size_t)kPartUnits * kMaxPieces * 128 * 4);
  n += al256((size_t)kPartUnits * 4);
  n += 512;
  return n;
}
DecodeWs decode_ws_carve(void* ws, int H, int I) {
  const size_t HB = H / 128, IB = I / 128;
  char* p = reinterpret_cast<char*>(ws);
  DecodeWs w;
  w.status = reinterpret_cast<int*>(p), p += 256;
  w.xq = reinterpret_cast<uint8_t*>(p), p += al256(HB * kActBlk > (size_t)H * 16 ? HB * kActBlk : (size_t)H * 16);
  w.h = reinterpret_cast<__nv_bfloat16*>(p), p += al256((size_t)kMaxSlots * 8 * I * 2);
  w.hq = reinterpret_cast<uint8_t*>(p), p += al256((size_t)kMaxSlots * IB * kActBlk);
  w.ypick = reinterpret_cast<float*>(p), p += al256((size_t)kMaxSlots * (H / 16) * 128 * 4);
  w.cnt_h = reinterpret_cast<int*>(p), p += al256((size_t)kMaxSlots * IB * 4);
  w.cnt_y = reinterpret_cast<int*>(p), p += al256((size_t)(H / 16) * 4);
  w.tab = reinterpret_cast<SlotTab*>(p), p += kSlotTabBytes;
  w.lpart = reinterpret_cast<float*>(p), p += al256((size_t)((H + 1023) / 1024) * kMaxRows * 512 * 4);
  w.sync = reinterpret_cast<StepSync*>(p), p += al256(sizeof(StepSync));
  w.part = reinterpret_cast<float*>(p), p += al256((size_t)kPartUnits * kMaxPieces * 128 * 4);
  w.cnt_u = reinterpret_cast<int*>(p), p += al256((size_t)kPartUnits * 4);
  w.r_idx = reinterpret_cast<int*>(p), w.r_w = reinterpret_cast<float*>(p + 256);
  return w;
}

// the routing fields only (dsgx_route reads nothing else)
static int check_route_shape(const dsgx_moe_shape* s) {
  if (!s) return DSGX_ERR_ARG;
  if (s->E < 1 || s->E > 512 || s->topk < 1 || s->topk > kMaxTopK || s->topk > s->E) return DSGX_ERR_SHAPE;
  if (s->n_group < 1 || s->n_group > 32 || s->E % s->n_group || s->topk_group < 1 || s->topk_group > s->n_group)
    return DSGX_ERR_SHAPE;
  if (s->n_group > 1 && (s->E / s->n_group < 2 || s->topk > s->topk_group * (s->E / s->n_group))) return DSGX_ERR_SHAPE;
  if (s->score_fn != DSGX_SCORE_SIGMOID && s->score_fn != DSGX_SCORE_SOFTMAX && s->score_fn != DSGX_SCORE_SQRTSOFTPLUS)
    return DSGX_ERR_SHAPE;
  return DSGX_OK;
}
static int check_shape(const dsgx_moe_shape* s) {
  if (!s) return DSGX_ERR_ARG;
  if (s->fmt == DSGX_FMT_NVFP4 || s->fmt == DSGX_FMT_RETIRED) return DSGX_ERR_FORMAT;
  if (!fmt_fp8_family(s->fmt) && s->fmt != DSGX_FMT_INT4 && s->fmt != DSGX_FMT_BF16) return DSGX_ERR_FORMAT;
  const int rc = check_route_shape(s);
  if (rc) return rc;
  if (s->H < 128 || s->I < 128 || s->H % 128 || s->I % 128) return DSGX_ERR_SHAPE;
  if (s->e_lo < 0 || s->e_hi > s->E || s->e_lo > s->e_hi) return DSGX_ERR_SHAPE;
  if (fmt_fp8_family(s->fmt) && (s->H > 4096 || s->I > 4096 || s->H % 256 || s->I % 256)) return DSGX_ERR_SHAPE;
  if ((s->fmt == DSGX_FMT_INT4 || s->fmt == DSGX_FMT_BF16) && (s->H % 512 || s->I % 512)) return DSGX_ERR_SHAPE;
  if (s->sh_lo || s->sh_hi) {  // a part of the shared expert: FP8 decode only, whole pieces of 512 channels
    if (!fmt_fp8_family(s->fmt) || s->sh_lo < 0 || s->sh_hi > s->I || s->sh_lo >= s->sh_hi || s->sh_lo % 512 ||
        (s->sh_hi % 512 && s->sh_hi != s->I))
      return DSGX_ERR_SHAPE;
  }
  if (!(s->swiglu_limit >= 0.f) || (s->swiglu_limit > 0.f && !fmt_fp8_family(s->fmt))) return DSGX_ERR_SHAPE;
  return DSGX_OK;
}

}  // namespace dsgx

using namespace dsgx;

extern "C" {

int dsgx_last_cuda_error(void) { return g_last_cuda.load(); }

const char* dsgx_status_name(int s) {
  switch (s) {
    case DSGX_OK: return "ok";
    case DSGX_ERR_ARG: return "bad argument";
    case DSGX_ERR_FORMAT: return "unknown or refused expert format";
    case DSGX_ERR_SHAPE: return "unsupported shape";
    case DSGX_ERR_CUDA: return "CUDA error";
    case DSGX_ERR_DEVICE_WAIT: return "a bounded device wait ran out";
    case DSGX_ERR_UNSUPPORTED: return "unsupported";
    case DSGX_ERR_LIMIT: return "beyond a fixed built-in size";
  }
  return "unknown status";
}

int dsgx_router_logits(const void* x, const float* wr, int M, int H, int E, float* logits, void* stream) {
  if (!x || !wr || !logits || M < 1) return DSGX_ERR_ARG;
  if (H < 128 || H % 128 || E < 1) return DSGX_ERR_SHAPE;
  if (((uintptr_t)x & 7) || ((uintptr_t)wr & 15)) return DSGX_ERR_ARG;
  cudaError_t e = launch_router_logits(reinterpret_cast<const __nv_bfloat16*>(x), wr, M, H, E, logits,
                                       (cudaStream_t)stream, true);
  return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
}

int dsgx_route(const dsgx_moe_shape* s, const float* logits, const float* bias, int M, int32_t* idx, float* w,
               void* stream) {
  const int rc = check_route_shape(s);
  if (rc) return rc;
  if (!logits || !idx || !w || M < 1) return DSGX_ERR_ARG;
  RouteParams p{s->E, s->topk, s->n_group, s->topk_group, s->score_fn, s->norm_topk, s->route_scale};
  cudaError_t e = launch_route(p, logits, bias, M, idx, w, (cudaStream_t)stream, true);
  return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
}

size_t dsgx_sort_ws_bytes(int T, int topk, int E) { return sort_ws_bytes(T, topk, E); }

int dsgx_sort_pack(const int32_t* idx, int T, int topk, int E, int32_t* counts, int32_t* offsets, int32_t* perm_tok,
                   int32_t* perm_slot, int32_t* pos_of, int32_t* row_order, void* ws, void* stream) {
  if (!idx || !counts || !offsets || !perm_tok || !perm_slot || !pos_of || !row_order || !ws) return DSGX_ERR_ARG;
  if (T < 0 || topk < 1 || topk > kMaxTopK || E < 1 || E > 512) return DSGX_ERR_SHAPE;
  if (T == 0) {
    cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int) * E, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(offsets, 0, sizeof(int) * (E + 1), (cudaStream_t)stream);
    return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
  }
  cudaError_t e = launch_sort_pack(idx, T, topk, E, counts, offsets, perm_tok, perm_slot, pos_of, row_order, ws,
                                   (cudaStream_t)stream);
  return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
}

int dsgx_sort_pack_static(const int32_t* idx, int T, int topk, int E, int32_t* counts, int32_t* offsets, int32_t* perm_tok,
                          int32_t* perm_slot, int32_t* pos_of, int32_t* row_order, void* stream) {
  if (!idx || !counts || !offsets || !perm_tok || !perm_slot || !pos_of || !row_order) return DSGX_ERR_ARG;
  if (T < 0 || topk < 1 || topk > kMaxTopK || E < 1 || E > 512) return DSGX_ERR_SHAPE;
  if (sort_ws_bytes(T, topk, E) > kSortStaticBytes) return DSGX_ERR_LIMIT;
  if (T == 0) {
    cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int) * E, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(offsets, 0, sizeof(int) * (E + 1), (cudaStream_t)stream);
    return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
  }
  cudaError_t e = launch_sort_pack_static(idx, T, topk, E, counts, offsets, perm_tok, perm_slot, pos_of, row_order,
                                          (cudaStream_t)stream);
  return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
}

int dsgx_finalize_peers(const dsgx_peer_set* ps, int M, int H, void* out, int32_t* status_word, void* stream) {
  if (!ps || !ps->parts || !ps->flags || !ps->state || (!out && !ps->outs) || !status_word) return DSGX_ERR_ARG;
  if ((ps->outs != nullptr) != (ps->done != nullptr)) return DSGX_ERR_ARG;
  if (ps->outs && H % 8) return DSGX_ERR_SHAPE;
  if (ps->world < 1 || ps->world > 32 || ps->rank < 0 || ps->rank >= ps->world || ps->shared_rank >= ps->world || ps->shared_rank < -2) return DSGX_ERR_ARG;
  if (ps->shared_rank == -2 && ps->outs) return DSGX_ERR_UNSUPPORTED;  // (parts of the shared expert: the decode form only)
  if (M < 1 || M > ps->rows_cap || H < 4 || H % 4 || (size_t)M * H / 4 > (size_t)1 << 30) return DSGX_ERR_SHAPE;
  PeerParams p;
  p.parts = ps->parts, p.flags = ps->flags, p.state = ps->state, p.rank = ps->rank, p.world = ps->world;
  p.rows_cap = ps->rows_cap, p.shared_rank = ps->shared_rank, p.M = M, p.H = H;
  p.out = reinterpret_cast<__nv_bfloat16*>(out), p.status = status_word;
  p.outs = reinterpret_cast<__nv_bfloat16* const*>(ps->outs), p.done = ps->done;
  cudaError_t e = launch_finalize_peers(p, (cudaStream_t)stream);
  return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
}

static int add_norm_args(const dsgx_add_norm* an, int H, AddNormParams& a) {
  if (!an || !an->norm_w || (an->norm_mode != 0 && an->norm_mode != 1) || !(an->eps >= 0.f)) return DSGX_ERR_ARG;
  if (H % 8 || H > 8192) return DSGX_ERR_SHAPE;
  if (((uintptr_t)an->res | (uintptr_t)an->res_out | (uintptr_t)an->norm_w | (uintptr_t)an->normed) & 15) return DSGX_ERR_ARG;
  a.res = reinterpret_cast<const __nv_bfloat16*>(an->res), a.res_out = reinterpret_cast<__nv_bfloat16*>(an->res_out);
  a.w = reinterpret_cast<const __nv_bfloat16*>(an->norm_w), a.normed = reinterpret_cast<__nv_bfloat16*>(an->normed);
  a.eps = an->eps, a.mode = an->norm_mode, a.add_f32 = an->add_f32 != 0, a.R = nullptr, a.S = nullptr, a.fin_mode = 0;
  return DSGX_OK;
}

int dsgx_finalize_peers_norm(const dsgx_peer_set* ps, int M, int H, void* out, const dsgx_add_norm* an, int32_t* status_word,
                             void* stream) {
  if (!ps || !ps->parts || !ps->flags || !ps->state || !status_word || ps->outs || ps->done) return DSGX_ERR_ARG;
  if (ps->world < 1 || ps->world > 32 || ps->rank < 0 || ps->rank >= ps->world || ps->shared_rank >= ps->world || ps->shared_rank < -2) return DSGX_ERR_ARG;
  if (M < 1 || M > ps->rows_cap || ((uintptr_t)out & 15)) return DSGX_ERR_SHAPE;
  AddNormParams a;
  const int rc = add_norm_args(an, H, a);
  if (rc) return rc;
  PeerParams p;
  p.parts = ps->parts, p.flags = ps->flags, p.state = ps->state, p.rank = ps->rank, p.world = ps->world;
  p.rows_cap = ps->rows_cap, p.shared_rank = ps->shared_rank, p.M = M, p.H = H;
  p.out = reinterpret_cast<__nv_bfloat16*>(out), p.status = status_word, p.outs = nullptr, p.done = nullptr;
  cudaError_t e = launch_add_norm(p, a, true, (cudaStream_t)stream, false);
  return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
}

int dsgx_finalize_add_norm(const float* R, const float* S, int M, int H, int mode, void* out, const dsgx_add_norm* an,
                           void* stream) {
  if (!R || M < 1 || (mode != 0 && mode != 1) || (((uintptr_t)R | (uintptr_t)S | (uintptr_t)out) & 15)) return DSGX_ERR_ARG;
  AddNormParams a;
  const int rc = add_norm_args(an, H, a);
  if (rc) return rc;
  a.R = R, a.S = S, a.fin_mode = mode;
  PeerParams p{};
  p.world = 1, p.rows_cap = M, p.shared_rank = -1, p.M = M, p.H = H, p.out = reinterpret_cast<__nv_bfloat16*>(out);
  cudaError_t e = launch_add_norm(p, a, false, (cudaStream_t)stream, true);
  return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
}

size_t dsgx_decode_ws_bytes(const dsgx_moe_shape* s) {
  if (check_shape(s)) return 0;
  return decode_ws_bytes(s->H, s->I);
}

int dsgx_moe_decode(const dsgx_moe_shape* s, const dsgx_layer_w* L, const void* x, const int32_t* idx, const float* w,
                    int M, void* ws, float* yr, float* ys, void* stream, const dsgx_decode_cfg* cfg) {
  const int rc = check_shape(s);
  if (rc) return rc;
  const dsgx_decode_cfg dflt = {0, 1, 0, 0, 0, {0, 0, 0}, nullptr, nullptr};
  if (!cfg) cfg = &dflt;
  const bool own_route = cfg->logits != nullptr;  // the step routes on the caller's logits: idx / w are not read
  if (!L || !x || (!own_route && (!idx || !w)) || !ws || !yr) return DSGX_ERR_ARG;
  if (M > kMaxRows && M <= DSGX_MAX_STEP_ROWS) {  // 9..16 rows: rows 0..7, then the rest, in stream order on the same workspace
    if (cfg->parts != 0 && cfg->parts != 3) return DSGX_ERR_ARG;  // (the bench hooks address one launch sequence)
    const int rc0 = dsgx_moe_decode(s, L, x, idx, w, kMaxRows, ws, yr, ys, stream, cfg);
    if (rc0) return rc0;
    const size_t r = kMaxRows;
    dsgx_decode_cfg c2 = *cfg;
    if (c2.logits) c2.logits += r * s->E;
    return dsgx_moe_decode(s, L, reinterpret_cast<const uint8_t*>(x) + r * s->H * 2, idx ? idx + r * s->topk : nullptr,
                           w ? w + r * s->topk : nullptr, M - kMaxRows, ws, yr + r * s->H, ys ? ys + r * s->H : nullptr, stream, &c2);
  }
  if (M < 1 || M > kMaxRows) return DSGX_ERR_ARG;
  if (L->fmt != s->fmt) return DSGX_ERR_FORMAT;
  RouteParams rp{s->E, s->topk, s->n_group, s->topk_group, s->score_fn, s->norm_topk, s->route_scale};
  if (!L->pool || !L->desc) return DSGX_ERR_ARG;
  if (((uintptr_t)L->pool & 255) || ((uintptr_t)ws & 255) || ((uintptr_t)x & 15)) return DSGX_ERR_ARG;
  const bool sh8 = L->sh.g != nullptr;
  if (sh8 && (!L->sh.u || !L->sh.d || !L->sh.gs || !L->sh.us || !L->sh.ds)) return DSGX_ERR_ARG;
  if (fmt_fp8_family(s->fmt)) {
    if (L->sh.bg || L->sh.bu || L->sh.bd || L->sh.bgu) return DSGX_ERR_FORMAT;  // an FP8 layer's shared expert is FP8
    if (sh8 && !ys && !cfg->ysum) return DSGX_ERR_ARG;
    DecodeParams p;
    p.H = s->H, p.I = s->I, p.E = s->E, p.topk = s->topk, p.M = M, p.e_lo = s->e_lo, p.e_hi = s->e_hi;
    p.pool = L->pool, p.desc = L->desc, p.sh = L->sh;
    p.ws = decode_ws_carve(ws, s->H, s->I);
    p.idx = own_route ? p.ws.r_idx : idx, p.w = own_route ? p.ws.r_w : w;
    p.yr = yr, p.ys = ys, p.ysum = cfg->ysum, p.out = nullptr;
    p.up = cfg->up, p.down = cfg->down;
    p.sh_lo = s->sh_lo, p.sh_hi = s->sh_hi ? s->sh_hi : s->I, p.limit = s->swiglu_limit;
    p.norm = FrontNorm{nullptr, nullptr, 0.f, 0};
    p.mx = s->fmt == DSGX_FMT_MXFP4, p.b16 = 0;
    if (p.up < 0 || p.up >= decode_fp8_up_variants() || p.down < 0 || p.down >= decode_fp8_down_variants()) return DSGX_ERR_ARG;
    cudaError_t e = launch_decode_fp8(p, reinterpret_cast<const __nv_bfloat16*>(x), (cudaStream_t)stream, cfg->pdl != 0,
                                      cfg->parts == 0 ? 3 : cfg->parts, own_route ? &rp : nullptr, cfg->logits, cfg->bias);
    return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
  }
  if (s->fmt == DSGX_FMT_INT4 || s->fmt == DSGX_FMT_BF16) {
    if (L->sh.g || L->sh.u || L->sh.d) return DSGX_ERR_FORMAT;  // an INT4 or BF16 layer's shared expert is bf16
    const bool shb = L->sh.bg != nullptr || L->sh.bgu != nullptr;
    if (shb && (!L->sh.bd || (L->sh.bgu ? (L->sh.bg || L->sh.bu) : !L->sh.bu))) return DSGX_ERR_ARG;  // one of the two forms
    if (shb && !ys && !cfg->ysum) return DSGX_ERR_ARG;
    if (!decode_int4_fits(s->H, M)) return DSGX_ERR_SHAPE;
    DecodeParams p;
    p.H = s->H, p.I = s->I, p.E = s->E, p.topk = s->topk, p.M = M, p.e_lo = s->e_lo, p.e_hi = s->e_hi;
    p.pool = L->pool, p.desc = L->desc, p.sh = L->sh;
    p.ws = decode_ws_carve(ws, s->H, s->I);
    p.idx = own_route ? p.ws.r_idx : idx, p.w = own_route ? p.ws.r_w : w;
    p.yr = yr, p.ys = ys, p.ysum = cfg->ysum, p.out = nullptr, p.up = 0, p.down = 0;
    p.sh_lo = s->sh_lo, p.sh_hi = s->sh_hi ? s->sh_hi : s->I, p.limit = s->swiglu_limit;
    p.norm = FrontNorm{nullptr, nullptr, 0.f, 0};
    p.mx = 0, p.b16 = s->fmt == DSGX_FMT_BF16;
    cudaError_t e = launch_decode_int4(p, reinterpret_cast<const __nv_bfloat16*>(x), (cudaStream_t)stream, cfg->pdl != 0,
                                       cfg->parts == 0 ? 3 : cfg->parts, own_route ? &rp : nullptr, cfg->logits, cfg->bias);
    return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
  }
  return DSGX_ERR_UNSUPPORTED;
}

int dsgx_finalize(const float* R, const float* S, int M, int H, void* out, int mode, void* stream) {
  if (!R || !out || M < 1 || H < 1 || (mode != 0 && mode != 1)) return DSGX_ERR_ARG;
  cudaError_t e = launch_finalize(R, S, M, H, reinterpret_cast<__nv_bfloat16*>(out), mode, (cudaStream_t)stream, true);
  return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
}

int dsgx_moe_layer_decode(const dsgx_moe_shape* s, const dsgx_layer_w* L, const void* x, int M,
                          const dsgx_layer_step* st, int finalize, void* stream) {
  if (!st || !st->wr || !st->logits || !st->idx || !st->w || !st->ws || !st->yr) return DSGX_ERR_ARG;
  if (finalize && !st->out_bf16) return DSGX_ERR_ARG;
  int rc = check_shape(s);
  if (rc) return rc;
  if (M > kMaxRows && M <= DSGX_MAX_STEP_ROWS) {  // 9..16 rows: two launch sequences, every buffer moved on by eight rows
    rc = dsgx_moe_layer_decode(s, L, x, kMaxRows, st, finalize, stream);
    if (rc) return rc;
    const size_t r = kMaxRows;
    dsgx_layer_step b = *st;
    b.logits += r * s->E, b.idx += r * s->topk, b.w += r * s->topk, b.yr += r * s->H;
    if (b.ys) b.ys += r * s->H;
    if (b.out_bf16) b.out_bf16 = reinterpret_cast<uint8_t*>(b.out_bf16) + r * s->H * 2;
    if (b.xn_out) b.xn_out = reinterpret_cast<uint8_t*>(b.xn_out) + r * s->H * 2;
    return dsgx_moe_layer_decode(s, L, reinterpret_cast<const uint8_t*>(x) + r * s->H * 2, M - kMaxRows, &b, finalize, stream);
  }
  {
    if (!L || !x || !L->pool || !L->desc || L->fmt != s->fmt) return DSGX_ERR_ARG;
    if (M < 1 || M > kMaxRows) return DSGX_ERR_ARG;
    if (((uintptr_t)L->pool & 255) || ((uintptr_t)st->ws & 255) || ((uintptr_t)x & 15) || ((uintptr_t)st->wr & 15))
      return DSGX_ERR_ARG;
    const bool fp8 = fmt_fp8_family(s->fmt), mx = s->fmt == DSGX_FMT_MXFP4;
    const bool sh8 = L->sh.g != nullptr, shb = L->sh.bg != nullptr || L->sh.bgu != nullptr;
    if (fp8 ? shb : sh8) return DSGX_ERR_FORMAT;
    if (sh8 && (!L->sh.u || !L->sh.d || !L->sh.gs || !L->sh.us || !L->sh.ds || !st->ys)) return DSGX_ERR_ARG;
    if (shb && (!L->sh.bd || !st->ys || (L->sh.bgu ? (L->sh.bg || L->sh.bu) : !L->sh.bu))) return DSGX_ERR_ARG;
    if (!fp8 && !decode_int4_fits(s->H, M)) return DSGX_ERR_SHAPE;
    DecodeParams p;
    p.H = s->H, p.I = s->I, p.E = s->E, p.topk = s->topk, p.M = M, p.e_lo = s->e_lo, p.e_hi = s->e_hi;
    p.pool = L->pool, p.desc = L->desc, p.sh = L->sh;
    p.idx = st->idx, p.w = st->w;
    p.ws = decode_ws_carve(st->ws, s->H, s->I);
    p.yr = st->yr, p.ys = st->ys, p.ysum = 0, p.up = 0, p.down = 0;
    p.sh_lo = s->sh_lo, p.sh_hi = s->sh_hi ? s->sh_hi : s->I, p.limit = s->swiglu_limit;
    p.norm = FrontNorm{reinterpret_cast<const __nv_bfloat16*>(st->norm_w), reinterpret_cast<__nv_bfloat16*>(st->xn_out),
                       st->norm_eps, st->norm_mode};
    if (st->norm_w && ((st->norm_mode != 0 && st->norm_mode != 1) || !(st->norm_eps >= 0.f) || s->H % 8 ||
                       (((uintptr_t)st->norm_w | (uintptr_t)st->xn_out) & 15)))
      return DSGX_ERR_ARG;
    p.out = finalize ? reinterpret_cast<__nv_bfloat16*>(st->out_bf16) : nullptr;
    p.mx = mx, p.b16 = s->fmt == DSGX_FMT_BF16;
    RouteParams rp{s->E, s->topk, s->n_group, s->topk_group, s->score_fn, s->norm_topk, s->route_scale};
    const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
    // the whole step as one persistent kernel: measured faster from three rows up (flags bit 2 forces it, bit 0 forbids it)
    // Three rows and more: the whole step as one persistent kernel.  One or two rows: the four-kernel step is faster
    // (measured): the routing chain is too long to hide behind the little work that needs no routing.
    // flags: bit 0 never the one kernel; bit 2 always; bit 3: route with two small kernels, experts in the one kernel.
    const bool sh_part = p.sh_lo != 0 || p.sh_hi != s->I;  // (a part of the shared expert: the separate kernels)
    if (fp8 && !mx && !sh_part && !(st->flags & 1) && (M >= 3 || (st->flags & 28)) && step_fp8_fits(s->H, s->I, s->E, M)) {
      StepParams sp;
      sp.pre_routed = (st->flags & 8) ? 1 : 0;
      sp.test_no_table = (st->flags & 16) && !sp.pre_routed ? 1 : 0;
      if (sp.pre_routed) {
        cudaError_t e0 = launch_front_route_only(p, rp, xb, st->wr, st->bias, st->logits, st->idx, st->w, (cudaStream_t)stream, true);
        if (e0 != cudaSuccess) return cuda_fail(e0);
      }
      sp.d = p, sp.rp = rp, sp.x = xb, sp.wr = st->wr, sp.bias = st->bias, sp.logits = st->logits, sp.idx = st->idx;
      sp.w = st->w, sp.sync = p.ws.sync, sp.R = 0, sp.sh_slot = 0, sp.has_sh = 0;
      sp.stamps = (st->flags & 2) ? reinterpret_cast<unsigned long long*>(st->reserved_ptr) : nullptr;
      cudaError_t e = launch_step_fp8(sp, (cudaStream_t)stream);
      return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
    }
    cudaError_t e = fp8 ? launch_layer_fp8(p, rp, xb, st->wr, st->bias, st->logits, st->idx, st->w, (cudaStream_t)stream, true)
                        : launch_layer_int4(p, rp, xb, st->wr, st->bias, st->logits, st->idx, st->w, (cudaStream_t)stream, true);
    return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
  }
}

// the device address of a host buffer the device can reach (pinned and mapped), else null
static void* mapped_alias(const void* host) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, host) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return at.type == cudaMemoryTypeHost ? at.devicePointer : nullptr;
}

int dsgx_moe_layer_decode_host(const dsgx_moe_shape* s, const dsgx_layer_w* L, const void* x_host, int M,
                               const dsgx_layer_step* st, void* out_host, void* stream) {
  if (!st || !st->x_stage || !x_host || !s) return DSGX_ERR_ARG;
  if (out_host && !st->out_bf16) return DSGX_ERR_ARG;
  if (M < 1 || M > DSGX_MAX_STEP_ROWS) return DSGX_ERR_ARG;
  const size_t bytes = (size_t)M * s->H * 2;
  // Host buffers the device can address (pinned, mapped memory) are used in place: a small kernel pulls x over PCIe
  // into the staging buffer, and the step's last kernel writes the rounded rows straight into out_host, instead of two
  // copy-engine transfers of a few KB whose fixed cost is several microseconds each.
  void* x_dev = mapped_alias(x_host);
  void* out_dev = out_host ? mapped_alias(out_host) : nullptr;
  cudaError_t e;
  if (x_dev && bytes % 16 == 0 && ((uintptr_t)x_dev & 15) == 0)
    e = launch_copy_in(x_dev, st->x_stage, bytes, (cudaStream_t)stream);
  else
    e = cudaMemcpyAsync(st->x_stage, x_host, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_fail(e);
  if (!out_host) return dsgx_moe_layer_decode(s, L, st->x_stage, M, st, 0, stream);  // the partial sums only
  if (out_dev && ((uintptr_t)out_dev & 15) == 0) {
    dsgx_layer_step direct = *st;
    direct.out_bf16 = out_dev;
    return dsgx_moe_layer_decode(s, L, st->x_stage, M, &direct, 1, stream);
  }
  const int rc = dsgx_moe_layer_decode(s, L, st->x_stage, M, st, 1, stream);
  if (rc) return rc;
  e = cudaMemcpyAsync(out_host, st->out_bf16, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
}

static int check_prefill_shape(const dsgx_moe_shape* s) {
  const int rc = check_shape(s);
  if (rc) return rc;
  if (!fmt_fp8_family(s->fmt)) return DSGX_ERR_UNSUPPORTED;  // (MXFP4 layers: through an FP8 copy of the same weights)
  if (s->sh_lo || (s->sh_hi && s->sh_hi != s->I)) return DSGX_ERR_UNSUPPORTED;  // (the prefill pass runs whole experts)
  if (s->H % 256 || s->I % 128) return DSGX_ERR_SHAPE;
  return DSGX_OK;
}

size_t dsgx_prefill_weights_bytes(const dsgx_moe_shape* s) {
  if (check_prefill_shape(s)) return 0;
  return prefill_weights_bytes(s->H, s->I, s->E);
}

int dsgx_prefill_prepare(const dsgx_moe_shape* s, const dsgx_layer_w* L, void* wbuf, void* stream) {
  const int rc = check_prefill_shape(s);
  if (rc) return rc;
  if (!L || !L->pool || !L->desc || !wbuf || L->fmt != s->fmt) return DSGX_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const int H = s->H, I = s->I, E = s->E;
  PrefillWeights pw = prefill_weights_carve(wbuf, H, I, E);
  const int nloc = s->e_hi - s->e_lo;
  dsgx_mat_desc* hd = nloc > 0 ? new dsgx_mat_desc[(size_t)nloc * 3] : nullptr;
  cudaError_t e = cudaSuccess;
  if (nloc > 0) e = cudaMemcpy(hd, L->desc + (size_t)s->e_lo * 3, sizeof(dsgx_mat_desc) * nloc * 3, cudaMemcpyDeviceToHost);
  int bad = 0;
  const size_t mat = (size_t)I * H, sc = (size_t)(I / 128) * (H / 128);
  // MXFP4 layers: the copy holds the same weights as e4m3 with a power-of-two scale per 128 x 128 block (exact while a
  // block's scale bytes spread over at most 14; the flag word, first bytes of the copy's scale area until then, says
  // otherwise); twice the MXFP4 bytes
  const bool mx = s->fmt == DSGX_FMT_MXFP4;
  int* flag = nullptr;
  if (mx && e == cudaSuccess) {
    e = cudaMalloc(&flag, 4);  // (load time)
    if (e == cudaSuccess) e = cudaMemsetAsync(flag, 0, 4, st);
  }
  for (int i = 0; e == cudaSuccess && i < nloc; ++i) {
    const int ex = s->e_lo + i;
    for (int m = 0; m < 3; ++m) {
      const dsgx_mat_desc& d = hd[i * 3 + m];
      if (d.fmt != s->fmt || (d.off & 255)) {
        bad = 1;
        break;
      }
      const uint8_t* src = L->pool + d.off;
      uint8_t* dst = (m == 0 ? pw.g : m == 1 ? pw.u : pw.d) + (size_t)ex * mat;
      float* sdst = (m == 0 ? pw.sg : m == 1 ? pw.su : pw.sd) + (size_t)ex * sc;
      if (mx) {
        e = convert_mx4_matrix(src, m == 2 ? H : I, m == 2 ? I : H, dst, sdst, flag, st);
      } else {
        const float* ssrc = reinterpret_cast<const float*>(L->pool + ((uint64_t)d.rsv[0] | (uint64_t)d.rsv[1] << 32));
        e = retile_matrix(src, ssrc, m == 2 ? H : I, m == 2 ? I : H, dst, sdst, st);
      }
      if (e != cudaSuccess) break;
    }
    if (bad) break;
  }
  delete[] hd;
  int wide = 0;
  if (flag) {
    if (e == cudaSuccess && !bad) e = cudaMemcpyAsync(&wide, flag, 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(flag);
  }
  if (bad) return DSGX_ERR_FORMAT;
  if (wide) return DSGX_ERR_UNSUPPORTED;
  if (e == cudaSuccess && L->sh.g) {
    if (!L->sh.u || !L->sh.d || !L->sh.gs || !L->sh.us || !L->sh.ds) return DSGX_ERR_ARG;
    e = retile_matrix(L->sh.g, L->sh.gs, I, H, pw.g + (size_t)E * mat, pw.sg + (size_t)E * sc, st);
    if (e == cudaSuccess) e = retile_matrix(L->sh.u, L->sh.us, I, H, pw.u + (size_t)E * mat, pw.su + (size_t)E * sc, st);
    if (e == cudaSuccess) e = retile_matrix(L->sh.d, L->sh.ds, H, I, pw.d + (size_t)E * mat, pw.sd + (size_t)E * sc, st);
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
}

size_t dsgx_prefill_ws_bytes(const dsgx_moe_shape* s, int T) {
  if (check_prefill_shape(s) || T < 1) return 0;
  return prefill_ws_bytes(T, s->H, s->I, s->E, s->topk);
}

int dsgx_moe_prefill_phases(const dsgx_moe_shape* s, const dsgx_layer_w* L, const void* wbuf, const void* x, const int32_t* idx,
                            const float* w, int T, void* ws, float* yr, float* ys, void* out, int ysum, int phases,
                            void* stream) {
  const int rc = check_prefill_shape(s);
  if (rc) return rc;
  if (!L || !wbuf || !x || !idx || !w || !ws || (!yr && !out) || T < 1) return DSGX_ERR_ARG;
  if (phases < 1 || phases > DSGX_PH_ALL) return DSGX_ERR_ARG;
  if (((uintptr_t)wbuf & 255) || ((uintptr_t)ws & 255) || ((uintptr_t)x & 15)) return DSGX_ERR_ARG;
  const bool sh = L->sh.g != nullptr;
  if (sh && !ys && !(ysum & 1) && !out) return DSGX_ERR_ARG;
  if ((size_t)T * s->topk > (size_t)1 << 30) return DSGX_ERR_SHAPE;
  PrefillParams q;
  q.T = T, q.H = s->H, q.I = s->I, q.E = s->E, q.topk = s->topk, q.has_shared = sh, q.ysum = ysum & 1, q.phases = phases;
  q.e_lo = s->e_lo, q.e_hi = s->e_hi, q.limit = s->swiglu_limit;
  q.x = reinterpret_cast<const __nv_bfloat16*>(x), q.idx = idx, q.w = w;
  q.pw = prefill_weights_carve(const_cast<void*>(wbuf), s->H, s->I, s->E);
  q.ws = prefill_ws_carve(ws, T, s->H, s->I, s->E, s->topk);
  q.yr = yr, q.ys = ys, q.out = reinterpret_cast<__nv_bfloat16*>(out);
  cudaError_t e = cudaSuccess;
  if (phases & DSGX_PH_BUCKET) e = cudaMemsetAsync(q.ws.status, 0, 4, (cudaStream_t)stream);
  if (e == cudaSuccess) e = launch_prefill_fp8(q, (cudaStream_t)stream);
  return e == cudaSuccess ? DSGX_OK : cuda_fail(e);
}

int dsgx_moe_prefill(const dsgx_moe_shape* s, const dsgx_layer_w* L, const void* wbuf, const void* x, const int32_t* idx,
                     const float* w, int T, void* ws, float* yr, float* ys, void* out, int ysum, void* stream) {
  return dsgx_moe_prefill_phases(s, L, wbuf, x, idx, w, T, ws, yr, ys, out, ysum, DSGX_PH_ALL, stream);
}

int dsgx_prefill_view_of(const dsgx_moe_shape* s, void* ws, int T, dsgx_prefill_view* v) {
  const int rc = check_prefill_shape(s);
  if (rc) return rc;
  if (!ws || !v || T < 1) return DSGX_ERR_ARG;
  const PrefillWs w = prefill_ws_carve(ws, T, s->H, s->I, s->E, s->topk);
  v->counts = w.counts, v->offsets = w.offsets, v->perm_tok = w.perm_tok, v->perm_slot = w.perm_slot;
  v->pos_of = w.pos_of, v->row_order = w.row_order, v->hq = w.hq, v->hs = w.hs, v->hq_shared = w.hq_sh, v->hs_shared = w.hs_sh;
  return DSGX_OK;
}

int dsgx_decode_up_variants(void) { return decode_fp8_up_variants(); }
int dsgx_decode_down_variants(void) { return decode_fp8_down_variants(); }
const char* dsgx_decode_up_name(int v) { return decode_fp8_variant_name(0, v); }
const char* dsgx_decode_down_name(int v) { return decode_fp8_variant_name(1, v); }

int dsgx_sort_static_status(void) {
  int word = 0;
  cudaError_t e = sort_static_status(&word);
  if (e != cudaSuccess) return cuda_fail(e);
  return word ? DSGX_ERR_ARG : DSGX_OK;
}

int dsgx_ws_status(const void* ws) {
  if (!ws) return DSGX_ERR_ARG;
  int v = 0;
  cudaError_t e = cudaMemcpy(&v, ws, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return cuda_fail(e);
  return v;
}

}  // extern "C"
