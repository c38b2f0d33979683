"""Host-side mirror of the engine's MoE operator interface over the C ABI, with torch tensors as device memory.

Names and argument meaning follow the reference's `gx::` functions (altar1 engine/experts/experts.h:99-193): `route`,
`moe_decode`, `finalize`, `decode_ws_bytes`; `router_logits` stands in for the runner's router GEMV
(altar1 engine/model/model.cu:309-311).  torch is plumbing here (allocation, streams); every computation is a kernel of
the CUDA library.
"""
import ctypes as C

import torch

from . import _lib
from ._lib import MoeShape, check, lib


def shape(H, I, E, topk, fmt=_lib.FMT_FP8, n_group=1, topk_group=1, score_fn=_lib.SCORE_SIGMOID, norm_topk=True,
          route_scale=1.0, e_lo=0, e_hi=None, sh_lo=0, sh_hi=0, swiglu_limit=0.0):
    return MoeShape(H, I, E, topk, n_group, topk_group, score_fn, int(norm_topk), route_scale, fmt, e_lo,
                    E if e_hi is None else e_hi, sh_lo, sh_hi, swiglu_limit, 0)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


def router_logits(x, wr):
    """x bf16 [M][H], wr f32 [E][H] -> logits f32 [M][E]."""
    M, H = x.shape
    E = wr.shape[0]
    out = torch.empty(M, E, dtype=torch.float32, device=x.device)
    check(lib().dsgx_router_logits(_ptr(x), _ptr(wr), M, H, E, _ptr(out), _stream()), "dsgx_router_logits")
    return out


def route(shp, logits, bias=None):
    """logits f32 [M][E] -> (idx int32 [M][topk], w f32 [M][topk])."""
    M = logits.shape[0]
    idx = torch.empty(M, shp.topk, dtype=torch.int32, device=logits.device)
    w = torch.empty(M, shp.topk, dtype=torch.float32, device=logits.device)
    check(lib().dsgx_route(C.byref(shp), _ptr(logits), _ptr(bias), M, _ptr(idx), _ptr(w), _stream()), "dsgx_route")
    return idx, w


def sort_pack(idx, E):
    T, k = idx.shape
    dev = idx.device
    i32 = dict(dtype=torch.int32, device=dev)
    out = dict(counts=torch.empty(E, **i32), offsets=torch.empty(E + 1, **i32), perm_tok=torch.empty(T * k, **i32),
               perm_slot=torch.empty(T * k, **i32), pos_of=torch.empty(T, k, **i32), row_order=torch.empty(T, k, **i32))
    ws = torch.empty(max(lib().dsgx_sort_ws_bytes(T, k, E), 256), dtype=torch.uint8, device=dev)
    check(lib().dsgx_sort_pack(_ptr(idx), T, k, E, _ptr(out["counts"]), _ptr(out["offsets"]), _ptr(out["perm_tok"]),
                               _ptr(out["perm_slot"]), _ptr(out["pos_of"]), _ptr(out["row_order"]), _ptr(ws), _stream()),
          "dsgx_sort_pack")
    return out


def decode_variants():
    """The names of the decode kernels' variants: (gate/up, down)."""
    L = lib()
    return ([L.dsgx_decode_up_name(i).decode() for i in range(L.dsgx_decode_up_variants())],
            [L.dsgx_decode_down_name(i).decode() for i in range(L.dsgx_decode_down_variants())])


def sort_pack_static(idx, E):
    """sort_pack through the entry point that takes no workspace and allocates nothing (fixed scratch in the library)."""
    T, k = idx.shape
    i32 = dict(dtype=torch.int32, device=idx.device)
    out = dict(counts=torch.empty(E, **i32), offsets=torch.empty(E + 1, **i32), perm_tok=torch.empty(T * k, **i32),
               perm_slot=torch.empty(T * k, **i32), pos_of=torch.empty(T, k, **i32), row_order=torch.empty(T, k, **i32))
    check(lib().dsgx_sort_pack_static(_ptr(idx), T, k, E, _ptr(out["counts"]), _ptr(out["offsets"]), _ptr(out["perm_tok"]),
                                      _ptr(out["perm_slot"]), _ptr(out["pos_of"]), _ptr(out["row_order"]), _stream()),
          "dsgx_sort_pack_static")
    return out


def decode_ws_bytes(shp):
    n = lib().dsgx_decode_ws_bytes(C.byref(shp))
    if n == 0:
        raise _lib.DsgxError(_lib.ERR_SHAPE, "dsgx_decode_ws_bytes")
    return n


def decode_ws(shp, device="cuda"):
    """A zeroed decode workspace (zeroed once; the kernels leave its counters at zero)."""
    return torch.zeros(decode_ws_bytes(shp), dtype=torch.uint8, device=device)


def moe_decode(shp, layer_w, x, idx, w, ws, yr=None, ys=None, ysum=False, pdl=True, parts=0, up=0, down=0, logits=None,
               bias=None):
    """x bf16 [M][H]; idx, w from route(); returns (yr, ys) f32 [M][H]: this GPU's partial sums.
    logits (f32 [M][E], with an optional selection bias): the step routes the rows itself, idx and w may be None."""
    M, H = x.shape
    if yr is None:
        yr = torch.empty(M, H, dtype=torch.float32, device=x.device)
    if ys is None:
        ys = torch.empty(M, H, dtype=torch.float32, device=x.device)
    cfg = _lib.DecodeCfg(int(ysum), int(pdl), int(parts), int(up), int(down), (C.c_int32 * 3)(0, 0, 0), _ptr(logits), _ptr(bias))
    check(lib().dsgx_moe_decode(C.byref(shp), C.byref(layer_w), _ptr(x), _ptr(idx), _ptr(w), M, _ptr(ws), _ptr(yr),
                                _ptr(ys), _stream(), C.byref(cfg)), "dsgx_moe_decode")
    return yr, ys


def finalize(R, S=None, mode=0):
    M, H = R.shape
    out = torch.empty(M, H, dtype=torch.bfloat16, device=R.device)
    check(lib().dsgx_finalize(_ptr(R), _ptr(S), M, H, _ptr(out), mode, _stream()), "dsgx_finalize")
    return out


def add_norm_args(norm_w, res=None, eps=1e-6, norm_mode=0, add_f32=False, res_out=None, normed=None):
    """The dsgx_add_norm struct over torch tensors (res_out / normed: given buffers, or made here when True)."""
    return _lib.AddNorm(_ptr(res), _ptr(res_out), _ptr(norm_w), _ptr(normed), eps, norm_mode, int(add_f32), 0)


def finalize_add_norm(R, S, norm_w, res=None, mode=0, eps=1e-6, norm_mode=0, add_f32=False):
    """One GPU: out = bf16(R + S), h = bf16(res + out), normed = RMSNorm(h): returns (out, h, normed), bf16 [M][H]."""
    M, H = R.shape
    out, h, normed = (torch.empty(M, H, dtype=torch.bfloat16, device=R.device) for _ in range(3))
    an = add_norm_args(norm_w, res, eps, norm_mode, add_f32, h, normed)
    check(lib().dsgx_finalize_add_norm(_ptr(R), _ptr(S), M, H, mode, _ptr(out), C.byref(an), _stream()), "dsgx_finalize_add_norm")
    return out, h, normed


def ws_status(ws):
    return lib().dsgx_ws_status(_ptr(ws))


class LayerStep:
    """The buffers of one layer step (router to rounded output) and the two step calls."""

    def __init__(self, shp, wr, bias=None, device="cuda", fused=None, stamps=None, norm_w=None, norm_eps=1e-6, norm_mode=0):
        """fused: None = the library's choice by row count, True = always the one-kernel step, False = never.
        norm_w (bf16 [H]): the step normalises its input rows first (RMSNorm fused into the front); self.xn gets a copy."""
        f32 = dict(dtype=torch.float32, device=device)
        self.shp, self.wr, self.bias = shp, wr, bias
        self.logits = torch.empty(_lib.MAX_STEP_ROWS, shp.E, **f32)
        self.idx = torch.empty(_lib.MAX_STEP_ROWS, shp.topk, dtype=torch.int32, device=device)
        self.w = torch.empty(_lib.MAX_STEP_ROWS, shp.topk, **f32)
        self.ws = decode_ws(shp, device)
        self.yr = torch.zeros(_lib.MAX_STEP_ROWS, shp.H, **f32)
        self.ys = torch.zeros(_lib.MAX_STEP_ROWS, shp.H, **f32)
        self.out = torch.zeros(_lib.MAX_STEP_ROWS, shp.H, dtype=torch.bfloat16, device=device)
        self.x_stage = torch.zeros(_lib.MAX_STEP_ROWS, shp.H, dtype=torch.bfloat16, device=device)
        self.c = _lib.LayerStep(_ptr(wr), _ptr(bias), _ptr(self.logits), _ptr(self.idx), _ptr(self.w), _ptr(self.ws),
                                _ptr(self.yr), _ptr(self.ys), _ptr(self.out), _ptr(self.x_stage),
                                (0 if fused is None else 4 if fused else 1) | (2 if stamps is not None else 0), 0, _ptr(stamps))
        self.norm_w = norm_w
        if norm_w is not None:
            self.xn = torch.zeros(_lib.MAX_STEP_ROWS, shp.H, dtype=torch.bfloat16, device=device)
            self.c.norm_w, self.c.xn_out, self.c.norm_eps, self.c.norm_mode = _ptr(norm_w), _ptr(self.xn), norm_eps, norm_mode

    def run(self, layer_w, x, finalize=True, yr=None, ys=None):
        """x bf16 [M][H] on the device -> self.out[:M] (bf16) when finalize, else self.yr / self.ys partial sums
        (or the f32 [8][H] buffers given as yr, ys: an expert-parallel rank's share of a peer-reduced step)."""
        M = x.shape[0]
        c = self.c
        if yr is not None:
            c = _lib.LayerStep.from_buffer_copy(self.c)
            c.yr, c.ys = _ptr(yr), _ptr(ys)
        check(lib().dsgx_moe_layer_decode(C.byref(self.shp), C.byref(layer_w), _ptr(x), M, C.byref(c),
                                          int(finalize), _stream()), "dsgx_moe_layer_decode")
        return self.out[:M]

    def run_host(self, layer_w, x_host, out_host, yr=None, ys=None):
        """x_host, out_host: pinned bf16 host tensors [M][H]; copies, the step and the read-back in stream order.
        out_host None: the step stops at the partial sums (in yr, ys when given: a peer-reduced step's buffers)."""
        M = x_host.shape[0]
        c = self.c
        if yr is not None:
            c = _lib.LayerStep.from_buffer_copy(self.c)
            c.yr, c.ys = _ptr(yr), _ptr(ys)
        check(lib().dsgx_moe_layer_decode_host(C.byref(self.shp), C.byref(layer_w), _ptr(x_host), M, C.byref(c),
                                               _ptr(out_host), _stream()), "dsgx_moe_layer_decode_host")
        return out_host


def prefill_view(shp, ws, T):
    v = _lib.PrefillView()
    check(lib().dsgx_prefill_view_of(C.byref(shp), _ptr(ws), T, C.byref(v)), "dsgx_prefill_view_of")
    return v


class PrefillLayer:
    """A layer prepared for the prefill path: the K-major weight copy (made once) and a workspace for up to T_max rows."""

    def __init__(self, shp, layer_w, T_max, device="cuda", wbuf=None):
        """wbuf: the prepared weight copy of another PrefillLayer of the same layer (a second workspace, e.g. for a
        second stream, shares it)."""
        self.shp, self.layer_w, self.T_max = shp, layer_w, T_max
        nb = lib().dsgx_prefill_weights_bytes(C.byref(shp))
        if nb == 0:
            raise _lib.DsgxError(_lib.ERR_SHAPE, "dsgx_prefill_weights_bytes")
        if wbuf is not None:
            self.wbuf = wbuf
        else:
            self.wbuf = torch.empty(nb, dtype=torch.uint8, device=device)
            check(lib().dsgx_prefill_prepare(C.byref(shp), C.byref(layer_w), _ptr(self.wbuf), _stream()), "dsgx_prefill_prepare")
        self.ws = torch.empty(lib().dsgx_prefill_ws_bytes(C.byref(shp), T_max), dtype=torch.uint8, device=device)

    def run(self, x, idx, w, yr=None, ys=None, out=None, ysum=False, parts=0, phases=None):
        """x bf16 [T][H]; idx, w from route(); returns (yr, ys, out): f32 partial sums and bf16(yr + ys).
        phases: DSGX_PH_* bits (default: the whole pass); parts 1 / 2: the routed gate/up / down GEMM alone."""
        T, H = x.shape
        assert T <= self.T_max
        f32 = dict(dtype=torch.float32, device=x.device)
        yr = torch.empty(T, H, **f32) if yr is None else (None if yr is False else yr)   # False: rounded rows only
        ys = torch.empty(T, H, **f32) if ys is None else (None if ys is False else ys)
        out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device) if out is None else (None if out is False else out)
        if phases is None:
            phases = {0: _lib.PH_ALL, 1: _lib.PH_UP, 2: _lib.PH_DOWN}[parts]
        check(lib().dsgx_moe_prefill_phases(C.byref(self.shp), C.byref(self.layer_w), _ptr(self.wbuf), _ptr(x), _ptr(idx),
                                            _ptr(w), T, _ptr(self.ws), _ptr(yr), _ptr(ys), _ptr(out), int(ysum), phases,
                                            _stream()), "dsgx_moe_prefill_phases")
        return yr, ys, out
