"""Loads the in-tree CUDA library through its C ABI (include/dsgx_moe.h).  There is no fallback: a missing or
unloadable library is an error, never a silent CPU path."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libdsgx_moe.so")

OK, ERR_ARG, ERR_FORMAT, ERR_SHAPE, ERR_CUDA, ERR_DEVICE_WAIT, ERR_UNSUPPORTED, ERR_LIMIT = range(8)
FMT_NVFP4, FMT_RETIRED, FMT_INT4, FMT_BF16, FMT_FP8, FMT_MXFP4 = range(6)
SCORE_SIGMOID, SCORE_SOFTMAX, SCORE_SQRTSOFTPLUS = 0, 1, 2
MAX_ROWS = 8         # rows one launch sequence takes
MAX_STEP_ROWS = 16   # rows a decode call takes (9..16: two sequences)
PH_BUCKET, PH_UP, PH_DOWN, PH_COMBINE, PH_SHARED, PH_ALL = 1, 2, 4, 8, 16, 31


class MatDesc(C.Structure):
    _fields_ = [("off", C.c_uint64), ("s2", C.c_float), ("fmt", C.c_uint32), ("rsv", C.c_uint32 * 12)]


class SharedW(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("g", "u", "d", "gs", "us", "ds", "bg", "bu", "bd", "bgu")]


class LayerW(C.Structure):
    _fields_ = [("pool", C.c_void_p), ("desc", C.c_void_p), ("sh", SharedW), ("fmt", C.c_uint32)]


class MoeShape(C.Structure):
    _fields_ = [("H", C.c_int32), ("I", C.c_int32), ("E", C.c_int32), ("topk", C.c_int32), ("n_group", C.c_int32),
                ("topk_group", C.c_int32), ("score_fn", C.c_int32), ("norm_topk", C.c_int32),
                ("route_scale", C.c_float), ("fmt", C.c_uint32), ("e_lo", C.c_int32), ("e_hi", C.c_int32),
                ("sh_lo", C.c_int32), ("sh_hi", C.c_int32), ("swiglu_limit", C.c_float), ("reserved", C.c_int32)]


class PeerSet(C.Structure):
    _fields_ = [("parts", C.c_void_p), ("flags", C.c_void_p), ("state", C.c_void_p), ("rank", C.c_int32),
                ("world", C.c_int32), ("rows_cap", C.c_int32), ("shared_rank", C.c_int32),
                ("outs", C.c_void_p), ("done", C.c_void_p)]


class PrefillView(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("counts", "offsets", "perm_tok", "perm_slot", "pos_of", "row_order", "hq", "hs",
                                          "hq_shared", "hs_shared")]


class DecodeCfg(C.Structure):
    _fields_ = [("ysum", C.c_int32), ("pdl", C.c_int32), ("parts", C.c_int32), ("up", C.c_int32),
                ("down", C.c_int32), ("reserved", C.c_int32 * 3), ("logits", C.c_void_p), ("bias", C.c_void_p)]


class LayerStep(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("wr", "bias", "logits", "idx", "w", "ws", "yr", "ys", "out_bf16", "x_stage")] + \
               [("flags", C.c_int32), ("reserved", C.c_int32), ("reserved_ptr", C.c_void_p),
                ("norm_w", C.c_void_p), ("xn_out", C.c_void_p), ("norm_eps", C.c_float), ("norm_mode", C.c_int32)]


class AddNorm(C.Structure):
    _fields_ = [("res", C.c_void_p), ("res_out", C.c_void_p), ("norm_w", C.c_void_p), ("normed", C.c_void_p),
                ("eps", C.c_float), ("norm_mode", C.c_int32), ("add_f32", C.c_int32), ("reserved", C.c_int32)]


# every symbol include/dsgx_moe.h declares: name -> (restype, argtypes)
_V, _I, _Z = C.c_void_p, C.c_int, C.c_size_t
SYMBOLS = {
    "dsgx_last_cuda_error": (_I, []),
    "dsgx_status_name": (C.c_char_p, [_I]),
    "dsgx_router_logits": (_I, [_V, _V, _I, _I, _I, _V, _V]),
    "dsgx_route": (_I, [C.POINTER(MoeShape), _V, _V, _I, _V, _V, _V]),
    "dsgx_sort_ws_bytes": (_Z, [_I, _I, _I]),
    "dsgx_sort_pack": (_I, [_V, _I, _I, _I, _V, _V, _V, _V, _V, _V, _V, _V]),
    "dsgx_finalize_peers": (_I, [_V, _I, _I, _V, _V, _V]),
    "dsgx_finalize_peers_norm": (_I, [_V, _I, _I, _V, C.POINTER(AddNorm), _V, _V]),
    "dsgx_finalize_add_norm": (_I, [_V, _V, _I, _I, _I, _V, C.POINTER(AddNorm), _V]),
    "dsgx_sort_pack_static": (_I, [_V, _I, _I, _I, _V, _V, _V, _V, _V, _V, _V]),
    "dsgx_decode_ws_bytes": (_Z, [C.POINTER(MoeShape)]),
    "dsgx_moe_decode": (_I, [C.POINTER(MoeShape), C.POINTER(LayerW), _V, _V, _V, _I, _V, _V, _V, _V,
                             C.POINTER(DecodeCfg)]),
    "dsgx_finalize": (_I, [_V, _V, _I, _I, _V, _I, _V]),
    "dsgx_moe_layer_decode": (_I, [C.POINTER(MoeShape), C.POINTER(LayerW), _V, _I, C.POINTER(LayerStep), _I, _V]),
    "dsgx_moe_layer_decode_host": (_I, [C.POINTER(MoeShape), C.POINTER(LayerW), _V, _I, C.POINTER(LayerStep), _V, _V]),
    "dsgx_prefill_weights_bytes": (_Z, [C.POINTER(MoeShape)]),
    "dsgx_prefill_prepare": (_I, [C.POINTER(MoeShape), C.POINTER(LayerW), _V, _V]),
    "dsgx_prefill_ws_bytes": (_Z, [C.POINTER(MoeShape), _I]),
    "dsgx_moe_prefill": (_I, [C.POINTER(MoeShape), C.POINTER(LayerW), _V, _V, _V, _V, _I, _V, _V, _V, _V, _I, _V]),
    "dsgx_moe_prefill_phases": (_I, [C.POINTER(MoeShape), C.POINTER(LayerW), _V, _V, _V, _V, _I, _V, _V, _V, _V, _I, _I, _V]),
    "dsgx_prefill_view_of": (_I, [C.POINTER(MoeShape), _V, _I, _V]),
    "dsgx_decode_up_variants": (_I, []),
    "dsgx_decode_down_variants": (_I, []),
    "dsgx_decode_up_name": (C.c_char_p, [_I]),
    "dsgx_decode_down_name": (C.c_char_p, [_I]),
    "dsgx_sort_static_status": (_I, []),
    "dsgx_ws_status": (_I, [_V]),
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m dsgx10_b200.build` "
                               "(there is no CPU fallback)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            f = getattr(L, name)  # AttributeError if the library lacks a declared symbol
            f.restype, f.argtypes = res, args
        _lib = L
    return _lib


class DsgxError(RuntimeError):
    def __init__(self, status, where):
        self.status = status
        name = lib().dsgx_status_name(status).decode()
        extra = f" (cuda error {lib().dsgx_last_cuda_error()})" if status == ERR_CUDA else ""
        super().__init__(f"{where}: {name}{extra}")


def check(status, where):
    if status != OK:
        raise DsgxError(status, where)
