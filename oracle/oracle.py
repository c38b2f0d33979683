"""ctypes front of the CPU oracle (oracle/moe_oracle.c) and of the reference shim (oracle/_ref/libref_shim.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by bench.py's cpu_baseline / reference
legs as the checker and the timed CPU arm; the library itself never imports it.

All arrays are numpy: bf16 travels as uint16 bit patterns, e4m3 as uint8 codes.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

SCORE_SIGMOID, SCORE_SOFTMAX, SCORE_SQRTSOFTPLUS = 0, 1, 2


def build(with_ref=True):
    """Compile liboracle.so and, when the reference tree is there (environment variable DSGX_REFERENCE, else the
    directory `reference` beside this repository), the shim over the reference's own host functions."""
    ref = os.environ.get("DSGX_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    cmd = ["make", "-s", "-C", HERE, "all" if with_ref else os.path.join(HERE, "liboracle.so")]
    if with_ref and os.path.isdir(ref):
        cmd.append("REF=" + ref)
    subprocess.run(cmd, check=True)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path):
            build(with_ref=False)
        L = C.CDLL(path)
        L.orc_bf16_to_f32.restype = C.c_float
        L.orc_bf16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_bf16.restype = C.c_uint16
        L.orc_f32_to_bf16.argtypes = [C.c_float]
        L.orc_e4m3_to_f32.restype = C.c_float
        L.orc_e4m3_to_f32.argtypes = [C.c_uint8]
        L.orc_f32_to_e4m3.restype = C.c_uint8
        L.orc_f32_to_e4m3.argtypes = [C.c_float]
        L.orc_route_sigmoid.restype = C.c_float
        L.orc_route_sigmoid.argtypes = [C.c_float]
        L.orc_route_sqrtsoftplus.restype = C.c_float
        L.orc_route_sqrtsoftplus.argtypes = [C.c_float]
        L.orc_read_int4_block.restype = C.c_uint16
        L.orc_num_threads.restype = C.c_int
        _LIB = L
    return _LIB


def ref():
    """The shim over the reference's own host functions, or None when it was not built."""
    global _REF
    if _REF is None:
        path = os.path.join(HERE, "_ref", "libref_shim.so")
        if not os.path.exists(path):
            return None
        R = C.CDLL(path)
        R.ref_route_sigmoid.restype = C.c_float
        R.ref_route_sigmoid.argtypes = [C.c_float]
        R.ref_e4m3_to_f.restype = C.c_float
        R.ref_e4m3_to_f.argtypes = [C.c_uint8]
        R.ref_f_to_bf16_bits.restype = C.c_uint16
        R.ref_f_to_bf16_bits.argtypes = [C.c_float]
        R.ref_i4_value_bits.restype = C.c_uint16
        R.ref_i4_value_bits.argtypes = [C.c_int, C.c_int, C.c_uint16]
        R.ref_read_fp8.restype = C.c_float
        R.ref_read_i4.restype = C.c_uint16
        R.ref_fp8_value.restype = C.c_float
        _REF = R
    return _REF


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


# ---------------------------------------------------------------------------------------------- scalar formats

def f32_to_bf16(a):
    """numpy f32 -> bf16 bits (uint16), round to nearest even."""
    u = _c(a, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r.reshape(np.shape(a))


def bf16_to_f32(b):
    return (_c(b, np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(np.shape(b))


_E4M3_LUT = None


def e4m3_to_f32(q):
    global _E4M3_LUT
    if _E4M3_LUT is None:
        L = lib()
        _E4M3_LUT = np.array([L.orc_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)
    return _E4M3_LUT[_c(q, np.uint8)]


def f32_to_e4m3(a):
    L = lib()
    a = _c(a, np.float32)
    return np.array([L.orc_f32_to_e4m3(float(v)) for v in a.ravel()], dtype=np.uint8).reshape(a.shape)


# ------------------------------------------------------------------------------------------------------ router

def router_logits(x_bf16, wr):
    x_bf16, wr = _c(x_bf16, np.uint16), _c(wr, np.float32)
    R, H = x_bf16.shape
    E = wr.shape[0]
    out = np.empty((R, E), np.float32)
    rc = lib().orc_router_logits(_p(x_bf16), _p(wr), R, H, E, _p(out))
    assert rc == 0
    return out


def rmsnorm(x_bf16, w_bf16, eps=1e-6, mode=0):
    """RMSNorm of bf16 rows (bits in, bits out); mode 0: bf16(w (x r)), mode 1: bf16(w bf16(x r))."""
    x_bf16, w_bf16 = _c(x_bf16, np.uint16), _c(w_bf16, np.uint16)
    R, H = x_bf16.shape
    y = np.empty((R, H), np.uint16)
    assert lib().orc_rmsnorm(_p(x_bf16), _p(w_bf16), R, H, C.c_float(eps), mode, _p(y)) == 0
    return y


def add_norm(v, res_bf16, w_bf16, eps=1e-6, mode=0, add_f32=False):
    """out = bf16(v); h = bf16(res + out) (or res + v); normed = RMSNorm(h).  Returns (out, h, normed) as bf16 bits."""
    v, w_bf16 = _c(v, np.float32), _c(w_bf16, np.uint16)
    R, H = v.shape
    res = None if res_bf16 is None else _c(res_bf16, np.uint16)
    out, h, normed = (np.empty((R, H), np.uint16) for _ in range(3))
    assert lib().orc_add_norm(_p(v), _p(res) if res is not None else None, _p(w_bf16), R, H, C.c_float(eps), mode,
                              int(add_f32), _p(out), _p(h), _p(normed)) == 0
    return out, h, normed


def route(logits, bias, topk, score_fn=SCORE_SIGMOID, n_group=1, topk_group=1, norm=True, route_scale=1.0):
    logits = _c(logits, np.float32)
    R, E = logits.shape
    bias = None if bias is None else _c(bias, np.float32)
    idx = np.empty((R, topk), np.int32)
    w = np.empty((R, topk), np.float32)
    rc = lib().orc_route(_p(logits), _p(bias), R, E, topk, score_fn, n_group, topk_group, int(norm),
                         C.c_float(route_scale), _p(idx), _p(w))
    if rc != 0:
        raise ValueError("orc_route: bad arguments")
    return idx, w


def sort_pack(idx, E):
    idx = _c(idx, np.int32)
    T, k = idx.shape
    counts = np.empty(E, np.int32)
    offsets = np.empty(E + 1, np.int32)
    perm_tok = np.empty(T * k, np.int32)
    perm_slot = np.empty(T * k, np.int32)
    pos_of = np.empty((T, k), np.int32)
    row_order = np.empty((T, k), np.int32)
    rc = lib().orc_sort_pack(_p(idx), T, k, E, _p(counts), _p(offsets), _p(perm_tok), _p(perm_slot), _p(pos_of),
                             _p(row_order))
    if rc != 0:
        raise ValueError("orc_sort_pack: expert id out of range")
    return dict(counts=counts, offsets=offsets, perm_tok=perm_tok, perm_slot=perm_slot, pos_of=pos_of,
                row_order=row_order)


# --------------------------------------------------------------------------------------------------------- FP8

def act_quant(v):
    """f32 [..., n] -> (e4m3 codes uint8 [..., n], f32 scales [..., n/128])."""
    v = _c(v, np.float32)
    n = v.shape[-1]
    rows = v.reshape(-1, n)
    q = np.empty(rows.shape, np.uint8)
    s = np.empty((rows.shape[0], n // 128), np.float32)
    L = lib()
    for r in range(rows.shape[0]):
        L.orc_act_quant(_p(rows[r]), n, _p(q[r]), _p(s[r]))
    return q.reshape(v.shape), s.reshape(v.shape[:-1] + (n // 128,))


def _ptr_array(arrs):
    a = (C.c_void_p * len(arrs))()
    for i, x in enumerate(arrs):
        a[i] = None if x is None else x.ctypes.data
    return a


def fp8_expert_row(x_bf16, wg, sg, wu, su, wd, sd, wroute=None, swiglu_limit=0.0):
    """One expert on one row.  Returns (y [H] f32 (bf16-rounded values), h [I] f32 (bf16-rounded values))."""
    I, H = wg.shape
    y = np.empty(H, np.float32)
    h = np.empty(I, np.float32)
    x_bf16 = _c(x_bf16, np.uint16)
    lib().orc_fp8_expert_row(_p(x_bf16), H, I, _p(wg), _p(sg), _p(wu), _p(su), _p(wd), _p(sd),
                             C.c_float(-1.0 if wroute is None else wroute), C.c_float(swiglu_limit), _p(y), _p(h))
    return y, h


def mx4_expert_row(x_bf16, wg, sg, wu, su, wd, sd, wroute=None, swiglu_limit=0.0):
    """One MXFP4 expert (nibble bytes [N][K/2], ue8m0 bytes [N][K/32]) on one row: (y [H], h [I]) as bf16-rounded f32."""
    I, H = wg.shape[0], wg.shape[1] * 2
    y, h = np.empty(H, np.float32), np.empty(I, np.float32)
    x_bf16 = _c(x_bf16, np.uint16)
    lib().orc_mx4_expert_row(_p(x_bf16), H, I, _p(wg), _p(sg), _p(wu), _p(su), _p(wd), _p(sd),
                             C.c_float(-1.0 if wroute is None else wroute), C.c_float(swiglu_limit), _p(y), _p(h))
    return y, h


def mx4_dequant(q, s):
    q, s = _c(q, np.uint8), _c(s, np.uint8)
    N, K = q.shape[0], q.shape[1] * 2
    out = np.empty((N, K), np.float32)
    lib().orc_mx4_dequant(_p(q), _p(s), N, K, _p(out))
    return out


def moe_fp8_layer(x_bf16, idx, w, experts, shared, e_lo=0, e_hi=None, with_shared=True, swiglu_limit=0.0,
                  pickmax=False, mx4=False):
    """experts: dict e -> (wg, sg, wu, su, wd, sd) canonical numpy arrays (only the picked experts need be present);
    shared: the same tuple or None.  mx4: the routed experts are MXFP4 (nibble bytes, ue8m0 bytes), the shared one FP8.
    Returns (acc f32 [T][H], out bf16 bits [T][H]) and, with pickmax, a third array
    f32 [T][H]: per element the largest magnitude among the bf16 outputs that were added there."""
    x_bf16, idx, w = _c(x_bf16, np.uint16), _c(idx, np.int32), _c(w, np.float32)
    T, H = x_bf16.shape
    k = idx.shape[1]
    E = max(list(experts.keys()) + [int(idx.max())]) + 1
    e_hi = E if e_hi is None else e_hi
    cols = [[None] * (E + 1) for _ in range(6)]
    I = None
    for e, tup in list(experts.items()) + ([(E, shared)] if shared is not None else []):
        for c in range(6):
            cols[c][e] = tup[c]
        I = tup[0].shape[0]
    acc = np.empty((T, H), np.float32)
    out = np.empty((T, H), np.uint16)
    pa = [_ptr_array(c) for c in cols]
    pm = np.empty((T, H), np.float32) if pickmax else None
    fn = lib().orc_moe_mx4_layer if mx4 else lib().orc_moe_fp8_layer
    rc = fn(_p(x_bf16), _p(idx), _p(w), T, H, I, E, k, pa[0], pa[1], pa[2], pa[3], pa[4], pa[5], e_lo, e_hi,
            int(with_shared), C.c_float(swiglu_limit), _p(acc), _p(out), _p(pm))
    assert rc == 0
    return (acc, out, pm) if pickmax else (acc, out)


def pack_fp8_tile(w):
    w = _c(w, np.uint8)
    out = np.empty(w.size, np.uint8)
    lib().orc_pack_fp8_tile(_p(w), w.shape[0], w.shape[1], _p(out))
    return out


def unpack_fp8_tile(m, N, K):
    m = _c(m, np.uint8)
    out = np.empty((N, K), np.uint8)
    lib().orc_unpack_fp8_tile(_p(m), N, K, _p(out))
    return out


# -------------------------------------------------------------------------------------------------------- INT4

def int4_dequant(wp, s, zp=None):
    """wp uint8 [N][K/2], s bf16 bits [N][K/32], zp uint32 [N/8][K/32] or None -> bf16 bits [N][K]."""
    wp, s = _c(wp, np.uint8), _c(s, np.uint16)
    zp = None if zp is None else _c(zp, np.uint32)
    N, K = wp.shape[0], wp.shape[1] * 2
    out = np.empty((N, K), np.uint16)
    lib().orc_int4_dequant(_p(wp), _p(s), _p(zp), N, K, _p(out))
    return out


def bf16w_expert_row(x_bf16, wg, wu, wd):
    I, H = wg.shape
    y = np.empty(H, np.float32)
    h = np.empty(I, np.float32)
    x_bf16 = _c(x_bf16, np.uint16)
    lib().orc_bf16w_expert_row(_p(x_bf16), H, I, _p(wg), _p(wu), _p(wd), _p(y), _p(h))
    return y, h


def moe_bf16w_layer(x_bf16, idx, w, experts, shared, e_lo=0, e_hi=None, with_shared=True):
    """experts: dict e -> (wg, wu, wd) bf16-bit arrays (dequantised INT4); shared likewise or None."""
    x_bf16, idx, w = _c(x_bf16, np.uint16), _c(idx, np.int32), _c(w, np.float32)
    T, H = x_bf16.shape
    k = idx.shape[1]
    E = max(list(experts.keys()) + [int(idx.max())]) + 1
    e_hi = E if e_hi is None else e_hi
    cols = [[None] * (E + 1) for _ in range(3)]
    I = None
    for e, tup in list(experts.items()) + ([(E, shared)] if shared is not None else []):
        for c in range(3):
            cols[c][e] = tup[c]
        I = tup[0].shape[0]
    acc = np.empty((T, H), np.float32)
    out = np.empty((T, H), np.uint16)
    pa = [_ptr_array(c) for c in cols]
    rc = lib().orc_moe_bf16w_layer(_p(x_bf16), _p(idx), _p(w), T, H, I, E, k, pa[0], pa[1], pa[2], e_lo, e_hi,
                                   int(with_shared), _p(acc), _p(out))
    assert rc == 0
    return acc, out


def pack_int4_block(wp, s, zp=None):
    wp, s = _c(wp, np.uint8), _c(s, np.uint16)
    zp = None if zp is None else _c(zp, np.uint32)
    N, K = wp.shape[0], wp.shape[1] * 2
    out = np.empty((N // 8) * (K // 512) * 2368, np.uint8)
    lib().orc_pack_int4_block(_p(wp), _p(s), _p(zp), N, K, _p(out))
    return out


def pack_bf16_tile(w):
    w = _c(w, np.uint16)
    out = np.empty(w.size * 2, np.uint8)
    lib().orc_pack_bf16_tile(_p(w), w.shape[0], w.shape[1], _p(out))
    return out


def num_threads():
    return lib().orc_num_threads()


def set_threads(n=None):
    """Use n host threads (default: every core this process may run on), whatever OMP_NUM_THREADS a launcher exported."""
    if n is None:
        n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_num_threads(int(n))
    return num_threads()
