"""The C-ABI library loads and exports every symbol include/dsgx_moe.h declares (no compute without a GPU)."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            src = open(os.path.join(inc, f)).read()
            src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
            names |= set(re.findall(r"\b(dsgx_[a-z0-9_]+)\s*\(", src))
    return names


def test_library_exports_every_declared_symbol():
    from dsgx10_b200 import _lib, build
    build.build()
    L = _lib.lib()
    declared = _declared()
    assert declared, "no declarations found"
    assert declared == set(_lib.SYMBOLS), (declared ^ set(_lib.SYMBOLS))
    for name in declared:
        assert hasattr(L, name), name


def test_status_names_and_host_side_refusals():
    import ctypes as C
    from dsgx10_b200 import _lib, moe
    L = _lib.lib()
    assert L.dsgx_status_name(0) == b"ok"
    for fmt in (_lib.FMT_NVFP4, _lib.FMT_RETIRED, 9):
        assert L.dsgx_decode_ws_bytes(C.byref(moe.shape(2048, 1024, 64, 6, fmt=fmt))) == 0
    assert L.dsgx_decode_ws_bytes(C.byref(moe.shape(2048, 1024, 64, 6))) > 0
    assert L.dsgx_decode_ws_bytes(C.byref(moe.shape(2048, 1000, 64, 6))) == 0      # I not a multiple of 128
    assert L.dsgx_decode_ws_bytes(C.byref(moe.shape(2048, 1024, 64, 9))) == 0      # topk > 8
    assert L.dsgx_decode_ws_bytes(C.byref(moe.shape(4096, 2048, 256, 8, n_group=8, topk_group=9))) == 0
    assert L.dsgx_sort_ws_bytes(16384, 6, 64) > 0
