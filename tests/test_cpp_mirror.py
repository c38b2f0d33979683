"""The header-only C++ mirror of the engines' operator interface (dsgx10_b200/csrc/gx_moe.hpp) compiles and links
against the library: a translation unit that calls every wrapper is built with nvcc (no GPU needed to build)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

TU = r"""
#include "gx_moe.hpp"
// every wrapper once, on null buffers: this program is compiled and linked, never run
int use_all(cudaStream_t st) {
  gx::MoeShape s{};
  gx::LayerW L{};
  gx::DecodeCfg cfg{};
  gx::PeerSet ps{};
  gx::LayerStep step{};
  const __nv_bfloat16* x = nullptr;
  __nv_bfloat16* out = nullptr;
  float* f = nullptr;
  int* i = nullptr;
  void* v = nullptr;
  try {
    gx::router_logits(x, f, 1, 128, 8, f, st);
    gx::route(s, f, f, 1, i, f, st);
    size_t n = gx::decode_ws_bytes(s);
    gx::moe_decode(s, L, x, i, f, 1, v, f, f, st, cfg);
    gx::moe_decode(s, L, x, i, f, 1, v, f, f, st);
    gx::finalize(f, f, 1, 128, out, st);
    gx::finalize(f, f, 1, 128, out, st, 1);
    n += gx::prefill_weights_bytes(s) + gx::prefill_ws_bytes(s, 16);
    gx::prefill_prepare(s, L, v, st);
    gx::moe_prefill(s, L, v, x, i, f, 16, v, f, f, st, out, true);
    gx::finalize_peers(ps, 1, 128, out, i, st);
    gx::layer_decode(s, L, x, 1, step, st);
    GX_EXTRA_CALLS
    return (int)n;
  } catch (const gx::Error& e) {
    return e.status;
  }
}
int main() { return 0; }
"""


def test_cpp_mirror_compiles_and_links(tmp_path):
    if shutil.which("nvcc") is None:
        pytest.skip("no nvcc on this machine")
    lib = os.path.join(ROOT, "dsgx10_b200", "libdsgx_moe.so")
    if not os.path.exists(lib):
        pytest.skip("libdsgx_moe.so is not built")
    hdr = open(os.path.join(ROOT, "dsgx10_b200", "csrc", "gx_moe.hpp")).read()
    extra = ""
    if "inline void sort_pack(" in hdr:
        extra += "gx::sort_pack(i, 16, 2, 8, i, i, i, i, i, i, v, st);\n"
    if "inline void moe_prefill_phases(" in hdr:
        extra += "gx::moe_prefill_phases(s, L, v, x, i, f, 16, v, f, f, st, gx::kPrefillAll, out);\n"
    if "inline int decode_up_variants(" in hdr:
        extra += "n += gx::decode_up_variants() + (gx::decode_up_name(0) != nullptr);\n"
    src = tmp_path / "use_gx.cu"
    src.write_text(TU.replace("GX_EXTRA_CALLS", extra))
    exe = tmp_path / "use_gx"
    r = subprocess.run(["nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I", os.path.join(ROOT, "include"),
                        "-I", os.path.join(ROOT, "dsgx10_b200", "csrc"), "-o", str(exe), str(src), lib, "-lcudart"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
