"""B200 (sm_100a) quantised mixture-of-experts FFN operator: a drop-in for the MoE op of dsgx10's engines.

`dsgx10_b200.moe` mirrors the engine's operator interface over the C ABI of `libdsgx_moe.so` (include/dsgx_moe.h);
`dsgx10_b200.synth` makes seeded synthetic layers in the engine's weight layouts; `dsgx10_b200.build` compiles the library.
"""
from . import _lib  # noqa: F401
