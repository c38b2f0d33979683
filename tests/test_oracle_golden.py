"""Pins the CPU oracle against outputs of the reference's own Python CPU modules (tests/golden/*.npz, made by
tests/golden/make_golden.py from ds41f ref/inference/model.py + ref/torchref/kernel.py and altar1 ref/glmref.py) and, for
the group-limited selection that neither engine runs, against the function altar1 docs/model.md names as its definition."""
import os
import zlib

import numpy as np
import pytest

from tests.util import rowmax_err

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _crc(*arrays):
    c = 0
    for a in arrays:
        c = zlib.crc32(np.ascontiguousarray(a).tobytes(), c)
    return np.uint32(c)


@pytest.mark.parametrize("name", ["fp8_sigmoid_small", "fp8_sigmoid_top6", "fp8_softmax", "fp8_sqrtsoftplus_clamp",
                                  "mx4_sqrtsoftplus_clamp"])
def test_fp8_layer_matches_reference_model_py(orc, name):
    from dsgx10_b200 import synth
    g = np.load(os.path.join(GOLD, name + ".npz"))
    H, I, E, topk, T, score, seed = (int(v) for v in g["meta"])
    limit = float(g["swiglu_limit"])   # (the last fixture: ds41f's sqrt(softplus) score and its SwiGLU clamp at 10)
    mx4 = name.startswith("mx4")   # (ds41f's layer: MXFP4 routed experts, FP8 shared expert)
    layer = (synth.Mx4Layer if mx4 else synth.Fp8Layer)(H, I, E, seed, device="cpu")
    experts = {e: layer.canonical(e) for e in range(E + 1)}
    if not all(_crc(*experts[e]) == g["weights_crc"][e] for e in range(E + 1)):
        pytest.skip("this torch build's CPU generator gives other weights than the fixture's (checksum)")
    wr = synth.router_weights(E, H, seed + 2000).numpy()
    x = g["x"]
    # logits: same sums in another order
    logits = orc.router_logits(x, wr)
    assert np.abs(logits - g["logits"]).max() <= 2e-5 * max(1.0, float(np.abs(g["logits"]).max()))
    # the selection on the reference's logits: same experts in the same order, same weights (its sum order may differ)
    idx, w = orc.route(g["logits"], None, topk, score, norm=True, route_scale=float(g["route_scale"]))
    assert (idx == g["idx"]).all()
    assert np.abs(w - g["w"]).max() <= 4e-7 * float(g["route_scale"])
    # and on the oracle's own logits too (no near-ties in these fixtures)
    idx2, _ = orc.route(logits, None, topk, score, norm=True, route_scale=float(g["route_scale"]))
    assert (idx2 == g["idx"]).all()
    # one routed expert and the shared expert on row 0 (bf16 outputs): a rounding flip at most
    e0 = int(g["e0"])
    row = orc.mx4_expert_row if mx4 else orc.fp8_expert_row
    y0, _ = row(x[0], *experts[e0], wroute=float(g["w"][0, 0]), swiglu_limit=limit)
    ysh, _ = orc.fp8_expert_row(x[0], *experts[E], swiglu_limit=limit)
    if limit:  # the clamp is at work in this fixture: without it the outputs are far off
        y_free, _ = orc.fp8_expert_row(x[0], *experts[E])
        assert rowmax_err(y_free, orc.bf16_to_f32(g["ysh"]).reshape(-1)) > 0.05
    for mine, theirs in ((y0, g["y0"]), (ysh, g["ysh"])):
        theirs = orc.bf16_to_f32(theirs).reshape(-1)
        assert rowmax_err(mine, theirs) <= 2e-3
        assert (orc.f32_to_bf16(mine) == orc.f32_to_bf16(theirs)).mean() > 0.98
    # the whole layer with the reference's routing
    shared = experts.pop(E)
    acc, out = orc.moe_fp8_layer(x, g["idx"], g["w"], experts, shared, swiglu_limit=limit, mx4=mx4)
    want = orc.bf16_to_f32(g["out"])
    assert rowmax_err(orc.bf16_to_f32(out), want) <= 2e-3 + 2 ** -8
    assert (out == g["out"]).mean() > 0.97


def test_int4_layer_matches_reference_glmref(orc):
    from dsgx10_b200 import synth
    import torch
    g = np.load(os.path.join(GOLD, "int4_sigmoid.npz"))
    H, I, E, topk, T, _, seed = (int(v) for v in g["meta"])
    shapes = ((I, H), (I, H), (H, I))
    raw = {e: [synth.int4_tensors(n, k, seed * 1000 + e * 3 + m) for m, (n, k) in enumerate(shapes)] for e in range(E)}
    sh = [synth.bf16_bits((torch.randn(n, k, generator=torch.Generator().manual_seed(seed + 9 + i)) * 0.02).to(torch.bfloat16))
          for i, (n, k) in enumerate(shapes)]
    crcs = [_crc(*[a for t in raw[e] for a in t]) for e in range(E)] + [_crc(*sh)]
    if not (np.array(crcs, np.uint32) == g["weights_crc"]).all():
        pytest.skip("this numpy / torch build's generators give other weights than the fixture's (checksum)")
    deq = {e: tuple(orc.int4_dequant(wp, s, None) for wp, s in raw[e]) for e in range(E)}
    assert (deq[0][0][:16] == g["deq0"]).all()          # the dequant contract, bit for bit
    wr = synth.bf16_bits(synth.router_weights(E, H, seed + 2000).to(torch.bfloat16))
    logits = orc.router_logits(g["x"], orc.bf16_to_f32(wr))
    idx, w = orc.route(logits, g["bias"], topk, orc.SCORE_SIGMOID, norm=True, route_scale=float(g["route_scale"]))
    safe = g["margin"] > 1e-5
    assert (idx[safe] == g["idx"][safe]).all()
    assert np.abs(w[safe] - g["w"][safe]).max() <= 1e-6
    acc, _ = orc.moe_bf16w_layer(g["x"], g["idx"], g["w"], deq, tuple(sh))
    assert rowmax_err(acc, g["out"]) <= 2e-3


def test_rmsnorm_matches_both_references(orc):
    """ds41f's model.py RMSNorm (one rounding) and altar1's glmref.rms_norm (the normalised value rounded first); the
    references sum the squares in torch's order, so a row's 1/rms may differ in its last bit: bf16 bits equal on all but a
    few elements, never more than one ulp apart.  Also the residual add in front (h = bf16(res + x))."""
    g = np.load(os.path.join(GOLD, "rmsnorm.npz"))

    def close(mine, theirs):
        assert (mine == theirs).mean() > 0.995
        a, b = mine.astype(np.int32), theirs.astype(np.int32)   # same sign (checked by the bound): bit patterns differ by one ulp
        assert np.abs(a - b).max() <= 1

    close(orc.rmsnorm(g["x"], g["w"], 1e-6, 0), g["y_model"])
    close(orc.rmsnorm(g["x"], g["w"], 1e-5, 1), g["y_glm"])
    out, h, normed = orc.add_norm(orc.bf16_to_f32(g["x"]), g["res"], g["w"], 1e-6, 0)
    assert (out == g["x"]).all() and (h == g["h"]).all()
    close(normed, g["y_model_h"])


def test_group_limited_routing_matches_the_named_definition(orc):
    """Config 2's router (8 groups, the best 4 kept; and two smaller shapes).  The fixture holds the outputs of
    transformers' GlmMoeDsa `route_tokens_to_experts` (altar1 docs/model.md:337-347 gives that function as the router's
    definition; the engines themselves run it with one group) on seeded logits: the same experts for every row, as sets
    (that function's top-k is unsorted), and the same weights."""
    g = np.load(os.path.join(GOLD, "group_route.npz"))
    for ci in range(int(g["n_cases"])):
        E, ng, tg, topk, T = (int(v) for v in g[f"meta{ci}"])
        scale = float(g[f"scale{ci}"])
        idx, w = orc.route(g[f"logits{ci}"], g[f"bias{ci}"], topk, orc.SCORE_SIGMOID, n_group=ng, topk_group=tg, norm=True,
                           route_scale=scale)
        order = np.argsort(idx, axis=1)
        idx, w = np.take_along_axis(idx, order, 1), np.take_along_axis(w, order, 1)
        assert float(g[f"margin{ci}"].min()) > 1e-5          # no decision of the fixture is a near-tie
        assert (idx == g[f"idx{ci}"]).all(), ci
        assert np.abs(w - g[f"w{ci}"]).max() <= 4e-7 * scale, ci
