"""GPU parity of the router front and the token sort: bit-exact against the oracle (ids, weight bits, permutation)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _mods():
    from dsgx10_b200 import _lib, moe, synth
    return _lib, moe, synth


CASES = [
    # H, E, topk, n_group, topk_group, score, scale, M
    (2048, 64, 6, 1, 1, 0, 1.0, 1),
    (2048, 64, 6, 1, 1, 0, 1.5, 8),
    (4096, 256, 8, 8, 4, 0, 1.0, 8),
    (4096, 256, 8, 8, 4, 0, 2.5, 5),
    (6144, 168, 8, 1, 1, 1, 1.0, 4),
    (6144, 168, 8, 1, 1, 0, 2.5, 8),
    (256, 8, 2, 1, 1, 0, 1.0, 3),
    (1280, 40, 3, 4, 2, 1, 1.0, 7),
    (1024, 512, 8, 16, 4, 0, 1.0, 2),     # the largest expert count, a CTA a row
    (1024, 512, 8, 8, 3, 1, 1.0, 33),     # the same through the warp-a-row kernel
    (5120, 384, 6, 1, 1, 2, 1.5, 4),      # ds41f's router: sqrt(softplus) scores, top-6 of 384, a CTA a row
    (5120, 384, 6, 1, 1, 2, 1.5, 40),     # the same through the warp-a-row kernel
    (2048, 64, 6, 1, 1, 2, 1.0, 1),
]


@pytest.mark.parametrize("H,E,topk,ng,tg,score,scale,M", CASES)
def test_router_logits_and_route_bit_exact(orc, H, E, topk, ng, tg, score, scale, M):
    _lib, moe, synth = _mods()
    shp = moe.shape(H, 256, E, topk, n_group=ng, topk_group=tg, score_fn=score, route_scale=scale)
    x = synth.activations(M, H, 1000 + H + M).cuda()
    wr = synth.router_weights(E, H, 2000 + E).cuda()
    bias = (torch.randn(E, generator=torch.Generator().manual_seed(5)) * 0.01).float().cuda()
    logits = moe.router_logits(x, wr)
    idx, w = moe.route(shp, logits, bias)
    torch.cuda.synchronize()
    from tests.util import oracle_route
    ol, oi, ow = oracle_route(orc, synth.bf16_bits(x), wr.cpu().numpy(), bias.cpu().numpy(), shp)
    assert (logits.cpu().numpy().view(np.uint32) == ol.view(np.uint32)).all()
    assert (idx.cpu().numpy() == oi).all()
    assert (w.cpu().numpy().view(np.uint32) == ow.view(np.uint32)).all()


@pytest.mark.parametrize("T", [1, 255, 1024, 4099])
def test_router_prefill_widths_bit_exact(orc, T):
    _lib, moe, synth = _mods()
    H, E, topk = 2048, 64, 6
    shp = moe.shape(H, 1024, E, topk)
    x = synth.activations(T, H, 77 + T).cuda()
    wr = synth.router_weights(E, H, 78).cuda()
    logits = moe.router_logits(x, wr)
    idx, w = moe.route(shp, logits, None)
    torch.cuda.synchronize()
    from tests.util import oracle_route
    ol, oi, ow = oracle_route(orc, synth.bf16_bits(x), wr.cpu().numpy(), None, shp)
    assert (logits.cpu().numpy().view(np.uint32) == ol.view(np.uint32)).all()
    assert (idx.cpu().numpy() == oi).all()
    assert (w.cpu().numpy().view(np.uint32) == ow.view(np.uint32)).all()


def test_route_engineered_ties(orc):
    """Many equal logits and a 3-way tie at the last place: ties go to the lower expert id, on the GPU as in the oracle."""
    _lib, moe, synth = _mods()
    E, topk, M = 168, 8, 19
    rng = np.random.default_rng(4)
    l = (rng.integers(0, 8, (M, E)) * 0.5).astype(np.float32)      # heavy ties
    for m in range(M):
        l[m, [(m * 13) % E, (m * 13 + 50) % E, (m * 13 + 101) % E]] = 2.25
    bias = np.full(E, 28.25, np.float32)
    shp = moe.shape(6144, 2048, E, topk, route_scale=2.5)
    idx, w = moe.route(shp, torch.from_numpy(l).cuda(), torch.from_numpy(bias).cuda())
    oi, ow = orc.route(l, bias, topk, route_scale=2.5)
    assert (idx.cpu().numpy() == oi).all()
    assert (w.cpu().numpy().view(np.uint32) == ow.view(np.uint32)).all()


@pytest.mark.parametrize("T,E,topk", [(1, 64, 6), (7, 8, 2), (256, 64, 6), (257, 64, 6), (16384, 64, 6), (5000, 256, 8)])
def test_sort_pack_bit_exact(orc, T, E, topk):
    _lib, moe, synth = _mods()
    rng = np.random.default_rng(T + E)
    # Zipf-like popularity so some experts get thousands of rows and some none
    p = 1.0 / np.arange(1, E + 1) ** 1.1
    p /= p.sum()
    idx = np.stack([rng.choice(E, topk, replace=False, p=p) for _ in range(T)]).astype(np.int32)
    got = moe.sort_pack(torch.from_numpy(idx).cuda(), E)
    torch.cuda.synchronize()
    want = orc.sort_pack(idx, E)
    for k in want:
        assert (got[k].cpu().numpy().reshape(want[k].shape) == want[k]).all(), k


def test_finalize_both_modes():
    """dsgx_finalize: mode 0 rounds the f32 sum once (the CPU references' order); mode 1 is the engine's
    bf16(bf16(R) + bf16(S)) (altar1 engine/experts/decode.cu:591-598).  Bit-exact against the same arithmetic in torch."""
    from dsgx10_b200 import moe
    g = torch.Generator().manual_seed(77)
    R = (torch.randn(5, 1024, generator=g) * 3).cuda()
    S = torch.randn(5, 1024, generator=g).cuda()
    out0 = moe.finalize(R, S, mode=0)
    out1 = moe.finalize(R, S, mode=1)
    out_r = moe.finalize(R, None, mode=0)
    torch.cuda.synchronize()
    assert torch.equal(out0, (R + S).to(torch.bfloat16))
    assert torch.equal(out1, (R.to(torch.bfloat16).float() + S.to(torch.bfloat16).float()).to(torch.bfloat16))
    assert torch.equal(out_r, R.to(torch.bfloat16))
    assert not torch.equal(out0, out1)   # (the two orders do differ on some elements of this input)


def test_group_limited_routing_against_the_golden_fixture():
    """The CUDA router on the fixture's logits (tests/golden/group_route.npz: transformers' GlmMoeDsa routing function, the
    definition altar1 docs/model.md names): the same experts as sets and the same weights, without the oracle in between."""
    import os
    _lib, moe, synth = _mods()
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "group_route.npz"))
    for ci in range(int(g["n_cases"])):
        E, ng, tg, topk, T = (int(v) for v in g[f"meta{ci}"])
        scale = float(g[f"scale{ci}"])
        shp = moe.shape(1024, 256, E, topk, n_group=ng, topk_group=tg, score_fn=0, route_scale=scale)
        idx, w = moe.route(shp, torch.from_numpy(g[f"logits{ci}"]).cuda(), torch.from_numpy(g[f"bias{ci}"]).cuda())
        torch.cuda.synchronize()
        idx, w = idx.cpu().numpy(), w.cpu().numpy()
        order = np.argsort(idx, axis=1)
        idx, w = np.take_along_axis(idx, order, 1), np.take_along_axis(w, order, 1)
        assert (idx == g[f"idx{ci}"]).all(), ci
        assert np.abs(w - g[f"w{ci}"]).max() <= 4e-7 * scale, ci
