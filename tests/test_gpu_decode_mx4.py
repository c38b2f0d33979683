"""GPU parity of the MXFP4 decode expert step (ds41f's routed format: e2m1 values, a ue8m0 scale per 32 along K, FP8
activations and FP8 shared expert) against the CPU oracle, through the C ABI.  Same tolerance rule as the FP8 step."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TOL = 2e-3


def _run(orc, H, I, E, topk, M, seed, shared=True, e_lo=0, e_hi=None, score=0, limit=0.0, x_scale=1.0, ng=1, tg=1):
    from dsgx10_b200 import _lib, moe, synth
    from tests.util import assert_rows_close, oracle_fp8_layer, oracle_route
    shp = moe.shape(H, I, E, topk, fmt=_lib.FMT_MXFP4, n_group=ng, topk_group=tg, e_lo=e_lo, e_hi=e_hi, score_fn=score,
                    swiglu_limit=limit)
    layer = synth.Mx4Layer(H, I, E, seed, device="cuda", shared=shared)
    x = (synth.activations(M, H, seed + 1000, device="cpu").float() * x_scale).to(torch.bfloat16).cuda()
    wr = synth.router_weights(E, H, seed + 2000, device="cpu").cuda()
    idx, w = moe.route(shp, moe.router_logits(x, wr), None)
    ws = moe.decode_ws(shp)
    outs = []
    for _ in range(2):  # twice on the same workspace: its counters must reset themselves
        yr, ys = moe.moe_decode(shp, layer.layer_w(), x, idx, w, ws)
        out = moe.finalize(yr, ys if shared else None)
        torch.cuda.synchronize()
        assert moe.ws_status(ws) == 0
        outs.append((yr.cpu().numpy(), ys.cpu().numpy(), synth.bf16_bits(out)))
    assert (outs[0][0] == outs[1][0]).all() and (outs[0][2] == outs[1][2]).all()  # deterministic
    xb = synth.bf16_bits(x)
    _, oi, ow = oracle_route(orc, xb, wr.cpu().numpy(), None, shp)
    assert (idx.cpu().numpy() == oi).all()
    acc_r, _, pm_r = oracle_fp8_layer(orc, layer, xb, oi, ow, e_lo, e_hi, with_shared=False, pickmax=True, swiglu_limit=limit)
    acc_all, out_all, pm_all = oracle_fp8_layer(orc, layer, xb, oi, ow, e_lo, e_hi, with_shared=shared, pickmax=True,
                                               swiglu_limit=limit)
    yr, ys, outb = outs[0]
    assert_rows_close(yr, acc_r, TOL, what="yr", pickmax=pm_r)
    if shared:
        assert_rows_close(yr + ys, acc_all, TOL, what="yr + ys", pickmax=pm_all)
    assert_rows_close(orc.bf16_to_f32(outb), orc.bf16_to_f32(out_all), TOL, what="out", pickmax=pm_all, rounded=True)
    return layer, shp, x, wr, outs[0]


@pytest.mark.parametrize("M", [1, 2, 3, 8])
def test_small_layer(orc, M):
    _run(orc, 512, 256, 16, 4, M, seed=40 + M)


def test_scale_range(orc):
    """Weights over many octaves, so the ue8m0 bytes of a block's four groups differ widely (the per-group promotion)."""
    from dsgx10_b200 import _lib, moe, synth
    from tests.util import assert_rows_close, oracle_fp8_layer, oracle_route
    H, I, E, topk, M = 512, 256, 8, 2, 4
    layer = synth.Mx4Layer(H, I, E, 61, device="cpu")
    # rescale groups of 32 by powers of two in [-6, 6]: the nibbles stay, the scale bytes move
    g = torch.Generator().manual_seed(7)
    for (e, m), (off, _) in layer._off.items():
        if e == E:
            continue
        N, K = (H, I) if m == 2 else (I, H)
        nb = synth.mx4_mat_bytes(N, K)
        q, sc = synth.untile_mx4(layer.pool[off:off + nb], N, K)
        sc = (sc.to(torch.int32) + torch.randint(-6, 7, sc.shape, generator=g)).clamp(1, 254).to(torch.uint8)
        layer.pool[off:off + nb] = synth.tile_mx4(q, sc)
    layer.to("cuda")
    shp = moe.shape(H, I, E, topk, fmt=_lib.FMT_MXFP4)
    x = synth.activations(M, H, 62, device="cpu").cuda()
    wr = synth.router_weights(E, H, 63, device="cpu").cuda()
    idx, w = moe.route(shp, moe.router_logits(x, wr), None)
    yr, ys = moe.moe_decode(shp, layer.layer_w(), x, idx, w, moe.decode_ws(shp))
    torch.cuda.synchronize()
    xb = synth.bf16_bits(x)
    _, oi, ow = oracle_route(orc, xb, wr.cpu().numpy(), None, shp)
    acc, _, pm = oracle_fp8_layer(orc, layer, xb, oi, ow, with_shared=False, pickmax=True)
    assert_rows_close(yr.cpu().numpy(), acc, TOL, what="yr", pickmax=pm)


def test_ds41f_like_shape(orc):
    """hidden 4096, experts of 2048 intermediate channels, top-6 of 32 by sqrt(softplus), SwiGLU clamp 10, + FP8 shared."""
    _run(orc, 4096, 2048, 32, 6, 2, seed=71, score=2, limit=10.0, x_scale=8.0)


def test_expert_range_and_no_shared(orc):
    _run(orc, 1024, 512, 16, 4, 3, seed=81, e_lo=4, e_hi=12)
    _run(orc, 1024, 512, 16, 4, 2, seed=82, shared=False)


def test_variants_split_and_layer_step(orc):
    """Every kernel variant, a launch that splits K across SMs (few experts) and one that does not, and the layer step with
    the router inside: the same bits."""
    from dsgx10_b200 import _lib, moe, synth
    layer, shp, x, wr, (yr0, ys0, out0) = _run(orc, 2048, 1024, 16, 4, 2, seed=91)
    idx, w = moe.route(shp, moe.router_logits(x, wr), None)
    ws = moe.decode_ws(shp)
    nu, nd = moe.decode_variants()
    for up in range(len(nu)):
        for down in range(len(nd)):
            yr, ys = moe.moe_decode(shp, layer.layer_w(), x, idx, w, ws, up=up, down=down)
            torch.cuda.synchronize()
            assert moe.ws_status(ws) == 0
            assert (yr.cpu().numpy() == yr0).all() and (ys.cpu().numpy() == ys0).all(), (up, down)
    step = moe.LayerStep(shp, wr)
    out = step.run(layer.layer_w(), x)
    torch.cuda.synchronize()
    assert moe.ws_status(step.ws) == 0
    assert (synth.bf16_bits(out) == out0).all()
    # batch invariance: row 0 alone gives row 0's bits
    yr1, ys1 = moe.moe_decode(shp, layer.layer_w(), x[:1], idx[:1], w[:1], ws)
    torch.cuda.synchronize()
    assert (yr1.cpu().numpy()[0] == yr0[0]).all()


def test_refusals():
    from dsgx10_b200 import _lib, moe, synth
    H, I, E, topk = 512, 256, 8, 2
    shp = moe.shape(H, I, E, topk, fmt=_lib.FMT_MXFP4)
    fp8 = synth.Fp8Layer(H, I, E, 5, device="cuda")
    x = synth.activations(1, H, 6, device="cpu").cuda()
    wr = synth.router_weights(E, H, 7, device="cpu").cuda()
    idx, w = moe.route(shp, moe.router_logits(x, wr), None)
    with pytest.raises(_lib.DsgxError):   # the layer's tag must be the shape's
        moe.moe_decode(shp, fp8.layer_w(), x, idx, w, moe.decode_ws(shp))
    L = fp8.layer_w()
    L.fmt = _lib.FMT_MXFP4                # descriptors of another format: refused on the device, recorded in the workspace
    ws = moe.decode_ws(shp)
    moe.moe_decode(shp, L, x, idx, w, ws)
    torch.cuda.synchronize()
    assert moe.ws_status(ws) == _lib.ERR_FORMAT


@pytest.mark.parametrize("T", [7, 300])
def test_prefill_through_the_fp8_copy(orc, T):
    """An MXFP4 layer's prefill pass: dsgx_prefill_prepare turns the routed experts into the grouped GEMM's FP8 operand with
    the weights unchanged (e4m3 values and a power-of-two scale per 128 x 128 block); parity as for an FP8 layer, and the
    one-token rows agree with the decode path within the rule."""
    from dsgx10_b200 import _lib, moe, synth
    from tests.util import assert_rows_close, oracle_fp8_layer
    H, I, E, topk = 512, 256, 8, 2
    shp = moe.shape(H, I, E, topk, fmt=_lib.FMT_MXFP4)
    layer = synth.Mx4Layer(H, I, E, 400 + T, device="cuda")
    x = synth.activations(T, H, 401).cuda()
    wr = synth.router_weights(E, H, 402).cuda()
    idx, w = moe.route(shp, moe.router_logits(x, wr), None)
    pl = moe.PrefillLayer(shp, layer.layer_w(), T)
    yr, ys, out = pl.run(x, idx, w)
    torch.cuda.synchronize()
    assert moe.ws_status(pl.ws) == 0
    xb = synth.bf16_bits(x)
    oi, ow = idx.cpu().numpy(), w.cpu().numpy()
    acc_r, _, pm_r = oracle_fp8_layer(orc, layer, xb, oi, ow, with_shared=False, pickmax=True)
    acc_all, out_all, pm_all = oracle_fp8_layer(orc, layer, xb, oi, ow, with_shared=True, pickmax=True)
    assert_rows_close(yr.cpu().numpy(), acc_r, TOL, what="yr", pickmax=pm_r)
    assert_rows_close(orc.bf16_to_f32(synth.bf16_bits(out)), orc.bf16_to_f32(out_all), TOL, what="out", pickmax=pm_all, rounded=True)
    # the decode path on the first rows: the same contract
    M = min(T, 8)
    yd, ysd = moe.moe_decode(shp, layer.layer_w(), x[:M].contiguous(), idx[:M].contiguous(), w[:M].contiguous(), moe.decode_ws(shp))
    torch.cuda.synchronize()
    assert_rows_close(yd.cpu().numpy(), yr[:M].cpu().numpy(), TOL, what="decode vs prefill", pickmax=pm_r[:M])


def test_prefill_refuses_scales_that_spread_too_widely():
    """A 128 x 128 block whose scale bytes differ by more than 14 has no exact FP8 form: the prepare call says so."""
    from dsgx10_b200 import _lib, moe, synth
    H, I, E, topk = 512, 256, 4, 2
    layer = synth.Mx4Layer(H, I, E, 410, device="cpu")
    off, _ = layer._off[(1, 0)]
    nb = synth.mx4_mat_bytes(I, H)
    q, sc = synth.untile_mx4(layer.pool[off:off + nb], I, H)
    sc[3, 2] = int(sc[3, 3]) - 20            # one group 20 octaves below its neighbours
    layer.pool[off:off + nb] = synth.tile_mx4(q, sc)
    layer.to("cuda")
    shp = moe.shape(H, I, E, topk, fmt=_lib.FMT_MXFP4)
    with pytest.raises(_lib.DsgxError) as e:
        moe.PrefillLayer(shp, layer.layer_w(), 16)
    assert e.value.status == _lib.ERR_UNSUPPORTED
    # a spread of 14 is still exact
    ok = synth.Mx4Layer(H, I, E, 411, device="cpu")
    off, _ = ok._off[(0, 2)]
    nb = synth.mx4_mat_bytes(H, I)
    q, sc = synth.untile_mx4(ok.pool[off:off + nb], H, I)
    blk = sc[:128, :4]
    sc[5, 1] = int(blk.max()) - 14
    ok.pool[off:off + nb] = synth.tile_mx4(q, sc)
    ok.to("cuda")
    moe.PrefillLayer(shp, ok.layer_w(), 16)
