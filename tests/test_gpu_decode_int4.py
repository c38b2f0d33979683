"""GPU parity of the INT4-g32 decode expert step (bf16 activations, bf16 shared expert) against the CPU oracle."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TOL = 2e-3


def _oracle(orc, layer, xb, idx, w, e_lo=0, e_hi=None, with_shared=True):
    picked = sorted(set(int(e) for e in np.asarray(idx).ravel()))
    e_hi = layer.E if e_hi is None else e_hi
    deq = {e: tuple(orc.int4_dequant(wp, s, None) for wp, s in layer.raw[e]) for e in picked if e_lo <= e < e_hi}
    if not deq:
        e = next(iter(layer.raw))
        deq = {e: tuple(orc.int4_dequant(wp, s, None) for wp, s in layer.raw[e])}
    sh = tuple(layer.sh_bits) if (layer.shared and with_shared) else None
    return orc.moe_bf16w_layer(xb, idx, w, deq, sh, e_lo=e_lo, e_hi=e_hi, with_shared=with_shared)


def _run(orc, H, I, E, topk, M, seed, score=1, scale=1.0, shared=True, e_lo=0, e_hi=None, picked_only=False):
    from dsgx10_b200 import _lib, moe, synth
    from tests.util import assert_rows_close, oracle_route, rowmax_err
    shp = moe.shape(H, I, E, topk, fmt=_lib.FMT_INT4, score_fn=score, route_scale=scale, e_lo=e_lo, e_hi=e_hi)
    x = synth.activations(M, H, seed + 1000).cuda()
    wr = synth.router_weights(E, H, seed + 2000).cuda()
    only = None
    if picked_only:  # a full-size layer: generate the experts these rows route to, nothing else (routing needs no expert)
        only = moe.route(shp, moe.router_logits(x, wr), None)[0].flatten().tolist()
    layer = synth.Int4Layer(H, I, E, seed, device="cuda", shared=shared, e_range=(e_lo, E if e_hi is None else e_hi),
                            experts=only)
    step = moe.LayerStep(shp, wr)
    outs = []
    for _ in range(2):
        out = step.run(layer.layer_w(), x)
        torch.cuda.synchronize()
        assert moe.ws_status(step.ws) == 0
        outs.append((step.yr[:M].cpu().numpy().copy(), step.ys[:M].cpu().numpy().copy(), synth.bf16_bits(out).copy()))
    assert (outs[0][0] == outs[1][0]).all() and (outs[0][2] == outs[1][2]).all()
    xb = synth.bf16_bits(x)
    _, oi, ow = oracle_route(orc, xb, wr.cpu().numpy(), None, shp)
    assert (step.idx[:M].cpu().numpy() == oi).all()
    assert (step.w[:M].cpu().numpy().view(np.uint32) == ow.view(np.uint32)).all()
    acc_r, _ = _oracle(orc, layer, xb, oi, ow, e_lo, e_hi, with_shared=False)
    acc_all, out_all = _oracle(orc, layer, xb, oi, ow, e_lo, e_hi, with_shared=shared)
    yr, ys, outb = outs[0]
    assert_rows_close(yr, acc_r, TOL, what="yr")
    if shared:
        assert_rows_close(yr + ys, acc_all, TOL, what="yr + ys")
    assert_rows_close(orc.bf16_to_f32(outb), orc.bf16_to_f32(out_all), TOL, what="out", rounded=True, max_outliers=1e-2)
    # the separate-call path (caller's idx / w) gives the same bits
    ws = moe.decode_ws(shp)
    yr2, ys2 = moe.moe_decode(shp, layer.layer_w(), x, step.idx[:M].contiguous(), step.w[:M].contiguous(), ws)
    torch.cuda.synchronize()
    assert (yr2.cpu().numpy() == yr).all()
    if shared:
        assert (ys2.cpu().numpy() == ys).all()


@pytest.mark.parametrize("M", [1, 2, 3, 4, 8])
def test_small_layer(orc, M):
    _run(orc, 1024, 512, 16, 4, M, seed=100 + M)


@pytest.mark.parametrize("M", [1, 4])
def test_config3_shapes_fewer_experts(orc, M):
    """hidden 6144, intermediate 2048, top-8 softmax, bf16 shared expert; 24 experts instead of 168 to stay small."""
    _run(orc, 6144, 2048, 24, 8, M, seed=20261103 + M)


def test_config3_full_expert_count(orc):
    """hidden 6144, all 168 experts of 2048, top-8 softmax, bf16 shared expert: the third benchmark configuration as it is
    benchmarked, one row."""
    _run(orc, 6144, 2048, 168, 8, 1, seed=20261120, picked_only=True)


def test_sigmoid_scaled_no_shared_and_expert_parallel(orc):
    _run(orc, 1024, 1024, 16, 8, 5, seed=120, score=0, scale=2.5, shared=False)
    _run(orc, 1024, 512, 16, 4, 6, seed=121, e_lo=8, e_hi=16, shared=False)
    _run(orc, 1024, 512, 16, 4, 6, seed=121, e_lo=0, e_hi=8)


def test_interleaved_shared_expert_same_bits(orc):
    """The bf16 shared expert as the reference's engine holds it (SharedW::bgu: gate and up rows interleaved in one
    matrix, altar1 engine/experts/experts.h:72-87) gives the bits of the three-matrix form."""
    import ctypes as C
    from dsgx10_b200 import _lib, moe, synth
    H, I, E, topk, M = 1024, 512, 16, 4, 5
    shp = moe.shape(H, I, E, topk, fmt=_lib.FMT_INT4, score_fn=1)
    layer = synth.Int4Layer(H, I, E, 140, device="cuda")
    x = synth.activations(M, H, 141).cuda()
    wr = synth.router_weights(E, H, 142).cuda()
    step = moe.LayerStep(shp, wr)
    step.run(layer.layer_w(), x)
    yr, ys = step.yr[:M].clone(), step.ys[:M].clone()
    gu = np.empty((2 * I, H), np.uint16)
    gu[0::2], gu[1::2] = layer.sh_bits[0], layer.sh_bits[1]
    bgu = torch.from_numpy(synth.tile_bf16(gu)).cuda()
    lw = layer.layer_w()
    lw.sh.bg, lw.sh.bu, lw.sh.bgu = None, None, bgu.data_ptr()
    step2 = moe.LayerStep(shp, wr)
    step2.run(lw, x)
    torch.cuda.synchronize()
    assert moe.ws_status(step2.ws) == 0
    assert torch.equal(step2.yr[:M], yr) and torch.equal(step2.ys[:M], ys)
    lw.sh.bu = layer.sh_dev[1].data_ptr()          # both forms at once are refused
    with pytest.raises(_lib.DsgxError):
        step2.run(lw, x)


def test_batch_invariance(orc):
    from dsgx10_b200 import _lib, moe, synth
    H, I, E, topk = 1024, 512, 16, 4
    shp = moe.shape(H, I, E, topk, fmt=_lib.FMT_INT4)
    layer = synth.Int4Layer(H, I, E, 131, device="cuda")
    x = synth.activations(8, H, 132).cuda()
    wr = synth.router_weights(E, H, 133).cuda()
    step = moe.LayerStep(shp, wr)
    step.run(layer.layer_w(), x)
    yr8, ys8 = step.yr.clone(), step.ys.clone()
    for r in range(8):
        step.run(layer.layer_w(), x[r:r + 1].contiguous())
        torch.cuda.synchronize()
        assert torch.equal(step.yr[0], yr8[r]) and torch.equal(step.ys[0], ys8[r])


def test_rows_9_to_16(orc):
    """Twelve rows through an INT4 layer: the rows of an eight-row and a four-row step, bit for bit."""
    from dsgx10_b200 import _lib, moe, synth
    H, I, E, topk, M = 1024, 512, 8, 2, 12
    shp = moe.shape(H, I, E, topk, fmt=_lib.FMT_INT4, score_fn=1)
    layer = synth.Int4Layer(H, I, E, 950, device="cuda")
    wr = synth.router_weights(E, H, 951, device="cpu").cuda()
    x = synth.activations(M, H, 952, device="cpu").cuda()
    big, small = moe.LayerStep(shp, wr), moe.LayerStep(shp, wr)
    out = big.run(layer.layer_w(), x).clone()
    a = small.run(layer.layer_w(), x[:8]).clone()
    b = small.run(layer.layer_w(), x[8:]).clone()
    torch.cuda.synchronize()
    assert moe.ws_status(big.ws) == 0 and torch.equal(out, torch.cat([a, b]))


@pytest.mark.parametrize("M", [1, 5, 8])
def test_bf16_routed_experts(orc, M):
    """A BF16 layer (format tag 3: altar-1's unquantised layers): the routed experts stream through the same kernels as the
    bf16 shared expert; parity against the oracle on the bf16 weights, same bits run after run and for a row alone."""
    from dsgx10_b200 import _lib, moe, synth
    from tests.util import assert_rows_close, oracle_route
    H, I, E, topk = 1024, 512, 8, 2
    shp = moe.shape(H, I, E, topk, fmt=_lib.FMT_BF16, score_fn=1)
    layer = synth.Bf16Layer(H, I, E, 970, device="cuda")
    wr = synth.router_weights(E, H, 971).cuda()
    x = synth.activations(M, H, 972 + M).cuda()
    step = moe.LayerStep(shp, wr)
    out = step.run(layer.layer_w(), x).clone()
    torch.cuda.synchronize()
    assert moe.ws_status(step.ws) == 0
    xb = synth.bf16_bits(x)
    _, oi, ow = oracle_route(orc, xb, wr.cpu().numpy(), None, shp)
    assert (step.idx[:M].cpu().numpy() == oi).all()
    experts = {int(e): tuple(layer.bits[int(e)]) for e in np.unique(oi)}
    acc, out_o = orc.moe_bf16w_layer(xb, oi, ow, experts, tuple(layer.sh_bits))
    assert_rows_close(step.yr[:M].cpu().numpy() + step.ys[:M].cpu().numpy(), acc, TOL, what="yr + ys")
    out2 = step.run(layer.layer_w(), x).clone()
    one = moe.LayerStep(shp, wr).run(layer.layer_w(), x[:1]).clone()
    torch.cuda.synchronize()
    assert torch.equal(out, out2) and torch.equal(one[0], out[0])
    # an INT4 layer's descriptors under the BF16 tag are refused on the device
    i4 = synth.Int4Layer(H, I, E, 973, device="cuda")
    L = i4.layer_w()
    L.fmt = _lib.FMT_BF16
    st2 = moe.LayerStep(shp, wr)
    st2.run(L, x)
    torch.cuda.synchronize()
    assert moe.ws_status(st2.ws) == _lib.ERR_FORMAT
