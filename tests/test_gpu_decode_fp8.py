"""GPU parity of the FP8 decode expert step against the CPU oracle, through the C ABI.

Tolerance (stated by the task): outputs within 2e-3 of the row's largest magnitude; router ids and weights bit-exact."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TOL = 2e-3


def _run(orc, H, I, E, topk, M, seed, ng=1, tg=1, scale=1.0, shared=True, e_lo=0, e_hi=None, ysum=False, score=0,
         limit=0.0, x_scale=1.0):
    from dsgx10_b200 import moe, synth
    from tests.util import assert_rows_close, bf16_ulp_hist, oracle_fp8_layer, oracle_route
    shp = moe.shape(H, I, E, topk, n_group=ng, topk_group=tg, route_scale=scale, e_lo=e_lo, e_hi=e_hi, score_fn=score,
                    swiglu_limit=limit)
    layer = synth.Fp8Layer(H, I, E, seed, device="cuda", shared=shared)
    x = (synth.activations(M, H, seed + 1000, device="cpu").float() * x_scale).to(torch.bfloat16).cuda()
    wr = synth.router_weights(E, H, seed + 2000, device="cpu").cuda()
    logits = moe.router_logits(x, wr)
    idx, w = moe.route(shp, logits, None)
    ws = moe.decode_ws(shp)
    outs = []
    for _ in range(2):  # twice on the same workspace: its counters must reset themselves
        yr, ys = moe.moe_decode(shp, layer.layer_w(), x, idx, w, ws, ysum=ysum)
        out = moe.finalize(yr, None if (ysum or not shared) else ys)
        torch.cuda.synchronize()
        assert moe.ws_status(ws) == 0
        outs.append((yr.cpu().numpy(), ys.cpu().numpy(), synth.bf16_bits(out)))
    assert (outs[0][0] == outs[1][0]).all() and (outs[0][2] == outs[1][2]).all()  # deterministic
    xb = synth.bf16_bits(x)
    _, oi, ow = oracle_route(orc, xb, wr.cpu().numpy(), None, shp)
    assert (idx.cpu().numpy() == oi).all() and (w.cpu().numpy().view(np.uint32) == ow.view(np.uint32)).all()
    acc_r, _, pm_r = oracle_fp8_layer(orc, layer, xb, oi, ow, e_lo, e_hi, with_shared=False, pickmax=True, swiglu_limit=limit)
    acc_all, out_all, pm_all = oracle_fp8_layer(orc, layer, xb, oi, ow, e_lo, e_hi, with_shared=shared, pickmax=True,
                                               swiglu_limit=limit)
    yr, ys, outb = outs[0]
    if ysum or not shared:
        assert_rows_close(yr, acc_all, TOL, what="yr", pickmax=pm_all)
    else:
        assert_rows_close(yr, acc_r, TOL, what="yr", pickmax=pm_r)
        assert_rows_close(yr + ys, acc_all, TOL, what="yr + ys", pickmax=pm_all)
    assert_rows_close(orc.bf16_to_f32(outb), orc.bf16_to_f32(out_all), TOL, what="out", pickmax=pm_all, rounded=True)
    print("bf16 ulp histogram of the rounded output:", bf16_ulp_hist(orc, outb, out_all))


@pytest.mark.parametrize("M", [1, 2, 3, 8])
def test_small_layer(orc, M):
    _run(orc, 512, 256, 16, 4, M, seed=10 + M)


def test_config1_single_row(orc):
    """hidden 2048, 64 experts of 1024, top-6 sigmoid, normalised, + shared expert, one row."""
    _run(orc, 2048, 1024, 64, 6, 1, seed=20261101)


@pytest.mark.parametrize("M", [1, 4, 8])
def test_config2_shapes_fewer_experts(orc, M):
    """hidden 4096, intermediate 2048, top-8 of 256 with group-limited selection (8 groups, 4 kept); the layer holds all
    256 experts' descriptors but the test generates a 32-expert layer to stay small: E = 32, groups of 4."""
    _run(orc, 4096, 2048, 32, 8, M, seed=20261102 + M, ng=8, tg=4)


@pytest.mark.parametrize("M", [1, 8])
def test_config2_full_expert_count(orc, M):
    """The headline configuration as it is benchmarked: all 256 experts (8 groups of 32, 4 kept, top-8), one row and eight."""
    _run(orc, 4096, 2048, 256, 8, M, seed=20261110 + M, ng=8, tg=4)


@pytest.mark.parametrize("M", [1, 5])
def test_sqrtsoftplus_score_and_swiglu_clamp(orc, M):
    """ds41f's router score and its SwiGLU clamp at 10 (ref/config.json), on activations large enough for the clamp to
    bite; both decode paths (the separate kernels at one row, the one-kernel step at five)."""
    from dsgx10_b200 import moe, synth
    _run(orc, 1024, 512, 32, 6, M, seed=500 + M, scale=1.5, score=2, limit=10.0, x_scale=48.0)
    # the layer step (router inside) on the same inputs: the same bits as the separate calls
    H, I, E, topk = 1024, 512, 32, 6
    shp = moe.shape(H, I, E, topk, route_scale=1.5, score_fn=2, swiglu_limit=10.0)
    layer = synth.Fp8Layer(H, I, E, 500 + M, device="cuda")
    x = (synth.activations(M, H, 500 + M + 1000).float() * 48.0).to(torch.bfloat16).cuda()
    wr = synth.router_weights(E, H, 500 + M + 2000).cuda()
    idx, w = moe.route(shp, moe.router_logits(x, wr), None)
    yr, ys = moe.moe_decode(shp, layer.layer_w(), x, idx, w, moe.decode_ws(shp))
    step = moe.LayerStep(shp, wr)
    out = step.run(layer.layer_w(), x)
    torch.cuda.synchronize()
    assert torch.equal(step.idx[:M], idx) and torch.equal(step.yr[:M], yr) and torch.equal(step.ys[:M], ys)
    assert torch.equal(out, moe.finalize(yr, ys))


def test_shared_expert_in_parts(orc):
    """Two ranks of an expert-parallel step on one GPU, one after the other: each takes half of the routed experts and
    half of the shared expert's intermediate channels; its ys is an unrounded partial sum.  The parts added and the
    shared expert's sum rounded once give the whole step's outputs within the parity rule; a part's outputs do not
    depend on the row count."""
    from dsgx10_b200 import moe, synth
    from tests.util import assert_rows_close, oracle_fp8_layer, oracle_route
    H, I, E, topk, M = 1024, 1024, 16, 4, 6
    layer = synth.Fp8Layer(H, I, E, 610, device="cuda")
    x = synth.activations(M, H, 611).cuda()
    wr = synth.router_weights(E, H, 612).cuda()
    whole = moe.shape(H, I, E, topk)
    idx, w = moe.route(whole, moe.router_logits(x, wr), None)
    parts = []
    for r in range(2):
        shp = moe.shape(H, I, E, topk, e_lo=r * E // 2, e_hi=(r + 1) * E // 2, sh_lo=r * I // 2, sh_hi=(r + 1) * I // 2)
        yr, ys = moe.moe_decode(shp, layer.layer_w(), x, idx, w, moe.decode_ws(shp))
        parts.append((yr.clone(), ys.clone()))
        y1, s1 = moe.moe_decode(shp, layer.layer_w(), x[2:3].contiguous(), idx[2:3].contiguous(), w[2:3].contiguous(),
                                moe.decode_ws(shp))
        torch.cuda.synchronize()
        assert torch.equal(y1[0], yr[2]) and torch.equal(s1[0], ys[2])
    yr = parts[0][0] + parts[1][0]
    ys = (parts[0][1] + parts[1][1]).to(torch.bfloat16).float()   # the shared expert's output: rounded once, as a whole
    xb = synth.bf16_bits(x)
    acc_r, _, pm_r = oracle_fp8_layer(orc, layer, xb, idx.cpu().numpy(), w.cpu().numpy(), with_shared=False, pickmax=True)
    acc_all, _, pm_all = oracle_fp8_layer(orc, layer, xb, idx.cpu().numpy(), w.cpu().numpy(), pickmax=True)
    assert_rows_close(yr.cpu().numpy(), acc_r, TOL, what="yr of two parts", pickmax=pm_r)
    assert_rows_close((yr + ys).cpu().numpy(), acc_all, TOL, what="yr + ys of two parts", pickmax=pm_all)
    # refusals: a part must be whole pieces of 512 channels
    from dsgx10_b200 import _lib
    with pytest.raises(_lib.DsgxError) as e:
        moe.decode_ws(moe.shape(H, I, E, topk, sh_lo=128, sh_hi=512))
    assert e.value.status == _lib.ERR_SHAPE


def test_no_shared_and_ysum(orc):
    _run(orc, 512, 512, 8, 2, 5, seed=31, shared=False)
    _run(orc, 512, 512, 8, 2, 5, seed=32, ysum=True)


def test_expert_parallel_partial_sums(orc):
    """Two ranks' partial sums (experts [0, E/2) and [E/2, E)) each match the oracle's share."""
    _run(orc, 512, 256, 16, 4, 6, seed=41, e_lo=0, e_hi=8)
    _run(orc, 512, 256, 16, 4, 6, seed=41, e_lo=8, e_hi=16, shared=False)


def test_batch_invariance(orc):
    """A row's bits do not depend on the other rows of the step (altar1 engine/experts/experts.h:15-16)."""
    from dsgx10_b200 import moe, synth
    H, I, E, topk = 1024, 512, 16, 4
    shp = moe.shape(H, I, E, topk)
    layer = synth.Fp8Layer(H, I, E, 55, device="cuda")
    x = synth.activations(8, H, 56).cuda()
    wr = synth.router_weights(E, H, 57).cuda()
    idx, w = moe.route(shp, moe.router_logits(x, wr), None)
    ws = moe.decode_ws(shp)
    yr8, ys8 = moe.moe_decode(shp, layer.layer_w(), x, idx, w, ws)
    yr8, ys8 = yr8.clone(), ys8.clone()
    for r in range(8):
        yr1, ys1 = moe.moe_decode(shp, layer.layer_w(), x[r:r + 1].contiguous(), idx[r:r + 1].contiguous(),
                                  w[r:r + 1].contiguous(), ws)
        torch.cuda.synchronize()
        assert torch.equal(yr1[0], yr8[r]) and torch.equal(ys1[0], ys8[r])


def test_refusals():
    """Bad arguments come back as status codes (the reference aborts: altar1 engine/experts/decode.cu:708-730)."""
    import ctypes as C
    from dsgx10_b200 import _lib, moe, synth
    shp = moe.shape(512, 256, 16, 4)
    layer = synth.Fp8Layer(512, 256, 16, 1, device="cuda")
    x = synth.activations(17, 512, 2).cuda()
    idx = torch.zeros(17, 4, dtype=torch.int32, device="cuda")
    w = torch.zeros(17, 4, device="cuda")
    ws = moe.decode_ws(shp)
    with pytest.raises(_lib.DsgxError) as e:
        moe.moe_decode(shp, layer.layer_w(), x, idx, w, ws)  # 17 rows: more than a decode call takes
    assert e.value.status == _lib.ERR_ARG
    for fmt in (_lib.FMT_NVFP4, _lib.FMT_RETIRED, 7):
        bad = moe.shape(512, 256, 16, 4, fmt=fmt)
        assert _lib.lib().dsgx_decode_ws_bytes(C.byref(bad)) == 0
        with pytest.raises(_lib.DsgxError) as e:
            moe.moe_decode(bad, layer.layer_w(), x[:1].contiguous(), idx[:1].contiguous(), w[:1].contiguous(), ws)
        assert e.value.status == _lib.ERR_FORMAT
    with pytest.raises(_lib.DsgxError) as e:
        moe.decode_ws(moe.shape(500, 256, 16, 4))
    assert e.value.status == _lib.ERR_SHAPE


@pytest.mark.parametrize("H,I,E,topk,M,ng,tg", [(2048, 1024, 64, 6, 1, 1, 1), (4096, 2048, 32, 8, 7, 8, 4), (1280, 512, 16, 4, 8, 1, 1)])
def test_layer_step_equals_separate_calls(orc, H, I, E, topk, M, ng, tg):
    """The fused layer step (logit slices + route + slot table + experts + rounding) gives the bits of the separate
    calls: same logits, ids, weights, partial sums and rounded output; and the host-buffer entry point the same again."""
    from dsgx10_b200 import moe, synth
    if H % 256:
        pytest.skip("FP8 kernels need H % 256 == 0")
    shp = moe.shape(H, I, E, topk, n_group=ng, topk_group=tg)
    layer = synth.Fp8Layer(H, I, E, 77, device="cuda")
    x = synth.activations(M, H, 78).cuda()
    wr = synth.router_weights(E, H, 79).cuda()
    bias = (torch.randn(E, generator=torch.Generator().manual_seed(5)) * 0.01).float().cuda()
    logits = moe.router_logits(x, wr)
    idx, w = moe.route(shp, logits, bias)
    ws = moe.decode_ws(shp)
    yr, ys = moe.moe_decode(shp, layer.layer_w(), x, idx, w, ws)
    out = moe.finalize(yr, ys)
    step = moe.LayerStep(shp, wr, bias)
    out2 = step.run(layer.layer_w(), x)
    torch.cuda.synchronize()
    assert moe.ws_status(step.ws) == 0
    assert torch.equal(step.logits[:M], logits)
    assert torch.equal(step.idx[:M], idx) and torch.equal(step.w[:M], w)
    assert torch.equal(step.yr[:M], yr) and torch.equal(step.ys[:M], ys)
    assert torch.equal(out2, out)
    xh = x.cpu().pin_memory()
    oh = torch.empty(M, H, dtype=torch.bfloat16).pin_memory()
    step.run_host(layer.layer_w(), xh, oh)
    torch.cuda.synchronize()
    assert torch.equal(oh, out.cpu())
    # pageable host memory goes through the copy engine instead of being used in place: the same bits
    xp, op = x.cpu().clone(), torch.zeros(M, H, dtype=torch.bfloat16)
    step.run_host(layer.layer_w(), xp, op)
    torch.cuda.synchronize()
    assert torch.equal(op, out.cpu())
    # the gate/up kernel alone (bench hook 5) over what a hook-1 call left in the workspace repeats its h
    moe.moe_decode(shp, layer.layer_w(), x, idx, w, ws, parts=1)
    torch.cuda.synchronize()
    snap = ws.clone()
    moe.moe_decode(shp, layer.layer_w(), x, idx, w, ws, parts=5)
    torch.cuda.synchronize()
    assert torch.equal(ws, snap) and moe.ws_status(ws) == 0


def test_fused_routing_on_callers_logits():
    """dsgx_decode_cfg.logits (the reference's DecodeCfg::logits, altar1 engine/experts/experts.h:123-127): the step routes
    the rows itself and gives the bits of route + moe_decode; idx and w are not read."""
    from dsgx10_b200 import moe, synth
    H, I, E, topk, M = 1024, 512, 32, 6, 5
    shp = moe.shape(H, I, E, topk, n_group=4, topk_group=2, route_scale=1.5)
    layer = synth.Fp8Layer(H, I, E, 95, device="cuda")
    x = synth.activations(M, H, 96).cuda()
    wr = synth.router_weights(E, H, 97).cuda()
    bias = (torch.randn(E, generator=torch.Generator().manual_seed(6)) * 0.01).float().cuda()
    logits = moe.router_logits(x, wr)
    idx, w = moe.route(shp, logits, bias)
    yr, ys = moe.moe_decode(shp, layer.layer_w(), x, idx, w, moe.decode_ws(shp))
    ws = moe.decode_ws(shp)
    for _ in range(2):
        yr2, ys2 = moe.moe_decode(shp, layer.layer_w(), x, None, None, ws, logits=logits, bias=bias)
        torch.cuda.synchronize()
        assert moe.ws_status(ws) == 0
        assert torch.equal(yr2, yr) and torch.equal(ys2, ys)


def test_kernel_variants_same_bits(orc):
    """Every up / down kernel variant (warps, chunking, ring depth) gives the same bits (cf. altar1
    engine/experts/tests/test_experts.cu:557-575)."""
    from dsgx10_b200 import moe, synth
    H, I, E, topk, M = 2048, 1024, 16, 4, 5
    shp = moe.shape(H, I, E, topk)
    layer = synth.Fp8Layer(H, I, E, 91, device="cuda")
    x = synth.activations(M, H, 92).cuda()
    wr = synth.router_weights(E, H, 93).cuda()
    idx, w = moe.route(shp, moe.router_logits(x, wr), None)
    ws = moe.decode_ws(shp)
    base = None
    ups, downs = moe.decode_variants()
    assert len(ups) == 7 and len(downs) == 5 and all(ups) and all(downs)
    for up in range(len(ups)):
        for down in range(len(downs)):
            if up and down:
                continue
            yr, ys = moe.moe_decode(shp, layer.layer_w(), x, idx, w, ws, up=up, down=down)
            torch.cuda.synchronize()
            if base is None:
                base = (yr.clone(), ys.clone())
            assert torch.equal(yr, base[0]) and torch.equal(ys, base[1]), (up, down)
    assert moe.ws_status(ws) == 0


@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 8])
def test_one_kernel_step_equals_separate_kernels(orc, M):
    """The persistent one-kernel layer step and the four-kernel step give the same bits, run after run on one workspace
    (its counters reset themselves), for every row count (activation blocks of 1, 2, 4, 8 rows)."""
    from dsgx10_b200 import moe, synth
    H, I, E, topk = 1024, 512, 32, 6
    shp = moe.shape(H, I, E, topk, n_group=4, topk_group=2)
    layer = synth.Fp8Layer(H, I, E, 400 + M, device="cuda")
    wr = synth.router_weights(E, H, 401).cuda()
    fused = moe.LayerStep(shp, wr, fused=True)
    sep = moe.LayerStep(shp, wr, fused=False)
    for it in range(3):
        x = synth.activations(M, H, 410 + it).cuda()
        a = fused.run(layer.layer_w(), x).clone()
        b = sep.run(layer.layer_w(), x).clone()
        torch.cuda.synchronize()
        assert moe.ws_status(fused.ws) == 0 and moe.ws_status(sep.ws) == 0
        assert torch.equal(fused.logits[:M], sep.logits[:M])
        assert torch.equal(fused.idx[:M], sep.idx[:M]) and torch.equal(fused.w[:M], sep.w[:M])
        assert torch.equal(fused.yr[:M], sep.yr[:M]) and torch.equal(fused.ys[:M], sep.ys[:M])
        assert torch.equal(a, b)


def test_one_kernel_step_reports_a_wait_that_runs_out():
    """The one-kernel step's CTAs wait for one another through counters; when what they wait for never comes (here: the
    table is never announced, a test switch of dsgx_layer_step.flags), the waits run out after about a second, the
    status word says so, and the workspace's counters are reset: with the status word cleared the next step is right."""
    import ctypes as C
    from dsgx10_b200 import _lib, moe, synth
    H, I, E, topk, M = 1024, 512, 32, 6, 4
    shp = moe.shape(H, I, E, topk)
    layer = synth.Fp8Layer(H, I, E, 700, device="cuda")
    wr = synth.router_weights(E, H, 701).cuda()
    x = synth.activations(M, H, 702).cuda()
    good = moe.LayerStep(shp, wr, fused=True)
    want = good.run(layer.layer_w(), x).clone()
    step = moe.LayerStep(shp, wr, fused=True)
    c = _lib.LayerStep.from_buffer_copy(step.c)
    c.flags = 4 | 16
    rc = _lib.lib().dsgx_moe_layer_decode(C.byref(shp), C.byref(layer.layer_w()), C.c_void_p(x.data_ptr()), M, C.byref(c), 1,
                                          C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0                                   # the launch itself is fine
    torch.cuda.synchronize()                         # (about a second: the bounded waits)
    assert moe.ws_status(step.ws) == _lib.ERR_DEVICE_WAIT
    step.ws[:4].zero_()                              # the caller clears the status word ...
    got = step.run(layer.layer_w(), x)               # ... and the workspace is ready: its counters were reset
    torch.cuda.synchronize()
    assert moe.ws_status(step.ws) == 0
    assert torch.equal(got, want)


@pytest.mark.parametrize("M", [9, 13, 16])
def test_rows_9_to_16(orc, M):
    """More than eight rows: two launch sequences of at most eight on one workspace; parity as any step, and the layer
    step's rows (with the fused norm) equal the rows of two smaller steps bit for bit."""
    _run(orc, 512, 256, 16, 4, M, seed=300 + M)
    from dsgx10_b200 import moe, synth
    H, I, E, topk = 1024, 512, 16, 4
    shp = moe.shape(H, I, E, topk)
    layer = synth.Fp8Layer(H, I, E, 310, device="cuda")
    wr = synth.router_weights(E, H, 311, device="cpu").cuda()
    x = synth.activations(M, H, 312, device="cpu").cuda()
    nw = (1.0 + 0.1 * torch.randn(H, generator=torch.Generator().manual_seed(313))).to(torch.bfloat16).cuda()
    for kw in ({}, {"norm_w": nw}):
        big, small = moe.LayerStep(shp, wr, **kw), moe.LayerStep(shp, wr, **kw)
        out = big.run(layer.layer_w(), x).clone()
        a = small.run(layer.layer_w(), x[:8]).clone()
        b = small.run(layer.layer_w(), x[8:]).clone()
        torch.cuda.synchronize()
        assert moe.ws_status(big.ws) == 0
        assert torch.equal(out, torch.cat([a, b]))
        assert torch.equal(big.idx[8:M], small.idx[:M - 8])
