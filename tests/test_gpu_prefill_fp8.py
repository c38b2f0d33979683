"""GPU parity of the FP8 prefill path (token sort + tcgen05 grouped GEMMs + combine) against the CPU oracle and the
decode path, through the C ABI."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TOL = 2e-3


def _setup(H, I, E, topk, T, seed, ng=1, tg=1, shared=True, e_lo=0, e_hi=None, zipf=False):
    from dsgx10_b200 import moe, synth
    shp = moe.shape(H, I, E, topk, n_group=ng, topk_group=tg, e_lo=e_lo, e_hi=e_hi)
    layer = synth.Fp8Layer(H, I, E, seed, device="cuda", shared=shared)
    x = synth.activations(T, H, seed + 1000).cuda()
    wr = synth.router_weights(E, H, seed + 2000).cuda()
    bias = None
    if zipf:  # a selection bias that makes expert popularity very uneven (empty and huge segments)
        p = 1.0 / np.arange(1, E + 1) ** 1.1
        bias = torch.from_numpy((0.25 * np.log(p / p.max())).astype(np.float32)).cuda()
    idx, w = moe.route(shp, moe.router_logits(x, wr), bias)
    return shp, layer, x, wr, bias, idx, w


def _check(orc, shp, layer, x, idx, w, yr, ys, out, shared=True, e_lo=0, e_hi=None, rows=None):
    from dsgx10_b200 import synth
    from tests.util import assert_rows_close, oracle_fp8_layer, rowmax_err
    rows = np.arange(x.shape[0]) if rows is None else np.asarray(rows)
    xb = synth.bf16_bits(x)[rows]
    oi, ow = idx.cpu().numpy()[rows], w.cpu().numpy()[rows]
    acc_r, _, pm_r = oracle_fp8_layer(orc, layer, xb, oi, ow, e_lo, e_hi, with_shared=False, pickmax=True)
    acc_all, out_all, pm_all = oracle_fp8_layer(orc, layer, xb, oi, ow, e_lo, e_hi, with_shared=shared, pickmax=True)
    yr, ys, out = yr.cpu().numpy()[rows], ys.cpu().numpy()[rows], synth.bf16_bits(out)[rows]
    assert_rows_close(yr, acc_r, TOL, what="yr", pickmax=pm_r)
    if shared:
        assert_rows_close(yr + ys, acc_all, TOL, what="yr + ys", pickmax=pm_all)
    assert_rows_close(orc.bf16_to_f32(out), orc.bf16_to_f32(out_all), TOL, what="out", pickmax=pm_all, rounded=True)
    return pm_r, pm_all


@pytest.mark.parametrize("T", [1, 7, 130, 300])
def test_small_layer(orc, T):
    from dsgx10_b200 import moe
    shp, layer, x, wr, bias, idx, w = _setup(512, 256, 8, 2, T, seed=200 + T)
    pl = moe.PrefillLayer(shp, layer.layer_w(), T)
    yr, ys, out = pl.run(x, idx, w)
    yr2, ys2, out2 = pl.run(x, idx, w)            # twice on one workspace: deterministic
    torch.cuda.synchronize()
    assert moe.ws_status(pl.ws) == 0
    assert torch.equal(yr, yr2) and torch.equal(out, out2)
    _check(orc, shp, layer, x, idx, w, yr, ys, out)


def test_ragged_segments_config1_shapes(orc):
    """hidden 2048, 64 experts of 1024, top-6: Zipf-biased routing gives empty experts and segments of many tiles;
    a sample of rows is checked against the oracle, all rows against the decode path (same contract)."""
    from dsgx10_b200 import moe
    T = 1500
    shp, layer, x, wr, bias, idx, w = _setup(2048, 1024, 64, 6, T, seed=20261104, zipf=True)
    counts = torch.bincount(idx.flatten().long(), minlength=64)
    assert int(counts.max()) > 512 and int((counts == 0).sum()) >= 0
    pl = moe.PrefillLayer(shp, layer.layer_w(), T)
    yr, ys, out = pl.run(x, idx, w)
    torch.cuda.synchronize()
    assert moe.ws_status(pl.ws) == 0
    rows = np.random.default_rng(0).choice(T, 12, replace=False)
    _check(orc, shp, layer, x, idx, w, yr, ys, out, rows=rows)
    # decode path on chunks of 8 rows: same numerics contract.  Both sides may have flipped one bf16 rounding of one
    # expert's output against the exact sums, so up to two ulps of the largest output added at an element are explained
    # (bf16_ulp(2 m) = 2 bf16_ulp(m)).
    from dsgx10_b200 import synth
    from tests.util import assert_rows_close, oracle_fp8_layer
    first = np.arange(64)
    _, _, pm = oracle_fp8_layer(orc, layer, synth.bf16_bits(x)[first], idx.cpu().numpy()[first], w.cpu().numpy()[first],
                                with_shared=False, pickmax=True)
    ws = moe.decode_ws(shp)
    for r0 in range(0, 64, 8):
        yd, sd = moe.moe_decode(shp, layer.layer_w(), x[r0:r0 + 8].contiguous(), idx[r0:r0 + 8].contiguous(),
                                w[r0:r0 + 8].contiguous(), ws)
        torch.cuda.synchronize()
        assert_rows_close(yr[r0:r0 + 8].cpu().numpy(), yd.cpu().numpy(), TOL, what="prefill vs decode yr",
                          pickmax=2 * pm[r0:r0 + 8], max_outliers=5e-3)
        assert_rows_close(ys[r0:r0 + 8].cpu().numpy(), sd.cpu().numpy(), TOL, what="prefill vs decode ys",
                          pickmax=2 * np.abs(sd.cpu().numpy()), max_outliers=5e-3)


def test_expert_parallel_and_no_shared(orc):
    from dsgx10_b200 import moe
    T = 200
    for e_lo, e_hi, shared in ((0, 4, True), (4, 8, False)):
        shp, layer, x, wr, bias, idx, w = _setup(512, 256, 8, 2, T, seed=260, shared=shared, e_lo=e_lo, e_hi=e_hi)
        pl = moe.PrefillLayer(shp, layer.layer_w(), T)
        yr, ys, out = pl.run(x, idx, w)
        torch.cuda.synchronize()
        assert moe.ws_status(pl.ws) == 0
        _check(orc, shp, layer, x, idx, w, yr, ys, out, shared=shared, e_lo=e_lo, e_hi=e_hi)


@pytest.mark.parametrize("H,I", [(4096, 2048), (1280, 768)])
def test_scale_staging_widths(orc, H, I):
    """The grouped GEMM brings a tile's scales into shared memory when K is a multiple of 512 and they fit (hidden 4096:
    32 k-blocks a row in the gate/up launch, 16 in the down launch), and fetches them from global memory block by block
    otherwise (hidden 1280, intermediate 768: 10 and 6 k-blocks): sampled rows of both against the oracle, segments of
    several tiles."""
    from dsgx10_b200 import moe
    T, E, topk = 700, 4, 2
    shp, layer, x, wr, bias, idx, w = _setup(H, I, E, topk, T, seed=295 + I)
    pl = moe.PrefillLayer(shp, layer.layer_w(), T)
    yr, ys, out = pl.run(x, idx, w)
    torch.cuda.synchronize()
    assert moe.ws_status(pl.ws) == 0
    rows = np.random.default_rng(1).choice(T, 6, replace=False)
    _check(orc, shp, layer, x, idx, w, yr, ys, out, rows=rows)


def test_pass_in_a_cuda_graph():
    """The whole pass (cluster launches chained as programmatic dependents) captured into a CUDA graph and replayed on new
    inputs gives the bits of the plain launches."""
    from dsgx10_b200 import moe
    T = 700
    shp, layer, x, wr, bias, idx, w = _setup(1024, 512, 16, 4, T, seed=287)
    shp2, _, x2, _, _, idx2, w2 = _setup(1024, 512, 16, 4, T, seed=288)
    pl = moe.PrefillLayer(shp, layer.layer_w(), T)
    out = torch.empty(T, 1024, dtype=torch.bfloat16, device="cuda")
    want1 = pl.run(x, idx, w, yr=False, ys=False)[2].clone()
    want2 = pl.run(x2, idx2, w2, yr=False, ys=False)[2].clone()
    xs, ids, ws_ = x.clone(), idx.clone(), w.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        pl.run(xs, ids, ws_, yr=False, ys=False, out=out)      # (first calls of a stream: nothing lazy left for the capture)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        pl.run(xs, ids, ws_, yr=False, ys=False, out=out)
    for xi, ii, wi, want in ((x, idx, w, want1), (x2, idx2, w2, want2), (x, idx, w, want1)):
        xs.copy_(xi), ids.copy_(ii), ws_.copy_(wi)
        graph.replay()
        torch.cuda.synchronize()
        assert moe.ws_status(pl.ws) == 0
        assert torch.equal(out, want)


def test_rounded_rows_only_and_gemm_hooks(orc):
    """Without the f32 outputs the rounded rows are the same; the bench hooks that launch one grouped GEMM alone over
    the workspace of a whole pass change nothing."""
    from dsgx10_b200 import moe
    T = 300
    shp, layer, x, wr, bias, idx, w = _setup(1024, 512, 16, 4, T, seed=280)
    pl = moe.PrefillLayer(shp, layer.layer_w(), T)
    yr, ys, out = pl.run(x, idx, w)
    out = out.clone()
    _, _, out2 = pl.run(x, idx, w, yr=False, ys=False)
    torch.cuda.synchronize()
    assert torch.equal(out2, out)
    snap = pl.ws.clone()
    for parts in (1, 2):
        pl.run(x, idx, w, yr=False, ys=False, parts=parts)
        torch.cuda.synchronize()
        assert torch.equal(pl.ws, snap) and moe.ws_status(pl.ws) == 0


def test_phases_in_separate_calls(orc):
    """dsgx_moe_prefill_phases (the reference's moe_prefill_phases, altar1 engine/experts/experts.h:191-193): the phases
    run one call each on one workspace give the whole pass's bits; the view names the workspace's intermediates."""
    from dsgx10_b200 import _lib, moe
    T = 300
    shp, layer, x, wr, bias, idx, w = _setup(1024, 512, 16, 4, T, seed=285)
    pl = moe.PrefillLayer(shp, layer.layer_w(), T)
    yr, ys, out = (t.clone() for t in pl.run(x, idx, w))
    pl.ws.zero_()
    f32 = dict(dtype=torch.float32, device="cuda")
    yr2, ys2, out2 = torch.zeros(T, 1024, **f32), torch.zeros(T, 1024, **f32), torch.zeros(T, 1024, dtype=torch.bfloat16, device="cuda")
    for ph in (_lib.PH_BUCKET, _lib.PH_UP, _lib.PH_DOWN, _lib.PH_SHARED, _lib.PH_COMBINE):
        pl.run(x, idx, w, yr=yr2, ys=ys2, out=out2, phases=ph)
    torch.cuda.synchronize()
    assert moe.ws_status(pl.ws) == 0
    assert torch.equal(yr2, yr) and torch.equal(ys2, ys) and torch.equal(out2, out)
    v = moe.prefill_view(shp, pl.ws, T)
    base = pl.ws.data_ptr()
    counts = pl.ws[v.counts - base: v.counts - base + 16 * 4].view(torch.int32)
    assert torch.equal(counts.long(), torch.bincount(idx.flatten().long(), minlength=16))


def test_chunk_invariance(orc):
    """A row's bits do not depend on the other rows of the chunk (altar1 engine/experts/tests/test_prefill.inc:293-302)."""
    from dsgx10_b200 import moe
    T = 260
    shp, layer, x, wr, bias, idx, w = _setup(512, 256, 8, 2, T, seed=270)
    pl = moe.PrefillLayer(shp, layer.layer_w(), T)
    yr, ys, out = pl.run(x, idx, w)
    yr, ys = yr.clone(), ys.clone()
    for a, b in ((0, 100), (100, 260), (37, 38)):
        yr2, ys2, _ = pl.run(x[a:b].contiguous(), idx[a:b].contiguous(), w[a:b].contiguous())
        torch.cuda.synchronize()
        assert torch.equal(yr2, yr[a:b]) and torch.equal(ys2, ys[a:b])


def test_full_size_16384_tokens_properties(orc):
    """The benchmark's size (hidden 2048, 64 experts x 1024, top-6, 16384 tokens, Zipf-skewed routing: segments from a few
    rows to thousands): properties that do not need the oracle over every row -- the sort is a permutation with the
    right counts, a chunk of rows run alone has the bits it has inside the whole pass, a second pass repeats the first
    bit for bit, and sampled rows (the hot expert's, a rare expert's, the first and the last) match the oracle."""
    from dsgx10_b200 import moe
    T, H, I, E, topk = 16384, 2048, 1024, 64, 6
    shp, layer, x, wr, bias, idx, w = _setup(H, I, E, topk, T, seed=20261104, zipf=True)
    counts = torch.bincount(idx.flatten().long(), minlength=E)
    assert int(counts.max()) > 2000 and int(counts.min()) < 256          # ragged: huge and tiny segments
    sp = moe.sort_pack(idx, E)
    assert torch.equal(sp["counts"].long(), counts)
    assert torch.equal(torch.sort(sp["perm_tok"].long() * topk + sp["perm_slot"].long()).values,
                       torch.arange(T * topk, device="cuda"))
    e_sorted = idx.flatten()[(sp["perm_tok"].long() * topk + sp["perm_slot"].long())]
    assert bool((e_sorted[1:] >= e_sorted[:-1]).all())                     # expert-major order
    pl = moe.PrefillLayer(shp, layer.layer_w(), T)
    yr, ys, out = pl.run(x, idx, w)
    yr, ys, out = yr.clone(), ys.clone(), out.clone()
    yr_b, ys_b, out_b = pl.run(x, idx, w)
    torch.cuda.synchronize()
    assert moe.ws_status(pl.ws) == 0
    assert torch.equal(yr_b, yr) and torch.equal(ys_b, ys) and torch.equal(out_b, out)   # run to run
    for a, b in ((0, 4096), (9000, 9300), (16383, 16384)):
        yr2, ys2, out2 = pl.run(x[a:b].contiguous(), idx[a:b].contiguous(), w[a:b].contiguous())
        torch.cuda.synchronize()
        assert torch.equal(yr2, yr[a:b]) and torch.equal(ys2, ys[a:b]) and torch.equal(out2, out[a:b])
    hot, rare = int(counts.argmax()), int(torch.where(counts > 0, counts, T * topk).argmin())
    rows = [0, T - 1]
    for e in (hot, rare):
        rows += torch.nonzero((idx == e).any(dim=1)).flatten()[:3].tolist()
    _check(orc, shp, layer, x, idx, w, yr, ys, out, rows=sorted(set(rows)))


def test_ragged_batch_config5(orc):
    """The mixed batch of the fifth benchmark configuration in ONE pass over the config-1 layer: 40 one-token decode rows, 16
    speculative-verify requests of 2-6 rows and 8 prefill chunks of 512-4096 rows (the seeded mix bench.py --workload ragged
    runs).  Rows of every request class are checked against the oracle, and the one-token rows also against the decode
    path (same contract: what differs is explained by rounding flips of single outputs)."""
    from dsgx10_b200 import moe, synth
    from tests.util import assert_rows_close, oracle_fp8_layer
    H, I, E, topk = 2048, 1024, 64, 6
    rng = np.random.default_rng(20261102 + 5)
    reqs = [1] * 40 + [int(v) for v in rng.integers(2, 7, 16)] + [int(v) for v in rng.integers(512, 4097, 8)]
    T = sum(reqs)
    starts = np.concatenate([[0], np.cumsum(reqs)])
    shp, layer, x, wr, bias, idx, w = _setup(H, I, E, topk, T, seed=20261105)
    pl = moe.PrefillLayer(shp, layer.layer_w(), T)
    yr, ys, out = pl.run(x, idx, w)
    torch.cuda.synchronize()
    assert moe.ws_status(pl.ws) == 0
    pick = np.random.default_rng(1)
    rows = list(pick.choice(40, 4, replace=False))                                   # decode rows
    rows += [int(starts[40 + j]) for j in pick.choice(16, 3, replace=False)]         # first row of three verify requests
    rows += [int(starts[40 + 16 - 1 + 1] - 1)]                                       # last row of the last verify request
    for j in range(8):                                                               # a row inside every prefill chunk
        rows.append(int(starts[56 + j] + pick.integers(0, reqs[56 + j])))
    rows += [T - 1]
    _check(orc, shp, layer, x, idx, w, yr, ys, out, rows=sorted(set(rows)))
    # the 40 one-token rows through the decode path, eight at a time
    first = np.arange(40)
    _, _, pm = oracle_fp8_layer(orc, layer, synth.bf16_bits(x)[first], idx.cpu().numpy()[first], w.cpu().numpy()[first],
                                with_shared=False, pickmax=True)
    ws = moe.decode_ws(shp)
    for r0 in range(0, 40, 8):
        yd, sd = moe.moe_decode(shp, layer.layer_w(), x[r0:r0 + 8].contiguous(), idx[r0:r0 + 8].contiguous(),
                                w[r0:r0 + 8].contiguous(), ws)
        torch.cuda.synchronize()
        assert_rows_close(yr[r0:r0 + 8].cpu().numpy(), yd.cpu().numpy(), TOL, what="ragged batch vs decode yr",
                          pickmax=2 * pm[r0:r0 + 8], max_outliers=5e-3)
        assert_rows_close(ys[r0:r0 + 8].cpu().numpy(), sd.cpu().numpy(), TOL, what="ragged batch vs decode ys",
                          pickmax=2 * np.abs(sd.cpu().numpy()), max_outliers=5e-3)


def test_512_experts(orc):
    """The largest expert count the interface accepts (the tile table has E + 1 entries: one more than threads build it)."""
    from dsgx10_b200 import moe
    T = 700
    shp, layer, x, wr, bias, idx, w = _setup(256, 256, 512, 8, T, seed=290)
    pl = moe.PrefillLayer(shp, layer.layer_w(), T)
    yr, ys, out = pl.run(x, idx, w)
    torch.cuda.synchronize()
    assert moe.ws_status(pl.ws) == 0
    _check(orc, shp, layer, x, idx, w, yr, ys, out, rows=np.arange(0, T, 23))
