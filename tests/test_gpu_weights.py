"""A layer written to a layer file and loaded back (dsgx10_b200/weights.py) runs through the operator with the bits of
the same layer built in memory: the file path's layouts, offsets and descriptors are the ones the kernels read."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def test_fp8_layer_from_file_same_bits(tmp_path):
    from dsgx10_b200 import moe, synth, weights as W
    H, I, E, topk, M = 1024, 512, 16, 4, 5
    mem = synth.Fp8Layer(H, I, E, 800, device="cpu")
    experts = {e: mem.canonical(e) for e in range(E)}
    path = str(tmp_path / "fp8.dsgx")
    W.write_layer_file(path, H, I, E, W.FMT_FP8, experts, shared=mem.canonical(E))
    layer = W.load_layer_file(path, device="cuda")
    mem.to("cuda")
    shp = moe.shape(H, I, E, topk)
    wr = synth.router_weights(E, H, 801).cuda()
    x = synth.activations(M, H, 802).cuda()
    a, b = moe.LayerStep(shp, wr), moe.LayerStep(shp, wr)
    out_a = a.run(mem.layer_w(), x).clone()
    out_b = b.run(layer.layer_w(), x).clone()
    torch.cuda.synchronize()
    assert moe.ws_status(a.ws) == 0 and moe.ws_status(b.ws) == 0
    assert torch.equal(a.yr[:M], b.yr[:M]) and torch.equal(a.ys[:M], b.ys[:M]) and torch.equal(out_a, out_b)
    # the prefill path re-tiles from the same pool
    T = 130
    xt = synth.activations(T, H, 803).cuda()
    idx, w = moe.route(shp, moe.router_logits(xt, wr), None)
    ya = moe.PrefillLayer(shp, mem.layer_w(), T).run(xt, idx, w)
    yb = moe.PrefillLayer(shp, layer.layer_w(), T).run(xt, idx, w)
    torch.cuda.synchronize()
    assert all(torch.equal(p, q) for p, q in zip(ya, yb))


def test_int4_layer_from_file_same_bits(tmp_path):
    from dsgx10_b200 import _lib, moe, synth, weights as W
    H, I, E, topk, M = 1024, 512, 8, 4, 3
    mem = synth.Int4Layer(H, I, E, 810, device="cuda")
    experts = {e: [(wp, s, None) for wp, s in mem.raw[e]] for e in range(E)}
    path = str(tmp_path / "int4.dsgx")
    W.write_layer_file(path, H, I, E, W.FMT_INT4, experts, shared=tuple(mem.sh_bits))
    layer = W.load_layer_file(path, device="cuda")
    shp = moe.shape(H, I, E, topk, fmt=_lib.FMT_INT4, score_fn=1)
    wr = synth.router_weights(E, H, 811).cuda()
    x = synth.activations(M, H, 812).cuda()
    a, b = moe.LayerStep(shp, wr), moe.LayerStep(shp, wr)
    a.run(mem.layer_w(), x)
    b.run(layer.layer_w(), x)      # (the file holds the shared expert as the interleaved gate/up matrix)
    torch.cuda.synchronize()
    assert moe.ws_status(a.ws) == 0 and moe.ws_status(b.ws) == 0
    assert torch.equal(a.yr[:M], b.yr[:M]) and torch.equal(a.ys[:M], b.ys[:M])


def test_mx4_layer_from_file_same_bits(tmp_path):
    from dsgx10_b200 import _lib, moe, synth, weights as W
    H, I, E, topk, M = 1024, 512, 8, 4, 3
    mem = synth.Mx4Layer(H, I, E, 820, device="cpu")
    experts = {e: mem.canonical(e) for e in range(E)}
    path = str(tmp_path / "mx4.dsgx")
    W.write_layer_file(path, H, I, E, W.FMT_MXFP4, experts, shared=mem.canonical(E))
    layer = W.load_layer_file(path, device="cuda")
    mem.to("cuda")
    shp = moe.shape(H, I, E, topk, fmt=_lib.FMT_MXFP4)
    wr = synth.router_weights(E, H, 821).cuda()
    x = synth.activations(M, H, 822).cuda()
    a, b = moe.LayerStep(shp, wr), moe.LayerStep(shp, wr)
    out_a = a.run(mem.layer_w(), x).clone()
    out_b = b.run(layer.layer_w(), x).clone()
    torch.cuda.synchronize()
    assert moe.ws_status(a.ws) == 0 and moe.ws_status(b.ws) == 0
    assert torch.equal(a.yr[:M], b.yr[:M]) and torch.equal(a.ys[:M], b.ys[:M]) and torch.equal(out_a, out_b)
