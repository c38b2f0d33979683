"""The two RMSNorm fusions around the experts, against the CPU oracle, bit for bit:
the norm in front of the router inside the layer step's first kernel, and the residual add + norm inside the kernel that
reduces the partial sums (one GPU's own sums, and the peer form run with a world of one)."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def _from_bits(b, device="cuda"):
    return torch.from_numpy(b.view(np.int16).copy()).view(torch.bfloat16).to(device)


def _norm_inputs(M, H, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(M, H, generator=g) * 3.0).to(torch.bfloat16).cuda()
    w = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).cuda()
    return x, w


@pytest.mark.parametrize("M,fused", [(1, False), (2, False), (5, False), (3, True), (8, True), (1, True)])
@pytest.mark.parametrize("mode", [0, 1])
def test_front_norm_fp8(orc, M, fused, mode):
    """x -> RMSNorm -> router + experts in one step equals normalising first (oracle) and running the plain step."""
    from dsgx10_b200 import moe, synth
    H, I, E, topk = 1024, 512, 16, 4
    shp = moe.shape(H, I, E, topk)
    layer = synth.Fp8Layer(H, I, E, 900 + M, device="cuda")
    wr = synth.router_weights(E, H, 901, device="cpu").cuda()
    x, nw = _norm_inputs(M, H, 902 + M)
    eps = 1e-6 if mode == 0 else 1e-5
    xn = orc.rmsnorm(_bits(x), _bits(nw), eps, mode)
    step = moe.LayerStep(shp, wr, fused=fused, norm_w=nw, norm_eps=eps, norm_mode=mode)
    plain = moe.LayerStep(shp, wr, fused=fused)
    for _ in range(2):
        got = step.run(layer.layer_w(), x).clone()
        want = plain.run(layer.layer_w(), _from_bits(xn)).clone()
        torch.cuda.synchronize()
        assert moe.ws_status(step.ws) == 0 and moe.ws_status(plain.ws) == 0
        assert (_bits(step.xn[:M]) == xn).all()
        assert torch.equal(step.logits[:M], plain.logits[:M]) and torch.equal(step.idx[:M], plain.idx[:M])
        assert torch.equal(got, want)
    # and the normalised rows matter: the un-normalised input routes differently or gives other outputs
    raw = plain.run(layer.layer_w(), x).clone()
    assert not torch.equal(raw, got)


def test_front_norm_config2_width(orc):
    """hidden 4096 (two chunks a thread in the sum of squares), 256 experts grouped, one row: normalised rows, logits and
    picks bit for bit against the oracle."""
    from dsgx10_b200 import moe, synth
    from tests.util import oracle_route
    H, I, E, topk = 4096, 256, 256, 8
    shp = moe.shape(H, I, E, topk, n_group=8, topk_group=4)
    x, nw = _norm_inputs(1, H, 77)
    wr = synth.router_weights(E, H, 78, device="cpu").cuda()
    xn = orc.rmsnorm(_bits(x), _bits(nw), 1e-6, 0)
    lg, oi, ow = oracle_route(orc, xn, wr.cpu().numpy(), None, shp)
    layer = synth.Fp8Layer(H, I, E, 79, device="cuda")
    step = moe.LayerStep(shp, wr, norm_w=nw)
    step.run(layer.layer_w(), x)
    torch.cuda.synchronize()
    assert moe.ws_status(step.ws) == 0
    assert (_bits(step.xn[:1]) == xn).all()
    assert (step.logits[:1].cpu().numpy().view(np.uint32) == lg.view(np.uint32)).all()
    assert (step.idx[:1].cpu().numpy() == oi).all()


@pytest.mark.parametrize("M", [1, 4])
def test_front_norm_int4(orc, M):
    from dsgx10_b200 import _lib, moe, synth
    H, I, E, topk = 1024, 512, 8, 2
    shp = moe.shape(H, I, E, topk, fmt=_lib.FMT_INT4, score_fn=1)
    layer = synth.Int4Layer(H, I, E, 910, device="cuda")
    wr = synth.router_weights(E, H, 911, device="cpu").cuda()
    x, nw = _norm_inputs(M, H, 912 + M)
    xn = orc.rmsnorm(_bits(x), _bits(nw), 1e-5, 1)
    step = moe.LayerStep(shp, wr, norm_w=nw, norm_eps=1e-5, norm_mode=1)
    plain = moe.LayerStep(shp, wr)
    got = step.run(layer.layer_w(), x).clone()
    want = plain.run(layer.layer_w(), _from_bits(xn)).clone()
    torch.cuda.synchronize()
    assert moe.ws_status(step.ws) == 0
    assert (_bits(step.xn[:M]) == xn).all()
    assert torch.equal(step.idx[:M], plain.idx[:M]) and torch.equal(got, want)


@pytest.mark.parametrize("M,H", [(1, 512), (8, 4096), (3, 6144), (300, 2048), (2, 8192)])
@pytest.mark.parametrize("fin_mode,norm_mode,add_f32", [(0, 0, False), (1, 1, False), (0, 1, True)])
def test_finalize_add_norm(orc, M, H, fin_mode, norm_mode, add_f32):
    from dsgx10_b200 import moe
    g = torch.Generator().manual_seed(M * 131 + H)
    R = torch.randn(M, H, generator=g).cuda()
    S = (torch.randn(M, H, generator=g) * 0.5).cuda()
    res = (torch.randn(M, H, generator=g) * 2).to(torch.bfloat16).cuda()
    nw = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).cuda()
    Rn, Sn = R.cpu().numpy(), S.cpu().numpy()
    v = (orc.bf16_to_f32(orc.f32_to_bf16(Rn)) + orc.bf16_to_f32(orc.f32_to_bf16(Sn))) if fin_mode == 1 else Rn + Sn
    want = orc.add_norm(v.astype(np.float32), _bits(res), _bits(nw), 1e-6, norm_mode, add_f32)
    got = moe.finalize_add_norm(R, S, nw, res, mode=fin_mode, eps=1e-6, norm_mode=norm_mode, add_f32=add_f32)
    torch.cuda.synchronize()
    for name, a, b in zip(("out", "h", "normed"), got, want):
        assert (_bits(a) == b).all(), name
    assert torch.equal(got[0], moe.finalize(R, S, mode=fin_mode))
    # no residual: h = out
    got2 = moe.finalize_add_norm(R, None, nw, None, mode=0, eps=1e-6, norm_mode=norm_mode)
    want2 = orc.add_norm(Rn, None, _bits(nw), 1e-6, norm_mode)
    torch.cuda.synchronize()
    for a, b in zip(got2, want2):
        assert (_bits(a) == b).all()


def test_peer_form_with_a_world_of_one(orc):
    """The peer kernel's own path (flags, parity halves, step counter) on one GPU: a peer set whose only rank is this
    GPU.  Three steps in a row; each equals the oracle and the one-GPU entry point."""
    from dsgx10_b200 import _lib, moe
    H, cap = 2048, 8
    parts = torch.zeros(2, 2, cap, H, device="cuda")
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    pp = torch.tensor([parts.data_ptr()], dtype=torch.int64, device="cuda")
    fp = torch.tensor([flags.data_ptr()], dtype=torch.int64, device="cuda")

    class PeerSet(C.Structure):
        _fields_ = [("parts", C.c_void_p), ("flags", C.c_void_p), ("state", C.c_void_p), ("rank", C.c_int32),
                    ("world", C.c_int32), ("rows_cap", C.c_int32), ("shared_rank", C.c_int32), ("outs", C.c_void_p),
                    ("done", C.c_void_p)]

    ps = PeerSet(pp.data_ptr(), fp.data_ptr(), state.data_ptr(), 0, 1, cap, 0, None, None)
    g = torch.Generator().manual_seed(5)
    nw = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).cuda()
    for step in range(1, 4):
        M = 2 + step
        R, S = torch.randn(M, H, generator=g).cuda(), torch.randn(M, H, generator=g).cuda()
        res = torch.randn(M, H, generator=g).to(torch.bfloat16).cuda()
        parts[step & 1, 0, :M] = R
        parts[step & 1, 1, :M] = S
        out, h, normed = (torch.empty(M, H, dtype=torch.bfloat16, device="cuda") for _ in range(3))
        an = moe.add_norm_args(nw, res, 1e-6, 0, False, h, normed)
        rc = _lib.lib().dsgx_finalize_peers_norm(C.byref(ps), M, H, out.data_ptr(), C.byref(an), status.data_ptr(),
                                                 torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0 and int(state[0].item()) == step
        want = orc.add_norm((R + S).cpu().numpy(), _bits(res), _bits(nw), 1e-6, 0)
        for a, b in zip((out, h, normed), want):
            assert (_bits(a) == b).all()
