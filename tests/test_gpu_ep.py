"""Expert parallelism on two GPUs (NCCL): the decode all-reduce scheme and the prefill all-to-all scheme against the
single-GPU result.  Skipped on a box with one GPU."""
import os
import socket
import sys

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from dsgx10_b200 import ep, moe, synth
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        H, I, E, topk = 1024, 512, 16, 4
        lo, hi = ep.expert_range(rank, world, E)
        full_shp = moe.shape(H, I, E, topk)
        my_shp = moe.shape(H, I, E, topk, e_lo=lo, e_hi=hi)
        full = synth.Fp8Layer(H, I, E, 300, device=dev)                       # the single-GPU reference layer
        mine = synth.Fp8Layer(H, I, E, 300, device=dev, shared=(rank == 0), e_range=(lo, hi))
        wr = synth.router_weights(E, H, 301).to(dev)
        res = {}
        # decode: all-reduce of the partial sums
        x = synth.activations(5, H, 302).to(dev)
        ref = moe.LayerStep(full_shp, wr, device=dev)
        ref.run(full.layer_w(), x)
        st = moe.LayerStep(my_shp, wr, device=dev)
        st.run(mine.layer_w(), x, finalize=False)
        if rank != 0:
            st.ys.zero_()
        ep.allreduce_partials(st.yr, st.ys)
        torch.cuda.synchronize()
        den = float(ref.yr[:5].abs().max())
        res["decode_yr"] = float((st.yr[:5] - ref.yr[:5]).abs().max()) / den
        res["decode_ys"] = float((st.ys[:5] - ref.ys[:5]).abs().max())
        res["decode_idx"] = bool(torch.equal(st.idx[:5], ref.idx[:5]))
        # decode: the same reduction by the library's own kernel over peer memory, three steps in a row (both halves of
        # the buffer and the step counter); the bits are those of bf16((yr0 + yr1) + ys0) and equal on both ranks
        pr = ep.PeerReduce(H, shared_rank=0)
        peer_ok, peer_same = True, True
        for step_no in range(1, 4):
            xs = synth.activations(3 + step_no, H, 310 + step_no).to(dev)
            M = xs.shape[0]
            st.run(mine.layer_w(), xs, finalize=False)
            if rank != 0:
                st.ys.zero_()
            want_parts = torch.stack([st.yr[:M], st.ys[:M]]).clone()
            gathered = [torch.empty_like(want_parts) for _ in range(world)]
            dist.all_gather(gathered, want_parts)
            want = moe.finalize(gathered[0][0] + gathered[1][0], gathered[0][1])
            yr_p, ys_p = pr.parts(pr.launched + 1)
            st.run(mine.layer_w(), xs, finalize=False, yr=yr_p, ys=ys_p)
            got = pr.finalize(M).clone()
            torch.cuda.synchronize()
            peer_ok = peer_ok and bool(torch.equal(got, want))
            both = [torch.empty_like(got) for _ in range(world)]
            dist.all_gather(both, got)
            peer_same = peer_same and bool(torch.equal(both[0], both[1]))
        res["peer_ok"], res["peer_same"], res["peer_status"] = peer_ok, peer_same, int(pr.status.item())
        # the reduction with the residual add and the next block's RMSNorm in the same kernel: out as before, h and normed
        # equal to the one-GPU entry point on the all-gathered sums, the same bits on both ranks
        g = torch.Generator().manual_seed(77)
        nw = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).to(dev)
        resid = torch.randn(4, H, generator=g).to(torch.bfloat16).to(dev)
        xs = synth.activations(4, H, 340).to(dev)
        st.run(mine.layer_w(), xs, finalize=False)
        if rank != 0:
            st.ys.zero_()
        mine_parts = torch.stack([st.yr[:4], st.ys[:4]]).clone()
        gathered = [torch.empty_like(mine_parts) for _ in range(world)]
        dist.all_gather(gathered, mine_parts)
        want3 = moe.finalize_add_norm(gathered[0][0] + gathered[1][0], gathered[0][1], nw, resid)
        yr_p, ys_p = pr.parts(pr.launched + 1)
        st.run(mine.layer_w(), xs, finalize=False, yr=yr_p, ys=ys_p)
        got3 = [t.clone() for t in pr.finalize_norm(4, nw, resid)]
        torch.cuda.synchronize()
        res["norm_ok"] = all(bool(torch.equal(a, b)) for a, b in zip(got3, want3)) and int(pr.status.item()) == 0
        # the shared expert in parts: each rank computes half of its intermediate channels, its ys is an unrounded partial
        # sum; the reduction adds the parts in rank order, rounds that sum to bf16 once and adds it to the sum of yr
        I2 = 1024
        full2 = synth.Fp8Layer(H, I2, E, 320, device=dev)
        ref2 = moe.LayerStep(moe.shape(H, I2, E, topk), wr, device=dev)
        st2 = moe.LayerStep(moe.shape(H, I2, E, topk, e_lo=lo, e_hi=hi, sh_lo=rank * 512, sh_hi=(rank + 1) * 512), wr, device=dev)
        pr2 = ep.PeerReduce(H, shared_rank=-2)
        parts_ok, parts_close = True, 0.0
        for step_no in range(1, 4):
            xs = synth.activations(2 + step_no, H, 330 + step_no).to(dev)
            M = xs.shape[0]
            want_one = ref2.run(full2.layer_w(), xs).clone()
            yr_p, ys_p = pr2.parts(pr2.launched + 1)
            st2.run(full2.layer_w(), xs, finalize=False, yr=yr_p, ys=ys_p)
            mine_parts = torch.stack([yr_p[:M], ys_p[:M]]).clone()
            got = pr2.finalize(M).clone()
            gathered = [torch.empty_like(mine_parts) for _ in range(world)]
            dist.all_gather(gathered, mine_parts)
            want = moe.finalize(gathered[0][0] + gathered[1][0], (gathered[0][1] + gathered[1][1]).to(torch.bfloat16).float())
            torch.cuda.synchronize()
            parts_ok = parts_ok and bool(torch.equal(got, want))
            den = want_one.float().abs().amax(dim=1, keepdim=True)
            parts_close = max(parts_close, float(((got.float() - want_one.float()).abs() / den).max()))
        res["parts_ok"], res["parts_close"], res["parts_status"] = parts_ok, parts_close, max(int(pr2.status.item()), moe.ws_status(st2.ws))
        # the same kernel over a prefill's rows (its many-CTA form): f32 partial sums of 600 rows, no shared-expert term
        prw = ep.PeerReduce(H, rows_cap=600, shared_rank=-1)
        wide_ok = True
        for step_no in range(1, 3):
            part = torch.randn(600, H, device=dev, generator=torch.Generator(device=dev).manual_seed(500 + 10 * step_no + rank))
            yr_p, _ = prw.parts(prw.launched + 1)
            yr_p.copy_(part)
            got = prw.finalize(600).clone()
            both = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(both, part)
            want = moe.finalize(both[0] + both[1])
            torch.cuda.synchronize()
            wide_ok = wide_ok and bool(torch.equal(got, want))
        res["peer_wide_ok"], res["peer_wide_status"] = wide_ok, int(prw.status.item())
        # and its sliced form: each rank reduces half of the rows and stores them into both ranks' output rows
        prs = ep.PeerReduce(H, rows_cap=601, shared_rank=-1, sliced=True)
        sl_ok = True
        for step_no in range(1, 4):
            part = torch.randn(601, H, device=dev, generator=torch.Generator(device=dev).manual_seed(700 + 10 * step_no + rank))
            yr_p, _ = prs.parts(prs.launched + 1)
            yr_p.copy_(part)
            got = prs.finalize(601).clone()
            both = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(both, part)
            want = moe.finalize(both[0] + both[1])
            torch.cuda.synchronize()
            sl_ok = sl_ok and bool(torch.equal(got, want))
        res["peer_sliced_ok"], res["peer_sliced_status"] = sl_ok, int(prs.status.item())
        # prefill: rows partitioned, all-to-all dispatch and combine
        T = 96
        xa = synth.activations(T, H, 303).to(dev)
        idx, w = moe.route(full_shp, moe.router_logits(xa, wr), None)
        pl_full = moe.PrefillLayer(full_shp, full.layer_w(), T, device=dev)
        yr_full, _, _ = pl_full.run(xa, idx, w)
        pl = moe.PrefillLayer(my_shp, mine.layer_w(), T, device=dev)
        rows = torch.arange(rank, T, world, device=dev)

        def local(xr, ir, wr_):
            yr, _, _ = pl.run(xr, ir, wr_)
            return yr.clone()

        acc = ep.all_to_all_experts(xa[rows].contiguous(), idx[rows].contiguous(), w[rows].contiguous(), E, local)
        torch.cuda.synchronize()
        res["prefill"] = float((acc - yr_full[rows]).abs().max()) / float(yr_full.abs().max())
        res["status"] = max(moe.ws_status(st.ws), moe.ws_status(pl.ws))
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


def test_two_gpus_match_one():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    for rank, res in sorted(q.get(timeout=5) for _ in range(2)):
        assert res["decode_idx"] and res["status"] == 0
        assert res["decode_yr"] <= 1e-6 and res["decode_ys"] == 0.0, res    # only the association of the f32 adds differs
        assert res["prefill"] <= 1e-6, res
        assert res["peer_ok"] and res["peer_same"] and res["peer_status"] == 0, res
        assert res["parts_ok"] and res["parts_status"] == 0, res
        assert res["norm_ok"], res
        assert res["parts_close"] <= 2e-3 + 2 ** -7, res     # against one GPU: a bf16 rounding flip of the output at most
        assert res["peer_wide_ok"] and res["peer_wide_status"] == 0, res
        assert res["peer_sliced_ok"] and res["peer_sliced_status"] == 0, res
