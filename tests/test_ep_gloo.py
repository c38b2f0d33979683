"""Expert-parallel host logic on CPU: two gloo ranks, the oracle as each rank's local compute.  Checks that both
exchange schemes (all-reduce of partial sums; all-to-all dispatch / combine of rows) reproduce the single-rank result."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, scheme, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from dsgx10_b200 import ep, synth
    from oracle import oracle as orc
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        H, I, E, topk, T = 256, 128, 8, 3, 10
        layer = synth.Fp8Layer(H, I, E, 77, device="cpu")
        experts = {e: layer.canonical(e) for e in range(E)}
        x = synth.activations(T, H, 78)
        wr = synth.router_weights(E, H, 79).numpy()
        xb = synth.bf16_bits(x)
        idx, w = orc.route(orc.router_logits(xb, wr), None, topk)
        full, _ = orc.moe_fp8_layer(xb, idx, w, experts, None, with_shared=False)
        lo, hi = ep.expert_range(rank, world, E)

        def local(xr, ir, wr_):
            acc, _ = orc.moe_fp8_layer(synth.bf16_bits(xr), ir.numpy(), wr_.numpy(), experts, None, e_lo=lo, e_hi=hi,
                                       with_shared=False)
            return torch.from_numpy(acc)

        if scheme == "reduce":
            yr = local(x, torch.from_numpy(idx), torch.from_numpy(w))
            ys = torch.zeros_like(yr)
            ep.allreduce_partials(yr, ys)
            got, want = yr.numpy(), full
        else:
            mine = np.arange(T)[rank::world]          # this rank's rows
            acc = ep.all_to_all_experts(x[mine], torch.from_numpy(idx[mine]), torch.from_numpy(w[mine]), E, local)
            got, want = acc.numpy(), full[mine]
        err = float(np.abs(got - want).max() / np.abs(want).max())
        q.put((rank, err))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("scheme", ["reduce", "all_to_all"])
def test_two_ranks_reproduce_one(scheme):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, scheme, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    res = sorted(q.get(timeout=5) for _ in range(2))
    for rank, err in res:
        assert err <= 1e-6, (rank, err)    # the partial sums are added in another association, nothing else differs


def test_dispatch_plan_and_ranges():
    import torch
    sys.path.insert(0, ROOT)
    from dsgx10_b200 import ep
    assert ep.expert_range(3, 8, 256) == (96, 128)
    idx = torch.tensor([[0, 5], [6, 7], [1, 2]], dtype=torch.int32)
    rows, mask = ep.dispatch_plan(idx, 2, 8)
    assert rows[0].tolist() == [0, 2] and rows[1].tolist() == [0, 1]
    assert mask.tolist() == [[True, True], [False, True], [True, False]]
