#!/usr/bin/env python
"""Benchmark of the MoE decode layer-step (the headline metric): DeepSeek-style FP8 layer, hidden 4096, 256 routed
experts of intermediate 2048, top-8 sigmoid routing with group-limited selection (8 groups, 4 kept), one shared expert,
one row by default (`--rows` 1..8).

  python bench.py --gpus N --steps K --warmup W          this library on N GPUs (torchrun for N > 1)
  python bench.py --impl reference ...                   the CPU path (the oracle port) on the host cores

A step = router logits + top-k + activation quantisation + expert gate/up (SwiGLU) + expert down + combine + rounding of
one batch of rows through one layer.  Weights are cold: steps cycle through `--layers` distinct layers and distinct
activations, so that no step finds its experts in L2 (each step streams ~231 MB, the L2 holds 126 MB).
One JSON line on stdout (rank 0).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG_BIG = dict(H=4096, I=2048, E=256, topk=8, n_group=8, topk_group=4, score_fn=0, fmt="fp8")                  # config 2
CFG = dict(CFG_BIG)
CFG_INT4 = dict(H=6144, I=2048, E=168, topk=8, n_group=1, topk_group=1, score_fn=1, fmt="int4")   # config 3
CFG_SMALL = dict(H=2048, I=1024, E=64, topk=6, n_group=1, topk_group=1, score_fn=0, fmt="fp8")      # config 1
# config 2's shapes with the routed experts in ds41f's own format (MXFP4: e2m1, a ue8m0 scale per 32) and the FP8 shared expert
CFG_MX4 = dict(H=4096, I=2048, E=256, topk=8, n_group=8, topk_group=4, score_fn=0, fmt="mx4")


def workload_name(rows):
    if CFG["fmt"] == "int4":
        return (f"config 3: INT4-g32 MoE decode layer-step, hidden 6144, 168 experts x 2048, top-8 softmax, "
                f"+ bf16 shared expert, rows {rows}")
    if CFG["fmt"] == "mx4":
        return (f"config 2 shapes, MXFP4 routed experts: MoE decode layer-step, hidden 4096, 256 experts x 2048 (e2m1, ue8m0 "
                f"scale per 32), top-8 grouped (8 groups / 4), + FP8 shared expert, rows {rows}")
    if CFG["H"] == 2048:
        return (f"config 1: FP8 MoE decode layer-step, hidden 2048, 64 experts x 1024, top-6 sigmoid, + shared expert, "
                f"rows {rows}")
    return (f"config 2: FP8 MoE decode layer-step, hidden 4096, 256 experts x 2048, top-8 grouped (8 groups / 4), "
            f"+ shared expert, rows {rows}")
SEED = 20261102


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i].lower() == "active"})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def step_bytes(rows_union, rows):
    """Algorithmic bytes of one step: each distinct picked expert and the shared expert once (three matrices and
    their block scales), the router weights, the activations in and out."""
    H, I, E = CFG["H"], CFG["I"], CFG["E"]
    if CFG["fmt"] == "int4":  # routed experts in 2368-byte blocks of 8 x 512 values, the shared expert bf16
        return rows_union * 3 * I * H * 2368 // 4096 + 3 * I * H * 2 + E * H * 4 + rows * H * 2 * 2
    expert = 3 * I * H + 3 * (I // 128) * (H // 128) * 4
    if CFG["fmt"] == "mx4":  # routed experts in 544-byte blocks of 8 x 128 values, the shared expert FP8
        return rows_union * 3 * (I // 8) * (H // 128) * 544 + expert + E * H * 4 + rows * H * 2 * 2
    return (rows_union + 1) * expert + E * H * 4 + rows * H * 2 * 2


def up_bytes(n_routed, shared_frac=1.0):
    """Algorithmic bytes of a gate/up launch: n_routed picked experts and shared_frac of the shared expert (two matrices
    and their scales each)."""
    H, I = CFG["H"], CFG["I"]
    if CFG["fmt"] == "int4":
        return n_routed * (2 * I * H * 2368 // 4096) + shared_frac * 2 * I * H * 2
    if CFG["fmt"] == "mx4":
        return n_routed * 2 * (I // 8) * (H // 128) * 544 + shared_frac * (2 * I * H + 2 * (I // 128) * (H // 128) * 4)
    return (n_routed + shared_frac) * (2 * I * H + 2 * (I // 128) * (H // 128) * 4)


# --------------------------------------------------------------------------------------------------------- CPU arm

def run_reference(args):
    """Times the CPU path (the oracle port of the reference's Python/C++ CPU references) on the host cores."""
    import numpy as np
    import torch
    from dsgx10_b200 import moe, synth
    from oracle import oracle as orc
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    orc.build(with_ref=False) if not os.path.exists(os.path.join(ROOT, "oracle", "liboracle.so")) else None
    orc.set_threads()  # every host core, whatever OMP_NUM_THREADS the launcher exported
    H, I, E, topk = CFG["H"], CFG["I"], CFG["E"], CFG["topk"]
    rows = args.rows
    shp = moe.shape(H, I, E, topk, n_group=CFG["n_group"], topk_group=CFG["topk_group"])
    x = synth.activations(rows, H, SEED + 1000)
    wr = synth.router_weights(E, H, SEED + 2000).numpy()
    xb = synth.bf16_bits(x)
    logits = orc.router_logits(xb, wr)
    idx, w = orc.route(logits, None, topk, 0, CFG["n_group"], CFG["topk_group"], True, 1.0)
    picked = sorted(set(int(e) for e in idx.ravel()))
    # canonical weights of the picked experts only (the other 247 are never read by a step)
    experts = {}
    for e in picked + [E]:
        t = []
        for m in range(3):
            N, K = (H, I) if m == 2 else (I, H)
            g = torch.Generator().manual_seed(SEED * 1000003 + e * 3 + m)
            q, s = synth.quant_fp8_128(torch.randn(N, K, generator=g) * 0.02)
            t += [q.numpy(), s.numpy()]
        experts[e] = tuple(t)
    shared = experts.pop(E)

    def one():
        lg = orc.router_logits(xb, wr)
        ii, ww = orc.route(lg, None, topk, 0, CFG["n_group"], CFG["topk_group"], True, 1.0)
        return orc.moe_fp8_layer(xb, ii, ww, experts, shared)

    for _ in range(max(1, min(args.warmup, 2))):
        one()
    steps = max(1, args.steps)
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    dt = (time.perf_counter() - t0) / steps
    us = dt * 1e6
    cores = orc.num_threads()
    line = {
        "impl": "reference", "metric": "moe_decode_layer_step_us", "value": us, "unit": "us", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp8_e4m3 (f32 accumulate)", "data": "synthetic",
        "config": {"workload": workload_name(rows), "rows": rows},
        "cpu_baseline": {"value": us, "unit": "us", "cores": cores, "kind": "port",
                         "sample": f"{steps} whole layer-steps ({rows} row(s), {len(picked)} experts + shared) through "
                                   "the C oracle (OpenMP)"},
        "e2e": {"value": us, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tokens_per_s": rows / dt,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------------- GPU arm

def dist_setup():
    """(world, rank, local rank, device); the process group is created once, on the first call."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this library has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    return world, rank, local, dev


def shared_part(rank, world, I):
    """The shared expert's intermediate channels of a rank: parts of whole 512-channel pieces, one a rank while they last."""
    if world == 1:
        return 0, I
    n = max(512, (I // world + 511) // 512 * 512)
    lo = rank * n
    return (lo, min(I, lo + n)) if lo < I else None


def parity_rule(got, want, pm):
    """The tests' rule on one step's rounded rows: within 2e-3 of the row maximum; what is left beyond that must be one
    bf16 rounding flip of one added output (pm) or of the final rounding.  Returns (ok, max error, elements beyond 2e-3)."""
    import numpy as np
    got, want, pm = (np.asarray(a, np.float64) for a in (got, want, pm))
    den = np.abs(want).max(axis=1, keepdims=True)
    den = np.where(den == 0, 1.0, den)
    diff = np.abs(got - want)
    ulp = lambda v: 2.0 ** (np.floor(np.log2(np.maximum(np.abs(v), 2.0 ** -126))) - 7)
    allow = 2e-3 * den + ulp(pm) + ulp(want)
    beyond = int((diff > 2e-3 * den).sum())
    return bool((diff <= allow).all() and beyond <= max(1, int(0.02 * diff.size))), float((diff / den).max()), beyond


def run_gpu(args, rows=None, steps=None, with_kernel=True, with_cpu=True):
    """One decode workload (the shapes in CFG) on this rank's GPU; returns rank 0's result line (None on other ranks)."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from dsgx10_b200 import _lib, moe, synth

    world, rank, local, dev = dist_setup()
    _lib.lib()
    rows = args.rows if rows is None else rows
    n_steps = args.steps if steps is None else steps

    H, I, E, topk = CFG["H"], CFG["I"], CFG["E"], CFG["topk"]
    e_lo, e_hi = rank * E // world, (rank + 1) * E // world
    int4, mx4 = CFG["fmt"] == "int4", CFG["fmt"] == "mx4"
    # several GPUs: contiguous expert ranges; an FP8 layer's shared expert is cut into parts of its intermediate channels,
    # one a rank (the INT4 layers' bf16 shared expert stays whole, on rank 0)
    part = (0, I) if world == 1 else (shared_part(rank, world, I) if not int4 else ((0, I) if rank == 0 else None))
    shp = moe.shape(H, I, E, topk, fmt=_lib.FMT_INT4 if int4 else _lib.FMT_MXFP4 if mx4 else _lib.FMT_FP8, n_group=CFG["n_group"],
                    topk_group=CFG["topk_group"], score_fn=CFG["score_fn"], e_lo=e_lo, e_hi=e_hi,
                    sh_lo=part[0] if (part and world > 1 and not int4) else 0,
                    sh_hi=part[1] if (part and world > 1 and not int4) else 0)
    NL, NX = args.layers, 16
    layers, steps_buf = [], []
    for l in range(NL):
        if int4:
            lay = synth.Int4Layer.on_device(H, I, E, SEED + 7919 * l, dev, shared=part is not None, e_range=(e_lo, e_hi))
        else:
            lay = (synth.Mx4Layer if mx4 else synth.Fp8Layer)(H, I, E, SEED + 7919 * l, device=dev, shared=part is not None,
                                                              e_range=(e_lo, e_hi))
        wr = synth.router_weights(E, H, SEED + 2000 + l, device="cpu").to(dev)
        layers.append((lay, lay.layer_w()))
        steps_buf.append(moe.LayerStep(shp, wr, None, device=dev, fused=False if args.separate else True if args.fused else None))
    xs = [synth.activations(rows, H, SEED + 1000 + i, device="cpu").to(dev) for i in range(NX)]
    xs_host = [x.cpu().pin_memory() for x in xs]
    out_host = torch.empty(rows, H, dtype=torch.bfloat16).pin_memory()
    red = torch.zeros(2, _lib.MAX_ROWS, H, dtype=torch.float32, device=dev) if world > 1 else None
    # several GPUs: the partial sums are reduced and rounded by the library's kernel over peer memory (--nccl: by an
    # NCCL all-reduce and the rounding kernel); the buffer half follows the step parity, so the graph holds an even count
    peer = None
    if world > 1 and not args.nccl:
        from dsgx10_b200 import ep
        peer = ep.PeerReduce(H, shared_rank=0 if int4 else -2)
        n_steps += n_steps & 1

    def step(i, host=False):
        lay, lw = layers[i % NL]
        sb = steps_buf[i % NL]
        if world == 1:
            if host:
                sb.run_host(lw, xs_host[i % NX], out_host)
                return out_host
            return sb.run(lw, xs[i % NX])
        x = xs[i % NX]
        if host and peer is None:
            sb.x_stage[:rows].copy_(xs_host[i % NX], non_blocking=True)
            x = sb.x_stage[:rows]
        if peer is not None:
            yr_p, ys_p = peer.parts(peer.launched + 1)
            if host:  # host buffers in place: copy-in kernel, partial sums, then the reduction writes the pinned rows
                sb.run_host(lw, xs_host[i % NX], None, yr=yr_p, ys=ys_p)
                return peer.finalize(rows, out=out_host)
            sb.run(lw, x, finalize=False, yr=yr_p, ys=ys_p)
            return peer.finalize(rows)
        sb.run(lw, x, finalize=False)
        red[0].copy_(sb.yr)
        if part is not None:
            red[1].copy_(sb.ys)
        else:
            red[1].zero_()
        dist.all_reduce(red)
        out = moe.finalize(red[0, :rows], red[1, :rows].to(torch.bfloat16).float())
        if host:
            out_host.copy_(out, non_blocking=True)
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        """Device time of exactly n steps.  One GPU: the n steps are captured in one CUDA graph (as a serving engine
        replays its step graph; the reference benches a graph of 64 steps, altar1
        engine/experts/tests/bench_experts.cu:46-82) and the replay is timed; with several GPUs the NCCL all-reduce is
        captured in the same graph."""
        graph = None
        if not args.eager:
            barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(n):
                    fn(i)
            graph.replay()  # one untimed replay (the launches the capture counted)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if graph is not None:
            graph.replay()
            if peer is not None:
                peer.launched += n  # a second run of the captured steps
        else:
            for i in range(n):
                fn(i)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for i in range(max(args.warmup, 3)):
        step(i)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(lambda i: step(i), n_steps)
    # end to end: host buffers in, host buffer out, copies inside the timed region
    for i in range(4):
        step(i, host=True)
    ms_e2e = timed(lambda i: step(i, host=True), n_steps)

    # the dominant kernel (gate/up stream) alone, for the roofline: same cold-weight rotation
    union = []
    for i in range(NL):
        sb = steps_buf[i]
        union.append(len(set(sb.idx[:rows].flatten().tolist()) & set(range(e_lo, e_hi))))

    # (FP8: the kernel alone, hook 5, over the table and quantised rows that one hook-1 call a layer leaves in the
    # workspace; INT4: with its preparation launch)
    def up_only(i, parts=1 if int4 else 5):
        lay, lw = layers[i % NL]
        sb = steps_buf[i % NL]
        moe.moe_decode(shp, lw, xs[i % NX], sb.idx, sb.w, sb.ws, sb.yr, sb.ys, parts=parts)
    ms_up = None
    if with_kernel:
        for i in range(NL):
            up_only(i, parts=1)
        for i in range(3):
            up_only(i)
        ms_up = timed(up_only, n_steps)
    clocks = sampler.stop() if rank == 0 else None
    status = max(moe.ws_status(sb.ws) for sb in steps_buf)
    if peer is not None:
        status = max(status, int(peer.status.item()))

    # ---- one step's rounded rows against the CPU oracle (outside every timed region; the oracle is only the checker):
    # every rank runs the oracle over its own experts, the partial sums are added across the ranks
    parity = None
    if not int4 and not args.no_parity:
        from oracle import oracle as orc
        got = step(0)
        torch.cuda.synchronize()
        got = got.float().cpu().numpy()
        sb, lay = steps_buf[0], layers[0][0]
        idx_np, w_np = sb.idx[:rows].cpu().numpy(), sb.w[:rows].cpu().numpy()
        mine = {int(e): lay.canonical(int(e)) for e in np.unique(idx_np) if e_lo <= e < e_hi}
        if not mine:
            mine = {e_lo: lay.canonical(e_lo)}   # (an expert no row picked: it gives the shapes, nothing is computed)
        sh = lay.canonical(E) if rank == 0 else None
        acc, _, pm = orc.moe_fp8_layer(synth.bf16_bits(xs[0]), idx_np, w_np, mine, sh, e_lo=e_lo, e_hi=e_hi,
                                       with_shared=rank == 0, pickmax=True, mx4=mx4)
        acc_t, pm_t = torch.from_numpy(acc).to(dev), torch.from_numpy(pm).to(dev)
        if world > 1:
            dist.all_reduce(acc_t)
            dist.all_reduce(pm_t, op=dist.ReduceOp.MAX)
        ok, err, beyond = parity_rule(got, acc_t.cpu().numpy(), pm_t.cpu().numpy())
        parity = {"ok": ok, "max_err_of_row_max": err, "elements_beyond_2e-3": beyond, "rows": rows,
                  "against": "the CPU oracle on the picked experts (every rank its own, partial sums added)"}

    if int4 and not args.no_parity and world == 1:
        # INT4: the timed layers are generated straight in the block layout on the device and keep no canonical tensors, so
        # the check runs one step over a layer packed from canonical tensors (the experts these rows pick, the same router)
        from oracle import oracle as orc
        sb = steps_buf[0]
        rc = min(rows, 2)  # (rows checked: packing an expert's canonical tensors on the host takes a second each)
        picked = sorted(set(int(e) for e in moe.route(shp, moe.router_logits(xs[0][:rc], sb.wr), None)[0].flatten().tolist()))
        chk = synth.Int4Layer(H, I, E, SEED + 99, device=dev, experts=picked)
        st = moe.LayerStep(shp, sb.wr, None, device=dev)
        got = st.run(chk.layer_w(), xs[0][:rc])
        torch.cuda.synchronize()
        idx_np, w_np = st.idx[:rc].cpu().numpy(), st.w[:rc].cpu().numpy()
        deq = {e: tuple(orc.int4_dequant(wp, s_, None) for wp, s_ in chk.raw[e]) for e in picked}
        acc, _ = orc.moe_bf16w_layer(synth.bf16_bits(xs[0][:rc]), idx_np, w_np, deq, tuple(chk.sh_bits))
        ok, err, beyond = parity_rule(got.float().cpu().numpy(), acc, np.zeros_like(acc))
        ok = ok and sorted(set(idx_np.ravel().tolist())) == picked and moe.ws_status(st.ws) == 0
        parity = {"ok": ok, "max_err_of_row_max": err, "elements_beyond_2e-3": beyond, "rows": rc,
                  "against": "the CPU oracle (dequantised INT4 experts, bf16 shared expert) on a layer packed from canonical "
                             "tensors: the picked experts, the same router and rows"}

    if rank != 0:
        return None
    peaks, peak_kind = measured_peaks()
    us = ms * 1e3 / n_steps
    us_e2e = ms_e2e * 1e3 / n_steps
    # distinct experts a step touches (all ranks): from the routed ids of the last steps (all ranks route identically)
    tot_union = sum(len(set(sb.idx[:rows].flatten().tolist())) for sb in steps_buf) / NL
    sb_bytes = step_bytes(tot_union, rows)
    line = {
        "metric": "moe_decode_layer_step_us", "value": us, "unit": "us", "n_gpus": world, "steps": n_steps,
        "warmup": max(args.warmup, 3), "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "int4-g32 weights, bf16 activations (f32 accumulate)" if int4 else
                                      "mxfp4 weights, fp8_e4m3 activations (f32 accumulate)" if mx4 else "fp8_e4m3 (f32 accumulate)",
        "data": "synthetic",
        "config": {"workload": workload_name(rows), "rows": rows,
                   "parallelism": f"ep{world}" + ("" if world == 1 else " (NCCL all-reduce)" if peer is None else
                                                   " (partial sums reduced over peer memory by k_finalize_peers; the shared "
                                                   "expert in parts across the ranks)"),
                   "cold_weights": f"{NL} layers x 16 activations cycled; inputs larger than L2",
                   "launch": "eager" if args.eager else "one CUDA graph of the timed steps"},
        "tokens_per_s": rows / (us * 1e-6),
        "step_hbm_gbs": sb_bytes / (us * 1e-6) / 1e9,
        "step_frac_of_measured_hbm": sb_bytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"],
        "step_frac_of_8tbs": sb_bytes / (us * 1e-6) / 1e9 / 8000.0,
        "step_algorithmic_bytes": sb_bytes,
        "e2e": {"value": us_e2e, "unit": "us", "h2d_bytes_per_step": rows * H * 2, "d2h_bytes_per_step": rows * H * 2},
        # this library's kernels a step: the one persistent kernel from three rows (or --fused), else front, routing, gate/up,
        # down; with several GPUs also the reduction kernel
        "gpu_launches": n_steps * ((1 if (args.fused or (rows >= 3 and not args.separate and not int4 and world == 1)) else 4)
                                   + (1 if world > 1 else 0)),
        "clocks": clocks,
        "device_status": status,
        "parity": parity,
    }
    if ms_up is not None:
        us_up = ms_up * 1e3 / n_steps
        sh_frac = ((part[1] - part[0]) / I) if part else 0.0
        upb = sum(up_bytes(u, sh_frac) for u in union) / NL  # this rank's picked experts + its part of the shared one
        ach = upb / (us_up * 1e-6) / 1e9
        line["roofline"] = {"bound": "hbm", "kernel": ("k_up_i4 (+ activation staging launch)" if int4 else "k_up_fp8"),
                            "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                            "peak_kind": peak_kind, "us_per_launch": us_up, "algorithmic_bytes": upb,
                            # one ncu capture of this kernel (its summary is among the committed profiles): 151.14 MB read +
                            # 3.91 MB written for 151.03 MB algorithmic; the traffic grows with the experts a launch streams
                            "traffic": None if (int4 or mx4) else upb * (151.142912 + 3.909120) / 151.031808,
                            "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of a 9-expert launch, scaled by "
                                              "this launch's algorithmic bytes"}
    if with_cpu and not args.no_cpu_baseline and world == 1 and not int4 and not mx4:
        line["cpu_baseline"] = cpu_baseline(rows, workload=args.workload)
    return line


# ------------------------------------------------------------------------------------------- prefill workload (GPU)

PF = dict(H=2048, I=1024, E=64, topk=6)   # the small layer's shapes: 16384 tokens, Zipf(1.1) expert popularity


def prefill_flops(T):
    """Useful FLOPs of the expert pass: every pick and the shared expert through three H x I matrices."""
    return T * (PF["topk"] + 1) * 3 * PF["H"] * PF["I"] * 2


def run_prefill_reference(args):
    """The oracle port on the host cores over a bounded sample of the same token stream (64 tokens a step)."""
    import numpy as np
    from dsgx10_b200 import synth
    from oracle import oracle as orc
    if int(os.environ.get("RANK", "0")) != 0:
        return
    orc.set_threads()
    H, I, E, topk = PF["H"], PF["I"], PF["E"], PF["topk"]
    Ts = 64
    lay = synth.Fp8Layer(H, I, E, SEED, device="cpu")
    x = synth.bf16_bits(synth.activations(Ts, H, SEED + 1000))
    wr = synth.router_weights(E, H, SEED + 2000).numpy()
    experts = {e: lay.canonical(e) for e in range(E)}
    shared = lay.canonical(E)

    def one():
        lg = orc.router_logits(x, wr)
        ii, ww = orc.route(lg, None, topk, 0, 1, 1, True, 1.0)
        picked = {int(e) for e in ii.ravel()}
        return orc.moe_fp8_layer(x, ii, ww, {e: experts[e] for e in picked}, shared)

    one()
    steps = max(1, args.steps)
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    dt = (time.perf_counter() - t0) / steps
    tf = prefill_flops(Ts) / dt / 1e12
    line = {
        "impl": "reference", "metric": "moe_prefill_grouped_gemm_tflops", "value": tf, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": 1, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 (f32 accumulate)", "data": "synthetic",
        "config": {"workload": "config 4: prefill MoE, hidden 2048, 64 experts x 1024, top-6, + shared expert", "tokens": Ts},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": orc.num_threads(), "kind": "port",
                         "sample": f"{steps} passes of {Ts} tokens through the C oracle (OpenMP)"},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tokens_per_s": Ts / dt,
    }
    print(json.dumps(line), flush=True)


def run_prefill(args, workload=None, steps=None, with_cpu=True, a2a=False):
    """Config 4: one layer's prefill over `--tokens` tokens whose expert popularity follows Zipf(1.1) (a router bias
    calibrated so that the realised pick histogram matches), experts sharded over the ranks, partial sums reduced over
    peer memory.  Config 5 (`ragged`): the mixed batch through the same pass.  a2a (several GPUs): the rows are partitioned
    over the ranks instead, every rank routes its own rows, an all-to-all (NCCL) sends each row to the ranks that own one
    of its picks, the f32 partial sums return by a second all-to-all and are added in rank order; the shared expert runs
    on the rows' own rank.  Returns rank 0's result line."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from dsgx10_b200 import _lib, moe, synth

    world, rank, local, dev = dist_setup()
    _lib.lib()
    workload = args.workload if workload is None else workload
    n_steps = args.steps if steps is None else steps
    H, I, E, topk = PF["H"], PF["I"], PF["E"], PF["topk"]
    T = args.tokens
    ragged = workload == "ragged"
    if ragged:  # config 5: 64 requests packed into one token-sorted pass: 40 decode rows, 16 verify rows, 8 prefill chunks
        rng = np.random.default_rng(SEED + 5)
        reqs = [1] * 40 + [int(v) for v in rng.integers(2, 7, 16)] + [int(v) for v in rng.integers(512, 4097, 8)]
        T = sum(reqs)
    e_lo, e_hi = rank * E // world, (rank + 1) * E // world
    shp_all = moe.shape(H, I, E, topk)
    shp = moe.shape(H, I, E, topk, e_lo=e_lo, e_hi=e_hi)
    a2a = a2a and world > 1
    lay = synth.Fp8Layer(H, I, E, SEED, device=dev, shared=(rank == 0) and not a2a, e_range=(e_lo, e_hi))
    NX = 3  # distinct activation sets: 3 x 67 MB of inputs, and ~1.5 GB of intermediates a pass: nothing stays in L2
    xs = [synth.activations(T, H, SEED + 1000 + i, device="cpu").to(dev) for i in range(NX)]
    xs_host = [x.cpu().pin_memory() for x in xs]
    out_host = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
    wr = synth.router_weights(E, H, SEED + 2000, device="cpu").to(dev)
    logits0 = moe.router_logits(xs[0], wr)

    def counts_for(b):
        idx, _ = moe.route(shp_all, logits0, torch.from_numpy(b).to(dev))
        return torch.bincount(idx.flatten().long(), minlength=E).cpu().numpy()
    if ragged:  # no popularity skew is asked for: the router's own picks
        alpha, b = 0.0, np.zeros(E, np.float32)
        counts = counts_for(b)
    else:
        alpha, b, counts = synth.calibrate_zipf_bias(counts_for, E, topk, SEED + 7)
    bias = torch.from_numpy(b).to(dev)
    pl = moe.PrefillLayer(shp, lay.layer_w(), T, device=dev)
    routed = []
    for x in xs:
        lg = moe.router_logits(x, wr)
        routed.append(moe.route(shp_all, lg, bias))
    f32 = dict(dtype=torch.float32, device=dev)
    yr, ys = torch.empty(T, H, **f32), torch.zeros(T, H, **f32)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    x_stage = torch.empty(T, H, dtype=torch.bfloat16, device=dev)

    # several GPUs: rank 0 adds the shared expert's output into its partial sums; the partial sums are written into
    # symmetric memory and one kernel a GPU adds them over NVLink and rounds (--nccl: an NCCL all-reduce instead)
    peer = None
    if world > 1 and not args.nccl:
        from dsgx10_b200 import ep
        # two GPUs: each reads the other's whole partial sums; more: each reduces 1 / N of the rows and stores them everywhere
        peer = ep.PeerReduce(H, rows_cap=T, shared_rank=-1, sliced=world > 2)

    if a2a:  # the shared expert of this rank's own rows: a layer with no routed expert, only the shared one
        from dsgx10_b200 import ep
        peer = None
        r_lo, r_hi = rank * T // world, (rank + 1) * T // world
        lay_sh = synth.Fp8Layer(H, I, E, SEED, device=dev, shared=True, e_range=(0, 0))
        pl_sh = moe.PrefillLayer(moe.shape(H, I, E, topk, e_lo=0, e_hi=0), lay_sh.layer_w(), r_hi - r_lo, device=dev)
        out_all = torch.empty(T, H, dtype=torch.bfloat16, device=dev)

        def local_routed(xr, ir, wr_):
            y, _, _ = pl.run(xr, ir, wr_, ys=False, out=False)
            return y

    def experts(i):
        idx, w = routed[i % NX]
        if a2a:
            x_loc, idx_loc, w_loc = xs[i % NX][r_lo:r_hi], idx[r_lo:r_hi].contiguous(), w[r_lo:r_hi].contiguous()
            acc = ep.all_to_all_experts(x_loc, idx_loc, w_loc, E, local_routed)
            _, ysh, _ = pl_sh.run(x_loc, idx_loc, w_loc, out=False)   # (its routed partial sums are zero: no expert)
            return moe.finalize(acc, ysh)     # this rank's rows
        if peer is not None:
            yr_p, _ = peer.parts(peer.launched + 1)
            pl.run(xs[i % NX], idx, w, yr=yr_p, ys=False, out=False, ysum=True)
            peer.finalize(T, out=None if peer.sliced else out)   # (sliced: the rounded rows land in peer.out on every rank)
            return peer.out if peer.sliced else out
        # one GPU: only the rounded rows; several: the f32 partial sums for the reduction
        pl.run(xs[i % NX], idx, w, yr=yr if world > 1 else False, ys=ys if world > 1 else False, out=out, ysum=world > 1)
        if world > 1:  # rank 0's partial sums hold the shared expert's output too: one buffer to reduce
            dist.all_reduce(yr)
            out.copy_(moe.finalize(yr))
        return out

    # end to end: host activations in, router, experts, host bf16 out; the pass is cut into chunks of tokens that go
    # round two streams (each with its own workspace), so that the copies of one chunk overlap the kernels of another
    NCH = args.chunks if T % args.chunks == 0 and T >= 4096 else 1
    TC = T // NCH
    NS = 3 if NCH > 2 else 2
    streams = [torch.cuda.Stream(device=dev) for _ in range(NS)]
    pls = [pl] + [moe.PrefillLayer(shp, lay.layer_w(), TC, device=dev, wbuf=pl.wbuf) for _ in range(NS - 1)] if NCH > 1 else [pl]

    def whole(i):
        xh = xs_host[i % NX]
        cur = torch.cuda.current_stream()
        for s in streams:
            s.wait_stream(cur)
        for c in range(NCH):
            s, p2 = streams[c % NS], pls[c % len(pls)]
            lo, hi = c * TC, (c + 1) * TC
            with torch.cuda.stream(s):
                x_stage[lo:hi].copy_(xh[lo:hi], non_blocking=True)
                lg = moe.router_logits(x_stage[lo:hi], wr)
                idx, w = moe.route(shp_all, lg, bias)
                p2.run(x_stage[lo:hi], idx, w, yr=yr[lo:hi] if world > 1 else False, ys=ys[lo:hi] if world > 1 else False,
                       out=out[lo:hi], ysum=world > 1)
                if world > 1:  # (the chunked end-to-end pipeline keeps the NCCL reduction: one reduction a chunk and stream)
                    dist.all_reduce(yr[lo:hi])
                    out[lo:hi].copy_(moe.finalize(yr[lo:hi]))
                out_host[lo:hi].copy_(out[lo:hi], non_blocking=True)
        for s in streams:
            cur.wait_stream(s)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            fn(i)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / n

    W = max(args.warmup, 3)
    for i in range(W):
        experts(i)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(experts, n_steps)
    if a2a:
        ms_e2e = ms   # (no separate end-to-end leg for this scheme: the sub-record carries the device-timed pass)
    else:
        for i in range(3):
            whole(i)
        ms_e2e = timed(whole, max(2, n_steps // 2))
    # the dominant kernel alone: the routed gate/up grouped GEMM over the operands the last pass left in the workspace
    idx, w = routed[(n_steps - 1) % NX]
    pl.run(xs[(n_steps - 1) % NX], idx, w, yr=yr, ys=ys, out=out)
    up = lambda i: pl.run(xs[0], idx, w, yr=yr, ys=ys, out=out, parts=1)
    for i in range(3):
        up(i)
    ms_up = timed(up, n_steps)
    clocks = sampler.stop() if rank == 0 else None
    status = moe.ws_status(pl.ws)
    # ---- sampled rows of one pass against the CPU oracle (outside the timed regions; the oracle is only the checker)
    parity = None
    if not args.no_parity:
        from oracle import oracle as orc
        idx0, w0 = routed[0]
        got = experts(0)
        if a2a:  # every rank holds its own rows: gathered for the check
            parts = [torch.empty((r + 1) * T // world - r * T // world, H, dtype=torch.bfloat16, device=dev) for r in range(world)]
            dist.all_gather(parts, got.contiguous())
            got = torch.cat(parts)
        torch.cuda.synchronize()
        rows_s = np.unique(np.concatenate([[0, T - 1], np.random.default_rng(3).integers(0, T, 14)]))
        got = got[torch.from_numpy(rows_s).to(dev)].float().cpu().numpy()
        idx_np, w_np = idx0.cpu().numpy()[rows_s], w0.cpu().numpy()[rows_s]
        mine = {int(e): lay.canonical(int(e)) for e in np.unique(idx_np) if e_lo <= e < e_hi}
        if not mine:
            mine = {e_lo: lay.canonical(e_lo)}
        sh_lay = lay_sh if a2a else lay
        acc, _, pm = orc.moe_fp8_layer(synth.bf16_bits(xs[0])[rows_s], idx_np, w_np, mine, sh_lay.canonical(E) if rank == 0 else None,
                                       e_lo=e_lo, e_hi=e_hi, with_shared=rank == 0, pickmax=True)
        acc_t, pm_t = torch.from_numpy(acc).to(dev), torch.from_numpy(pm).to(dev)
        if world > 1:
            dist.all_reduce(acc_t)
            dist.all_reduce(pm_t, op=dist.ReduceOp.MAX)
        ok, err, beyond = parity_rule(got, acc_t.cpu().numpy(), pm_t.cpu().numpy())
        parity = {"ok": ok, "max_err_of_row_max": err, "elements_beyond_2e-3": beyond, "rows": int(len(rows_s)),
                  "against": "the CPU oracle on sampled rows (every rank its own experts, partial sums added)"}
    if rank != 0:
        return None
    peaks, peak_kind = measured_peaks()
    local_picks = int(counts[e_lo:e_hi].sum())
    fl_up = local_picks * 2 * H * I * 2
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    ach = fl_up / (ms_up * 1e-3) / 1e12
    tf = prefill_flops(T) / (ms * 1e-3) / 1e12
    tf_e2e = prefill_flops(T) / (ms_e2e * 1e-3) / 1e12
    c = np.sort(counts)[::-1]
    line = {
        "metric": "moe_prefill_grouped_gemm_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": world, "steps": n_steps,
        "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp8_e4m3 (f32 accumulate)", "data": "synthetic",
        "config": {"workload": (f"config 5: ragged batch of 64 requests (40 x 1, 16 x 2-6, 8 x 512-4096 tokens) in one pass, "
                                f"hidden 2048, 64 experts x 1024, top-6, + shared expert, {T} tokens" if ragged else
                                f"config 4: prefill MoE, hidden 2048, 64 experts x 1024, top-6, + shared expert, {T} tokens, "
                                f"Zipf(1.1) expert popularity (router bias scale {alpha})"), "tokens": T,
                   "segments": {"max": int(c[0]), "median": int(np.median(c)), "min": int(c[-1])},
                   "parallelism": f"ep{world}" + ("" if world == 1 else
                                                   " (rows partitioned; NCCL all-to-all dispatch of rows to the ranks that own "
                                                   "a pick, all-to-all return of f32 partial sums)" if a2a else
                                                   " (NCCL all-reduce)" if peer is None else
                                                   " (partial sums reduced over peer memory by k_finalize_peers)"),
                   "cold_inputs": f"{NX} activation sets cycled; inputs and intermediates larger than L2",
                   "step": "sort/permute + quantise + gate/up GEMM (SwiGLU) + down GEMM + shared expert + combine",
                   "e2e": f"{NCH} chunks of {TC} tokens over {NS} streams: copy in, router, expert pass, copy out"},
        "tokens_per_s": T / (ms * 1e-3),
        "roofline": {"bound": "tensor", "kernel": "k_gemm_fp8<up> (routed gate/up grouped GEMM, SwiGLU and h quantisation fused)",
                     "achieved": ach, "peak": fp8_peak, "unit": "TFLOP/s", "frac": ach / fp8_peak,
                     "peak_kind": f"2 x {peak_kind} bf16 burst (no FP8 figure is measured on this pool)",
                     "frac_of_nominal_4500": ach / 4500.0, "us_per_launch": ms_up * 1e3, "algorithmic_flops": fl_up,
                     "traffic": None},
        "e2e": {"value": tf_e2e, "unit": "TFLOP/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": T * H * 2,
                "d2h_bytes_per_step": T * H * 2},
        "gpu_launches": n_steps * (11 + (1 if world > 1 else 0)),
        "clocks": clocks,
        "device_status": status,
        "parity": parity,
    }
    if with_cpu and not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_baseline(1, workload="prefill")
    return line


def cpu_baseline(rows, workload="decode"):
    """The oracle port on the host cores, a bounded sample: ten whole layer-steps of the same workload."""
    r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", "10", "--warmup", "1",
                        "--rows", str(rows), "--workload", workload], capture_output=True, text=True, timeout=600)
    try:
        d = json.loads(r.stdout.strip().splitlines()[-1])
        return d["cpu_baseline"]
    except Exception as ex:  # report, do not hide
        return {"value": None, "unit": "us", "cores": os.cpu_count(), "kind": "port", "sample": f"failed: {ex}: {r.stderr[-300:]}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--workload", default="decode", choices=["decode", "decode1", "int4", "mx4", "prefill", "ragged"],
                    help="decode: the headline layer-step (config 2); decode1: the small layer's step (config 1); int4: "
                         "config 3; mx4: config 2's shapes with MXFP4 routed experts; prefill: the grouped GEMM pass of config 4; ragged: the mixed batch of config 5 "
                         "through the same pass")
    ap.add_argument("--tokens", type=int, default=16384, help="prefill: tokens a pass")
    ap.add_argument("--chunks", type=int, default=4, help="prefill end to end: chunks of tokens the pass is cut into")
    ap.add_argument("--layers", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    dv = ap.add_argument_group("development switches (profiling and A/B runs; none belongs to the benchmark contract)")
    dv.add_argument("--eager", action="store_true", help="no CUDA graph: launch every kernel from the host")
    dv.add_argument("--nccl", action="store_true", help="several GPUs: reduce with an NCCL all-reduce instead of the peer kernel")
    dv.add_argument("--separate", action="store_true", help="always run the step as four kernels")
    dv.add_argument("--fused", action="store_true", help="always run the step as the one persistent kernel")
    dv.add_argument("--experts", type=int, default=0,
                    help="a layer with fewer routed experts (same matrices), to keep an ncu capture small")
    ap.add_argument("--no-parity", action="store_true", help="skip the check of one step's rows against the CPU oracle")
    ap.add_argument("--no-others", action="store_true",
                    help="the headline workload only (default: the other configurations follow, briefly, as sub-records)")
    args = ap.parse_args()

    def select(workload):
        """CFG and the layer count of a decode workload."""
        CFG.update(CFG_BIG)
        layers = args.layers
        if workload == "decode1":  # config 1: the same decode bench over the small FP8 layer
            CFG.update(CFG_SMALL)
            layers = 12 if args.layers == 3 else args.layers  # 12 x 50 MB of picked experts between reuses: larger than L2
        if workload == "int4":  # config 3: the same decode bench over an INT4-g32 layer
            CFG.update(CFG_INT4)
            layers = 2 if args.layers == 3 else args.layers
        if workload == "mx4":
            CFG.update(CFG_MX4)
        if args.experts:
            CFG["E"] = args.experts
        return layers

    if args.workload in ("prefill", "ragged") and args.steps == 200:
        args.steps = 20
    if args.impl == "reference":
        args.layers = select(args.workload)
        run_prefill_reference(args) if args.workload in ("prefill", "ragged") else run_reference(args)
        return

    import copy
    import gc

    def one(workload, rows, steps, brief):
        """A workload's line; brief: a sub-record (fewer steps, no CPU leg), cut down to its figures."""
        import torch
        a = copy.copy(args)
        a.workload = workload
        if workload in ("prefill", "ragged", "ragged_a2a"):
            line = run_prefill(a, workload="ragged" if workload == "ragged_a2a" else workload, steps=steps, with_cpu=not brief,
                               a2a=workload == "ragged_a2a")
        else:
            a.layers = select(workload)
            line = run_gpu(a, rows=rows, steps=steps, with_kernel=True, with_cpu=not brief)
        gc.collect()
        torch.cuda.empty_cache()
        if line is None or not brief:
            return line
        keep = {k: line[k] for k in ("metric", "value", "unit", "ms_per_step", "tokens_per_s", "step_frac_of_measured_hbm",
                                     "device_status", "parity") if k in line}
        keep["workload"] = line["config"]["workload"]
        keep["e2e"] = line["e2e"]["value"]
        if "roofline" in line:
            keep["roofline"] = {k: line["roofline"][k] for k in ("kernel", "achieved", "unit", "frac", "us_per_launch")}
        keep["clocks"] = line["clocks"]
        return keep

    head = one(args.workload, args.rows, args.steps, brief=False)
    others = {}
    default_run = args.workload == "decode" and args.rows == 1 and not (args.no_others or args.eager or args.experts
                                                                        or args.separate or args.fused or args.nccl)
    if default_run:
        world = int(os.environ.get("WORLD_SIZE", "1"))
        plan = [("config2_rows8", "decode", 8, 30)]
        if world == 1:
            plan += [("config1_rows1", "decode1", 1, 60), ("mxfp4_rows1", "mx4", 1, 30), ("mxfp4_rows4", "mx4", 4, 20),
                     ("config3_int4_rows1", "int4", 1, 30),
                     ("config3_int4_rows4", "int4", 4, 20), ("config4_prefill_16384", "prefill", 1, 6),
                     ("config5_ragged_batch", "ragged", 1, 6)]
        else:
            plan += [("config4_prefill_16384", "prefill", 1, 6), ("config5_ragged_batch_all_to_all", "ragged_a2a", 1, 6)]
        for name, wl, rows, steps in plan:
            try:
                others[name] = one(wl, rows, steps, brief=True)
            except Exception as ex:  # a sub-record that fails is reported, the headline stands
                others[name] = {"error": f"{type(ex).__name__}: {ex}"[:300]}
    if head is not None:
        if others:
            head["others"] = others
        print(json.dumps(head), flush=True)
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
