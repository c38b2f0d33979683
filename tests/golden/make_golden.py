#!/usr/bin/env python
"""Generates tests/golden/*.npz by running the reference's own Python CPU modules on small seeded layers.

Run in a container that has the reference tree (its location: the environment variable DSGX_REFERENCE); the fixtures it writes are committed, this
script is how they were made.  Nothing of the reference is copied: its modules are imported from where they lie.

  FP8:  ds41f ref/inference/model.py (Gate, Expert, MoE) over ref/torchref/kernel.py, switched to the "g128" recipe the
        benchmark configurations name: fp8_block_size 128, f32 scales (scale_fmt None), default dtype bf16.
  INT4: altar1 ref/glmref.py (int4_dequant, moe) with its module constants set to the small shape.
  group-limited routing: transformers' GlmMoeDsa routing function, which altar1 docs/model.md names as the definition.

Weights are not stored: the tests rebuild them from the same seeds (dsgx10_b200.synth, CPU generator) and check a
checksum kept in the fixture, so a fixture only holds activations, routing and outputs (a few KB).
"""
import os
import sys
import zlib
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = os.environ.get("DSGX_REFERENCE")
if not REF:
    raise SystemExit("set DSGX_REFERENCE to the reference project's directory")

from dsgx10_b200 import synth  # noqa: E402


def crc(*arrays):
    c = 0
    for a in arrays:
        c = zlib.crc32(np.ascontiguousarray(a).tobytes(), c)
    return np.uint32(c)


# ------------------------------------------------------------------------------------------------------------- FP8

def fp8_case(name, H, I, E, topk, T, score, seed, route_scale=1.0, swiglu_limit=0.0, x_scale=1.0, mx4=False):
    """mx4: the routed experts in ds41f's own format (expert_dtype "fp4": e2m1 with a ue8m0 scale per 32), the shared
    expert FP8."""
    sys.path[:0] = [os.path.join(REF, "ds41f-4xgx10-switchless/ref/torchref"),
                    os.path.join(REF, "ds41f-4xgx10-switchless/ref/inference")]
    import model as M  # the reference's model.py; `kernel` resolves to torchref/kernel.py
    M.fp8_block_size, M.scale_fmt, M.scale_dtype = 128, None, torch.float32
    M.default_dtype = torch.float8_e4m3fn
    M.world_size, M.rank = 1, 0
    torch.set_default_dtype(torch.bfloat16)
    try:
        args = M.ModelArgs(dim=H, moe_inter_dim=I, n_routed_experts=E, n_activated_experts=topk, score_func=score,
                           route_scale=route_scale, expert_dtype="fp4" if mx4 else None, n_layers=1,
                           swiglu_limit=swiglu_limit)
        moe = M.MoE(0, args)
    finally:
        torch.set_default_dtype(torch.float32)
    layer = (synth.Mx4Layer if mx4 else synth.Fp8Layer)(H, I, E, seed, device="cpu")
    wr = synth.router_weights(E, H, seed + 2000)
    x = synth.activations(T, H, seed + 1000)
    if x_scale != 1.0:  # (large activations, so that the SwiGLU clamp has something to clamp)
        x = (x.float() * x_scale).to(torch.bfloat16)
    sums = []
    with torch.no_grad():
        moe.gate.weight = torch.nn.Parameter(wr.clone(), requires_grad=False)
        moe.gate.bias = torch.nn.Parameter(torch.zeros(E), requires_grad=False)
        for e in range(E + 1):
            ex = moe.experts[e] if e < E else moe.shared_experts
            wg, sg, wu, su, wd, sd = layer.canonical(e)
            sums.append(crc(wg, sg, wu, su, wd, sd))
            for lin, q, s in ((ex.w1, wg, sg), (ex.w3, wu, su), (ex.w2, wd, sd)):
                if mx4 and e < E:
                    lin.weight = torch.nn.Parameter(torch.from_numpy(q.copy()).view(torch.float4_e2m1fn_x2), requires_grad=False)
                    lin.weight.scale = lin.scale = torch.nn.Parameter(torch.from_numpy(s.copy()).view(torch.float8_e8m0fnu),
                                                                      requires_grad=False)
                    continue
                lin.weight = torch.nn.Parameter(torch.from_numpy(q.copy()).view(torch.float8_e4m3fn), requires_grad=False)
                lin.weight.scale = lin.scale = torch.nn.Parameter(torch.from_numpy(s.copy()), requires_grad=False)
        torch.set_default_dtype(torch.bfloat16)
        try:
            weights, indices = moe.gate(x)
            out = moe(x)
            # one expert on one row, for the oracle's per-expert pin
            e0 = int(indices[0, 0])
            y0 = moe.experts[e0](x[:1], weights[:1, :1].float())
            ysh = moe.shared_experts(x[:1])
            logits = M.linear(x.float(), moe.gate.weight.float())
        finally:
            torch.set_default_dtype(torch.float32)
    np.savez_compressed(os.path.join(HERE, name + ".npz"),
                        meta=np.array([H, I, E, topk, T, {"sigmoid": 0, "softmax": 1, "sqrtsoftplus": 2}[score], seed], np.int64),
                        route_scale=np.float32(route_scale), swiglu_limit=np.float32(swiglu_limit), weights_crc=np.array(sums, np.uint32),
                        x=synth.bf16_bits(x), logits=logits.float().numpy(), idx=indices.numpy().astype(np.int32),
                        w=weights.float().numpy(), out=synth.bf16_bits(out), e0=np.int32(e0), y0=synth.bf16_bits(y0),
                        ysh=synth.bf16_bits(ysh))
    print(name, "ok", out.shape)


# ------------------------------------------------------------------------------------------------------------ INT4

int4_tensors = synth.int4_tensors


def int4_case(name, H, I, E, topk, T, seed, route_scale=2.5):
    sys.path.insert(0, os.path.join(REF, "altar1-4xgx10-switchless/ref"))
    import glmref as G
    G.D, G.NE, G.K8, G.DFF, G.ROUTE_SCALE, G.COMBINE = H, E, topk, I, route_scale, "f32"
    rng = np.random.default_rng(seed + 5)
    x = synth.activations(T, H, seed + 1000)
    wr = synth.router_weights(E, H, seed + 2000).to(torch.bfloat16)   # altar-1's gate weight is bf16
    bias = torch.from_numpy((rng.standard_normal(E) * 0.01).astype(np.float32))
    sh = [(torch.randn(n, k, generator=torch.Generator().manual_seed(seed + 9 + i)) * 0.02).to(torch.bfloat16)
          for i, (n, k) in enumerate(((I, H), (I, H), (H, I)))]
    ex = {e: [int4_tensors(n, k, seed * 1000 + e * 3 + m) for m, (n, k) in enumerate(((I, H), (I, H), (H, I)))]
          for e in range(E)}
    sums = [crc(*[a for t in ex[e] for a in t]) for e in range(E)] + [crc(*[synth.bf16_bits(t) for t in sh])]

    def W(nm):
        return {"mlp.gate.weight": wr, "mlp.gate.e_score_correction_bias": bias,
                "mlp.shared_experts.gate_proj.weight": sh[0], "mlp.shared_experts.up_proj.weight": sh[1],
                "mlp.shared_experts.down_proj.weight": sh[2]}[nm]

    class Src:
        def load(self, e):
            return e

        def prepare(self, e):
            out = []
            for (wp, s), (n, k) in zip(ex[e], ((I, H), (I, H), (H, I))):
                packed = torch.from_numpy(wp.view(np.int32).reshape(n, k // 8).copy())
                zp = torch.full((n // 8, k // 32), -2004318072, dtype=torch.int32)      # 0x88888888: zero point 8
                out.append(G.int4_dequant(packed, torch.from_numpy(s.view(np.int16).copy()).view(torch.bfloat16), zp))
            return ("bf16", *out)

    with ThreadPoolExecutor(2) as pool, torch.no_grad():
        out, route, _ = G.moe(x, W, 0, pool, Src())
    deq = Src().prepare(0)[1]
    np.savez_compressed(os.path.join(HERE, name + ".npz"),
                        meta=np.array([H, I, E, topk, T, 0, seed], np.int64), route_scale=np.float32(route_scale),
                        weights_crc=np.array(sums, np.uint32), x=synth.bf16_bits(x), bias=bias.numpy(),
                        idx=route["route_idx"].astype(np.int32), w=route["route_w"], margin=route["route_margin"],
                        out=out.float().numpy(), deq0=synth.bf16_bits(deq)[:16])
    print(name, "ok", out.shape)


# --------------------------------------------------------------------------------------------------------- RMSNorm

def norm_case(name, T, H, seed):
    """Both references' RMSNorm on the same rows: ds41f model.py RMSNorm (one rounding) and altar1 glmref.rms_norm."""
    sys.path[:0] = [os.path.join(REF, "ds41f-4xgx10-switchless/ref/torchref"),
                    os.path.join(REF, "ds41f-4xgx10-switchless/ref/inference")]
    import model as M
    sys.path.insert(0, os.path.join(REF, "altar1-4xgx10-switchless/ref"))
    import glmref as G
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(T, H, generator=g) * 3.0).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    res = torch.randn(T, H, generator=g).to(torch.bfloat16)
    with torch.no_grad():
        torch.set_default_dtype(torch.bfloat16)
        try:
            norm = M.RMSNorm(H, 1e-6)
            norm.weight = torch.nn.Parameter(w.clone(), requires_grad=False)
            y_model = norm(x)
            h = res + x                       # the residual add in bf16 (model.py: x = x + ffn(x))
            y_model_h = norm(h)
        finally:
            torch.set_default_dtype(torch.float32)
        y_glm = G.rms_norm(x, w, 1e-5)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), x=synth.bf16_bits(x), w=synth.bf16_bits(w), res=synth.bf16_bits(res),
                        y_model=synth.bf16_bits(y_model), y_glm=synth.bf16_bits(y_glm), h=synth.bf16_bits(h),
                        y_model_h=synth.bf16_bits(y_model_h))
    print(name, "ok", y_model.shape)


# ------------------------------------------------------------------------------------------- group-limited routing

def group_route_case(name, cases):
    """The group-limited selection (config 2's router: 8 groups, the best 4 kept).  Neither engine of the reference runs it
    (altar-1's n_group = topk_group = 1, ds41f has no groups); altar1 docs/model.md:337-347 names the function that defines
    it: transformers' modeling code of GlmMoeDsa, `route_tokens_to_experts` (group score = the sum of a group's two largest
    sigmoid + bias scores, the best topk_group groups kept, top-k of the kept scores, weights from the sigmoid without the
    bias, normalised with + 1e-20, times the scaling factor).  That function is third-party code present in this
    container (transformers, version recorded in the fixture); its own body is run here on seeded logits, through a
    stand-in object that carries the attributes it reads."""
    import types
    import transformers
    from transformers.models.glm_moe_dsa import modeling_glm_moe_dsa as M
    out = {"transformers_version": np.array(transformers.__version__)}
    for ci, (E, ng, tg, topk, scale, T, seed) in enumerate(cases):
        g = torch.Generator().manual_seed(seed)
        logits = torch.randn(T, E, generator=g) * 1.5
        bias = torch.randn(E, generator=g) * 0.05
        stub = types.SimpleNamespace(n_group=ng, topk_group=tg, n_routed_experts=E, top_k=topk, norm_topk_prob=True,
                                     routed_scaling_factor=scale, gate=types.SimpleNamespace(e_score_correction_bias=bias))
        with torch.no_grad():
            idx, w = M.GlmMoeDsaMoE.route_tokens_to_experts(stub, logits.clone())
        order = idx.argsort(dim=-1)
        idx, w = idx.gather(1, order), w.gather(1, order)
        # how far every decision is from a tie: the kept groups against the dropped ones, the picks against the rest
        sel = logits.sigmoid() + bias
        gs = sel.view(T, ng, E // ng).topk(2, dim=-1)[0].sum(-1)
        gsort = gs.sort(dim=-1, descending=True).values
        gmargin = (gsort[:, tg - 1] - gsort[:, tg]) if tg < ng else torch.full((T,), 1.0)
        keep = torch.zeros(T, ng).scatter_(1, gs.topk(tg, dim=-1)[1], 1.0).bool().repeat_interleave(E // ng, dim=1)
        ssort = sel.masked_fill(~keep, 0.0).sort(dim=-1, descending=True).values
        margin = torch.minimum(gmargin, ssort[:, topk - 1] - ssort[:, topk])
        out.update({f"meta{ci}": np.array([E, ng, tg, topk, T], np.int64), f"scale{ci}": np.float32(scale),
                    f"logits{ci}": logits.numpy(), f"bias{ci}": bias.numpy(), f"idx{ci}": idx.numpy().astype(np.int32),
                    f"w{ci}": w.numpy(), f"margin{ci}": margin.numpy()})
    np.savez_compressed(os.path.join(HERE, name + ".npz"), n_cases=np.int64(len(cases)), **out)
    print(name, "ok", len(cases), "cases")


if __name__ == "__main__":
    group_route_case("group_route", [(256, 8, 4, 8, 2.5, 64, 3401), (64, 4, 2, 6, 1.0, 48, 3402), (32, 8, 3, 4, 1.5, 40, 3403)])
    norm_case("rmsnorm", 6, 4096, 3301)
    fp8_case("fp8_sigmoid_small", 512, 256, 8, 2, 6, "sigmoid", 3101)
    fp8_case("fp8_sigmoid_top6", 1024, 512, 32, 6, 5, "sigmoid", 3102, route_scale=1.5)
    fp8_case("fp8_softmax", 512, 512, 16, 4, 4, "softmax", 3103)
    # ds41f's own router score and its SwiGLU clamp (ref/config.json: scoring_func sqrtsoftplus, swiglu_limit 10)
    fp8_case("fp8_sqrtsoftplus_clamp", 512, 256, 16, 6, 5, "sqrtsoftplus", 3104, route_scale=1.5, swiglu_limit=10.0, x_scale=48.0)
    # ds41f's routed format: MXFP4 experts, FP8 shared expert, its score and clamp
    fp8_case("mx4_sqrtsoftplus_clamp", 512, 256, 16, 6, 5, "sqrtsoftplus", 3105, route_scale=1.5, swiglu_limit=10.0, x_scale=32.0,
             mx4=True)
    int4_case("int4_sigmoid", 1024, 512, 16, 8, 5, 3201)
