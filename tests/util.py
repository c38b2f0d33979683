"""Shared helpers of the parity tests: run the oracle on a synthetic layer, compare with the row-max rule."""
import numpy as np


def oracle_route(orc, x_bits, wr, bias, shp):
    """The oracle's full routing front: logits in the library's summation order, then the selection."""
    logits = orc.router_logits(x_bits, wr)
    idx, w = orc.route(logits, bias, shp.topk, shp.score_fn, shp.n_group, shp.topk_group, bool(shp.norm_topk),
                       shp.route_scale)
    return logits, idx, w


def oracle_fp8_layer(orc, layer, x_bits, idx, w, e_lo=0, e_hi=None, with_shared=True, pickmax=False, swiglu_limit=0.0):
    """The oracle's layer on the picked experts.  Returns (acc, out bits) and, with pickmax, per element the largest
    magnitude among the bf16 outputs added there (see assert_rows_close)."""
    picked = sorted(set(int(e) for e in np.asarray(idx).ravel()))
    experts = {e: layer.canonical(e) for e in picked if (e_hi is None or e < e_hi) and e >= e_lo}
    if not experts:
        experts = {picked[0]: layer.canonical(picked[0])}
    shared = layer.canonical(layer.E) if (layer.shared and with_shared) else None
    return orc.moe_fp8_layer(x_bits, idx, w, experts, shared, e_lo=e_lo, e_hi=e_hi if e_hi is not None else layer.E,
                             with_shared=with_shared, pickmax=pickmax, swiglu_limit=swiglu_limit,
                             mx4=getattr(layer, "fmt", None) == 5)   # (an MXFP4 layer: routed nibbles, FP8 shared expert)


def rowmax_err(got, want):
    """max over rows of max_c |got - want| / max_c |want| (the reference's 2e-3 rule: altar1
    engine/experts/tests/test_prefill.inc:232-247)."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    den = np.abs(want).max(axis=-1, keepdims=True)
    den = np.where(den == 0, 1.0, den)
    return float((np.abs(got - want) / den).max())


def bf16_ulp_hist(orc, got_bits, want_bits):
    """Histogram of |difference| in bf16 ulps: {0: n, 1: n, 2: n, '>2': n}."""
    def key(b):
        b = b.astype(np.int32)
        return np.where(b & 0x8000, -(b & 0x7FFF), b & 0x7FFF)
    d = np.abs(key(np.asarray(got_bits)) - key(np.asarray(want_bits)))
    return {0: int((d == 0).sum()), 1: int((d == 1).sum()), 2: int((d == 2).sum()), ">2": int((d > 2).sum())}


def bf16_ulp(v):
    """The spacing of bf16 numbers at magnitude |v| (8 significant bits)."""
    v = np.abs(np.asarray(v, np.float64))
    return 2.0 ** (np.floor(np.log2(np.maximum(v, 2.0 ** -126))) - 7)


def assert_rows_close(got, want, tol=2e-3, what="", pickmax=None, rounded=False, max_outliers=1e-3):
    """The parity rule of the FFN outputs: every element within `tol` of its row's largest magnitude (the reference's
    own 2e-3 rule, altar1 engine/experts/tests/test_prefill.inc:232-247).

    The FP8 contract rounds every expert's output to bf16 before the f32 adds, so two correct implementations whose f32
    sums differ in the last bits can round one of those outputs to the neighbouring bf16 number.  The rule does not
    excuse that wholesale: with `pickmax` (per element the largest magnitude among the bf16 outputs the oracle added
    there) an element outside `tol` passes only if what is left after `tol` is at most ONE bf16 ulp of that magnitude,
    and such elements must be rarer than `max_outliers`.  `rounded`: the compared values were rounded to bf16 once more
    (the layer's final output), which may flip one ulp of the value itself whenever the f32 sum lies close to the middle
    between two bf16 numbers: that is allowed on up to 2 % of the elements.  Without `pickmax` and `rounded` (the INT4
    contract's f32 sums) the bound is hard.  Returns (max error, number of explained outliers)."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    den = np.abs(want).max(axis=-1, keepdims=True)
    den = np.where(den == 0, 1.0, den)
    diff = np.abs(got - want)
    out = diff > tol * den
    n_out = int(out.sum())
    if rounded:
        max_outliers = max(max_outliers, 2e-2)
    if n_out:
        allow = tol * den * np.ones_like(diff)
        if pickmax is not None:
            allow = allow + bf16_ulp(pickmax) * (1 + 1e-6)
        if rounded:
            allow = allow + bf16_ulp(want) * (1 + 1e-6)
        bad = out & (diff > allow)
        worst = float((diff / den).max())
        assert pickmax is not None or rounded, f"{what}: {n_out} elements beyond {tol} of the row maximum (max {worst:.4g})"
        assert not bad.any(), (f"{what}: {int(bad.sum())} elements beyond {tol} of the row maximum are not explained by one "
                               f"bf16 rounding flip (max {worst:.4g}; worst unexplained excess "
                               f"{float((diff - allow)[bad].max()):.4g})")
        assert n_out <= max(1, int(max_outliers * diff.size)), \
            f"{what}: {n_out} of {diff.size} elements needed the one-ulp explanation (more than {max_outliers})"
    return float((diff / den).max()), n_out
