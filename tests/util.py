"""Shared helpers of the parity tests: run the oracle on a synthetic layer, compare with the row-max rule."""
import numpy as np


def oracle_route(orc, x_bits, wr, bias, shp):
    """The oracle's full routing front: logits in the library's summation order, then the selection."""
    logits = orc.router_logits(x_bits, wr)
    idx, w = orc.route(logits, bias, shp.topk, shp.score_fn, shp.n_group, shp.topk_group, bool(shp.norm_topk),
                       shp.route_scale)
    return logits, idx, w


def oracle_fp8_layer(orc, layer, x_bits, idx, w, e_lo=0, e_hi=None, with_shared=True):
    picked = sorted(set(int(e) for e in np.asarray(idx).ravel()))
    experts = {e: layer.canonical(e) for e in picked if (e_hi is None or e < e_hi) and e >= e_lo}
    if not experts:
        experts = {picked[0]: layer.canonical(picked[0])}
    shared = layer.canonical(layer.E) if (layer.shared and with_shared) else None
    return orc.moe_fp8_layer(x_bits, idx, w, experts, shared, e_lo=e_lo, e_hi=e_hi if e_hi is not None else layer.E,
                             with_shared=with_shared)


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


def assert_rows_close(got, want, tol=2e-3, frac=0.999, what=""):
    """The parity rule of the FFN outputs.  Errors are measured against the row's largest magnitude (the reference's own
    2e-3 rule).  The FP8 contract rounds every pick's output (and h, g, u) to bf16, so two correct implementations whose
    f32 sums differ in the last bits can differ by one bf16 ulp of a pick's output on isolated elements, which at the
    scale of the row maximum is up to 2^-7: so at least `frac` of the elements must be within tol, and every element
    within tol + 2^-7."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    den = np.abs(want).max(axis=-1, keepdims=True)
    den = np.where(den == 0, 1.0, den)
    err = np.abs(got - want) / den
    inside = float((err <= tol).mean())
    assert inside >= frac, f"{what}: only {inside:.5f} of the elements within {tol} of the row maximum (max {err.max():.4g})"
    assert err.max() <= tol + 2.0 ** -7, f"{what}: max error {err.max():.4g} of the row maximum"
    return float(err.max()), inside
