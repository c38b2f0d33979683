"""Pins the CPU oracle against the reference's own host functions (oracle/_ref, built from the reference tree by
oracle/Makefile) and against known-answer cases the reference's tests hold for this path
(altar1 engine/experts/tests/test_experts.cu:62-213, 289-319)."""
import ctypes as C

import numpy as np
import pytest


def _mix64(x):
    m = (1 << 64) - 1
    x = (x + 0x9E3779B97F4A7C15) & m
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & m
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & m
    return x ^ (x >> 31)


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def test_bf16_and_e4m3_scalars(orc, ref):
    L = orc.lib()
    # every e4m3 code: decode equals the reference's, re-encode is the identity (NaN codes aside)
    for b in range(256):
        mine, theirs = L.orc_e4m3_to_f32(b), ref.ref_e4m3_to_f(b)
        if (b & 0x7F) == 0x7F:
            assert np.isnan(mine) and np.isnan(theirs)
            continue
        assert mine == theirs
        assert L.orc_f32_to_e4m3(mine) == b or (mine == 0.0 and (b & 0x7F) == 0)
    rng = np.random.default_rng(1)
    vals = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s for s in (1e-3, 1.0, 100.0)])
    for v in vals[:3000]:
        assert L.orc_f32_to_bf16(float(v)) == ref.ref_f_to_bf16_bits(float(v))
    assert (orc.f32_to_bf16(vals) == np.array([L.orc_f32_to_bf16(float(v)) for v in vals], np.uint16)).all()


def test_e4m3_encode_matches_torch(orc):
    """f32 -> e4m3 round-to-nearest-even equals torch's conversion (what the Python reference's act_quant uses:
    ds41f ref/torchref/kernel.py:30-31), including ties, subnormals and the saturation edge."""
    import torch
    rng = np.random.default_rng(2)
    L = orc.lib()
    lut = np.array([L.orc_e4m3_to_f32(i) for i in range(127)], np.float32)
    mids = (lut[:-1] + lut[1:]) / 2          # exact ties between neighbours
    vals = np.concatenate([lut, mids, np.nextafter(mids, np.float32(0)), np.nextafter(mids, np.float32(1e9)),
                           rng.uniform(-448, 448, 4000).astype(np.float32),
                           rng.standard_normal(4000).astype(np.float32) * 0.01]).astype(np.float32)
    vals = np.concatenate([vals, -vals])
    t = torch.from_numpy(vals).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    mine = orc.f32_to_e4m3(vals)
    same = (mine == t) | ((vals == 0) & ((mine & 0x7F) == 0) & ((t & 0x7F) == 0))
    assert same.all(), (vals[~same][:5], mine[~same][:5], t[~same][:5])


def test_route_sigmoid_bits(orc, ref):
    L = orc.lib()
    xs = np.concatenate([np.linspace(-100, 100, 4001), np.random.default_rng(3).standard_normal(4000) * 3]).astype(np.float32)
    for x in xs:
        a, b = L.orc_route_sigmoid(float(x)), ref.ref_route_sigmoid(float(x))
        assert np.float32(a).view(np.uint32) == np.float32(b).view(np.uint32), x


def _ref_logits(M, E, seed, ties):
    l = np.empty(M * E, np.float32)
    for i in range(M * E):
        h = _mix64(seed * 13 + i)
        l[i] = np.float32((np.float32((h >> 40)) * np.float32(2.0 ** -24) - np.float32(0.5)) * np.float32(6.0))
        if ties and (h & 7) == 0:
            l[i] = 1.25
    return l.reshape(M, E)


@pytest.mark.parametrize("case", ["random", "many_ties", "tie_at_8th"])
def test_route_matches_reference_route_ref(orc, ref, case):
    """ids and weight bits equal the reference's route_ref at its own shape (168 experts, top-8, x2.5) on its own three
    routing test inputs: random logits, many equal logits with equal bias, a 3-way tie at the 8th place
    (altar1 engine/experts/tests/test_experts.cu:289-319)."""
    E, K = ref.ref_kE(), ref.ref_kTopK()
    assert (E, K) == (168, 8)
    ties = {"random": 0, "many_ties": 1, "tie_at_8th": 2}[case]
    M = 16 + 3 * (ties > 0)
    l = _ref_logits(M, E, 11 + ties, ties == 1)
    if ties:
        bias = np.full(E, 28.25, np.float32)
    else:
        bias = np.array([28.2 + np.float32(0.37) * np.float32((_mix64(e) % 1000) / 1000.0) for e in range(E)], np.float32)
    if ties == 2:
        for m in range(M):
            for e in range(E):
                l[m, e] = np.float32(-4.0) + np.float32(0.01) * np.float32((e * 37 + m * 11) % E)
            a, b, c, top = (m * 13) % E, (m * 13 + 50) % E, (m * 13 + 101) % E, (m * 13 + 7) % E
            for r in range(7):
                l[m, (top + 3 * r) % E] = 5.0 + r
            l[m, a] = l[m, b] = l[m, c] = 4.5
    l = np.ascontiguousarray(l)
    ri = np.empty((M, K), np.int32)
    rw = np.empty((M, K), np.float32)
    ref.ref_route(_p(l), _p(bias), M, _p(ri), _p(rw))
    idx, w = orc.route(l, bias, K, orc.SCORE_SIGMOID, norm=True, route_scale=2.5)
    assert (idx == ri).all()
    assert (w.view(np.uint32) == rw.view(np.uint32)).all()
    if ties == 2:  # the tie is broken towards the lower id
        for m in range(M):
            tied = sorted([(m * 13) % E, (m * 13 + 50) % E, (m * 13 + 101) % E])
            assert idx[m, 7] == tied[0]


def test_route_engineered_ties_order_and_sum(orc):
    """The reference's host check of its routing reference: three experts tied above the rest; picks in descending
    key order with ties to the lower id; weights sum to the route scale (test_experts.cu:187-212)."""
    E, K, M = 168, 8, 64
    l = _ref_logits(M, E, 3, True)
    for m in range(M):
        for j in range(3):
            l[m, (m * 29 + 53 * j) % E] = 3.5
    bias = np.full(E, 28.25, np.float32)
    idx, w = orc.route(l, bias, K, route_scale=2.5)
    L = orc.lib()
    ties = 0
    for m in range(M):
        assert abs(float(w[m].astype(np.float64).sum()) - 2.5) < 1e-5
        for k in range(1, K):
            a, b = idx[m, k - 1], idx[m, k]
            ka = np.float32(L.orc_route_sigmoid(float(l[m, a]))) + bias[a]
            kb = np.float32(L.orc_route_sigmoid(float(l[m, b]))) + bias[b]
            assert ka > kb or (ka == kb and a < b)
            ties += ka == kb
    assert ties > 0


def test_int4_contract_matches_reference(orc, ref):
    """W = bf16((u - u_z) * s), exhaustive over (u, u_z) and a spread of scales incl. subnormal and extreme ones
    (test_experts.cu:62-68, 89-123), through the oracle's dequant of a canonical tensor."""
    scales = [0x0001, 0x007F, 0x0080, 0x3C00, 0x3B80, 0x3BFF, 0x2000, 0x7F00, 0x7F7F, 0x1234]
    scales += [int(((118 + i % 4) << 7) | ((i * 37) & 0x7F)) for i in range(135)]
    N, K = 8, 32 * len(scales)
    for uz in range(16):
        wp = np.zeros((N, K // 2), np.uint8)
        s = np.zeros((N, K // 32), np.uint16)
        zp = np.zeros((1, K // 32), np.uint32)
        for c, sc in enumerate(scales):
            s[:, c] = sc
            zp[0, c] = sum(uz << (4 * r) for r in range(8))
            for i in range(32):
                u = i % 16
                k = 32 * c + i
                wp[:, k // 2] |= np.uint8(u << (4 * (k & 1)))
        out = orc.int4_dequant(wp, s, zp)
        for c, sc in enumerate(scales):
            for u in range(16):
                assert out[0, 32 * c + u] == ref.ref_i4_value_bits(u, uz, sc), (u, uz, hex(sc))
    # symmetric: zero point 8 everywhere equals zp = None
    wp = np.random.default_rng(5).integers(0, 256, (16, 64), dtype=np.uint8)
    s = np.full((16, 4), 0x3C00, np.uint16)
    zp8 = np.full((2, 4), 0x88888888, np.uint32)
    assert (orc.int4_dequant(wp, s, zp8) == orc.int4_dequant(wp, s, None)).all()


def test_packers_match_reference(orc, ref):
    """The engine layouts byte for byte against the reference's packers, and value by value against its readers
    (altar1 engine/experts/layout.h:78-119; test_experts.cu:159-186)."""
    rng = np.random.default_rng(7)
    N, K = 32, 1024
    w8 = rng.integers(0, 256, (N, K), dtype=np.uint8)
    mine = orc.pack_fp8_tile(w8)
    theirs = np.empty_like(mine)
    ref.ref_pack_fp8(_p(w8), N, K, _p(theirs))
    assert (mine == theirs).all()
    assert (orc.unpack_fp8_tile(mine, N, K) == w8).all()
    L = orc.lib()
    for n, k in [(0, 0), (7, 127), (8, 128), (31, 1023), (13, 700)]:
        if (w8[n, k] & 0x7F) != 0x7F:
            assert ref.ref_read_fp8(_p(theirs), K, n, k) == L.orc_e4m3_to_f32(int(w8[n, k]))
    wp = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    s = ((118 + rng.integers(0, 4, (N, K // 32))) << 7 | rng.integers(0, 128, (N, K // 32))).astype(np.uint16)
    zp = rng.integers(0, 2 ** 32, (N // 8, K // 32), dtype=np.uint64).astype(np.uint32)
    mine = orc.pack_int4_block(wp, s, zp)
    theirs = np.empty_like(mine)
    ref.ref_pack_int4(_p(wp), _p(s), _p(zp), N, K, _p(theirs))
    assert (mine == theirs).all()
    deq = orc.int4_dequant(wp, s, zp)
    for n in range(N):
        for k in range(0, K, 7):
            assert ref.ref_read_i4(_p(theirs), K, n, k) == deq[n, k]
            assert L.orc_read_int4_block(_p(mine), K, n, k) == deq[n, k]
    wb = rng.integers(0, 65536, (N, K), dtype=np.uint16)
    mine = orc.pack_bf16_tile(wb)
    theirs = np.empty_like(mine)
    ref.ref_pack_bf16(_p(wb), N, K, _p(theirs))
    assert (mine == theirs).all()
