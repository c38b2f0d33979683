"""The weight-file path (dsgx10_b200/weights.py): the packers against the oracle's (which are pinned byte for byte to the
reference's own packers, tests/test_oracle_pins.py), the rank slices, the layer file's round trip and its checks."""
import os

import numpy as np
import pytest

from dsgx10_b200 import weights as W


def _fp8_expert(rng, H, I):
    t = []
    for N, K in ((I, H), (I, H), (H, I)):
        t += [rng.integers(0, 256, (N, K), dtype=np.uint8), rng.random((N // 128, K // 128), dtype=np.float32) + 0.5]
    return tuple(t)


def _int4_expert(rng, H, I, zp=True):
    t = []
    for N, K in ((I, H), (I, H), (H, I)):
        wp = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
        s = rng.integers(0x3B00, 0x3C80, (N, K // 32)).astype(np.uint16)
        z = rng.integers(0, 2 ** 32, (N // 8, K // 32), dtype=np.uint64).astype(np.uint32) if zp else None
        t.append((wp, s, z))
    return t


def test_packers_equal_the_oracles(orc):
    rng = np.random.default_rng(1)
    q = rng.integers(0, 256, (64, 512), dtype=np.uint8)
    assert (W.pack_fp8(q) == orc.pack_fp8_tile(q)).all()
    assert (W.unpack_fp8(W.pack_fp8(q), 64, 512) == q).all()
    (wp, s, zp), _, _ = _int4_expert(rng, 1024, 64)
    assert (W.pack_int4(wp, s, zp) == orc.pack_int4_block(wp, s, zp)).all()
    assert (W.pack_int4(wp, s, None) == orc.pack_int4_block(wp, s, None)).all()
    w = rng.integers(0, 65536, (32, 256)).astype(np.uint16)
    assert (W.pack_bf16(w) == orc.pack_bf16_tile(w)).all()


def test_rank_slices():
    rng = np.random.default_rng(2)
    H, I = 256, 512
    t = _fp8_expert(rng, H, I)
    parts = [W.rank_slice_fp8(t, r, 2) for r in range(2)]
    assert (np.concatenate([p[0] for p in parts]) == t[0]).all()            # gate rows
    assert (np.concatenate([p[1] for p in parts]) == t[1]).all()            # ... and their scale rows
    assert (np.concatenate([p[4] for p in parts], axis=1) == t[4]).all()    # down's input columns
    assert (np.concatenate([p[5] for p in parts], axis=1) == t[5]).all()
    H, I = 1024, 1024
    ti = _int4_expert(rng, H, I)
    pi = [W.rank_slice_int4(ti, r, 2) for r in range(2)]
    assert (np.concatenate([p[0][0] for p in pi]) == ti[0][0]).all() and (np.concatenate([p[0][2] for p in pi]) == ti[0][2]).all()
    assert (np.concatenate([p[2][0] for p in pi], axis=1) == ti[2][0]).all()
    assert (np.concatenate([p[2][1] for p in pi], axis=1) == ti[2][1]).all()
    with pytest.raises(AssertionError):
        W.rank_slice_fp8(_fp8_expert(rng, 256, 384), 0, 2)                  # 192 rows a rank: not whole scale blocks


def test_layer_file_round_trip_and_checks(tmp_path):
    rng = np.random.default_rng(3)
    H, I, E = 256, 256, 6
    experts = {e: _fp8_expert(rng, H, I) for e in range(E)}
    shared = _fp8_expert(rng, H, I)
    path = str(tmp_path / "layer.dsgx")
    size = W.write_layer_file(path, H, I, E, W.FMT_FP8, experts, shared=shared, e_range=(2, 5))
    assert size == os.path.getsize(path) and size % W.ALIGN == 0
    hdr, entries, data = W.read_layer_file(path)
    assert (hdr["H"], hdr["I"], hdr["E"], hdr["fmt"], hdr["e_lo"], hdr["e_hi"]) == (H, I, E, W.FMT_FP8, 2, 5)
    assert [e["id"] for e in entries] == [2, 3, 4, E]
    for ent in entries:                                                     # every matrix and scale tensor byte for byte
        t = shared if ent["id"] == E else experts[ent["id"]]
        base = ent["offset"] - hdr["data"]
        assert base % W.ALIGN == 0 and all(o % 256 == 0 for o in ent["moff"] + ent["soff"])
        for m in range(3):
            N, K = (H, I) if m == 2 else (I, H)
            got = W.unpack_fp8(data[base + ent["moff"][m]: base + ent["moff"][m] + N * K], N, K)
            assert (got == t[2 * m]).all()
            sc = data[base + ent["soff"][m]: base + ent["soff"][m] + t[2 * m + 1].size * 4].view(np.float32)
            assert (sc == t[2 * m + 1].reshape(-1)).all()
    # a flipped byte in the data, a short file, a foreign file
    raw = bytearray(open(path, "rb").read())
    raw[hdr["data"] + 1000] ^= 0x40
    bad = str(tmp_path / "bad.dsgx")
    open(bad, "wb").write(raw)
    with pytest.raises(W.LayerFileError, match="checksum"):
        W.read_layer_file(bad)
    W.read_layer_file(bad, verify=False)
    open(bad, "wb").write(raw[:-4096])
    with pytest.raises(W.LayerFileError, match="truncated"):
        W.read_layer_file(bad)
    open(bad, "wb").write(b"ALTR1W01" + bytes(raw[8:]))
    with pytest.raises(W.LayerFileError, match="magic"):
        W.read_layer_file(bad)
    with pytest.raises(ValueError):
        W.expert_entry(1, experts[0])                                        # the retired tag


def test_int4_layer_file_with_bf16_shared(tmp_path, orc):
    rng = np.random.default_rng(4)
    H, I, E = 1024, 1024, 3
    experts = {e: _int4_expert(rng, H, I, zp=(e == 1)) for e in range(E)}
    sh = tuple(rng.integers(0, 65536, s).astype(np.uint16) for s in ((I, H), (I, H), (H, I)))
    path = str(tmp_path / "layer4.dsgx")
    W.write_layer_file(path, H, I, E, W.FMT_INT4, experts, shared=sh, tp=(1, 2))
    hdr, entries, data = W.read_layer_file(path)
    assert hdr["I"] == I // 2 and hdr["tp_rank"] == 1 and hdr["tp_world"] == 2
    ent = entries[1]
    sl = W.rank_slice_int4(experts[1], 1, 2)
    base = ent["offset"] - hdr["data"]
    for m in range(3):
        want = orc.pack_int4_block(*sl[m])
        assert (data[base + ent["moff"][m]: base + ent["moff"][m] + want.size] == want).all()
    s_ent = entries[-1]
    assert s_ent["id"] == E and s_ent["fmt"] == W.FMT_BF16
    gu = W.interleave_gate_up(sh[0][I // 2:], sh[1][I // 2:])
    b = s_ent["offset"] - hdr["data"] + s_ent["moff"][0]
    assert (data[b: b + gu.size * 2] == orc.pack_bf16_tile(gu)).all()


def test_mx4_packer_slices_and_file(tmp_path, orc):
    """MXFP4 (tag 5): the packer is the synthetic layers' tiler (torch) byte for byte and round-trips; every value of a
    packed block dequantises as the oracle dequantises the canonical tensor; rank slices; a layer file with an FP8 shared
    expert."""
    import torch
    from dsgx10_b200 import synth
    rng = np.random.default_rng(5)
    N, K = 64, 512
    q = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    s = rng.integers(100, 140, (N, K // 32), dtype=np.uint8)
    packed = W.pack_mx4(q, s)
    assert packed.size == (N // 8) * (K // 128) * 576
    assert (packed == synth.tile_mx4(torch.from_numpy(q), torch.from_numpy(s)).numpy()).all()
    q2, s2 = W.unpack_mx4(packed, N, K)
    assert (q2 == q).all() and (s2 == s).all()
    # the layout as the header states it, value by value: lane (g, t), group G of block b holds k = 128 b + 32 G + 8 t + 0..7
    deq = orc.mx4_dequant(q, s)
    mags = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], np.float32)
    blk = packed.reshape(N // 8, K // 128, 576)
    for n8, b, g, t, G in ((0, 0, 0, 0, 0), (3, 2, 5, 1, 2), (7, 3, 7, 3, 3)):
        word = int(blk[n8, b, (4 * g + t) * 16 + 4 * G:][:4].view(np.uint32)[0])
        e = int(blk[n8, b, 512 + 8 * g + 2 * G:][:2].view(np.uint16)[0]) >> 7     # the scale as bf16: byte << 7
        k = 128 * b + 32 * G + 8 * t
        got = np.array([(-1.0 if (word >> (8 * i + 7 if i < 4 else 8 * (i - 4) + 3)) & 1 else 1.0) * mags[(word >> (4 * i)) & 7]
                        for i in range(8)], np.float32) * np.float32(2.0) ** (e - 127)
        assert (got == deq[8 * n8 + g, k:k + 8]).all()
    H, I = 256, 512
    t = []
    for n, k in ((I, H), (I, H), (H, I)):
        t += [rng.integers(0, 256, (n, k // 2), dtype=np.uint8), rng.integers(110, 130, (n, k // 32), dtype=np.uint8)]
    parts = [W.rank_slice_mx4(tuple(t), r, 2) for r in range(2)]
    assert (np.concatenate([p[0] for p in parts]) == t[0]).all() and (np.concatenate([p[1] for p in parts]) == t[1]).all()
    assert (np.concatenate([p[4] for p in parts], axis=1) == t[4]).all()
    assert (np.concatenate([p[5] for p in parts], axis=1) == t[5]).all()
    path = str(tmp_path / "mx4.dsgx")
    shared = _fp8_expert(rng, H, I)
    W.write_layer_file(path, H, I, 2, W.FMT_MXFP4, {0: tuple(t), 1: tuple(t)}, shared=shared)
    hdr, entries, data = W.read_layer_file(path)
    assert hdr["fmt"] == W.FMT_MXFP4 and [e["fmt"] for e in entries] == [W.FMT_MXFP4, W.FMT_MXFP4, W.FMT_FP8]
    e0 = entries[0]
    got = data[e0["offset"] - hdr["data"] + e0["moff"][2]:][:W.pack_mx4(t[4], t[5]).size]
    assert (got == W.pack_mx4(t[4], t[5])).all()
