"""The weight-file path of one MoE layer: checkpoint tensors -> the kernels' tile layouts -> a per-rank layer file ->
device pool + descriptors.

It stands in for the part of the reference's converter / loader that feeds the expert kernels (altar1
engine/weights/int4_pack.py:113-205: `rank_slice`, `pack`, `expert_entry`, `expert_descs`; the per-rank container of
engine/weights/glw.h: header, table of contents, 4 KiB-aligned data, a checksum per entry) for the formats this library
runs: routed FP8-128 experts (tag 4: `tile_fp8` values + f32 [N/128][K/128] scales), INT4-g32 experts (tag 2), MXFP4
experts (tag 5: e2m1 values + their power-of-two scales in 576-byte blocks) and the shared expert (FP8, or BF16 as the interleaved gate/up matrix + down).  Nothing is quantised here: every stored code,
scale and zero point is the checkpoint's, only re-tiled.  numpy only on the packing side; torch carries the pool to the
device.

    experts = {e: (wg, sg, wu, su, wd, sd)}                 # canonical e4m3 codes [N][K] and f32 scales [N/128][K/128]
    write_layer_file(path, H, I, E, FMT_FP8, experts, shared=(...), tp=(rank, world))
    layer = load_layer_file(path, device="cuda")            # verifies every entry's CRC-32, builds pool + descriptors
    step.run(layer.layer_w(), x)

File layout (little endian):
    [0, 4096)        header: magic "DSGXMOE1", version, H, I, E, fmt, first and end of the stored expert range, the
                     tensor-parallel (rank, world) the slices were cut for, entry count, table offset, data offset, size
    [toc, ...)       one 128-byte entry per stored expert (id E: the shared expert): id, format tag, offset and size of
                     its bytes, the offsets of gate / up / down inside them and of their scale tensors, CRC-32
    [data, size)     the entries' bytes, each starting on a 4 KiB boundary; the device address of an entry is
                     pool + (entry offset - data offset)
"""
import struct
import zlib

import numpy as np

FMT_INT4, FMT_BF16, FMT_FP8, FMT_MXFP4 = 2, 3, 4, 5
MAGIC = b"DSGXMOE1"
VERSION = 1
ALIGN = 4096
HEADER = struct.Struct("<8sIIIIIIIIIIQQQ")   # magic, version, H, I, E, fmt, e_lo, e_hi, tp_rank, tp_world, n, toc, data, size
ENTRY = struct.Struct("<IIQQ3Q3QI")           # id, fmt, offset, bytes, matrix offsets, scale offsets, crc32
ENTRY_BYTES = 128
I4_BLK, B16_BLK, MX4_BLK = 2368, 2048, 576


def _al(n, a=ALIGN):
    return (n + a - 1) // a * a


# ------------------------------------------------------------------------------------------------------------ packers

def pack_fp8(q):
    """canonical e4m3 codes uint8 [N][K] -> the tile_fp8 byte stream [N/8][K/128][32 lanes][32 B]: lane 4 g + t holds
    row 8 n8 + g, k = 128 j + 64 q + 16 t + i at byte 16 q + i (altar1 engine/experts/layout.h:108-119)."""
    q = np.ascontiguousarray(q, np.uint8)
    N, K = q.shape
    assert N % 8 == 0 and K % 128 == 0
    v = q.reshape(N // 8, 8, K // 128, 2, 4, 16)                 # n8, g, j, q, t, i
    return np.ascontiguousarray(v.transpose(0, 2, 1, 4, 3, 5)).reshape(-1)   # n8, j, g, t, q, i


def unpack_fp8(m, N, K):
    v = np.ascontiguousarray(m, np.uint8).reshape(N // 8, K // 128, 8, 4, 2, 16)
    return np.ascontiguousarray(v.transpose(0, 2, 1, 4, 3, 5)).reshape(N, K)


def mx4_words(q):
    """canonical nibble bytes uint8 [N][K/2] -> the stored words uint32 [N][K/8]: magnitudes in place, the sign of value
    i < 4 of a word at bit 8 i + 7, of value i >= 4 at bit 8 (i - 4) + 3."""
    w = np.ascontiguousarray(q, np.uint8).view(np.uint32)
    out = w & np.uint32(0x77777777)
    for i in range(8):
        out |= ((w >> np.uint32(4 * i + 3)) & np.uint32(1)) << np.uint32(8 * i + 7 if i < 4 else 8 * (i - 4) + 3)
    return out


def mx4_unwords(w):
    w = np.ascontiguousarray(w, np.uint32)
    out = w & np.uint32(0x77777777)
    for i in range(8):
        out |= ((w >> np.uint32(8 * i + 7 if i < 4 else 8 * (i - 4) + 3)) & np.uint32(1)) << np.uint32(4 * i + 3)
    return out.view(np.uint8)


def pack_mx4(q, s):
    """canonical MXFP4 (e2m1 nibble bytes uint8 [N][K/2], the lower k in the low nibble; ue8m0 scale bytes uint8 [N][K/32];
    ds41f ref/torchref/kernel.py:111-118) -> this library's blocks of 8 rows x 128 k, 576 B, [N/8][K/128]:
    [32 lanes 4 g + t][4 groups G][one word = k 128 b + 32 G + 8 t + 0..7 of row 8 n8 + g, the sign bits moved inside the
    word (mx4_words)], then [8 g][4 G] the scales 2^(byte - 127) written as bf16 (byte << 7; 0x0040 for byte 0): the same
    numbers, one shift from a float on the device
    (it stands in for ds41f's own re-tiling, engine/kernels/dsk.h:176-180 tile_fp4, for these kernels' operand order)."""
    q, s = np.ascontiguousarray(q, np.uint8), np.ascontiguousarray(s, np.uint8)
    N, K = q.shape[0], q.shape[1] * 2
    assert N % 8 == 0 and K % 128 == 0 and s.shape == (N, K // 32)
    qw = mx4_words(q).view(np.uint8).reshape(N, K // 2)
    vals = np.ascontiguousarray(qw.reshape(N // 8, 8, K // 128, 4, 4, 4).transpose(0, 2, 1, 4, 3, 5))  # n8, b, g, t, G, byte
    sb = np.where(s == 0, 0x40, s.astype(np.uint16) << 7).astype(np.uint16)
    sc = np.ascontiguousarray(sb.reshape(N // 8, 8, K // 128, 4).transpose(0, 2, 1, 3))                 # n8, b, g, G
    out = np.empty((N // 8, K // 128, MX4_BLK), np.uint8)
    out[..., :512] = vals.reshape(N // 8, K // 128, 512)
    out[..., 512:] = sc.view(np.uint8).reshape(N // 8, K // 128, 64)
    return out.reshape(-1)


def unpack_mx4(m, N, K):
    blk = np.ascontiguousarray(m, np.uint8).reshape(N // 8, K // 128, MX4_BLK)
    q = np.ascontiguousarray(blk[..., :512].reshape(N // 8, K // 128, 8, 4, 4, 4).transpose(0, 2, 1, 4, 3, 5)).reshape(N, K // 2)
    q = mx4_unwords(q.view(np.uint32)).reshape(N, K // 2)
    sb = np.ascontiguousarray(blk[..., 512:]).view(np.uint16).reshape(N // 8, K // 128, 8, 4)
    s = np.where(sb == 0x40, 0, sb >> 7).astype(np.uint8)
    return q, np.ascontiguousarray(s.transpose(0, 2, 1, 3)).reshape(N, K // 32)


def pack_int4(wp, s, zp=None):
    """canonical INT4-g32 (compressed-tensors pack-quantized: wp uint8 [N][K/2], value k in byte k/2, low nibble = even
    k, stored nibble u = q + 8; s bf16 bits [N][K/32]; zp uint32 [N/8][K/32], row n's zero-point nibble at bits 4 (n % 8),
    None: 8 everywhere) -> blocks of 8 rows x 512 k, 2368 B each, [N/8][K/512] (layout.h:50-58, 78-95;
    int4_pack.py:151-162)."""
    wp, s = np.ascontiguousarray(wp, np.uint8), np.ascontiguousarray(s, np.uint16)
    N, K = wp.shape[0], wp.shape[1] * 2
    assert N % 8 == 0 and K % 512 == 0
    B, N8 = K // 512, N // 8
    v = wp.reshape(N8, 8, B, 4, 2, 4, 8).transpose(0, 2, 3, 1, 5, 4, 6).reshape(N8, B, 2048)   # n8, b, jj, g, t, q, byte
    sc = s.reshape(N8, 8, B, 8, 2).transpose(0, 2, 1, 4, 3).reshape(N8, B, 128)                # n8, b, g, h, j
    out = np.empty((N8, B, I4_BLK), np.uint8)
    out[:, :, :2048] = v
    out[:, :, 2048:2304] = np.ascontiguousarray(sc).view(np.uint8).reshape(N8, B, 256)
    if zp is None:
        out[:, :, 2304:] = 0x88
    else:
        zp = np.ascontiguousarray(zp, np.uint32)                                            # [N8][K/32]
        nib = ((zp[:, None, :] >> (4 * np.arange(8, dtype=np.uint32))[None, :, None]) & 15).astype(np.uint8)   # [N8][g][K/32]
        z = nib.reshape(N8, 8, B, 8, 2).transpose(0, 2, 1, 4, 3)                            # n8, b, g, h, j
        out[:, :, 2304:] = (z[..., 0::2] | (z[..., 1::2] << 4)).reshape(N8, B, 64)
    return out.reshape(-1)


def pack_bf16(w):
    """bf16 bits uint16 [N][K] -> blocks of 8 rows x 128 k, 2048 B, [N/8][K/128]: the lane's 16 B at 512 p + 16 (4 g + t)
    are k = 64 (p >> 1) + 16 t + 8 (p & 1) + 0..7 (layout.h:96-107; int4_pack.py:165-170)."""
    w = np.ascontiguousarray(w, np.uint16)
    N, K = w.shape
    assert N % 8 == 0 and K % 128 == 0
    v = w.reshape(N // 8, 8, K // 128, 2, 4, 2, 8)                                            # n8, g, b, q, t, half, 8
    return np.ascontiguousarray(v.transpose(0, 2, 3, 5, 1, 4, 6)).reshape(-1).view(np.uint8)


def interleave_gate_up(g, u):
    """[I][K], [I][K] -> [2 I][K]: row 2 i gate, 2 i + 1 up of channel i (the engine's SharedW::bgu order)."""
    out = np.empty((2 * g.shape[0],) + g.shape[1:], g.dtype)
    out[0::2], out[1::2] = g, u
    return out


# --------------------------------------------------------------------------------------------- slices of a checkpoint

def rank_slice_fp8(tensors, rank, world):
    """Tensor-parallel rank `rank` of `world` of one FP8 expert (wg, sg, wu, su, wd, sd): gate / up rows and down's input
    columns [I r / world, I (r + 1) / world) with their block scales (int4_pack.py:113-140 for this format); the cut
    must fall on 128-row block borders."""
    wg, sg, wu, su, wd, sd = tensors
    I = wg.shape[0]
    assert I % (128 * world) == 0, "a rank's slice must be whole 128 x 128 scale blocks"
    lo, hi = I * rank // world, I * (rank + 1) // world
    b0, b1 = lo // 128, hi // 128
    c = np.ascontiguousarray
    return (c(wg[lo:hi]), c(sg[b0:b1]), c(wu[lo:hi]), c(su[b0:b1]), c(wd[:, lo:hi]), c(sd[:, b0:b1]))


def rank_slice_mx4(tensors, rank, world):
    """The same for an MXFP4 expert (wg, sg, wu, su, wd, sd: nibble bytes and ue8m0 bytes): gate / up rows and down's input
    columns; the cut falls on whole 128-k blocks of the down matrix."""
    wg, sg, wu, su, wd, sd = tensors
    I = wg.shape[0]
    assert I % (128 * world) == 0
    lo, hi = I * rank // world, I * (rank + 1) // world
    c = np.ascontiguousarray
    return (c(wg[lo:hi]), c(sg[lo:hi]), c(wu[lo:hi]), c(su[lo:hi]), c(wd[:, lo // 2:hi // 2]), c(sd[:, lo // 32:hi // 32]))


def rank_slice_int4(tensors, rank, world):
    """The same for an INT4-g32 expert ((wp, s, zp) for gate, up, down; zp may be None): every cut is group- and
    word-aligned (int4_pack.py:113-140)."""
    out = []
    for m, (wp, s, zp) in enumerate(tensors):
        N, K = wp.shape[0], wp.shape[1] * 2
        if m < 2:
            lo, hi = N * rank // world, N * (rank + 1) // world
            assert lo % 8 == 0 and hi % 8 == 0
            out.append((np.ascontiguousarray(wp[lo:hi]), np.ascontiguousarray(s[lo:hi]),
                        None if zp is None else np.ascontiguousarray(zp[lo // 8:hi // 8])))
        else:
            lo, hi = K * rank // world, K * (rank + 1) // world
            assert lo % 512 == 0 and hi % 512 == 0
            out.append((np.ascontiguousarray(wp[:, lo // 2:hi // 2]), np.ascontiguousarray(s[:, lo // 32:hi // 32]),
                        None if zp is None else np.ascontiguousarray(zp[:, lo // 32:hi // 32])))
    return out


# ------------------------------------------------------------------------------------------------------------ entries

def _place(parts):
    """Concatenate byte arrays, each on a 256-byte boundary; returns (bytes, offsets)."""
    offs, n = [], 0
    for p in parts:
        n = _al(n, 256)
        offs.append(n)
        n += p.size
    buf = np.zeros(_al(n, 256), np.uint8)
    for o, p in zip(offs, parts):
        buf[o:o + p.size] = p
    return buf, offs


def expert_entry(fmt, tensors):
    """One expert's bytes in the kernels' layouts and where its matrices lie in them: (bytes, matrix offsets [3], scale
    offsets [3]); stands in for int4_pack.expert_entry (:179-195).  fmt FMT_FP8: tensors = (wg, sg, wu, su, wd, sd);
    FMT_INT4: ((wp, s, zp) x 3); FMT_BF16 (the INT4 layers' shared expert): (wg, wu, wd) bf16 bits, stored as the
    interleaved gate/up matrix and the down matrix (matrix offsets: gate/up, -, down)."""
    if fmt == FMT_FP8:
        wg, sg, wu, su, wd, sd = tensors
        parts = [pack_fp8(wg), pack_fp8(wu), pack_fp8(wd)] + [np.ascontiguousarray(s, np.float32).view(np.uint8).reshape(-1)
                                                              for s in (sg, su, sd)]
        buf, offs = _place(parts)
        return buf, offs[:3], offs[3:]
    if fmt == FMT_MXFP4:
        wg, sg, wu, su, wd, sd = tensors
        buf, offs = _place([pack_mx4(wg, sg), pack_mx4(wu, su), pack_mx4(wd, sd)])
        return buf, offs, [0, 0, 0]
    if fmt == FMT_INT4:
        buf, offs = _place([pack_int4(*t) for t in tensors])
        return buf, offs, [0, 0, 0]
    if fmt == FMT_BF16:
        wg, wu, wd = tensors
        buf, offs = _place([pack_bf16(interleave_gate_up(wg, wu)), pack_bf16(wd)])
        return buf, [offs[0], 0, offs[1]], [0, 0, 0]
    raise ValueError(f"expert format {fmt}: not INT4 (2), BF16 (3), FP8 (4) or MXFP4 (5); NVFP4 (0) and the retired tag 1 are refused")


def write_layer_file(path, H, I, E, fmt, experts, shared=None, shared_fmt=None, tp=(0, 1), e_range=None):
    """experts: {id: canonical tensors} (the ids of e_range, default all E); shared: the shared expert's tensors (FP8 for an
    FP8 layer; bf16 bits (wg, wu, wd) for an INT4 layer) or None; tp = (rank, world): every expert is cut with
    rank_slice_* first, so the file holds intermediate size I / world."""
    rank, world = tp
    lo, hi = e_range if e_range is not None else (0, E)
    Ir = I // world
    entries, blobs = [], []
    off = 0

    def add(eid, f, tensors):
        nonlocal off
        buf, moff, soff = expert_entry(f, tensors)
        entries.append((eid, f, off, buf.size, moff, soff, zlib.crc32(buf.tobytes()) & 0xFFFFFFFF))
        blobs.append(buf)
        off += _al(buf.size)

    for e in range(lo, hi):
        t = experts[e]
        if world > 1:
            t = (rank_slice_fp8 if fmt == FMT_FP8 else rank_slice_mx4 if fmt == FMT_MXFP4 else rank_slice_int4)(t, rank, world)
        add(e, fmt, t)
    if shared is not None:
        sf = shared_fmt if shared_fmt is not None else (FMT_FP8 if fmt in (FMT_FP8, FMT_MXFP4) else FMT_BF16)
        if world > 1:
            if sf == FMT_FP8:
                shared = rank_slice_fp8(shared, rank, world)
            else:
                wg, wu, wd = shared
                a, b = wg.shape[0] * rank // world, wg.shape[0] * (rank + 1) // world
                shared = (np.ascontiguousarray(wg[a:b]), np.ascontiguousarray(wu[a:b]), np.ascontiguousarray(wd[:, a:b]))
        add(E, sf, shared)
    toc = _al(HEADER.size)
    data = _al(toc + len(entries) * ENTRY_BYTES)
    size = data + off
    with open(path, "wb") as f:
        f.write(HEADER.pack(MAGIC, VERSION, H, Ir, E, fmt, lo, hi, rank, world, len(entries), toc, data, size))
        f.seek(toc)
        for eid, ef, o, n, moff, soff, crc in entries:
            f.write(ENTRY.pack(eid, ef, data + o, n, *moff, *soff, crc).ljust(ENTRY_BYTES, b"\0"))
        for (eid, ef, o, n, moff, soff, crc), buf in zip(entries, blobs):
            f.seek(data + o)
            f.write(buf.tobytes())
        f.truncate(size)
    return size


class LayerFileError(RuntimeError):
    pass


def read_layer_file(path, verify=True):
    """-> (header dict, entries [dict], data bytes as a numpy array); raises LayerFileError on a bad magic, version,
    size or (with verify) checksum."""
    raw = np.fromfile(path, np.uint8)
    if raw.size < HEADER.size:
        raise LayerFileError("not a layer file: too short")
    magic, ver, H, I, E, fmt, lo, hi, rank, world, n, toc, data, size = HEADER.unpack(raw[:HEADER.size].tobytes())
    if magic != MAGIC:
        raise LayerFileError("not a layer file: bad magic")
    if ver != VERSION:
        raise LayerFileError(f"layer file version {ver}, this reader knows {VERSION}")
    if size != raw.size or toc + n * ENTRY_BYTES > data or data > size:
        raise LayerFileError("layer file is truncated or its header is inconsistent")
    if fmt not in (FMT_INT4, FMT_FP8, FMT_MXFP4):
        raise LayerFileError(f"layer format {fmt}: this library runs INT4 (2), FP8 (4) and MXFP4 (5) layers")
    entries = []
    for i in range(n):
        rec = ENTRY.unpack(raw[toc + i * ENTRY_BYTES: toc + i * ENTRY_BYTES + ENTRY.size].tobytes())
        eid, ef, off, nbytes = rec[:4]
        ent = dict(id=eid, fmt=ef, offset=off, bytes=nbytes, moff=list(rec[4:7]), soff=list(rec[7:10]), crc=rec[10])
        if off < data or off + nbytes > size or off % ALIGN:
            raise LayerFileError(f"entry {eid}: outside the data region")
        if verify and (zlib.crc32(raw[off:off + nbytes].tobytes()) & 0xFFFFFFFF) != ent["crc"]:
            raise LayerFileError(f"entry {eid}: checksum mismatch")
        entries.append(ent)
    hdr = dict(H=H, I=I, E=E, fmt=fmt, e_lo=lo, e_hi=hi, tp_rank=rank, tp_world=world, data=data, size=size)
    return hdr, entries, raw[data:]


class LoadedLayer:
    """A layer file on a device: the pool (the file's data region, byte for byte), the descriptors [E][3] and the shared
    expert's pointers; `layer_w()` is what the operator takes."""

    def __init__(self, hdr, entries, pool, desc):
        self.hdr, self.entries, self.pool, self.desc = hdr, entries, pool, desc
        self.H, self.I, self.E, self.fmt = hdr["H"], hdr["I"], hdr["E"], hdr["fmt"]
        self.shared = next((e for e in entries if e["id"] == self.E), None)

    def layer_w(self):
        from . import _lib
        L = _lib.LayerW()
        L.pool, L.desc, L.fmt = self.pool.data_ptr(), self.desc.data_ptr(), self.fmt
        s = self.shared
        if s is not None:
            base = self.pool.data_ptr() + s["offset"] - self.hdr["data"]
            if s["fmt"] == FMT_FP8:
                L.sh.g, L.sh.u, L.sh.d = (base + o for o in s["moff"])
                L.sh.gs, L.sh.us, L.sh.ds = (base + o for o in s["soff"])
            else:
                L.sh.bgu, L.sh.bd = base + s["moff"][0], base + s["moff"][2]
        return L


def load_layer_file(path, device="cuda", verify=True):
    """Reads and verifies a layer file, copies its data region to the device in one piece and builds the descriptors
    (dsgx_mat_desc: off relative to the pool, s2 1.0, the format tag, for FP8 the scales' offset in rsv[0..1]); stands in
    for the loader's expert part and int4_pack.expert_descs (:198-205)."""
    import torch
    from . import _lib
    hdr, entries, data = read_layer_file(path, verify=verify)
    desc = (_lib.MatDesc * (hdr["E"] * 3))()
    for ent in entries:
        if ent["id"] >= hdr["E"]:
            continue
        base = ent["offset"] - hdr["data"]
        for m in range(3):
            d = desc[ent["id"] * 3 + m]
            d.off, d.s2, d.fmt = base + ent["moff"][m], 1.0, ent["fmt"]
            if ent["fmt"] == FMT_FP8:
                so = base + ent["soff"][m]
                d.rsv[0], d.rsv[1] = so & 0xFFFFFFFF, so >> 32
    pool = torch.from_numpy(np.ascontiguousarray(data)).to(device)
    desc_t = torch.frombuffer(bytearray(bytes(desc)), dtype=torch.uint8).to(device)
    return LoadedLayer(hdr, entries, pool, desc_t)
