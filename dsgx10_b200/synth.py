"""Seeded synthetic MoE layers in the engine's weight layouts (pool + descriptors), for the tests and the bench.

The reference benches and tests its expert kernels on hashed synthetic layers too (altar1
engine/experts/tests/testdata.h:52-198); the distributions here are the ones the benchmark configurations name:
FP8 weights quantised from N(0, 0.02) per 128x128 block (scale = amax / 448), INT4 nibbles uniform in [-8, 7] with bf16
group scales in [2^-9, 2^-7), router weights f32 N(0, 0.02), activations bf16 N(0, 1).
"""
import numpy as np
import torch

from . import _lib

F8 = torch.float8_e4m3fn


def _gen(device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def al256(n):
    return (n + 255) & ~255


# ------------------------------------------------------------------------------------------------------ FP8 tensors

def quant_fp8_128(w):
    """f32 [N][K] -> (e4m3 codes uint8 [N][K], f32 scales [N/128][K/128]); scale = amax / 448 per 128x128 block."""
    N, K = w.shape
    blk = w.view(N // 128, 128, K // 128, 128)
    amax = blk.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    s = amax * (1.0 / 448.0)
    q = (blk / s[:, None, :, None]).clamp(-448.0, 448.0).to(F8)
    return q.view(N, K).view(torch.uint8), s.float().contiguous()


def tile_fp8(q):
    """canonical e4m3 codes [N][K] -> the tile_fp8 byte stream [N/8][K/128][32 lanes][32 B]
    (lane 4 g + t: row 8 n8 + g, k = 128 j + 64 q + 16 t + i at byte 16 q + i; altar1 engine/experts/layout.h:108-119)."""
    N, K = q.shape
    v = q.view(N // 8, 8, K // 128, 2, 4, 16)          # n8, g, j, q, t, i
    return v.permute(0, 2, 1, 4, 3, 5).contiguous().view(-1)   # n8, j, g, t, q, i


def untile_fp8(m, N, K):
    v = m.view(N // 8, K // 128, 8, 4, 2, 16)           # n8, j, g, t, q, i
    return v.permute(0, 2, 1, 4, 3, 5).contiguous().view(N, K)


class Fp8Layer:
    """One FP8 layer: `E` routed experts + (optionally) a shared expert, all in one device pool."""

    def __init__(self, H, I, E, seed, device="cpu", shared=True, std=0.02, e_range=None):
        """e_range = (lo, hi): only these experts are generated and stored (an expert-parallel rank's share); an
        expert's weights depend on (seed, expert id) alone, whatever the range."""
        self.H, self.I, self.E, self.fmt = H, I, E, _lib.FMT_FP8
        self.device = torch.device(device)
        mat_b = I * H
        sc_b = al256((I // 128) * (H // 128) * 4)
        per_expert = 3 * mat_b + 3 * sc_b
        lo, hi = e_range if e_range is not None else (0, E)
        ids = list(range(lo, hi)) + ([E] if shared else [])
        self.pool = torch.empty(max(len(ids), 1) * per_expert, dtype=torch.uint8, device=self.device)
        self.desc_host = (_lib.MatDesc * (E * 3))()
        self._off = {}
        for n, e in enumerate(ids):
            base = n * per_expert
            for m in range(3):
                N, K = (H, I) if m == 2 else (I, H)
                g = _gen(self.device, seed * 1000003 + e * 3 + m)
                w = torch.randn(N, K, generator=g, device=self.device, dtype=torch.float32) * std
                q, s = quant_fp8_128(w)
                off = base + m * mat_b
                soff = base + 3 * mat_b + m * sc_b
                self.pool[off:off + mat_b] = tile_fp8(q)
                self.pool[soff:soff + s.numel() * 4] = s.view(-1).view(torch.uint8)
                self._off[(e, m)] = (off, soff)
                if e < E:
                    d = self.desc_host[e * 3 + m]
                    d.off, d.s2, d.fmt = off, 1.0, _lib.FMT_FP8
                    d.rsv[0], d.rsv[1] = soff & 0xFFFFFFFF, soff >> 32
        self.desc = torch.frombuffer(bytearray(bytes(self.desc_host)), dtype=torch.uint8).to(self.device)
        self.shared = shared

    def to(self, device):
        """The same layer with its pool and descriptors on another device (built on the CPU, it reaches the GPU in two
        copies instead of hundreds of small generation kernels)."""
        self.device = torch.device(device)
        self.pool, self.desc = self.pool.to(self.device), self.desc.to(self.device)
        return self

    def layer_w(self):
        L = _lib.LayerW()
        L.pool, L.desc, L.fmt = self.pool.data_ptr(), self.desc.data_ptr(), _lib.FMT_FP8
        if self.shared:
            p = self.pool.data_ptr()
            (g, gs), (u, us), (d, ds) = (self._off[(self.E, m)] for m in range(3))
            L.sh.g, L.sh.u, L.sh.d, L.sh.gs, L.sh.us, L.sh.ds = p + g, p + u, p + d, p + gs, p + us, p + ds
        return L

    def canonical(self, e):
        """(wg, sg, wu, su, wd, sd) of expert e (e == E: the shared expert) as numpy arrays, un-tiled from the pool."""
        out = []
        for m in range(3):
            N, K = (self.H, self.I) if m == 2 else (self.I, self.H)
            off, soff = self._off[(e, m)]
            q = untile_fp8(self.pool[off:off + N * K], N, K).cpu().numpy()
            ns = (N // 128) * (K // 128)
            s = self.pool[soff:soff + ns * 4].cpu().view(torch.float32).view(N // 128, K // 128).numpy().copy()
            out += [q, s]
        return tuple(out)

    def expert_bytes(self):
        """Algorithmic bytes of one expert: three matrices and their block scales."""
        return 3 * self.I * self.H + 3 * (self.I // 128) * (self.H // 128) * 4


# ---------------------------------------------------------------------------------------------------- MXFP4 tensors

def quant_mx4(w):
    """f32 [N][K] -> (e2m1 nibbles uint8 [N][K/2], the lower k in the low nibble; ue8m0 scale bytes uint8 [N][K/32]):
    scale = 2^ceil(log2(amax / 6)) per 32 along K, values rounded to nearest, ties to the even mantissa (ds41f
    ref/torchref/kernel.py:20-50, 86-100: the quantiser of its fp4 tensors)."""
    N, K = w.shape
    blk = w.float().view(N, K // 32, 32)
    v = blk.abs().amax(-1).clamp_min(6 * 2.0 ** -126) * torch.tensor(1.0 / 6.0, dtype=torch.float32, device=w.device)
    bits = v.view(torch.int32)
    e = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).to(torch.int32)          # the biased exponent of 2^ceil(log2 v)
    s = torch.ldexp(torch.ones_like(v), (e - 127).float())
    a = (blk / s[..., None]).clamp(-6.0, 6.0)
    mag = a.abs()
    code = torch.zeros_like(mag, dtype=torch.uint8)
    for thr, incl in ((0.25, False), (0.75, True), (1.25, False), (1.75, True), (2.5, False), (3.5, True), (5.0, False)):
        code += ((mag >= thr) if incl else (mag > thr)).to(torch.uint8)
    code |= ((a < 0) | ((a == 0) & torch.signbit(a))).to(torch.uint8) << 3
    code = code.view(N, K // 2, 2)
    return (code[..., 0] | code[..., 1] << 4).contiguous(), e.to(torch.uint8).contiguous()


def ue8m0_to_bf16_bits(s):
    """ue8m0 bytes -> the bf16 bit patterns of 2^(byte - 127): byte << 7, and 0x0040 (a subnormal) for byte 0."""
    s = s.to(torch.int32)
    return torch.where(s == 0, torch.full_like(s, 0x40), s << 7).to(torch.int16)


def _u32_bytes(v):
    """int64 values in [0, 2^32) -> their little-endian bytes (uint8, four a value)."""
    return torch.where(v >= 2 ** 31, v - 2 ** 32, v).to(torch.int32).view(torch.uint8)


def mx4_words(q):
    """canonical nibble bytes [N][K/2] -> the stored 32-bit words, as bytes [N][K/2]: the eight magnitude codes of
    k = 8 j .. 8 j + 7 stay in their nibbles; the sign of value i < 4 goes to bit 8 i + 7, of value i >= 4 to bit
    8 (i - 4) + 3 (where the kernels' e4m3 operands want them)."""
    w = q.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    out = w & 0x77777777
    for i in range(8):
        out |= ((w >> (4 * i + 3)) & 1) << (8 * i + 7 if i < 4 else 8 * (i - 4) + 3)
    return _u32_bytes(out)


def mx4_unwords(b):
    w = b.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    out = w & 0x77777777
    for i in range(8):
        out |= ((w >> (8 * i + 7 if i < 4 else 8 * (i - 4) + 3)) & 1) << (4 * i + 3)
    return _u32_bytes(out)


def tile_mx4(q, s):
    """canonical MXFP4 (nibble bytes [N][K/2], ue8m0 [N][K/32]) -> blocks of 8 rows x 128 k, 576 B, [N/8][K/128]:
    [32 lanes 4 g + t][4 groups G][one word (mx4_words): k = 128 b + 32 G + 8 t + 0..7 of row 8 n8 + g], then [8 g][4 G] the
    scales 2^(byte - 127) as bf16."""
    N, K = q.shape[0], q.shape[1] * 2
    v = mx4_words(q).view(N // 8, 8, K // 128, 4, 4, 4)      # n8, g, b, G, t, 4 bytes
    vals = v.permute(0, 2, 1, 4, 3, 5).contiguous().view(N // 8, K // 128, 512)   # n8, b, g, t, G, bytes
    sc = ue8m0_to_bf16_bits(s).view(N // 8, 8, K // 128, 4).permute(0, 2, 1, 3).contiguous().view(torch.uint8)
    return torch.cat([vals, sc.view(N // 8, K // 128, 64)], dim=-1).contiguous().view(-1)


def untile_mx4(m, N, K):
    blk = m.view(N // 8, K // 128, MX4_BLK)
    vals = mx4_unwords(blk[..., :512].reshape(N // 8, K // 128, 8, 4, 4, 4).permute(0, 2, 1, 4, 3, 5).contiguous().view(N, K // 2))
    sb = blk[..., 512:].contiguous().view(torch.int16).to(torch.int32) & 0xFFFF       # n8, b, g * 4 + G
    sc = torch.where(sb == 0x40, torch.zeros_like(sb), sb >> 7).to(torch.uint8)
    sc = sc.view(N // 8, K // 128, 8, 4).permute(0, 2, 1, 3).contiguous().view(N, K // 32)
    return vals, sc


MX4_BLK = 576


def mx4_mat_bytes(N, K):
    return (N // 8) * (K // 128) * MX4_BLK


class Mx4Layer(Fp8Layer):
    """One MXFP4 layer as ds41f stores it: `E` routed experts in e2m1 with a ue8m0 scale per 32 along K, and an FP8
    (128x128 block-scaled) shared expert, in one device pool."""

    def __init__(self, H, I, E, seed, device="cpu", shared=True, std=0.02, e_range=None, experts=None):
        """experts: the routed ids to generate (default: all of e_range); the others' descriptors stay empty."""
        self.H, self.I, self.E, self.fmt = H, I, E, _lib.FMT_MXFP4
        self.device = torch.device(device)
        mat8, sc8 = I * H, al256((I // 128) * (H // 128) * 4)
        mat4 = al256(mx4_mat_bytes(I, H))           # (gate, up and down have the same number of bytes)
        lo, hi = e_range if e_range is not None else (0, E)
        ids = list(range(lo, hi)) if experts is None else sorted(experts)
        self.pool = torch.empty(max(len(ids) * 3 * mat4 + (3 * mat8 + 3 * sc8 if shared else 0), 256), dtype=torch.uint8,
                                device=self.device)
        self.desc_host = (_lib.MatDesc * (E * 3))()
        self._off = {}
        for n, e in enumerate(ids):
            for m in range(3):
                N, K = (H, I) if m == 2 else (I, H)
                g = _gen(self.device, seed * 1000003 + e * 3 + m)
                w = torch.randn(N, K, generator=g, device=self.device, dtype=torch.float32) * std
                off = (n * 3 + m) * mat4
                self.pool[off:off + mx4_mat_bytes(N, K)] = tile_mx4(*quant_mx4(w))
                self._off[(e, m)] = (off, 0)
                d = self.desc_host[e * 3 + m]
                d.off, d.s2, d.fmt = off, 1.0, _lib.FMT_MXFP4
        if shared:
            base = len(ids) * 3 * mat4
            for m in range(3):
                N, K = (H, I) if m == 2 else (I, H)
                g = _gen(self.device, seed * 1000003 + E * 3 + m)
                w = torch.randn(N, K, generator=g, device=self.device, dtype=torch.float32) * std
                q, sc = quant_fp8_128(w)
                off, soff = base + m * mat8, base + 3 * mat8 + m * sc8
                self.pool[off:off + mat8] = tile_fp8(q)
                self.pool[soff:soff + sc.numel() * 4] = sc.view(-1).view(torch.uint8)
                self._off[(E, m)] = (off, soff)
        self.desc = torch.frombuffer(bytearray(bytes(self.desc_host)), dtype=torch.uint8).to(self.device)
        self.shared = shared

    def layer_w(self):
        L = super().layer_w()
        L.fmt = _lib.FMT_MXFP4
        return L

    def canonical(self, e):
        """Routed expert e: (wg, sg, wu, su, wd, sd) = nibble bytes [N][K/2] and ue8m0 bytes [N][K/32]; e == E: the FP8
        shared expert's tuple (Fp8Layer.canonical)."""
        if e == self.E:
            return super().canonical(e)
        out = []
        for m in range(3):
            N, K = (self.H, self.I) if m == 2 else (self.I, self.H)
            off, _ = self._off[(e, m)]
            q, sc = untile_mx4(self.pool[off:off + mx4_mat_bytes(N, K)], N, K)
            out += [q.cpu().numpy(), sc.cpu().numpy()]
        return tuple(out)

    def expert_bytes(self):
        """Algorithmic bytes of one routed expert: three matrices of e2m1 values with one scale byte per 32 (the stored
        blocks spend two bytes a scale: 576 instead of 544 bytes)."""
        return 3 * (self.I // 8) * (self.H // 128) * 544

    def shared_bytes(self):
        return 3 * self.I * self.H + 3 * (self.I // 128) * (self.H // 128) * 4


# ---------------------------------------------------------------------------------------------- router / activations

def router_weights(E, H, seed, device="cpu", std=0.02):
    g = _gen(device, seed)
    return torch.randn(E, H, generator=g, device=device, dtype=torch.float32) * std


def activations(M, H, seed, device="cpu"):
    g = _gen(device, seed)
    return torch.randn(M, H, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)


def bf16_bits(t):
    """torch bf16 tensor -> numpy uint16 bit patterns."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


# ----------------------------------------------------------------------------------------------------- INT4 tensors

def int4_tensors(N, K, seed):
    """Canonical symmetric INT4-g32 tensor (compressed-tensors pack-quantized order; altar1 engine/experts/layout.h:24-31):
    wp uint8 [N][K/2] (value k in byte k/2, low nibble = even k, stored nibble u = q + 8, q uniform in [-8, 7]) and
    bf16 scale bits [N][K/32] in [2^-9, 2^-7) with a random mantissa (the range of the reference's generator,
    tests/testdata.h:45-48); the zero point is 8 everywhere."""
    rng = np.random.default_rng(seed)
    wp = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    s = (((118 + rng.integers(0, 2, (N, K // 32))) << 7) | rng.integers(0, 128, (N, K // 32))).astype(np.uint16)
    return wp, s


def pack_int4_block(wp, s):
    """canonical symmetric INT4 (wp uint8 [N][K/2], s bf16 bits [N][K/32]) -> the engine's blocks of 8 rows x 512 k,
    2368 B each, [N/8][K/512] (altar1 engine/experts/layout.h:50-58, 78-95); the zero point is 8 everywhere."""
    N, K = wp.shape[0], wp.shape[1] * 2
    B = K // 512
    v = wp.reshape(N // 8, 8, B, 4, 2, 4, 8)                       # n8, g, b, jj, q, t, byte
    vals = np.ascontiguousarray(v.transpose(0, 2, 3, 1, 5, 4, 6)).reshape(N // 8, B, 2048)   # n8, b, jj, g, t, q, byte
    sc = s.reshape(N // 8, 8, B, 4, 2, 2)                          # n8, g, b, jj, q, h   (group 16 b + 4 jj + 2 q + h)
    sc = np.ascontiguousarray(sc.transpose(0, 2, 1, 5, 3, 4)).reshape(N // 8, B, 128)        # n8, b, g, h, jj, q
    out = np.empty((N // 8, B, 2368), np.uint8)
    out[:, :, :2048] = vals
    out[:, :, 2048:2304] = sc.view(np.uint8).reshape(N // 8, B, 256)
    out[:, :, 2304:] = 0x88
    return out.reshape(-1)


def tile_bf16(w):
    """bf16 bits [N][K] (torch int16 / numpy uint16) -> blocks of 8 rows x 128 k, 2048 B, [N/8][K/128]: the lane's 16 B
    at 512 p + 16 (4 g + t) are k = 64 (p >> 1) + 16 t + 8 (p & 1) + 0..7 (altar1 engine/experts/layout.h:96-107)."""
    N, K = w.shape
    v = w.reshape(N // 8, 8, K // 128, 2, 4, 2, 8)                  # n8, g, b, q, t, half, 8 values
    return np.ascontiguousarray(v.transpose(0, 2, 3, 5, 1, 4, 6)).reshape(-1).view(np.uint8)  # n8, b, q, half, g, t, 8


class Int4Layer:
    """One INT4-g32 layer: `E` routed experts in the engine's block layout + (optionally) a bf16 shared expert."""

    def __init__(self, H, I, E, seed, device="cpu", shared=True, e_range=None, experts=None):
        """experts: the ids to generate (default: all of e_range); the other experts' descriptors stay empty, so a step
        must not pick them (a test of a full-size layer generates only what its rows route to)."""
        self.H, self.I, self.E, self.fmt = H, I, E, _lib.FMT_INT4
        self.device = torch.device(device)
        shapes = ((I, H), (I, H), (H, I))
        mat_b = (I // 8) * (H // 512) * 2368
        assert mat_b == (H // 8) * (I // 512) * 2368 and mat_b % 256 == 0
        lo, hi = e_range if e_range is not None else (0, E)
        ids = [e for e in (range(lo, hi) if experts is None else sorted(set(experts))) if lo <= e < hi]
        self.raw = {}
        pool = np.empty(max(len(ids), 1) * 3 * mat_b, np.uint8)
        self.desc_host = (_lib.MatDesc * (E * 3))()
        for n, e in enumerate(ids):
            self.raw[e] = []
            for m, (N, K) in enumerate(shapes):
                wp, s = int4_tensors(N, K, seed * 1000 + e * 3 + m)
                self.raw[e].append((wp, s))
                off = (n * 3 + m) * mat_b
                pool[off:off + mat_b] = pack_int4_block(wp, s)
                d = self.desc_host[e * 3 + m]
                d.off, d.s2, d.fmt = off, 1.0, _lib.FMT_INT4
        self.pool = torch.from_numpy(pool).to(self.device)
        self.desc = torch.frombuffer(bytearray(bytes(self.desc_host)), dtype=torch.uint8).to(self.device)
        self.shared = shared
        if shared:
            self.sh_bits = [bf16_bits((torch.randn(n, k, generator=_gen("cpu", seed + 9 + i)) * 0.02).to(torch.bfloat16))
                            for i, (n, k) in enumerate(shapes)]
            self.sh_dev = [torch.from_numpy(tile_bf16(b)).to(self.device) for b in self.sh_bits]

    @classmethod
    def on_device(cls, H, I, E, seed, device, shared=True, e_range=None):
        """A layer of the same format and value ranges built straight in the block layout on the device (uniform
        nibbles, bf16 scales in [2^-9, 2^-7), zero point 8, bf16 shared expert N(0, 0.02)): for benchmarks of full-size
        layers, where packing 168 experts through numpy takes minutes.  It keeps no canonical copy for the oracle."""
        self = cls.__new__(cls)
        self.H, self.I, self.E, self.fmt = H, I, E, _lib.FMT_INT4
        self.device = torch.device(device)
        shapes = ((I, H), (I, H), (H, I))
        mat_b = (I // 8) * (H // 512) * 2368
        lo, hi = e_range if e_range is not None else (0, E)
        g = _gen(self.device, seed)
        nblk = max(hi - lo, 1) * 3 * mat_b // 2368
        pool = torch.empty(nblk, 2368, dtype=torch.uint8, device=self.device)
        pool[:, :2048] = torch.randint(0, 256, (nblk, 2048), generator=g, device=self.device, dtype=torch.uint8)
        sc = pool[:, 2048:2304].view(nblk, 128, 2)           # little-endian bf16: random mantissa, exponent of 2^-9..2^-8
        sc[:, :, 0] = torch.randint(0, 256, (nblk, 128), generator=g, device=self.device, dtype=torch.uint8)
        sc[:, :, 1] = 0x3B
        pool[:, 2304:] = 0x88
        self.pool = pool.view(-1)
        self.raw = {}
        self.desc_host = (_lib.MatDesc * (E * 3))()
        for n, e in enumerate(range(lo, hi)):
            for m in range(3):
                d = self.desc_host[e * 3 + m]
                d.off, d.s2, d.fmt = (n * 3 + m) * mat_b, 1.0, _lib.FMT_INT4
        self.desc = torch.frombuffer(bytearray(bytes(self.desc_host)), dtype=torch.uint8).to(self.device)
        self.shared = shared
        if shared:
            self.sh_dev = [(torch.randn(n * k, generator=g, device=self.device) * 0.02).to(torch.bfloat16).view(torch.uint8)
                           for n, k in shapes]   # any order of N(0, 0.02) values is a tiled N(0, 0.02) matrix
        return self

    def layer_w(self):
        L = _lib.LayerW()
        L.pool, L.desc, L.fmt = self.pool.data_ptr(), self.desc.data_ptr(), _lib.FMT_INT4
        if self.shared:
            L.sh.bg, L.sh.bu, L.sh.bd = (t.data_ptr() for t in self.sh_dev)
        return L

    def expert_bytes(self):
        return 3 * (self.I // 8) * (self.H // 512) * 2368

    def shared_bytes(self):
        return 3 * self.I * self.H * 2


class Bf16Layer(Int4Layer):
    """One BF16 layer (altar-1 keeps a few layers' routed experts in BF16; altar1 engine/experts/experts.h:28-39, format tag
    3): `E` routed experts and the shared expert in blocks of 8 rows x 128 k of bf16 (tile_bf16)."""

    def __init__(self, H, I, E, seed, device="cpu", shared=True, e_range=None, std=0.02):
        self.H, self.I, self.E, self.fmt = H, I, E, _lib.FMT_BF16
        self.device = torch.device(device)
        shapes = ((I, H), (I, H), (H, I))
        mat_b = I * H * 2
        lo, hi = e_range if e_range is not None else (0, E)
        self.bits = {}
        pool = np.empty(max(hi - lo, 1) * 3 * mat_b, np.uint8)
        self.desc_host = (_lib.MatDesc * (E * 3))()
        for n, e in enumerate(range(lo, hi)):
            self.bits[e] = []
            for m, (N, K) in enumerate(shapes):
                w = bf16_bits((torch.randn(N, K, generator=_gen("cpu", seed * 1000 + e * 3 + m)) * std).to(torch.bfloat16))
                self.bits[e].append(w)
                off = (n * 3 + m) * mat_b
                pool[off:off + mat_b] = tile_bf16(w)
                d = self.desc_host[e * 3 + m]
                d.off, d.s2, d.fmt = off, 1.0, _lib.FMT_BF16
        self.pool = torch.from_numpy(pool).to(self.device)
        self.desc = torch.frombuffer(bytearray(bytes(self.desc_host)), dtype=torch.uint8).to(self.device)
        self.shared = shared
        if shared:
            self.sh_bits = [bf16_bits((torch.randn(n, k, generator=_gen("cpu", seed + 9 + i)) * std).to(torch.bfloat16))
                            for i, (n, k) in enumerate(shapes)]
            self.sh_dev = [torch.from_numpy(tile_bf16(b)).to(self.device) for b in self.sh_bits]

    def layer_w(self):
        L = super().layer_w()
        L.fmt = _lib.FMT_BF16
        return L

    def expert_bytes(self):
        return 3 * self.I * self.H * 2


# ------------------------------------------------------------------------------------------- Zipf-skewed routing bias

def zipf_target_shares(E, topk, s=1.1):
    """Pick shares of E experts under Zipf(s), with no expert above 1 / topk of the picks (a token picks an expert at
    most once): the excess of the capped experts is spread over the others in proportion (water-filling)."""
    p = 1.0 / np.arange(1, E + 1) ** s
    p /= p.sum()
    cap = 1.0 / topk
    for _ in range(E):
        over = p > cap
        if not over.any():
            break
        excess = (p[over] - cap).sum()
        p[over] = cap
        p[~over] += excess * p[~over] / p[~over].sum()
    return p


def zipf_bias(E, alpha, seed, s=1.1):
    """Selection bias b_e = alpha * ln(p_e / p_max) over a seeded permutation of the experts, p_e ~ rank^-s."""
    p = 1.0 / np.arange(1, E + 1) ** s
    perm = np.random.default_rng(seed).permutation(E)
    b = np.empty(E, np.float32)
    b[perm] = (alpha * np.log(p / p.max())).astype(np.float32)
    return b


def calibrate_zipf_bias(route_counts, E, topk, seed, s=1.1, alphas=None):
    """route_counts(bias np.float32 [E]) -> pick counts [E].  Returns (alpha, bias, counts) whose sorted pick shares are
    closest (least squares) to zipf_target_shares: the realised histogram of a benchmark's routing follows Zipf(s)."""
    target = np.sort(zipf_target_shares(E, topk, s))[::-1]
    best = None
    for a in (alphas if alphas is not None else [0.005, 0.01, 0.015, 0.02, 0.03, 0.04, 0.06, 0.08, 0.12, 0.16, 0.24]):
        b = zipf_bias(E, a, seed, s)
        c = np.asarray(route_counts(b), np.float64)
        err = float(((np.sort(c / c.sum())[::-1] - target) ** 2).sum())
        if best is None or err < best[0]:
            best = (err, a, b, c)
    return best[1], best[2], best[3]
