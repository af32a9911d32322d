"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no checkpoint or dataset is involved anywhere).

Everything is numpy on the host; weights are generated once and uploaded.
The quantisers here only *produce inputs* (weights in the storage formats of
reference c/st.h:88-89); they are not on the measured path.
"""
import numpy as np

# V4-Flash dimensions (reference-0731/config.json).
DIM = 4096
INTER = 2048
N_EXPERTS = 256
TOPK = 6
ROUTE_SCALE = 1.5
SWIGLU_LIMIT = 10.0

_E4M3_VALUES = None


def e4m3_table():
    """f32 value of each E4M3 code 0..255 (reference c/fp4.h:255-260)."""
    global _E4M3_VALUES
    if _E4M3_VALUES is None:
        c = np.arange(256)
        e = (c >> 3) & 15
        m = c & 7
        mag = np.where(e > 0, (8 + m) * np.exp2(e - 10.0), m * np.exp2(-9.0))
        _E4M3_VALUES = np.where(c & 0x80, -mag, mag).astype(np.float32)
    return _E4M3_VALUES


def e4m3_quant(x):
    """Round-to-nearest-even f32 -> E4M3 codes with clamp to +-448."""
    x = np.asarray(x, dtype=np.float32)
    a = np.minimum(np.abs(x), np.float32(448.0))
    grid = e4m3_table()[:0x7F].astype(np.float64)          # codes 0..0x7e ascending
    idx = np.searchsorted(grid, a.astype(np.float64), side="left")
    idx = np.clip(idx, 1, len(grid) - 1)
    lo, hi = grid[idx - 1], grid[idx]
    d_lo, d_hi = a - lo, hi - a
    pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & ((idx & 1) == 0))
    code = np.where(pick_hi, idx, idx - 1).astype(np.uint8)
    code = np.where(a == 0, 0, code).astype(np.uint8)
    return code | (np.signbit(x).astype(np.uint8) << 7)


def bf16_round(x):
    """RNE to BF16, returned as f32 (reference c/fp4.h:262-270)."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def bf16_bits(x):
    return (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


def fp4_weight(rng, O, K, scale_lo=120, scale_hi=126):
    """MXFP4 matrix: E2M1 nibbles uniform over all 16 codes, one UE8M0 scale
    byte per 32 along K uniform in [scale_lo, scale_hi]."""
    packed = rng.integers(0, 256, size=(O, K // 2), dtype=np.uint8)
    scales = rng.integers(scale_lo, scale_hi + 1, size=(O, K // 32), dtype=np.uint8)
    return packed, scales


def fp8_weight(rng, O, K, std=0.02):
    """FP8 matrix: N(0, std) quantised to E4M3 per 128x128 tile with a
    power-of-two scale whose UE8M0 byte is uniform in {119, 120, 121}
    (= [0.5, 2] x 2^-7 restricted to powers of two, the storage the reference
    reads: c/fp8.h:11-14)."""
    w = (rng.standard_normal((O, K)) * std).astype(np.float32)
    tb = rng.integers(119, 122, size=((O + 127) // 128, (K + 127) // 128), dtype=np.uint8)
    s = np.exp2(tb.astype(np.float32) - 127.0)
    s_full = np.repeat(np.repeat(s, 128, axis=0)[:O], 128, axis=1)[:, :K]
    return e4m3_quant(w / s_full), tb


def activations(rng, T, K, std=1.0):
    """BF16-valued f32 activations ~ N(0, std)."""
    return bf16_round((rng.standard_normal((T, K)) * std).astype(np.float32))


class MoeWeights:
    """All tensors of one synthetic MoE sublayer (reference c/moe.h:37-63).

    Every expert is drawn from its own generator stream keyed by (seed, expert
    id), so a rank of an expert-parallel job can materialise only its shard
    [e_lo, e_hi) and still agree bit for bit with a full-size instance."""

    def __init__(self, seed=0, E=N_EXPERTS, dim=DIM, inter=INTER, topk=TOPK,
                 hash_vocab=0, route_scale=ROUTE_SCALE, limit=SWIGLU_LIMIT,
                 e_lo=0, e_hi=None):
        rng = np.random.default_rng([seed, 1 << 20])
        self.E, self.dim, self.inter, self.topk = E, dim, inter, topk
        self.route_scale, self.limit = route_scale, limit
        self.e_lo, self.e_hi = e_lo, E if e_hi is None else e_hi
        self.gate_w = bf16_round((rng.standard_normal((E, dim)) * 0.01).astype(np.float32))
        self.gate_bias = (rng.standard_normal(E) * 0.01).astype(np.float32)
        self.sw1 = fp8_weight(rng, inter, dim)
        self.sw3 = fp8_weight(rng, inter, dim)
        self.sw2 = fp8_weight(rng, dim, inter)
        self.tid2eid = None
        if hash_vocab:
            self.tid2eid = np.stack([rng.permutation(E)[:topk] for _ in range(hash_vocab)]
                                    ).astype(np.int64)
        # expert-major contiguous storage of the local shard, one slab per tensor
        nl = self.e_hi - self.e_lo
        self.w1p = np.empty((nl, inter, dim // 2), np.uint8)
        self.w1s = np.empty((nl, inter, dim // 32), np.uint8)
        self.w3p = np.empty((nl, inter, dim // 2), np.uint8)
        self.w3s = np.empty((nl, inter, dim // 32), np.uint8)
        self.w2p = np.empty((nl, dim, inter // 2), np.uint8)
        self.w2s = np.empty((nl, dim, inter // 32), np.uint8)
        for le in range(nl):
            er = np.random.default_rng([seed, self.e_lo + le])
            self.w1p[le], self.w1s[le] = fp4_weight(er, inter, dim)
            self.w3p[le], self.w3s[le] = fp4_weight(er, inter, dim)
            self.w2p[le], self.w2s[le] = fp4_weight(er, dim, inter)

    def expert_bytes(self):
        return (self.w1p[0].nbytes + self.w1s[0].nbytes + self.w3p[0].nbytes
                + self.w3s[0].nbytes + self.w2p[0].nbytes + self.w2s[0].nbytes)

    def moew(self):
        """Build the ApusMoeW view; keeps the expert arrays alive on self.
        Experts outside [e_lo, e_hi) get NULL views."""
        import ctypes as C
        from . import capi
        E = self.E
        self._a1 = (capi.QW * E)()
        self._a2 = (capi.QW * E)()
        self._a3 = (capi.QW * E)()
        for e in range(self.e_lo, self.e_hi):
            le = e - self.e_lo
            self._a1[e] = capi.qw(self.w1p[le], self.w1s[le], self.inter, self.dim)
            self._a3[e] = capi.qw(self.w3p[le], self.w3s[le], self.inter, self.dim)
            self._a2[e] = capi.qw(self.w2p[le], self.w2s[le], self.dim, self.inter)
        w = capi.MoeW()
        w.E, w.topk, w.inter, w.dim = E, self.topk, self.inter, self.dim
        w.hash = 1 if self.tid2eid is not None else 0
        w.route_scale, w.limit = self.route_scale, self.limit
        w.gate_w = capi.ptr(self.gate_w)
        w.gate_bias = None if w.hash else capi.ptr(self.gate_bias)
        w.tid2eid = capi.ptr(self.tid2eid) if w.hash else None
        w.w1 = C.cast(self._a1, C.POINTER(capi.QW))
        w.w2 = C.cast(self._a2, C.POINTER(capi.QW))
        w.w3 = C.cast(self._a3, C.POINTER(capi.QW))
        w.sw1 = capi.qw(self.sw1[0], self.sw1[1], self.inter, self.dim)
        w.sw3 = capi.qw(self.sw3[0], self.sw3[1], self.inter, self.dim)
        w.sw2 = capi.qw(self.sw2[0], self.sw2[1], self.dim, self.inter)
        w.layer_id = 0
        return w
