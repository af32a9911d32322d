"""Random-init DeepSeek-V4-Flash for the token-loop benchmark: every tensor of
the architecture (reference-0731/config.json) is generated on the GPU with the
value distributions of the benchmark's single-operator configurations, and
handed to the C library as DEVICE pointers inside the same descriptors a host
loader would fill (the library uses device buffers in place).

torch is used here only as the device allocator and random generator; all
arithmetic of the token loop is the library's.
"""
import ctypes as C
import math
from dataclasses import dataclass, field

import numpy as np

from . import capi


@dataclass
class FlashConfig:
    """Sizes of the real model (reference-0731/config.json; c/layer.h:32-43)."""
    dim: int = 4096
    n_heads: int = 64
    head_dim: int = 512
    rope_dim: int = 64
    q_lora: int = 1024
    o_groups: int = 8
    o_lora: int = 1024
    window: int = 128
    inter: int = 2048
    n_experts: int = 256
    topk: int = 6
    idx_heads: int = 64
    idx_dim: int = 128
    idx_topk: int = 512
    hc_mult: int = 4
    hc_iters: int = 20
    hc_eps: float = 1e-6
    norm_eps: float = 1e-6
    vocab: int = 129280
    n_layers: int = 43
    n_hash_layers: int = 3
    route_scale: float = 1.5
    swiglu_limit: float = 10.0
    rope_theta: float = 10000.0
    compress_rope_theta: float = 160000.0
    rope_factor: float = 16.0
    original_seq_len: int = 65536
    beta_fast: int = 32
    beta_slow: int = 1
    # per-layer compression ratio: 0 = sliding window, 4 = compressed sparse
    # (indexer), 128 = heavily compressed dense
    ratios: list = field(default_factory=lambda: [0, 0] + [4, 128] * 20 + [4])

    def layer_kinds(self):
        return [self.ratios[i] for i in range(self.n_layers)]


def rope_tables(cfg, compressed, rows):
    """cos/sin [rows, rope_dim/2] as the reference builds them (c/attn.h:247-281):
    f32 frequencies (YaRN ramp scalars in double for compressed layers), then
    cos/sin of the f32 angle."""
    dim = cfg.rope_dim
    half = dim // 2
    base = cfg.compress_rope_theta if compressed else cfg.rope_theta
    j = np.arange(half, dtype=np.float32)
    freqs = (np.float32(1.0) / np.power(np.float32(base), (2 * j) / np.float32(dim), dtype=np.float32)).astype(np.float32)
    if compressed and cfg.original_seq_len > 0:
        l2pi = 2.0 * math.pi
        low = math.floor(dim * math.log(cfg.original_seq_len / (cfg.beta_fast * l2pi)) / (2.0 * math.log(base)))
        high = math.ceil(dim * math.log(cfg.original_seq_len / (cfg.beta_slow * l2pi)) / (2.0 * math.log(base)))
        low, high = max(low, 0), min(high, dim - 1)
        if low == high:
            high += 0.001
        ramp = ((np.arange(half, dtype=np.float64) - low) / (high - low)).astype(np.float32)
        ramp = np.clip(ramp, np.float32(0), np.float32(1))
        smooth = (np.float32(1.0) - ramp).astype(np.float32)
        freqs = (freqs / np.float32(cfg.rope_factor) * (np.float32(1.0) - smooth) + freqs * smooth).astype(np.float32)
    ang = (np.arange(rows, dtype=np.float32)[:, None] * freqs[None, :]).astype(np.float32)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


class RandomFlashModel:
    """All weights of the model on one device (experts [e_lo, e_hi) only) plus
    the ApusCudaModelDesc that points at them.  Keeps every tensor alive."""

    def __init__(self, cfg, seed, device, e_lo=0, e_hi=None, max_pos=1024):
        import torch
        self.cfg, self.device = cfg, device
        self.e_lo, self.e_hi = e_lo, cfg.n_experts if e_hi is None else e_hi
        self.keep = []
        self.bytes = 0
        # replicated tensors come from one generator stream per layer and every
        # expert from its own stream keyed by (seed, layer, expert), so that the
        # ranks of an expert-parallel job hold the same model
        self.seed = seed
        self.g = torch.Generator(device=device)
        self.g.manual_seed(seed)
        self.ge = torch.Generator(device=device)
        self.torch = torch
        self.rope = {c: rope_tables(cfg, c, max_pos) for c in (False, True)}
        descs = [self._layer(i, r) for i, r in enumerate(cfg.layer_kinds())]
        self._descs = (capi.LayerDesc * cfg.n_layers)(*descs)
        self.g.manual_seed(self.seed * 1000003 + 999983)
        d = capi.ModelDesc()
        d.n_layers, d.dim, d.hc_mult, d.hc_sinkhorn_iters, d.vocab = (cfg.n_layers, cfg.dim, cfg.hc_mult,
                                                                      cfg.hc_iters, cfg.vocab)
        d.hc_eps, d.norm_eps = cfg.hc_eps, cfg.norm_eps
        d.layers = C.cast(self._descs, C.POINTER(capi.LayerDesc))
        hc, dim = cfg.hc_mult, cfg.dim
        d.embed, d.embed_bf16 = self._bf16((cfg.vocab, dim), 1.0), 1
        d.head, d.head_bf16 = self._bf16((cfg.vocab, dim), 0.02), 1
        d.norm_w = self._f32((dim,), 0.05, 1.0)
        d.hc_head_fn = self._f32((hc, hc * dim), 0.01)
        d.hc_head_base = self._f32((hc,), 0.5)
        d.hc_head_scale = 0.8
        self.desc = d

    # ---- tensor factories (device pointers) ------------------------------------------
    def _hold(self, t):
        self.keep.append(t)
        self.bytes += t.numel() * t.element_size()
        return t.data_ptr()

    def _f32(self, shape, std, mean=0.0, bf16=False):
        torch = self.torch
        t = torch.randn(shape, generator=self.g, device=self.device, dtype=torch.float32) * std + mean
        if bf16:                        # f32 storage carrying BF16 values, like the reference's widened tensors
            t = t.to(torch.bfloat16).to(torch.float32)
        return self._hold(t.contiguous())

    def _bf16(self, shape, std):
        torch = self.torch
        t = (torch.randn(shape, generator=self.g, device=self.device, dtype=torch.float32) * std).to(torch.bfloat16)
        return self._hold(t.view(torch.int16).contiguous())

    def _bytes(self, shape, lo, hi):
        torch = self.torch
        return self._hold(torch.randint(lo, hi, shape, generator=self.g, device=self.device, dtype=torch.uint8))

    def _fp8(self, O, K, std=0.02):
        """E4M3 codes of N(0, std) / 2^-7 with UE8M0 tile-scale bytes in {119, 120, 121}."""
        torch = self.torch
        w = torch.randn((O, K), generator=self.g, device=self.device, dtype=torch.float32) * (std * 128.0)
        codes = w.to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
        del w
        scales = torch.randint(119, 122, ((O + 127) // 128, K // 128), generator=self.g, device=self.device,
                               dtype=torch.uint8)
        return capi.QW(self._hold(codes), self._hold(scales), O, K)

    def _fp4_slab(self, layer, which, O, K):
        """The local experts' MXFP4 matrices, expert-major: uniform nibbles, scale
        bytes uniform in [120, 126]; expert e is drawn from its own stream."""
        torch = self.torch
        n = self.e_hi - self.e_lo
        codes = torch.empty((n, O, K // 2), device=self.device, dtype=torch.uint8)
        scales = torch.empty((n, O, K // 32), device=self.device, dtype=torch.uint8)
        for le in range(n):
            self.ge.manual_seed(((self.seed * 64 + layer) * 1024 + self.e_lo + le) * 4 + which)
            codes[le].random_(0, 256, generator=self.ge)
            scales[le].random_(120, 127, generator=self.ge)
        return self._hold(codes), self._hold(scales)

    # ---- one layer ----------------------------------------------------------------------------
    def _layer(self, i, ratio):
        cfg, torch = self.cfg, self.torch
        self.g.manual_seed(self.seed * 1000003 + i)
        dim, h, hd = cfg.dim, cfg.n_heads, cfg.head_dim
        G, ol, ql = cfg.o_groups, cfg.o_lora, cfg.q_lora
        csa = ratio == 4
        acfg = capi.AttnCfg(dim, h, hd, cfg.rope_dim, ql, G, ol, cfg.window, ratio, int(csa), cfg.idx_heads,
                            cfg.idx_dim, cfg.idx_topk, cfg.norm_eps, 1 << 20)
        aw = capi.AttnW()
        aw.wq_a, aw.wq_b = self._fp8(ql, dim), self._fp8(h * hd, ql)
        aw.wkv, aw.wo_b = self._fp8(hd, dim), self._fp8(dim, G * ol)
        aw.wo_a = self._bf16((G * ol, h * hd // G), 0.02)
        aw.q_norm, aw.kv_norm = self._f32((ql,), 0.05, 1.0), self._f32((hd,), 0.05, 1.0)
        aw.sink = self._f32((h,), 0.5)

        def comp(dd, overlap, rotate):
            cd = (1 + overlap) * dd
            return capi.CompW(self._f32((cd, dim), 0.02, bf16=True), self._f32((cd, dim), 0.02, bf16=True),
                              self._f32((max(ratio, 1), cd), 0.5), self._f32((dd,), 0.05, 1.0),
                              ratio, overlap, dd, cfg.rope_dim, rotate, cfg.norm_eps)
        if ratio:
            aw.comp = comp(hd, int(csa), 0)
        if csa:
            aw.idx_comp = comp(cfg.idx_dim, 1, 1)
            aw.idx_wq_b = self._fp8(cfg.idx_heads * cfg.idx_dim, ql)
            aw.idx_wproj = self._f32((cfg.idx_heads, dim), 0.02, bf16=True)

        E, inter, nl = cfg.n_experts, cfg.inter, self.e_hi - self.e_lo
        mw = capi.MoeW()
        mw.E, mw.topk, mw.inter, mw.dim = E, cfg.topk, inter, dim
        mw.hash = int(i < cfg.n_hash_layers)
        mw.route_scale, mw.limit = cfg.route_scale, cfg.swiglu_limit
        mw.gate_w = self._f32((E, dim), 0.01, bf16=True)
        if mw.hash:
            t = torch.rand((cfg.vocab, E), generator=self.g, device=self.device).argsort(dim=1)[:, :cfg.topk]
            mw.tid2eid = self._hold(t.to(torch.int64).contiguous())
        else:
            mw.gate_bias = self._f32((E,), 0.01)
        p1, s1 = self._fp4_slab(i, 0, inter, dim)
        p3, s3 = self._fp4_slab(i, 1, inter, dim)
        p2, s2 = self._fp4_slab(i, 2, dim, inter)
        a1, a2, a3 = (capi.QW * E)(), (capi.QW * E)(), (capi.QW * E)()
        c13, z13 = inter * dim // 2, inter * dim // 32
        for e in range(self.e_lo, self.e_hi):
            le = e - self.e_lo
            a1[e] = capi.QW(p1 + le * c13, s1 + le * z13, inter, dim)
            a3[e] = capi.QW(p3 + le * c13, s3 + le * z13, inter, dim)
            a2[e] = capi.QW(p2 + le * c13, s2 + le * z13, dim, inter)
        self.keep += [a1, a2, a3]
        mw.w1, mw.w2, mw.w3 = (C.cast(a, C.POINTER(capi.QW)) for a in (a1, a2, a3))
        mw.sw1, mw.sw3, mw.sw2 = self._fp8(inter, dim), self._fp8(inter, dim), self._fp8(dim, inter)
        mw.layer_id = i

        hc = cfg.hc_mult
        nmix = (2 + hc) * hc
        d = capi.LayerDesc()
        d.acfg, d.aw, d.mw = acfg, aw, mw
        d.attn_norm_w, d.ffn_norm_w = self._f32((dim,), 0.05, 1.0), self._f32((dim,), 0.05, 1.0)
        d.hc_attn_fn, d.hc_attn_base = self._f32((nmix, hc * dim), 0.01), self._f32((nmix,), 0.5)
        d.hc_attn_scale = self._hold(torch.tensor([0.7, 1.3, 0.9], device=self.device))
        d.hc_ffn_fn, d.hc_ffn_base = self._f32((nmix, hc * dim), 0.01), self._f32((nmix,), 0.5)
        d.hc_ffn_scale = self._hold(torch.tensor([0.7, 1.3, 0.9], device=self.device))
        cos, sin = self.rope[ratio != 0]
        d.cos, d.sin, d.rope_rows = capi.ptr(cos), capi.ptr(sin), cos.shape[0]
        return d
