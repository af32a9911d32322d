"""Random-init DeepSeek-V4-Flash for the token-loop benchmark: every tensor of
the architecture (reference-0731/config.json) is generated on the GPU with the
value distributions of the benchmark's single-operator configurations, and
handed to the C library as DEVICE pointers inside the same descriptors a host
loader would fill (the library uses device buffers in place).

The values come from the library's counter-based generator
(include/apus_synth.h), which has a host twin: the same model, or any layers
of it, can be regenerated in host memory for a CPU checker.  torch is used
here only as the device allocator; all arithmetic of the token loop is the
library's.
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


# tensor ids of the synthetic model (the `tensor` argument of apus_synth_key); the
# layer argument is the layer index, TOP for the tensors outside the blocks
TOP = 1000
TENSOR_IDS = {n: i for i, n in enumerate((
    "wq_a", "wq_a.s", "wq_b", "wq_b.s", "wkv", "wkv.s", "wo_b", "wo_b.s", "wo_a", "q_norm", "kv_norm", "sink",
    "comp.wkv", "comp.wgate", "comp.ape", "comp.norm", "idx.wkv", "idx.wgate", "idx.ape", "idx.norm",
    "idx_wq_b", "idx_wq_b.s", "idx_wproj", "gate_w", "gate_bias", "tid2eid",
    "w1", "w1.s", "w3", "w3.s", "w2", "w2.s", "sw1", "sw1.s", "sw3", "sw3.s", "sw2", "sw2.s",
    "attn_norm", "ffn_norm", "hc_attn_fn", "hc_attn_base", "hc_ffn_fn", "hc_ffn_base",
    "embed", "head", "norm", "hc_head_fn", "hc_head_base", "prompt",
    "e_proj", "e_proj.s", "h_proj", "h_proj.s", "enorm", "hnorm",
    "main_proj", "main_proj.s", "main_norm", "markov_w1", "markov_w2", "conf_proj"))}
# the MTP draft head's block is generated as layer MTP_LAYER + idx (c/mtp.h:223-226: "mtp.<idx>.*")
MTP_LAYER = 2000
# apus_synth.h kinds
K_U8, K_U8_RANGE, K_F32, K_F32_BF16, K_BF16, K_E4M3, K_I64_MOD, K_I64_SUBSET = range(8)


def prompt_ids(seed, first_seq, n_seq, n_prompt, vocab):
    """Prompt token ids [n_seq, n_prompt] of the sequences first_seq..: uniform over
    the vocabulary, one generator key per GLOBAL sequence index, so rank r of an
    N-rank job (sequences r*B..) and a single-GPU job agree on sequence 0..B-1."""
    import apus_b200
    L = apus_b200.lib()
    out = np.empty((n_seq, n_prompt), np.int64)
    for b in range(n_seq):
        key = L.apus_synth_key(seed, TOP, TENSOR_IDS["prompt"], first_seq + b)
        apus_b200.check(L.apus_synth_fill_host(out[b].ctypes.data, K_I64_MOD, n_prompt, key, float(vocab), 0.0, 1),
                        "synth_fill_host")
    return out


class RandomFlashModel:
    """All weights of the model (experts [e_lo, e_hi) only) plus the
    ApusCudaModelDesc that points at them.  Keeps every tensor alive.

    Every tensor is filled by the library's counter-based generator
    (include/apus_synth.h) from a key (seed, layer, tensor id, expert): with
    device = a CUDA device the tensors are generated in HBM and the descriptors
    carry device pointers (the library uses them in place); with device =
    "host" the SAME bits are generated into numpy arrays, which is how a CPU
    checker runs the reference on the identical model, whole or layer by layer.
    Ranks of an expert-parallel job build the same model by construction."""

    def __init__(self, cfg, seed, device, e_lo=0, e_hi=None, max_pos=1024, rope=None, layer_ids=None):
        import apus_b200
        self.lib = apus_b200.lib()
        self.check = apus_b200.check
        self.cfg, self.device = cfg, device
        self.host = device == "host"
        self.e_lo, self.e_hi = e_lo, cfg.n_experts if e_hi is None else e_hi
        self.keep = []
        self.named = {}                  # (layer, tensor name) -> the array / tensor that holds it
        self.bytes = 0
        self.seed = seed
        if not self.host:
            import torch
            self.torch = torch
            self.stream = torch.cuda.current_stream(device).cuda_stream
        # rope tables are inputs (host cos/sin); `rope` = {False: (cos, sin), True: (cos, sin)} overrides
        # the ones computed here, e.g. with the very tables a committed reference run used
        self.rope = rope or {c: rope_tables(cfg, c, max_pos) for c in (False, True)}
        # layer_ids: instantiate only these layers of the model (their true indices select
        # the kind, the routing mode and the generator keys), e.g. to check one layer on a CPU
        self.layer_ids = list(range(cfg.n_layers)) if layer_ids is None else list(layer_ids)
        descs = [self._layer(i, cfg.ratios[i]) for i in self.layer_ids]
        self._descs = (capi.LayerDesc * len(descs))(*descs)
        d = capi.ModelDesc()
        d.n_layers, d.dim, d.hc_mult, d.hc_sinkhorn_iters, d.vocab = (len(descs), cfg.dim, cfg.hc_mult,
                                                                      cfg.hc_iters, cfg.vocab)
        d.hc_eps, d.norm_eps = cfg.hc_eps, cfg.norm_eps
        d.layers = C.cast(self._descs, C.POINTER(capi.LayerDesc))
        hc, dim = cfg.hc_mult, cfg.dim
        d.embed, d.embed_bf16 = self._fill(TOP, "embed", K_BF16, (cfg.vocab, dim), 0.0, 1.0), 1
        d.head, d.head_bf16 = self._fill(TOP, "head", K_BF16, (cfg.vocab, dim), 0.0, 0.02), 1
        d.norm_w = self._fill(TOP, "norm", K_F32, (dim,), 1.0, 0.05)
        d.hc_head_fn = self._fill(TOP, "hc_head_fn", K_F32, (hc, hc * dim), 0.0, 0.01)
        d.hc_head_base = self._fill(TOP, "hc_head_base", K_F32, (hc,), 0.0, 0.5)
        d.hc_head_scale = 0.8
        self.desc = d
        if not self.host:
            self.torch.cuda.synchronize(device)

    # ---- tensor factory (device or host pointers) ---------------------------------------
    _NP = {K_U8: np.uint8, K_U8_RANGE: np.uint8, K_F32: np.float32, K_F32_BF16: np.float32, K_BF16: np.uint16,
           K_E4M3: np.uint8, K_I64_MOD: np.int64, K_I64_SUBSET: np.int64}

    def _alloc(self, shape, npdtype):
        if self.host:
            t = np.empty(shape, npdtype)
            p, nbytes = t.ctypes.data, t.nbytes
        else:
            torch = self.torch
            td = {np.uint8: torch.uint8, np.float32: torch.float32, np.uint16: torch.int16, np.int64: torch.int64}[npdtype]
            t = torch.empty(shape, device=self.device, dtype=td)
            p, nbytes = t.data_ptr(), t.numel() * t.element_size()
        self.keep.append(t)
        self.bytes += nbytes
        return t, p

    def _fill_at(self, ptr, layer, name, kind, n, a, b, expert=0):
        key = self.lib.apus_synth_key(self.seed, layer, TENSOR_IDS[name], expert)
        if self.host:
            self.check(self.lib.apus_synth_fill_host(ptr, kind, n, key, a, b, 0), "synth_fill_host")
        else:
            self.check(self.lib.apus_synth_fill_dev(ptr, kind, n, key, a, b, self.stream), "synth_fill_dev")

    def _fill(self, layer, name, kind, shape, a=0.0, b=0.0, expert=0):
        t, p = self._alloc(shape, self._NP[kind])
        self._fill_at(p, layer, name, kind, int(np.prod(shape)), a, b, expert)
        self.named[(layer, name)] = t
        return p

    def _const(self, values):
        if self.host:
            t = np.asarray(values, np.float32)
            self.keep.append(t)
            return t.ctypes.data
        t = self.torch.tensor(values, device=self.device, dtype=self.torch.float32)
        self.keep.append(t)
        return t.data_ptr()

    def _fp8(self, layer, name, O, K, std=0.02):
        """E4M3 codes of N(0, std) / 2^-7 with UE8M0 tile-scale bytes in {119, 120, 121}."""
        codes = self._fill(layer, name, K_E4M3, (O, K), 0.0, std * 128.0)
        scales = self._fill(layer, name + ".s", K_U8_RANGE, ((O + 127) // 128, K // 128), 119, 121)
        return capi.QW(codes, scales, O, K)

    def _fp4_slab(self, layer, name, O, K):
        """The local experts' MXFP4 matrices, expert-major: uniform nibbles, scale
        bytes uniform in [120, 126]; expert e has its own generator key."""
        n = self.e_hi - self.e_lo
        _, pc = self._alloc((n, O, K // 2), np.uint8)
        _, ps = self._alloc((n, O, K // 32), np.uint8)
        if not self.host and n:                # one launch per slab; the same bytes as the per-expert fills below
            T = TENSOR_IDS
            self.check(self.lib.apus_synth_fill_slab_dev(pc, K_U8, O * (K // 2), n, self.seed, layer, T[name], self.e_lo,
                                                         0.0, 0.0, self.stream), "synth_fill_slab_dev")
            self.check(self.lib.apus_synth_fill_slab_dev(ps, K_U8_RANGE, O * (K // 32), n, self.seed, layer, T[name + ".s"],
                                                         self.e_lo, 120.0, 126.0, self.stream), "synth_fill_slab_dev")
            return pc, ps
        for le in range(n):
            self._fill_at(pc + le * O * (K // 2), layer, name, K_U8, O * (K // 2), 0, 0, self.e_lo + le)
            self._fill_at(ps + le * O * (K // 32), layer, name + ".s", K_U8_RANGE, O * (K // 32), 120, 126,
                          self.e_lo + le)
        return pc, ps

    def mtp_desc(self, idx=0):
        """ApusCudaMtpDesc of MTP draft head `idx` (reference c/mtp.h:66-76): a sliding-window block
        with scored routing and the full expert set, the FP8 [dim, dim] e/h projections, the three
        norm weights and its own mHC head parameters -- random-init like everything else."""
        cfg, L = self.cfg, MTP_LAYER + idx
        dim, hc = cfg.dim, cfg.hc_mult
        d = capi.MtpDesc()
        d.block = self._layer(L, 0)
        d.e_proj, d.h_proj = self._fp8(L, "e_proj", dim, dim), self._fp8(L, "h_proj", dim, dim)
        d.enorm_w = self._fill(L, "enorm", K_F32, (dim,), 1.0, 0.05)
        d.hnorm_w = self._fill(L, "hnorm", K_F32, (dim,), 1.0, 0.05)
        d.norm_w = self._fill(L, "norm", K_F32, (dim,), 1.0, 0.05)
        d.hc_head_fn = self._fill(L, "hc_head_fn", K_F32, (hc, hc * dim), 0.0, 0.01)
        d.hc_head_base = self._fill(L, "hc_head_base", K_F32, (hc,), 0.0, 0.5)
        d.hc_head_scale = 0.8
        if not self.host:
            self.torch.cuda.synchronize(self.device)
        self.keep.append(d)
        return d

    def dspark_desc(self, n_stages=3, block_size=5, targets=(13, 27, 41), noise_id=0, rank=64):
        """ApusCudaDsparkDesc of a random-init DSpark draft module (reference c/dspark.h:88-107): `n_stages`
        sliding-window blocks generated as layers MTP_LAYER + k (stage 0 is the block the MTP head uses),
        the FP8 main projection over the mean hiddens of the `targets` layers, norms, the last stage's
        mHC head, the two bigram matrices and the confidence projection.  The checkpoint's own values of
        block size, targets and rank are not known here; these are stand-ins of the same shape."""
        cfg = self.cfg
        dim, hc, V = cfg.dim, cfg.hc_mult, cfg.vocab
        targets = [t for t in targets if t < cfg.n_layers] or [cfg.n_layers - 1]
        L = MTP_LAYER + n_stages - 1
        stages = [self._layer(MTP_LAYER + k, 0) for k in range(n_stages)]
        arr = (capi.LayerDesc * n_stages)(*stages)
        d = capi.DsparkDesc()
        d.n_stages, d.block_size, d.noise_id, d.markov_rank, d.n_targets = n_stages, block_size, noise_id, rank, len(targets)
        for i, t in enumerate(targets):
            d.targets[i] = t
        d.stages = C.cast(arr, C.POINTER(capi.LayerDesc))
        d.main_proj = self._fp8(MTP_LAYER, "main_proj", dim, len(targets) * dim)
        d.main_norm_w = self._fill(MTP_LAYER, "main_norm", K_F32, (dim,), 1.0, 0.05)
        d.norm_w = self._fill(L, "norm", K_F32, (dim,), 1.0, 0.05)
        d.hc_head_fn = self._fill(L, "hc_head_fn", K_F32, (hc, hc * dim), 0.0, 0.01)
        d.hc_head_base = self._fill(L, "hc_head_base", K_F32, (hc,), 0.0, 0.5)
        d.hc_head_scale = 0.8
        d.markov_w1 = self._fill(L, "markov_w1", K_F32_BF16, (V, rank), 0.0, 0.1)
        d.markov_w2 = self._fill(L, "markov_w2", K_F32_BF16, (V, rank), 0.0, 0.1)
        d.conf_proj = self._fill(L, "conf_proj", K_F32_BF16, (dim + rank,), 0.0, 0.02)
        if not self.host:
            self.torch.cuda.synchronize(self.device)
        self.keep += [arr, d]
        return d

    def mark(self):
        """A point to which drop() frees what was generated since (draft modules of a bench arm)."""
        return len(self.keep), self.bytes

    def drop(self, mark):
        del self.keep[mark[0]:]
        self.bytes = mark[1]
        for k in [k for k in self.named if k[0] >= MTP_LAYER]:
            del self.named[k]
        if not self.host:
            self.torch.cuda.empty_cache()

    # ---- one layer ----------------------------------------------------------------------------
    def _layer(self, i, ratio):
        cfg = self.cfg
        dim, h, hd = cfg.dim, cfg.n_heads, cfg.head_dim
        G, ol, ql = cfg.o_groups, cfg.o_lora, cfg.q_lora
        csa = ratio == 4
        acfg = capi.AttnCfg(dim, h, hd, cfg.rope_dim, ql, G, ol, cfg.window, ratio, int(csa), cfg.idx_heads,
                            cfg.idx_dim, cfg.idx_topk, cfg.norm_eps, 1 << 20)
        aw = capi.AttnW()
        aw.wq_a, aw.wq_b = self._fp8(i, "wq_a", ql, dim), self._fp8(i, "wq_b", h * hd, ql)
        aw.wkv, aw.wo_b = self._fp8(i, "wkv", hd, dim), self._fp8(i, "wo_b", dim, G * ol)
        aw.wo_a = self._fill(i, "wo_a", K_BF16, (G * ol, h * hd // G), 0.0, 0.02)
        aw.q_norm = self._fill(i, "q_norm", K_F32, (ql,), 1.0, 0.05)
        aw.kv_norm = self._fill(i, "kv_norm", K_F32, (hd,), 1.0, 0.05)
        aw.sink = self._fill(i, "sink", K_F32, (h,), 0.0, 0.5)

        def comp(pre, dd, overlap, rotate):
            cd = (1 + overlap) * dd
            return capi.CompW(self._fill(i, pre + ".wkv", K_F32_BF16, (cd, dim), 0.0, 0.02),
                              self._fill(i, pre + ".wgate", K_F32_BF16, (cd, dim), 0.0, 0.02),
                              self._fill(i, pre + ".ape", K_F32, (max(ratio, 1), cd), 0.0, 0.5),
                              self._fill(i, pre + ".norm", K_F32, (dd,), 1.0, 0.05),
                              ratio, overlap, dd, cfg.rope_dim, rotate, cfg.norm_eps)
        if ratio:
            aw.comp = comp("comp", hd, int(csa), 0)
        if csa:
            aw.idx_comp = comp("idx", cfg.idx_dim, 1, 1)
            aw.idx_wq_b = self._fp8(i, "idx_wq_b", cfg.idx_heads * cfg.idx_dim, ql)
            aw.idx_wproj = self._fill(i, "idx_wproj", K_F32_BF16, (cfg.idx_heads, dim), 0.0, 0.02)

        E, inter = cfg.n_experts, cfg.inter
        mw = capi.MoeW()
        mw.E, mw.topk, mw.inter, mw.dim = E, cfg.topk, inter, dim
        mw.hash = int(i < cfg.n_hash_layers)
        mw.route_scale, mw.limit = cfg.route_scale, cfg.swiglu_limit
        mw.gate_w = self._fill(i, "gate_w", K_F32_BF16, (E, dim), 0.0, 0.01)
        if mw.hash:
            mw.tid2eid = self._fill(i, "tid2eid", K_I64_SUBSET, (cfg.vocab, cfg.topk), float(E), float(cfg.topk))
        else:
            mw.gate_bias = self._fill(i, "gate_bias", K_F32, (E,), 0.0, 0.01)
        p1, s1 = self._fp4_slab(i, "w1", inter, dim)
        p3, s3 = self._fp4_slab(i, "w3", inter, dim)
        p2, s2 = self._fp4_slab(i, "w2", dim, inter)
        a1, a2, a3 = (capi.QW * E)(), (capi.QW * E)(), (capi.QW * E)()
        c13, z13 = inter * dim // 2, inter * dim // 32
        for e in range(self.e_lo, self.e_hi):
            le = e - self.e_lo
            a1[e] = capi.QW(p1 + le * c13, s1 + le * z13, inter, dim)
            a3[e] = capi.QW(p3 + le * c13, s3 + le * z13, inter, dim)
            a2[e] = capi.QW(p2 + le * c13, s2 + le * z13, dim, inter)
        self.keep += [a1, a2, a3]
        mw.w1, mw.w2, mw.w3 = (C.cast(a, C.POINTER(capi.QW)) for a in (a1, a2, a3))
        mw.sw1, mw.sw3 = self._fp8(i, "sw1", inter, dim), self._fp8(i, "sw3", inter, dim)
        mw.sw2 = self._fp8(i, "sw2", dim, inter)
        mw.layer_id = i

        hc = cfg.hc_mult
        nmix = (2 + hc) * hc
        d = capi.LayerDesc()
        d.acfg, d.aw, d.mw = acfg, aw, mw
        d.attn_norm_w = self._fill(i, "attn_norm", K_F32, (dim,), 1.0, 0.05)
        d.ffn_norm_w = self._fill(i, "ffn_norm", K_F32, (dim,), 1.0, 0.05)
        d.hc_attn_fn = self._fill(i, "hc_attn_fn", K_F32, (nmix, hc * dim), 0.0, 0.01)
        d.hc_attn_base = self._fill(i, "hc_attn_base", K_F32, (nmix,), 0.0, 0.5)
        d.hc_attn_scale = self._const([0.7, 1.3, 0.9])
        d.hc_ffn_fn = self._fill(i, "hc_ffn_fn", K_F32, (nmix, hc * dim), 0.0, 0.01)
        d.hc_ffn_base = self._fill(i, "hc_ffn_base", K_F32, (nmix,), 0.0, 0.5)
        d.hc_ffn_scale = self._const([0.7, 1.3, 0.9])
        cos, sin = self.rope[ratio != 0]
        d.cos, d.sin, d.rope_rows = capi.ptr(cos), capi.ptr(sin), cos.shape[0]
        return d
