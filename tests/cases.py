"""Small seeded parity cases shared by the golden-vector generator and the tests.

Each case builder returns a dict of numpy inputs; they are deterministic in the
seed, so the committed golden file only stores the reference's outputs.
"""
import numpy as np

from apus_b200 import synth


def linear_case(seed, fmt, M, O, K, edge=False):
    rng = np.random.default_rng(seed)
    if fmt == 4:
        codes, scales = synth.fp4_weight(rng, O, K, 118, 130)
        if edge:                      # scale-byte corners: 0 (2^-127), 1, 254
            scales[0, 0] = 0
            scales[1, 1] = 1
            scales[2, 0] = 254
            codes[3, :16] = 0         # an all-zero block
            codes[4, :16] = 0xFF      # all -6
    else:
        codes, scales = synth.fp8_weight(rng, O, K, std=0.05)
        if edge:
            scales[0, 0] = 0
            scales[-1, -1] = 1
            scales[0, -1] = 200
    x = synth.activations(rng, M, K, std=3.0)
    if edge and M > 1:
        x[1, :] = 0.0                 # all-zero row -> amax floor
        x[-1, K // 2:] *= 100.0       # large second half
    return dict(codes=codes, scales=scales, x=x)


def expert_case(seed, kind, rows, dim, inter):
    rng = np.random.default_rng(seed)
    if kind == 0:
        w1, w3 = synth.fp4_weight(rng, inter, dim), synth.fp4_weight(rng, inter, dim)
        w2 = synth.fp4_weight(rng, dim, inter)
    else:
        w1, w3 = synth.fp8_weight(rng, inter, dim), synth.fp8_weight(rng, inter, dim)
        w2 = synth.fp8_weight(rng, dim, inter)
    x = synth.activations(rng, rows, dim)
    return dict(w1=w1, w2=w2, w3=w3, x=x)


def moe_case(seed, s, E=16, topk=3, dim=256, inter=128, hash_vocab=0):
    W = synth.MoeWeights(seed=seed, E=E, dim=dim, inter=inter, topk=topk, hash_vocab=hash_vocab)
    rng = np.random.default_rng(seed + 1000)
    x = synth.activations(rng, s, dim)
    ids = rng.integers(0, max(hash_vocab, 1), size=s).astype(np.int64)
    return W, x, ids


def topk_case(seed, rows, n, k, ties):
    rng = np.random.default_rng(seed)
    sc = rng.standard_normal((rows, n)).astype(np.float32)
    if ties:                          # BF16-rounded scores: ties everywhere
        sc = synth.bf16_round(sc)
        sc[0, : n // 3] = -np.inf     # masked prefix
        if rows > 1:
            sc[1, :] = 0.25           # one value only
    return sc


def sparse_attn_case(seed, s, h, d, na, nb, idxw, pattern):
    rng = np.random.default_rng(seed)
    q = synth.activations(rng, s * h, d).reshape(s, h, d)
    kv_a = synth.activations(rng, max(na, 1), d)[:na]
    kv_b = synth.activations(rng, max(nb, 1), d)[:nb]
    sink = (rng.standard_normal(h) * 0.5).astype(np.float32)
    idx = np.full((s, idxw), -1, np.int32)
    tot = na + nb
    for t in range(s):
        if pattern == "empty" and t == 0:
            continue
        n = int(rng.integers(1, idxw + 1))
        if pattern == "full":
            n = idxw
        ids = rng.integers(0, tot, size=n)
        if pattern == "dups":
            ids[: n // 2] = ids[0]
        pos = np.sort(rng.choice(idxw, size=n, replace=False)) if pattern == "holes" \
            else np.arange(n)
        idx[t, pos] = ids
    return dict(q=q, kv_a=kv_a, kv_b=kv_b, sink=sink, idx=idx)


def mhc_case(seed, rows, d, n=4):
    rng = np.random.default_rng(seed)
    nmix = (2 + n) * n
    x4 = synth.activations(rng, rows, n * d, std=1.5)
    fn = (rng.standard_normal((nmix, n * d)) * 0.05).astype(np.float32)
    scale = np.array([0.7, 1.3, 0.9], np.float32)
    base = (rng.standard_normal(nmix) * 0.5).astype(np.float32)
    hfn = (rng.standard_normal((n, n * d)) * 0.05).astype(np.float32)
    hbase = (rng.standard_normal(n) * 0.5).astype(np.float32)
    f = synth.activations(rng, rows, d)
    norm_w = (1.0 + 0.05 * rng.standard_normal(d)).astype(np.float32)
    return dict(x4=x4, fn=fn, scale=scale, base=base, hfn=hfn, hbase=hbase, f=f, norm_w=norm_w)


# ---- attention sublayer ------------------------------------------------------------------
ATTN_DIMS = dict(dim=256, n_heads=4, head_dim=128, rope_dim=64, q_lora=128, o_groups=2, o_lora=128,
                 window=8, idx_heads=4, idx_dim=128, idx_topk=4, max_pos=256)


class AttnLayer:
    """Synthetic weights + ctypes views of one attention sublayer (reference
    c/attn.h:114-143).  kind: 'swa' (ratio 0), 'csa' (ratio 4 + indexer),
    'hca' (dense compressed attention, ratio 8 here instead of 128 so that a
    short sequence completes several blocks)."""

    def __init__(self, seed, kind, dims=None):
        from apus_b200 import capi
        D = dict(ATTN_DIMS)
        D.update(dims or {})
        self.D, self.kind = D, kind
        rng = np.random.default_rng(seed)
        ratio = {"swa": 0, "csa": 4, "hca": 8, "hca128": 128}[kind]
        self.ratio = ratio
        dim, h, d, ql = D["dim"], D["n_heads"], D["head_dim"], D["q_lora"]
        G, ol, ih, idm = D["o_groups"], D["o_lora"], D["idx_heads"], D["idx_dim"]
        hd = h * d
        f8 = lambda O, K, std: synth.fp8_weight(rng, O, K, std=std)
        self.wq_a, self.wq_b = f8(ql, dim, 0.06), f8(hd, ql, 0.09)
        self.wkv, self.wo_b = f8(d, dim, 0.06), f8(dim, G * ol, 0.06)
        self.wo_a = synth.bf16_bits((rng.standard_normal((G * ol, hd // G)) * 0.04).astype(np.float32))
        nrm = lambda n: (1 + 0.05 * rng.standard_normal(n)).astype(np.float32)
        self.q_norm, self.kv_norm = nrm(ql), nrm(d)
        self.sink = (rng.standard_normal(h) * 0.5).astype(np.float32)
        bfw = lambda *s, std=0.05: synth.bf16_round((rng.standard_normal(s) * std).astype(np.float32))

        def comp(dd, overlap):
            cd = (1 + overlap) * dd
            return dict(wkv=bfw(cd, dim), wgate=bfw(cd, dim), ape=(rng.standard_normal((max(ratio, 1), cd)) * 0.5
                                                                ).astype(np.float32), norm=nrm(dd))
        self.comp = comp(d, int(ratio == 4))
        self.idx_comp = comp(idm, 1)
        self.idx_wq_b = f8(ih * idm, ql, 0.09)
        self.idx_wproj = bfw(ih, dim)
        cfg = capi.AttnCfg(dim, h, d, D["rope_dim"], ql, G, ol, D["window"], ratio, int(kind == "csa"), ih, idm,
                           D["idx_topk"], 1e-6, D["max_pos"])
        w = capi.AttnW()
        w.wq_a, w.wq_b = capi.qw(*self.wq_a, ql, dim), capi.qw(*self.wq_b, hd, ql)
        w.wkv, w.wo_b = capi.qw(*self.wkv, d, dim), capi.qw(*self.wo_b, dim, G * ol)
        w.wo_a, w.q_norm, w.kv_norm, w.sink = (capi.ptr(self.wo_a), capi.ptr(self.q_norm),
                                               capi.ptr(self.kv_norm), capi.ptr(self.sink))

        def cw(c, dd, overlap, rotate):
            return capi.CompW(capi.ptr(c["wkv"]), capi.ptr(c["wgate"]), capi.ptr(c["ape"]), capi.ptr(c["norm"]),
                              ratio, overlap, dd, D["rope_dim"], rotate, 1e-6)
        w.comp = cw(self.comp, d, int(ratio == 4), 0)
        w.idx_comp = cw(self.idx_comp, idm, 1, 1)
        w.idx_wq_b = capi.qw(*self.idx_wq_b, ih * idm, ql)
        w.idx_wproj = capi.ptr(self.idx_wproj)
        self.cfg, self.w = cfg, w

    def weight_ptrs(self):
        """Host addresses the backend may have cached device copies for."""
        arrs = [self.wq_a[0], self.wq_b[0], self.wkv[0], self.wo_b[0], self.wo_a, self.q_norm, self.kv_norm,
                self.sink, self.idx_wq_b[0], self.idx_wproj]
        for c in (self.comp, self.idx_comp):
            arrs += [c["wkv"], c["wgate"], c["ape"], c["norm"]]
        return arrs


class AttnState:
    """Host-side ApusAttnS built from numpy arrays (reference c/attn.h:747-760,
    1494-1504)."""

    def __init__(self, L):
        from apus_b200 import capi
        D, ratio = L.D, L.ratio
        self.win = np.zeros((D["window"], D["head_dim"]), np.float32)
        st = capi.AttnS()
        st.pos = 0
        st.win = capi.ptr(self.win)
        self.keep = []

        def comp(dd, overlap):
            coff = 1 + overlap
            rows, cols = coff * ratio, coff * dd
            kv = np.zeros((rows, cols), np.float32)
            sc = np.full((rows, cols), -np.inf, np.float32)
            max_nb = D["max_pos"] // ratio + 2
            cache = np.zeros((max_nb, dd), np.float32)
            self.keep += [kv, sc, cache]
            return capi.CompS(rows, cols, capi.ptr(kv), capi.ptr(sc), capi.ptr(cache), 0, max_nb, dd, max_nb), \
                (kv, sc, cache)
        if ratio:
            st.comp, self.comp = comp(D["head_dim"], int(ratio == 4))
            if L.kind == "csa":
                st.idx_comp, self.idx = comp(D["idx_dim"], 1)
        self.st = st


def attn_inputs(seed, n_tokens, dim):
    rng = np.random.default_rng(seed)
    return synth.activations(rng, n_tokens, dim)


# ---- block / model ------------------------------------------------------------------------
MODEL_DIMS = dict(hc=4, iters=20, hc_eps=1e-6, norm_eps=1e-6, vocab=384, E=8, topk=2, inter=128)
# one block at the real model's sizes (reference-0731/config.json) with 8 routed experts
FLASH_ATTN_DIMS = dict(dim=4096, n_heads=64, head_dim=512, rope_dim=64, q_lora=1024, o_groups=8, o_lora=1024,
                       window=128, idx_heads=64, idx_dim=128, idx_topk=512, max_pos=256)
FLASH_MOE_DIMS = dict(E=8, topk=6, inter=2048)


class BlockLayer:
    """One full block (reference c/layer.h:45-71): attention sublayer, MoE
    sublayer, the two RMSNorm weights and the two sets of mHC mixing
    parameters, plus the ApusCudaLayerDesc that points at them.  cos/sin are
    the reference's rope tables for this layer kind (read from the committed
    golden file; the reference builds them in c/layer.h:167-190)."""

    def __init__(self, seed, kind, cos, sin, hash_vocab=0, dims=None, attn_dims=None):
        from apus_b200 import capi
        M = dict(MODEL_DIMS)
        M.update(dims or {})
        self.M = M
        self.attn = AttnLayer(seed, kind, attn_dims)
        dim, hc = self.attn.D["dim"], M["hc"]
        self.moe = synth.MoeWeights(seed=seed + 500, E=M["E"], dim=dim, inter=M["inter"], topk=M["topk"],
                                    hash_vocab=hash_vocab)
        rng = np.random.default_rng(seed + 900)
        nmix = (2 + hc) * hc
        nrm = lambda n: (1 + 0.05 * rng.standard_normal(n)).astype(np.float32)
        self.attn_norm_w, self.ffn_norm_w = nrm(dim), nrm(dim)
        mk = lambda: ((rng.standard_normal((nmix, hc * dim)) * 0.05).astype(np.float32),
                      (rng.standard_normal(nmix) * 0.5).astype(np.float32),
                      (np.array([0.7, 1.3, 0.9], np.float32) * (1 + 0.1 * rng.standard_normal(3))).astype(np.float32))
        self.hc_attn, self.hc_ffn = mk(), mk()
        self.cos, self.sin = np.ascontiguousarray(cos), np.ascontiguousarray(sin)
        d = capi.LayerDesc()
        d.acfg, d.aw, d.mw = self.attn.cfg, self.attn.w, self.moe.moew()
        d.attn_norm_w, d.ffn_norm_w = capi.ptr(self.attn_norm_w), capi.ptr(self.ffn_norm_w)
        d.hc_attn_fn, d.hc_attn_base, d.hc_attn_scale = (capi.ptr(a) for a in self.hc_attn)
        d.hc_ffn_fn, d.hc_ffn_base, d.hc_ffn_scale = (capi.ptr(a) for a in self.hc_ffn)
        d.cos, d.sin, d.rope_rows = capi.ptr(self.cos), capi.ptr(self.sin), self.cos.shape[0]
        self.desc = d


class TinyModel:
    """A few blocks + embedding, final norm, mHC head and BF16 vocabulary head
    (reference c/model.h:58-84) at toy sizes: layer 0 sliding-window with hash
    routing, then compressed-sparse (indexer) and dense-compressed layers,
    i.e. every layer kind of the real model once."""

    KINDS = ("swa", "csa", "hca", "swa")

    def __init__(self, seed, rope, n_layers=3):
        from apus_b200 import capi
        M = dict(MODEL_DIMS)
        self.M = M
        dim, hc, V = ATTN_DIMS["dim"], M["hc"], M["vocab"]
        self.layers = []
        for i in range(n_layers):
            kind = self.KINDS[i % len(self.KINDS)]
            cos, sin = rope["plain" if kind == "swa" else "yarn"]
            self.layers.append(BlockLayer(seed + 10 * i, kind, cos, sin, hash_vocab=V if i == 0 else 0))
        rng = np.random.default_rng(seed + 77)
        self.embed = synth.bf16_bits(rng.standard_normal((V, dim)).astype(np.float32))
        self.head = synth.bf16_bits((rng.standard_normal((V, dim)) * 0.05).astype(np.float32))
        self.norm_w = (1 + 0.05 * rng.standard_normal(dim)).astype(np.float32)
        self.hc_head_fn = (rng.standard_normal((hc, hc * dim)) * 0.05).astype(np.float32)
        self.hc_head_base = (rng.standard_normal(hc) * 0.5).astype(np.float32)
        self._descs = (capi.LayerDesc * n_layers)(*[L.desc for L in self.layers])
        d = capi.ModelDesc()
        d.n_layers, d.dim, d.hc_mult, d.hc_sinkhorn_iters, d.vocab = n_layers, dim, hc, M["iters"], V
        d.hc_eps, d.norm_eps = M["hc_eps"], M["norm_eps"]
        import ctypes as C
        d.layers = C.cast(self._descs, C.POINTER(capi.LayerDesc))
        d.embed, d.embed_bf16, d.head, d.head_bf16 = capi.ptr(self.embed), 1, capi.ptr(self.head), 1
        d.norm_w, d.hc_head_fn, d.hc_head_base = capi.ptr(self.norm_w), capi.ptr(self.hc_head_fn), \
            capi.ptr(self.hc_head_base)
        d.hc_head_scale = 0.8
        self.desc = d

    def states(self):
        """Fresh host attention states, one per layer, as a contiguous ApusAttnS array."""
        from apus_b200 import capi
        S = [AttnState(L.attn) for L in self.layers]
        arr = (capi.AttnS * len(S))(*[s.st for s in S])
        return S, arr


class TinyMtp:
    """The MTP draft head of a TinyModel (reference c/mtp.h:66-76): one more sliding-window block
    with scored routing, the two FP8 [dim, dim] projections, three norm weights and its own
    mHC head parameters."""

    def __init__(self, seed, rope):
        from apus_b200 import capi
        M = dict(MODEL_DIMS)
        dim, hc = ATTN_DIMS["dim"], M["hc"]
        cos, sin = rope["plain"]
        self.block = BlockLayer(seed, "swa", cos, sin)
        rng = np.random.default_rng(seed + 31)
        self.e_proj, self.h_proj = synth.fp8_weight(rng, dim, dim, std=0.06), synth.fp8_weight(rng, dim, dim, std=0.06)
        nrm = lambda n: (1 + 0.05 * rng.standard_normal(n)).astype(np.float32)
        self.enorm_w, self.hnorm_w, self.norm_w = nrm(dim), nrm(dim), nrm(dim)
        self.hc_head_fn = (rng.standard_normal((hc, hc * dim)) * 0.05).astype(np.float32)
        self.hc_head_base = (rng.standard_normal(hc) * 0.5).astype(np.float32)
        d = capi.MtpDesc()
        d.block = self.block.desc
        d.e_proj, d.h_proj = capi.qw(*self.e_proj, dim, dim), capi.qw(*self.h_proj, dim, dim)
        d.enorm_w, d.hnorm_w, d.norm_w = capi.ptr(self.enorm_w), capi.ptr(self.hnorm_w), capi.ptr(self.norm_w)
        d.hc_head_fn, d.hc_head_base, d.hc_head_scale = capi.ptr(self.hc_head_fn), capi.ptr(self.hc_head_base), 0.9
        self.desc = d

    def state(self):
        S = AttnState(self.block.attn)
        return S, S.st


class TinyDspark:
    """The DSpark draft module of a TinyModel (reference c/dspark.h:88-107): `n_stages` sliding-window blocks
    with scored routing, the FP8 [dim, n_targets * dim] main projection and its norm, the last stage's norm
    and mHC head, the two [vocab, rank] bigram matrices and the confidence projection."""

    def __init__(self, seed, rope, targets, n_stages=2, block_size=3, noise_id=5, rank=16):
        import ctypes as C
        from apus_b200 import capi
        M = dict(MODEL_DIMS)
        dim, hc, V = ATTN_DIMS["dim"], M["hc"], M["vocab"]
        cos, sin = rope["plain"]
        self.stages = [BlockLayer(seed + 10 * k, "swa", cos, sin) for k in range(n_stages)]
        rng = np.random.default_rng(seed + 57)
        nt = len(targets)
        self.main_proj = synth.fp8_weight(rng, dim, nt * dim, std=0.05)
        nrm = lambda n: (1 + 0.05 * rng.standard_normal(n)).astype(np.float32)
        self.main_norm_w, self.norm_w = nrm(dim), nrm(dim)
        self.hc_head_fn = (rng.standard_normal((hc, hc * dim)) * 0.05).astype(np.float32)
        self.hc_head_base = (rng.standard_normal(hc) * 0.5).astype(np.float32)
        bf = lambda *sh, std: synth.bf16_round((rng.standard_normal(sh) * std).astype(np.float32))
        self.markov_w1, self.markov_w2 = bf(V, rank, std=0.5), bf(V, rank, std=0.5)
        self.conf_proj = bf(dim + rank, std=0.05)
        self._descs = (capi.LayerDesc * n_stages)(*[L.desc for L in self.stages])
        d = capi.DsparkDesc()
        d.n_stages, d.block_size, d.noise_id, d.markov_rank, d.n_targets = n_stages, block_size, noise_id, rank, nt
        for i, t in enumerate(targets):
            d.targets[i] = t
        d.stages = C.cast(self._descs, C.POINTER(capi.LayerDesc))
        d.main_proj = capi.qw(*self.main_proj, dim, nt * dim)
        d.main_norm_w, d.norm_w = capi.ptr(self.main_norm_w), capi.ptr(self.norm_w)
        d.hc_head_fn, d.hc_head_base, d.hc_head_scale = capi.ptr(self.hc_head_fn), capi.ptr(self.hc_head_base), 0.85
        d.markov_w1, d.markov_w2, d.conf_proj = capi.ptr(self.markov_w1), capi.ptr(self.markov_w2), capi.ptr(self.conf_proj)
        self.desc, self.block_size = d, block_size

    def states(self):
        from apus_b200 import capi
        S = [AttnState(L.attn) for L in self.stages]
        arr = (capi.AttnS * len(S))(*[s.st for s in S])
        return S, arr


def block_inputs(seed, n_tokens, hc, dim):
    rng = np.random.default_rng(seed)
    return synth.activations(rng, n_tokens, hc * dim, std=1.2).reshape(n_tokens, hc, dim)


def prompt_ids(seed, batch, n, vocab):
    return np.random.default_rng(seed).integers(0, vocab, size=(batch, n)).astype(np.int64)


# ---- sampling -------------------------------------------------------------------------
def sample_case(seed, rows, n, kind):
    """Logit rows + one uniform per row.  kind: 'peaked' (a few dominant tokens),
    'flat' (near-uniform, the nucleus reaches deep into the tail), 'ties'
    (BF16-rounded logits: many exactly equal probabilities)."""
    rng = np.random.default_rng(seed)
    if kind == "peaked":
        lg = (rng.standard_normal((rows, n)) * 4.0).astype(np.float32)
    elif kind == "flat":
        lg = (rng.standard_normal((rows, n)) * 0.05).astype(np.float32)
    else:
        lg = synth.bf16_round((rng.standard_normal((rows, n)) * 0.5).astype(np.float32))
        lg = (np.round(lg * 8) / 8).astype(np.float32)
    u = rng.random(rows)
    return lg, u
