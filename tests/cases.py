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
