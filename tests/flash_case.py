"""The benchmarked model at its real dimensions, cut to its first six layers, as a
parity case: hidden 4096, 64 heads x 512, 256 routed MXFP4 experts (top-6) + FP8
shared expert per layer, vocabulary 129,280; layers 0-1 sliding window, 2 and 4
compressed-sparse with indexer, 3 and 5 heavily compressed (ratio 128); layers
0-2 hash-routed.  The weights are the counter-based synthetic model of
apus_b200/flash.py with the benchmark's seed, so these ARE the first six layers
(and the embedding / head) of the model bench.py times; the host build of the
same generator hands the identical bits to the reference.

Shared by tests/golden/make_golden.py (runs the unmodified reference on the
host) and tests/test_gpu_flash_parity.py (runs the CUDA path).
"""
import ctypes as C

import numpy as np

from apus_b200 import capi
from apus_b200.flash import FlashConfig, RandomFlashModel, prompt_ids

CASE = dict(seed=0, n_layers=6, n_prompt=100, n_gen=64, batch=4, max_pos=192)
SUB_STRIDE = 61          # every 61st logit of a row is kept in the golden file
TOPN = 8                 # and its eight largest entries (index, value)


def config(n_layers=None):
    cfg = FlashConfig()
    cfg.n_layers = n_layers or CASE["n_layers"]
    return cfg


def prompts(cfg, batch=None, n_prompt=None):
    return prompt_ids(CASE["seed"], 0, batch or CASE["batch"], n_prompt or CASE["n_prompt"], cfg.vocab)


def rope_arrays():
    """The rope tables of the case as the golden file stores them (cos/sin come from the
    host's math library, so the tables the reference run used travel with its outputs)."""
    from apus_b200.flash import rope_tables
    cfg = config()
    out = {}
    for name, compressed in (("plain", False), ("yarn", True)):
        cos, sin = rope_tables(cfg, compressed, CASE["max_pos"])
        out[f"rope.{name}.cos"], out[f"rope.{name}.sin"] = cos, sin
    return out


def rope_from(G):
    return {c: (np.ascontiguousarray(G[f"rope.{n}.cos"]), np.ascontiguousarray(G[f"rope.{n}.sin"]))
            for n, c in (("plain", False), ("yarn", True))}


def host_states(cfg, max_pos):
    """Fresh host attention states (reference c/attn.h:147-160, 747-760), one per layer."""
    keep, sts = [], []
    for ratio in cfg.layer_kinds():
        st = capi.AttnS()
        st.pos = 0
        win = np.zeros((cfg.window, cfg.head_dim), np.float32)
        keep.append(win)
        st.win = capi.ptr(win)

        def comp(dd, overlap):
            coff = 1 + overlap
            rows, cols = coff * ratio, coff * dd
            kv = np.zeros((rows, cols), np.float32)
            sc = np.full((rows, cols), -np.inf, np.float32)
            max_nb = max_pos // ratio + 2
            cache = np.zeros((max_nb, dd), np.float32)
            keep.extend([kv, sc, cache])
            return capi.CompS(rows, cols, capi.ptr(kv), capi.ptr(sc), capi.ptr(cache), 0, max_nb, dd, max_nb)
        if ratio:
            st.comp = comp(cfg.head_dim, int(ratio == 4))
            if ratio == 4:
                st.idx_comp = comp(cfg.idx_dim, 1)
        sts.append(st)
    return keep, (capi.AttnS * len(sts))(*sts)


def rel(a, b):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))


def summarise(row):
    """What the golden file keeps of one logits row."""
    top = np.argsort(-row, kind="stable")[:TOPN].astype(np.int32)
    return dict(sub=row[::SUB_STRIDE].copy(), top_idx=top, top_val=row[top].copy(),
                norm=np.float64(np.linalg.norm(row.astype(np.float64))))


def run_reference(L, batch=None, n_prompt=None, n_gen=None, n_layers=None, progress=False, perturb=False,
                  feed=None):
    """Greedy loop of the unmodified reference (c/apus.c:895-944, temperature 0) on the
    host build of the model, one sequence at a time.  Returns tokens [B, n_gen] and the
    per-step summaries of the logits rows.

    perturb: the lowest mantissa bit of ONE BF16 embedding value (element 0 of the row of
    each sequence's first prompt token) is flipped before the run, and the tokens fed back
    are `feed` [B, n_gen] (those of the unperturbed run) -- the reference's own sensitivity
    to a one-ulp change of one input value, the yardstick for any other implementation's
    distance from it."""
    batch, n_prompt, n_gen = batch or CASE["batch"], n_prompt or CASE["n_prompt"], n_gen or CASE["n_gen"]
    cfg = config(n_layers)
    W = RandomFlashModel(cfg, CASE["seed"], "host", max_pos=CASE["max_pos"])
    V = cfg.vocab
    P = capi.ptr
    L.ref_model_forward.restype = None
    L.ref_model_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int]
    ids = prompts(cfg, batch, n_prompt)
    if perturb:
        from apus_b200.flash import TOP
        embed = W.named[(TOP, "embed")]
        for b in range(batch):
            embed[ids[b, 0], 0] ^= 1
    n_sub = len(range(0, V, SUB_STRIDE))
    G = dict(tokens=np.zeros((batch, n_gen), np.int32), gap=np.zeros((batch, n_gen), np.float32),
             sub=np.zeros((batch, n_gen, n_sub), np.float32), top_idx=np.zeros((batch, n_gen, TOPN), np.int32),
             top_val=np.zeros((batch, n_gen, TOPN), np.float32), norm=np.zeros((batch, n_gen), np.float64))
    for b in range(batch):
        keep, st = host_states(cfg, CASE["max_pos"])
        pos = C.c_int64(0)
        lg = np.empty(V, np.float32)
        L.ref_model_forward(C.byref(W.desc), st, C.byref(pos), P(np.ascontiguousarray(ids[b])), n_prompt, P(lg), 0)
        for g in range(n_gen):
            s = summarise(lg)
            tok = int(np.argmax(lg))
            G["tokens"][b, g] = tok
            G["gap"][b, g] = s["top_val"][0] - s["top_val"][1]
            for k in ("sub", "top_idx", "top_val", "norm"):
                G[k][b, g] = s[k]
            if g + 1 < n_gen:
                nxt = np.array([tok if feed is None else feed[b, g]], np.int64)
                L.ref_model_forward(C.byref(W.desc), st, C.byref(pos), P(nxt), 1, P(lg), 0)
        if progress:
            print(f"  sequence {b}: tokens {G['tokens'][b, :8].tolist()}..., min gap {G['gap'][b].min():.4f}", flush=True)
    return G


# ---- one layer at a time, stage by stage ---------------------------------------------------
LAYER_CHUNKS = [4, 1, 1, 1]        # tokens per apus_block_forward call: a prefill, then decode steps
LAYER_KEYS = ("attn_norm_out", "o_out", "ffn_norm_out", "moe_out", "out")


def layer_inputs(cfg, li):
    """Seeded hidden states [tokens, hc, dim] (BF16-valued) and token ids for the layer case."""
    from apus_b200 import synth
    total = sum(LAYER_CHUNKS)
    rng = np.random.default_rng([CASE["seed"], 77, li])
    h = synth.activations(rng, total, cfg.hc_mult * cfg.dim, std=1.2).reshape(total, cfg.hc_mult, cfg.dim)
    ids = prompt_ids(CASE["seed"], 100 + li, 1, total, cfg.vocab)[0]
    return h, np.ascontiguousarray(ids)


def one_layer_config(cfg, li):
    one = config(1)
    one.ratios = [cfg.ratios[li]]
    return one


class RefInterm(C.Structure):
    """The reference's ApusInterm (c/layer.h:88-104)."""
    _fields_ = [("attn_hc_pre", C.c_void_p), ("attn_hc_post", C.c_void_p), ("attn_hc_comb", C.c_void_p),
                ("attn_norm_out", C.c_void_p), ("attn", capi.AttnInterm), ("post_attn_h", C.c_void_p),
                ("ffn_hc_pre", C.c_void_p), ("ffn_hc_post", C.c_void_p), ("ffn_hc_comb", C.c_void_p),
                ("ffn_norm_out", C.c_void_p), ("moe", capi.MoeInterm), ("moe_out", C.c_void_p)]


def run_reference_layers(L, progress=False):
    """Layers 0..5 of the model one at a time through the reference's apus_block_forward
    (c/layer.h:495-545) on seeded hidden states, with the stage outputs its ApusInterm
    exposes.  Everything kept is BF16-valued and stored as BF16 bits."""
    from apus_b200 import synth
    cfg = config()
    hc, dim = cfg.hc_mult, cfg.dim
    total = sum(LAYER_CHUNKS)
    L.ref_block_forward_interm.restype = None
    L.ref_block_forward_interm.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_float, C.c_void_p, C.c_void_p,
                                           C.c_void_p, C.c_int, C.c_int64, C.c_void_p]
    G = {}
    for li in range(cfg.n_layers):
        W = RandomFlashModel(cfg, CASE["seed"], "host", max_pos=CASE["max_pos"], layer_ids=[li])
        d = W._descs[0]
        d.mw.layer_id = li
        h_in, ids = layer_inputs(cfg, li)
        A = {k: np.zeros((total, dim), np.float32) for k in LAYER_KEYS[:-1]}
        keep, st = host_states(one_layer_config(cfg, li), CASE["max_pos"])
        out = h_in.copy()
        # the reference reads the vocabulary size for hash routing from the layer's cfg, which
        # the descriptor adapter leaves 0: bounds are not checked there, the lookup is by id
        pos = 0
        for n in LAYER_CHUNKS:
            it = RefInterm()
            it.attn_norm_out, it.ffn_norm_out, it.moe_out = (capi.ptr(A[k][pos:pos + n]) for k in
                                                             ("attn_norm_out", "ffn_norm_out", "moe_out"))
            it.attn.o_out = capi.ptr(A["o_out"][pos:pos + n])
            L.ref_block_forward_interm(C.byref(d), hc, cfg.hc_iters, cfg.hc_eps, cfg.norm_eps, C.byref(st[0]),
                                       capi.ptr(out[pos:pos + n]), capi.ptr(ids[pos:pos + n]), n, pos, C.byref(it))
            pos += n
        A["out"] = out
        for k, v in A.items():
            assert np.array_equal(synth.bf16_round(v), v), k      # BF16-valued: the bits lose nothing
            G[f"layer{li}.{k}"] = synth.bf16_bits(v)
        if progress:
            print(f"  layer {li} (ratio {cfg.ratios[li]}, hash {int(li < cfg.n_hash_layers)}) done", flush=True)
    return G
