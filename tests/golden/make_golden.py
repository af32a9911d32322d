#!/usr/bin/env python3
"""Regenerates the committed golden vectors from the reference itself.

Run in a container where the reference checkout is mounted (its location: the
APUS_REFERENCE environment variable, else a directory named `reference` beside this repository):

  1. m3/ and m4a/: the reference's OWN golden generators
     (tests/m3/gen_golden.py, tests/m4a/gen_golden.py; seed 20260729) are
     imported and run with their output directory redirected here.  These are
     the known-answer fixtures its C tests check the kernels against.
  2. ref_cases.npz: outputs of the unmodified reference C code
     (oracle/_ref/libapus_ref.so) on the seeded cases of tests/cases.py.
  3. ckpt_case.npz (argument `ckpt`), mtp_case.npz (argument `mtp`) and flash_case.npz
     (argument `flash`): the reference's loader + greedy loop on a written checkpoint
     directory, its hidden-collecting forwards, MTP draft head and speculative loop on the
     small model, and its greedy loop on six real-dimension layers of the benchmarked model.

Nothing on the GPU box reads the reference checkout; it only reads these files.
"""
import ctypes as C
import importlib.util
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))
import cases                                   # noqa: E402
from _oracle import P, ref, reference_dir      # noqa: E402
REF = reference_dir()
from apus_b200 import capi                     # noqa: E402


def run_reference_generators():
    for name in ("m3", "m4a"):
        spec = importlib.util.spec_from_file_location(
            f"gen_{name}", REF / "tests" / name / "gen_golden.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.OUT = str(HERE / name)
        os.makedirs(mod.OUT, exist_ok=True)
        mod.main()


def ref_linear(L, fmt, c):
    M, K = c["x"].shape
    O = c["codes"].shape[0]
    out = np.empty((M, O), np.float32)
    w = capi.qw(c["codes"], c["scales"], O, K)
    (L.apus_fp4_linear if fmt == 4 else L.apus_fp8_linear)(C.byref(w), P(c["x"]), P(out), M, K, O)
    xb = np.empty_like(c["x"])
    codes = np.empty((M, K), np.uint8)
    scales = np.empty((M, K // 128), np.float32)
    L.ref_act_quant_rows(P(c["x"]), P(xb), P(codes), P(scales), M, K)
    raw = np.empty((M, O), np.float32)
    scratch = np.empty((M, K), np.float32)
    (L.apus_fp4_gemm_mt if fmt == 4 else L.apus_fp8_gemm_mt)(
        P(c["codes"]), P(c["scales"]), P(codes), P(scales), P(scratch), P(raw), M, O, K)
    return dict(out=out, acodes=codes, ascales=scales, raw=raw)


def rope_tables(L, D, compressed):
    """cos/sin [max_pos, rd/2] exactly as the reference's layers build them
    (c/layer.h:147-149: plain theta 1e4 for sliding-window layers, YaRN factor 16
    over 65536 with theta 1.6e5 for compressed ones)."""
    half = D["rope_dim"] // 2
    cos = np.empty((D["max_pos"], half), np.float32)
    sin = np.empty((D["max_pos"], half), np.float32)
    L.apus_rope_precompute.restype = None
    L.apus_rope_precompute.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_double,
                                       C.c_double, C.c_int, C.c_int]
    if compressed:
        L.apus_rope_precompute(P(cos), P(sin), D["rope_dim"], D["max_pos"], 65536, 160000.0, 16.0, 32, 1)
    else:
        L.apus_rope_precompute(P(cos), P(sin), D["rope_dim"], D["max_pos"], 0, 10000.0, 1.0, 32, 1)
    return cos, sin


def ref_attention(L, seed, kind, chunks):
    """Runs the reference apus_attention over consecutive chunks of tokens
    (first chunk = prefill at position 0, the rest single-token decodes or
    mid-stream batches) and returns outputs + final state."""
    Lyr = cases.AttnLayer(seed, kind)
    S = cases.AttnState(Lyr)
    D = Lyr.D
    cos, sin = rope_tables(L, D, kind != "swa")
    total = sum(chunks)
    x = cases.attn_inputs(seed + 7, total, D["dim"])
    out = np.empty((total, D["dim"]), np.float32)
    L.apus_attention.restype = None
    L.apus_attention.argtypes = [C.c_void_p] * 4 + [C.c_int, C.c_int64] + [C.c_void_p] * 4
    pos = 0
    for n in chunks:
        L.apus_attention(C.byref(Lyr.cfg), C.byref(Lyr.w), C.byref(S.st), P(x[pos:pos + n]), n, pos, P(cos), P(sin),
                         P(out[pos:pos + n]), None)
        pos += n
    r = dict(out=out, win=S.win.copy(), cos=cos, sin=sin)
    if Lyr.ratio:
        r.update(comp_kv=S.comp[0].copy(), comp_sc=S.comp[1].copy(),
                 comp_cache=S.comp[2][:S.st.comp.nb].copy())
        if kind == "csa":
            r.update(idx_kv=S.idx[0].copy(), idx_sc=S.idx[1].copy(), idx_cache=S.idx[2][:S.st.idx_comp.nb].copy())
    return r


def rope_pair(L):
    D = cases.ATTN_DIMS
    return {"plain": rope_tables(L, D, False), "yarn": rope_tables(L, D, True)}


class RefInterm(C.Structure):
    """The reference's ApusInterm (c/layer.h:88-104)."""
    _fields_ = [("attn_hc_pre", C.c_void_p), ("attn_hc_post", C.c_void_p), ("attn_hc_comb", C.c_void_p),
                ("attn_norm_out", C.c_void_p), ("attn", capi.AttnInterm), ("post_attn_h", C.c_void_p),
                ("ffn_hc_pre", C.c_void_p), ("ffn_hc_post", C.c_void_p), ("ffn_hc_comb", C.c_void_p),
                ("ffn_norm_out", C.c_void_p), ("moe", capi.MoeInterm), ("moe_out", C.c_void_p)]


def ref_block(L, seed, kind, chunks, flash=False):
    """The reference's apus_block_forward over consecutive chunks (prefill at
    position 0, then decodes) through the shim's descriptor adapter, with the
    stage outputs its ApusInterm exposes."""
    rope = rope_pair(L)
    cos, sin = rope["plain" if kind == "swa" else "yarn"]
    B = cases.BlockLayer(seed, kind, cos, sin, dims=cases.FLASH_MOE_DIMS, attn_dims=cases.FLASH_ATTN_DIMS) \
        if flash else cases.BlockLayer(seed, kind, cos, sin)
    S = cases.AttnState(B.attn)
    M, dim = B.M, B.attn.D["dim"]
    hc = M["hc"]
    total = sum(chunks)
    h = cases.block_inputs(seed + 3, total, hc, dim)
    out = h.copy()
    ids = np.zeros(total, np.int64)
    A = {k: np.zeros((total,) + sh, np.float32) for k, sh in dict(
        attn_hc_post=(hc,), attn_hc_comb=(hc, hc), attn_norm_out=(dim,), o_out=(dim,), post_attn_h=(hc, dim),
        ffn_hc_post=(hc,), ffn_hc_comb=(hc, hc), ffn_norm_out=(dim,), moe_out=(dim,)).items()}
    L.ref_block_forward_interm.restype = None
    L.ref_block_forward_interm.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_float, C.c_void_p,
                                           C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_void_p]
    pos = 0
    for n in chunks:
        it = RefInterm()
        for k, a in A.items():
            if k == "o_out":
                it.attn.o_out = P(a[pos:pos + n])
            else:
                setattr(it, k, P(a[pos:pos + n]))
        L.ref_block_forward_interm(C.byref(B.desc), hc, M["iters"], M["hc_eps"], M["norm_eps"], C.byref(S.st),
                                   P(out[pos:pos + n]), P(ids[pos:pos + n]), n, pos, C.byref(it))
        pos += n
    if flash:          # real sizes: keep the hidden states of the listed tokens only, as BF16 bits
        from apus_b200.synth import bf16_bits
        keep = FLASH_KEEP[kind]
        return dict(out_bits=bf16_bits(out[keep]), o_bits=bf16_bits(A["o_out"][keep]),
                    moe_bits=bf16_bits(A["moe_out"][keep]))
    return dict(out=out, win=S.win.copy(), **A)


def ref_generate(L, seed, n_layers, batch, n_prompt, n_gen, temp=0.0, top_p=1.0, rng_seed=0):
    """Greedy token loop on the reference's apus_model_forward (c/apus.c:895-944
    with temperature 0: argmax, lowest index on ties), one sequence at a time."""
    Mdl = cases.TinyModel(seed, rope_pair(L), n_layers)
    V = Mdl.M["vocab"]
    prompts = cases.prompt_ids(seed + 5, batch, n_prompt, V)
    L.ref_model_forward.restype = None
    L.ref_model_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int]
    toks = np.zeros((batch, n_gen), np.int32)
    logits = np.zeros((batch, n_gen, V), np.float32)
    L.apus_sample_logits_u.restype = C.c_int
    L.apus_sample_logits_u.argtypes = [C.c_void_p, C.c_size_t, C.c_float, C.c_float, C.c_double, C.c_void_p]
    L.apus_rng_uniform.restype = C.c_double
    scratch = np.empty(2 * V, np.float32)
    for b in range(batch):
        rng_state = C.c_uint64(rng_seed + b)             # sequence b draws from the stream seeded seed + b
        keep, st = Mdl.states()
        pos = C.c_int64(0)
        lg = np.empty(V, np.float32)
        ids = np.ascontiguousarray(prompts[b])
        L.ref_model_forward(C.byref(Mdl.desc), st, C.byref(pos), P(ids), n_prompt, P(lg), 0)
        for g in range(n_gen):
            logits[b, g] = lg
            if temp > 0:                                  # c/sample.h:173-178 apus_sample
                toks[b, g] = L.apus_sample_logits_u(P(lg), V, temp, top_p, L.apus_rng_uniform(C.byref(rng_state)),
                                                    P(scratch))
            else:
                toks[b, g] = int(np.argmax(lg))
            if g + 1 < n_gen:
                nxt = np.array([toks[b, g]], np.int64)
                L.ref_model_forward(C.byref(Mdl.desc), st, C.byref(pos), P(nxt), 1, P(lg), 0)
        assert pos.value == n_prompt + n_gen - 1
    return dict(tokens=toks, logits=logits)


def ref_checkpoint(L, seed, n_layers, n_prompt, n_gen):
    """The model of tests/ckpt_util.py written as a checkpoint directory, loaded
    by the reference's own apus_model_load and run through its greedy loop
    (oracle/ref_shim.c ref_ckpt_run): what the reference makes of the files."""
    import tempfile
    import ckpt_util
    tm = cases.TinyModel(seed, rope_pair(L), n_layers)
    V, D = tm.M["vocab"], cases.ATTN_DIMS
    prompt = cases.prompt_ids(seed + 5, 1, n_prompt, V)[0]
    toks = np.zeros(n_gen, np.int32)
    logits = np.zeros((n_gen, V), np.float32)
    cfg = capi.CkptCfg()
    ratios, hash_ = np.zeros(n_layers, np.int32), np.zeros(n_layers, np.int32)
    wo = np.zeros_like(tm.layers[0].attn.wo_a)
    rows, half = D["max_pos"], D["rope_dim"] // 2
    rope = [np.zeros((rows, half), np.float32) for _ in range(4)]
    err = C.create_string_buffer(256)
    with tempfile.TemporaryDirectory() as d:
        ckpt_util.write_checkpoint(d, tm, seed=seed)
        L.ref_ckpt_run.restype = C.c_int
        L.ref_ckpt_run.argtypes = [C.c_char_p, C.c_void_p, C.c_int, C.c_int] + [C.c_void_p] * 6 + \
            [C.c_size_t, C.c_int] + [C.c_void_p] * 4 + [C.c_char_p, C.c_size_t]
        rc = L.ref_ckpt_run(d.encode(), P(prompt), n_prompt, n_gen, P(toks), P(logits), C.addressof(cfg),
                            P(ratios), P(hash_), P(wo), wo.size, rows, P(rope[0]), P(rope[1]), P(rope[2]),
                            P(rope[3]), err, 256)
        assert rc == 0, err.value
    assert np.array_equal(wo, tm.layers[0].attn.wo_a)
    return dict(tokens=toks, logits=logits, cfg=np.frombuffer(bytes(cfg), np.uint8).copy(), ratios=ratios,
                hash=hash_, wo_a0=wo, cos_plain=rope[0], sin_plain=rope[1], cos_yarn=rope[2], sin_yarn=rope[3])


def main_flash():
    """The real-dimension six-layer case (tests/flash_case.py): tokens, top-1 margins and a
    summary of every logits row of the reference's greedy loop -> flash_case.npz."""
    import flash_case
    L = ref()
    assert L is not None, "reference build not available"
    G = flash_case.run_reference(L, progress=True)
    # the reference against itself with one input value moved by one BF16 ulp, teacher-forced
    Gp = flash_case.run_reference(L, progress=True, perturb=True, feed=G["tokens"])
    G["sens"] = np.array([[flash_case.rel(Gp["sub"][b, g], G["sub"][b, g]) for g in range(G["sub"].shape[1])]
                          for b in range(G["sub"].shape[0])])
    G["sens_flips"] = (Gp["tokens"] != G["tokens"])
    G.update(flash_case.rope_arrays())
    G.update(flash_case.run_reference_layers(L, progress=True))
    # the same loop on the model cut after its first layer: depth 1 is where the stated
    # logits / token bars can be held (see tests/test_gpu_flash_parity.py)
    G.update({f"one.{k}": v for k, v in flash_case.run_reference(L, batch=2, n_layers=1, progress=True).items()})
    np.savez_compressed(HERE / "flash_case.npz", **G)
    print("wrote flash_case.npz:", {k: v.shape for k, v in G.items()})


def main_ckpt():
    L = ref()
    assert L is not None, "reference build not available"
    G = ref_checkpoint(L, **CKPT_CASE)
    np.savez_compressed(HERE / "ckpt_case.npz", **G)
    print("wrote ckpt_case.npz:", {k: v.shape for k, v in G.items()})


def ref_mtp(L, seed, n_layers, n_prompt, n_gen, depth, targets):
    """The reference's hidden-collecting forwards (c/model.h:731-743), its MTP head over the
    prompt's true (hidden, token) pairs and one chained call (c/mtp.h:303-357), and its
    speculative loop with that head as the proposer (c/mtp.h:472-616), greedy."""
    Mdl = cases.TinyModel(seed, rope_pair(L), n_layers)
    Mtp = cases.TinyMtp(seed + 3, rope_pair(L))
    V, hd, dim = Mdl.M["vocab"], Mdl.M["hc"] * cases.ATTN_DIMS["dim"], cases.ATTN_DIMS["dim"]
    prompt = np.ascontiguousarray(cases.prompt_ids(seed + 5, 1, n_prompt, V)[0])
    vp = C.c_void_p
    L.ref_model_forward_hm.restype = None
    L.ref_model_forward_hm.argtypes = [vp, vp, vp, vp, C.c_int, vp, C.c_int, vp, vp, C.c_int, vp]
    L.ref_mtp_forward.restype = None
    L.ref_mtp_forward.argtypes = [vp, vp, vp, vp, vp, C.c_int, C.c_int64, vp, vp]
    L.ref_spec_generate_mtp.restype = C.c_int
    L.ref_spec_generate_mtp.argtypes = [vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, vp, vp, vp]
    out = {}
    # forward_h with every position's logits
    keep, st = Mdl.states()
    pos = C.c_int64(0)
    lg_all, h_all = np.empty((n_prompt, V), np.float32), np.empty((n_prompt, hd), np.float32)
    L.ref_model_forward_hm(C.byref(Mdl.desc), st, C.byref(pos), P(prompt), n_prompt, P(lg_all), 1, P(h_all), None, 0, None)
    out["h_all"], out["logits_all"] = h_all, lg_all
    # forward_mh
    keep2, st2 = Mdl.states()
    pos = C.c_int64(0)
    tg = np.array(targets, np.int32)
    mh, lg = np.empty((n_prompt, len(targets) * dim), np.float32), np.empty(V, np.float32)
    L.ref_model_forward_hm(C.byref(Mdl.desc), st2, C.byref(pos), P(prompt), n_prompt, P(lg), 0, None, P(tg), len(targets), P(mh))
    out["mh_all"] = mh
    assert np.array_equal(lg, lg_all[-1])
    # the head over the true pairs, then one chained position
    keepm, stm = Mtp.state()
    ml, mhl = np.empty(V, np.float32), np.empty(hd, np.float32)
    L.ref_mtp_forward(C.byref(Mdl.desc), C.byref(Mtp.desc), C.byref(stm), P(h_all), P(prompt), n_prompt, 0, P(ml), P(mhl))
    out["mtp_logits"], out["mtp_h_last"] = ml.copy(), mhl.copy()
    d1 = np.array([int(np.argmax(ml))], np.int64)
    own = mhl.copy()                                    # the head's own hidden is the chaining input
    L.ref_mtp_forward(C.byref(Mdl.desc), C.byref(Mtp.desc), C.byref(stm), P(own), P(d1), 1, n_prompt, P(ml), P(mhl))
    out["mtp_logits_chained"], out["mtp_h_chained"] = ml.copy(), mhl.copy()
    out["mtp_win"] = keepm.win.copy()
    # the speculative loop
    keep3, st3 = Mdl.states()
    keepm2, stm2 = Mtp.state()
    toks, stats, fd = np.zeros(n_gen, np.int32), np.zeros(8, np.uint64), np.zeros(depth, np.int64)
    n = L.ref_spec_generate_mtp(C.byref(Mdl.desc), C.byref(Mtp.desc), st3, C.byref(stm2), P(prompt), n_prompt, n_gen, depth,
                                P(toks), P(stats), P(fd))
    assert n == n_gen
    out["spec_tokens"], out["spec_stats"], out["spec_first_drafts"] = toks, stats, fd
    # and the plain greedy stream it must reproduce
    plain = ref_generate(L, seed, n_layers, 1, n_prompt, n_gen)["tokens"][0]
    assert np.array_equal(plain, toks), (plain, toks)
    return out


def ref_dspark(L, seed, n_layers, n_prompt, n_gen, targets, n_stages, block_size, noise_id, rank, temp, top_p, rng_seed,
               draft_seed):
    """The reference's DSpark module on the small model (c/dspark.h): the stage rings built from the prompt's
    main hiddens and one draft round after them (drafts, final logits, confidence, every stage's block
    output), and its speculative loop (greedy), which must emit the plain greedy stream."""
    Mdl = cases.TinyModel(seed, rope_pair(L), n_layers)
    Ds = cases.TinyDspark(seed + 4, rope_pair(L), targets, n_stages, block_size, noise_id, rank)
    V, hd, dim = Mdl.M["vocab"], Mdl.M["hc"] * cases.ATTN_DIMS["dim"], cases.ATTN_DIMS["dim"]
    prompt = np.ascontiguousarray(cases.prompt_ids(seed + 5, 1, n_prompt, V)[0])
    vp = C.c_void_p
    L.ref_model_forward_hm.restype = None
    L.ref_model_forward_hm.argtypes = [vp, vp, vp, vp, C.c_int, vp, C.c_int, vp, vp, C.c_int, vp]
    L.ref_dspark_prefill_round.restype = None
    L.ref_dspark_prefill_round.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int64, vp, vp, vp, vp]
    L.ref_spec_generate_dspark.restype = C.c_int
    L.ref_spec_generate_dspark.argtypes = [vp, vp, vp, vp, vp, C.c_int, C.c_int, vp, vp]
    out = {}
    keep, st = Mdl.states()
    pos = C.c_int64(0)
    tg = np.array(targets, np.int32)
    mh, lg = np.empty((n_prompt, len(targets) * dim), np.float32), np.empty(V, np.float32)
    L.ref_model_forward_hm(C.byref(Mdl.desc), st, C.byref(pos), P(prompt), n_prompt, P(lg), 0, None, P(tg), len(targets), P(mh))
    anchor = int(np.argmax(lg))
    keeps, sst = Ds.states()
    drafts, conf = np.zeros(block_size, np.int64), np.zeros(block_size, np.float32)
    lf, sh = np.zeros((block_size, V), np.float32), np.zeros((n_stages, block_size, hd), np.float32)
    L.ref_dspark_prefill_round(C.byref(Mdl.desc), C.byref(Ds.desc), sst, P(mh), n_prompt, anchor, P(drafts), P(conf), P(lf), P(sh))
    out.update(mh_all=mh, anchor=np.array([anchor]), drafts=drafts, confidence=conf, logits_final=lf, stage_h=sh,
               rings=np.stack([k.win.copy() for k in keeps]))
    keep3, st3 = Mdl.states()
    keeps2, sst2 = Ds.states()
    toks, stats = np.zeros(n_gen, np.int32), np.zeros(7, np.uint64)
    n = L.ref_spec_generate_dspark(C.byref(Mdl.desc), C.byref(Ds.desc), st3, sst2, P(prompt), n_prompt, n_gen, P(toks), P(stats))
    assert n == n_gen
    plain = ref_generate(L, seed, n_layers, 1, n_prompt, n_gen)["tokens"][0]
    assert np.array_equal(plain, toks), (plain, toks)
    out.update(spec_tokens=toks, spec_stats=stats)
    # sampled: the draft picks of a round drawn from the module's own stream, and the loop with a sampled main stream
    L.ref_dspark_prefill_round_t.restype = None
    L.ref_dspark_prefill_round_t.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int64, C.c_float, C.c_uint64, vp, vp, vp, vp]
    L.ref_spec_generate_dspark_t.restype = C.c_int
    L.ref_spec_generate_dspark_t.argtypes = [vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_float, C.c_float, C.c_uint64, C.c_uint64, vp, vp]
    keeps4, sst4 = Ds.states()
    d_s, lf_s = np.zeros(block_size, np.int64), np.zeros((block_size, V), np.float32)
    L.ref_dspark_prefill_round_t(C.byref(Mdl.desc), C.byref(Ds.desc), sst4, P(mh), n_prompt, anchor, temp, draft_seed, P(d_s), None,
                                 P(lf_s), None)
    keep5, st5 = Mdl.states()
    keeps5, sst5 = Ds.states()
    toks_s, stats_s = np.zeros(n_gen, np.int32), np.zeros(7, np.uint64)
    n = L.ref_spec_generate_dspark_t(C.byref(Mdl.desc), C.byref(Ds.desc), st5, sst5, P(prompt), n_prompt, n_gen, temp, top_p, rng_seed,
                                     draft_seed, P(toks_s), P(stats_s))
    assert n == n_gen
    out.update(drafts_sampled=d_s, logits_final_sampled=lf_s, spec_sampled_tokens=toks_s, spec_sampled_stats=stats_s)
    return out


def main_dspark():
    L = ref()
    assert L is not None, "reference build not available"
    G = ref_dspark(L, **DSPARK_CASE)
    np.savez_compressed(HERE / "dspark_case.npz", **G)
    print("wrote dspark_case.npz:", {k: v.shape for k, v in G.items()}, "stats", G["spec_stats"].tolist(), "drafts", G["drafts"].tolist(),
          "sampled drafts", G["drafts_sampled"].tolist(), "sampled stats", G["spec_sampled_stats"].tolist())


def main_mtp():
    L = ref()
    assert L is not None, "reference build not available"
    G = ref_mtp(L, **MTP_CASE)
    np.savez_compressed(HERE / "mtp_case.npz", **G)
    print("wrote mtp_case.npz:", {k: v.shape for k, v in G.items()}, "stats", G["spec_stats"].tolist())


def main():
    L = ref()
    assert L is not None, "reference build not available"
    run_reference_generators()
    G = {}
    for tag, args in LINEAR_CASES.items():
        r = ref_linear(L, args[1], cases.linear_case(*args))
        for k, v in r.items():
            G[f"{tag}.{k}"] = v
    for tag, args in EXPERT_CASES.items():
        c = cases.expert_case(*args)
        _, kind, rows, dim, inter = args
        out = np.empty((rows, dim), np.float32)
        w1, w2, w3 = capi.qw(*c["w1"], inter, dim), capi.qw(*c["w2"], dim, inter), capi.qw(*c["w3"], inter, dim)
        for t in range(rows):                 # the reference's expert is per token
            L.ref_expert(C.byref(w1), C.byref(w2), C.byref(w3), kind, 10.0,
                         P(c["x"][t]), dim, inter, P(out[t]))
        G[f"{tag}.out"] = out
    for tag, kw in MOE_CASES.items():
        W, x, ids = cases.moe_case(**kw)
        s = x.shape[0]
        w = W.moew()
        out = np.empty((s, W.dim), np.float32)
        sp = np.empty((s, W.E), np.float32)
        biased = np.zeros((s, W.E), np.float32)
        rw = np.empty((s, W.topk), np.float32)
        ri = np.empty((s, W.topk), np.int32)
        routed = np.empty((s, W.dim), np.float32)
        shared = np.empty((s, W.dim), np.float32)
        it = capi.MoeInterm(P(sp), P(biased), P(rw), P(ri), P(routed), P(shared))
        L.apus_moe_forward(C.byref(w), P(x), P(ids), s, P(out), C.byref(it))
        G.update({f"{tag}.out": out, f"{tag}.sp": sp, f"{tag}.biased": biased, f"{tag}.w": rw,
                  f"{tag}.idx": ri, f"{tag}.routed": routed, f"{tag}.shared": shared})
    for tag, args in TOPK_CASES.items():
        sc = cases.topk_case(*args)
        rows, n = sc.shape
        k = args[3]
        idx = np.empty((rows, k), np.int32)
        for r in range(rows):
            L.apus_topk_stable(P(sc[r]), n, k, P(idx[r]))
        G[f"{tag}.idx"] = idx
    for tag, args in ATTN_CASES.items():
        c = cases.sparse_attn_case(*args)
        _, s, h, d, na, nb, idxw, _ = args
        o = np.empty((s, h, d), np.float32)
        L.ref_sparse_attn(P(c["q"]), P(c["sink"]), h, d, P(c["idx"]), idxw, s, d ** -0.5,
                          P(c["kv_a"]), na, P(c["kv_b"]), P(o))
        G[f"{tag}.o"] = o
    for tag, args in MHC_CASES.items():
        c = cases.mhc_case(*args)
        _, rows, d = args
        n = 4
        pre = np.empty((rows, n), np.float32)
        post = np.empty((rows, n), np.float32)
        comb = np.empty((rows, n, n), np.float32)
        y = np.empty((rows, d), np.float32)
        y4 = np.empty((rows, n, d), np.float32)
        yh = np.empty((rows, d), np.float32)
        for t in range(rows):
            L.apus_mhc_prepost_scalar(P(c["x4"][t]), d, n, P(c["fn"]), P(c["scale"]), P(c["base"]),
                                      1e-6, 1e-6, 20, P(pre[t]), P(post[t]), P(comb[t]), None)
            L.apus_mhc_collapse_scalar(P(c["x4"][t]), P(pre[t]), P(y[t]), d, n)
            L.apus_mhc_apply_scalar(P(c["f"][t]), P(c["x4"][t]), P(post[t]), P(comb[t]), P(y4[t]), d, n)
            L.apus_mhc_head_scalar(P(c["x4"][t]), d, n, P(c["hfn"]), 0.8, P(c["hbase"]), 1e-6, 1e-6,
                                   P(yh[t]), None)
        yn = np.empty((rows, d), np.float32)
        from apus_b200.synth import bf16_round
        yb = bf16_round(y)
        for t in range(rows):
            L.apus_rms_norm(P(yb[t]), P(c["norm_w"]), 1e-6, P(yn[t]), d)
        G.update({f"{tag}.pre": pre, f"{tag}.post": post, f"{tag}.comb": comb, f"{tag}.y": y,
                  f"{tag}.y4": y4, f"{tag}.yhead": yh, f"{tag}.ynorm": yn})
    for tag, (seed, kind, chunks) in ATTN_LAYER_CASES.items():
        G.update({f"{tag}.{k}": v for k, v in ref_attention(L, seed, kind, chunks).items()})
    for name, (cos, sin) in rope_pair(L).items():
        G[f"rope.{name}.cos"], G[f"rope.{name}.sin"] = cos, sin
    for tag, (seed, kind, chunks) in BLOCK_CASES.items():
        G.update({f"{tag}.{k}": v for k, v in ref_block(L, seed, kind, chunks).items()})
    for tag, (seed, kind, chunks) in BLOCK_FLASH_CASES.items():
        G.update({f"{tag}.{k}": v for k, v in ref_block(L, seed, kind, chunks, flash=True).items()})
        print(tag, "done", flush=True)
    for tag, args in MODEL_CASES.items():
        G.update({f"{tag}.{k}": v for k, v in ref_generate(L, *args).items()})
    for tag, args in MODEL_SAMPLED_CASES.items():
        G.update({f"{tag}.{k}": v for k, v in ref_generate(L, *args).items()})
    L.apus_sample_logits_u.restype = C.c_int
    L.apus_sample_logits_u.argtypes = [C.c_void_p, C.c_size_t, C.c_float, C.c_float, C.c_double, C.c_void_p]
    for tag, (seed, rows, n, kind, temp, top_p) in SAMPLE_CASES.items():
        lg, u = cases.sample_case(seed, rows, n, kind)
        scratch = np.empty(2 * n, np.float32)
        G[f"{tag}.tokens"] = np.array([L.apus_sample_logits_u(P(lg[r]), n, temp, top_p, float(u[r]), P(scratch))
                                       for r in range(rows)], np.int32)
    st = C.c_uint64(20260729)
    L.apus_rng_uniform.restype = C.c_double
    G["rng.uniforms"] = np.array([L.apus_rng_uniform(C.byref(st)) for _ in range(16)], np.float64)
    np.savez_compressed(HERE / "ref_cases.npz", **G)
    print(f"wrote {len(G)} arrays; avx2 hits {L.ref_avx2_hits()}, threads {L.ref_pool_threads()}")


# the checkpoint-directory case (tests/ckpt_util.py)
CKPT_CASE = dict(seed=91, n_layers=3, n_prompt=6, n_gen=8)
# tag -> arguments of the case builders in tests/cases.py
LINEAR_CASES = {
    "fp4_small": (11, 4, 3, 64, 256, True),
    "fp4_wide": (12, 4, 9, 256, 1024, False),
    "fp8_small": (13, 8, 8, 320, 384, True),
    "fp8_wide": (14, 8, 5, 256, 1024, False),
}
EXPERT_CASES = {
    "expert_fp4": (21, 0, 3, 256, 128),
    "expert_fp8": (22, 1, 3, 256, 128),
}
MOE_CASES = {
    "moe_bias": dict(seed=31, s=5),
    "moe_hash": dict(seed=32, s=4, hash_vocab=50),
    "moe_one": dict(seed=33, s=1),
    "moe_many": dict(seed=34, s=70, E=8, topk=2),
}
TOPK_CASES = {
    "topk_plain": (41, 3, 300, 6, False),
    "topk_ties": (42, 3, 2000, 512, True),
    "topk_all": (43, 2, 64, 64, True),
}
ATTN_CASES = {
    "attn_holes": (51, 3, 4, 64, 16, 40, 24, "holes"),
    "attn_empty": (52, 2, 2, 64, 8, 8, 12, "empty"),
    "attn_dups": (53, 2, 3, 128, 0, 50, 33, "dups"),
    "attn_full": (54, 1, 2, 64, 128, 30, 140, "full"),
}
# tag -> (seed, layer kind, token chunks fed to apus_attention one call each)
ATTN_LAYER_CASES = {
    "attn_swa": (71, "swa", [11] + [1] * 9),
    "attn_csa": (72, "csa", [13] + [1] * 14 + [3]),
    "attn_hca": (73, "hca", [10] + [1] * 16),
    "attn_csa_decode_only": (74, "csa", [1] * 26),
}
# tag -> (seed, layer kind, token chunks fed to apus_block_forward one call each)
BLOCK_CASES = {
    "block_swa": (81, "swa", [6] + [1] * 6),
    "block_csa": (82, "csa", [9] + [1] * 12),
    "block_hca": (83, "hca", [10] + [1] * 10),
}
# one block at the real model's sizes; hca128 completes its first compressed entry at token 127
BLOCK_FLASH_CASES = {
    "flash_swa": (101, "swa", [3] + [1] * 4),
    "flash_csa": (102, "csa", [6] + [1] * 7),
    "flash_hca": (103, "hca128", [2] + [1] * 130),
}
FLASH_KEEP = {"swa": list(range(7)), "csa": list(range(13)), "hca128": [0, 1, 2, 64, 126, 127, 128, 129, 130, 131]}
# tag -> (seed, layers, sequences, prompt tokens, generated tokens)
MODEL_CASES = {
    "model_one": (91, 3, 1, 9, 14),
    "model_batch": (92, 4, 3, 7, 12),
}
# the same plus (temperature, top_p, generator seed): sampled continuation (c/apus.c:895-944 with --temp)
MODEL_SAMPLED_CASES = {
    "model_sampled": (93, 3, 2, 6, 12, 0.8, 0.9, 1234),
}
# tag -> (seed, rows, vocabulary, logit pattern, temperature, top_p); c/sample.h
SAMPLE_CASES = {
    "sample_peaked": (111, 24, 4096, "peaked", 0.8, 0.95),
    "sample_flat": (112, 24, 4096, "flat", 1.0, 0.9),
    "sample_all": (113, 16, 3000, "flat", 1.0, 1.0),
    "sample_ties": (114, 24, 2048, "ties", 0.7, 0.5),
    "sample_top1": (115, 8, 1000, "peaked", 1.0, 0.0),
    "sample_vocab": (116, 6, 129280, "peaked", 0.8, 0.95),
    "sample_vocab_flat": (117, 4, 129280, "flat", 1.0, 1.0),
    "sample_greedy": (118, 8, 5000, "ties", 0.0, 0.9),
}
MHC_CASES = {"mhc_a": (61, 3, 64), "mhc_b": (62, 2, 256)}
# the MTP draft head on the small model (c/mtp.h): targets = the layers whose mean hidden forward_mh collects
MTP_CASE = dict(seed=91, n_layers=3, n_prompt=9, n_gen=24, depth=3, targets=[0, 2])
# the DSpark draft module on the small model (c/dspark.h); the prompt is longer than the window of 8
DSPARK_CASE = dict(seed=91, n_layers=3, n_prompt=11, n_gen=24, targets=[0, 2], n_stages=2, block_size=3, noise_id=5, rank=16,
                   temp=0.8, top_p=0.9, rng_seed=1234, draft_seed=77)

if __name__ == "__main__":
    import sys
    if sys.argv[1:] == ["ckpt"]:      # only the checkpoint case (its own file)
        main_ckpt()
    elif sys.argv[1:] == ["mtp"]:     # only the MTP draft-head case (its own file)
        main_mtp()
    elif sys.argv[1:] == ["dspark"]:  # only the DSpark case (its own file)
        main_dspark()
    elif sys.argv[1:] == ["flash"]:   # only the real-dimension model case (its own file; ~23 GB of host memory)
        main_flash()
    else:
        main()
        main_ckpt()
        main_mtp()
        main_dspark()
        main_flash()
