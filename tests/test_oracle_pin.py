"""Pins the CPU oracle (oracle/apus_oracle.c) to the reference.

Three anchors, all on CPU:
  * the reference's own golden fixtures (tests/golden/m3, m4a — produced by
    its generators, the known-answer vectors its C tests use);
  * outputs of the unmodified reference C code committed in
    tests/golden/ref_cases.npz (bitwise for everything without libm calls
    inside, which is everything but exp/log1p-bearing stages — those are
    bitwise too when run on the same libm);
  * the live reference build (oracle/_ref), when present, on fresh seeds.
"""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

import cases
from _oracle import P, ora, ora_act_quant, ora_expert, ora_moe, ora_qlinear, oqw, ref, rel_l2
from golden.make_golden import (ATTN_CASES, EXPERT_CASES, LINEAR_CASES, MHC_CASES, MOE_CASES,
                                TOPK_CASES)

GOLD = Path(__file__).resolve().parent / "golden"
G = np.load(GOLD / "ref_cases.npz")


def manifest(path):
    return {k: v for k, v in (ln.split("=") for ln in path.read_text().split())}


# ---- reference golden fixtures ---------------------------------------------------------
def test_m3_golden_act_quant_bitwise_and_gemm():
    d = GOLD / "m3"
    mf = manifest(d / "manifest.txt")
    M, O, K = int(mf["M"]), int(mf["O"]), int(mf["K"])
    x = np.fromfile(d / "act_x.bin", np.float32).reshape(M, K)
    codes = np.fromfile(d / "act_codes.bin", np.uint8).reshape(M, K)
    scales = np.fromfile(d / "act_scales.bin", np.float32).reshape(M, K // 128)
    c2 = np.empty_like(codes)
    s2 = np.empty_like(scales)
    for m in range(M):                # golden quantises the raw f32 rows (no BF16 round)
        ora().ora_act_quant_row(P(x[m]), K, P(c2[m]), P(s2[m]))
    assert np.array_equal(c2, codes) and np.array_equal(s2, scales)
    wp = np.fromfile(d / "w_packed.bin", np.uint8).reshape(O, K // 2)
    ws = np.fromfile(d / "w_scales.bin", np.uint8).reshape(O, K // 32)
    truth = np.fromfile(d / "out.bin", np.float64).reshape(M, O)
    out = np.empty((M, O), np.float32)
    ora().ora_fp4_gemm(P(wp), P(ws), P(codes), P(scales), P(out), M, O, K)
    # the reference's bound: |err| <= 2e-5 * sum of |block contributions| (tests/m3/test_fp4.c:66-100)
    esc = fp4_esc(wp, ws, codes, scales)
    assert np.all(np.abs(out - truth) <= 2e-5 * esc + 1e-30)


def fp4_esc(wp, ws, codes, scales):
    from apus_b200.synth import e4m3_table
    lut = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, 0, -.5, -1, -1.5, -2, -3, -4, -6], np.float64)
    O, K = wp.shape[0], wp.shape[1] * 2
    w = np.empty((O, K))
    w[:, 0::2] = lut[wp & 15]
    w[:, 1::2] = lut[wp >> 4]
    a = e4m3_table()[codes].astype(np.float64)
    sb = np.exp2(ws.astype(np.float64) - 127)
    esc = np.zeros((a.shape[0], O))
    for kb in range(K // 32):
        dot = a[:, kb * 32:(kb + 1) * 32] @ w[:, kb * 32:(kb + 1) * 32].T
        esc += np.abs(dot * scales[:, kb // 4].astype(np.float64)[:, None] * sb[:, kb][None, :])
    return esc


def test_m4a_golden_fp8_gemm():
    d = GOLD / "m4a"
    mf = manifest(d / "fp8_manifest.txt")
    M, O, K = int(mf["M"]), int(mf["O"]), int(mf["K"])
    wc = np.fromfile(d / "fp8_w_codes.bin", np.uint8).reshape(O, K)
    ws = np.fromfile(d / "fp8_w_scales.bin", np.uint8).reshape((O + 127) // 128, K // 128)
    x = np.fromfile(d / "fp8_act_x.bin", np.float32).reshape(M, K)
    codes = np.fromfile(d / "fp8_act_codes.bin", np.uint8).reshape(M, K)
    scales = np.fromfile(d / "fp8_act_scales.bin", np.float32).reshape(M, K // 128)
    c2 = np.empty_like(codes)
    s2 = np.empty_like(scales)
    for m in range(M):
        ora().ora_act_quant_row(P(x[m]), K, P(c2[m]), P(s2[m]))
    assert np.array_equal(c2, codes) and np.array_equal(s2, scales)
    truth = np.fromfile(d / "fp8_out.bin", np.float64).reshape(M, O)
    esc = np.fromfile(d / "fp8_esc.bin", np.float64).reshape(M, O)
    out = np.empty((M, O), np.float32)
    ora().ora_fp8_gemm(P(wc), P(ws), P(codes), P(scales), P(out), M, O, K)
    # 0 * (act_scale * 2^127) is NaN on the all-zero tile with scale byte 254 when
    # the scale product overflows; the reference's own check skips those outputs
    # (a NaN ratio never raises its running maximum, tests/m4a/test_fp8.c:239-242)
    fin = np.isfinite(out) & np.isfinite(esc)
    assert np.all(np.abs(out[fin] - truth[fin]) <= 2e-5 * np.maximum(esc[fin], 1e-30))


def test_m4a_golden_mhc():
    d = GOLD / "m4a"
    mf = manifest(d / "mhc_manifest.txt")
    T, D, N, IT = int(mf["T"]), int(mf["D"]), int(mf["N"]), int(mf["ITERS"])
    ne, he = float(mf["NORM_EPS"]), float(mf["HC_EPS"])
    x4 = np.fromfile(d / "mhc_x4.bin", np.float32).reshape(T, N * D)
    fn = np.fromfile(d / "mhc_fn.bin", np.float32)
    scale = np.fromfile(d / "mhc_scale.bin", np.float32)
    base = np.fromfile(d / "mhc_base.bin", np.float32)
    g_pre = np.fromfile(d / "mhc_pre.bin", np.float64).reshape(T, N)
    g_post = np.fromfile(d / "mhc_post.bin", np.float64).reshape(T, N)
    g_comb = np.fromfile(d / "mhc_comb.bin", np.float64).reshape(T, N, N)
    g_ypre = np.fromfile(d / "mhc_ypre.bin", np.float64).reshape(T, D)
    g_ypost = np.fromfile(d / "mhc_ypost.bin", np.float64).reshape(T, N, D)
    g_yhead = np.fromfile(d / "mhc_yhead.bin", np.float64).reshape(T, D)
    f = np.fromfile(d / "mhc_f.bin", np.float32).reshape(T, D)
    hfn = np.fromfile(d / "mhc_hfn.bin", np.float32)
    hscale = float(np.fromfile(d / "mhc_hscale.bin", np.float32)[0])
    hbase = np.fromfile(d / "mhc_hbase.bin", np.float32)
    for t in range(T):
        pre = np.empty(N, np.float32); post = np.empty(N, np.float32); comb = np.empty((N, N), np.float32)
        ora().ora_mhc_prepost(P(x4[t]), D, N, P(fn), P(scale), P(base), ne, he, IT, P(pre), P(post), P(comb), None)
        assert np.allclose(pre, g_pre[t], rtol=2e-6, atol=1e-7)
        assert np.allclose(post, g_post[t], rtol=2e-6, atol=1e-7)
        assert np.allclose(comb, g_comb[t], rtol=5e-6, atol=1e-7)
        y = np.empty(D, np.float32)
        ora().ora_mhc_collapse(P(x4[t]), P(pre), P(y), D, N)
        assert np.allclose(y, g_ypre[t], rtol=1e-4, atol=1e-3)
        y4 = np.empty((N, D), np.float32)
        ora().ora_mhc_apply(P(f[t]), P(x4[t]), P(post), P(comb), P(y4), D, N)
        assert np.allclose(y4, g_ypost[t], rtol=1e-4, atol=1e-3)
        yh = np.empty(D, np.float32)
        ora().ora_mhc_head(P(x4[t]), D, N, P(hfn), hscale, P(hbase), ne, he, P(yh))
        assert np.allclose(yh, g_yhead[t], rtol=1e-4, atol=1e-3)
    # Sinkhorn against the last of the 40 recorded stages
    mfT2 = int(mf["T2"])
    logits = np.fromfile(d / "mhc_sk_logits.bin", np.float32).reshape(mfT2, N, N)
    stages = np.fromfile(d / "mhc_sk_stages.bin", np.float64).reshape(mfT2, 40, N, N)
    for t in range(mfT2):
        c = logits[t].copy()
        ora().ora_sinkhorn(P(c), N, IT, he)
        assert np.allclose(c, stages[t, -1], rtol=5e-6, atol=1e-9)


# ---- committed outputs of the reference C code: bitwise ------------------------------------
@pytest.mark.parametrize("tag", list(LINEAR_CASES))
def test_linear_bitwise_vs_reference_outputs(tag):
    args = LINEAR_CASES[tag]
    c = cases.linear_case(*args)
    fmt = args[1]
    codes, scales = ora_act_quant(c["x"])
    assert np.array_equal(codes, G[f"{tag}.acodes"])
    assert np.array_equal(scales, G[f"{tag}.ascales"])
    M, K = c["x"].shape
    O = c["codes"].shape[0]
    raw = np.empty((M, O), np.float32)
    (ora().ora_fp4_gemm if fmt == 4 else ora().ora_fp8_gemm)(
        P(c["codes"]), P(c["scales"]), P(codes), P(scales), P(raw), M, O, K)
    assert np.array_equal(raw.view(np.uint32), G[f"{tag}.raw"].view(np.uint32))
    out = ora_qlinear(0 if fmt == 4 else 1, c["codes"], c["scales"], c["x"], O)
    assert np.array_equal(out.view(np.uint32), G[f"{tag}.out"].view(np.uint32))


@pytest.mark.parametrize("tag", list(EXPERT_CASES))
def test_expert_bitwise(tag):
    args = EXPERT_CASES[tag]
    c = cases.expert_case(*args)
    _, kind, rows, dim, inter = args
    out = ora_expert(kind, c["w1"], c["w2"], c["w3"], c["x"], inter, 10.0)
    assert np.array_equal(out.view(np.uint32), G[f"{tag}.out"].view(np.uint32))


@pytest.mark.parametrize("tag", list(MOE_CASES))
def test_moe_bitwise(tag):
    W, x, ids = cases.moe_case(**MOE_CASES[tag])
    out, idx, wgt, routed, shared = ora_moe(W, x, ids)
    assert np.array_equal(idx, G[f"{tag}.idx"])
    assert np.array_equal(wgt.view(np.uint32), G[f"{tag}.w"].view(np.uint32))
    assert np.array_equal(routed.view(np.uint32), G[f"{tag}.routed"].view(np.uint32))
    assert np.array_equal(shared.view(np.uint32), G[f"{tag}.shared"].view(np.uint32))
    assert np.array_equal(out.view(np.uint32), G[f"{tag}.out"].view(np.uint32))


@pytest.mark.parametrize("tag", list(TOPK_CASES))
def test_topk_exact(tag):
    args = TOPK_CASES[tag]
    sc = cases.topk_case(*args)
    k = args[3]
    for r in range(sc.shape[0]):
        idx = np.empty(k, np.int32)
        ora().ora_topk_stable(P(sc[r]), sc.shape[1], k, P(idx))
        assert np.array_equal(idx, G[f"{tag}.idx"][r])


@pytest.mark.parametrize("tag", list(ATTN_CASES))
def test_sparse_attn_bitwise(tag):
    args = ATTN_CASES[tag]
    c = cases.sparse_attn_case(*args)
    _, s, h, d, na, nb, idxw, _ = args
    o = np.empty((s, h, d), np.float32)
    ora().ora_sparse_attn(P(c["q"]), P(c["sink"]), h, d, P(c["idx"]), idxw, s, d ** -0.5,
                          P(c["kv_a"]), na, P(c["kv_b"]), P(o))
    assert np.array_equal(o.view(np.uint32), G[f"{tag}.o"].view(np.uint32))


@pytest.mark.parametrize("tag", list(MHC_CASES))
def test_mhc_bitwise(tag):
    args = MHC_CASES[tag]
    c = cases.mhc_case(*args)
    _, rows, d = args
    n = 4
    for t in range(rows):
        pre = np.empty(n, np.float32); post = np.empty(n, np.float32); comb = np.empty((n, n), np.float32)
        ora().ora_mhc_prepost(P(c["x4"][t]), d, n, P(c["fn"]), P(c["scale"]), P(c["base"]), 1e-6, 1e-6, 20,
                              P(pre), P(post), P(comb), None)
        assert np.array_equal(pre.view(np.uint32), G[f"{tag}.pre"][t].view(np.uint32))
        assert np.array_equal(post.view(np.uint32), G[f"{tag}.post"][t].view(np.uint32))
        assert np.array_equal(comb.view(np.uint32), G[f"{tag}.comb"][t].view(np.uint32))
        y = np.empty(d, np.float32)
        ora().ora_mhc_collapse(P(c["x4"][t]), P(pre), P(y), d, n)
        assert np.array_equal(y.view(np.uint32), G[f"{tag}.y"][t].view(np.uint32))
        y4 = np.empty((n, d), np.float32)
        ora().ora_mhc_apply(P(c["f"][t]), P(c["x4"][t]), P(post), P(comb), P(y4), d, n)
        assert np.array_equal(y4.view(np.uint32), G[f"{tag}.y4"][t].view(np.uint32))
        yh = np.empty(d, np.float32)
        ora().ora_mhc_head(P(c["x4"][t]), d, n, P(c["hfn"]), 0.8, P(c["hbase"]), 1e-6, 1e-6, P(yh))
        assert np.array_equal(yh.view(np.uint32), G[f"{tag}.yhead"][t].view(np.uint32))


# ---- scalar conversions: exhaustive -----------------------------------------------------------
def test_format_helpers_exhaustive():
    from apus_b200 import synth
    tab = synth.e4m3_table()
    for c in range(256):
        assert ora().ora_e4m3_to_f32(c) == tab[c]
        if (c & 0x7f) != 0x7f:
            assert ora().ora_e4m3_from_f32(float(tab[c])) == (c if c != 0x80 else 0x80)
    assert ora().ora_ue8m0(0) == np.float32(2.0) ** -127
    assert ora().ora_ue8m0(127) == 1.0 and np.isinf(ora().ora_ue8m0(255))
    rng = np.random.default_rng(5)
    xs = np.concatenate([rng.standard_normal(20000).astype(np.float32) * 100,
                         (rng.standard_normal(20000) * 1e-2).astype(np.float32),
                         np.array([448, 464, 480, 1e9, -1e9, 2 ** -9, 2 ** -10, 1.5 * 2 ** -10,
                                   3 * 2 ** -10, 0.0, -0.0, 2 ** -7 * 1.0625], np.float32)])
    mine = synth.e4m3_quant(xs)
    theirs = np.array([ora().ora_e4m3_from_f32(float(v)) for v in xs], np.uint8)
    assert np.array_equal(mine, theirs)
    bf = np.array([ora().ora_bf16_round(float(v)) for v in xs[:5000]], np.float32)
    assert np.array_equal(bf.view(np.uint32), synth.bf16_round(xs[:5000]).view(np.uint32))


# ---- live reference, fresh seeds ------------------------------------------------------------------
needs_ref = pytest.mark.skipif(ref() is None, reason="reference build not present")


@needs_ref
def test_live_reference_conversions():
    L = ref()
    for c in range(256):
        assert ora().ora_e4m3_to_f32(c) == L.apus_e4m3_dequant_f32(c)
        assert ora().ora_ue8m0(c) == L.apus_ue8m0_f32(c) or (c == 255)
    rng = np.random.default_rng(7)
    xs = np.concatenate([rng.standard_normal(30000).astype(np.float32) * 200,
                         (rng.standard_normal(30000) * 3e-2).astype(np.float32)])
    for v in xs:
        assert ora().ora_e4m3_from_f32(float(v)) == L.apus_e4m3_quant_f32(float(v))
        assert np.float32(ora().ora_bf16_round(float(v))) == np.float32(L.apus_bf16_round(float(v)))


@needs_ref
@pytest.mark.parametrize("seed,fmt,M,O,K", [(101, 4, 2, 128, 512), (102, 8, 3, 256, 512),
                                           (103, 4, 1, 2048, 4096), (104, 8, 1, 512, 4096)])
def test_live_reference_linear(seed, fmt, M, O, K):
    L = ref()
    from apus_b200 import capi
    c = cases.linear_case(seed, fmt, M, O, K)
    out = np.empty((M, O), np.float32)
    w = capi.qw(c["codes"], c["scales"], O, K)
    (L.apus_fp4_linear if fmt == 4 else L.apus_fp8_linear)(C.byref(w), P(c["x"]), P(out), M, K, O)
    mine = ora_qlinear(0 if fmt == 4 else 1, c["codes"], c["scales"], c["x"], O)
    assert np.array_equal(mine.view(np.uint32), out.view(np.uint32))


def row_helper_inputs():
    rng = np.random.default_rng(99)
    x = (rng.standard_normal((6, 128)) * rng.choice([1e-3, 1.0, 30.0], size=(6, 1))).astype(np.float32)
    x[1, :32] = 0.0
    x[2, 5] = -0.0
    x[3, :8] = [6, -6, 0.25, 0.75, 1.25, 2.5, 3.5, 5.0]
    cos = np.cos(rng.standard_normal(32)).astype(np.float32)
    sin = np.sin(rng.standard_normal(32)).astype(np.float32)
    return x, cos, sin


@needs_ref
def test_live_reference_row_helpers_bitwise():
    L = ref()
    x, cos, sin = row_helper_inputs()
    for fn_o, fn_r, args in (("ora_hadamard", "apus_hadamard", (128,)),
                             ("ora_fp8_qat_sim", "apus_fp8_qat_sim", (64, 64)),
                             ("ora_fp8_qat_sim", "apus_fp8_qat_sim", (128, 64)),
                             ("ora_fp4_qat_sim", "apus_fp4_qat_sim", (128,))):
        a, b = x.copy(), x.copy()
        for r in range(x.shape[0]):
            getattr(ora(), fn_o)(P(a[r]), *args)
            getattr(L, fn_r)(P(b[r]), *args)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), fn_o
    for inv in (0, 1):
        a, b = x.copy(), x.copy()
        for r in range(x.shape[0]):
            ora().ora_apply_rope(P(a[r, 64:]), P(cos), P(sin), 64, inv)
            L.apus_apply_rope(P(b[r, 64:]), P(cos), P(sin), 64, inv)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_rope_tables_match_the_reference():
    """apus_b200.flash.rope_tables restates c/attn.h:247-281; the committed tables
    were written by the reference's apus_rope_precompute (plain theta 1e4 and the
    YaRN-scaled compressed-layer table).  powf/cosf/sinf come from different
    math libraries (a frequency one ulp off moves the f32 angle at position 200
    by a few 1e-6), hence an absolute bar of 2e-5 instead of bit equality."""
    from apus_b200.flash import FlashConfig, rope_tables
    G = np.load(Path(__file__).resolve().parent / "golden" / "ref_cases.npz")
    cfg = FlashConfig()
    for name, compressed in (("plain", False), ("yarn", True)):
        cos, sin = rope_tables(cfg, compressed, 256)
        assert np.abs(cos - G[f"rope.{name}.cos"]).max() <= 2e-5
        assert np.abs(sin - G[f"rope.{name}.sin"]).max() <= 2e-5


def test_sampler_matches_the_reference():
    """Temperature + nucleus sampling and the splitmix64 stream (c/sample.h) against
    tokens and uniforms produced by the unmodified reference."""
    from golden.make_golden import SAMPLE_CASES
    G = np.load(Path(__file__).resolve().parent / "golden" / "ref_cases.npz")
    O = ora()
    for tag, (seed, rows, n, kind, temp, top_p) in SAMPLE_CASES.items():
        lg, u = cases.sample_case(seed, rows, n, kind)
        p, ordr, tmp = np.empty(n, np.float32), np.empty(n, np.int32), np.empty(n, np.int32)
        got = [O.ora_sample_logits_u(P(lg[r]), n, temp, top_p, float(u[r]), P(p), P(ordr), P(tmp)) for r in range(rows)]
        assert got == G[f"{tag}.tokens"].tolist(), tag
    st = C.c_uint64(20260729)
    assert [O.ora_rng_uniform(C.byref(st)) for _ in range(16)] == G["rng.uniforms"].tolist()
