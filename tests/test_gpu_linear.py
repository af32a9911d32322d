"""GPU parity: activation quantisation and the MXFP4 / FP8 block-scaled products,
called through the C ABI, against the CPU oracle and the committed reference
outputs.

Tolerances (north star: GEMV/GEMM outputs within rel-L2 <= 1e-3 of the
reference's f32-accumulated result):
  * activation codes and scales: bit-exact;
  * raw GEMM outputs: rel-L2 <= 1e-5 (the only difference is the order of the
    f32 additions inside one 32- or 128-wide block), and the reference's own
    error bound err <= 2e-5 * esc against the f64 truth of its fixtures;
  * BF16-rounded linears: rel-L2 <= 1e-3, at most 1 BF16 step anywhere.
"""
from pathlib import Path

import numpy as np
import pytest

import cases
from _gpu import bf16_ulps, bits, cuda_act_quant, cuda_expert, cuda_qgemm, cuda_qlinear, lib
from _oracle import P, ora, ora_act_quant, ora_expert, ora_qlinear, rel_l2
from golden.make_golden import EXPERT_CASES, LINEAR_CASES
from test_oracle_pin import fp4_esc, manifest

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
G = np.load(GOLD / "ref_cases.npz")


def test_enable_and_counters():
    L = lib()
    assert L.apus_cuda_is_enabled() == 1
    d0 = L.apus_cuda_dispatches()
    x = np.ones((1, 128), np.float32)
    cuda_act_quant(x)
    assert L.apus_cuda_dispatches() > d0


@pytest.mark.parametrize("M,K", [(1, 128), (3, 4096), (33, 2048), (257, 1024)])
def test_act_quant_bitwise(M, K):
    rng = np.random.default_rng(M * 7 + K)
    x = (rng.standard_normal((M, K)) * rng.choice([1e-6, 1e-3, 1.0, 50.0, 3e4], size=(M, 1))
         ).astype(np.float32)
    x[0, :5] = [0.0, -0.0, 448.0, -1e-7, 1e-5]
    if M > 2:
        x[2] = 0.0
    c0, s0 = ora_act_quant(x)
    c1, s1 = cuda_act_quant(x)
    assert np.array_equal(s0, s1)
    assert np.array_equal(c0, c1)


def test_act_quant_golden_fixture():
    d = GOLD / "m3"
    mf = manifest(d / "manifest.txt")
    M, K = int(mf["M"]), int(mf["K"])
    from apus_b200.synth import bf16_round
    x = bf16_round(np.fromfile(d / "act_x.bin", np.float32).reshape(M, K))
    c0, s0 = ora_act_quant(x)
    c1, s1 = cuda_act_quant(x)
    assert np.array_equal(c0, c1) and np.array_equal(s0, s1)


def test_fp4_gemm_reference_fixture_f64_truth():
    d = GOLD / "m3"
    mf = manifest(d / "manifest.txt")
    M, O, K = int(mf["M"]), int(mf["O"]), int(mf["K"])
    wp = np.fromfile(d / "w_packed.bin", np.uint8).reshape(O, K // 2)
    ws = np.fromfile(d / "w_scales.bin", np.uint8).reshape(O, K // 32)
    codes = np.fromfile(d / "act_codes.bin", np.uint8).reshape(M, K)
    scales = np.fromfile(d / "act_scales.bin", np.float32).reshape(M, K // 128)
    truth = np.fromfile(d / "out.bin", np.float64).reshape(M, O)
    out = cuda_qgemm(4, wp, ws, codes, scales, O)
    esc = fp4_esc(wp, ws, codes, scales)
    assert np.all(np.abs(out - truth) <= 2e-5 * esc + 1e-30)


def test_fp8_gemm_reference_fixture_f64_truth():
    d = GOLD / "m4a"
    mf = manifest(d / "fp8_manifest.txt")
    M, O, K = int(mf["M"]), int(mf["O"]), int(mf["K"])
    wc = np.fromfile(d / "fp8_w_codes.bin", np.uint8).reshape(O, K)
    ws = np.fromfile(d / "fp8_w_scales.bin", np.uint8).reshape((O + 127) // 128, K // 128)
    codes = np.fromfile(d / "fp8_act_codes.bin", np.uint8).reshape(M, K)
    scales = np.fromfile(d / "fp8_act_scales.bin", np.float32).reshape(M, K // 128)
    truth = np.fromfile(d / "fp8_out.bin", np.float64).reshape(M, O)
    esc = np.fromfile(d / "fp8_esc.bin", np.float64).reshape(M, O)
    out = cuda_qgemm(8, wc, ws, codes, scales, O)
    fin = np.isfinite(out) & np.isfinite(esc)
    assert fin.mean() > 0.7
    assert np.all(np.abs(out[fin] - truth[fin]) <= 2e-5 * np.maximum(esc[fin], 1e-30))


@pytest.mark.parametrize("tag", list(LINEAR_CASES))
def test_linear_vs_reference_outputs(tag):
    args = LINEAR_CASES[tag]
    fmt = args[1]
    c = cases.linear_case(*args)
    O = c["codes"].shape[0]
    raw = cuda_qgemm(fmt, c["codes"], c["scales"], G[f"{tag}.acodes"], G[f"{tag}.ascales"], O)
    ref_raw = G[f"{tag}.raw"]
    fin = np.isfinite(ref_raw)
    assert np.array_equal(np.isfinite(raw), fin)
    assert rel_l2(raw[fin], ref_raw[fin]) <= 1e-5
    out = cuda_qlinear(fmt, c["codes"], c["scales"], c["x"], O)
    ref_out = G[f"{tag}.out"]
    fin = np.isfinite(ref_out)
    assert rel_l2(out[fin], ref_out[fin]) <= 1e-3
    assert bf16_ulps(out[fin], ref_out[fin]).max() <= 1


@pytest.mark.parametrize("fmt,M,O,K", [(4, 1, 2048, 4096), (4, 8, 2048, 4096), (4, 5, 4096, 2048),
                                       (4, 17, 256, 512), (4, 40, 128, 1024), (8, 1, 2048, 4096),
                                       (8, 7, 4096, 2048), (8, 32, 1024, 4096), (8, 70, 256, 1024),
                                       (8, 300, 512, 2048), (8, 128, 256, 8192)])
def test_linear_vs_oracle_model_shapes(fmt, M, O, K):
    c = cases.linear_case(1000 + M + O + K + fmt, fmt, M, O, K)
    want = ora_qlinear(0 if fmt == 4 else 1, c["codes"], c["scales"], c["x"], O)
    got = cuda_qlinear(fmt, c["codes"], c["scales"], c["x"], O)
    assert rel_l2(got, want) <= 1e-3
    u = bf16_ulps(got, want)
    assert u.max() <= 1
    # run-to-run determinism: a second call returns the same bits
    again = cuda_qlinear(fmt, c["codes"], c["scales"], c["x"], O)
    assert np.array_equal(bits(got), bits(again))


def test_linear_m_independence():
    """Row m of an M-row call equals the M=1 call on that row (reference
    tests/m9e: batched == per-token)."""
    c = cases.linear_case(77, 4, 11, 512, 1024)
    full = cuda_qlinear(4, c["codes"], c["scales"], c["x"], 512)
    for m in (0, 5, 10):
        one = cuda_qlinear(4, c["codes"], c["scales"], c["x"][m:m + 1].copy(), 512)
        assert np.array_equal(bits(one[0]), bits(full[m]))


def test_fp8_many_rows_equal_single_rows():
    """The 128-rows-per-CTA FP8 kernel (M >= 64) returns for every row the bits of
    the M = 1 call (32-row kernel): same block dots, same block-ordered fold."""
    c = cases.linear_case(78, 8, 200, 384, 1024)
    full = cuda_qlinear(8, c["codes"], c["scales"], c["x"], 384)
    for m in (0, 63, 127, 128, 199):
        one = cuda_qlinear(8, c["codes"], c["scales"], c["x"][m:m + 1].copy(), 384)
        assert np.array_equal(bits(one[0]), bits(full[m])), m


@pytest.mark.parametrize("M,O,K", [(1, 512, 4096), (8, 1024, 4096), (7, 4096, 8192), (3, 256, 384), (2, 128, 1024)])
def test_fp8_split_k_is_the_single_fold_bit_for_bit(M, O, K):
    """With few activation rows an FP8 matrix with few output tiles is split along K over
    CTAs; the chunks park every block's term and the last CTA adds them in block order.
    That is the single in-order fold value for value: the rows must equal, bit for bit,
    the same rows inside a 40-row call (which is not split), and stay within the bars
    against the reference restatement; the FP8 SwiGLU pair takes the same path."""
    L = lib()
    c = cases.linear_case(500 + M + O, 8, 40, O, K)
    full = cuda_qlinear(8, c["codes"], c["scales"], c["x"], O)
    few = cuda_qlinear(8, c["codes"], c["scales"], c["x"][:M].copy(), O)
    assert L.apus_cuda_kernel_status(1) == 0
    assert np.array_equal(bits(few), bits(full[:M]))
    want = ora_qlinear(8, c["codes"], c["scales"], c["x"][:M].copy(), O)
    assert rel_l2(few, want) <= 1e-3 and (bf16_ulps(few, want) > 0).mean() <= 2e-3
    e = cases.expert_case(600 + M, 1, 40, 512, 256)
    ge_full = cuda_expert(1, e["w1"], e["w2"], e["w3"], e["x"], 256, 10.0)
    ge_few = cuda_expert(1, e["w1"], e["w2"], e["w3"], e["x"][:M].copy(), 256, 10.0)
    assert np.array_equal(bits(ge_few), bits(ge_full[:M]))
    assert rel_l2(ge_few, ora_expert(1, e["w1"], e["w2"], e["w3"], e["x"][:M].copy(), 256, 10.0)) <= 1e-3


@pytest.mark.parametrize("tag", list(EXPERT_CASES))
def test_expert_vs_reference_outputs(tag):
    args = EXPERT_CASES[tag]
    _, kind, rows, dim, inter = args
    c = cases.expert_case(*args)
    got = cuda_expert(kind, c["w1"], c["w2"], c["w3"], c["x"], inter, 10.0)
    assert rel_l2(got, G[f"{tag}.out"]) <= 1e-3


def test_expert_config0_shape():
    """Config 0: one MXFP4 SwiGLU expert, x [8,4096], 2048 intermediate."""
    c = cases.expert_case(0, 0, 8, 4096, 2048)
    want = ora_expert(0, c["w1"], c["w2"], c["w3"], c["x"], 2048, 10.0)
    got = cuda_expert(0, c["w1"], c["w2"], c["w3"], c["x"], 2048, 10.0)
    assert np.isfinite(got).all()
    assert rel_l2(got, want) <= 1e-3
    assert (bf16_ulps(got, want) > 0).mean() < 5e-3


def test_grouped_gemm_matches_per_entry():
    import ctypes as C
    from apus_b200 import capi, synth
    rng = np.random.default_rng(5)
    O, K, rows = 256, 512, 23
    x = synth.activations(rng, rows, K)
    codes, scales = ora_act_quant(x)
    ents, outs, ws = [], [], []
    spans = [(0, 1), (1, 9), (10, 13)]
    arr = (capi.Fp4GemmEnt * len(spans))()
    for i, (m0, M) in enumerate(spans):
        w = synth.fp4_weight(rng, O, K)
        ws.append(w)
        o = np.zeros((M, O), np.float32)
        outs.append(o)
        arr[i] = capi.Fp4GemmEnt(capi.ptr(w[0]), capi.ptr(w[1]), capi.ptr(o), m0, M)
    rc = lib().apus_cuda_fp4_gemm_grouped(arr, len(spans), capi.ptr(codes), capi.ptr(scales), rows, O, K)
    assert rc == 0
    for w in ws:
        lib().apus_cuda_forget(capi.ptr(w[0]))
    for (m0, M), w, o in zip(spans, ws, outs):
        single = cuda_qgemm(4, w[0], w[1], codes[m0:m0 + M].copy(), scales[m0:m0 + M].copy(), O)
        assert np.array_equal(bits(single), bits(o))


def test_unsupported_shape_fails_loudly():
    import ctypes as C
    from apus_b200 import capi
    codes = np.zeros((24, 48), np.uint8)
    scales = np.zeros((24, 3), np.uint8)
    x = np.zeros((1, 96), np.float32)
    out = np.zeros((1, 24), np.float32)
    w = capi.qw(codes, scales, 24, 96)
    assert lib().apus_cuda_fp4_linear(C.byref(w), capi.ptr(x), capi.ptr(out), 1, 96, 24) != 0
    assert b"multiple" in lib().apus_cuda_last_error()
