"""GPU parity of the tcgen05 block-scaled MXFP4 kernel (TMA-unpacked weights in
the reference storage, UE8M0 scale factors in tensor memory) against the CPU
oracle, the reference fixtures and the mma.sync kernel.

Tolerance: raw GEMM rel-L2 <= 1e-5 (f32 summation order only) and the
reference's err <= 2e-5 * esc bound on its f64-truth fixture.
"""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

import cases
from _gpu import bits, cuda_moe, lib
from _oracle import P, ora, ora_act_quant, ora_moe, rel_l2
from apus_b200 import capi, synth
from golden.make_golden import LINEAR_CASES

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
G = np.load(GOLD / "ref_cases.npz")


def tc_gemm(w, ws, codes, scales, O):
    M, K = codes.shape
    out = np.full((M, O), np.nan, np.float32)
    rc = lib().apus_cuda_fp4_gemm_tc(P(w), P(ws), P(codes), P(scales), P(out), M, O, K)
    assert rc == 0, lib().apus_cuda_last_error()
    return out


@pytest.mark.parametrize("M,O,K", [(1, 128, 512), (5, 128, 1024), (32, 256, 512), (33, 256, 512),
                                   (1, 2048, 4096), (8, 2048, 4096), (40, 4096, 2048), (100, 128, 1024)])
def test_tc_gemm_vs_oracle(M, O, K):
    rng = np.random.default_rng(M + O + K)
    w, ws = synth.fp4_weight(rng, O, K, 118, 130)
    x = synth.activations(rng, M, K, std=3.0)
    if M > 2:
        x[1] = 0.0
        x[2, K // 2:] *= 100.0
    codes, scales = ora_act_quant(x)
    want = np.empty((M, O), np.float32)
    ora().ora_fp4_gemm(P(w), P(ws), P(codes), P(scales), P(want), M, O, K)
    got = tc_gemm(w, ws, codes, scales, O)
    assert rel_l2(got, want) <= 1e-5
    again = tc_gemm(w, ws, codes, scales, O)
    assert np.array_equal(bits(got), bits(again))
    assert lib().apus_cuda_kernel_status(1) == 0


def test_tc_gemm_scale_byte_corners():
    """UE8M0 corners: byte 0 (2^-127), 1, 254; all-zero and all -6 blocks."""
    c = cases.linear_case(11, 4, 3, 128, 512, True)
    codes, scales = ora_act_quant(c["x"])
    want = np.empty((3, 128), np.float32)
    ora().ora_fp4_gemm(P(c["codes"]), P(c["scales"]), P(codes), P(scales), P(want), 3, 128, 512)
    got = tc_gemm(c["codes"], c["scales"], codes, scales, 128)
    fin = np.isfinite(want)
    assert np.array_equal(np.isfinite(got), fin)
    assert rel_l2(got[fin], want[fin]) <= 1e-5


def test_tc_moe_matches_oracle_and_mma_sync_kernel():
    W = synth.MoeWeights(seed=311, E=16, topk=4)
    rng = np.random.default_rng(4)
    x = synth.activations(rng, 20, W.dim)
    want = ora_moe(W, x)
    L = lib()
    w = W.moew()
    outs = {}
    for tc in (1, 0):
        h = L.apus_cuda_moe_get(C.byref(w))
        assert h
        assert L.apus_cuda_moe_use_tc(h, tc) == tc
        out = np.empty((20, W.dim), np.float32)
        routed = np.empty((20, W.dim), np.float32)
        idx = np.empty((20, W.topk), np.int32)
        it = capi.MoeInterm(None, None, None, P(idx), P(routed), None)
        assert L.apus_cuda_moe_forward(C.byref(w), P(x), None, 20, P(out), C.byref(it)) == 0, \
            L.apus_cuda_last_error()
        outs[tc] = (out, routed, idx)
    L.apus_cuda_forget(P(W.gate_w))
    assert np.array_equal(outs[1][2], want[1]) and np.array_equal(outs[0][2], want[1])
    for tc in (1, 0):
        assert rel_l2(outs[tc][1], want[3]) <= 1e-3
        assert rel_l2(outs[tc][0], want[0]) <= 1e-3
    assert rel_l2(outs[1][1], outs[0][1]) <= 1e-3
