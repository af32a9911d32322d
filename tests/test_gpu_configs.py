"""The single-operator configurations at their stated sizes against the unmodified reference
(oracle/_ref, all host cores): the FP8 block-scaled GEMM W [4096, 4096] with M = 1, 32, 512, 4096
(c/attn.h:408-449 apus_fp8_linear), and one MoE sublayer at the model's sizes -- 256 routed MXFP4
experts, top-6, FP8 shared expert -- for T = 1, 32 and 512 tokens (c/moe.h:369-595).  The MoE
weights are one layer of the benchmarked model (the counter-based generator's host build)."""
import ctypes as C

import numpy as np
import pytest

from _gpu import bf16_ulps, bits, lib, ok
from _oracle import P, ref, rel_l2
from apus_b200 import capi, synth

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(ref() is None, reason="reference build not present")]


@pytest.mark.parametrize("M", [1, 32, 512, 4096])
def test_fp8_gemm_4096x4096_vs_reference(M):
    rng = np.random.default_rng(4096 + M)
    O = K = 4096
    codes, scales = synth.fp8_weight(rng, O, K, std=0.02)
    x = synth.activations(rng, M, K)
    w = capi.qw(codes, scales, O, K)
    want, got = np.empty((M, O), np.float32), np.empty((M, O), np.float32)
    ref().apus_fp8_linear(C.byref(w), P(x), P(want), M, K, O)
    ok(lib().apus_cuda_fp8_linear(C.byref(w), P(x), P(got), M, K, O), "fp8_linear")
    lib().apus_cuda_forget(P(codes))
    off = bf16_ulps(got, want)
    print("M", M, "rel-L2", rel_l2(got, want), "elements one BF16 step off", float((off > 0).mean()))
    assert rel_l2(got, want) <= 1e-3
    # one BF16 step at most, wherever a step means something: an output that cancels to almost nothing
    # carries the products' different summation order in its leading bits
    floor = 0.05 * float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    big = np.abs(want) >= floor
    assert off[big].max() <= 1 and (off > 0).mean() <= 2e-2
    assert np.abs(got - want)[~big].max() <= floor * 2.0 ** -6


@pytest.fixture(scope="module")
def flash_moe():
    """The MoE sublayer of layer 3 of the benchmarked model (scored routing, 256 experts) on the host."""
    import flash_case
    from apus_b200.flash import RandomFlashModel
    cfg = flash_case.config(6)
    W = RandomFlashModel(cfg, flash_case.CASE["seed"], "host", max_pos=64, layer_ids=[3])
    yield cfg, W
    lib().apus_cuda_disable()                  # drops the device copy of the 256 experts


@pytest.mark.parametrize("T", [1, 32, 512])
def test_moe_layer_256_experts_vs_reference(flash_moe, T):
    cfg, W = flash_moe
    mw = W.desc.layers[0].mw
    assert mw.E == 256 and mw.topk == 6 and not mw.hash
    x = synth.activations(np.random.default_rng(900 + T), T, cfg.dim)
    ids = np.zeros(T, np.int64)

    def run(fn):
        out = np.empty((T, cfg.dim), np.float32)
        r = dict(sp=np.empty((T, mw.E), np.float32), biased=np.zeros((T, mw.E), np.float32), w=np.empty((T, mw.topk), np.float32),
                 idx=np.empty((T, mw.topk), np.int32), routed=np.empty((T, cfg.dim), np.float32),
                 shared=np.empty((T, cfg.dim), np.float32))
        it = capi.MoeInterm(P(r["sp"]), P(r["biased"]), P(r["w"]), P(r["idx"]), P(r["routed"]), P(r["shared"]))
        rc = fn(C.byref(mw), P(x), P(ids), T, P(out), C.byref(it))
        r["out"] = out
        return rc, r
    _, want = run(ref().apus_moe_forward)
    rc, got = run(lib().apus_cuda_moe_forward)
    assert rc == 0, lib().apus_cuda_last_error()
    same = np.all(got["idx"] == want["idx"], axis=1)                 # a token whose sixth expert is a near-tie may differ
    print("T", T, "tokens with the reference's experts", int(same.sum()), "of", T,
          "out rel-L2", rel_l2(got["out"][same], want["out"][same]))
    assert same.mean() >= 0.99
    assert rel_l2(got["sp"], want["sp"]) <= 1e-5
    assert rel_l2(got["out"][same], want["out"][same]) <= 1e-3
    assert rel_l2(got["routed"][same], want["routed"][same]) <= 1e-3
    assert rel_l2(got["shared"], want["shared"]) <= 1e-3
    w_, g_ = want["out"][same], got["out"][same]
    # an output is six weighted expert rows plus the shared expert, each BF16-rounded at the size of the
    # row: where they cancel, one step of a term is many steps of the sum -- count steps on the outputs
    # that are as large as their terms, bound the rest in absolute terms
    rms = float(np.sqrt(np.mean(w_.astype(np.float64) ** 2)))
    assert bf16_ulps(g_, w_)[np.abs(w_) >= rms].max() <= 2
    assert np.abs(g_ - w_).max() <= rms * 2.0 ** -5
