"""GPU parity of the attention sublayer (q path, window KV, compressors,
indexer, gathered attention, o-projection) and its row helpers through the C
ABI against outputs and final states of the reference's apus_attention.

Bars: row helpers bit-exact; per-token sublayer outputs rel-L2 <= 5e-3 against
the reference (BF16 outputs after a chain of BF16-rounded stages whose sums
are ordered differently), compressed caches and ring within 1 BF16 step on
all but a small fraction of elements, entry counts exact.
"""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

import cases
from _gpu import bf16_ulps, bits, lib
from _oracle import P, ora, rel_l2
from apus_b200 import capi
from golden.make_golden import ATTN_LAYER_CASES
from test_oracle_pin import row_helper_inputs

pytestmark = pytest.mark.gpu
G = np.load(Path(__file__).resolve().parent / "golden" / "ref_cases.npz")


def test_row_helpers_bitwise():
    L = lib()
    x, cos, sin = row_helper_inputs()
    for ora_fn, cuda_call in (
            (lambda r: ora().ora_hadamard(P(r), 128), lambda a: L.apus_cuda_hadamard(P(a), 128, a.shape[0])),
            (lambda r: ora().ora_fp8_qat_sim(P(r), 64, 64), lambda a: L.apus_cuda_fp8_qat_sim(P(a), 128, 64, a.shape[0])),
            (lambda r: ora().ora_fp8_qat_sim(P(r), 128, 64), lambda a: L.apus_cuda_fp8_qat_sim(P(a), 128, 128, a.shape[0])),
            (lambda r: ora().ora_fp4_qat_sim(P(r), 128), lambda a: L.apus_cuda_fp4_qat_sim(P(a), 128, a.shape[0]))):
        want, got = x.copy(), x.copy()
        for r in range(x.shape[0]):
            ora_fn(want[r])
        assert cuda_call(got) == 0, L.apus_cuda_last_error()
        assert np.array_equal(bits(got), bits(want))
    for inv in (0, 1):
        want, got = x.copy(), x.copy()
        for r in range(x.shape[0]):
            ora().ora_apply_rope(P(want[r, 64:]), P(cos), P(sin), 64, inv)
        assert L.apus_cuda_apply_rope(P(got), P(cos), P(sin), 128, 64, inv, x.shape[0]) == 0
        assert np.array_equal(bits(got), bits(want))


def run_cuda(seed, kind, chunks, cos, sin, interm=False):
    L = lib()
    Lyr = cases.AttnLayer(seed, kind)
    S = cases.AttnState(Lyr)
    D = Lyr.D
    total = sum(chunks)
    x = cases.attn_inputs(seed + 7, total, D["dim"])
    out = np.empty((total, D["dim"]), np.float32)
    pos = 0
    for n in chunks:
        rc = L.apus_cuda_attention(C.byref(Lyr.cfg), C.byref(Lyr.w), C.byref(S.st), P(x[pos:pos + n]), n, pos,
                                   P(cos), P(sin), P(out[pos:pos + n]), None)
        assert rc == 0, L.apus_cuda_last_error()
        pos += n
    for a in Lyr.weight_ptrs():
        L.apus_cuda_forget(P(a))
    return Lyr, S, out


@pytest.mark.parametrize("tag", list(ATTN_LAYER_CASES))
def test_attention_vs_reference(tag):
    seed, kind, chunks = ATTN_LAYER_CASES[tag]
    cos, sin = np.ascontiguousarray(G[f"{tag}.cos"]), np.ascontiguousarray(G[f"{tag}.sin"])
    Lyr, S, out = run_cuda(seed, kind, chunks, cos, sin)
    want = G[f"{tag}.out"]
    per_tok = [rel_l2(out[t], want[t]) for t in range(out.shape[0])]
    print(tag, "max per-token rel-L2", max(per_tok))
    assert rel_l2(out, want) <= 5e-3
    assert max(per_tok) <= 2e-2
    # final state
    assert (bf16_ulps(S.win, G[f"{tag}.win"]) > 1).mean() <= 0.01
    if Lyr.ratio:
        cache = G[f"{tag}.comp_cache"]
        assert S.st.comp.nb == cache.shape[0]
        assert (bf16_ulps(S.comp[2][:cache.shape[0]], cache) > 1).mean() <= 0.01
        assert np.allclose(S.comp[0], G[f"{tag}.comp_kv"], rtol=1e-5, atol=1e-5)
        m = np.isfinite(G[f"{tag}.comp_sc"])
        assert np.array_equal(np.isfinite(S.comp[1]), m)
        assert np.allclose(S.comp[1][m], G[f"{tag}.comp_sc"][m], rtol=1e-5, atol=1e-5)
        if kind == "csa":
            ic = G[f"{tag}.idx_cache"]
            assert S.st.idx_comp.nb == ic.shape[0]
            assert (bf16_ulps(S.idx[2][:ic.shape[0]], ic) > 1).mean() <= 0.02


def test_attention_chunking_invariance():
    """Feeding the same tokens as one call or token by token gives the same
    bits (reference tests/m4c: prefill == prefill + decodes)."""
    tag = "attn_csa"
    seed, kind, chunks = ATTN_LAYER_CASES[tag]
    cos, sin = np.ascontiguousarray(G[f"{tag}.cos"]), np.ascontiguousarray(G[f"{tag}.sin"])
    total = sum(chunks)
    _, S1, o1 = run_cuda(seed, kind, [total], cos, sin)
    _, S2, o2 = run_cuda(seed, kind, [1] * total, cos, sin)
    assert np.array_equal(bits(o1), bits(o2))
    assert np.array_equal(bits(S1.win), bits(S2.win))
    assert np.array_equal(bits(S1.comp[2]), bits(S2.comp[2]))
