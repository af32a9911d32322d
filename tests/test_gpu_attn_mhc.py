"""GPU parity: stable top-k, sparse attention, mHC, RMSNorm and the dense f32 /
bf16 linears through the C ABI, against the CPU oracle and the committed
reference outputs.

Bars: top-k indices bit-exact (ties included: the rule is deterministic);
sparse-attention and mHC outputs within rel-L2 <= 1e-3 (exp/expf are
tolerance-class across libms) and at most 1 BF16 step on rounded outputs;
f32 linears rel-L2 <= 1e-5 (summation order only).
"""
import ctypes as C

import numpy as np
import pytest

import cases
from _gpu import bf16_ulps, bits, lib
from _oracle import P, ora, rel_l2
from apus_b200 import capi, synth
from golden.make_golden import ATTN_CASES, MHC_CASES, TOPK_CASES

pytestmark = pytest.mark.gpu
G = np.load(__import__("pathlib").Path(__file__).resolve().parent / "golden" / "ref_cases.npz")


def cuda_topk(sc, k):
    rows, n = sc.shape
    idx = np.empty((rows, k), np.int32)
    assert lib().apus_cuda_topk_stable(P(sc), n, k, P(idx), rows) == 0, lib().apus_cuda_last_error()
    return idx


@pytest.mark.parametrize("tag", list(TOPK_CASES))
def test_topk_vs_reference(tag):
    args = TOPK_CASES[tag]
    sc = cases.topk_case(*args)
    assert np.array_equal(cuda_topk(sc, args[3]), G[f"{tag}.idx"])


@pytest.mark.parametrize("n,k,ties", [(256, 6, False), (2048, 512, True), (32768, 512, True),
                                      (262144, 512, False), (262144, 512, True), (5, 5, True),
                                      (1000, 1, True)])
def test_topk_vs_oracle_long_rows(n, k, ties):
    """Indexer rows up to the 1M-context size (n = ctx/4 = 262144, k = 512); the
    BF16-rounded variant has ties everywhere, resolved by lowest index."""
    rng = np.random.default_rng(n + k)
    sc = rng.standard_normal((2, n)).astype(np.float32)
    if ties:
        sc = synth.bf16_round(sc)
        sc[1, n // 2:] = -np.inf
    want = np.empty((2, k), np.int32)
    # the O(n*k) oracle is slow at n = 262144: use numpy's stable sort, which
    # is the same order (descending score, ascending index), checked against
    # the oracle on the short rows
    for r in range(2):
        order = np.lexsort((np.arange(n), -sc[r].astype(np.float64)))
        want[r] = order[:k]
        if n <= 4096:
            o = np.empty(k, np.int32)
            ora().ora_topk_stable(P(sc[r]), n, k, P(o))
            assert np.array_equal(o, want[r])
    assert np.array_equal(cuda_topk(sc, k), want)


def cuda_sparse_attn(c, s, h, d, na, nb, idxw):
    o = np.empty((s, h, d), np.float32)
    rc = lib().apus_cuda_sparse_attn(P(c["q"]), P(c["sink"]), h, d, P(c["idx"]), idxw, s, d ** -0.5,
                                     P(c["kv_a"]), na, P(c["kv_b"]), nb, P(o))
    assert rc == 0, lib().apus_cuda_last_error()
    return o


@pytest.mark.parametrize("tag", list(ATTN_CASES))
def test_sparse_attn_vs_reference(tag):
    args = ATTN_CASES[tag]
    _, s, h, d, na, nb, idxw, _ = args
    c = cases.sparse_attn_case(*args)
    got = cuda_sparse_attn(c, s, h, d, na, nb, idxw)
    want = G[f"{tag}.o"]
    assert rel_l2(got, want) <= 1e-3
    assert bf16_ulps(got, want).max() <= 1


def test_sparse_attn_flash_dims_csa_decode():
    """Config 3 shape, CSA decode: 64 heads x 512, 128 ring rows + 512 selected of
    a compressed cache, 2 queries (the oracle needs seconds per query)."""
    s, h, d, na, nb, idxw = 2, 64, 512, 128, 2048, 640
    rng = np.random.default_rng(3)
    c = cases.sparse_attn_case(303, s, h, d, na, nb, idxw, "full")
    sel = np.stack([np.concatenate([np.arange(na), na + rng.choice(nb, 512, replace=False)])
                    for _ in range(s)]).astype(np.int32)
    c["idx"] = sel
    want = np.empty((s, h, d), np.float32)
    ora().ora_sparse_attn(P(c["q"]), P(c["sink"]), h, d, P(c["idx"]), idxw, s, d ** -0.5,
                          P(c["kv_a"]), na, P(c["kv_b"]), P(want))
    got = cuda_sparse_attn(c, s, h, d, na, nb, idxw)
    assert rel_l2(got, want) <= 1e-3
    assert (bf16_ulps(got, want) > 0).mean() < 1e-2


def test_sparse_attn_bf16_cache_dev_matches_f32_host_path():
    """The device-resident entry point takes BF16 caches; values are identical,
    so the result must equal the host-pointer path bit for bit."""
    import torch
    s, h, d, na, nb, idxw = 3, 8, 128, 16, 100, 40
    c = cases.sparse_attn_case(77, s, h, d, na, nb, idxw, "holes")
    host = cuda_sparse_attn(c, s, h, d, na, nb, idxw)
    dev = torch.device("cuda")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    q, sink, idx = t(c["q"]), t(c["sink"]), t(c["idx"])
    ka = t(synth.bf16_bits(c["kv_a"]).view(np.int16))
    kb = t(synth.bf16_bits(c["kv_b"]).view(np.int16))
    o = torch.empty(s, h, d, device=dev)
    rc = lib().apus_cuda_sparse_attn_dev(q.data_ptr(), sink.data_ptr(), h, d, idx.data_ptr(), idxw, s,
                                         d ** -0.5, ka.data_ptr(), na, kb.data_ptr(), nb, o.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert np.array_equal(bits(o.cpu().numpy()), bits(host))


@pytest.mark.parametrize("tag", list(MHC_CASES))
def test_mhc_vs_reference(tag):
    args = MHC_CASES[tag]
    _, rows, d = args
    n = 4
    c = cases.mhc_case(*args)
    L = lib()
    pre = np.empty((rows, n), np.float32); post = np.empty((rows, n), np.float32)
    comb = np.empty((rows, n, n), np.float32)
    assert L.apus_cuda_mhc_prepost(P(c["x4"]), d, n, P(c["fn"]), P(c["scale"]), P(c["base"]), 1e-6, 1e-6,
                                   20, P(pre), P(post), P(comb), rows) == 0
    # reference sum order: only exp (double-evaluated here, host libm there) can differ
    assert np.allclose(pre, G[f"{tag}.pre"], rtol=5e-6, atol=1e-7)
    assert np.allclose(post, G[f"{tag}.post"], rtol=5e-6, atol=1e-7)
    assert np.allclose(comb, G[f"{tag}.comb"], rtol=5e-6, atol=1e-7)
    # hc_pre: collapse + BF16 round fused with RMSNorm
    y = np.empty((rows, d), np.float32); yn = np.empty((rows, d), np.float32)
    post2 = np.empty_like(post); comb2 = np.empty_like(comb)
    assert L.apus_cuda_hc_pre(P(c["x4"]), d, n, P(c["fn"]), P(c["scale"]), P(c["base"]), 1e-6, 1e-6, 20,
                              P(c["norm_w"]), 1e-6, P(y), P(yn), P(post2), P(comb2), rows) == 0
    want_y = synth.bf16_round(G[f"{tag}.y"])
    assert bf16_ulps(y, want_y).max() <= 1
    assert rel_l2(y, want_y) <= 1e-3
    assert rel_l2(yn, G[f"{tag}.ynorm"]) <= 2e-3
    assert np.array_equal(bits(post2), bits(post))
    # hc_post on the reference's own post/comb: elementwise, bit-exact
    y4 = np.empty((rows, n, d), np.float32)
    rp, rc_ = np.ascontiguousarray(G[f"{tag}.post"]), np.ascontiguousarray(G[f"{tag}.comb"])
    assert L.apus_cuda_hc_post(P(c["f"]), P(c["x4"]), P(rp), P(rc_), P(y4), d, n, rows) == 0
    assert np.array_equal(bits(y4), bits(synth.bf16_round(G[f"{tag}.y4"])))
    yh = np.empty((rows, d), np.float32)
    assert L.apus_cuda_hc_head(P(c["x4"]), d, n, P(c["hfn"]), 0.8, P(c["hbase"]), 1e-6, 1e-6, P(yh), rows) == 0
    want_h = synth.bf16_round(G[f"{tag}.yhead"])
    assert bf16_ulps(yh, want_h).max() <= 1
    L.apus_cuda_forget(P(c["fn"])); L.apus_cuda_forget(P(c["hfn"]))


def test_mhc_flash_dims():
    """hc_mult 4 x hidden 4096: the 24 x 16384 map matrix of the real model."""
    rows, d, n = 3, 4096, 4
    c = cases.mhc_case(404, rows, d)
    pre = np.empty((rows, n), np.float32); post = np.empty((rows, n), np.float32)
    comb = np.empty((rows, n, n), np.float32)
    assert lib().apus_cuda_mhc_prepost(P(c["x4"]), d, n, P(c["fn"]), P(c["scale"]), P(c["base"]), 1e-6,
                                       1e-6, 20, P(pre), P(post), P(comb), rows) == 0
    for t in range(rows):
        p = np.empty(n, np.float32); q = np.empty(n, np.float32); cb = np.empty((n, n), np.float32)
        ora().ora_mhc_prepost(P(c["x4"][t]), d, n, P(c["fn"]), P(c["scale"]), P(c["base"]), 1e-6, 1e-6, 20,
                              P(p), P(q), P(cb), None)
        assert np.allclose(pre[t], p, rtol=5e-6, atol=1e-7)
        assert np.allclose(post[t], q, rtol=5e-6, atol=1e-7)
        assert np.allclose(comb[t], cb, rtol=5e-6, atol=1e-7)
    lib().apus_cuda_forget(P(c["fn"]))


@pytest.mark.parametrize("rows,n", [(1, 4096), (5, 1024), (3, 512), (2, 128)])
def test_rmsnorm(rows, n):
    rng = np.random.default_rng(n)
    x = synth.activations(rng, rows, n, std=2.0)
    w = (1 + 0.05 * rng.standard_normal(n)).astype(np.float32)
    y = np.empty_like(x)
    assert lib().apus_cuda_rmsnorm(P(x), P(w), 1e-6, P(y), n, rows) == 0
    want = np.empty_like(x)
    for r in range(rows):
        ora().ora_rms_norm(P(x[r]), P(w), 1e-6, P(want[r]), n)
    assert bf16_ulps(y, want).max() <= 1 and rel_l2(y, want) <= 1e-3


@pytest.mark.parametrize("M,K,O,flags", [(1, 4096, 256, 0), (32, 4096, 256, 0), (3, 4096, 64, 3),
                                         (2, 4096, 1024, 6), (9, 512, 40, 0)])
def test_f32_linear(M, K, O, flags):
    rng = np.random.default_rng(M + K + O)
    x = (rng.standard_normal((M, K))).astype(np.float32)
    wf = synth.bf16_round((rng.standard_normal((O, K)) * 0.02).astype(np.float32))
    w = synth.bf16_bits(wf) if flags & 4 else wf
    out = np.empty((M, O), np.float32); want = np.empty((M, O), np.float32)
    assert lib().apus_cuda_f32_linear(P(w), P(x), P(out), M, K, O, flags) == 0
    ora().ora_f32_linear(P(w), P(x), P(want), M, K, O, flags)
    lib().apus_cuda_forget(P(w))
    if flags & 2:
        assert bf16_ulps(out, want).max() <= 1
    assert rel_l2(out, want) <= 1e-5 if not flags & 2 else rel_l2(out, want) <= 1e-3


@pytest.mark.parametrize("M", [1, 5, 32])
@pytest.mark.parametrize("flags", [0, 1, 4, 5, 7])
def test_f32_linear_bitwise_reference_order(M, flags):
    """Reference sum order, bit for bit, over tiles that take the fused walk (BF16
    operands: one FMA per term is the same number) and tiles that must not (true f32
    inputs, products in the subnormal range, huge values)."""
    rng = np.random.default_rng(100 * M + flags)
    K, O = 1024, 96
    x = rng.standard_normal((M, K)).astype(np.float32)
    if flags & 1 or flags == 4:
        x = synth.bf16_round(x)                       # BF16 values: fused tiles
    else:
        x[:, :256] = synth.bf16_round(x[:, :256])     # mixed: tiles 0,1 fused, the rest not
    wf = synth.bf16_round((rng.standard_normal((O, K)) * 0.02).astype(np.float32))
    wf[:, 5] = 0.0; x[:, 7] = 0.0; x[0, 9] = -0.0
    # subnormal-range products and operands outside the exact window in tiles 4 and 5
    x[:, 520] = np.float32(1.5e-22); wf[:, 520] = synth.bf16_round(np.float32(1.3e-20).reshape(1))[0]
    x[:, 650] = synth.bf16_round(np.float32(3e25).reshape(1))[0]
    x[-1, 651] = np.float32(1e-41)                    # a subnormal input
    w = synth.bf16_bits(wf) if flags & 4 else wf
    out = np.empty((M, O), np.float32); want = np.empty((M, O), np.float32)
    assert lib().apus_cuda_f32_linear(P(w), P(x), P(out), M, K, O, flags) == 0
    ora().ora_f32_linear(P(w), P(x), P(want), M, K, O, flags)
    lib().apus_cuda_forget(P(w))
    assert np.array_equal(out.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("M,K,O", [(1, 4096, 1280), (5, 512, 256), (32, 4096, 1024), (70, 1024, 384), (3, 448, 128)])
@pytest.mark.parametrize("flags", [4, 5, 7])
def test_bf16_linear_on_the_tensor_core(M, K, O, flags):
    """BF16 weights in tree order run on the tcgen05 BF16 kernel (one or several K
    chunks, one to three row groups): products are exact, only the order of the f32
    adds differs from the reference's chain -- rel-L2 <= 1e-5 unrounded, within one
    BF16 step on <= 0.2 % of the outputs when rounded; run to run identical bits."""
    rng = np.random.default_rng(M * 7 + K + O + flags)
    x = synth.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    w = synth.bf16_bits((rng.standard_normal((O, K)) * 0.02).astype(np.float32))
    out, again, want = (np.empty((M, O), np.float32) for _ in range(3))
    L = lib()
    old = L.apus_cuda_set_tree_ops(-1)
    try:
        L.apus_cuda_set_tree_ops(511)
        assert L.apus_cuda_f32_linear(P(w), P(x), P(out), M, K, O, flags) == 0, L.apus_cuda_last_error()
        assert L.apus_cuda_f32_linear(P(w), P(x), P(again), M, K, O, flags) == 0
    finally:
        L.apus_cuda_set_tree_ops(old)
    L.apus_cuda_forget(P(w))
    ora().ora_f32_linear(P(w), P(x), P(want), M, K, O, flags)
    assert L.apus_cuda_kernel_status(1) == 0
    assert np.array_equal(out.view(np.uint32), again.view(np.uint32))
    if flags & 2:
        u = bf16_ulps(out, want)
        big = np.abs(want) > 1e-3 * np.abs(want).max()       # an output next to zero has no meaningful step count
        assert u[big].max() <= 1 and (u > 0).mean() <= 2e-3, (u[big].max(), (u > 0).mean())
        assert rel_l2(out, want) <= 1e-3
    else:
        assert rel_l2(out, want) <= 1e-5, rel_l2(out, want)


def test_head_gemv_bf16_and_hook_table():
    rng = np.random.default_rng(9)
    O, K = 12928, 4096                         # a tenth of the 129280-row LM head
    w = synth.bf16_bits((rng.standard_normal((O, K)) * 0.02).astype(np.float32))
    x = synth.activations(rng, 1, K)
    out = np.empty(O, np.float32); want = np.empty(O, np.float32)
    assert lib().apus_cuda_head_gemv_bf16(P(w), P(x), P(out), O, K) == 0
    ora().ora_head_gemv_bf16(P(w), P(x), P(want), O, K)
    assert rel_l2(out, want) <= 1e-5
    assert int(np.argmax(out)) == int(np.argmax(want))
    # the plugin table: three non-NULL slots that compute the same thing
    hooks = capi.Hooks()
    assert lib().apus_cuda_fill_hooks(C.byref(hooks), 160, 240) == 0
    assert hooks.fp8_linear and hooks.f32_linear and hooks.head_gemv

    class StTensor(C.Structure):               # reference c/st.h:49-56
        _fields_ = [("name", C.c_char * 160), ("dtype", C.c_int), ("ndim", C.c_int),
                    ("shape", C.c_int64 * 8), ("data", C.c_void_p), ("nbytes", C.c_size_t)]
    assert StTensor.dtype.offset == 160 and StTensor.data.offset == 232
    assert lib().apus_cuda_fill_hooks(C.byref(hooks), StTensor.dtype.offset, StTensor.data.offset) == 0
    t = StTensor(dtype=4, data=P(w), nbytes=w.nbytes)
    fn = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64)(hooks.head_gemv)
    out2 = np.empty(O, np.float32)
    assert fn(C.addressof(t), P(x), P(out2), O, K) == 0
    assert np.array_equal(bits(out2), bits(out))
    lib().apus_cuda_forget(P(w))
