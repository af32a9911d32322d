"""Chunks of positions (batched prefill and mid-stream batches; reference c/attn.h:1576-1680,
c/model.h:651-720) against one step per position: the reference defines the two to be equal
(tests/m4c chunk invariance), and here they are compared bit for bit -- logits, the tokens
decoded afterwards, the attention state -- on the small committed cases and on the benchmarked
model's first six layers at their real dimensions, in both sum orders."""
import ctypes as C
import time
from pathlib import Path

import numpy as np
import pytest

import cases
import flash_case
from _gpu import lib
from _oracle import P

pytestmark = pytest.mark.gpu
G = np.load(Path(__file__).resolve().parent / "golden" / "ref_cases.npz")
GOLD = Path(__file__).resolve().parent / "golden" / "flash_case.npz"
ORDERS = ["reference", "default"]


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def rope():
    return {k: (np.ascontiguousarray(G[f"rope.{k}.cos"]), np.ascontiguousarray(G[f"rope.{k}.sin"]))
            for k in ("plain", "yarn")}


def state_of(A, S):
    """Everything apus_cuda_attention leaves behind (reference c/attn.h:147-160)."""
    out = {"win": S.win.copy()}
    if A.ratio:
        out.update(comp_kv=S.comp[0].copy(), comp_sc=S.comp[1].copy(), comp_cache=S.comp[2].copy(),
                   comp_nb=np.array([S.st.comp.nb]))
        if A.kind == "csa":
            out.update(idx_kv=S.idx[0].copy(), idx_sc=S.idx[1].copy(), idx_cache=S.idx[2].copy(),
                       idx_nb=np.array([S.st.idx_comp.nb]))
    return out


@pytest.fixture
def sum_order(request):
    L = lib()
    old = L.apus_cuda_set_tree_ops(-1)
    L.apus_cuda_set_tree_ops(0 if request.param == "reference" else L.apus_cuda_set_tree_ops(-2))
    yield request.param
    L.apus_cuda_set_tree_ops(old)


@pytest.fixture
def chunk_rows():
    L = lib()
    old = L.apus_cuda_set_prefill_chunk(-1)
    yield lambda rows: L.apus_cuda_set_prefill_chunk(rows)
    L.apus_cuda_set_prefill_chunk(old)


@pytest.mark.parametrize("sum_order", ORDERS, indirect=True)
@pytest.mark.parametrize("kind", ["swa", "csa", "hca"])
def test_attention_chunks_equal_steps(kind, sum_order, chunk_rows):
    """apus_cuda_attention over 41 positions in one pass, as 1-position calls and as uneven pieces
    (a piece that starts mid-stream reads the ring and the carries the one before left): outputs,
    ring, compressed caches, carries and entry counts equal bit for bit."""
    L = lib()
    cos, sin = rope()["plain" if kind == "swa" else "yarn"]
    total = 41

    def run(parts, rows):
        chunk_rows(rows)
        A = cases.AttnLayer(7, kind)
        S = cases.AttnState(A)
        x = cases.attn_inputs(11, total, A.D["dim"])
        out = np.zeros_like(x)
        pos = 0
        for n in parts:
            rc = L.apus_cuda_attention(C.byref(A.cfg), C.byref(A.w), C.byref(S.st), P(x[pos:pos + n]), n, pos, P(cos), P(sin),
                                       P(out[pos:pos + n]), None)
            assert rc == 0, L.apus_cuda_last_error()
            pos += n
        L.apus_cuda_disable()
        return out, state_of(A, S)

    ref_out, ref_state = run([1] * total, 0)
    for parts in ([total], [5, 1, 17, 2, 16], [40, 1]):
        out, state = run(parts, 2048)
        assert np.array_equal(bits(out), bits(ref_out)), (kind, parts)
        for k in ref_state:
            assert np.array_equal(np.asarray(state[k]).view(np.uint8), np.asarray(ref_state[k]).view(np.uint8)), (kind, parts, k)


@pytest.mark.parametrize("sum_order", ORDERS, indirect=True)
def test_model_chunks_equal_steps(sum_order, chunk_rows):
    """A 3-sequence prompt of 37 tokens through the small model: as steps, as one chunk, as chunks
    of 7 and of 2 positions; then a 5-position mid-stream call and 8 greedy steps.  Logits and
    tokens equal bit for bit."""
    L = lib()
    Mdl = cases.TinyModel(91, rope(), 4)
    B, n_prompt, n_mid, n_gen = 3, 37, 5, 8
    V = Mdl.M["vocab"]
    prompts = cases.prompt_ids(17, B, n_prompt, V)
    mid = cases.prompt_ids(18, B, n_mid, V)

    def run(rows, keep=None):
        chunk_rows(rows)
        h = keep or L.apus_cuda_model_create(C.byref(Mdl.desc), B, 64)
        assert h, L.apus_cuda_last_error()
        try:
            assert L.apus_cuda_model_reset(h) == 0
            lg1, lg2 = np.empty((B, V), np.float32), np.empty((B, V), np.float32)
            nxt = np.empty(B, np.int32)
            assert L.apus_cuda_model_forward(h, P(prompts), n_prompt, P(lg1), None) == 0, L.apus_cuda_last_error()
            assert L.apus_cuda_model_forward(h, P(mid), n_mid, P(lg2), P(nxt)) == 0, L.apus_cuda_last_error()
            assert L.apus_cuda_model_pos(h) == n_prompt + n_mid
            toks = [nxt.copy()]
            for _ in range(n_gen):
                feed = np.ascontiguousarray(toks[-1].astype(np.int64).reshape(B, 1))
                assert L.apus_cuda_model_forward(h, P(feed), 1, None, P(nxt)) == 0, L.apus_cuda_last_error()
                toks.append(nxt.copy())
            # generate() consumes its prompt the same way
            assert L.apus_cuda_model_reset(h) == 0
            gen = np.empty((B, n_gen), np.int32)
            assert L.apus_cuda_model_generate(h, P(prompts), n_prompt, n_gen, P(gen), None, None) == 0
        finally:
            if not keep:
                L.apus_cuda_model_destroy(h)
        return lg1, lg2, np.stack(toks), gen

    want = run(0)
    # one model through steps (its decode step gets recorded), a chunk (workspaces grow and move: the
    # recorded step must be taken again), steps
    h = L.apus_cuda_model_create(C.byref(Mdl.desc), B, 64)
    try:
        for rows in (0, 2048, 0):
            got = run(rows, keep=h)
            assert np.array_equal(bits(got[1]), bits(want[1])) and np.array_equal(got[2], want[2]) and np.array_equal(got[3], want[3])
    finally:
        L.apus_cuda_model_destroy(h)
    for rows in (2048, 7 * B, 2 * B):
        got = run(rows)
        assert np.array_equal(bits(got[0]), bits(want[0])), rows
        assert np.array_equal(bits(got[1]), bits(want[1])), rows
        assert np.array_equal(got[2], want[2]) and np.array_equal(got[3], want[3]), rows
    L.apus_cuda_disable()


@pytest.mark.parametrize("sum_order", ORDERS, indirect=True)
def test_six_real_layers_prompt_in_chunks_equals_steps(sum_order, chunk_rows):
    """The benchmarked model's first six layers (all three layer kinds, hash and scored routing, 256
    experts, vocabulary 129,280): a 100-token prompt of 4 sequences as steps, as one 400-row chunk
    and as 48-row chunks; last-position logits and 16 greedy tokens equal bit for bit."""
    if not GOLD.exists():
        pytest.skip("tests/golden/flash_case.npz is not present")
    import torch
    from apus_b200.flash import RandomFlashModel
    L = lib()
    gold = np.load(GOLD)
    cfg = flash_case.config(6)
    W = RandomFlashModel(cfg, flash_case.CASE["seed"], torch.device("cuda", 0), max_pos=flash_case.CASE["max_pos"],
                         rope=flash_case.rope_from(gold))
    B, n_prompt, n_gen = 4, flash_case.CASE["n_prompt"], 16
    ids = np.ascontiguousarray(flash_case.prompts(cfg, B, n_prompt))
    h = L.apus_cuda_model_create(C.byref(W.desc), B, flash_case.CASE["max_pos"])
    assert h, L.apus_cuda_last_error()
    res, ms = {}, {}
    try:
        for rows in (0, 2048, 48):
            chunk_rows(rows)
            assert L.apus_cuda_model_reset(h) == 0
            lg = np.empty((B, cfg.vocab), np.float32)
            t0 = time.perf_counter()
            assert L.apus_cuda_model_forward(h, P(ids), n_prompt, P(lg), None) == 0, L.apus_cuda_last_error()
            ms[rows] = (time.perf_counter() - t0) * 1e3
            assert L.apus_cuda_model_reset(h) == 0
            toks = np.zeros((B, n_gen), np.int32)
            assert L.apus_cuda_model_generate(h, P(ids), n_prompt, n_gen, P(toks), None, None) == 0, L.apus_cuda_last_error()
            res[rows] = (lg, toks)
    finally:
        L.apus_cuda_model_destroy(h)
        L.apus_cuda_disable()
    print(sum_order, "prompt of", n_prompt, "x", B, "ms (host clock): steps %.0f, one chunk %.0f, 48-row chunks %.0f" % (ms[0], ms[2048], ms[48]))
    for rows in (2048, 48):
        assert np.array_equal(bits(res[rows][0]), bits(res[0][0])), rows
        assert np.array_equal(res[rows][1], res[0][1]), rows
