"""The hidden-collecting forwards (reference c/model.h:731-743), the MTP draft head
(c/mtp.h:303-357) and the speculative loop it drives (c/mtp.h:472-616) against outputs of the
unmodified reference on the small model (tests/golden/mtp_case.npz, made by
tests/golden/make_golden.py mtp)."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

import cases
from _gpu import lib
from _oracle import P
from golden.make_golden import MTP_CASE

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent
G = np.load(HERE / "golden" / "ref_cases.npz")
M = np.load(HERE / "golden" / "mtp_case.npz")


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def rope():
    return {k: (np.ascontiguousarray(G[f"rope.{k}.cos"]), np.ascontiguousarray(G[f"rope.{k}.sin"]))
            for k in ("plain", "yarn")}


@pytest.fixture
def setup():
    L = lib()
    Mdl = cases.TinyModel(MTP_CASE["seed"], rope(), MTP_CASE["n_layers"])
    Mtp = cases.TinyMtp(MTP_CASE["seed"] + 3, rope())
    prompt = np.ascontiguousarray(cases.prompt_ids(MTP_CASE["seed"] + 5, 1, MTP_CASE["n_prompt"], Mdl.M["vocab"]))
    handles = []

    def model(batch=1):
        h = L.apus_cuda_model_create(C.byref(Mdl.desc), batch, 64)
        assert h, L.apus_cuda_last_error()
        handles.append(("model", h))
        return h

    def head(h):
        mt = L.apus_cuda_mtp_create(h, C.byref(Mtp.desc))
        assert mt, L.apus_cuda_last_error()
        handles.append(("mtp", mt))
        return mt
    yield L, Mdl, Mtp, prompt, model, head
    for kind, h in reversed(handles):
        (L.apus_cuda_mtp_destroy if kind == "mtp" else L.apus_cuda_model_destroy)(h)
    L.apus_cuda_disable()


def test_forward_h_and_mh_equal_the_reference(setup):
    L, Mdl, _, prompt, model, _ = setup
    V, hd, dim, n = Mdl.M["vocab"], Mdl.M["hc"] * cases.ATTN_DIMS["dim"], cases.ATTN_DIMS["dim"], MTP_CASE["n_prompt"]
    h = model()
    lg, hh, nxt = np.empty((1, n, V), np.float32), np.empty((1, n, hd), np.float32), np.empty((1, n), np.int32)
    assert L.apus_cuda_model_forward_h(h, P(prompt), n, P(lg), 1, P(nxt), P(hh)) == 0, L.apus_cuda_last_error()
    assert np.array_equal(bits(hh[0]), bits(M["h_all"]))                    # hidden after the last block, every position
    assert np.array_equal(bits(lg[0]), bits(M["logits_all"]))
    assert nxt[0].tolist() == np.argmax(M["logits_all"], axis=1).tolist()
    assert L.apus_cuda_model_pos(h) == n
    # last-position form
    assert L.apus_cuda_model_reset(h) == 0
    lg1, n1 = np.empty((1, V), np.float32), np.empty(1, np.int32)
    assert L.apus_cuda_model_forward_h(h, P(prompt), n, P(lg1), 0, P(n1), P(hh)) == 0
    assert np.array_equal(bits(lg1[0]), bits(M["logits_all"][-1])) and np.array_equal(bits(hh[0]), bits(M["h_all"]))
    # mean hidden after the target layers
    assert L.apus_cuda_model_reset(h) == 0
    tg = np.array(MTP_CASE["targets"], np.int32)
    mh = np.empty((1, n, len(tg) * dim), np.float32)
    assert L.apus_cuda_model_forward_mh(h, P(prompt), n, None, 0, None, P(tg), len(tg), P(mh)) == 0, L.apus_cuda_last_error()
    assert np.array_equal(bits(mh[0]), bits(M["mh_all"]))
    one, bad = prompt[:, :1].copy(), np.array([7], np.int32)
    assert L.apus_cuda_model_forward_mh(h, P(one), 1, None, 0, None, P(bad), 1, P(mh)) != 0
    assert b"target layer" in L.apus_cuda_last_error()


def test_forward_h_batch_rows_are_the_single_sequences(setup):
    L, Mdl, _, _, model, _ = setup
    V, hd, n, B = Mdl.M["vocab"], Mdl.M["hc"] * cases.ATTN_DIMS["dim"], 11, 3
    ids = cases.prompt_ids(44, B, n, V)
    hb = model(B)
    lg, hh = np.empty((B, n, V), np.float32), np.empty((B, n, hd), np.float32)
    assert L.apus_cuda_model_forward_h(hb, P(ids), n, P(lg), 1, None, P(hh)) == 0, L.apus_cuda_last_error()
    h1 = model(1)
    for b in range(B):
        assert L.apus_cuda_model_reset(h1) == 0
        l1, x1 = np.empty((1, n, V), np.float32), np.empty((1, n, hd), np.float32)
        row = np.ascontiguousarray(ids[b:b + 1])
        assert L.apus_cuda_model_forward_h(h1, P(row), n, P(l1), 1, None, P(x1)) == 0
        assert np.array_equal(bits(l1[0]), bits(lg[b])) and np.array_equal(bits(x1[0]), bits(hh[b]))


def test_mtp_head_equals_the_reference(setup):
    """The head over the prompt's true (hidden, token) pairs in one pass, then one chained position
    fed its own hidden and its own pick."""
    L, Mdl, _, prompt, model, head = setup
    V, hd, n = Mdl.M["vocab"], Mdl.M["hc"] * cases.ATTN_DIMS["dim"], MTP_CASE["n_prompt"]
    h = model()
    mt = head(h)
    h_all = np.ascontiguousarray(M["h_all"].reshape(1, n, hd))
    lg, nxt, hl = np.empty((1, V), np.float32), np.empty(1, np.int32), np.empty((1, hd), np.float32)
    assert L.apus_cuda_mtp_forward(mt, P(h_all), P(prompt), n, 0, P(lg), P(nxt), P(hl)) == 0, L.apus_cuda_last_error()
    print("mtp logits rel-L2", rel_l2(lg[0], M["mtp_logits"]), "hidden", rel_l2(hl[0], M["mtp_h_last"]))
    assert np.array_equal(bits(hl[0]), bits(M["mtp_h_last"]))
    assert np.array_equal(bits(lg[0]), bits(M["mtp_logits"]))
    assert nxt[0] == int(np.argmax(M["mtp_logits"]))
    d1 = np.array([[nxt[0]]], np.int64)
    assert L.apus_cuda_mtp_forward(mt, P(hl), P(d1), 1, n, P(lg), P(nxt), P(hl)) == 0, L.apus_cuda_last_error()
    assert np.array_equal(bits(hl[0]), bits(M["mtp_h_chained"])) and np.array_equal(bits(lg[0]), bits(M["mtp_logits_chained"]))
    # the same pairs position by position leave the same head
    assert L.apus_cuda_mtp_reset(mt) == 0
    for t in range(n):
        h_t, id_t = h_all[:, t:t + 1].copy(), prompt[:, t:t + 1].copy()
        assert L.apus_cuda_mtp_forward(mt, P(h_t), P(id_t), 1, t, P(lg), None, P(hl)) == 0
    assert np.array_equal(bits(hl[0]), bits(M["mtp_h_last"])) and np.array_equal(bits(lg[0]), bits(M["mtp_logits"]))


def test_speculative_loop_with_the_mtp_head(setup):
    """Tokens: the reference's speculative stream, which is its plain greedy stream; counters: the
    reference's (batches, batch tokens, re-fed tokens, offered, accepted, d1 offered / hits)."""
    L, Mdl, _, prompt, model, head = setup
    n, n_gen, depth = MTP_CASE["n_prompt"], MTP_CASE["n_gen"], MTP_CASE["depth"]
    h = model()
    mt = head(h)
    toks, stats = np.zeros(n_gen, np.int32), np.zeros(8, np.uint64)
    rc = L.apus_cuda_model_spec_generate_mtp(h, mt, P(prompt), n, n_gen, depth, P(toks), P(stats))
    assert rc == 0, L.apus_cuda_last_error()
    assert toks.tolist() == M["spec_tokens"].tolist()
    assert stats[1:].tolist() == M["spec_stats"][1:].tolist(), (stats, M["spec_stats"])
    plain = np.zeros((1, n_gen), np.int32)
    assert L.apus_cuda_model_reset(h) == 0
    assert L.apus_cuda_model_generate(h, P(prompt), n, n_gen, P(plain), None, None) == 0
    assert plain[0].tolist() == toks.tolist()
    # a second run on the same objects reproduces the first
    assert L.apus_cuda_model_reset(h) == 0
    toks2 = np.zeros(n_gen, np.int32)
    assert L.apus_cuda_model_spec_generate_mtp(h, mt, P(prompt), n, n_gen, depth, P(toks2), None) == 0
    assert toks2.tolist() == toks.tolist()


def test_mtp_head_loaded_from_a_checkpoint_directory(tmp_path):
    """The head written as "mtp.0.*" tensors beside the model (reference c/mtp.h:213-281) and read back by
    apus_cuda_mtp_load: the same logits and hidden, bit for bit, as the head handed over in memory."""
    import ckpt_util
    L = lib()
    Mdl = cases.TinyModel(MTP_CASE["seed"], rope(), MTP_CASE["n_layers"])
    Mtp = cases.TinyMtp(MTP_CASE["seed"] + 3, rope())
    ckpt_util.write_checkpoint(tmp_path, Mdl, seed=3, mtp=Mtp)         # also rewrites every wo_a as a loader derives it
    V, hd, n = Mdl.M["vocab"], Mdl.M["hc"] * cases.ATTN_DIMS["dim"], MTP_CASE["n_prompt"]
    prompt = np.ascontiguousarray(cases.prompt_ids(MTP_CASE["seed"] + 5, 1, n, V))
    h_mem = L.apus_cuda_model_create(C.byref(Mdl.desc), 1, 64)
    h_dir = L.apus_cuda_model_load(str(tmp_path).encode(), 1, 64, 0, -1)
    assert h_mem and h_dir, L.apus_cuda_last_error()
    mt_mem = L.apus_cuda_mtp_create(h_mem, C.byref(Mtp.desc))
    mt_dir = L.apus_cuda_mtp_load(h_dir, str(tmp_path).encode(), 0)
    assert mt_mem and mt_dir, L.apus_cuda_last_error()
    try:
        outs = []
        for h, mt in ((h_mem, mt_mem), (h_dir, mt_dir)):
            hh, lg, hl = np.empty((1, n, hd), np.float32), np.empty((1, V), np.float32), np.empty((1, hd), np.float32)
            assert L.apus_cuda_model_forward_h(h, P(prompt), n, P(lg), 0, None, P(hh)) == 0, L.apus_cuda_last_error()
            assert L.apus_cuda_mtp_forward(mt, P(hh), P(prompt), n, 0, P(lg), None, P(hl)) == 0, L.apus_cuda_last_error()
            outs.append((hh, lg, hl))
        for a, b in zip(outs[0], outs[1]):
            assert np.array_equal(bits(a), bits(b))
        assert not L.apus_cuda_mtp_load(h_dir, str(tmp_path).encode(), 1)
        assert b"no MTP block 1" in L.apus_cuda_last_error()
    finally:
        L.apus_cuda_mtp_destroy(mt_mem); L.apus_cuda_mtp_destroy(mt_dir)
        L.apus_cuda_model_destroy(h_mem); L.apus_cuda_model_destroy(h_dir)
        L.apus_cuda_disable()
