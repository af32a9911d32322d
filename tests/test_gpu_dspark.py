"""The DSpark draft module (reference c/dspark.h) against outputs of the unmodified reference on the small
model (tests/golden/dspark_case.npz, made by tests/golden/make_golden.py dspark): stage rings from the
prompt's main hiddens, one draft round, the speculative loop."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

import cases
from _gpu import lib
from _oracle import P
from golden.make_golden import DSPARK_CASE as D

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent
G = np.load(HERE / "golden" / "ref_cases.npz")
R = np.load(HERE / "golden" / "dspark_case.npz")


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def rope():
    return {k: (np.ascontiguousarray(G[f"rope.{k}.cos"]), np.ascontiguousarray(G[f"rope.{k}.sin"]))
            for k in ("plain", "yarn")}


@pytest.fixture
def setup():
    L = lib()
    Mdl = cases.TinyModel(D["seed"], rope(), D["n_layers"])
    Ds = cases.TinyDspark(D["seed"] + 4, rope(), D["targets"], D["n_stages"], D["block_size"], D["noise_id"], D["rank"])
    prompt = np.ascontiguousarray(cases.prompt_ids(D["seed"] + 5, 1, D["n_prompt"], Mdl.M["vocab"]))
    h = L.apus_cuda_model_create(C.byref(Mdl.desc), 1, 64)
    assert h, L.apus_cuda_last_error()
    ds = L.apus_cuda_dspark_create(h, C.byref(Ds.desc))
    assert ds, L.apus_cuda_last_error()
    yield L, Mdl, Ds, prompt, h, ds
    L.apus_cuda_dspark_destroy(ds)
    L.apus_cuda_model_destroy(h)
    L.apus_cuda_disable()


def one_round(L, Mdl, ds, pieces):
    """Stage rings fed in `pieces`, then the draft round after the last prompt position."""
    V, hd, B, n = Mdl.M["vocab"], Mdl.M["hc"] * cases.ATTN_DIMS["dim"], D["block_size"], D["n_prompt"]
    mh = np.ascontiguousarray(R["mh_all"])
    assert L.apus_cuda_dspark_reset(ds) == 0
    pos = 0
    for k in pieces:
        part = np.ascontiguousarray(mh[pos:pos + k])
        assert L.apus_cuda_dspark_feed(ds, P(part), pos, k) == 0, L.apus_cuda_last_error()
        pos += k
    drafts, conf = np.zeros(B, np.int64), np.zeros(B, np.float32)
    lf, sh = np.zeros((B, V), np.float32), np.zeros((D["n_stages"], B, hd), np.float32)
    last = np.ascontiguousarray(mh[n - 1])
    rc = L.apus_cuda_dspark_draft_round(ds, int(R["anchor"][0]), P(last), n - 1, P(drafts), P(conf), P(lf), P(sh))
    assert rc == 0, L.apus_cuda_last_error()
    return drafts, conf, lf, sh


def test_draft_round_equals_the_reference(setup):
    L, Mdl, _, _, _, ds = setup
    n = D["n_prompt"]
    for pieces in ([n], [6, n - 6], [1] * n):             # whole prompt / prefill + catch-up / position by position
        drafts, conf, lf, sh = one_round(L, Mdl, ds, pieces)
        for k in range(D["n_stages"]):
            assert np.array_equal(bits(sh[k]), bits(R["stage_h"][k])), (pieces, k)
        assert np.array_equal(bits(lf), bits(R["logits_final"])), pieces
        assert drafts.tolist() == R["drafts"].tolist(), pieces
        assert np.array_equal(bits(conf), bits(R["confidence"])), (pieces, conf, R["confidence"])


def test_speculative_loop_with_dspark(setup):
    """Tokens: the reference's speculative stream = its plain greedy stream; counters: the reference's."""
    L, _, _, prompt, h, ds = setup
    n, n_gen = D["n_prompt"], D["n_gen"]
    toks, stats = np.zeros(n_gen, np.int32), np.zeros(7, np.uint64)
    rc = L.apus_cuda_model_spec_generate_dspark(h, ds, P(prompt), n, n_gen, P(toks), P(stats))
    assert rc == 0, L.apus_cuda_last_error()
    assert toks.tolist() == R["spec_tokens"].tolist()
    assert stats[1:].tolist() == R["spec_stats"][1:].tolist(), (stats, R["spec_stats"])
    plain = np.zeros((1, n_gen), np.int32)
    assert L.apus_cuda_model_reset(h) == 0
    assert L.apus_cuda_model_generate(h, P(prompt), n, n_gen, P(plain), None, None) == 0
    assert plain[0].tolist() == toks.tolist()
    assert L.apus_cuda_model_reset(h) == 0
    toks2 = np.zeros(n_gen, np.int32)
    assert L.apus_cuda_model_spec_generate_dspark(h, ds, P(prompt), n, n_gen, P(toks2), None) == 0
    assert toks2.tolist() == toks.tolist()


def test_sampled_drafts_and_sampled_loop(setup):
    """Draft picks drawn at a temperature from the module's own generator stream (c/dspark.h:666-676): the
    drafts of a round and the final logits behind them (every row's bigram bias follows the token drawn for
    the row before) equal apus_dspark_draft_round with the same seed; the loop with a sampled main stream and
    sampled drafts emits the reference's tokens and counters, which are those of plain sampled decoding."""
    L, Mdl, _, prompt, h, ds = setup
    n, n_gen = D["n_prompt"], D["n_gen"]
    assert L.apus_cuda_dspark_set_sampling(ds, D["temp"], D["draft_seed"]) == 0, L.apus_cuda_last_error()
    drafts, _, lf, _ = one_round(L, Mdl, ds, [n])
    assert drafts.tolist() == R["drafts_sampled"].tolist()
    assert np.array_equal(bits(lf), bits(R["logits_final_sampled"]))
    assert drafts.tolist() != R["drafts"].tolist()                      # the case does tell greedy from sampled
    # the loop: both streams seeded as apus_dspec_init seeds them
    assert L.apus_cuda_model_reset(h) == 0
    assert L.apus_cuda_model_set_sampling(h, D["temp"], D["top_p"], D["rng_seed"]) == 0
    assert L.apus_cuda_dspark_set_sampling(ds, D["temp"], D["draft_seed"]) == 0
    toks, stats = np.zeros(n_gen, np.int32), np.zeros(7, np.uint64)
    rc = L.apus_cuda_model_spec_generate_dspark(h, ds, P(prompt), n, n_gen, P(toks), P(stats))
    assert rc == 0, L.apus_cuda_last_error()
    assert toks.tolist() == R["spec_sampled_tokens"].tolist()
    assert stats[1:].tolist() == R["spec_sampled_stats"][1:].tolist(), (stats, R["spec_sampled_stats"])
    plain = np.zeros((1, n_gen), np.int32)
    assert L.apus_cuda_model_reset(h) == 0
    assert L.apus_cuda_model_set_sampling(h, D["temp"], D["top_p"], D["rng_seed"]) == 0
    assert L.apus_cuda_model_generate(h, P(prompt), n, n_gen, P(plain), None, None) == 0
    assert plain[0].tolist() == toks.tolist()
    # back to greedy drafts: the round of the greedy case again
    assert L.apus_cuda_dspark_set_sampling(ds, 0.0, 0) == 0
    assert one_round(L, Mdl, ds, [n])[0].tolist() == R["drafts"].tolist()


def test_dspark_loaded_from_a_checkpoint_directory(tmp_path):
    """The module written as "mtp.<k>.*" tensors with its config section (reference c/dspark.h:272-341,
    c/model.h:336-373) and read back by apus_cuda_dspark_load: the draft round of the in-memory module."""
    import ckpt_util
    L = lib()
    Mdl = cases.TinyModel(D["seed"], rope(), D["n_layers"])
    Ds = cases.TinyDspark(D["seed"] + 4, rope(), D["targets"], D["n_stages"], D["block_size"], D["noise_id"], D["rank"])
    ckpt_util.write_checkpoint(tmp_path, Mdl, seed=3, dspark=Ds)
    h_mem = L.apus_cuda_model_create(C.byref(Mdl.desc), 1, 64)
    h_dir = L.apus_cuda_model_load(str(tmp_path).encode(), 1, 64, 0, -1)
    assert h_mem and h_dir, L.apus_cuda_last_error()
    ds_mem = L.apus_cuda_dspark_create(h_mem, C.byref(Ds.desc))
    ds_dir = L.apus_cuda_dspark_load(h_dir, str(tmp_path).encode())
    assert ds_mem and ds_dir, L.apus_cuda_last_error()
    try:
        a = one_round(L, Mdl, ds_mem, [D["n_prompt"]])
        b = one_round(L, Mdl, ds_dir, [D["n_prompt"]])
        assert a[0].tolist() == b[0].tolist()
        for x, y in zip(a[1:], b[1:]):
            assert np.array_equal(bits(x), bits(y))
    finally:
        L.apus_cuda_dspark_destroy(ds_mem); L.apus_cuda_dspark_destroy(ds_dir)
        L.apus_cuda_model_destroy(h_mem); L.apus_cuda_model_destroy(h_dir)
        L.apus_cuda_disable()
