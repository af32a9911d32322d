"""The NDJSON serve loop (reference c/apus.c:451-662) on file descriptors, against the
token loop it wraps and the reference's committed greedy / sampled continuations."""
import ctypes as C
import json
import os
from pathlib import Path

import numpy as np
import pytest

import cases
from _gpu import lib
from _oracle import P
from golden.make_golden import MODEL_CASES, MODEL_SAMPLED_CASES

pytestmark = pytest.mark.gpu
G = np.load(Path(__file__).resolve().parent / "golden" / "ref_cases.npz")


def rope():
    return {k: (np.ascontiguousarray(G[f"rope.{k}.cos"]), np.ascontiguousarray(G[f"rope.{k}.sin"]))
            for k in ("plain", "yarn")}


def serve(L, h, requests, tmp_path, eos=-1):
    inp, out = tmp_path / "in.ndjson", tmp_path / "out.ndjson"
    inp.write_text("".join(r if isinstance(r, str) else json.dumps(r) + "\n" for r in requests))
    fi, fo = os.open(inp, os.O_RDONLY), os.open(out, os.O_WRONLY | os.O_CREAT | os.O_TRUNC)
    try:
        assert L.apus_cuda_serve(h, fi, fo, eos) == 0, L.apus_cuda_last_error()
    finally:
        os.close(fi); os.close(fo)
    return [json.loads(l) for l in out.read_text().splitlines()]


def test_serve_loop(tmp_path):
    L = lib()
    seed, n_layers, B, n_prompt, n_gen = MODEL_CASES["model_one"]
    Mdl = cases.TinyModel(seed, rope(), n_layers)
    prompt = cases.prompt_ids(seed + 5, B, n_prompt, Mdl.M["vocab"])
    h = L.apus_cuda_model_create(C.byref(Mdl.desc), 1, 64)
    assert h, L.apus_cuda_last_error()
    try:
        want = np.zeros((1, n_gen), np.int32)
        assert L.apus_cuda_model_generate(h, P(prompt), n_prompt, n_gen, P(want), None, None) == 0
        assert want[0, :8].tolist() == G["model_one.tokens"][0, :8].tolist()     # the reference's own stream
        ids = [int(t) for t in prompt[0]]
        reqs = [
            {"id": 1, "cmd": "generate", "ids": ids, "max_tokens": n_gen, "temperature": 0},
            "this is not json\n",
            {"id": "two", "cmd": "nothing"},
            {"id": 3, "cmd": "generate", "text": "hello"},
            {"id": 4, "cmd": "generate", "ids": []},
            {"id": 5, "cmd": "generate", "ids": [1] * 64},
            {"id": [6, {"k": "v\"q"}], "cmd": "generate", "ids": ids, "max_tokens": 5, "temperature": 0},
            {"id": 7, "cmd": "encode", "text": "x"},
            {"id": 8, "cmd": "generate", "ids": ids, "max_tokens": 1000, "temperature": 0},
            {"id": 10, "cmd": "generate", "ids": [Mdl.M["vocab"]]},
        ]
        out = serve(L, h, reqs, tmp_path)
        by = lambda i: [o for o in out if o["id"] == i]
        r1 = by(1)
        assert r1[0] == {"id": 1, "type": "prompt", "prompt_tokens": n_prompt}
        assert [o["token_id"] for o in r1 if o["type"] == "token"] == want[0].tolist()
        assert r1[-1] == {"id": 1, "type": "done", "finish_reason": "length", "prompt_tokens": n_prompt,
                          "completion_tokens": n_gen, "text": ""}
        assert {"id": None, "type": "error", "message": "bad request line (not a JSON object)"} in out
        assert by("two") == [{"id": "two", "type": "error", "message": "unknown cmd (want encode|generate)"}]
        assert by(3)[0]["message"] == "no tokenizer in model dir" and by(7)[0]["message"] == "no tokenizer in model dir"
        assert by(4)[0]["message"] == "empty prompt"
        assert by(5)[0]["message"] == "prompt too long for model max_pos"
        r6 = by([6, {"k": "v\"q"}])                      # any JSON value is echoed as the id
        assert [o["token_id"] for o in r6 if o["type"] == "token"] == want[0, :5].tolist()
        r8 = by(8)                                        # the completion is cut to the position table
        assert r8[-1]["completion_tokens"] == 64 - n_prompt and r8[-1]["finish_reason"] == "length"
        assert by(10)[-1]["type"] == "error" and "outside [0," in by(10)[-1]["message"]   # refused on the host
        # the end-of-sequence token ends the completion and is not emitted
        eos = int(want[0, 3])
        first = want[0].tolist().index(eos)
        out = serve(L, h, [{"id": 9, "cmd": "generate", "ids": ids, "max_tokens": n_gen, "temperature": 0}], tmp_path, eos=eos)
        assert [o["token_id"] for o in out if o["type"] == "token"] == want[0, :first].tolist()
        assert out[-1]["finish_reason"] == "stop" and out[-1]["completion_tokens"] == first
    finally:
        L.apus_cuda_model_destroy(h)
        L.apus_cuda_disable()


def test_serve_sampled_equals_the_reference_stream(tmp_path):
    """temperature / top_p / seed of a request drive the device sampler: the tokens of the
    reference's sampled continuation (its own loop, same seed)."""
    L = lib()
    seed, n_layers, B, n_prompt, n_gen, temp, top_p, rng_seed = MODEL_SAMPLED_CASES["model_sampled"]
    Mdl = cases.TinyModel(seed, rope(), n_layers)
    prompt = cases.prompt_ids(seed + 5, B, n_prompt, Mdl.M["vocab"])
    h = L.apus_cuda_model_create(C.byref(Mdl.desc), 1, 64)
    assert h, L.apus_cuda_last_error()
    try:
        out = serve(L, h, [{"id": 0, "cmd": "generate", "ids": [int(t) for t in prompt[0]], "max_tokens": n_gen,
                            "temperature": temp, "top_p": top_p, "seed": rng_seed}], tmp_path)
        got = [o["token_id"] for o in out if o["type"] == "token"]
        want = G["model_sampled.tokens"][0].tolist()
        agree = next((i for i, (a, b) in enumerate(zip(got, want)) if a != b), len(want))
        print("sampled stream equal to the reference's for", agree, "of", len(want), "tokens")
        assert agree >= 8
    finally:
        L.apus_cuda_model_destroy(h)
        L.apus_cuda_disable()
