"""The checkpoint reader (host code, no GPU): config parsing, safetensors shards,
conversions and rope tables against what was written and against what the
reference's own loader made of the same directory (tests/golden/ckpt_case.npz,
written by tests/golden/make_golden.py through apus_model_load); error messages
for the malformed inputs the reference's tests cover (tests/m1).  The GPU half
(apus_cuda_model_load) is in tests/test_gpu_model.py.
"""
import ctypes as C
import json
import shutil
import struct
from pathlib import Path

import numpy as np
import pytest

import cases
import ckpt_util
from apus_b200 import capi
from golden.make_golden import CKPT_CASE

GOLD = Path(__file__).resolve().parent / "golden"
K = np.load(GOLD / "ckpt_case.npz")
R = np.load(GOLD / "ref_cases.npz")
P = capi.ptr
_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = capi.load()
    return _lib


def rope_pair():
    return {n: (R[f"rope.{n}.cos"], R[f"rope.{n}.sin"]) for n in ("plain", "yarn")}


def open_ckpt(path):
    err = C.create_string_buffer(512)
    return lib().apus_cuda_ckpt_open(str(path).encode(), err, 512), err.value.decode()


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    d = tmp_path_factory.mktemp("ckpt")
    tm = cases.TinyModel(CKPT_CASE["seed"], rope_pair(), CKPT_CASE["n_layers"])
    written = ckpt_util.write_checkpoint(d, tm, seed=CKPT_CASE["seed"])
    h, err = open_ckpt(d)
    assert h, err
    yield dict(dir=d, tm=tm, written=written, h=h)
    lib().apus_cuda_ckpt_close(h)


def test_config_equals_the_reference_parse(ckpt):
    cfg = lib().apus_cuda_ckpt_cfg(ckpt["h"]).contents
    assert bytes(cfg) == K["cfg"].tobytes()                       # every field, bit for bit
    assert cfg.n_layers == 3 and cfg.vocab_size == 384 and cfg.rope_factor == 16.0
    for i in range(cfg.n_layers):
        r, h = C.c_int(), C.c_int()
        assert lib().apus_cuda_ckpt_layer_kind(ckpt["h"], i, C.byref(r), C.byref(h)) == 0
        assert (r.value, h.value) == (int(K["ratios"][i]), int(K["hash"][i]))
    assert lib().apus_cuda_ckpt_layer_kind(ckpt["h"], 3, None, None) == 1


def test_every_tensor_reads_back(ckpt):
    h = ckpt["h"]
    for name, (dtype, shape, payload) in ckpt["written"].items():
        dt, nd, nb = C.c_int(), C.c_int(), C.c_uint64()
        sh = (C.c_int64 * 8)()
        assert lib().apus_cuda_ckpt_tensor(h, name.encode(), C.byref(dt), C.byref(nd), sh, C.byref(nb)) == 0
        assert capi.ST_DTYPES[dt.value] == dtype and tuple(sh[: nd.value]) == shape and nb.value == len(payload)
        buf = np.empty(len(payload), np.uint8)
        assert lib().apus_cuda_ckpt_read(h, name.encode(), P(buf), buf.size) == 0
        assert buf.tobytes() == payload
        if dtype in ("BF16", "F32"):
            n = int(np.prod(shape))
            out = np.empty(n, np.float32)
            assert lib().apus_cuda_ckpt_read_f32(h, name.encode(), P(out), n) == 0
            want = np.frombuffer(payload, np.float32) if dtype == "F32" else \
                (np.frombuffer(payload, np.uint16).astype(np.uint32) << 16).view(np.float32)
            assert np.array_equal(out.view(np.uint32), want.view(np.uint32))
    assert lib().apus_cuda_ckpt_tensor(h, b"layers.0.nope", None, None, None, None) == 1
    assert lib().apus_cuda_ckpt_read(h, b"norm.weight", P(np.empty(4, np.uint8)), 4) == 1   # size mismatch
    assert b"norm.weight" in lib().apus_cuda_last_error()


def test_wo_a_conversion_equals_the_reference_loader(ckpt):
    tm = ckpt["tm"]
    for i, L in enumerate(tm.layers):
        out = np.zeros_like(L.attn.wo_a)
        assert lib().apus_cuda_ckpt_wo_a(ckpt["h"], i, P(out), out.size) == 0
        assert np.array_equal(out, L.attn.wo_a)                   # the numpy restatement
    out = np.zeros_like(tm.layers[0].attn.wo_a)
    lib().apus_cuda_ckpt_wo_a(ckpt["h"], 0, P(out), out.size)
    assert np.array_equal(out, K["wo_a0"])                        # apus_layer_load's own result


def test_rope_tables_equal_the_reference(ckpt):
    rows, half = cases.ATTN_DIMS["max_pos"], cases.ATTN_DIMS["rope_dim"] // 2
    for ratio, name in ((0, "plain"), (4, "yarn"), (128, "yarn")):
        cos, sin = np.empty((rows, half), np.float32), np.empty((rows, half), np.float32)
        assert lib().apus_cuda_ckpt_rope(ckpt["h"], ratio, rows, P(cos), P(sin)) == 0
        # the tables are host-libm cosf/sinf values on both sides: identical on one libc
        assert np.array_equal(cos.view(np.uint32), K[f"cos_{name}"].view(np.uint32))
        assert np.array_equal(sin.view(np.uint32), K[f"sin_{name}"].view(np.uint32))
        assert np.array_equal(cos, R[f"rope.{name}.cos"]) and np.array_equal(sin, R[f"rope.{name}.sin"])


@pytest.mark.parametrize("coalesce", [True, False])
def test_expert_slab_is_one_read_when_adjacent(tmp_path, coalesce):
    tm = cases.TinyModel(5, rope_pair(), 2)
    ckpt_util.write_checkpoint(tmp_path, tm, seed=5, n_shards=1, coalesce=coalesce)
    h, err = open_ckpt(tmp_path)
    assert h, err
    Mo = tm.layers[1].moe
    slab = np.empty(Mo.expert_bytes(), np.uint8)
    w = [capi.QW() for _ in range(3)]
    assert lib().apus_cuda_ckpt_expert(h, 1, 0, P(slab), slab.size - 1, *[C.byref(q) for q in w]) == 1   # too small
    n0, b0 = lib().apus_cuda_ckpt_read_count(h), lib().apus_cuda_ckpt_read_bytes(h)
    for e in (3, 0, Mo.E - 1):
        assert lib().apus_cuda_ckpt_expert(h, 1, e, P(slab), slab.size, *[C.byref(q) for q in w]) == 0
        for q, (pk, sc, O, Kd) in zip(w, ((Mo.w1p, Mo.w1s, Mo.inter, Mo.dim), (Mo.w2p, Mo.w2s, Mo.dim, Mo.inter),
                                           (Mo.w3p, Mo.w3s, Mo.inter, Mo.dim))):
            assert (q.O, q.K) == (O, Kd)
            got_p = np.ctypeslib.as_array(C.cast(q.codes, capi.u8p), (O * Kd // 2,))
            got_s = np.ctypeslib.as_array(C.cast(q.scales, capi.u8p), (O * Kd // 32,))
            assert np.array_equal(got_p, pk[e].ravel()) and np.array_equal(got_s, sc[e].ravel())
    reads = lib().apus_cuda_ckpt_read_count(h) - n0
    assert reads == (3 if coalesce else 18)
    assert lib().apus_cuda_ckpt_read_bytes(h) - b0 == 3 * Mo.expert_bytes()
    assert lib().apus_cuda_ckpt_expert(h, 1, Mo.E, P(slab), slab.size, None, None, None) == 1
    lib().apus_cuda_ckpt_close(h)


def test_weights_subdirectory_layout(tmp_path):
    tm = cases.TinyModel(6, rope_pair(), 1)
    ckpt_util.write_checkpoint(tmp_path, tm, seed=6, n_shards=1, subdir=True)
    h, err = open_ckpt(tmp_path)
    assert h, err
    out = np.empty(cases.ATTN_DIMS["dim"], np.float32)
    assert lib().apus_cuda_ckpt_read_f32(h, b"norm.weight", P(out), out.size) == 0
    assert np.array_equal(out, tm.norm_w)
    lib().apus_cuda_ckpt_close(h)


REAL_CONFIG = {       # the keys of the real checkpoint's config.json (HF schema), toy values
    "hidden_size": 256, "num_attention_heads": 4, "head_dim": 128, "qk_rope_head_dim": 64, "q_lora_rank": 128,
    "o_groups": 2, "o_lora_rank": 128, "sliding_window": 8, "moe_intermediate_size": 128, "n_routed_experts": 8,
    "num_experts_per_tok": 2, "index_n_heads": 4, "index_head_dim": 128, "index_topk": 4, "hc_mult": 4,
    "hc_sinkhorn_iters": 20, "vocab_size": 384, "max_position_embeddings": 1048576, "hc_eps": 1e-06,
    "rms_norm_eps": 1e-06, "routed_scaling_factor": 1.5, "swiglu_limit": 10.0, "rope_theta": 10000,
    "compress_rope_theta": 160000, "bos_token_id": 0, "eos_token_id": 1, "num_hidden_layers": 5,
    "num_hash_layers": 2, "num_nextn_predict_layers": 1, "compress_ratios": [0, 0, 4, 128, 4, 0],
    "rope_scaling": {"beta_fast": 32, "beta_slow": 1, "factor": 16, "original_max_position_embeddings": 65536,
                     "type": "yarn"},
}


def write_cfg_only(d, cfg):
    (d / "config.json").write_text(json.dumps(cfg))
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {}}))


def test_real_checkpoint_config_schema(tmp_path):
    write_cfg_only(tmp_path, REAL_CONFIG)
    h, err = open_ckpt(tmp_path)
    assert h, err
    c = lib().apus_cuda_ckpt_cfg(h).contents
    assert (c.dim, c.n_heads, c.rope_head_dim, c.window_size, c.moe_inter_dim, c.n_activated_experts,
            c.max_pos, c.n_layers) == (256, 4, 64, 8, 128, 2, 1048576, 5)
    assert (c.rope_factor, c.beta_fast, c.beta_slow, c.compress_rope_theta) == (16.0, 32, 1, 160000.0)
    # the reference leaves original_seq_len at 0 when rope_scaling carries the key (it assigns only
    # when its lookup FAILS, c/model.h:254-255); parity follows the reference
    assert c.original_seq_len == 0
    assert (c.n_mtp, c.mtp_ratio, c.mtp_hash, c.dspark, c.bos_id, c.eos_id) == (1, 0, 0, 0, 0, 1)
    kinds = []
    for i in range(5):
        r, hh = C.c_int(), C.c_int()
        lib().apus_cuda_ckpt_layer_kind(h, i, C.byref(r), C.byref(hh))
        kinds.append((r.value, hh.value))
    assert kinds == [(0, 1), (0, 1), (4, 0), (128, 0), (4, 0)]
    lib().apus_cuda_ckpt_close(h)
    # DSpark keys: the trailing ratios are speculative stages, no classic MTP block (c/model.h:316-324)
    cfg = dict(REAL_CONFIG, dspark_block_size=5, dspark_noise_token_id=7, dspark_target_layer_ids=[2, 3, 4],
               dspark_markov_rank=16, compress_ratios=[0, 0, 4, 128, 4, 0, 0, 0])
    write_cfg_only(tmp_path, cfg)
    h, err = open_ckpt(tmp_path)
    assert h, err
    c = lib().apus_cuda_ckpt_cfg(h).contents
    assert (c.dspark, c.n_mtp, c.n_layers) == (1, 0, 5)
    lib().apus_cuda_ckpt_close(h)


def test_config_parse_against_the_live_reference(tmp_path):
    """Both schemas and the error strings, side by side with the reference's parser
    (skipped where the reference build is absent)."""
    from _oracle import ref
    L = ref()
    if L is None or not hasattr(L, "ref_parse_config"):
        pytest.skip("reference build not present")
    L.ref_parse_config.restype = C.c_int
    L.ref_parse_config.argtypes = [C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_char_p, C.c_size_t]
    variants = [dict(REAL_CONFIG)]
    v = dict(REAL_CONFIG); v["rope_scaling"] = {"factor": 8, "beta_fast": 16}; variants.append(v)
    v = dict(REAL_CONFIG); v.pop("rope_scaling"); v.update(original_seq_len=4096, rope_factor=4, beta_fast=8, beta_slow=2)
    variants.append(v)
    v = dict(REAL_CONFIG, dspark_block_size=5, compress_ratios=[0, 0, 4, 128, 4, 0, 0, 0]); variants.append(v)
    v = dict(v, dspark_noise_token_id=7, dspark_target_layer_ids=[2, 3, 4], dspark_markov_rank=16); variants.append(v)
    v = dict(REAL_CONFIG, dspark={"block_size": 5, "noise_token_id": 1, "target_layer_ids": [0], "markov_rank": 8,
                                  "n_mtp_layers": 2}); variants.append(v)
    v = dict(REAL_CONFIG); v.pop("eos_token_id"); v.pop("num_hidden_layers"); variants.append(v)
    v = dict(REAL_CONFIG); v.pop("index_topk"); variants.append(v)                  # an error case
    v = dict(REAL_CONFIG); v["vocab_size"] = "many"; variants.append(v)              # wrong type
    tm = cases.TinyModel(3, rope_pair(), 2)
    v = ckpt_util.model_config(tm); v["mtp"] = [{"compress_ratio": 0, "hash": False}]; variants.append(v)
    for cfg in variants:
        write_cfg_only(tmp_path, cfg)
        want, r, hh = capi.CkptCfg(), (C.c_int * 16)(), (C.c_int * 16)()
        rerr = C.create_string_buffer(256)
        rc = L.ref_parse_config(str(tmp_path / "config.json").encode(), C.addressof(want), r, hh, 16, rerr, 256)
        h, err = open_ckpt(tmp_path)
        if rc:
            assert not h and err == rerr.value.decode()
            continue
        assert h, err
        got = lib().apus_cuda_ckpt_cfg(h).contents
        assert bytes(got) == bytes(want), cfg
        for i in range(got.n_layers):
            a, b = C.c_int(), C.c_int()
            lib().apus_cuda_ckpt_layer_kind(h, i, C.byref(a), C.byref(b))
            assert (a.value, b.value) == (r[i], hh[i])
        lib().apus_cuda_ckpt_close(h)


@pytest.mark.parametrize("mutate,msg", [
    (lambda c: c.pop("hidden_size"), "config: missing dim"),
    (lambda c: c.pop("routed_scaling_factor"), "config: missing route_scale"),
    (lambda c: c.pop("compress_ratios"), "config: no layer schedule (layers|compress_ratios)"),
    (lambda c: c.update(compress_ratios=[0, 4]), "config: num_hidden_layers != compress_ratios"),
    (lambda c: c.update(layers=[{"hash": True}]), "config: layers[0].compress_ratio"),
])
def test_config_errors_name_the_key(tmp_path, mutate, msg):
    cfg = dict(REAL_CONFIG)
    mutate(cfg)
    write_cfg_only(tmp_path, cfg)
    h, err = open_ckpt(tmp_path)
    assert not h and err == msg
    assert lib().apus_cuda_last_error().decode() == msg


def test_missing_files_and_broken_shards(tmp_path, ckpt):
    h, err = open_ckpt(tmp_path / "nowhere")
    assert not h and "cannot open" in err
    (tmp_path / "config.json").write_text("{ not json")
    h, err = open_ckpt(tmp_path)
    assert not h and err.startswith("json:")
    d = tmp_path / "m"
    shutil.copytree(ckpt["dir"], d)
    (d / "model.safetensors.index.json").unlink()
    h, err = open_ckpt(d)
    assert not h and "model.safetensors.index.json" in err
    # a shard cut short: its tensors end past the end of the file (tests/m1 truncation case)
    d2 = tmp_path / "t"
    shutil.copytree(ckpt["dir"], d2)
    shard = d2 / "apus-00001.safetensors"
    raw = shard.read_bytes()
    shard.write_bytes(raw[: len(raw) - 1000])
    h, err = open_ckpt(d2)
    assert h, err                                                  # headers are parsed on first use
    assert lib().apus_cuda_ckpt_tensor(h, b"norm.weight", None, None, None, None) == 1
    assert b"tensor past EOF" in lib().apus_cuda_last_error()
    lib().apus_cuda_ckpt_close(h)
    # a header length that exceeds the file
    shard.write_bytes(struct.pack("<Q", 1 << 40) + raw[8:])
    h, err = open_ckpt(d2)
    assert lib().apus_cuda_ckpt_tensor(h, b"norm.weight", None, None, None, None) == 1
    assert b"bad header" in lib().apus_cuda_last_error()
    lib().apus_cuda_ckpt_close(h)


@pytest.mark.parametrize("delta", [+64, -64])
def test_shard_whose_offsets_disagree_with_the_shape_is_rejected(tmp_path, ckpt, delta):
    """The loader sizes its buffers from a tensor's shape, so a header whose data_offsets
    hold more (or fewer) bytes than dtype x shape must be refused when the shard is
    parsed, not copied: grow / shrink one tensor's payload range in the header."""
    d = tmp_path / "bad"
    shutil.copytree(ckpt["dir"], d)
    shard = d / "apus-00001.safetensors"
    raw = shard.read_bytes()
    hlen = struct.unpack("<Q", raw[:8])[0]
    hdr = json.loads(raw[8:8 + hlen])
    names = [n for n in hdr if n != "__metadata__"]
    last = max(names, key=lambda n: hdr[n]["data_offsets"][1] - hdr[n]["data_offsets"][0])   # the largest payload
    hdr[last]["data_offsets"][1] += delta
    doc = json.dumps(hdr, separators=(",", ":")).encode()
    doc += b" " * ((-len(doc)) % 8)
    body = raw[8 + hlen:] + (b"\0" * delta if delta > 0 else b"")
    shard.write_bytes(struct.pack("<Q", len(doc)) + doc + body)
    h, err = open_ckpt(d)
    assert h, err
    assert lib().apus_cuda_ckpt_tensor(h, last.encode(), None, None, None, None) == 1
    assert b"its shape and dtype need" in lib().apus_cuda_last_error()
    # nothing half-parsed is left behind: asking again fails the same way
    assert lib().apus_cuda_ckpt_tensor(h, last.encode(), None, None, None, None) == 1
    lib().apus_cuda_ckpt_close(h)
    # negative and absurd shapes
    hdr[last]["data_offsets"][1] -= delta
    hdr[last]["shape"] = [-4, 7]
    doc = json.dumps(hdr, separators=(",", ":")).encode()
    doc += b" " * ((-len(doc)) % 8)
    shard.write_bytes(struct.pack("<Q", len(doc)) + doc + raw[8 + hlen:])
    h, err = open_ckpt(d)
    assert lib().apus_cuda_ckpt_tensor(h, last.encode(), None, None, None, None) == 1
    assert b"bad shape" in lib().apus_cuda_last_error()
    lib().apus_cuda_ckpt_close(h)


def fnv1a(chunks):
    h = 1469598103934665603
    n = 0
    for c in chunks:
        b = bytes(c)
        n += len(b)
        for x in b:
            h = ((h ^ x) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h, n


def layer_chunks(L, e_lo, e_hi):
    """The tensors of a block as a loader must hand them over, in descriptor order
    (reference c/layer.h:202-330): FP8 views raw, wo_a as BF16 bits, everything loaded
    through apus_load_f32 widened to f32, local experts raw."""
    A, Mo = L.attn, L.moe
    f = lambda a: np.ascontiguousarray(a, np.float32).tobytes()
    out = []
    for cs in (A.wq_a, A.wq_b, A.wkv, A.wo_b):
        out += [cs[0].tobytes(), cs[1].tobytes()]
    out.append(A.wo_a.tobytes())
    out += [f(A.q_norm), f(A.kv_norm), f(A.sink), f(L.attn_norm_w), f(L.ffn_norm_w)]
    if A.ratio:
        c = A.comp
        out += [f(c["wkv"]), f(c["wgate"]), f(c["ape"]), f(c["norm"])]
        if A.ratio == 4:
            ic = A.idx_comp
            out += [f(A.idx_wproj), f(ic["wkv"]), f(ic["wgate"]), f(ic["ape"]), f(ic["norm"])]
    out.append(f(Mo.gate_w))
    if Mo.tid2eid is None:
        out.append(f(Mo.gate_bias))
    for fn, base, scale in (L.hc_attn, L.hc_ffn):
        out += [f(fn), f(base), f(scale)]
    if Mo.tid2eid is not None:
        out.append(Mo.tid2eid.tobytes())
    for e in range(e_lo, e_hi):
        for p, s in ((Mo.w1p, Mo.w1s), (Mo.w2p, Mo.w2s), (Mo.w3p, Mo.w3s)):
            out += [p[e].tobytes(), s[e].tobytes()]
    for cs in (Mo.sw1, Mo.sw2, Mo.sw3):
        out += [cs[0].tobytes(), cs[1].tobytes()]
    if A.ratio == 4:
        out += [A.idx_wq_b[0].tobytes(), A.idx_wq_b[1].tobytes()]
    return out


@pytest.mark.parametrize("threads", ["1", "3", "8"])
def test_whole_layers_load_like_the_model_receives_them(ckpt, threads, monkeypatch):
    """apus_cuda_ckpt_layer_digest runs the host half of apus_cuda_model_load (every
    conversion, experts read by the I/O threads): same digest as the tensors written,
    whatever the number of threads; an expert range loads only its experts."""
    monkeypatch.setenv("APUS_IO_THREADS", threads)
    tm = ckpt["tm"]
    E = tm.M["E"]
    for i, L in enumerate(tm.layers):
        want, nbytes = fnv1a(layer_chunks(L, 0, E))
        d, n = C.c_uint64(), C.c_uint64()
        assert lib().apus_cuda_ckpt_layer_digest(ckpt["h"], i, 0, -1, C.byref(d), C.byref(n)) == 0, \
            lib().apus_cuda_last_error()
        assert (d.value, n.value) == (want, nbytes), i
    want, nbytes = fnv1a(layer_chunks(tm.layers[1], 2, 6))
    d, n = C.c_uint64(), C.c_uint64()
    assert lib().apus_cuda_ckpt_layer_digest(ckpt["h"], 1, 2, 6, C.byref(d), C.byref(n)) == 0
    assert (d.value, n.value) == (want, nbytes)
    assert lib().apus_cuda_ckpt_layer_digest(ckpt["h"], 9, 0, -1, None, None) == 1


@pytest.mark.parametrize("kind", ["mtp", "dspark"])
def test_draft_module_sections_of_a_checkpoint(tmp_path, kind):
    """A checkpoint that also carries a draft module ("mtp.<k>.*" tensors and the config entry that declares
    them, reference c/model.h:336-373): the config fields say so, every written tensor resolves by name with
    its dtype and shape, and the loaders refuse a missing model with a message (no GPU needed for that)."""
    tm = cases.TinyModel(91, rope_pair(), 3)
    extra = {"mtp": cases.TinyMtp(94, rope_pair())} if kind == "mtp" else \
        {"dspark": cases.TinyDspark(95, rope_pair(), [0, 2], 2, 3, 5, 16)}
    written = ckpt_util.write_checkpoint(tmp_path, tm, seed=3, **extra)
    h, err = open_ckpt(tmp_path)
    assert h, err
    cfg = lib().apus_cuda_ckpt_cfg(h).contents
    assert (cfg.n_mtp, cfg.mtp_ratio, cfg.mtp_hash, cfg.dspark) == ((1, 0, 0, 0) if kind == "mtp" else (0, 0, 0, 1))   # the stage count of a DSpark section is its own field
    names = [n for n in written if n.startswith("mtp.")]
    assert any(n.endswith("e_proj.weight") for n in names) == (kind == "mtp")
    assert any("markov_head" in n for n in names) == (kind == "dspark")
    for name in names:
        dtype, shape, payload = written[name]
        dt, nd, nb = C.c_int(), C.c_int(), C.c_uint64()
        sh = (C.c_int64 * 8)()
        assert lib().apus_cuda_ckpt_tensor(h, name.encode(), C.byref(dt), C.byref(nd), sh, C.byref(nb)) == 0, name
        assert capi.ST_DTYPES[dt.value] == dtype and tuple(sh[: nd.value]) == tuple(shape) and nb.value == len(payload)
    lib().apus_cuda_ckpt_close(h)
    assert not lib().apus_cuda_mtp_load(None, str(tmp_path).encode(), 0)
    assert b"NULL model" in lib().apus_cuda_last_error()
    assert not lib().apus_cuda_dspark_load(None, str(tmp_path).encode())
    assert b"NULL model" in lib().apus_cuda_last_error()
