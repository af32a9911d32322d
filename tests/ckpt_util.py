"""Writes a tests.cases.TinyModel as a checkpoint directory in the reference's
container format (c/st.h:5-9, c/model.h:396-423, tensor names of
c/layer.h:202-330): config.json in the fixture schema, safetensors shards written
by hand (8-byte little-endian header length, JSON header, payloads) and
model.safetensors.index.json.  Test infrastructure only.
"""
import json
import struct
from pathlib import Path

import numpy as np

from apus_b200 import synth
import cases

DTYPE_SIZE = {"I8": 1, "U8": 1, "F8_E8M0": 1, "F8_E4M3": 1, "BF16": 2, "F16": 2, "F32": 4, "I32": 4, "I64": 8}


def wo_a_bits(codes, scales):
    """c/layer.h:226-247 in numpy: FP8 codes [O,K] and UE8M0 tile scales -> BF16 bits."""
    tab = synth.e4m3_table()
    sc = np.where(scales == 0, np.uint32(0x00400000), scales.astype(np.uint32) << 23).view(np.float32)
    full = np.repeat(np.repeat(sc, 128, axis=0), 128, axis=1)[: codes.shape[0], : codes.shape[1]]
    return synth.bf16_bits((tab[codes] * full).astype(np.float32))


def bf16_payload(a):
    """BF16-valued f32 array -> its BF16 bytes."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    assert not (u & 0xFFFF).any(), "not BF16-valued"
    return (u >> 16).astype(np.uint16).tobytes()


def write_shard(path, tensors, metadata=True):
    """tensors: [(name, dtype, shape, payload bytes)] in file order."""
    header, off = {}, 0
    if metadata:
        header["__metadata__"] = {"format": "pt"}
    for name, dtype, shape, payload in tensors:
        n = DTYPE_SIZE[dtype] * int(np.prod(shape, dtype=np.int64))
        assert len(payload) == n, (name, len(payload), n)
        header[name] = {"dtype": dtype, "shape": [int(s) for s in shape], "data_offsets": [off, off + n]}
        off += n
    doc = json.dumps(header, separators=(",", ":")).encode()
    doc += b" " * ((-len(doc)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(doc)))
        f.write(doc)
        for _, _, _, payload in tensors:
            f.write(payload)


def model_config(tm):
    A, M = cases.ATTN_DIMS, tm.M
    return {
        "dim": A["dim"], "n_heads": A["n_heads"], "head_dim": A["head_dim"], "rope_head_dim": A["rope_dim"],
        "q_lora_rank": A["q_lora"], "o_groups": A["o_groups"], "o_lora_rank": A["o_lora"],
        "window_size": A["window"], "moe_inter_dim": M["inter"], "n_routed_experts": M["E"],
        "n_activated_experts": M["topk"], "index_n_heads": A["idx_heads"], "index_head_dim": A["idx_dim"],
        "index_topk": A["idx_topk"], "hc_mult": M["hc"], "hc_sinkhorn_iters": M["iters"],
        "vocab_size": M["vocab"], "max_pos": A["max_pos"], "beta_fast": 32, "beta_slow": 1,
        "original_seq_len": 65536, "rope_factor": 16.0, "hc_eps": M["hc_eps"], "norm_eps": M["norm_eps"],
        "route_scale": synth.ROUTE_SCALE, "swiglu_limit": synth.SWIGLU_LIMIT, "rope_theta": 10000.0,
        "compress_rope_theta": 160000.0, "bos_token_id": 0, "eos_token_id": 1,
        "layers": [{"compress_ratio": L.attn.ratio, "hash": bool(L.moe.tid2eid is not None)} for L in tm.layers],
    }


def layer_tensors(i, L, seed, coalesce, px=None):
    """The tensors of block i (or of the block under prefix `px`) in file order.  wo_a is drawn
    here as FP8 and the layer's in-memory BF16 copy is overwritten with what a loader must derive."""
    A, W, Mo = L.attn, L.attn, L.moe
    D = A.D
    px = px or f"layers.{i}"
    out = []
    f32 = lambda name, a: out.append((f"{px}.{name}", "F32", a.shape, np.ascontiguousarray(a, np.float32).tobytes()))
    bf16 = lambda name, a: out.append((f"{px}.{name}", "BF16", a.shape, bf16_payload(a)))

    def fp8(name, cs):
        codes, scales = cs
        out.append((f"{px}.{name}.weight", "F8_E4M3", codes.shape, codes.tobytes()))
        out.append((f"{px}.{name}.scale", "F8_E8M0", scales.shape, scales.tobytes()))
    fp8("attn.wq_a", W.wq_a); fp8("attn.wq_b", W.wq_b); fp8("attn.wkv", W.wkv); fp8("attn.wo_b", W.wo_b)
    rng = np.random.default_rng([seed, i, 7])
    wo = synth.fp8_weight(rng, D["o_groups"] * D["o_lora"], D["n_heads"] * D["head_dim"] // D["o_groups"], std=0.04)
    W.wo_a[...] = wo_a_bits(*wo)
    fp8("attn.wo_a", wo)
    f32("attn.q_norm.weight", W.q_norm); f32("attn.kv_norm.weight", W.kv_norm); f32("attn.attn_sink", W.sink)
    f32("attn_norm.weight", L.attn_norm_w); f32("ffn_norm.weight", L.ffn_norm_w)
    if A.ratio:
        c = W.comp
        bf16("attn.compressor.wkv.weight", c["wkv"]); bf16("attn.compressor.wgate.weight", c["wgate"])
        f32("attn.compressor.ape", c["ape"]); f32("attn.compressor.norm.weight", c["norm"])
        if A.ratio == 4:
            ic = W.idx_comp
            fp8("attn.indexer.wq_b", W.idx_wq_b)
            bf16("attn.indexer.weights_proj.weight", W.idx_wproj)
            bf16("attn.indexer.compressor.wkv.weight", ic["wkv"])
            bf16("attn.indexer.compressor.wgate.weight", ic["wgate"])
            f32("attn.indexer.compressor.ape", ic["ape"]); f32("attn.indexer.compressor.norm.weight", ic["norm"])
    bf16("ffn.gate.weight", Mo.gate_w)
    if Mo.tid2eid is not None:
        out.append((f"{px}.ffn.gate.tid2eid", "I64", Mo.tid2eid.shape, Mo.tid2eid.tobytes()))
    else:
        f32("ffn.gate.bias", Mo.gate_bias)
    late = []
    for e in range(Mo.E):
        six = []
        for wn, (p, s) in (("w1", (Mo.w1p, Mo.w1s)), ("w2", (Mo.w2p, Mo.w2s)), ("w3", (Mo.w3p, Mo.w3s))):
            six.append((f"{px}.ffn.experts.{e}.{wn}.weight", "I8", p[e].shape, p[e].tobytes()))
            six.append((f"{px}.ffn.experts.{e}.{wn}.scale", "F8_E8M0", s[e].shape, s[e].tobytes()))
        if coalesce:
            out += six                      # the converter's slab: six adjacent tensors per expert
        else:
            out += six[0::2]                # weights here, scales after everything else
            late += six[1::2]
    fp8("ffn.shared_experts.w1", Mo.sw1); fp8("ffn.shared_experts.w2", Mo.sw2); fp8("ffn.shared_experts.w3", Mo.sw3)
    for kind, (fn, base, scale) in (("attn", L.hc_attn), ("ffn", L.hc_ffn)):
        f32(f"hc_{kind}_fn", fn); f32(f"hc_{kind}_base", base); f32(f"hc_{kind}_scale", scale)
    return out + late


def draft_tensors(mtp=None, dspark=None, seed=0, coalesce=True):
    """The "mtp.<k>.*" tensors of an MTP head (cases.TinyMtp, c/mtp.h:213-281) or of a DSpark module
    (cases.TinyDspark, c/dspark.h:272-341) and the config entries that declare them."""
    out, cfg = [], {}
    f32 = lambda name, a: out.append((name, "F32", np.shape(a), np.ascontiguousarray(a, np.float32).tobytes()))
    bf16 = lambda name, a: out.append((name, "BF16", np.shape(a), bf16_payload(a)))

    def fp8(name, cs):
        out.append((f"{name}.weight", "F8_E4M3", cs[0].shape, cs[0].tobytes()))
        out.append((f"{name}.scale", "F8_E8M0", cs[1].shape, cs[1].tobytes()))
    if mtp is not None:
        cfg["mtp"] = [{"compress_ratio": 0, "hash": False}]
        out += layer_tensors(1000, mtp.block, seed, coalesce, px="mtp.0")
        fp8("mtp.0.e_proj", mtp.e_proj); fp8("mtp.0.h_proj", mtp.h_proj)
        f32("mtp.0.enorm.weight", mtp.enorm_w); f32("mtp.0.hnorm.weight", mtp.hnorm_w); f32("mtp.0.norm.weight", mtp.norm_w)
        f32("mtp.0.hc_head_fn", mtp.hc_head_fn); f32("mtp.0.hc_head_base", mtp.hc_head_base)
        f32("mtp.0.hc_head_scale", np.array([mtp.desc.hc_head_scale], np.float32))
    if dspark is not None:
        d = dspark.desc
        cfg["dspark"] = {"block_size": int(d.block_size), "noise_token_id": int(d.noise_id), "markov_rank": int(d.markov_rank),
                         "target_layer_ids": [int(d.targets[i]) for i in range(d.n_targets)], "n_mtp_layers": int(d.n_stages)}
        last = d.n_stages - 1
        for k, L in enumerate(dspark.stages):
            out += layer_tensors(1000 + k, L, seed, coalesce, px=f"mtp.{k}")
        fp8("mtp.0.main_proj", dspark.main_proj)
        f32("mtp.0.main_norm.weight", dspark.main_norm_w); f32(f"mtp.{last}.norm.weight", dspark.norm_w)
        f32(f"mtp.{last}.hc_head_fn", dspark.hc_head_fn); f32(f"mtp.{last}.hc_head_base", dspark.hc_head_base)
        f32(f"mtp.{last}.hc_head_scale", np.array([d.hc_head_scale], np.float32))
        bf16(f"mtp.{last}.markov_head.markov_w1.weight", dspark.markov_w1)
        bf16(f"mtp.{last}.markov_head.markov_w2.weight", dspark.markov_w2)
        bf16(f"mtp.{last}.confidence_head.proj.weight", dspark.conf_proj)
    return out, cfg


def write_checkpoint(path, tm, seed=0, n_shards=2, coalesce=True, subdir=False, mtp=None, dspark=None):
    """Writes `tm` under `path`; returns {tensor name: (dtype, shape, payload)}.
    subdir: shards + index under <path>/weights (the fixture layout, c/model.h:414-417).
    mtp / dspark: a draft module to write beside the model (both use the "mtp.*" names: one at a time)."""
    path = Path(path)
    wdir = path / "weights" if subdir else path
    wdir.mkdir(parents=True, exist_ok=True)
    config = model_config(tm)
    extra, extra_cfg = draft_tensors(mtp, dspark, seed, coalesce)
    config.update(extra_cfg)
    (path / "config.json").write_text(json.dumps(config, indent=1))
    shards = [[] for _ in range(n_shards)]
    shards[0] += extra
    for i, L in enumerate(tm.layers):
        shards[i % n_shards] += layer_tensors(i, L, seed, coalesce)
    V, dim, hc = tm.M["vocab"], cases.ATTN_DIMS["dim"], tm.M["hc"]
    shards[-1] += [
        ("embed.weight", "BF16", (V, dim), tm.embed.tobytes()), ("head.weight", "BF16", (V, dim), tm.head.tobytes()),
        ("norm.weight", "F32", (dim,), tm.norm_w.tobytes()),
        ("hc_head_fn", "F32", tm.hc_head_fn.shape, tm.hc_head_fn.tobytes()),
        ("hc_head_base", "F32", (hc,), tm.hc_head_base.tobytes()),
        ("hc_head_scale", "F32", (1,), np.float32(tm.desc.hc_head_scale).tobytes()),
    ]
    weight_map, written = {}, {}
    for k, ts in enumerate(shards):
        fname = f"apus-{k:05d}.safetensors"
        write_shard(wdir / fname, ts)
        for name, dtype, shape, payload in ts:
            weight_map[name] = fname
            written[name] = (dtype, tuple(int(s) for s in shape), payload)
    (wdir / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    return written
