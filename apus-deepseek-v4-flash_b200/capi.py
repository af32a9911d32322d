"""ctypes view of include/apus_b200.h: structures and function signatures.

The structures are layout-identical to the reference's (c/st.h:88-89,
c/moe.h:37-71, c/fp4.h:184-188), so the same Python objects can be handed to
this library and, in the tests, to the reference build.
"""
import ctypes as C
import re
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
HEADER = ROOT.parent / "include" / "apus_b200.h"
LIB_PATH = ROOT / "libapus_b200.so"

u8p = C.POINTER(C.c_uint8)
f32p = C.POINTER(C.c_float)
i32p = C.POINTER(C.c_int32)
i64p = C.POINTER(C.c_int64)
u16p = C.POINTER(C.c_uint16)


class QW(C.Structure):
    """ApusFp8W / ApusFp4W (c/st.h:88-89): codes|packed, scales, O, K."""
    _fields_ = [("codes", C.c_void_p), ("scales", C.c_void_p),
                ("O", C.c_int64), ("K", C.c_int64)]


DRAFT_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_int64, C.POINTER(C.c_int64), C.c_int)
RESOLVE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_int,
                         C.POINTER(QW), C.POINTER(QW), C.POINTER(QW))
HINT_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_int, C.c_int)
LAYER_END_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_int)


class MoeW(C.Structure):
    """ApusMoeW (c/moe.h:37-63)."""
    _fields_ = [("E", C.c_int), ("topk", C.c_int), ("inter", C.c_int),
                ("dim", C.c_int), ("hash", C.c_int),
                ("route_scale", C.c_float), ("limit", C.c_float),
                ("gate_w", C.c_void_p), ("gate_bias", C.c_void_p),
                ("tid2eid", C.c_void_p),
                ("w1", C.POINTER(QW)), ("w2", C.POINTER(QW)), ("w3", C.POINTER(QW)),
                ("sw1", QW), ("sw2", QW), ("sw3", QW),
                ("hook_ctx", C.c_void_p),
                ("hook_resolve", C.c_void_p), ("hook_hint", C.c_void_p),
                ("hook_layer_end", C.c_void_p),
                ("hook_hint_ctx", C.c_void_p), ("hook_layer_end_ctx", C.c_void_p),
                ("layer_id", C.c_int)]


class MoeInterm(C.Structure):
    """ApusMoeInterm (c/moe.h:67-71)."""
    _fields_ = [("router_scores", C.c_void_p), ("router_scores_biased", C.c_void_p),
                ("router_w", C.c_void_p), ("router_idx", C.c_void_p),
                ("moe_routed", C.c_void_p), ("moe_shared", C.c_void_p)]


class AttnCfg(C.Structure):
    """ApusAttnCfg (c/attn.h:114-122)."""
    _fields_ = [(n, C.c_int) for n in ("dim", "n_heads", "head_dim", "rope_dim", "q_lora", "o_groups",
                                        "o_lora", "window", "ratio", "has_indexer", "idx_heads",
                                        "idx_dim", "idx_topk")] + [("eps", C.c_float), ("max_pos", C.c_int)]


class CompW(C.Structure):
    """ApusCompW (c/attn.h:126-130)."""
    _fields_ = [("wkv", C.c_void_p), ("wgate", C.c_void_p), ("ape", C.c_void_p), ("norm", C.c_void_p),
                ("ratio", C.c_int), ("overlap", C.c_int), ("d", C.c_int), ("rd", C.c_int),
                ("rotate", C.c_int), ("eps", C.c_float)]


class AttnW(C.Structure):
    """ApusAttnW (c/attn.h:132-143)."""
    _fields_ = [("wq_a", QW), ("wq_b", QW), ("wkv", QW), ("wo_b", QW), ("wo_a", C.c_void_p),
                ("q_norm", C.c_void_p), ("kv_norm", C.c_void_p), ("sink", C.c_void_p),
                ("comp", CompW), ("idx_comp", CompW), ("idx_wq_b", QW), ("idx_wproj", C.c_void_p)]


class CompS(C.Structure):
    """ApusCompS (c/attn.h:147-153)."""
    _fields_ = [("rows", C.c_int), ("cols", C.c_int), ("kv", C.c_void_p), ("sc", C.c_void_p),
                ("cache", C.c_void_p), ("nb", C.c_int), ("max_nb", C.c_int), ("d", C.c_int),
                ("cap", C.c_int)]


class AttnS(C.Structure):
    """ApusAttnS (c/attn.h:155-160)."""
    _fields_ = [("pos", C.c_int64), ("win", C.c_void_p), ("comp", CompS), ("idx_comp", CompS)]


class AttnInterm(C.Structure):
    """ApusAttnInterm (c/attn.h:168-173)."""
    _fields_ = [("q", C.c_void_p), ("win_kv", C.c_void_p), ("comp_kv", C.c_void_p),
                ("idx_comp_kv", C.c_void_p), ("idx_scores", C.c_void_p), ("idx_topk", C.c_void_p),
                ("attn_out", C.c_void_p), ("o_out", C.c_void_p), ("comp_nb", C.c_int),
                ("idx_nb", C.c_int), ("idx_k", C.c_int)]


class LayerDesc(C.Structure):
    """ApusCudaLayerDesc: what apus_block_forward reads of ApusLayer (c/layer.h:45-71)."""
    _fields_ = [("acfg", AttnCfg), ("aw", AttnW), ("mw", MoeW),
                ("attn_norm_w", C.c_void_p), ("ffn_norm_w", C.c_void_p),
                ("hc_attn_fn", C.c_void_p), ("hc_attn_base", C.c_void_p), ("hc_attn_scale", C.c_void_p),
                ("hc_ffn_fn", C.c_void_p), ("hc_ffn_base", C.c_void_p), ("hc_ffn_scale", C.c_void_p),
                ("cos", C.c_void_p), ("sin", C.c_void_p), ("rope_rows", C.c_int)]


class ModelDesc(C.Structure):
    """ApusCudaModelDesc: top-level tensors and sizes (c/model.h:58-84)."""
    _fields_ = [("n_layers", C.c_int), ("dim", C.c_int), ("hc_mult", C.c_int), ("hc_sinkhorn_iters", C.c_int),
                ("vocab", C.c_int), ("hc_eps", C.c_float), ("norm_eps", C.c_float),
                ("layers", C.POINTER(LayerDesc)), ("embed", C.c_void_p), ("embed_bf16", C.c_int),
                ("head", C.c_void_p), ("head_bf16", C.c_int), ("norm_w", C.c_void_p),
                ("hc_head_fn", C.c_void_p), ("hc_head_base", C.c_void_p), ("hc_head_scale", C.c_float)]


class MtpDesc(C.Structure):
    """ApusCudaMtpDesc: what apus_mtp_forward reads of ApusMtp (c/mtp.h:66-76)."""
    _fields_ = [("block", LayerDesc), ("e_proj", QW), ("h_proj", QW), ("enorm_w", C.c_void_p), ("hnorm_w", C.c_void_p),
                ("norm_w", C.c_void_p), ("hc_head_fn", C.c_void_p), ("hc_head_base", C.c_void_p),
                ("hc_head_scale", C.c_float)]


class DsparkDesc(C.Structure):
    """ApusCudaDsparkDesc: what the DSpark functions read of ApusDspark (c/dspark.h:88-107)."""
    _fields_ = [("n_stages", C.c_int), ("block_size", C.c_int), ("noise_id", C.c_int), ("markov_rank", C.c_int),
                ("n_targets", C.c_int), ("targets", C.c_int * 8), ("stages", C.POINTER(LayerDesc)), ("main_proj", QW),
                ("main_norm_w", C.c_void_p), ("norm_w", C.c_void_p), ("hc_head_fn", C.c_void_p), ("hc_head_base", C.c_void_p),
                ("hc_head_scale", C.c_float), ("markov_w1", C.c_void_p), ("markov_w2", C.c_void_p), ("conf_proj", C.c_void_p)]


class Fp4GemmEnt(C.Structure):
    """ApusFp4GemmEnt (c/fp4.h:184-188)."""
    _fields_ = [("w", C.c_void_p), ("ws", C.c_void_p), ("out", C.c_void_p),
                ("m0", C.c_size_t), ("M", C.c_size_t)]


class Hooks(C.Structure):
    """ApusCudaHooks == ApusBackendHooks (c/backend_metal.h:73-80)."""
    _fields_ = [("fp8_linear", C.c_void_p), ("f32_linear", C.c_void_p),
                ("head_gemv", C.c_void_p)]


class CkptCfg(C.Structure):
    """ApusCudaCkptCfg: the reference's ApusCfg (c/layer.h:32-41) + what its config parser returns beside it."""
    _fields_ = [(n, C.c_int) for n in (
        "dim", "n_heads", "head_dim", "rope_head_dim", "q_lora_rank", "o_groups", "o_lora_rank", "window_size",
        "moe_inter_dim", "n_routed_experts", "n_activated_experts", "index_n_heads", "index_head_dim",
        "index_topk", "hc_mult", "hc_sinkhorn_iters", "original_seq_len", "beta_fast", "beta_slow",
        "vocab_size", "max_pos")] + \
        [(n, C.c_float) for n in ("route_scale", "swiglu_limit", "hc_eps", "norm_eps")] + \
        [(n, C.c_double) for n in ("rope_theta", "compress_rope_theta", "rope_factor")] + \
        [(n, C.c_int) for n in ("n_layers", "bos_id", "eos_id", "n_mtp", "mtp_ratio", "mtp_hash", "dspark")]


ST_DTYPES = ("I8", "U8", "F8_E8M0", "F8_E4M3", "BF16", "F16", "F32", "I32", "I64", "OTHER")


def ptr(a):
    """Address of a numpy array's (or torch tensor's) first element."""
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    if hasattr(a, "data_ptr"):
        return a.data_ptr()
    return a


def qw(codes, scales, O, K):
    return QW(ptr(codes), ptr(scales), int(O), int(K))


def declared_symbols():
    """Every function name the headers under include/ declare."""
    names = set()
    for h in sorted(HEADER.parent.glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        names |= set(re.findall(r"\b(apus_(?:cuda|synth)_\w+|apus_fnv1a)\s*\(", text))
    return sorted(names)


def load(path=LIB_PATH):
    """dlopen the backend and attach argument/return types."""
    if not Path(path).exists():
        raise RuntimeError(
            f"{path} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()'); "
            "there is no CPU fallback")
    lib = C.CDLL(str(path))
    vp, ci, cf, sz, i64 = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_int64
    sigs = {
        "apus_cuda_enable": (ci, [C.c_char_p, sz]),
        "apus_cuda_disable": (None, []),
        "apus_cuda_is_enabled": (ci, []),
        "apus_cuda_bytes_uploaded": (C.c_uint64, []),
        "apus_cuda_dispatches": (C.c_uint64, []),
        "apus_cuda_fill_hooks": (ci, [C.POINTER(Hooks), sz, sz]),
        "apus_cuda_last_error": (C.c_char_p, []),
        "apus_cuda_forget": (None, [vp]),
        "apus_cuda_kernel_status": (ci, [ci]),
        "apus_cuda_fp8_linear": (ci, [C.POINTER(QW), vp, vp, ci, ci, ci]),
        "apus_cuda_fp4_linear": (ci, [C.POINTER(QW), vp, vp, ci, ci, ci]),
        "apus_cuda_f32_linear": (ci, [vp, vp, vp, ci, ci, ci, ci]),
        "apus_cuda_head_gemv_bf16": (ci, [vp, vp, vp, i64, i64]),
        "apus_cuda_fp8_gemm": (ci, [vp, vp, vp, vp, vp, ci, ci, ci]),
        "apus_cuda_fp4_gemm": (ci, [vp, vp, vp, vp, vp, ci, ci, ci]),
        "apus_cuda_fp4_gemm_tc": (ci, [vp, vp, vp, vp, vp, ci, ci, ci]),
        "apus_cuda_fp4_gemm_grouped": (ci, [C.POINTER(Fp4GemmEnt), sz, vp, vp, sz, sz, sz]),
        "apus_cuda_fp8_act_quant": (ci, [vp, ci, ci, vp, vp]),
        "apus_cuda_rmsnorm": (ci, [vp, vp, cf, vp, i64, i64]),
        "apus_cuda_expert": (ci, [vp, vp, vp, ci, cf, vp, ci, ci, ci, vp]),
        "apus_cuda_topk_stable": (ci, [vp, ci, ci, vp, ci]),
        "apus_cuda_router_score": (ci, [C.POINTER(MoeW), vp, ci, vp, vp]),
        "apus_cuda_moe_forward": (ci, [C.POINTER(MoeW), vp, vp, ci, vp, C.POINTER(MoeInterm)]),
        "apus_cuda_sparse_attn": (ci, [vp, vp, ci, ci, vp, ci, ci, cf, vp, i64, vp, i64, vp]),
        "apus_cuda_attention": (ci, [C.POINTER(AttnCfg), C.POINTER(AttnW), C.POINTER(AttnS), vp, ci, i64,
                                    vp, vp, vp, C.POINTER(AttnInterm)]),
        "apus_cuda_set_sum_order": (ci, [ci]),
        "apus_cuda_set_tree_ops": (ci, [ci]),
        "apus_cuda_set_prefill_chunk": (ci, [ci]),
        "apus_cuda_block_forward": (ci, [C.POINTER(LayerDesc), ci, ci, cf, cf, C.POINTER(AttnS), vp, vp, ci, i64]),
        "apus_cuda_block_forward_v": (ci, [C.POINTER(LayerDesc), ci, ci, cf, cf, C.POINTER(AttnS), vp, vp, ci, i64, i64]),
        "apus_cuda_model_create": (vp, [C.POINTER(ModelDesc), ci, ci]),
        "apus_cuda_model_create_ep": (vp, [C.POINTER(ModelDesc), ci, ci, ci, ci]),
        "apus_cuda_model_load": (vp, [C.c_char_p, ci, ci, ci, ci]),
        "apus_cuda_model_set_stream": (ci, [vp, vp, ci]),
        "apus_cuda_model_spec_generate": (ci, [vp, vp, ci, ci, ci, DRAFT_FN, vp, vp, vp]),
        "apus_cuda_model_snapshot": (vp, [vp, vp]),
        "apus_cuda_model_restore": (ci, [vp, vp]),
        "apus_cuda_snap_free": (None, [vp]),
        "apus_cuda_model_forward_group": (ci, [vp, ci, vp, ci, vp, vp]),
        "apus_cuda_model_generate_group": (ci, [vp, ci, vp, ci, ci, vp, C.POINTER(cf), C.POINTER(cf)]),
        "apus_cuda_ckpt_open": (vp, [C.c_char_p, C.c_char_p, sz]),
        "apus_cuda_ckpt_close": (None, [vp]),
        "apus_cuda_ckpt_cfg": (C.POINTER(CkptCfg), [vp]),
        "apus_cuda_ckpt_layer_kind": (ci, [vp, ci, C.POINTER(ci), C.POINTER(ci)]),
        "apus_cuda_ckpt_tensor": (ci, [vp, C.c_char_p, C.POINTER(ci), C.POINTER(ci), i64p, C.POINTER(C.c_uint64)]),
        "apus_cuda_ckpt_read": (ci, [vp, C.c_char_p, vp, C.c_uint64]),
        "apus_cuda_ckpt_read_f32": (ci, [vp, C.c_char_p, vp, C.c_uint64]),
        "apus_cuda_ckpt_wo_a": (ci, [vp, ci, vp, C.c_uint64]),
        "apus_cuda_ckpt_rope": (ci, [vp, ci, i64, vp, vp]),
        "apus_cuda_ckpt_expert": (ci, [vp, ci, ci, vp, C.c_uint64, C.POINTER(QW), C.POINTER(QW), C.POINTER(QW)]),
        "apus_cuda_ckpt_layer_digest": (ci, [vp, ci, ci, ci, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
        "apus_cuda_ckpt_read_count": (C.c_uint64, [vp]),
        "apus_cuda_ckpt_read_bytes": (C.c_uint64, [vp]),
        "apus_cuda_use_stream": (ci, [vp, ci]),
        "apus_cuda_model_set_ids": (ci, [vp, vp]),
        "apus_cuda_model_begin_step": (ci, [vp]),
        "apus_cuda_model_attn_half": (ci, [vp, ci]),
        "apus_cuda_model_ffn_input": (vp, [vp, ci]),
        "apus_cuda_model_ffn_output": (ci, [vp, ci, vp]),
        "apus_cuda_model_end_step": (ci, [vp, ci, ci]),
        "apus_cuda_model_capturing": (ci, [vp, ci]),
        "apus_cuda_model_note_step": (ci, [vp]),
        "apus_cuda_model_ids": (vp, [vp]),
        "apus_cuda_model_read": (ci, [vp, vp, vp]),
        "apus_cuda_model_destroy": (None, [vp]),
        "apus_cuda_model_reset": (ci, [vp]),
        "apus_cuda_model_pos": (i64, [vp]),
        "apus_cuda_model_moe": (vp, [vp, ci]),
        "apus_cuda_model_info": (ci, [vp, C.POINTER(ci), C.POINTER(ci), C.POINTER(ci), C.POINTER(ci)]),
        "apus_cuda_serve": (ci, [vp, ci, ci, ci]),
        "apus_cuda_model_use_graph": (ci, [vp, ci]),
        "apus_cuda_model_set_sampling": (ci, [vp, cf, cf, C.c_uint64]),
        "apus_cuda_sample_logits_u": (ci, [vp, C.c_size_t, cf, cf, vp, vp, ci]),
        "apus_cuda_moe_timing_enabled": (ci, [vp]),
        "apus_cuda_moe_work_items": (C.c_longlong, [vp, ci]),
        "apus_cuda_model_forward": (ci, [vp, vp, ci, vp, vp]),
        "apus_cuda_model_forward_all": (ci, [vp, vp, ci, vp, vp]),
        "apus_cuda_model_forward_h": (ci, [vp, vp, ci, vp, ci, vp, vp]),
        "apus_cuda_model_forward_mh": (ci, [vp, vp, ci, vp, ci, vp, vp, ci, vp]),
        "apus_cuda_mtp_create": (vp, [vp, vp]),
        "apus_cuda_mtp_destroy": (None, [vp]),
        "apus_cuda_mtp_reset": (ci, [vp]),
        "apus_cuda_mtp_forward": (ci, [vp, vp, vp, ci, C.c_int64, vp, vp, vp]),
        "apus_cuda_model_spec_generate_mtp": (ci, [vp, vp, vp, ci, ci, ci, vp, vp]),
        "apus_cuda_dspark_create": (vp, [vp, vp]),
        "apus_cuda_dspark_load": (vp, [vp, C.c_char_p]),
        "apus_cuda_mtp_load": (vp, [vp, C.c_char_p, ci]),
        "apus_cuda_dspark_destroy": (None, [vp]),
        "apus_cuda_dspark_reset": (ci, [vp]),
        "apus_cuda_dspark_set_sampling": (ci, [vp, C.c_float, C.c_uint64]),
        "apus_cuda_dspark_feed": (ci, [vp, vp, C.c_int64, ci]),
        "apus_cuda_dspark_draft_round": (ci, [vp, C.c_int64, vp, C.c_int64, vp, vp, vp, vp]),
        "apus_cuda_model_spec_generate_dspark": (ci, [vp, vp, vp, ci, ci, vp, vp]),
        "apus_cuda_model_generate": (ci, [vp, vp, ci, ci, vp, C.POINTER(cf), C.POINTER(cf)]),
        "apus_cuda_apply_rope": (ci, [vp, vp, vp, ci, ci, ci, ci]),
        "apus_cuda_hadamard": (ci, [vp, ci, ci]),
        "apus_cuda_fp8_qat_sim": (ci, [vp, ci, ci, ci]),
        "apus_cuda_fp4_qat_sim": (ci, [vp, ci, ci]),
        "apus_cuda_mhc_prepost": (ci, [vp, sz, sz, vp, vp, vp, cf, cf, ci, vp, vp, vp, ci]),
        "apus_cuda_hc_pre": (ci, [vp, sz, sz, vp, vp, vp, cf, cf, ci, vp, cf, vp, vp, vp, vp, ci]),
        "apus_cuda_hc_pre_noalloc_dev": (ci, [vp, sz, sz, vp, vp, vp, cf, cf, ci, vp, cf, vp, vp, vp, vp, ci, vp]),
        "apus_cuda_hc_post": (ci, [vp, vp, vp, vp, vp, sz, sz, ci]),
        "apus_cuda_hc_head": (ci, [vp, sz, sz, vp, cf, vp, cf, cf, vp, ci]),
        "apus_cuda_moe_create": (vp, [C.POINTER(MoeW), ci, ci]),
        "apus_cuda_moe_destroy": (None, [vp]),
        "apus_cuda_moe_bytes": (C.c_uint64, [vp]),
        "apus_cuda_moe_set_hash_table": (ci, [vp, vp, i64]),
        "apus_cuda_moe_get": (vp, [C.POINTER(MoeW)]),
        "apus_cuda_moe_use_tc": (ci, [vp, ci]),
        "apus_cuda_moe_timing": (None, [vp, ci]),
        "apus_cuda_moe_timing_read": (ci, [vp, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(ci)]),
        "apus_cuda_moe_route_dev": (ci, [vp, vp, vp, ci, vp, vp, vp, vp, vp]),
        "apus_cuda_moe_experts_dev": (ci, [vp, vp, ci, vp, vp, ci, vp, vp]),
        "apus_cuda_moe_combine_dev": (ci, [vp, vp, vp, vp, ci, vp, vp, vp]),
        "apus_cuda_moe_shared_dev": (ci, [vp, vp, ci, vp, vp]),
        "apus_cuda_moe_ep_plan_dev": (ci, [vp, ci, ci, ci, ci, vp, vp, vp]),
        "apus_cuda_moe_ep_rows_dev": (ci, [vp, ci, vp, ci, ci, ci, vp, vp]),
        "apus_cuda_moe_ep_row_bytes": (C.c_size_t, [vp]),
        "apus_cuda_moe_ep_pack_dev": (ci, [vp, vp, ci, vp, ci, vp, vp]),
        "apus_cuda_moe_experts_q_dev": (ci, [vp, vp, ci, vp, vp, vp]),
        "apus_cuda_moe_ep_unpack_dev": (ci, [vp, ci, vp, ci, vp, vp]),
        "apus_cuda_moe_forward_dev": (ci, [vp, vp, vp, ci, vp, vp]),
        "apus_cuda_moe_last_routing": (ci, [vp, ci, vp, vp, vp]),
        "apus_cuda_fp4_upload": (vp, [C.POINTER(QW)]),
        "apus_cuda_fp8_upload": (vp, [C.POINTER(QW)]),
        "apus_cuda_fp4_free": (None, [vp]),
        "apus_cuda_fp8_free": (None, [vp]),
        "apus_cuda_fp4_linear_dev": (ci, [vp, vp, vp, ci, vp]),
        "apus_cuda_fp8_linear_dev": (ci, [vp, vp, vp, ci, vp]),
        "apus_cuda_expert_fp4_dev": (ci, [vp, vp, vp, cf, vp, ci, vp, vp]),
        "apus_cuda_topk_stable_dev": (ci, [vp, ci, ci, vp, ci, vp]),
        "apus_cuda_sparse_attn_dev": (ci, [vp, vp, ci, ci, vp, ci, ci, cf, vp, i64, vp, i64, vp, vp]),
        "apus_cuda_sparse_attn_batch_dev": (ci, [vp, vp, ci, ci, vp, ci, ci, cf, vp, i64, i64, vp, i64, i64, vp, vp]),
        "apus_synth_key": (C.c_uint64, [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32]),
        "apus_synth_fill_host": (ci, [vp, ci, C.c_uint64, C.c_uint64, C.c_double, C.c_double, ci]),
        "apus_synth_fill_dev": (ci, [vp, ci, C.c_uint64, C.c_uint64, C.c_double, C.c_double, vp]),
        "apus_synth_fill_slab_dev": (ci, [vp, ci, C.c_uint64, C.c_uint32, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32,
                                          C.c_double, C.c_double, vp]),
        "apus_fnv1a": (C.c_uint64, [vp, C.c_uint64, C.c_uint64]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib
