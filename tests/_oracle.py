"""ctypes loaders for the CPU checkers (test infrastructure only).

  ora()  oracle/liboracle.so       plain-C restatement, built on demand with gcc
  ref()  oracle/_ref/libapus_ref.so the unmodified reference, prebuilt where the
                                    reference checkout is mounted (None if absent)
"""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORA_DIR = ROOT / "oracle"

vp, ci, cf, sz, i64 = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_int64
_ora = None
_ref = None


class OraQW(C.Structure):
    _fields_ = [("codes", vp), ("scales", vp), ("O", i64), ("K", i64)]


def P(a):
    return None if a is None else a.ctypes.data


def ora():
    global _ora
    if _ora is None:
        so = ORA_DIR / "liboracle.so"
        src = ORA_DIR / "apus_oracle.c"
        if not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
            subprocess.check_call(["make", "-C", str(ORA_DIR), "liboracle.so"],
                                  stdout=subprocess.DEVNULL)
        L = C.CDLL(str(so))
        q = C.POINTER(OraQW)
        sig = {
            "ora_bf16_round": (cf, [cf]), "ora_ue8m0": (cf, [C.c_uint8]),
            "ora_e4m3_to_f32": (cf, [C.c_uint8]), "ora_e4m3_from_f32": (C.c_uint8, [cf]),
            "ora_act_quant_row": (None, [vp, sz, vp, vp]),
            "ora_act_quant": (None, [vp, ci, ci, vp, vp, vp]),
            "ora_fp4_gemm": (None, [vp, vp, vp, vp, vp, sz, sz, sz]),
            "ora_fp8_gemm": (None, [vp, vp, vp, vp, vp, sz, sz, sz]),
            "ora_qlinear": (None, [ci, vp, vp, vp, vp, ci, ci, ci]),
            "ora_f32_linear": (None, [vp, vp, vp, ci, ci, ci, ci]),
            "ora_head_gemv_bf16": (None, [vp, vp, vp, i64, i64]),
            "ora_rms_norm": (None, [vp, vp, cf, vp, sz]),
            "ora_swiglu": (None, [vp, vp, vp, sz, cf]),
            "ora_expert": (None, [q, q, q, ci, cf, vp, ci, ci, ci, vp]),
            "ora_topk_stable": (None, [vp, ci, ci, vp]),
            "ora_sample_logits_u": (ci, [vp, C.c_size_t, C.c_float, C.c_float, C.c_double, vp, vp, vp]),
            "ora_sample_argmax": (ci, [vp, C.c_size_t]),
            "ora_rng_uniform": (C.c_double, [vp]),
            "ora_router_score": (None, [vp, vp, ci, ci, vp, ci, vp, vp]),
            "ora_moe_forward": (None, [ci, ci, ci, ci, ci, cf, cf, vp, vp, vp, vp, vp, vp,
                                       q, q, q, vp, vp, ci, vp, vp, vp, vp, vp]),
            "ora_sparse_attn": (None, [vp, vp, ci, ci, vp, ci, ci, cf, vp, i64, vp, vp]),
            "ora_sinkhorn": (None, [vp, ci, ci, cf]),
            "ora_mhc_prepost": (None, [vp, sz, sz, vp, vp, vp, cf, cf, ci, vp, vp, vp, vp]),
            "ora_mhc_collapse": (None, [vp, vp, vp, sz, sz]),
            "ora_mhc_apply": (None, [vp, vp, vp, vp, vp, sz, sz]),
            "ora_mhc_head": (None, [vp, sz, sz, vp, cf, vp, cf, cf, vp]),
            "ora_apply_rope": (None, [vp, vp, vp, ci, ci]),
            "ora_hadamard": (None, [vp, ci]),
            "ora_fp8_qat_sim": (None, [vp, sz, sz]),
            "ora_fp4_qat_sim": (None, [vp, sz]),
        }
        for n, (r, a) in sig.items():
            f = getattr(L, n)
            f.restype, f.argtypes = r, a
        _ora = L
    return _ora


def reference_dir():
    """Where the reference checkout lies when it is mounted: $APUS_REFERENCE, else a
    directory named `reference` beside this repository."""
    import os
    env = os.environ.get("APUS_REFERENCE")
    return Path(env) if env else ROOT.parent / "reference"


def ref():
    """The unmodified reference build, or None when it is not available."""
    global _ref
    if _ref is None:
        so = ORA_DIR / "_ref" / "libapus_ref.so"
        if not so.exists():
            if (reference_dir() / "c").exists():
                subprocess.check_call(["make", "-C", str(ORA_DIR), "ref"],
                                      stdout=subprocess.DEVNULL)
            else:
                return None
        L = C.CDLL(str(so))
        from apus_b200 import capi
        q = C.POINTER(capi.QW)
        sig = {
            "apus_bf16_round": (cf, [cf]), "apus_ue8m0_f32": (cf, [C.c_uint8]),
            "apus_e4m3_dequant_f32": (cf, [C.c_uint8]), "apus_e4m3_quant_f32": (C.c_uint8, [cf]),
            "apus_fp4_act_quant_scalar": (None, [vp, sz, vp, vp]),
            "ref_act_quant_rows": (None, [vp, vp, vp, vp, ci, ci]),
            "apus_fp4_gemm_mt": (None, [vp, vp, vp, vp, vp, vp, sz, sz, sz]),
            "apus_fp8_gemm_mt": (None, [vp, vp, vp, vp, vp, vp, sz, sz, sz]),
            "apus_fp4_gemm_scalar": (None, [vp, vp, vp, vp, vp, vp, sz, sz, sz]),
            "apus_fp8_gemm_scalar": (None, [vp, vp, vp, vp, vp, vp, sz, sz, sz]),
            "apus_fp4_linear": (None, [q, vp, vp, ci, ci, ci]),
            "apus_fp8_linear": (None, [q, vp, vp, ci, ci, ci]),
            "apus_bf16_linear": (None, [vp, vp, vp, ci, ci, ci]),
            "apus_f32_linear": (None, [vp, vp, vp, ci, ci, ci]),
            "apus_rms_norm": (None, [vp, vp, cf, vp, sz]),
            "apus_topk_stable": (None, [vp, ci, ci, vp]),
            "apus_router_score": (None, [C.POINTER(capi.MoeW), vp, ci, vp, vp]),
            "apus_moe_forward": (None, [C.POINTER(capi.MoeW), vp, vp, ci, vp,
                                        C.POINTER(capi.MoeInterm)]),
            "ref_expert": (None, [q, q, q, ci, cf, vp, ci, ci, vp]),
            "ref_expert_swiglu": (None, [vp, vp, vp, sz, cf]),
            "ref_sparse_attn": (None, [vp, vp, ci, ci, vp, ci, ci, cf, vp, i64, vp, vp]),
            "apus_mhc_sinkhorn": (None, [vp, sz, ci, cf]),
            "apus_apply_rope": (None, [vp, vp, vp, ci, ci]),
            "apus_hadamard": (None, [vp, ci]),
            "apus_fp8_qat_sim": (None, [vp, sz, sz]),
            "apus_fp4_qat_sim": (None, [vp, sz]),
            "apus_mhc_prepost_scalar": (None, [vp, sz, sz, vp, vp, vp, cf, cf, ci, vp, vp, vp, vp]),
            "apus_mhc_collapse_scalar": (None, [vp, vp, vp, sz, sz]),
            "apus_mhc_apply_scalar": (None, [vp, vp, vp, vp, vp, sz, sz]),
            "apus_mhc_head_scalar": (None, [vp, sz, sz, vp, cf, vp, cf, cf, vp, vp]),
            "ref_avx2_hits": (C.c_uint64, []), "ref_pool_threads": (ci, []),
        }
        for n, (r, a) in sig.items():
            f = getattr(L, n)
            f.restype, f.argtypes = r, a
        _ref = L
    return _ref


def oqw(codes, scales, O, K):
    return OraQW(P(codes), P(scales), int(O), int(K))


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / den) if den else float(np.linalg.norm(a - b))


# ---- oracle front-ends on numpy arrays ------------------------------------------------
def ora_qlinear(kind, codes, scales, x, O):
    M, K = x.shape
    out = np.empty((M, O), np.float32)
    ora().ora_qlinear(kind, P(codes), P(scales), P(x), P(out), M, K, O)
    return out


def ora_act_quant(x):
    M, K = x.shape
    codes = np.empty((M, K), np.uint8)
    scales = np.empty((M, (K + 127) // 128), np.float32)
    ora().ora_act_quant(P(x), M, K, None, P(codes), P(scales))
    return codes, scales


def ora_expert(kind, w1, w2, w3, x, inter, limit):
    rows, dim = x.shape
    out = np.empty((rows, dim), np.float32)
    a, b, c = oqw(*w1, inter, dim), oqw(*w2, dim, inter), oqw(*w3, inter, dim)
    ora().ora_expert(C.byref(a), C.byref(b), C.byref(c), kind, limit, P(x), rows, dim, inter, P(out))
    return out


def ora_moe(W, x, ids=None):
    """ora_moe_forward on a synth.MoeWeights; returns out, idx, wgt, routed, shared."""
    s = x.shape[0]
    E = W.E
    a1 = (OraQW * E)(*[oqw(W.w1p[e], W.w1s[e], W.inter, W.dim) for e in range(E)])
    a2 = (OraQW * E)(*[oqw(W.w2p[e], W.w2s[e], W.dim, W.inter) for e in range(E)])
    a3 = (OraQW * E)(*[oqw(W.w3p[e], W.w3s[e], W.inter, W.dim) for e in range(E)])
    s1, s2, s3 = oqw(*W.sw1, W.inter, W.dim), oqw(*W.sw2, W.dim, W.inter), oqw(*W.sw3, W.inter, W.dim)
    out = np.empty((s, W.dim), np.float32)
    idx = np.empty((s, W.topk), np.int32)
    wgt = np.empty((s, W.topk), np.float32)
    routed = np.empty((s, W.dim), np.float32)
    shared = np.empty((s, W.dim), np.float32)
    hash_ = W.tid2eid is not None
    ora().ora_moe_forward(E, W.topk, W.inter, W.dim, int(hash_), W.route_scale, W.limit,
                          P(W.gate_w), None if hash_ else P(W.gate_bias),
                          P(W.tid2eid) if hash_ else None,
                          C.cast(a1, vp), C.cast(a2, vp), C.cast(a3, vp),
                          C.byref(s1), C.byref(s2), C.byref(s3), P(x),
                          P(ids) if ids is not None else None, s, P(out), P(idx), P(wgt),
                          P(routed), P(shared))
    return out, idx, wgt, routed, shared
