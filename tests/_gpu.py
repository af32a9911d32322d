"""Helpers for the GPU parity tests: every call goes through the C ABI."""
import ctypes as C

import numpy as np

import apus_b200
from apus_b200 import capi

P = capi.ptr


def lib():
    L = apus_b200.lib()
    err = C.create_string_buffer(512)
    if L.apus_cuda_enable(err, 512) != 0:
        raise RuntimeError("apus_cuda_enable: " + err.value.decode())
    return L


def ok(rc, what):
    apus_b200.check(rc, what)


def cuda_qlinear(fmt, codes, scales, x, O):
    M, K = x.shape
    out = np.empty((M, O), np.float32)
    w = capi.qw(codes, scales, O, K)
    fn = lib().apus_cuda_fp4_linear if fmt == 4 else lib().apus_cuda_fp8_linear
    ok(fn(C.byref(w), P(x), P(out), M, K, O), "qlinear")
    lib().apus_cuda_forget(P(codes))      # numpy may reuse this address for other weights
    return out


def cuda_qgemm(fmt, codes, scales, acodes, ascales, O):
    M, K = acodes.shape
    out = np.empty((M, O), np.float32)
    fn = lib().apus_cuda_fp4_gemm if fmt == 4 else lib().apus_cuda_fp8_gemm
    ok(fn(P(codes), P(scales), P(acodes), P(ascales), P(out), M, O, K), "qgemm")
    lib().apus_cuda_forget(P(codes))
    return out


def cuda_act_quant(x):
    M, K = x.shape
    codes = np.empty((M, K), np.uint8)
    scales = np.empty((M, K // 128), np.float32)
    ok(lib().apus_cuda_fp8_act_quant(P(x), M, K, P(codes), P(scales)), "act_quant")
    return codes, scales


def cuda_expert(kind, w1, w2, w3, x, inter, limit):
    rows, dim = x.shape
    out = np.empty((rows, dim), np.float32)
    a, b, c = capi.qw(*w1, inter, dim), capi.qw(*w2, dim, inter), capi.qw(*w3, inter, dim)
    ok(lib().apus_cuda_expert(C.byref(a), C.byref(b), C.byref(c), kind, limit, P(x), rows, dim,
                              inter, P(out)), "expert")
    for w in (w1, w2, w3):
        lib().apus_cuda_forget(P(w[0]))
    return out


def cuda_moe(W, x, ids=None, want_interm=True):
    s = x.shape[0]
    w = W.moew()
    out = np.empty((s, W.dim), np.float32)
    r = dict(sp=np.empty((s, W.E), np.float32), biased=np.zeros((s, W.E), np.float32),
             w=np.empty((s, W.topk), np.float32), idx=np.empty((s, W.topk), np.int32),
             routed=np.empty((s, W.dim), np.float32), shared=np.empty((s, W.dim), np.float32))
    it = capi.MoeInterm(P(r["sp"]), P(r["biased"]), P(r["w"]), P(r["idx"]), P(r["routed"]), P(r["shared"]))
    ok(lib().apus_cuda_moe_forward(C.byref(w), P(x), P(ids) if ids is not None else None, s, P(out),
                                   C.byref(it) if want_interm else None), "moe_forward")
    lib().apus_cuda_forget(P(W.gate_w))
    r["out"] = out
    return r


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def bf16_ulps(a, b):
    """Distance in BF16 steps between two BF16-valued f32 arrays."""
    ia = (bits(a) >> 16).astype(np.int64)
    ib = (bits(b) >> 16).astype(np.int64)
    sa = np.where(ia & 0x8000, 0x8000 - ia, ia)
    sb = np.where(ib & 0x8000, 0x8000 - ib, ib)
    return np.abs(sa - sb)
