"""The C-ABI library loads and exports every symbol include/apus_b200.h declares
(no compute calls: this runs without a GPU)."""
import ctypes as C

import pytest

from apus_b200 import capi


def test_library_exports_every_declared_symbol():
    import apus_b200
    apus_b200.build()
    lib = C.CDLL(str(capi.LIB_PATH))
    names = capi.declared_symbols()
    assert len(names) >= 40
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_ctypes_signatures_cover_header():
    lib = capi.load()
    for n in capi.declared_symbols():
        assert getattr(lib, n).argtypes is not None, f"{n} has no ctypes signature"


def test_struct_layouts_match_reference():
    # c/st.h:88-89: two pointers + two int64; c/moe.h:37-63
    assert C.sizeof(capi.QW) == 32
    assert capi.MoeW.gate_w.offset == 32 and capi.MoeW.w1.offset == 56
    assert capi.MoeW.sw1.offset == 80 and capi.MoeW.hook_ctx.offset == 176
    assert C.sizeof(capi.MoeW) == 232
    assert C.sizeof(capi.Fp4GemmEnt) == 40


def test_no_gpu_calls_fail_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    lib = capi.load()
    err = C.create_string_buffer(256)
    assert lib.apus_cuda_enable(err, 256) != 0
    assert b"no CPU fallback" in err.value or b"CUDA" in err.value
