"""apus_b200 — B200 (sm_100a) backend for the apus DeepSeek-V4-Flash token loop.

The product is the C-ABI shared library ``libapus_b200.so`` built from
``csrc/`` (declared in ``include/apus_b200.h``).  This package is the thin host
side: it builds and loads the library, mirrors the reference's operator
interface for the MoE sublayer (``moe.py``) and generates synthetic inputs
(``synth.py``).  There is no CPU fallback: without the built library and a CUDA
device every operator raises.
"""
from . import capi, synth            # noqa: F401
from ._build import build            # noqa: F401

_lib = None


def lib():
    """The loaded backend (ctypes CDLL with typed signatures)."""
    global _lib
    if _lib is None:
        _lib = capi.load()
    return _lib


def check(rc, what="apus_cuda call"):
    """Raise with the library's message when a C-ABI call returned nonzero."""
    if rc != 0:
        msg = lib().apus_cuda_last_error()
        raise RuntimeError(f"{what} failed (rc={rc}): {msg.decode() if msg else '?'}")
