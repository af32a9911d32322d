import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))
os.environ.setdefault("APUS_THREADS", str(min(os.cpu_count() or 1, 16)))
# The parity tests written against the reference's bits run the long f32 sums in the
# reference's loop order; the tests of the default (tree / tensor-core) order select it
# themselves with apus_cuda_set_tree_ops (tests/test_gpu_flash_parity.py and others).
os.environ.setdefault("APUS_TREE_OPS", "0")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this environment")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)
