"""Expert parallelism on real NCCL: two ranks, two GPUs (skipped with fewer)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent


def test_two_gpu_expert_parallel_tokens_equal_one_gpu(tmp_path):
    """The expert-parallel loop over two GPUs (NCCL all-to-all dispatch / combine, the steps
    replayed from a CUDA graph) emits, for every sequence of the job, exactly the tokens
    the one-GPU loop emits for it (tests/ep2_worker.py)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = tmp_path / "ep2.json"
    env = dict(os.environ, NCCL_DEBUG="WARN")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29617", str(HERE / "ep2_worker.py"), str(out)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.loads(out.read_text())
    assert res["equal"], res
