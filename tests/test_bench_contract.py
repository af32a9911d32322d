"""bench.py's output contract, on the CPU: the reference arm prints exactly one JSON
line on stdout (whatever libraries write while it runs goes to stderr), with the keys
the driver reads; ranks other than 0 of a multi-rank launch print nothing."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
BASE = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
        "vs_baseline", "dtype", "data", "config"}


def run(args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    p = subprocess.run([sys.executable, str(ROOT / "bench.py")] + args, capture_output=True, text=True, env=e,
                       timeout=600, cwd=str(ROOT))
    assert p.returncode == 0, p.stderr[-2000:]
    return p.stdout


def test_reference_arm_prints_one_json_line():
    out = run(["--impl", "reference", "--workload", "moe_layer", "--experts", "8", "--steps", "1", "--warmup", "0"])
    lines = [ln for ln in out.split("\n") if ln.strip()]
    assert len(lines) == 1, out
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    if "unavailable" in line:                       # no reference build on this machine
        assert isinstance(line["unavailable"], str) and line["unavailable"]
        return
    assert BASE <= set(line), sorted(BASE - set(line))
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["e2e"]["value"] == line["value"] and line["e2e"]["unit"] == line["unit"]
    cb = line["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["sample"] and cb["value"] == line["value"]
    assert line["config"]["workload"] and "model" not in line["config"]
    assert line["vs_baseline"] is None and line["higher_is_better"] is True


def test_other_ranks_of_the_reference_arm_stay_silent():
    out = run(["--impl", "reference", "--workload", "moe_layer", "--experts", "8", "--steps", "1", "--warmup", "0",
               "--gpus", "2"], env={"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert out.strip() == ""
