"""Builds libapus_b200.so from csrc/*.cu with nvcc for sm_100a (in-tree)."""
import os
import shutil
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OUT = ROOT / "libapus_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
    "-std=c++17", "-Xcompiler", "-fPIC", "--use_fast_math=false",
    "-Xptxas", "-v", "-I", str(ROOT.parent / "include"),
]


def _stale(target, sources):
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources)


def build(force=False, verbose=False):
    """Compile every csrc/*.cu to an object and link the shared library.

    Returns the path of the library.  Incremental: an object is rebuilt only
    when its source or a header changed."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        if OUT.exists():
            return OUT            # prebuilt library travelled with the tree
        raise RuntimeError("nvcc not found and no prebuilt libapus_b200.so")
    objdir = ROOT / "build"
    objdir.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + \
        list((ROOT.parent / "include").glob("*.h"))
    objs = []
    logs = []
    procs = []
    for src in sorted(CSRC.glob("*.cu")):
        obj = objdir / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc] + [f for f in NVCC_FLAGS if f != "--use_fast_math=false"] + \
                ["-c", str(src), "-o", str(obj)]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE,
                                                stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        logs.append(f"== {src.name}\n{out}")
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{out}")
    if force or _stale(OUT, objs):
        cmd = [nvcc, "-shared", "-o", str(OUT)] + [str(o) for o in objs] + \
            ["-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}")
    (objdir / "ptxas.log").write_text("\n".join(logs)) if logs else None
    if verbose:
        print("\n".join(logs))
    return OUT
