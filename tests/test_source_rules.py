"""A source-level invariant of the CUDA sources that no compiler checks.

Every kernel launched through launch_k (programmatic dependent launch, csrc/common.cuh) must execute
APUS_PDL_WAIT before it touches global memory: without it the kernel may start while the kernel before it
on the stream is still writing its inputs.  The test finds the kernels named at launch_k call sites and
checks that each one's body has the wait among its first statements.
"""
import re
from pathlib import Path

SRC = Path(__file__).resolve().parent.parent / "apus-deepseek-v4-flash_b200" / "csrc"
FILES = sorted(SRC.glob("*.cu")) + sorted(SRC.glob("*.cuh"))


def kernel_bodies(text):
    """{kernel name: body text} of every __global__ function defined in `text`."""
    out = {}
    for m in re.finditer(r"__global__", text):
        # walk to the body's opening brace; the name is the identifier before the last top-level "(...)" group
        k, depth, name, last_word = m.end(), 0, None, None
        while k < len(text):
            c = text[k]
            if c == "(":
                if depth == 0:
                    name = last_word
                depth += 1
            elif c == ")":
                depth -= 1
            elif depth == 0 and c in ";{":
                break
            elif depth == 0:
                w = re.match(r"[A-Za-z_]\w*", text[k:])
                if w:
                    last_word = w.group(0)
                    k += len(last_word)
                    continue
            k += 1
        if k >= len(text) or text[k] != "{" or not name:
            continue                                   # a declaration
        depth, e = 0, k
        while e < len(text):
            depth += text[e] == "{"
            depth -= text[e] == "}"
            if depth == 0:
                break
            e += 1
        out[name] = text[k:e + 1]
    return out


def test_kernels_launched_programmatically_wait_first():
    bodies, launched = {}, set()
    for f in FILES:
        t = f.read_text()
        bodies.update(kernel_bodies(t))
        launched |= set(re.findall(r"launch_k\(\s*(\w+)", t))
        for m in re.finditer(r"auto\s+(\w+)\s*=\s*(\w+)<", t):          # auto kern = kernel<...>; launch_k(kern, ...)
            if m.group(1) in launched:
                launched.add(m.group(2))
    launched -= {"kern", "kernel", "void"}
    assert len(launched) > 40, sorted(launched)
    missing = [k for k in sorted(launched) if k in bodies and "APUS_PDL_WAIT()" not in bodies[k][:400]]
    unknown = [k for k in sorted(launched) if k not in bodies]
    assert not missing, f"launched with launch_k but no APUS_PDL_WAIT at the top: {missing}"
    assert not unknown, f"launch_k names no kernel defined in csrc/: {unknown}"
