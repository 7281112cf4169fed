"""In-tree build of the CUDA library (sm_100a only).

``python fusedtok_b200/_build.py`` compiles ``csrc/fusedtok_b200.cu`` into
``fusedtok_b200/libfusedtok_b200.so`` with nvcc. The library is the whole
product: there is no other backend and no CPU fallback, so importing the
package without it fails.
"""

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libfusedtok_b200.so")
SOURCES = ["fusedtok_b200.cu"]
HEADERS = sorted(f for f in os.listdir(CSRC) if f.endswith(".cuh")) + [
    os.path.join("..", "..", "include", "fusedtok_b200.h")]

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared", "-cudart", "static",
]


def stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False, defines=(), out=None):
    """Compile the library. `defines` / `out` produce a variant build next to the product (for example
    ``defines=["FTK_TIMELINE"]``: per-CTA timestamps in the tensor-core decode kernel, read back with
    ``ftk_debug_timeline``); the product itself is always built without defines."""
    target = out or LIB
    if not force and not defines and not stale():
        return LIB
    cmd = ["nvcc"] + NVCC_FLAGS + ["-D" + d for d in defines]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES] + ["-o", target]
    subprocess.check_call(cmd)
    return target


if __name__ == "__main__":
    # python fusedtok_b200/_build.py [--force] [-v] [-DNAME ...] [--out path]
    defs = [a[2:] for a in sys.argv[1:] if a.startswith("-D")]
    out_path = sys.argv[sys.argv.index("--out") + 1] if "--out" in sys.argv else None
    if defs and not out_path:
        raise SystemExit("a build with -D defines needs --out: the product library is built without defines")
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, defines=defs, out=out_path))
