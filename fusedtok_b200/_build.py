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


# The self-checking variant (tests/test_bounds_build_gpu.py): same sources with -DFTK_BOUNDS.
BOUNDS_LIB = os.path.join(HERE, "libfusedtok_b200_bounds.so")


def stale(target=None):
    target = target or LIB
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def _command(defines, target, verbose=False):
    cmd = ["nvcc"] + NVCC_FLAGS + ["-D" + d for d in defines]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    return cmd + [os.path.join(CSRC, s) for s in SOURCES] + ["-o", target]


def build_all(force=False):
    """The product and the self-checking variant, whichever is out of date, compiled side by side (each
    is one long nvcc run)."""
    jobs = [(t, subprocess.Popen(_command(d, t))) for d, t in (((), LIB), (("FTK_BOUNDS",), BOUNDS_LIB))
            if force or stale(t)]
    failed = [t for t, job in jobs if job.wait() != 0]
    if failed:
        raise RuntimeError("nvcc failed for " + ", ".join(failed))
    return LIB


def build(force=False, verbose=False, defines=(), out=None):
    """Compile the library. `defines` / `out` produce a variant build next to the product (for example
    ``defines=["FTK_TIMELINE"]``: per-CTA timestamps in the tensor-core decode kernel, read back with
    ``ftk_debug_timeline``); the product itself is always built without defines."""
    target = out or LIB
    if not force and not defines and not stale():
        return LIB
    subprocess.check_call(_command(defines, target, verbose))
    return target


if __name__ == "__main__":
    # python fusedtok_b200/_build.py [--force] [-v] [-DNAME ...] [--out path] | --all
    if "--all" in sys.argv:
        print(build_all(force="--force" in sys.argv))
        sys.exit(0)
    defs = [a[2:] for a in sys.argv[1:] if a.startswith("-D")]
    out_path = sys.argv[sys.argv.index("--out") + 1] if "--out" in sys.argv else None
    if defs and not out_path:
        raise SystemExit("a build with -D defines needs --out: the product library is built without defines")
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, defines=defs, out=out_path))
