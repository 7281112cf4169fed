"""Build recipe for the CPU oracle (TEST INFRASTRUCTURE ONLY).

Two artefacts, both used only by the tests, the smoke check and the
benchmark's CPU-baseline leg - never by the shipped package:

* ``oracle/liboracle.so``  - gcc build of ``attention_oracle.c`` (the plain-C
  restatement of the reference's CPU decode attention).
* ``oracle/_ref/libfusedtok_ref.so`` - the reference's OWN implementation:
  nvcc compiles the reference's ``src/attention.cu`` and ``src/rope.cu`` where they lie in the
  reference checkout (nothing is copied) together with ``ref_shim.cpp``, a
  C-ABI shim. It carries the reference's CPU functions (the parity pin) and
  its GPU launchers (timed beside ours). Only built when a reference checkout
  is present; the prebuilt file travels with the repository snapshot.

The reference checkout is found through the environment variable
``FUSEDTOK_REFERENCE_DIR`` or, when that is unset, as a directory named
``reference`` beside this repository. ``python oracle/build_oracle.py --ref``
fails with a message if neither exists.

Run ``python oracle/build_oracle.py`` (``--force`` rebuilds).
"""

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.environ.get("FUSEDTOK_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libfusedtok_ref.so")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(s) and os.path.getmtime(s) > t for s in sources)


def build_oracle(force=False):
    """gcc -O2, no fast-math and no FMA contraction: the summation order and
    rounding must match the reference's host code."""
    src = os.path.join(HERE, "attention_oracle.c")
    if force or _stale(ORACLE_SO, [src]):
        cmd = ["gcc", "-O2", "-std=c99", "-fPIC", "-shared", "-ffp-contract=off",
               "-o", ORACLE_SO, src, "-lm"]
        subprocess.check_call(cmd)
    return ORACLE_SO


def reference_present():
    return os.path.exists(os.path.join(REF_DIR, "src", "attention.cu"))


def build_ref(force=False):
    """Compile the reference's attention.cu in place plus the shim. Returns
    the path, or None when no reference checkout is available and no prebuilt
    library exists."""
    shim = os.path.join(HERE, "ref_shim.cpp")
    if not reference_present():
        return REF_SO if os.path.exists(REF_SO) else None
    ref_src = os.path.join(REF_DIR, "src", "attention.cu")
    rope_src = os.path.join(REF_DIR, "src", "rope.cu")
    if force or _stale(REF_SO, [shim, ref_src, rope_src]):
        os.makedirs(os.path.dirname(REF_SO), exist_ok=True)
        cmd = ["nvcc", "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
               "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
               "-I", os.path.join(REF_DIR, "include"),
               "-I", os.path.join(REF_DIR, "src"),
               "-x", "cu", ref_src, "-x", "cu", rope_src, "-x", "cu", shim, "-o", REF_SO]
        subprocess.check_call(cmd)
    return REF_SO


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_oracle(force))
    if "--ref" in sys.argv and not reference_present():
        raise SystemExit("no reference checkout: set FUSEDTOK_REFERENCE_DIR to fusedtok's source tree "
                         "(looked in %s)" % REF_DIR)
    print(build_ref(force))
