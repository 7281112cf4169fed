"""The reference's own attention test files, run unmodified against this library (through the tests-only
``fusedtok`` package under tests/shim, which forwards to ``fusedtok_b200``).

Needs a checkout of the reference (``FUSEDTOK_REFERENCE_DIR``, or a directory named ``reference`` beside this
repository); skipped where there is none. On a machine without a GPU the reference's files skip their GPU
classes themselves, so what runs is every host-route case: shapes, GQA mapping, lens handling, paged layout and
the whole error contract of ``attention_decode`` / ``attention_decode_paged`` / ``attention_prefill``, with this
library's wrappers doing the validation and the CPU oracle doing the arithmetic the reference does on the CPU.
The GPU classes of those files are mirrored, case by case, by tests/test_decode_gpu.py, test_paged_gpu.py,
test_prefill.py and test_validation_gpu.py.
"""

import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("FUSEDTOK_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
FILES = [os.path.join(REF, "tests", name) for name in ("test_attention.py", "test_attention_paged.py")]


@pytest.mark.skipif(not all(os.path.exists(f) for f in FILES), reason="no reference checkout on this machine")
def test_reference_attention_suites_pass_against_this_library(tmp_path):
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([os.path.join(ROOT, "tests", "shim"), ROOT, os.path.join(ROOT, "tests")])
    env["CUDA_VISIBLE_DEVICES"] = ""          # host routes only: the GPU classes are mirrored elsewhere
    cmd = [sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider", "--rootdir", str(tmp_path)] + FILES
    res = subprocess.run(cmd, env=env, cwd=str(tmp_path), capture_output=True, text=True, timeout=900)
    tail = res.stdout.strip().splitlines()[-1] if res.stdout.strip() else res.stderr[-500:]
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-1000:]
    passed = int(re.search(r"(\d+) passed", tail).group(1))
    assert "failed" not in tail and "error" not in tail, tail
    assert passed >= 35, tail             # every host-route case of the two files
