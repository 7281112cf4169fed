"""bench.py's reference arm runs on host cores only: its JSON line can be checked without a GPU."""

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*flags):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + list(flags), capture_output=True, text=True,
                         timeout=240, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    return json.loads(out.stdout.strip().splitlines()[-1])


@pytest.mark.parametrize("workload,metric,unit", [("c2", "decode_attn_kv_read_GBps", "GB/s"),
                                                  ("pf_ref", "prefill_attn_TFLOPs", "TFLOP/s")])
def test_reference_arm_line(workload, metric, unit):
    d = run_bench("--impl", "reference", "--workload", workload, "--steps", "1", "--warmup", "0")
    assert d["impl"] == "reference" and d["metric"] == metric and d["unit"] == unit
    assert d["higher_is_better"] is True and d["value"] > 0 and d["steps"] == 1 and d["n_gpus"] == 1
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["cpu_baseline"]["value"] == d["value"] and d["cpu_baseline"]["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["gpu_launches"] == 0 and "workload" in d["config"]
