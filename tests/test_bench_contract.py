"""The JSON line of bench.py carries the keys its readers rely on (both arms)."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

BASE_KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
             "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches"}


def _run(*args, timeout=600):
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True,
                         timeout=timeout, cwd=str(ROOT))
    assert res.returncode == 0, res.stdout + res.stderr
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, "exactly one JSON line"
    return json.loads(lines[0])


def test_reference_arm_prints_the_contract_line_without_a_gpu():
    line = _run("--impl", "reference", "--config", "c1", "--steps", "1", "--warmup", "1")
    assert BASE_KEYS <= set(line) and line["impl"] == "reference"
    assert line["metric"] == "decode_attention_kv_GBps" and line["unit"] == "GB/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["gpu_launches"] == 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"] and "sample" in line["cpu_baseline"]
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in line["config"] and "BASELINE config 1" in line["config"]["workload"]


@pytest.mark.gpu
def test_our_arm_prints_the_contract_line(cuda_device):
    line = _run("--config", "c1", "--steps", "3", "--warmup", "3", "--min-seconds", "0.02", "--no-variants")
    assert BASE_KEYS | {"roofline", "cpu_baseline", "clocks", "errors", "calls_per_step"} <= set(line)
    assert "impl" not in line and line["n_gpus"] == 1 and line["value"] > 0
    roof = line["roofline"]
    assert roof["bound"] == "hbm" and roof["unit"] == "GB/s" and roof["peak"] > 0
    assert abs(roof["frac"] - roof["achieved"] / roof["peak"]) < 1e-3
    assert {"traffic", "errors", "variants", "kernel_us"} <= set(roof)
    assert line["errors"]["within_tol"] is True and roof["errors"]["e2e_within_tol"] is True
    e2e = line["e2e"]
    assert e2e["value"] > 0 and e2e["h2d_bytes_per_step"] > 0 and e2e["d2h_bytes_per_step"] > 0
    assert e2e["value"] < line["value"]  # host buffers in and out cost something
    assert line["gpu_launches"] == line["steps"] * line["calls_per_step"]  # one kernel per loop call
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["value"] > 0
    assert set(line["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}
