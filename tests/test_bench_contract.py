"""The JSON line of bench.py: the reference arm runs on CPU (the reference's NumPy path on a
bounded sample), so its line can be checked here; the GPU arm's line is checked on the GPU box."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

BASE_KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
             "scaling", "vs_baseline", "dtype", "data", "config"}


def _last_json_line(stdout: str) -> dict:
    lines = [l for l in stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, stdout
    return json.loads(lines[0])


def test_reference_arm_prints_one_contract_line():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "0", "--workload", "bf16_smoke"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    line = _last_json_line(r.stdout)
    assert BASE_KEYS <= set(line)
    assert line["impl"] == "reference" and line["metric"] == "GEMM TFLOPS" and line["unit"] == "TFLOP/s"
    assert line["higher_is_better"] is True and line["vs_baseline"] is None
    assert line["value"] > 0 and line["n_gpus"] == 1 and line["steps"] == 1
    assert line["config"]["workload"] == "bf16_smoke"
    assert line["cpu_baseline"]["kind"] in ("port", "reference") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["e2e"]["value"] == line["value"]


@pytest.mark.gpu
def test_gpu_arm_prints_one_contract_line():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--steps", "5", "--warmup", "3", "--workload",
                        "bf16_smoke", "--e2e-steps", "2"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    line = _last_json_line(r.stdout)
    assert BASE_KEYS <= set(line)
    for key in ("roofline", "cpu_baseline", "e2e", "clocks", "gpu_launches"):
        assert key in line
    assert line["gpu_launches"] == 5 and line["warmup"] == 3 and line["steps"] == 5
    assert set(line["roofline"]) >= {"bound", "achieved", "peak", "unit", "frac", "traffic"}
    assert line["e2e"]["h2d_bytes_per_step"] > 0 and line["e2e"]["d2h_bytes_per_step"] > 0
    assert line["e2e"]["matches_device_path"] is True
    assert set(line["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}
