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


def test_cpu_baseline_helpers():
    """The pieces of the CPU baseline that need no GPU: the BLAS description, and the block-scaled
    sample (codes and scale bytes -> fp32 -> matmul) on a budget small enough for a unit test, with
    the few-row proportion of a decode workload kept."""
    sys.path.insert(0, str(ROOT))
    import bench
    threads, blas = bench.blas_info()
    assert threads >= 1 and isinstance(blas, str) and blas
    oracle = bench._load_oracle()
    rate, sample, secs = bench.cpu_fp4_rate(oracle, 16, 28672, 512, budget_s=0.05)
    assert rate > 0 and secs > 0 and sample.startswith("16x") and sample.split("x")[2].startswith("512")
    rate, sample, secs = bench.cpu_fp4_rate(oracle, 8192, 8192, 256, budget_s=0.05)
    rows, cols = int(sample.split("x")[0]), int(sample.split("x")[1])
    assert rate > 0 and rows >= 16 and cols >= 128


def test_reference_arm_of_a_block_scaled_workload():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "0", "--workload", "decode_m16"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    line = _last_json_line(r.stdout)
    assert line["impl"] == "reference" and line["dtype"] == "e2m1" and line["value"] > 0
    assert "blas" in line["cpu_baseline"] and line["cpu_baseline"]["cores"] >= 1
