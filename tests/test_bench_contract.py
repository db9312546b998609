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
    assert "workloads" not in line          # a named workload is timed alone


@pytest.mark.gpu
def test_default_run_carries_every_workload_of_the_metric():
    """Without --workload the one line leads with BF16 8192^3 and carries a sub-record for NVFP4
    8192^3, the three decode shapes and the large BF16 GEMM, each with its own timing, roofline
    (with the algorithmic work `frac` is computed from), clocks and, for the FP4 ones, an
    end-to-end figure through the FP4 host-buffer context."""
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--steps", "20", "--warmup", "5", "--e2e-steps", "2",
                        "--no-cpu-baseline"], capture_output=True, text=True, timeout=1200)
    assert r.returncode == 0, r.stderr[-2000:]
    line = _last_json_line(r.stdout)
    assert line["config"]["workload"] == "bf16_8192" and line["steps"] == 20 and line["gpu_launches"] == 20
    subs = line["workloads"]
    assert set(subs) == {"nvfp4_8192", "decode_m16", "decode_m64", "decode_m128", "bf16_large"}
    for name, rec in subs.items():
        assert rec["ms_per_step"] > 0 and rec["steps"] >= 5 and rec["config"]["workload"] == name
        roof = rec["roofline"]
        assert set(roof) >= {"bound", "achieved", "peak", "unit", "frac", "traffic",
                             "algorithmic_flops_per_launch", "algorithmic_bytes_per_launch", "launch_ms"}
        work = roof["algorithmic_bytes_per_launch"] / 1e9 if roof["bound"] == "hbm" else roof["algorithmic_flops_per_launch"] / 1e12
        assert abs(work / (roof["launch_ms"] * 1e-3) / roof["achieved"] - 1) < 1e-6
        assert abs(roof["achieved"] / roof["peak"] / roof["frac"] - 1) < 1e-9
        assert set(rec["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}
        if name != "bf16_large":
            assert rec["e2e"]["matches_device_path"] is True and rec["e2e"]["h2d_bytes_per_step"] > 0
    assert subs["decode_m16"]["roofline"]["bound"] == "hbm" and subs["nvfp4_8192"]["roofline"]["bound"] == "tensor"


def test_both_arms_print_the_same_config():
    sys.path.insert(0, str(ROOT))
    import bench
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "0", "--workload", "bf16_smoke", "--gpus", "1"], capture_output=True, text=True, timeout=300)
    assert _last_json_line(r.stdout)["config"] == bench.config_for("bf16_smoke", 1)
    # The GPU arm builds its `config` from the same function (bench.measure); nothing else goes in.
    assert set(bench.config_for("bf16_8192", 8)) == {"workload", "description", "shape_mnk", "sharding"}


def test_reference_arm_ignores_a_one_thread_launcher_setting():
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its children; the CPU baseline must still
    use the cores the process may run on, and say how many."""
    import os
    env = dict(os.environ, OMP_NUM_THREADS="1", OPENBLAS_NUM_THREADS="1")
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "0", "--workload", "bf16_smoke"], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stderr
    line = _last_json_line(r.stdout)
    assert line["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))


def test_traffic_table_points_at_committed_profiles():
    """Every DRAM-traffic figure bench.py may report is keyed by a kernel configuration and names
    the ncu summary under profiles/ that holds it; the algorithmic bytes it is compared with are
    computed at run time."""
    sys.path.insert(0, str(ROOT))
    import bench
    for (workload, kernel), (nbytes, source) in bench.NCU_TRAFFIC.items():
        assert workload in bench.WORKLOADS and kernel
        text = (ROOT / source).read_text()
        mb = nbytes / 1e6
        assert f"{nbytes:,}".replace(",", " ") in text or str(nbytes) in text, (workload, source, mb)
        kind, m, n, k, fill, _ = bench.WORKLOADS[workload]
        algo = (m * k + n * k + m * n) * 2 if kind == "bf16" else n * k // 2 + n * k // 32 + m * k // 2 + m * k // 32 + 2 * m * n
        # Re-reads at most triple the minimum; the 5 GB problem, whose operands cannot stay in L2, is
        # recorded as measured (nine times its operands, see its profile summary).
        assert 0.9 <= nbytes / algo <= (9.0 if workload == "bf16_large" else 3.0), (workload, nbytes / algo)


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
