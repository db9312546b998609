"""Output files of this repository's drivers against output files of the reference's own GPU
drivers (built unchanged from the reference sources into oracle/_ref by oracle/Makefile), same
shape, same fill, on the same GPU.  Skipped where oracle/_ref has not been built.  Timings of both
sides are written to a JSON file for the record (SMB_AB_RECORD if set, else reference_ab.json
in the test's temporary folder); only parity is asserted."""
import json
import os
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
OURS = ROOT / "strata-masonry_b200" / "bin"
REF = ROOT / "oracle" / "_ref"
RESULTS = {}


def _run(exe, args, timeout=300):
    r = subprocess.run([str(exe), *args], capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    m = re.search(r"([0-9.]+) ms\s+([0-9.]+) (?:NVFP4_)?TFLOPS", r.stdout)
    return (float(m.group(1)), float(m.group(2))) if m else None


def _pair(kind, m, k, n, fill, tmp_path, benchmark):
    name = f"kernel_sm100a_dense_gemm_{kind}"
    if not (REF / name).exists():
        pytest.skip("oracle/_ref not built (reference tree not mounted at build time)")
    outs, times = [], []
    for side, exe in (("ref", REF / name), ("ours", OURS / name)):
        out = tmp_path / f"{side}.bf16"
        args = [f"--shape={m},{k},{n}", f"--fill={fill}", "--no-gpu-verify", f"--dump-output={out}"]
        if not benchmark:
            args.append("--no-benchmark")
        times.append(_run(exe, args))
        outs.append(np.fromfile(out, dtype="<u2").reshape(m, n))
    if benchmark and times[0] and times[1]:
        RESULTS[f"{kind} M={m} N={n} K={k} fill={fill}"] = {
            "reference_ms": times[0][0], "reference_tflops": times[0][1],
            "ours_ms": times[1][0], "ours_tflops": times[1][1]}
        record = Path(os.environ.get("SMB_AB_RECORD", str(tmp_path.parent / "reference_ab.json")))
        record.parent.mkdir(parents=True, exist_ok=True)
        record.write_text(json.dumps(RESULTS, indent=1))
    return outs


@pytest.mark.parametrize("fill", [1, 2, 3, 4])
def test_bf16_smoke_files_match_reference_kernel(oracle, cuda_device, tmp_path, fill):
    ref, ours = _pair("bf16", 256, 64, 128, fill, tmp_path, benchmark=False)
    # K = 64: four instructions per output tile on both sides; fp32 sums may differ in order.
    diff = np.abs(ref.astype(np.int32) - ours.astype(np.int32))
    assert diff.max() <= 1 and (diff == 0).mean() > 0.99
    ok, bad = oracle.check_verifier_bf16(ours, oracle.bf16_to_f32(ref))
    assert ok, bad


@pytest.mark.parametrize("fill", [1, 2, 3, 4])
def test_fp4_smoke_files_match_reference_kernel(oracle, cuda_device, tmp_path, fill):
    ref, ours = _pair("nvfp4", 256, 256, 128, fill, tmp_path, benchmark=False)
    if fill in (1, 3):
        np.testing.assert_array_equal(ref, ours)
    ok, bad = oracle.check_verifier_nvfp4(ours, oracle.bf16_to_f32(ref))
    assert ok, bad
    assert np.abs(ref.astype(np.int32) - ours.astype(np.int32)).max() <= 1


@pytest.mark.parametrize("shape", [(8192, 4096, 8192), (14080, 2048, 5120), (30720, 4096, 2048)])
def test_bf16_large_files_match_reference_kernel(oracle, cuda_device, tmp_path, shape):
    m, k, n = shape
    ref, ours = _pair("bf16", m, k, n, 2, tmp_path, benchmark=True)
    ok, bad = oracle.check_verifier_bf16(ours, oracle.bf16_to_f32(ref))
    assert ok, bad
    diff = np.abs(ref.astype(np.int32) - ours.astype(np.int32))
    assert (diff <= 1).mean() > 0.999


@pytest.mark.parametrize("shape", [(8192, 8192, 8192), (30720, 8192, 4096)])
def test_fp4_large_files_match_reference_kernel(oracle, cuda_device, tmp_path, shape):
    m, k, n = shape
    ref, ours = _pair("nvfp4", m, k, n, 2, tmp_path, benchmark=True)
    ok, bad = oracle.check_verifier_nvfp4(ours, oracle.bf16_to_f32(ref))
    assert ok, bad
