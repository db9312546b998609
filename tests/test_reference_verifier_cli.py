"""The reference's own verifier command lines, unchanged, on output files this repository's drivers
wrote on a B200 (tests/golden/gpu_dumps).  Runs only where the reference tree is mounted."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
DUMPS = ROOT / "tests" / "golden" / "gpu_dumps"
GEMM = Path(os.environ.get("SMB_REFERENCE_DIR", "/root/reference")) / "src" / "kernels" / "gemm" / "sm100a"
VERIFIERS = {"bf16": GEMM / "dense_gemm_bf16_cpu_verifier.py",
             "nvfp4": GEMM / "nvfp4" / "dense_gemm_nvfp4_cpu_verifier.py"}


@pytest.mark.parametrize("kind", ["bf16", "nvfp4"])
@pytest.mark.parametrize("fill", [1, 2, 3, 4])
def test_unchanged_reference_verifier_accepts_gpu_dump(kind, fill):
    verifier = VERIFIERS[kind]
    if not verifier.exists():
        pytest.skip("reference tree not mounted")
    dump = DUMPS / f"{kind}_smoke_f{fill}.bf16"
    assert dump.stat().st_size == 256 * 128 * 2
    # --samples larger than M*N makes the verifier check every element, not its default sample.
    r = subprocess.run([sys.executable, str(verifier), "verify", "--case", "smoke", "--fill", str(fill),
                        "--samples", "40000", "--actual", str(dump)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    result = json.loads(r.stdout)
    assert result["passed"] is True and result["mismatches"] == 0 and result["samples"] == 256 * 128


@pytest.mark.parametrize("kind", ["bf16", "nvfp4"])
def test_unchanged_reference_verifier_rejects_wrong_size(kind, tmp_path):
    verifier = VERIFIERS[kind]
    if not verifier.exists():
        pytest.skip("reference tree not mounted")
    bad = tmp_path / "short.bf16"
    bad.write_bytes(b"\0" * 100)
    r = subprocess.run([sys.executable, str(verifier), "verify", "--case", "smoke", "--actual", str(bad)],
                       capture_output=True, text=True, timeout=60)
    assert r.returncode == 2
