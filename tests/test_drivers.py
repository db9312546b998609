"""The two command-line drivers: the reference executables' contract (flags, stdout lines, dump
file, exit codes).  Argument handling is checked on the CPU; the full flow needs a GPU."""
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "strata-masonry_b200" / "bin"
BF16 = BIN / "kernel_sm100a_dense_gemm_bf16"
FP4 = BIN / "kernel_sm100a_dense_gemm_nvfp4"


def _run(exe, *args, env=None):
    return subprocess.run([str(exe), *args], capture_output=True, text=True, timeout=600, env=env)


@pytest.fixture(scope="module", autouse=True)
def _built(smb):
    assert BF16.exists() and FP4.exists(), "drivers not built (python strata-masonry_b200/build.py)"


def test_bf16_driver_rejects_bad_arguments():
    assert _run(BF16, "--bogus").returncode == 1
    r = _run(BF16, "--fill=9")
    assert r.returncode == 1 and "--fill must be" in r.stderr
    r = _run(BF16, "--shape=256,64")
    assert r.returncode == 1 and "--shape must be M,K,N" in r.stderr


def test_fp4_driver_rejects_bad_arguments():
    r = _run(FP4, "--bogus")
    assert r.returncode == 1 and "unknown or empty argument" in r.stderr
    assert _run(FP4, "--fill=0").returncode == 1
    assert _run(FP4, "--shape=256,256,0").returncode == 1
    assert _run(FP4, "--dump-output=").returncode == 1
    r = _run(FP4, "--shape=256,100,128")
    assert r.returncode == 1 and "multiple of 32" in r.stderr
    r = _run(FP4, "--help")
    assert r.returncode == 0 and "Usage" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("fill", [1, 2])
def test_bf16_driver_smoke_flow(oracle, golden, cuda_device, tmp_path, fill):
    """README flow of the reference: run --shape=256,64,128, dump, check the file as the reference
    verifier does (size, its sample coordinates, fp32 reference, max(0.05, 0.05 |ref|))."""
    out = tmp_path / "gemm-smoke.bf16"
    r = _run(BF16, "--shape=256,64,128", f"--fill={fill}", "--no-benchmark", "--no-gpu-verify",
             f"--dump-output={out}")
    assert r.returncode == 0, r.stderr
    assert "K0 dense_gemm_bf16" in r.stdout
    assert "shape (   256,    128,   64): untimed" in r.stdout
    assert f"wrote 32768 BF16 values to {out}" in r.stdout
    data = np.fromfile(out, dtype="<u2")
    assert data.size == 256 * 128
    rows, cols = oracle.sample_coordinates(256, 128, 64)
    want = oracle.bf16_to_f32(golden[f"bf16_smoke_out_m{fill}"])
    ok, bad = oracle.check_verifier_bf16(data.reshape(256, 128)[rows, cols], want[rows, cols])
    assert ok, bad
    ok, bad = oracle.check_verifier_bf16(data.reshape(256, 128), want)
    assert ok, bad


@pytest.mark.gpu
def test_bf16_driver_benchmark_and_self_check(cuda_device, tmp_path):
    js = tmp_path / "r.json"
    r = _run(BF16, "--shape=1024,512,768", "--fill=5", f"--json={js}")
    assert r.returncode == 0, r.stderr
    assert " ms " in r.stdout and "TFLOPS" in r.stdout
    assert "verify (M=1024,N=768,K=512)" in r.stdout and "tight=OK" in r.stdout
    assert js.exists()
    r = _run(BF16, "--shape=512,256,384", "--raster=along-m")
    assert r.returncode == 0 and "tight=OK" in r.stdout
    assert _run(BF16, "--dump-output=/tmp/x.bf16").returncode == 1
    assert _run(BF16, "--shape=256,60,128").returncode == 1


@pytest.mark.gpu
@pytest.mark.parametrize("fill", [1, 2, 3, 4])
def test_fp4_driver_smoke_flow(oracle, golden, cuda_device, tmp_path, fill):
    out = tmp_path / "nvfp4-smoke.bf16"
    r = _run(FP4, "--shape=256,256,128", f"--fill={fill}", "--no-benchmark", f"--dump-output={out}")
    assert r.returncode == 0, r.stdout + r.stderr
    assert "K1 dense_gemm_nvfp4" in r.stdout
    assert "untimed" in r.stdout and "OK" in r.stdout
    data = np.fromfile(out, dtype="<u2")
    assert data.size == 256 * 128
    want = oracle.bf16_to_f32(golden[f"fp4_smoke_out_m{fill}"])
    ok, bad = oracle.check_verifier_nvfp4(data.reshape(256, 128), want)
    assert ok, bad


@pytest.mark.gpu
def test_fp4_driver_benchmark_line_and_env_fill(cuda_device):
    import os
    r = _run(FP4, "--shape=1024,1024,1024", "--fill=5")
    assert r.returncode == 0, r.stdout + r.stderr
    assert "mean=" in r.stdout and "NVFP4_TFLOPS" in r.stdout
    assert "sampled ref x2048): fail=0 nan=0 OK" in r.stdout
    env = dict(os.environ, FILL="3")
    r = _run(FP4, "--shape=512,512,256", "--no-benchmark", env=env)
    assert r.returncode == 0 and "(real scales): max_rel=0.00e+00 nan=0 OK" in r.stdout


def test_drivers_reject_bad_shards():
    r = _run(BF16, "--shard=2/2", "--shape=256,64,128")
    assert r.returncode == 1 and "--shard must be RANK/WORLD" in r.stderr
    r = _run(FP4, "--shard=x", "--shape=256,64,128")
    assert r.returncode == 1 and "--shard must be RANK/WORLD" in r.stderr
    assert _run(BF16, "--device=-1").returncode == 1


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["bf16", "fp4"])
def test_sharded_driver_slabs_make_up_the_unsharded_output(cuda_device, tmp_path, which):
    """--shard=RANK/WORLD: each process computes the column slab of its rank from operands generated
    with global indices; the slabs side by side are the single-process dump bit for bit (here the
    ranks run one after the other on the same GPU).  A split that breaks 16-byte rows is refused."""
    exe = BF16 if which == "bf16" else FP4
    m, k, n, world = 512, 256, 768, 3
    whole = tmp_path / "whole.bf16"
    r = _run(exe, f"--shape={m},{k},{n}", "--fill=2", "--no-benchmark", f"--dump-output={whole}")
    assert r.returncode == 0, r.stderr + r.stdout
    want = np.fromfile(whole, dtype="<u2").reshape(m, n)
    slabs = []
    for rank in range(world):
        out = tmp_path / f"slab{rank}.bf16"
        r = _run(exe, f"--shape={m},{k},{n}", "--fill=2", "--no-benchmark", f"--shard={rank}/{world}",
                 "--device=0", f"--dump-output={out}")
        assert r.returncode == 0, r.stderr + r.stdout
        lo, hi = rank * n // world, (rank + 1) * n // world
        assert f"shard {rank}/{world}: columns [{lo}, {hi}) of N={n} on device 0" in r.stdout
        assert "OK" in r.stdout   # the driver's own check ran on the slab
        slabs.append(np.fromfile(out, dtype="<u2").reshape(m, n // world))
    assert np.array_equal(np.concatenate(slabs, axis=1), want)
    r = _run(exe, f"--shape={m},{k},{n}", "--shard=0/5")
    assert r.returncode == 1 and "unsupported --shard" in r.stderr


def test_drivers_reject_bad_box_options():
    r = _run(BF16, "--allgather", "--shape=256,64,128")
    assert r.returncode == 1 and "--allgather requires --gpus" in r.stderr
    r = _run(FP4, "--gpus=0", "--shape=256,256,128")
    assert r.returncode == 1 and "--gpus must be" in r.stderr
    r = _run(BF16, "--gpus=2", "--shard=0/2", "--shape=256,64,128")
    assert r.returncode == 1 and "exclude each other" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["bf16", "fp4"])
@pytest.mark.parametrize("gpus", [1, 2])
def test_box_mode_gathers_the_unsharded_output(cuda_device, tmp_path, which, gpus):
    """--gpus=G --allgather: one process drives G devices, every device computes its column slab,
    the slabs are exchanged with the library's NCCL all-gather and unshard copy, and the dump of
    the gathered D is the single-GPU dump bit for bit.  Without --allgather the dump is assembled
    from the slabs on the host and must be the same file."""
    import torch
    if torch.cuda.device_count() < gpus:
        pytest.skip(f"needs {gpus} GPUs")
    exe = BF16 if which == "bf16" else FP4
    m, k, n = 512, 256, 768
    whole = tmp_path / "whole.bf16"
    r = _run(exe, f"--shape={m},{k},{n}", "--fill=2", "--no-benchmark", f"--dump-output={whole}")
    assert r.returncode == 0, r.stderr + r.stdout
    want = np.fromfile(whole, dtype="<u2")
    for extra in (["--allgather"], []):
        out = tmp_path / f"box{len(extra)}.bf16"
        r = _run(exe, f"--shape={m},{k},{n}", "--fill=2", f"--gpus={gpus}", *extra, f"--dump-output={out}")
        assert r.returncode == 0, r.stderr + r.stdout
        assert f"box of {gpus} GPUs" in r.stdout and "OK" in r.stdout
        if extra:
            assert f"all-gather of D over {gpus} GPUs" in r.stdout
        assert np.array_equal(np.fromfile(out, dtype="<u2"), want)
