"""Build the sm_100a shared library and the two reference-compatible drivers with nvcc.

Usage:  python strata-masonry_b200/build.py [--force] [--verbose]

Outputs (all ignored by git, all next to this file):
  lib/libstrata_masonry_b200.so          the C-ABI library
  bin/kernel_sm100a_dense_gemm_bf16      drop-in for the reference driver of that name
  bin/kernel_sm100a_dense_gemm_nvfp4     drop-in for the reference driver of that name
  build/*.o, build/ptxas.log             objects and the -Xptxas -v resource report

Target names follow the reference build (CMakeLists.txt:104-113 there).
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "build"
LIB = HERE / "lib" / "libstrata_masonry_b200.so"
BIN = HERE / "bin"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
          "--expt-relaxed-constexpr"]

LIB_SOURCES = ["runtime.cu", "fills.cu", "gemm_bf16.cu", "gemm_bf16_streamk.cu", "api_bf16.cu", "gemm_nvfp4.cu",
               "gemm_nvfp4_arun.cu", "gemm_nvfp4_decode.cu", "api_nvfp4.cu", "peer.cu", "gather.cu", "selftest.cu"]
DRIVERS = {"kernel_sm100a_dense_gemm_bf16": "driver_bf16.cu",
           "kernel_sm100a_dense_gemm_nvfp4": "driver_nvfp4.cu"}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the CUDA extension cannot be built")


def _deps_mtime() -> float:
    files = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [HERE.parent / "include" / "strata_masonry_b200.h"]
    return max(f.stat().st_mtime for f in files)


def _stale(out: Path, src: Path, dep_mtime: float) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return t < src.stat().st_mtime or t < dep_mtime


def _run(cmd, log: Path | None = None, verbose=False):
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        # One resource report per source file, rewritten whenever that file is compiled.
        with open(log, "w") as f:
            f.write("$ " + " ".join(map(str, cmd)) + "\n" + proc.stderr + proc.stdout + "\n")
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stderr)
        sys.stderr.write(proc.stdout)
    if proc.returncode != 0:
        raise RuntimeError(f"command failed ({proc.returncode}): {' '.join(map(str, cmd))}")


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    BUILD.mkdir(exist_ok=True)
    LIB.parent.mkdir(exist_ok=True)
    BIN.mkdir(exist_ok=True)
    dep_mtime = _deps_mtime()
    jobs = []
    objects = []
    for name in LIB_SOURCES:
        src = CSRC / name
        obj = BUILD / (src.stem + ".o")
        objects.append(obj)
        if force or _stale(obj, src, dep_mtime):
            jobs.append(([nvcc, *ARCH_FLAGS, *COMMON, "-c", str(src), "-o", str(obj)],
                         BUILD / f"ptxas_{src.stem}.log"))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(lambda job: _run(job[0], job[1], verbose), jobs))
        # The complete -Xptxas -v record of the library: every source's latest report, in build order.
        with open(BUILD / "ptxas.log", "w") as full:
            for name in LIB_SOURCES:
                part = BUILD / f"ptxas_{Path(name).stem}.log"
                if part.exists():
                    full.write(part.read_text())
    if jobs or not LIB.exists():
        _run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(LIB), *map(str, objects), "-lcudart_static",
              "-ldl", "-lpthread", "-lrt"], None, verbose)

    for exe, src_name in DRIVERS.items():
        src = CSRC / src_name
        out = BIN / exe
        if force or jobs or _stale(out, src, dep_mtime):
            _run([nvcc, *ARCH_FLAGS, "-std=c++17", "-O2", str(src), "-o", str(out),
                  f"-L{LIB.parent}", "-lstrata_masonry_b200", "-Xlinker", "-rpath", "-Xlinker",
                  "$ORIGIN/../lib"], None, verbose)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
