"""Generate tests/golden/reference_vectors.npz from the reference's own CPU verifiers.

Run where the reference tree is mounted (it is read, never modified or copied):

    python tests/golden/make_golden.py [/path/to/reference]

The two verifier modules are imported by path, unchanged, and called directly:
  src/kernels/gemm/sm100a/dense_gemm_bf16_cpu_verifier.py
  src/kernels/gemm/sm100a/nvfp4/dense_gemm_nvfp4_cpu_verifier.py
Only their outputs (numbers) are stored.  The oracle and the C/CUDA fills are tested against
this file, which travels with the repository; the reference tree does not.
"""
from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def _load(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main() -> None:
    ref_root = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SMB_REFERENCE_DIR", "/root/reference"))
    gemm_dir = ref_root / "src" / "kernels" / "gemm" / "sm100a"
    vb = _load(gemm_dir / "dense_gemm_bf16_cpu_verifier.py", "ref_bf16_verifier")
    vf = _load(gemm_dir / "nvfp4" / "dense_gemm_nvfp4_cpu_verifier.py", "ref_nvfp4_verifier")

    out: dict[str, np.ndarray] = {}
    rng = np.random.default_rng(7)

    # ---- bf16 helpers and fills
    f32 = np.concatenate([
        rng.standard_normal(2000).astype(np.float32) * np.float32(3.0),
        np.array([0.0, -0.0, 1.0, 1.00390625, 1.0078125, 1.01171875, 0.1, -0.1, 255.5, 65504.0,
                  3.0e-39, 1.0e-30, 0.33333334], dtype=np.float32),
        (np.arange(1, 600, dtype=np.uint32) * np.uint32(0x00008000) + np.uint32(0x3F800000)).view(np.float32),
    ])
    out["f32_samples"] = f32
    out["f32_to_bf16"] = vb.f32_to_bf16(f32).astype(np.uint16)
    out["bf16_to_f32"] = vb.bf16_to_f32(out["f32_to_bf16"])

    idx = np.unique(np.concatenate([
        np.arange(0, 4096, dtype=np.uint64),
        rng.integers(0, 2 ** 32, size=4096, dtype=np.uint64),
        np.array([2 ** 31 - 1, 2 ** 31, 2 ** 32 - 1, 2 ** 32, 2 ** 32 + 5, 2 ** 33 + 12345,
                  32768 * 8192 - 1, 57344 * 8192 - 1], dtype=np.uint64),
    ]))
    out["fill_indices"] = idx
    for mode in (1, 2, 3, 4):
        for seed in (1, 2):
            out[f"bf16_fill_m{mode}_s{seed}"] = vb.fill(idx, mode, seed).astype(np.float32)

    for (m, n, count) in ((256, 128, 64), (14080, 5120, 64), (8192, 8192, 256), (7, 5, 100)):
        rows, cols = vb.sample_coordinates(m, n, count, 20260827)
        out[f"sample_rows_{m}_{n}_{count}"] = rows.astype(np.int64)
        out[f"sample_cols_{m}_{n}_{count}"] = cols.astype(np.int64)

    # Full smoke outputs (256 x 128, K = 64) as the reference CPU path computes them.
    case = vb.CASES["smoke"]
    for mode in (1, 2, 3, 4):
        a = vb.fill(np.arange(case["m"] * case["k"]), mode, 1).reshape(case["m"], case["k"])
        b = vb.fill(np.arange(case["k"] * case["n"]), mode, 2).reshape(case["k"], case["n"])
        out[f"bf16_smoke_out_m{mode}"] = vb.f32_to_bf16(a @ b).astype(np.uint16)

    # Sampled references of two larger reference cases.
    for name in ("und-qkv", "gen-o"):
        c = vb.CASES[name]
        rows, cols = vb.sample_coordinates(c["m"], c["n"], 64, 20260827)
        for mode in (1, 2):
            out[f"bf16_{name}_ref_m{mode}"] = vb.references(c, rows, cols, mode).astype(np.float32)
        out[f"bf16_{name}_rows"] = rows.astype(np.int64)
        out[f"bf16_{name}_cols"] = cols.astype(np.int64)
        out[f"bf16_{name}_shape"] = np.array([c["m"], c["k"], c["n"]], dtype=np.int64)

    # ---- nvfp4 helpers and fills
    hx = np.concatenate([np.arange(0, 2048, dtype=np.uint64),
                         rng.integers(0, 2 ** 32, size=2048, dtype=np.uint64)])
    out["hash_inputs"] = hx
    out["hash32"] = vf.hash32(hx).astype(np.uint64)
    out["e2m1_table"] = vf.E2M1.astype(np.float32)
    for mode in (1, 2, 3, 4):
        out[f"fp4_data_m{mode}_A"] = vf.data_values(idx, mode, vf.SEED_A).astype(np.float32)
        out[f"fp4_data_m{mode}_B"] = vf.data_values(idx, mode, vf.SEED_B).astype(np.float32)
    srows = rng.integers(0, 2 ** 20, size=4096, dtype=np.uint64)
    sblk = rng.integers(0, 1024, size=4096, dtype=np.uint64)
    out["scale_rows"] = srows
    out["scale_blocks"] = sblk
    for mode in (1, 2, 3, 4):
        for which in (0, 1):
            out[f"fp4_scale_m{mode}_w{which}"] = vf.scale_values(srows, sblk, mode, which).astype(np.float32)

    case = vf.CASES["smoke"]
    for mode in (1, 2, 3, 4):
        ref = np.empty((case["m"], case["n"]), dtype=np.float32)
        for m in range(case["m"]):
            for n in range(case["n"]):
                ref[m, n] = vf.reference_value(m, n, case["k"], mode)
        out[f"fp4_smoke_out_m{mode}"] = vf.f32_to_bf16(ref).astype(np.uint16)

    c = vf.CASES["flagship"]
    rows, cols = vf.sample_coordinates(c["m"], c["n"], 48, 20260827)
    out["fp4_flagship_rows"] = rows.astype(np.int64)
    out["fp4_flagship_cols"] = cols.astype(np.int64)
    out["fp4_flagship_shape"] = np.array([c["m"], c["k"], c["n"]], dtype=np.int64)
    for mode in (2, 4):
        out[f"fp4_flagship_ref_m{mode}"] = np.array(
            [vf.reference_value(int(m), int(n), c["k"], mode) for m, n in zip(rows, cols)],
            dtype=np.float32)

    # ---- every benchmark configuration through the verifiers' own sampling and reference code.
    # The verifiers only know their built-in CASES; a shape outside them is added to the imported
    # module's CASES at run time (the files on disk are never edited) and then served by the same
    # sample_coordinates / references / reference_value functions verify() itself calls.  The GPU
    # tests hold the CUDA output at these coordinates to these values under verify()'s mismatch rule.
    config_samples = 256
    bf16_configs = {"bf16_8192": (8192, 8192, 8192), "bf16_ragged": (4095, 4160, 12289),
                    "bf16_large": (32768, 8192, 57344)}
    for name, (m, k, n) in bf16_configs.items():
        vb.CASES[name] = {"m": m, "k": k, "n": n, "production_m": m}
        c = vb.CASES[name]
        rows, cols = vb.sample_coordinates(c["m"], c["n"], config_samples, 20260827)
        out[f"cfg_{name}_rows"] = rows.astype(np.int64)
        out[f"cfg_{name}_cols"] = cols.astype(np.int64)
        out[f"cfg_{name}_shape"] = np.array([m, k, n], dtype=np.int64)
        out[f"cfg_{name}_ref_m2"] = vb.references(c, rows, cols, 2).astype(np.float32)
    fp4_configs = {"nvfp4_8192": (8192, 8192, 8192), "decode_m16": (16, 8192, 28672),
                   "decode_m64": (64, 8192, 28672), "decode_m128": (128, 8192, 28672)}
    for name, (m, k, n) in fp4_configs.items():
        vf.CASES[name] = {"m": m, "k": k, "n": n, "production_m": m}
        c = vf.CASES[name]
        rows, cols = vf.sample_coordinates(c["m"], c["n"], config_samples, 20260827)
        out[f"cfg_{name}_rows"] = rows.astype(np.int64)
        out[f"cfg_{name}_cols"] = cols.astype(np.int64)
        out[f"cfg_{name}_shape"] = np.array([m, k, n], dtype=np.int64)
        out[f"cfg_{name}_ref_m2"] = np.array(
            [vf.reference_value(int(r), int(cc), c["k"], 2) for r, cc in zip(rows, cols)], dtype=np.float32)
    out["cfg_tolerances"] = np.array([0.05, 0.05, 16.0, 0.008], dtype=np.float64)   # bf16 atol, rtol; nvfp4 atol, rtol

    np.savez_compressed(HERE / "reference_vectors.npz", **out)
    total = sum(v.nbytes for v in out.values())
    print(f"wrote {len(out)} arrays, {total / 1024:.0f} KiB raw, "
          f"{(HERE / 'reference_vectors.npz').stat().st_size / 1024:.0f} KiB on disk")


if __name__ == "__main__":
    main()
