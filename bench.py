#!/usr/bin/env python
"""Headline benchmark of the dense GEMM path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one pass of the hot path over one batch of synthetic input: one GEMM of the
named workload.  The headline workload is BF16 8192^3 (operands N(0,1)*0.1 stand-in, FP32
accumulate, BF16 out); run without --workload the same line carries, under "workloads", one
sub-record for every other half of the metric: NVFP4 8192^3, the three decode shapes (N = 1) and
the large BF16 GEMM 32768 x 57344 x 8192 (every N; at N > 1 with the all-gather of D, NCCL +
unshard copy through the C ABI, timed apart from the GEMM).

With N > 1 (launched under torch.distributed.run, one rank per GPU) the N dimension is sharded
column-parallel: rank r computes D[:, r*N/g : (r+1)*N/g] with no communication in the kernel.

Rank 0 prints ONE JSON line.  `value` is whole-job TFLOP/s with operands resident in HBM
(device-timed with CUDA events, max over ranks); `e2e` is the same metric through the
host-buffer entry points of the C ABI with the host<->device copies inside the timed region
(at N > 1 every rank sends its 1/g of A once and the GPUs complete A over NVLink); `roofline`
relates the kernel to the measured tensor or HBM peak; `cpu_baseline` is the reference's NumPy
CPU path timed on this host's cores on a bounded sample.

`--impl reference` times that NumPy CPU path alone (the reference has no other CPU
implementation of this path), on the same metric and config.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (kind, M, N, K, fill, description)
    "bf16_8192": ("bf16", 8192, 8192, 8192, 5, "dense BF16 GEMM M=N=K=8192, operands N(0,1)*0.1 stand-in"),
    "nvfp4_8192": ("nvfp4", 8192, 8192, 8192, 5, "dense NVFP4 GEMM M=N=K=8192, quantised N(0,1) stand-in"),
    "nvf4b16_8192": ("nvfp4", 8192, 8192, 8192, 16,
                     "dense NVFP4-proper GEMM M=N=K=8192: E4M3 scale per 16 K, quantised N(0,1) (secondary workload)"),
    "bf16_large": ("bf16", 32768, 57344, 8192, 6, "dense BF16 GEMM 32768x57344x8192, operands N(0,1)*0.05 stand-in"),
    "bf16_smoke": ("bf16", 256, 128, 64, 2, "reference smoke shape 256x128x64, fill 2"),
    "decode_m16": ("decode", 16, 28672, 8192, 5, "NVFP4 decode GEMM M=16, N=28672, K=8192 (HBM-bound)"),
    "decode_m16_b16": ("decode", 16, 28672, 8192, 16,
                       "NVFP4-proper decode GEMM M=16, N=28672, K=8192: E4M3 scale per 16 K (secondary workload)"),
    "decode_m64": ("decode", 64, 28672, 8192, 5, "NVFP4 decode GEMM M=64, N=28672, K=8192 (HBM-bound)"),
    "decode_m128": ("decode", 128, 28672, 8192, 5, "NVFP4 decode GEMM M=128, N=28672, K=8192 (HBM-bound)"),
}
HEADLINE = "bf16_8192"
# Sub-records of the default run: (name, steps; None = as many as fill about 0.25 s, only at these N; None = all).
SUB_WORKLOADS = [("nvfp4_8192", 300, None), ("decode_m16", 300, (1,)), ("decode_m64", 300, (1,)),
                 ("decode_m128", 300, (1,)), ("bf16_large", None, None)]
# A timed loop of back-to-back launches longer than this runs under the power cap: its tensor
# roofline uses the sustained cuBLAS figure, a shorter one the burst figure.
SUSTAINED_AFTER_S = 0.1
DECODE_WEIGHT_SETS = 4   # rotate weight buffers so that every step streams from HBM, not from L2

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel, from
# one ncu capture each at 1 GPU.  Keyed by workload AND by the kernel configuration the plan
# reports at run time (smb_*_plan_describe), so that a changed tile choice reads as "no capture"
# (null) instead of a stale figure; each entry names the summary under profiles/ that holds it.
NCU_TRAFFIC = {
    ("bf16_8192", "bf16 tile 256x512 store=tma resident=1"): (1_067_447_040, "profiles/bf16_gemm_8192.md"),
    ("nvfp4_8192", "fp4 tile 256x384 store=tma"): (205_597_184, "profiles/nvfp4_gemm_8192.md"),
    ("bf16_large", "bf16 tile 256x512 store=tma resident=1"): (42_861_576_960, "profiles/bf16_gemm_32768x57344x8192.md"),
    ("decode_m16", "fp4 decode m_pad=16 tile-pairs"): (128_733_440, "profiles/nvfp4_decode_m16.md"),
    ("decode_m64", "fp4 decode m_pad=64 tile-pairs"): (128_104_704, "profiles/nvfp4_decode_m16.md"),
    ("decode_m128", "fp4 decode m_pad=128 tile-pairs"): (129_742_080, "profiles/nvfp4_decode_m16.md"),
}

MIN_WARM_S = 0.3
BURST_AFTER_S = 0.03   # decode workloads: a first, short timing this long into the warm-up

THROTTLE_BITS = {
    0x4: "sw_power_cap",
    0x8: "hw_slowdown",
    0x20: "sw_thermal_slowdown",
    0x40: "hw_thermal_slowdown",
    0x80: "hw_power_brake_slowdown",
}


def _load_oracle():
    import importlib.util
    spec = importlib.util.spec_from_file_location("smb_oracle", ROOT / "oracle" / "oracle.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    def __init__(self, uuid: str | None, index: int, period_s: float = 0.002):
        self.period = period_s
        self.samples: list[tuple[int, int, float]] = []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            h = None
            if uuid:
                try:
                    h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if isinstance(uuid, str) else uuid)
                except Exception:
                    h = None
            if h is None:
                h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self._h = h
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._h = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                mhz = int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                reasons = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                try:
                    watts = nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0
                except Exception:
                    watts = float("nan")
                self.samples.append((mhz, reasons, watts))
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self):
        if not self.samples:
            return None
        mhz = sorted(s[0] for s in self.samples)
        bits = 0
        for s in self.samples:
            bits |= s[1]
        reasons = [name for bit, name in THROTTLE_BITS.items() if bits & bit]
        watts = [s[2] for s in self.samples if s[2] == s[2]]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(mhz), "power_w_max": round(max(watts), 1) if watts else None}


def _peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def host_cores() -> int:
    """CPUs this process may run on (the container's share of the host, not the host's count)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return os.cpu_count() or 1


class blas_threads:
    """Run the BLAS behind NumPy on all of this process's cores for the duration.  A launcher
    such as torch.distributed.run exports OMP_NUM_THREADS=1, which would silently make the CPU
    baseline a single-thread figure."""

    def __init__(self, threads: int | None = None):
        self.threads = threads or host_cores()
        self._ctx = None

    def __enter__(self):
        try:
            from threadpoolctl import threadpool_limits
            self._ctx = threadpool_limits(limits=self.threads, user_api="blas")
            self._ctx.__enter__()
        except Exception:
            self._ctx = None
        return self

    def __exit__(self, *exc):
        if self._ctx is not None:
            self._ctx.__exit__(*exc)


def blas_info():
    """(threads, description) of the BLAS behind NumPy's matmul, the library the reference's CPU path
    spends its time in; threads falls back to the core count when the pool cannot be inspected."""
    cores = host_cores()
    try:
        from threadpoolctl import threadpool_info
        for pool in threadpool_info():
            if pool.get("user_api") == "blas":
                return int(pool.get("num_threads") or cores), (
                    f"{pool.get('internal_api')} {pool.get('version')} "
                    f"({pool.get('threading_layer')}, {pool.get('architecture')})")
    except Exception:
        pass
    return cores, "unknown BLAS"


def reference_cpu_gemm():
    """The reference's own CPU GEMM functions where its tree is present (this container; never
    the GPU box): (bf16_fn(a_bits, bt_bits) -> bits, kind).  Falls back to the oracle's
    restatement ("port") of dense_gemm_bf16_cpu_verifier.py:99-103."""
    oracle = _load_oracle()
    ref_dir = Path(os.environ.get("SMB_REFERENCE_DIR", "/root/reference"))
    path = ref_dir / "src" / "kernels" / "gemm" / "sm100a" / "dense_gemm_bf16_cpu_verifier.py"
    if path.exists():
        try:
            import importlib.util
            spec = importlib.util.spec_from_file_location("smb_ref_bf16_verifier", path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            if hasattr(mod, "bf16_to_f32") and hasattr(mod, "f32_to_bf16"):
                def run(a_bits, bt_bits):
                    # write_smoke_reference's arithmetic (:99-103) with the verifier's own helpers,
                    # on operands that already are bf16 bit patterns.
                    a = mod.bf16_to_f32(a_bits)
                    b = mod.bf16_to_f32(bt_bits).T
                    return mod.f32_to_bf16(a @ b)
                return run, "reference"
        except Exception:
            pass
    return oracle.gemm_bf16_reference, "port"


def cpu_gemm_rate(oracle, a_bits, bt_bits, budget_s: float, fn=None):
    """Time the reference's CPU path (bf16 -> fp32, fp32 matmul, round to bf16) on as large a
    square sub-block as fits the time budget.  Returns (TFLOP/s, description, seconds)."""
    fn = fn or oracle.gemm_bf16_reference
    k = a_bits.shape[1]
    probe = min(512, a_bits.shape[0], bt_bits.shape[0])
    with blas_threads():
        t0 = time.perf_counter()
        fn(a_bits[:probe], bt_bits[:probe])
        dt = max(time.perf_counter() - t0, 1e-4)
        rate = 2.0 * probe * probe * k / dt
        side = int((budget_s * rate / (2.0 * k)) ** 0.5)
        side = max(min(256, a_bits.shape[0], bt_bits.shape[0]),
                   min(side // 256 * 256, a_bits.shape[0], bt_bits.shape[0]))
        best = None
        for _ in range(2):
            t0 = time.perf_counter()
            fn(a_bits[:side], bt_bits[:side])
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
    return 2.0 * side * side * k / best / 1e12, f"{side}x{side}x{k} sub-block of the workload, best of 2", best


def cpu_fp4_rate(oracle, m, n, k, budget_s: float):
    """Time the reference's CPU path for the block-scaled GEMM (codes and scale bytes -> fp32,
    fp32 matmul, round to bf16) on a rows x cols x K sub-block sized for the time budget.
    Returns (TFLOP/s, description, seconds)."""
    rows, cols = min(m, 2048), min(n, 2048)
    ac, asf = oracle.fp4_operand(min(rows, 256), k, 2, 0)
    bc, bsf = oracle.fp4_operand(min(cols, 256), k, 2, 1)
    ra, rb = max(1, rows // ac.shape[0]), max(1, cols // bc.shape[0])
    # Tiled copies of a small generated block: the timing does not depend on the values.
    ac, asf, bc, bsf = np.tile(ac, (ra, 1)), np.tile(asf, (ra, 1)), np.tile(bc, (rb, 1)), np.tile(bsf, (rb, 1))
    probe_r, probe_c = min(128, ac.shape[0]), min(128, bc.shape[0])
    with blas_threads():
        t0 = time.perf_counter()
        oracle.gemm_nvfp4_reference(ac[:probe_r], asf[:probe_r], bc[:probe_c], bsf[:probe_c])
        rate = 2.0 * probe_r * probe_c * k / max(time.perf_counter() - t0, 1e-4)
        # Keep the M : N proportion of the workload (decode shapes have few rows).
        area = budget_s * rate / (2.0 * k)
        r = int(min(ac.shape[0], max(16, (area * m / n) ** 0.5)))
        c = int(min(bc.shape[0], max(128, area / max(r, 1))))
        r, c = max(1, r // 16 * 16) if r >= 16 else r, max(128, c // 128 * 128)
        best = None
        for _ in range(2):
            t0 = time.perf_counter()
            oracle.gemm_nvfp4_reference(ac[:r], asf[:r], bc[:c], bsf[:c])
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
    return 2.0 * r * c * k / best / 1e12, f"{r}x{c}x{k} sub-block of the workload, best of 2", best


def config_for(name: str, g: int) -> dict:
    """The `config` object of a line: a function of the workload and the GPU count only, so that
    this arm and the reference arm print the same one."""
    kind, m, n, k, fill, desc = WORKLOADS[name]
    return {"workload": name, "description": desc, "shape_mnk": [m, n, k],
            "sharding": f"N column-parallel over {g} GPU(s), {n // g} columns each"}


def dtype_for(kind: str) -> str:
    return "bf16" if kind == "bf16" else "e2m1"


# --------------------------------------------------------------------------------------------
# Reference arm: the reference's NumPy CPU GEMM on this host's cores
# --------------------------------------------------------------------------------------------
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    name = args.workload or HEADLINE
    kind, m, n, k, fill, desc = WORKLOADS[name]
    oracle = _load_oracle()
    steps, warmup = args.steps, args.warmup
    # The whole workload per step where that costs about a second (8192^3 does); a bounded
    # sub-block of it for the larger shapes, so that the run ends within a few minutes.
    per_step_budget = max(0.05, min(3.0, 150.0 / max(1, steps + warmup)))
    impl_kind = "port"
    with blas_threads() as pool:
        cores, blas = blas_info()
        if kind == "bf16":
            fn, impl_kind = reference_cpu_gemm()
            rows, cols = min(m, 8192), min(n, 8192)
            a_bits, bt_bits = oracle.bf16_operands(min(rows, 1024), min(cols, 1024), k, 2 if fill > 4 else fill)
            # Tile the small generated block up to the sample size: the timing does not depend on values.
            a_bits = np.tile(a_bits, (max(1, rows // a_bits.shape[0]), 1))
            bt_bits = np.tile(bt_bits, (max(1, cols // bt_bits.shape[0]), 1))
            run = lambda r, c: fn(a_bits[:r], bt_bits[:c])
            lim_r, lim_c = a_bits.shape[0], bt_bits.shape[0]
        else:
            rows, cols = min(m, 8192), min(n, 8192)
            ac, asf = oracle.fp4_operand(min(rows, 512), k, 2, 0)
            bc, bsf = oracle.fp4_operand(min(cols, 512), k, 2, 1)
            ac, asf = np.tile(ac, (max(1, rows // ac.shape[0]), 1)), np.tile(asf, (max(1, rows // asf.shape[0]), 1))
            bc, bsf = np.tile(bc, (max(1, cols // bc.shape[0]), 1)), np.tile(bsf, (max(1, cols // bsf.shape[0]), 1))
            run = lambda r, c: oracle.gemm_nvfp4_reference(ac[:r], asf[:r], bc[:c], bsf[:c])
            lim_r, lim_c = ac.shape[0], bc.shape[0]
        pr, pc = min(256, lim_r), min(256, lim_c)
        t0 = time.perf_counter()
        run(pr, pc)
        rate = 2.0 * pr * pc * k / max(time.perf_counter() - t0, 1e-4)
        # Sample: keep the workload's M : N proportion, cap both at the workload's own extent.
        area = per_step_budget * rate / (2.0 * k)
        full = (lim_r == m and lim_c == n and float(m) * n <= area * 4.0)
        if full:
            r, c = m, n
        else:
            r = int(min(lim_r, max(min(16, lim_r), (area * m / n) ** 0.5)))
            c = int(min(lim_c, max(min(128, lim_c), area / max(r, 1))))
            r = max(1, r // 128 * 128) if r >= 128 else r
            c = max(1, c // 128 * 128) if c >= 128 else c
        for _ in range(warmup):
            run(r, c)
        t0 = time.perf_counter()
        for _ in range(steps):
            run(r, c)
        dt = time.perf_counter() - t0
    value = 2.0 * r * c * k * steps / dt / 1e12
    sample = (f"the whole {m}x{n}x{k} workload per step" if (r, c) == (m, n)
              else f"{r}x{c}x{k} sub-block of the workload per step")
    line = {
        "impl": "reference", "metric": "GEMM TFLOPS", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": dt / steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": dtype_for(kind), "data": "synthetic",
        "config": config_for(name, args.gpus),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": impl_kind,
                         "sample": f"{sample}, {steps} steps", "host_cpus": os.cpu_count(),
                         "cpus_usable": host_cores(), "blas": blas},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------------------------
# Our arm
# --------------------------------------------------------------------------------------------
class Env:
    """Process-wide state of one bench run: device, stream, rank, library handles."""

    def __init__(self):
        import torch
        import __graft_entry__ as entry
        self.torch = torch
        self.smb = entry.load_package()
        self.lib = self.smb.capi.lib()   # fails loudly if the CUDA library is missing: there is no CPU fallback
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
        self.stream = torch.cuda.current_stream()
        self.stream_ptr = int(self.stream.cuda_stream)
        self.peaks, self.peak_kind = _peaks()
        try:
            self.uuid = "GPU-" + str(torch.cuda.get_device_properties(self.dev).uuid)
        except Exception:
            self.uuid = None
        self._comm = None
        self.launches = 0

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        if self.dist is None:
            return x
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def comm(self):
        """The library's own NCCL communicator (C ABI), bootstrapped over torch.distributed."""
        if self._comm is None:
            torch = self.torch
            ident = torch.zeros(self.smb.capi.COMM_ID_BYTES, dtype=torch.uint8, device=self.dev)
            if self.rank == 0:
                raw = self.smb.gemm.Comm.unique_id()
                ident.copy_(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
            self.dist.broadcast(ident, 0)
            self._comm = self.smb.gemm.Comm(bytes(ident.cpu().numpy().tobytes()), self.world, self.rank)
        return self._comm

    def event(self):
        return self.torch.cuda.Event(enable_timing=True)


class Workload:
    """Operands of one workload resident in HBM on this rank, and the plans that multiply them."""

    def __init__(self, env: Env, name: str):
        torch, smb = env.torch, env.smb
        self.env, self.name = env, name
        self.kind, self.m, self.n, self.k, self.fill, self.desc = WORKLOADS[name]
        try:
            shard = smb.sharding.column_shard(self.n, env.world, env.rank)
        except ValueError as err:
            raise SystemExit(str(err))
        self.n_local, self.n0 = shard.n_local, shard.n0
        m, n, k, n_local, n0, fill, dev, stream = self.m, self.n, self.k, self.n_local, self.n0, self.fill, env.dev, env.stream
        self.plans, self.weights = [], []
        self.sfa = self.sfb = self.bt = None
        if self.kind == "bf16":
            self.a = torch.empty(m, k, device=dev, dtype=torch.bfloat16)
            self.bt = torch.empty(n_local, k, device=dev, dtype=torch.bfloat16)
            self.d = torch.empty(m, n_local, device=dev, dtype=torch.bfloat16)
            smb.gemm.bf16_operands_device(self.a, self.bt, m, n_local, k, fill, n0=n0, n_total=n, stream=stream)
            self.plans = [smb.gemm.Bf16Plan(self.a, self.bt, self.d, m, n_local, k, flags=smb.capi.FLAG_OPERANDS_STATIC)]
            self.resident_bytes = (self.a.numel() + self.bt.numel() + self.d.numel()) * 2
        elif self.kind == "decode":
            self.a = torch.empty(m, k // 2, device=dev, dtype=torch.uint8)
            self.sfa = torch.empty(smb.gemm.sf_packed_bytes(m, k), device=dev, dtype=torch.uint8)
            self.sfa_rm = torch.empty(m, k // 32, device=dev, dtype=torch.uint8)
            smb.gemm.fill_fp4_device(self.a, self.sfa, self.sfa_rm, m, k, 6, 0, 0, stream=stream)
            self.d = torch.empty(m, n_local, device=dev, dtype=torch.bfloat16)
            block16 = (fill == 16)
            if block16:
                self.sfa, gs_a = self._quantize_b16(m, self.a, 99)
            for i in range(DECODE_WEIGHT_SETS):
                w = torch.empty(n_local, k // 2, device=dev, dtype=torch.uint8)
                sfw_rm = None
                if block16:
                    sfw, gs_w = self._quantize_b16(n_local, w, 1000 + env.rank * 16 + i)
                    pl = smb.gemm.Fp4Plan(self.a, self.sfa, w, sfw, self.d, m, n_local, k, flags=smb.capi.FLAG_SCALE_BLOCK16)
                    pl.set_alpha(1.0 / (gs_a * gs_w))
                else:
                    sfw = torch.empty(smb.gemm.sf_packed_bytes(n_local, k), device=dev, dtype=torch.uint8)
                    if i == 0:
                        sfw_rm = torch.empty(n_local, k // 32, device=dev, dtype=torch.uint8)
                    # Different rows of the same logical generator for every set.
                    smb.gemm.fill_fp4_device(w, sfw, sfw_rm, n_local, k, fill, 1, n0 + i * n, stream=stream)
                    pl = smb.gemm.Fp4Plan(self.a, self.sfa, w, sfw, self.d, m, n_local, k)
                self.weights.append((w, sfw, sfw_rm))
                self.plans.append(pl)
            self.resident_bytes = DECODE_WEIGHT_SETS * (self.weights[0][0].numel() + self.weights[0][1].numel())
        else:
            self.a = torch.empty(m, k // 2, device=dev, dtype=torch.uint8)
            self.bt = torch.empty(n_local, k // 2, device=dev, dtype=torch.uint8)
            self.d = torch.empty(m, n_local, device=dev, dtype=torch.bfloat16)
            if fill == 16:
                # NVFP4 proper: Gaussian data quantised on the device, E4M3 scale per 16 K, the two
                # per-tensor factors folded into the plan's output factor.
                self.sfa, gs_a = self._quantize_b16(m, self.a, 1234 + env.rank)
                self.sfb, gs_b = self._quantize_b16(n_local, self.bt, 4321 + env.rank)
                pl = smb.gemm.Fp4Plan(self.a, self.sfa, self.bt, self.sfb, self.d, m, n_local, k,
                                      flags=smb.capi.FLAG_OPERANDS_STATIC | smb.capi.FLAG_SCALE_BLOCK16)
                pl.set_alpha(1.0 / (gs_a * gs_b))
            else:
                self.sfa = torch.empty(smb.gemm.sf_packed_bytes(m, k), device=dev, dtype=torch.uint8)
                self.sfb = torch.empty(smb.gemm.sf_packed_bytes(n_local, k), device=dev, dtype=torch.uint8)
                self.sfa_rm = torch.empty(m, k // 32, device=dev, dtype=torch.uint8)
                self.sfb_rm = torch.empty(n_local, k // 32, device=dev, dtype=torch.uint8)
                smb.gemm.fill_fp4_device(self.a, self.sfa, self.sfa_rm, m, k, fill, 0, 0, stream=stream)
                smb.gemm.fill_fp4_device(self.bt, self.sfb, self.sfb_rm, n_local, k, fill, 1, n0, stream=stream)
                pl = smb.gemm.Fp4Plan(self.a, self.sfa, self.bt, self.sfb, self.d, m, n_local, k,
                                      flags=smb.capi.FLAG_OPERANDS_STATIC)
            self.plans = [pl]
            self.resident_bytes = (self.a.numel() + self.bt.numel() + self.sfa.numel() + self.sfb.numel()
                                   + self.d.numel() * 2)
        torch.cuda.synchronize()
        # The decode steps are shorter (18 us) than a Python method call chain: launch through the
        # C entry point directly, with the handles and the stream pointer looked up once.
        self.run_fn = env.lib.smb_bf16_plan_run if self.kind == "bf16" else env.lib.smb_fp4_plan_run
        self.handles = [pl._h for pl in self.plans]
        self.kernel_config = self.plans[0].describe()
        self.flops_step = 2.0 * m * n * k
        sf_k = 16 if fill == 16 else 32   # K values per scale byte
        if self.kind == "bf16":
            self.algo_bytes = (m * k + n_local * k + m * n_local) * 2
        else:
            # Weights + weight scales + activations + their scales + D.
            self.algo_bytes = n_local * k // 2 + n_local * k // sf_k + m * k // 2 + m * k // sf_k + 2 * m * n_local

    def _quantize_b16(self, rows, codes, seed):
        """Gaussian data quantised on the device: E2M1 + E4M3 scale per 16 K."""
        env, torch, smb, k = self.env, self.env.torch, self.env.smb, self.k
        sf = torch.empty(smb.gemm.sf_packed_bytes(rows, 2 * k), device=env.dev, dtype=torch.uint8)
        gen = torch.Generator(device=env.dev).manual_seed(seed)
        x = torch.randn(rows, k, device=env.dev, generator=gen)
        gs = 448.0 * 6.0 / float(x.abs().max())
        smb.capi.check(env.lib.smb_quantize_nvf4_device(x.data_ptr(), k, C.c_float(gs), codes.data_ptr(), k // 2,
                                                        sf.data_ptr(), None, rows, k, env.stream_ptr))
        torch.cuda.synchronize()
        return sf, gs

    def step(self, i: int) -> None:
        if self.run_fn(self.handles[i % len(self.handles)], self.env.stream_ptr) != 0:
            raise RuntimeError(self.env.smb.capi.last_error())

    def check(self):
        for pl in self.plans:
            pl.check(self.env.stream)

    def close(self):
        for pl in self.plans:
            pl.close()
        self.plans = []


def time_workload(env: Env, wl: Workload, steps: int | None, warmup: int, extra_warmup: bool) -> dict:
    """W warm-up steps, then K steps between CUDA events on the launching stream, a barrier and a
    device synchronize on both sides, max over ranks; clocks sampled during the timed region."""
    torch = env.torch
    for i in range(warmup):
        wl.step(i)
    wl.check()
    if steps is None:
        # As many steps as fill about a quarter of a second (the same on all ranks).
        p0, p1 = env.event(), env.event()
        env.barrier()
        p0.record(env.stream)
        for i in range(3):
            wl.step(i)
        p1.record(env.stream)
        env.barrier()
        est_ms = env.max_over_ranks(p0.elapsed_time(p1)) / 3
        steps = int(max(5, min(300, round(250.0 / max(est_ms, 1e-3)))))
    # A GPU that has been idle takes a moment to reach its working clocks; the decode shapes
    # (300 steps are 6 ms) would otherwise be timed on the ramp: the first process on a fresh box
    # read 23.5 us per step, every later one 21.0.  Keep warming those up until the device has been
    # busy for MIN_WARM_S: by then the clocks have also settled where the board's power management
    # holds them under this load (1.4-1.7 GHz with sw_power_cap reported), so `value` is the
    # sustained figure.  The same number of steps timed early in that warm-up, at full clocks, is
    # reported beside it as `burst`.  The tensor-bound workloads keep exactly the W warm-up steps
    # asked for.
    warm_t0 = time.perf_counter()
    extra_warm = 0
    burst = None
    while (wl.kind == "decode" and extra_warmup and time.perf_counter() - warm_t0 < MIN_WARM_S
           and extra_warm < 100000):
        for i in range(20):
            wl.step(extra_warm + i)
        extra_warm += 20
        torch.cuda.synchronize()
        if burst is None and time.perf_counter() - warm_t0 >= BURST_AFTER_S:
            b0, b1 = env.event(), env.event()
            b0.record(env.stream)
            for i in range(steps):
                wl.step(i)
            b1.record(env.stream)
            torch.cuda.synchronize()
            burst = b0.elapsed_time(b1) / steps
            extra_warm += steps
    e0, e1 = env.event(), env.event()
    env.barrier()
    with ClockSampler(env.uuid, env.local_rank) as sampler:
        e0.record(env.stream)
        for i in range(steps):
            wl.step(i)
        e1.record(env.stream)
        env.barrier()
    wl.check()
    env.launches += steps
    ms_local = e0.elapsed_time(e1)
    ms_total = env.max_over_ranks(ms_local)
    ms_step = ms_total / steps
    rec = {"ms_per_step": ms_step, "steps": steps, "warmup": warmup, "extra_warmup_steps": extra_warm,
           "value": wl.flops_step / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s",
           "clocks": sampler.summary(), "kernel": wl.kernel_config}
    rec["roofline"] = roofline_for(env, wl, ms_local / steps, ms_total * 1e-3, burst, steps)
    if rec["clocks"] and rec["clocks"].get("sm_mhz"):
        # Launch time in SM clocks at the clock sampled under load: what to compare when two runs
        # (or two kernels) were held at different clocks by the power cap.
        rec["roofline"]["mcycles_per_launch_at_sampled_clock"] = (ms_local / steps) * rec["clocks"]["sm_mhz"] * 1e-3
    return rec


def roofline_for(env: Env, wl: Workload, launch_ms: float, timed_s: float, burst, steps: int) -> dict:
    peaks, peak_kind = env.peaks, env.peak_kind
    g = env.world
    hit = NCU_TRAFFIC.get((wl.name, wl.kernel_config)) if g == 1 else None
    traffic, traffic_src = (hit if hit else (None, None))
    flops_launch = 2.0 * wl.m * wl.n_local * wl.k
    if wl.kind == "decode":
        gbs = wl.algo_bytes / (launch_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": gbs / peaks["hbm_gbs"], "traffic": traffic,
                "peak_source": f"{peak_kind} device copy GB/s", "nominal_frac": gbs / 8000.0}
        if burst is not None:
            # Not the headline: the same launches timed 30 ms into the warm-up, before the clocks
            # have come down to where they stay under this load.
            roof["burst"] = {"us_per_step": burst * 1e3, "achieved": wl.algo_bytes / (burst * 1e-3) / 1e9,
                             "unit": "GB/s", "nominal_frac": wl.algo_bytes / (burst * 1e-3) / 1e9 / 8000.0,
                             "steps": steps, "after_warm_s": BURST_AFTER_S}
    else:
        achieved = flops_launch / (launch_ms * 1e-3) / 1e12
        sustained = timed_s >= SUSTAINED_AFTER_S
        base = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) if sustained else peaks["bf16_tflops"]
        if wl.kind == "bf16":
            peak = base
            note = f"{peak_kind} cuBLAS bf16 {'sustained' if sustained else 'burst'} TFLOP/s"
        else:
            # No FP4 entry in the measured peaks: four times the measured dense bf16 rate (the ratio
            # of the nominal dense FP4 and BF16 figures, 9 and 2.25 PFLOP/s).
            peak = 4.0 * base
            note = f"4 x {peak_kind} cuBLAS bf16 {'sustained' if sustained else 'burst'} TFLOP/s (no measured FP4 figure)"
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": traffic, "peak_source": note,
                "frac_of_burst": achieved / (peaks["bf16_tflops"] * (1 if wl.kind == "bf16" else 4)),
                "nominal_frac": achieved / (2250.0 if wl.kind == "bf16" else 9000.0)}
    # What `achieved` divides: the algorithmic work of one launch on this rank.
    roof["algorithmic_flops_per_launch"] = flops_launch
    roof["algorithmic_bytes_per_launch"] = wl.algo_bytes
    roof["launch_ms"] = launch_ms
    if traffic_src:
        roof["traffic_source"] = f"one ncu capture of this kernel configuration, {traffic_src}"
    return roof


def e2e_for(env: Env, wl: Workload, steps: int) -> dict | None:
    """The same GEMM through the host-buffer contexts of the C ABI: pinned host operands go up,
    the result comes back, all inside the timed region (wall clock, max over ranks).  With more
    than one GPU every rank sends its M / g rows of A and its own shard of B; the GPUs complete A
    over NVLink (NCCL all-gather inside the context's run)."""
    torch, smb = env.torch, env.smb
    m, n_local, k, g = wl.m, wl.n_local, wl.k, env.world
    if wl.fill == 16 or (g > 1 and m % g != 0):
        return None
    comm = env.comm() if g > 1 else None
    rows = m // g
    r0 = env.rank * rows

    def pinned(t):
        out = torch.empty(t.shape, dtype=t.dtype).pin_memory()
        out.copy_(t)
        return out

    d_host = torch.empty(m, n_local, dtype=torch.int16).pin_memory()
    if wl.kind == "bf16":
        a_host = pinned(wl.a[r0:r0 + rows].view(torch.int16))
        bt_host = pinned(wl.bt.view(torch.int16))
        ctx = smb.gemm.Bf16HostContext(m, n_local, k, comm=comm)
        run = lambda: ctx.run(a_host, bt_host, d_host)
        h2d = a_host.numel() * 2 + bt_host.numel() * 2
        api = "smb_bf16_host_ctx_run"
        wl.host_a, wl.host_bt = (a_host, bt_host) if g == 1 else (None, None)
    else:
        a_host = pinned(wl.a[r0:r0 + rows])
        sfa_host = pinned(wl.sfa_rm[r0:r0 + rows])
        if wl.kind == "decode":
            w, _, sfw_rm = wl.weights[0]
            b_host, sfb_host = pinned(w), pinned(sfw_rm)
        else:
            b_host, sfb_host = pinned(wl.bt), pinned(wl.sfb_rm)
        ctx = smb.gemm.Fp4HostContext(m, n_local, k, comm=comm)
        if wl.kind == "decode":
            # A decode step: the weights were loaded once (here: by the first, untimed run) and
            # stay on the device; a step sends the activations and their scales, and reads D back.
            ctx.run(a_host, sfa_host, b_host, sfb_host, d_host)
            run = lambda: ctx.run(a_host, sfa_host, None, None, d_host)
            h2d = a_host.numel() + sfa_host.numel()
            api = "smb_fp4_host_ctx_run, weights resident on the device (b = NULL)"
        else:
            run = lambda: ctx.run(a_host, sfa_host, b_host, sfb_host, d_host)
            h2d = a_host.numel() + sfa_host.numel() + b_host.numel() + sfb_host.numel()
            api = "smb_fp4_host_ctx_run"
    if g > 1:
        api += f" on a sharded context (rank r sends rows r*M/{g}.. of A, NCCL all-gather of A inside the run)"
    for _ in range(2):
        run()
    env.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    env.barrier()
    e2e_s = env.max_over_ranks(time.perf_counter() - t0) / steps
    # The plan for the timed loop wrote the same operands' product into wl.d (weight set 0 for decode).
    if wl.kind == "decode":
        wl.d.fill_(0)
        wl.step(0)
        wl.check()
    same = bool(torch.equal(d_host, wl.d.view(torch.int16).cpu()))
    ctx.close()
    return {"value": wl.flops_step / e2e_s / 1e12, "unit": "TFLOP/s",
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d_host.numel() * 2),
            "ms_per_step": e2e_s * 1e3, "steps": steps, "matches_device_path": same,
            "api": api + " (pinned host buffers, per-GPU figures for the byte counts)"}


def cpu_baseline_for(wl: Workload, budget_s: float) -> dict:
    oracle = _load_oracle()
    if wl.kind == "bf16":
        fn, impl_kind = reference_cpu_gemm()
        rows, cols = min(wl.m, 4096), min(wl.n, 4096)
        if getattr(wl, "host_a", None) is not None:
            a_np = wl.host_a[:rows].numpy().view(np.uint16)
            bt_np = wl.host_bt[:cols].numpy().view(np.uint16)
        else:
            a_np, bt_np = oracle.bf16_operands(min(rows, 512), min(cols, 512), wl.k, 2)
            a_np = np.tile(a_np, (max(1, rows // a_np.shape[0]), 1))
            bt_np = np.tile(bt_np, (max(1, cols // bt_np.shape[0]), 1))
        rate, sample, secs = cpu_gemm_rate(oracle, a_np, bt_np, budget_s, fn)
        what = "reference NumPy CPU path: bf16 operands -> fp32, a @ b, round to bf16"
    else:
        impl_kind = "port"
        rate, sample, secs = cpu_fp4_rate(oracle, wl.m, wl.n, wl.k, budget_s)
        what = "reference NumPy CPU path: E2M1 codes and UE8M0 scales -> fp32, a @ b, round to bf16"
    with blas_threads():
        threads, blas = blas_info()
    return {"value": rate, "unit": "TFLOP/s", "cores": threads, "kind": impl_kind,
            "sample": sample + f" ({secs:.2f} s)", "host_cpus": os.cpu_count(), "cpus_usable": host_cores(),
            "blas": blas, "what": what}


def allgather_study(env: Env, wl: Workload, ms_step: float) -> dict:
    """The optional exchange, timed apart from the GEMM: NCCL all-gather of the [M, N/g] slabs
    through the library's own communicator (smb_allgather_columns), then the unshard copy."""
    torch, smb = env.torch, env.smb
    g, m, n, n_local = env.world, wl.m, wl.n, wl.n_local
    comm = env.comm()
    gathered = torch.empty(g, m, n_local, device=env.dev, dtype=torch.bfloat16)
    full = torch.empty(m, n, device=env.dev, dtype=torch.bfloat16)
    reps = 5

    def timed(fn):
        for _ in range(2):
            fn()
        env.barrier()
        t0, t1 = env.event(), env.event()
        t0.record(env.stream)
        for _ in range(reps):
            fn()
        t1.record(env.stream)
        env.barrier()
        return env.max_over_ranks(t0.elapsed_time(t1)) / reps

    ag_ms = timed(lambda: comm.allgather_columns(wl.d, gathered, None, m, n_local, stream=env.stream))
    un_ms = timed(lambda: smb.gemm.unshard_columns_device(gathered, full, g, m, n_local, stream=env.stream))
    both_ms = timed(lambda: comm.allgather_columns(wl.d, gathered, full, m, n_local, stream=env.stream))
    # Every rank's full D holds every rank's slab: own slab equal to the GEMM's output, and one
    # checksum over the whole matrix equal on all ranks.
    own_ok = bool(torch.equal(full[:, wl.n0:wl.n0 + n_local].view(torch.int16), wl.d.view(torch.int16)))
    checksum = full.view(torch.int16).to(torch.int64).sum().reshape(1)
    lo, hi = checksum.clone(), checksum.clone()
    env.dist.all_reduce(lo, op=env.dist.ReduceOp.MIN)
    env.dist.all_reduce(hi, op=env.dist.ReduceOp.MAX)
    ok_t = torch.tensor([1 if own_ok else 0], device=env.dev)
    env.dist.all_reduce(ok_t, op=env.dist.ReduceOp.MIN)
    recv = (g - 1) * m * n_local * 2
    out = {"ms": ag_ms, "recv_gb_per_s_per_gpu": recv / (ag_ms * 1e-3) / 1e9,
           "layout": "rank-major [g, M, N/g]", "unshard_ms": un_ms,
           "unshard_gb_per_s": 2.0 * m * n * 2 / (un_ms * 1e-3) / 1e9,
           "allgather_plus_unshard_ms": both_ms, "unfused_total_ms": ms_step + ag_ms + un_ms,
           "api": "smb_allgather_columns (NCCL over NVLink) + smb_unshard_columns_device",
           "full_d_consistent_on_all_ranks": bool(ok_t.item() == 1 and lo.item() == hi.item()),
           "nvlink_bound_ms_at_770_gb_s": recv / 770e9 * 1e3}
    del gathered, full
    return out


def decode_from_bf16_study(env: Env, wl: Workload, steps: int, warmup: int) -> dict:
    """The step as a model runs it: the activations arrive as BF16 and are quantised on the device
    (inside the decode kernel up to 16 rows, by a kernel chained in front above that).  Secondary
    figure; the headline starts from quantised activations, as the reference's metric does."""
    torch, smb = env.torch, env.smb
    m, k, n_local = wl.m, wl.k, wl.n_local
    x16 = torch.empty(m, k, device=env.dev, dtype=torch.bfloat16)
    smb.gemm.fill_bf16_device(x16, m, k, 5, 1, stream=env.stream)

    def timed(flags):
        plans = [smb.gemm.Fp4Plan.from_bf16_activations(x16, w, sfw, wl.d, m, n_local, k, flags=flags)
                 for (w, sfw, _) in wl.weights]
        handles = [pl._h for pl in plans]
        for i in range(max(3, warmup)):
            plans[i % len(plans)].run(env.stream)
        plans[0].check(env.stream)
        a0, a1 = env.event(), env.event()
        env.barrier()
        a0.record(env.stream)
        for i in range(steps):
            if wl.run_fn(handles[i % len(handles)], env.stream_ptr) != 0:
                raise RuntimeError(smb.capi.last_error())
        a1.record(env.stream)
        env.barrier()
        for pl in plans:
            pl.check(env.stream)
            pl.close()
        return env.max_over_ranks(a0.elapsed_time(a1)) / steps

    act_ms = timed(0)
    plain_ms = timed(smb.capi.FLAG_NO_LAUNCH_OVERLAP)
    act_bytes = wl.algo_bytes + m * k * 2   # + the BF16 activations read by the quantiser
    return {"us_per_step": act_ms * 1e3, "us_per_step_plain_stream_order": plain_ms * 1e3,
            "gb_per_s": act_bytes / (act_ms * 1e-3) / 1e9,
            "api": "smb_fp4_plan_create_bf16_activations + smb_fp4_plan_run"}


def swiglu_study(env: Env, wl: Workload, ms_step: float, steps: int) -> dict | None:
    """The rows of BT are read as interleaved (up, gate) pairs; the fused plan writes
    silu(gate) * up, half as wide, against the plain GEMM followed by the same activation as
    separate PyTorch element-wise kernels on its bf16 output."""
    torch, smb = env.torch, env.smb
    m, k, n_local = wl.m, wl.k, wl.n_local
    if wl.kind == "decode" or n_local % 2 != 0:
        return None
    d_act = torch.empty(m, n_local // 2, device=env.dev, dtype=torch.bfloat16)
    sflags = smb.capi.FLAG_OPERANDS_STATIC | smb.capi.FLAG_EPILOGUE_SWIGLU
    if wl.kind == "bf16":
        splan = smb.gemm.Bf16Plan(wl.a, wl.bt, d_act, m, n_local, k, ldd=n_local // 2, flags=sflags)
    else:
        splan = smb.gemm.Fp4Plan(wl.a, wl.sfa, wl.bt, wl.sfb, d_act, m, n_local, k, ldd=n_local // 2, flags=sflags)
    reps = max(5, min(steps, 100))

    def timed(fn):
        for _ in range(3):
            fn()
        env.barrier()
        t0, t1 = env.event(), env.event()
        t0.record(env.stream)
        for _ in range(reps):
            fn()
        t1.record(env.stream)
        env.barrier()
        return env.max_over_ranks(t0.elapsed_time(t1)) / reps

    def unfused():
        wl.plans[0].run(env.stream)
        torch.mul(torch.nn.functional.silu(wl.d[:, 1::2]), wl.d[:, 0::2], out=d_act)

    fused_ms = timed(lambda: splan.run(env.stream))
    splan.check(env.stream)
    unfused_ms = timed(unfused)
    splan.close()
    return {"fused_ms": fused_ms, "gemm_then_torch_elementwise_ms": unfused_ms, "gemm_only_ms": ms_step,
            "d_bytes_fused": m * (n_local // 2) * 2,
            "tflops_fused": wl.flops_step / env.world / (fused_ms * 1e-3) / 1e12}


def fused_allgather_study(env: Env, wl: Workload, ms_step: float, steps: int) -> dict | None:
    """GEMM + all-gather in one kernel: every rank holds a full row-major D [M, N] that all
    processes map; the epilogue of rank r stores its column slab into all g of them (plain stores
    over NVLink for the g - 1 remote ones)."""
    torch, smb, dist = env.torch, env.smb, env.dist
    if wl.kind == "decode":
        return None
    m, n, k, n_local, g = wl.m, wl.n, wl.k, wl.n_local, env.world
    shared = smb.sharding.SharedOutput(m, n, dist)
    d_full = shared.local_tensor()
    if wl.kind == "bf16":
        fplan = smb.gemm.Bf16Plan(wl.a, wl.bt, shared.slab_address(), m, n_local, k, ldd=n,
                                  flags=smb.capi.FLAG_OPERANDS_STATIC)
    else:
        fplan = smb.gemm.Fp4Plan(wl.a, wl.sfa, wl.bt, wl.sfb, shared.slab_address(), m, n_local, k, ldd=n,
                                 flags=smb.capi.FLAG_OPERANDS_STATIC)
    fplan.set_peer_copies(shared.peer_targets(), n)
    for _ in range(3):
        fplan.run(env.stream)
    fplan.check(env.stream)
    env.barrier()
    f0, f1 = env.event(), env.event()
    reps = max(5, min(steps, 50))
    f0.record(env.stream)
    for _ in range(reps):
        fplan.run(env.stream)
    f1.record(env.stream)
    env.barrier()
    fplan.check(env.stream)
    fused_ms = env.max_over_ranks(f0.elapsed_time(f1)) / reps
    own_ok = bool(torch.equal(d_full[:, wl.n0:wl.n0 + n_local].view(torch.int16), wl.d.view(torch.int16)))
    checksum = d_full.view(torch.int16).to(torch.int64).sum().reshape(1)
    lo, hi = checksum.clone(), checksum.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    ok_t = torch.tensor([1 if own_ok else 0], device=env.dev)
    dist.all_reduce(ok_t, op=dist.ReduceOp.MIN)
    sent = (g - 1) * m * n_local * 2
    out = {"fused_ms": fused_ms, "gemm_only_ms": ms_step,
           "fused_sent_gb_per_s_per_gpu": sent / (fused_ms * 1e-3) / 1e9,
           "fused_matches_unfused": bool(ok_t.item() == 1 and lo.item() == hi.item()),
           "fused_bound_ms": {"nvlink_at_770_gb_s": sent / 770e9 * 1e3, "gemm": ms_step},
           "fused_layout": "row-major [M, N] on every GPU"}
    fplan.close()
    del d_full
    shared.close()
    return out


def fused_reduce_scatter_study(env: Env, wl: Workload, steps: int) -> dict | None:
    """Row-parallel form of the same problem: rank r multiplies [M, K/g] by [N, K/g]; the sum of the
    g partial products is scattered by rows.  Fused: the epilogue stores row block b of the partial
    product into slot r of rank b's receive buffer (peer-mapped memory), a one-element all-reduce
    orders the ranks, a slot-sum kernel adds the g slots.  Unfused: GEMM + NCCL reduce_scatter."""
    torch, smb, dist = env.torch, env.smb, env.dist
    m, n, k, g, fill = wl.m, wl.n, wl.k, env.world, wl.fill
    if wl.kind != "bf16" or k % g != 0 or m % (256 * g) != 0:
        return None
    kl = k // g
    a_r = torch.empty(m, kl, device=env.dev, dtype=torch.bfloat16)
    bt_r = torch.empty(n, kl, device=env.dev, dtype=torch.bfloat16)
    smb.gemm.fill_bf16_device(a_r, m, kl, fill, 11 + env.rank, stream=env.stream)
    smb.gemm.fill_bf16_device(bt_r, n, kl, fill, 101 + env.rank, stream=env.stream)
    slots = smb.sharding.ScatterSlots(m, n, dist)
    rows = slots.rows_per_block
    partial = torch.empty(m, n, device=env.dev, dtype=torch.bfloat16)
    mine = torch.empty(rows, n, device=env.dev, dtype=torch.bfloat16)
    mine_nccl = torch.empty(rows, n, device=env.dev, dtype=torch.bfloat16)
    token = torch.zeros(1, device=env.dev, dtype=torch.float32)
    rplan = smb.gemm.Bf16Plan(a_r, bt_r, partial, m, n, kl, flags=smb.capi.FLAG_OPERANDS_STATIC)
    rplan.set_row_route(slots.targets(), rows, n, slots.first_block())
    uplan = smb.gemm.Bf16Plan(a_r, bt_r, partial, m, n, kl, flags=smb.capi.FLAG_OPERANDS_STATIC)

    def fused_step():
        rplan.run(env.stream)
        dist.all_reduce(token)          # every rank's deliveries are complete behind this point
        smb.gemm.sum_slots_bf16_device(slots.local, mine, g, rows * n, stream=env.stream)
        dist.all_reduce(token)          # nobody overwrites a slot that is still being summed

    def unfused_step():
        uplan.run(env.stream)
        dist.reduce_scatter_tensor(mine_nccl, partial)

    def timed(fn, reps):
        for _ in range(2):
            fn()
        env.barrier()
        t0, t1 = env.event(), env.event()
        t0.record(env.stream)
        for _ in range(reps):
            fn()
        t1.record(env.stream)
        env.barrier()
        return env.max_over_ranks(t0.elapsed_time(t1)) / reps

    reps = max(5, min(steps, 30))
    fused_ms = timed(fused_step, reps)
    rplan.check(env.stream)
    unfused_ms = timed(unfused_step, reps)
    gemm_ms = timed(lambda: uplan.run(env.stream), reps)
    # Same sums up to the order of additions and one rounding.
    diff = (mine.float() - mine_nccl.float()).abs().max()
    scale = mine_nccl.float().abs().max().clamp_min(1e-30)
    agree = torch.tensor([float(diff / scale)], device=env.dev)
    dist.all_reduce(agree, op=dist.ReduceOp.MAX)
    sent = (g - 1) * rows * n * 2
    out = {"fused_ms": fused_ms, "gemm_plus_nccl_reduce_scatter_ms": unfused_ms, "gemm_only_ms": gemm_ms,
           "shape_per_rank_mnk": [m, n, kl], "fused_sent_gb_per_s_per_gpu": sent / (fused_ms * 1e-3) / 1e9,
           "max_rel_diff_vs_nccl": float(agree.item()),
           "bound_ms": {"nvlink_at_770_gb_s": sent / 770e9 * 1e3, "gemm": gemm_ms}}
    rplan.close()
    uplan.close()
    del partial, mine, mine_nccl, a_r, bt_r
    slots.close()
    return out


def measure(env: Env, name: str, steps: int | None, warmup: int, args, headline: bool) -> dict:
    """One workload, start to finish: operands, timed region, roofline, end-to-end leg, CPU
    baseline; for the headline also the optional studies named on the command line."""
    wl = Workload(env, name)
    rec = time_workload(env, wl, steps, warmup, not args.no_extra_warmup)
    rec["dtype"] = dtype_for(wl.kind)
    rec["config"] = config_for(name, env.world)
    rec["l2"] = (f"operands + output resident per GPU = {wl.resident_bytes / 1e6:.0f} MB > 126 MB L2 (no flush)"
                 if wl.kind != "decode" else
                 f"{DECODE_WEIGHT_SETS} rotating weight sets = {wl.resident_bytes / 1e6:.0f} MB > 126 MB L2")
    rec["per_gpu_tflops"] = rec["value"] / env.world
    ms_step = rec["ms_per_step"]
    if wl.kind == "decode" and wl.fill != 16:
        rec["from_bf16_activations"] = decode_from_bf16_study(env, wl, rec["steps"], warmup)
    if env.dist is not None and (args.allgather or (not headline and name == "bf16_large")):
        rec["allgather"] = allgather_study(env, wl, ms_step)
    if headline:
        if args.swiglu:
            rec["swiglu"] = swiglu_study(env, wl, ms_step, rec["steps"])
        if env.dist is not None and args.fused_allgather:
            fused = fused_allgather_study(env, wl, ms_step, rec["steps"])
            if fused:
                rec["allgather"] = {**(rec.get("allgather") or {}), **fused}
        if env.dist is not None and args.fused_reduce_scatter:
            rec["reduce_scatter"] = fused_reduce_scatter_study(env, wl, rec["steps"])
    # End to end through host buffers.  The 5 GB large workload is left out: its step is a copy
    # benchmark of 1.5 GB up and 3.8 GB down.
    rec["e2e"] = None
    if name != "bf16_large" and args.e2e_steps > 0:
        rec["e2e"] = e2e_for(env, wl, args.e2e_steps)
    rec["cpu_baseline"] = None
    if env.rank == 0 and env.world == 1 and not args.no_cpu_baseline:
        rec["cpu_baseline"] = cpu_baseline_for(wl, 8.0 if headline else 2.5)
    wl.close()
    del wl
    env.torch.cuda.empty_cache()
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="time this workload alone (default: the headline BF16 8192^3 plus the sub-records "
                         "of the other workloads of the metric)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-workloads", action="store_true", help="headline only, no sub-records")
    ap.add_argument("--allgather", action="store_true", help="also time the all-gather of D (N > 1)")
    ap.add_argument("--fused-allgather", action="store_true",
                    help="also time the GEMM whose epilogue writes D into every GPU's full D (N > 1)")
    ap.add_argument("--fused-reduce-scatter", action="store_true",
                    help="also time the K-sharded form: GEMM whose epilogue delivers row blocks to their owners, "
                         "then a slot sum, against GEMM + NCCL reduce-scatter (BF16 workloads, N > 1)")
    ap.add_argument("--swiglu", action="store_true",
                    help="also time the GEMM with the gated-activation epilogue (D = silu(gate) * up, [M, N/2])")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra-warmup", action="store_true",
                    help="decode workloads: skip the 0.3 s warm-up (for profiler captures, where few "
                         "launches should precede the captured one)")
    ap.add_argument("--e2e-steps", type=int, default=8)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        return run_reference(args)

    env = Env()
    name = args.workload or HEADLINE
    head = measure(env, name, args.steps, args.warmup, args, headline=True)
    workloads = None
    if args.workload is None and not args.no_workloads:
        workloads = {}
        for sub, sub_steps, only_n in SUB_WORKLOADS:
            if only_n is not None and env.world not in only_n:
                continue
            workloads[sub] = measure(env, sub, sub_steps, max(3, min(args.warmup, 10)), args, headline=False)
    if env.rank == 0:
        kind = WORKLOADS[name][0]
        config = dict(head["config"])
        line = {
            "metric": "GEMM TFLOPS", "value": head["value"], "unit": "TFLOP/s", "n_gpus": env.world,
            "steps": head["steps"], "warmup": head["warmup"], "ms_per_step": head["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": dtype_for(kind), "data": "synthetic", "config": config,
            "notes": {"l2": head["l2"], "per_gpu_tflops": head["per_gpu_tflops"], "kernel": head["kernel"],
                      "extra_warmup_steps": head["extra_warmup_steps"],
                      "launch": "operands static across steps: consecutive launches may overlap head and tail "
                                "(programmatic dependent launch); stores to D stay ordered"},
            "clocks": head["clocks"], "roofline": head["roofline"], "cpu_baseline": head["cpu_baseline"],
            "e2e": head["e2e"], "gpu_launches": head["steps"],
        }
        for key in ("allgather", "from_bf16_activations", "swiglu", "reduce_scatter"):
            if head.get(key) is not None:
                line[key] = head[key]
        if workloads is not None:
            line["workloads"] = workloads
            line["gpu_launches_all_timed_regions"] = env.launches
        print(json.dumps(line))
    if env.dist is not None:
        if env._comm is not None:
            env._comm.close()
        env.dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
