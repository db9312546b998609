#!/usr/bin/env python
"""Headline benchmark of the dense GEMM path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one pass of the hot path over one batch of synthetic input: one GEMM of the
named workload (default: BF16 8192^3, operands N(0,1)*0.1 stand-in, FP32 accumulate, BF16 out).
With N > 1 (launched under torch.distributed.run, one rank per GPU) the N dimension is sharded
column-parallel: rank r computes D[:, r*N/g : (r+1)*N/g] with no communication in the kernel;
the optional all-gather of D is timed separately and reported under "allgather" (--allgather: NCCL
all-gather + the library's unshard copy; --fused-allgather: the GEMM whose epilogue writes its
slab into the full D of every GPU over peer-mapped memory).

Rank 0 prints ONE JSON line.  `value` is whole-job TFLOP/s with operands resident in HBM
(device-timed, max over ranks); `e2e` is the same metric through the host-buffer entry point of
the C ABI with the host<->device copies inside the timed region; `roofline` relates the kernel
to the measured tensor peak; `cpu_baseline` is the reference's NumPy CPU path timed on this
host's cores on a bounded sample.

`--impl reference` times that NumPy CPU path alone (the reference has no other CPU
implementation of this path), on the same metric and config.
"""
from __future__ import annotations

import argparse
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
# A timed loop of back-to-back launches longer than this runs under the power cap: its tensor
# roofline uses the sustained cuBLAS figure, a shorter one the burst figure.
SUSTAINED_AFTER_S = 0.1
DECODE_WEIGHT_SETS = 4   # rotate weight buffers so that every step streams from HBM, not from L2

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of the
# dominant kernel on this workload at 1 GPU; the summaries are under profiles/).
NCU_TRAFFIC_BYTES = {"bf16_8192": 970_156_544, "nvfp4_8192": 255_423_744, "decode_m16": 128_138_240,
                     "decode_m128": 128_483_072}

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

    def __init__(self, uuid: str | None, index: int, period_s: float = 0.005):
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


def blas_info():
    """(threads, description) of the BLAS behind NumPy's matmul, the library the reference's CPU path
    spends its time in; threads falls back to the core count when the pool cannot be inspected."""
    cores = os.cpu_count() or 1
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


def cpu_gemm_rate(oracle, a_bits, bt_bits, budget_s: float):
    """Time the reference's CPU path (bf16 -> fp32, fp32 matmul, round to bf16) on as large a
    square sub-block as fits the time budget.  Returns (TFLOP/s, description, seconds)."""
    k = a_bits.shape[1]
    probe = min(512, a_bits.shape[0], bt_bits.shape[0])
    t0 = time.perf_counter()
    oracle.gemm_bf16_reference(a_bits[:probe], bt_bits[:probe])
    dt = max(time.perf_counter() - t0, 1e-4)
    rate = 2.0 * probe * probe * k / dt
    side = int((budget_s * rate / (2.0 * k)) ** 0.5)
    side = max(256, min(side // 256 * 256, a_bits.shape[0], bt_bits.shape[0]))
    best = None
    for _ in range(2):
        t0 = time.perf_counter()
        oracle.gemm_bf16_reference(a_bits[:side], bt_bits[:side])
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


def run_reference(args):
    """The reference arm: the reference's NumPy CPU GEMM on this host's cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    kind, m, n, k, fill, desc = WORKLOADS[args.workload]
    oracle = _load_oracle()
    cores, blas = blas_info()
    steps, warmup = args.steps, args.warmup
    # Bounded sample: the whole run must end within a few minutes.
    per_step_budget = max(0.05, min(2.0, 120.0 / max(1, steps + warmup)))
    rows = min(m, 4096)
    cols = min(n, 4096)
    if kind == "bf16":
        a_bits, bt_bits = oracle.bf16_operands(min(rows, 1024), min(cols, 1024), k, 2 if fill > 4 else fill)
        # Tile the small generated block up to the sample size: the timing does not depend on values.
        a_bits = np.tile(a_bits, (max(1, rows // a_bits.shape[0]), 1))
        bt_bits = np.tile(bt_bits, (max(1, cols // bt_bits.shape[0]), 1))
        run = lambda side: oracle.gemm_bf16_reference(a_bits[:side], bt_bits[:side])
    else:
        ac, asf = oracle.fp4_operand(min(rows, 512), k, 2, 0)
        bc, bsf = oracle.fp4_operand(min(cols, 512), k, 2, 1)
        reps = max(1, rows // ac.shape[0])
        ac, asf = np.tile(ac, (reps, 1)), np.tile(asf, (reps, 1))
        bc, bsf = np.tile(bc, (reps, 1)), np.tile(bsf, (reps, 1))
        run = lambda side: oracle.gemm_nvfp4_reference(ac[:side], asf[:side], bc[:side], bsf[:side])
    limit = min(a_bits.shape[0], bt_bits.shape[0]) if kind == "bf16" else min(ac.shape[0], bc.shape[0])
    probe = min(256, limit)
    t0 = time.perf_counter()
    run(probe)
    rate = 2.0 * probe * probe * k / max(time.perf_counter() - t0, 1e-4)
    side = int((per_step_budget * rate / (2.0 * k)) ** 0.5)
    side = max(128, min(side // 128 * 128, limit))
    for _ in range(warmup):
        run(side)
    t0 = time.perf_counter()
    for _ in range(steps):
        run(side)
    dt = time.perf_counter() - t0
    flops = 2.0 * side * side * k * steps
    value = flops / dt / 1e12
    line = {
        "impl": "reference", "metric": "GEMM TFLOPS", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": dt / steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16" if kind == "bf16" else "e2m1", "data": "synthetic",
        "config": {"workload": args.workload, "description": desc, "shape_mnk": [m, n, k],
                   "step": f"reference NumPy CPU path on a {side}x{side}x{k} sub-block"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"{side}x{side}x{k} sub-block per step, {steps} steps",
                         "host_cpus": os.cpu_count(), "blas": blas},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="bf16_8192", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
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

    import torch
    import __graft_entry__ as entry

    smb = entry.load_package()
    smb.capi.lib()   # fails loudly if the CUDA library is missing: there is no CPU fallback
    oracle = None

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    g = world

    kind, m, n, k, fill, desc = WORKLOADS[args.workload]
    try:
        shard = smb.sharding.column_shard(n, g, rank)
    except ValueError as err:
        raise SystemExit(str(err))
    n_local, n0 = shard.n_local, shard.n0
    stream = torch.cuda.current_stream()
    plans = None
    lib_q = smb.capi.lib()

    # ---------------------------------------------------------------- operands, resident in HBM
    if kind == "bf16":
        a = torch.empty(m, k, device=dev, dtype=torch.bfloat16)
        bt = torch.empty(n_local, k, device=dev, dtype=torch.bfloat16)
        d = torch.empty(m, n_local, device=dev, dtype=torch.bfloat16)
        smb.gemm.bf16_operands_device(a, bt, m, n_local, k, fill, n0=n0, n_total=n, stream=stream)
        plan = smb.gemm.Bf16Plan(a, bt, d, m, n_local, k, flags=smb.capi.FLAG_OPERANDS_STATIC)
        resident_bytes = a.numel() * 2 + bt.numel() * 2 + d.numel() * 2
        dtype = "bf16"
    elif kind == "decode":
        a = torch.empty(m, k // 2, device=dev, dtype=torch.uint8)
        sfa = torch.empty(smb.gemm.sf_packed_bytes(m, k), device=dev, dtype=torch.uint8)
        smb.gemm.fill_fp4_device(a, sfa, None, m, k, 6, 0, 0, stream=stream)
        d = torch.empty(m, n_local, device=dev, dtype=torch.bfloat16)
        weights, plans = [], []
        block16 = (fill == 16)

        def quantize_b16(rows_, codes_, seed_):
            """Gaussian data quantised on the device: E2M1 + E4M3 scale per 16 K."""
            import ctypes as C
            sf_ = torch.empty(smb.gemm.sf_packed_bytes(rows_, 2 * k), device=dev, dtype=torch.uint8)
            gen = torch.Generator(device=dev).manual_seed(seed_)
            x = torch.randn(rows_, k, device=dev, generator=gen)
            gs = 448.0 * 6.0 / float(x.abs().max())
            smb.capi.check(lib_q.smb_quantize_nvf4_device(x.data_ptr(), k, C.c_float(gs), codes_.data_ptr(), k // 2,
                                                          sf_.data_ptr(), None, rows_, k, int(stream.cuda_stream)))
            torch.cuda.synchronize()
            return sf_, gs

        if block16:
            sfa, gs_a = quantize_b16(m, a, 99)
        for i in range(DECODE_WEIGHT_SETS):
            w = torch.empty(n_local, k // 2, device=dev, dtype=torch.uint8)
            if block16:
                sfw, gs_w = quantize_b16(n_local, w, 1000 + rank * 16 + i)
                pl = smb.gemm.Fp4Plan(a, sfa, w, sfw, d, m, n_local, k, flags=smb.capi.FLAG_SCALE_BLOCK16)
                pl.set_alpha(1.0 / (gs_a * gs_w))
            else:
                sfw = torch.empty(smb.gemm.sf_packed_bytes(n_local, k), device=dev, dtype=torch.uint8)
                # Different rows of the same logical generator for every set.
                smb.gemm.fill_fp4_device(w, sfw, None, n_local, k, fill, 1, n0 + i * n, stream=stream)
                pl = smb.gemm.Fp4Plan(a, sfa, w, sfw, d, m, n_local, k)
            weights.append((w, sfw))
            plans.append(pl)
        plan = plans[0]
        resident_bytes = DECODE_WEIGHT_SETS * (weights[0][0].numel() + weights[0][1].numel())
        dtype = "e2m1"
    else:
        a = torch.empty(m, k // 2, device=dev, dtype=torch.uint8)
        sfa = torch.empty(smb.gemm.sf_packed_bytes(m, k), device=dev, dtype=torch.uint8)
        bt = torch.empty(n_local, k // 2, device=dev, dtype=torch.uint8)
        sfb = torch.empty(smb.gemm.sf_packed_bytes(n_local, k), device=dev, dtype=torch.uint8)
        d = torch.empty(m, n_local, device=dev, dtype=torch.bfloat16)
        if fill == 16:
            # NVFP4 proper: Gaussian data quantised on the device, E4M3 scale per 16 K, the two
            # per-tensor factors folded into the plan's output factor.
            import ctypes as C
            sfa = torch.empty(smb.gemm.sf_packed_bytes(m, 2 * k), device=dev, dtype=torch.uint8)
            sfb = torch.empty(smb.gemm.sf_packed_bytes(n_local, 2 * k), device=dev, dtype=torch.uint8)
            gen = torch.Generator(device=dev).manual_seed(1234 + rank)
            factors = []
            for rows_, codes_, sf_ in ((m, a, sfa), (n_local, bt, sfb)):
                x = torch.randn(rows_, k, device=dev, generator=gen)
                gs = 448.0 * 6.0 / float(x.abs().max())
                smb.capi.check(lib_q.smb_quantize_nvf4_device(x.data_ptr(), k, C.c_float(gs), codes_.data_ptr(), k // 2,
                                                              sf_.data_ptr(), None, rows_, k, int(stream.cuda_stream)))
                factors.append(gs)
                torch.cuda.synchronize()
                del x
            plan = smb.gemm.Fp4Plan(a, sfa, bt, sfb, d, m, n_local, k,
                                    flags=smb.capi.FLAG_OPERANDS_STATIC | smb.capi.FLAG_SCALE_BLOCK16)
            plan.set_alpha(1.0 / (factors[0] * factors[1]))
        else:
            smb.gemm.fill_fp4_device(a, sfa, None, m, k, fill, 0, 0, stream=stream)
            smb.gemm.fill_fp4_device(bt, sfb, None, n_local, k, fill, 1, n0, stream=stream)
            plan = smb.gemm.Fp4Plan(a, sfa, bt, sfb, d, m, n_local, k, flags=smb.capi.FLAG_OPERANDS_STATIC)
        resident_bytes = a.numel() + bt.numel() + sfa.numel() + sfb.numel() + d.numel() * 2
        dtype = "e2m1"
    torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # The decode steps are shorter (18 us) than a Python method call chain: launch through the
    # C entry point directly, with the handles and the stream pointer looked up once.
    lib = smb.capi.lib()
    stream_ptr = int(stream.cuda_stream)
    run_fn = lib.smb_bf16_plan_run if kind == "bf16" else lib.smb_fp4_plan_run
    handles = [pl._h for pl in (plans or [plan])]

    def run_step(i: int) -> None:
        if run_fn(handles[i % len(handles)], stream_ptr) != 0:
            raise RuntimeError(smb.capi.last_error())

    # ---------------------------------------------------------------- device-timed region
    for i in range(args.warmup):
        run_step(i)
    plan.check(stream)
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
    while (kind == "decode" and not args.no_extra_warmup and time.perf_counter() - warm_t0 < MIN_WARM_S
           and extra_warm < 100000):
        for i in range(20):
            run_step(extra_warm + i)
        extra_warm += 20
        torch.cuda.synchronize()
        if burst is None and time.perf_counter() - warm_t0 >= BURST_AFTER_S:
            b0 = torch.cuda.Event(enable_timing=True)
            b1 = torch.cuda.Event(enable_timing=True)
            b0.record(stream)
            for i in range(args.steps):
                run_step(i)
            b1.record(stream)
            torch.cuda.synchronize()
            burst = b0.elapsed_time(b1) / args.steps
            extra_warm += args.steps
    uuid = None
    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(dev).uuid)
    except Exception:
        uuid = None
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(uuid, local_rank) as sampler:
        e0.record(stream)
        for i in range(args.steps):
            run_step(i)
        e1.record(stream)
        barrier()
    for pl in (plans or [plan]):
        pl.check(stream)
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_local = e0.elapsed_time(e1)
    ms_step = ms_total / args.steps
    flops_step = 2.0 * m * n * k
    value = flops_step / (ms_step * 1e-3) / 1e12
    clocks = sampler.summary()

    # ---------------------------------------------------------------- roofline of the kernel
    peaks, peak_kind = _peaks()
    launch_ms = ms_local / args.steps
    achieved = 2.0 * m * n_local * k / (launch_ms * 1e-3) / 1e12
    timed_s = ms_total * 1e-3
    if kind == "decode":
        # Algorithmic bytes of one launch: weights + weight scales + activations + their scales + D.
        sf_k = 16 if fill == 16 else 32   # K values per scale byte
        algo_bytes = n_local * k // 2 + n_local * k // sf_k + m * k // 2 + m * k // sf_k + 2 * m * n_local
        gbs = algo_bytes / (launch_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": gbs / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES.get(args.workload) if g == 1 else None,
                    "peak_source": f"{peak_kind} device copy GB/s", "nominal_frac": gbs / 8000.0,
                    "algorithmic_bytes_per_launch": algo_bytes}
        if burst is not None:
            # Not the headline: the same launches timed 30 ms into the warm-up, before the clocks
            # have come down to where they stay under this load.
            roofline["burst"] = {"us_per_step": burst * 1e3, "achieved": algo_bytes / (burst * 1e-3) / 1e9,
                                 "unit": "GB/s", "nominal_frac": algo_bytes / (burst * 1e-3) / 1e9 / 8000.0,
                                 "steps": args.steps, "after_warm_s": BURST_AFTER_S}
    elif kind == "bf16":
        sustained = timed_s >= SUSTAINED_AFTER_S
        peak = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) if sustained else peaks["bf16_tflops"]
        peak_note = f"{peak_kind} cuBLAS bf16 {'sustained' if sustained else 'burst'} TFLOP/s"
    else:
        # No FP4 entry in the measured peaks: four times the measured dense bf16 rate (the ratio
        # of the nominal dense FP4 and BF16 figures, 9 and 2.25 PFLOP/s).
        sustained = timed_s >= SUSTAINED_AFTER_S
        base = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) if sustained else peaks["bf16_tflops"]
        peak = 4.0 * base
        peak_note = f"4 x {peak_kind} cuBLAS bf16 TFLOP/s (no measured FP4 figure)"
    if kind != "decode":
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(args.workload) if g == 1 else None,
                    "peak_source": peak_note,
                    "frac_of_burst": achieved / (peaks["bf16_tflops"] * (1 if kind == "bf16" else 4)),
                    "nominal_frac": achieved / (2250.0 if kind == "bf16" else 9000.0)}

    # ---------------------------------------------------------------- decode step from BF16 activations
    # The step as a model runs it: the activations arrive as BF16 and are quantised on the device
    # by a kernel chained in front of every GEMM (two launches per step).  Secondary figure; the
    # headline above starts from quantised activations, as the reference's metric does.
    act_step = None
    if kind == "decode" and fill != 16:
        x16 = torch.empty(m, k, device=dev, dtype=torch.bfloat16)
        smb.gemm.fill_bf16_device(x16, m, k, 5, 1, stream=stream)
        aplans = [smb.gemm.Fp4Plan.from_bf16_activations(x16, w, sfw, d, m, n_local, k) for (w, sfw) in weights]
        ahandles = [pl._h for pl in aplans]
        for i in range(max(3, args.warmup)):
            aplans[i % len(aplans)].run(stream)
        aplans[0].check(stream)
        a0 = torch.cuda.Event(enable_timing=True)
        a1 = torch.cuda.Event(enable_timing=True)
        barrier()
        a0.record(stream)
        for i in range(args.steps):
            if run_fn(ahandles[i % len(ahandles)], stream_ptr) != 0:
                raise RuntimeError(smb.capi.last_error())
        a1.record(stream)
        barrier()
        for pl in aplans:
            pl.check(stream)
        act_ms = max_over_ranks(a0.elapsed_time(a1)) / args.steps
        # The same two kernels in plain stream order (no early start of the GEMM's weight loads).
        nplans = [smb.gemm.Fp4Plan.from_bf16_activations(x16, w, sfw, d, m, n_local, k,
                                                         flags=smb.capi.FLAG_NO_LAUNCH_OVERLAP)
                  for (w, sfw) in weights]
        for i in range(3):
            nplans[i % len(nplans)].run(stream)
        barrier()
        a0.record(stream)
        nhandles = [pl._h for pl in nplans]
        for i in range(args.steps):
            if run_fn(nhandles[i % len(nhandles)], stream_ptr) != 0:
                raise RuntimeError(smb.capi.last_error())
        a1.record(stream)
        barrier()
        for pl in nplans:
            pl.check(stream)
            pl.close()
        plain_ms = max_over_ranks(a0.elapsed_time(a1)) / args.steps
        act_bytes = algo_bytes + m * k * 2   # + the BF16 activations read by the quantiser
        act_step = {"us_per_step": act_ms * 1e3, "us_per_step_plain_stream_order": plain_ms * 1e3,
                    "gpu_launches_per_step": 2,
                    "gb_per_s": act_bytes / (act_ms * 1e-3) / 1e9,
                    "api": "smb_fp4_plan_create_bf16_activations + smb_fp4_plan_run"}
        for pl in aplans:
            pl.close()

    # ---------------------------------------------------------------- optional all-gather of D
    allgather = None
    if dist is not None and args.allgather:
        gathered = torch.empty(g, m, n_local, device=dev, dtype=torch.bfloat16)
        for _ in range(2):
            dist.all_gather_into_tensor(gathered, d)
        barrier()
        g0 = torch.cuda.Event(enable_timing=True)
        g1 = torch.cuda.Event(enable_timing=True)
        g0.record()
        reps = 5
        for _ in range(reps):
            dist.all_gather_into_tensor(gathered, d)
        g1.record()
        barrier()
        ag_ms = max_over_ranks(g0.elapsed_time(g1)) / reps
        # Rank-major [g, M, N/g] -> row-major [M, N] (the library's copy kernel).
        full = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        smb.gemm.unshard_columns_device(gathered, full, g, m, n_local, stream=torch.cuda.current_stream())
        barrier()
        u0 = torch.cuda.Event(enable_timing=True)
        u1 = torch.cuda.Event(enable_timing=True)
        u0.record()
        for _ in range(reps):
            smb.gemm.unshard_columns_device(gathered, full, g, m, n_local, stream=torch.cuda.current_stream())
        u1.record()
        barrier()
        un_ms = max_over_ranks(u0.elapsed_time(u1)) / reps
        recv = (g - 1) * m * n_local * 2
        allgather = {"ms": ag_ms, "recv_gb_per_s_per_gpu": recv / (ag_ms * 1e-3) / 1e9,
                     "layout": "rank-major [g, M, N/g]", "unshard_ms": un_ms,
                     "unshard_gb_per_s": 2.0 * m * n * 2 / (un_ms * 1e-3) / 1e9,
                     "unfused_total_ms": ms_step + ag_ms + un_ms}
        del gathered, full

    # ---------------------------------------------------------------- gated-activation epilogue
    # The rows of BT are read as interleaved (up, gate) pairs; the fused plan writes
    # silu(gate) * up, half as wide, against the plain GEMM followed by the same activation as
    # separate PyTorch element-wise kernels on its bf16 output.
    swiglu = None
    if args.swiglu and kind != "decode" and n_local % 2 == 0:
        d_act = torch.empty(m, n_local // 2, device=dev, dtype=torch.bfloat16)
        sflags = smb.capi.FLAG_OPERANDS_STATIC | smb.capi.FLAG_EPILOGUE_SWIGLU
        if kind == "bf16":
            splan = smb.gemm.Bf16Plan(a, bt, d_act, m, n_local, k, ldd=n_local // 2, flags=sflags)
        else:
            splan = smb.gemm.Fp4Plan(a, sfa, bt, sfb, d_act, m, n_local, k, ldd=n_local // 2, flags=sflags)
        reps = max(5, min(args.steps, 100))

        def timed(fn):
            for _ in range(3):
                fn()
            barrier()
            t0 = torch.cuda.Event(enable_timing=True)
            t1 = torch.cuda.Event(enable_timing=True)
            t0.record(stream)
            for _ in range(reps):
                fn()
            t1.record(stream)
            barrier()
            return max_over_ranks(t0.elapsed_time(t1)) / reps

        def unfused():
            plan.run(stream)
            torch.mul(torch.nn.functional.silu(d[:, 1::2]), d[:, 0::2], out=d_act)

        fused_ms = timed(lambda: splan.run(stream))
        splan.check(stream)
        unfused_ms = timed(unfused)
        swiglu = {"fused_ms": fused_ms, "gemm_then_torch_elementwise_ms": unfused_ms,
                  "gemm_only_ms": ms_step, "d_bytes_fused": m * (n_local // 2) * 2,
                  "tflops_fused": flops_step / g / (fused_ms * 1e-3) / 1e12}
        splan.close()
        del d_act

    # ---------------------------------------------------------------- GEMM + all-gather in one kernel
    # Every rank holds a full row-major D [M, N] that all processes map; the epilogue of rank r
    # stores its column slab into all g of them (plain stores over NVLink for the g - 1 remote
    # ones).  Timed like the main region: barrier + synchronize on both sides, max over ranks.
    if dist is not None and args.fused_allgather and kind != "decode":
        shared = smb.sharding.SharedOutput(m, n, dist)
        d_full = shared.local_tensor()
        if kind == "bf16":
            fplan = smb.gemm.Bf16Plan(a, bt, shared.slab_address(), m, n_local, k, ldd=n,
                                      flags=smb.capi.FLAG_OPERANDS_STATIC)
        else:
            fplan = smb.gemm.Fp4Plan(a, sfa, bt, sfb, shared.slab_address(), m, n_local, k, ldd=n,
                                     flags=smb.capi.FLAG_OPERANDS_STATIC)
        fplan.set_peer_copies(shared.peer_targets(), n)
        for _ in range(3):
            fplan.run(stream)
        fplan.check(stream)
        barrier()
        f0 = torch.cuda.Event(enable_timing=True)
        f1 = torch.cuda.Event(enable_timing=True)
        reps = max(5, min(args.steps, 50))
        f0.record(stream)
        for _ in range(reps):
            fplan.run(stream)
        f1.record(stream)
        barrier()
        fplan.check(stream)
        fused_ms = max_over_ranks(f0.elapsed_time(f1)) / reps
        # Every rank's full D must hold every rank's slab: own slab equals the unfused result, and
        # a checksum over the whole matrix is the same on all ranks.
        own_ok = bool(torch.equal(d_full[:, n0:n0 + n_local].view(torch.int16), d.view(torch.int16)))
        checksum = d_full.view(torch.int16).to(torch.int64).sum().reshape(1)
        lo, hi = checksum.clone(), checksum.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        ok_t = torch.tensor([1 if own_ok else 0], device=dev)
        dist.all_reduce(ok_t, op=dist.ReduceOp.MIN)
        sent = (g - 1) * m * n_local * 2
        allgather = dict(allgather or {})
        allgather.update({
            "fused_ms": fused_ms, "gemm_only_ms": ms_step,
            "fused_sent_gb_per_s_per_gpu": sent / (fused_ms * 1e-3) / 1e9,
            "fused_matches_unfused": bool(ok_t.item() == 1 and lo.item() == hi.item()),
            "fused_bound_ms": {"nvlink_at_770_gb_s": sent / 770e9 * 1e3, "gemm": ms_step},
            "fused_layout": "row-major [M, N] on every GPU"})
        fplan.close()
        del d_full
        shared.close()

    # ---------------------------------------------------------------- K-sharded GEMM + reduce-scatter
    # Row-parallel form of the same problem: rank r multiplies [M, K/g] by [N, K/g]; the sum of the
    # g partial products is scattered by rows (rank b owns rows [b M/g, (b+1) M/g)).  Fused: the
    # epilogue stores row block b of the partial product straight into slot r of rank b's receive
    # buffer (peer-mapped memory, plain stores), a one-element all-reduce on the stream orders
    # the ranks, and a slot-sum kernel adds the g slots.  Unfused: GEMM into a local [M, N]
    # buffer, then NCCL reduce_scatter_tensor.
    reduce_scatter = None
    if dist is not None and args.fused_reduce_scatter and kind == "bf16" and k % g == 0 and m % (256 * g) == 0:
        kl = k // g
        a_r = torch.empty(m, kl, device=dev, dtype=torch.bfloat16)
        bt_r = torch.empty(n, kl, device=dev, dtype=torch.bfloat16)
        smb.gemm.fill_bf16_device(a_r, m, kl, fill, 11 + rank, stream=stream)
        smb.gemm.fill_bf16_device(bt_r, n, kl, fill, 101 + rank, stream=stream)
        slots = smb.sharding.ScatterSlots(m, n, dist)
        rows = slots.rows_per_block
        partial = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        mine = torch.empty(rows, n, device=dev, dtype=torch.bfloat16)
        mine_nccl = torch.empty(rows, n, device=dev, dtype=torch.bfloat16)
        token = torch.zeros(1, device=dev, dtype=torch.float32)
        rplan = smb.gemm.Bf16Plan(a_r, bt_r, partial, m, n, kl, flags=smb.capi.FLAG_OPERANDS_STATIC)
        rplan.set_row_route(slots.targets(), rows, n, slots.first_block())
        uplan = smb.gemm.Bf16Plan(a_r, bt_r, partial, m, n, kl, flags=smb.capi.FLAG_OPERANDS_STATIC)

        def fused_step():
            rplan.run(stream)
            dist.all_reduce(token)          # every rank's deliveries are complete behind this point
            smb.gemm.sum_slots_bf16_device(slots.local, mine, g, rows * n, stream=stream)
            dist.all_reduce(token)          # nobody overwrites a slot that is still being summed

        def unfused_step():
            uplan.run(stream)
            dist.reduce_scatter_tensor(mine_nccl, partial)

        def timed_rs(fn, reps):
            for _ in range(2):
                fn()
            barrier()
            t0 = torch.cuda.Event(enable_timing=True)
            t1 = torch.cuda.Event(enable_timing=True)
            t0.record(stream)
            for _ in range(reps):
                fn()
            t1.record(stream)
            barrier()
            return max_over_ranks(t0.elapsed_time(t1)) / reps

        reps = max(5, min(args.steps, 30))
        fused_rs_ms = timed_rs(fused_step, reps)
        rplan.check(stream)
        unfused_rs_ms = timed_rs(unfused_step, reps)
        gemm_rs_ms = timed_rs(lambda: uplan.run(stream), reps)
        # Same sums up to the order of additions and one rounding.
        diff = (mine.float() - mine_nccl.float()).abs().max()
        scale = mine_nccl.float().abs().max().clamp_min(1e-30)
        agree = torch.tensor([float(diff / scale)], device=dev)
        dist.all_reduce(agree, op=dist.ReduceOp.MAX)
        sent = (g - 1) * rows * n * 2
        reduce_scatter = {"fused_ms": fused_rs_ms, "gemm_plus_nccl_reduce_scatter_ms": unfused_rs_ms,
                          "gemm_only_ms": gemm_rs_ms, "shape_per_rank_mnk": [m, n, kl],
                          "fused_sent_gb_per_s_per_gpu": sent / (fused_rs_ms * 1e-3) / 1e9,
                          "max_rel_diff_vs_nccl": float(agree.item()),
                          "bound_ms": {"nvlink_at_770_gb_s": sent / 770e9 * 1e3, "gemm": gemm_rs_ms}}
        rplan.close()
        uplan.close()
        del partial, mine, mine_nccl, a_r, bt_r
        slots.close()

    # ---------------------------------------------------------------- end to end, host buffers
    e2e = None
    if kind == "bf16":
        a_host = torch.empty(m, k, dtype=torch.int16).pin_memory()
        bt_host = torch.empty(n_local, k, dtype=torch.int16).pin_memory()
        d_host = torch.empty(m, n_local, dtype=torch.int16).pin_memory()
        a_host.copy_(a.view(torch.int16))
        bt_host.copy_(bt.view(torch.int16))
        ctx = smb.gemm.Bf16HostContext(m, n_local, k)
        for _ in range(2):
            ctx.run(a_host, bt_host, d_host)
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            ctx.run(a_host, bt_host, d_host)
        barrier()
        e2e_s = max_over_ranks(time.perf_counter() - t0) / args.e2e_steps
        same = bool(torch.equal(d_host, d.view(torch.int16).cpu()))
        e2e = {"value": flops_step / e2e_s / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(a_host.numel() * 2 + bt_host.numel() * 2),
               "d2h_bytes_per_step": int(d_host.numel() * 2), "ms_per_step": e2e_s * 1e3,
               "steps": args.e2e_steps, "matches_device_path": same,
               "api": "smb_bf16_host_ctx_run (pinned host buffers, per-GPU shard)"}
        ctx.close()

    # ---------------------------------------------------------------- CPU baseline (rank 0, N = 1)
    cpu_baseline = None
    if rank == 0 and g == 1 and not args.no_cpu_baseline and kind != "bf16":
        oracle = _load_oracle()
        rate, sample, secs = cpu_fp4_rate(oracle, m, n, k, budget_s=6.0)
        threads, blas = blas_info()
        cpu_baseline = {"value": rate, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                        "sample": sample + f" ({secs:.2f} s)", "host_cpus": os.cpu_count(), "blas": blas,
                        "what": "reference NumPy CPU path: E2M1 codes and UE8M0 scales -> fp32, a @ b, "
                                "round to bf16"}
    if rank == 0 and g == 1 and not args.no_cpu_baseline and kind == "bf16":
        oracle = _load_oracle()
        rows = min(m, 4096)
        a_np = a_host[:rows].numpy().view(np.uint16)
        bt_np = bt_host[:min(n_local, 4096)].numpy().view(np.uint16)
        rate, sample, secs = cpu_gemm_rate(oracle, a_np, bt_np, budget_s=8.0)
        threads, blas = blas_info()
        cpu_baseline = {"value": rate, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                        "sample": sample + f" ({secs:.2f} s)", "host_cpus": os.cpu_count(), "blas": blas,
                        "what": "reference NumPy CPU path: bf16 operands -> fp32, a @ b, round to bf16"}

    for pl in (plans or [plan]):
        pl.close()
    if rank == 0:
        line = {
            "metric": "GEMM TFLOPS", "value": value, "unit": "TFLOP/s", "n_gpus": g,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": dtype, "data": "synthetic",
            "config": {"workload": args.workload, "description": desc, "shape_mnk": [m, n, k],
                       "sharding": f"N column-parallel over {g} GPU(s), {n_local} columns each",
                       "l2": (f"operands + output resident per GPU = {resident_bytes / 1e6:.0f} MB > 126 MB L2 (no flush)"
                              if kind != "decode" else
                              f"{DECODE_WEIGHT_SETS} rotating weight sets = {resident_bytes / 1e6:.0f} MB > 126 MB L2"),
                       "per_gpu_tflops": value / g,
                       "extra_warmup_steps": extra_warm,
                       "launch": "operands static across steps: consecutive launches may overlap head and tail "
                                 "(programmatic dependent launch); stores to D stay ordered"},
            "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": args.steps, "allgather": allgather, "from_bf16_activations": act_step, "swiglu": swiglu, "reduce_scatter": reduce_scatter,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
