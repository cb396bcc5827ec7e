#!/usr/bin/env python
"""Headline benchmark: fused SwiGLU gate/up stage, 32768 x 3072 x 12288, bf16.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A *step* is one pass of the hot path over the whole batch: one call of
``matmul_fused_swiglu(x, W)`` with x [32768, 3072] and the packed weight
W [3072, 24576] = [W_up | W_gate] (synthetic N(0,1) / N(0,1/sqrt(K)) values).
With N GPUs the 32768 rows are sharded across the ranks (weights replicated, no
collective), so total work is fixed: strong scaling.  Launched under torchrun
for N > 1; rank 0 prints ONE JSON line.

Fields beyond the common contract:
  roofline      tensor-core roofline of the kernel: algorithmic FLOPs per launch
                divided by the average launch duration (CUDA events over the
                timed region) against the measured cuBLAS bf16 peak of this pool;
  cpu_baseline  the reference's fp32 check expression (CPU oracle) timed on the
                host cores on a bounded row sample of the same workload;
  e2e           the same metric through the public operator with HOST buffers:
                pinned x and W copied in, h copied out, every step;
  silu_mul      the reference's other operator (`matmul_silu_mul`) on the same
                shape, device-resident, for the record.

``--impl reference`` times the reference's CPU path (its fp32 check expression,
restated in oracle/) on the host cores, rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

M_TOTAL, K_DIM, N_OUT = 32768, 3072, 12288
WORKLOAD = "c3_fused: matmul_fused_swiglu 32768x3072x12288 bf16, W=[W_up|W_gate] packed [3072,24576]"
METRIC = "fused_swiglu_tflops"
UNIT = "TFLOP/s"
PUBLISHED_V4_TFLOPS = 1257.0   # the reference README's V4 figure (README.md:106): 1x B200, same shape
# DRAM traffic of one full-size launch on one GPU: dram__bytes_read.sum + dram__bytes_write.sum
# from a one-pass ncu capture of this workload (profiles/swiglu_kernel_fused_c3_full_dram_traffic.md).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 2.27e9


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"tflops": float(d["bf16_tflops_sustained"]), "tflops_burst": float(d["bf16_tflops"]),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured (MEASURED_PEAKS.json, sustained)"}
    return {"tflops": 1400.0, "tflops_burst": 1590.0, "hbm_gbs": 6650.0,
            "source": "fallback (earlier measurement on this pool)"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap",
        0x8: "hw_slowdown", 0x10: "sync_boost", 0x20: "sw_thermal_slowdown",
        0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, index: int, period_s: float = 0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.mask, self.max_mhz = [], 0, None
        self._stop_evt = threading.Event()
        self.error = None

    def run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            while not self._stop_evt.is_set():
                self.samples.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                self.mask |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
                time.sleep(self.period)
        except Exception as e:  # NVML missing: report, do not fail the benchmark
            self.error = repr(e)

    def stop(self) -> dict:
        self._stop_evt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        reasons = [n for b, n in self.REASONS.items() if self.mask & b and n != "gpu_idle"]
        out = {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
               "reasons": reasons, "samples": len(s)}
        if self.error:
            out["error"] = self.error
        return out


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except (ValueError, IndexError):
            pass
    return local_rank


def cpu_reference_rate(target_s: float, threads: int) -> dict:
    """Times the reference's fp32 check expression on a row sample of the workload."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import swiglu_oracle as orc
    from swiglu_fused_b200.workloads import make_inputs

    torch.set_num_threads(threads)
    w = make_inputs(8, K_DIM, N_OUT, form="fused_swiglu", seed=0)["w"]
    x_all = make_inputs(M_TOTAL, K_DIM, 8, form="fused_swiglu", seed=1)["x"]
    orc.fused_swiglu(x_all[:256], w)                   # warm-up (thread pool, pages)
    # Grow the sample until it takes about target_s (or covers the whole workload).
    rows_target, dt = 1024, 0.0
    while True:
        t0 = time.perf_counter()
        orc.fused_swiglu(x_all[:rows_target], w)
        dt = time.perf_counter() - t0
        if rows_target >= M_TOTAL or dt >= 0.5 * target_s:
            break
        grow = max(2.0, min(16.0, 0.8 * target_s / max(dt, 1e-3)))
        rows_target = int(min(M_TOTAL, rows_target * grow)) // 128 * 128
    flops = 2.0 * rows_target * K_DIM * 2 * N_OUT
    return {"value": flops / dt / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{rows_target} of {M_TOTAL} rows of the c3 workload, full K and N, "
                      f"torch fp32 CPU, {dt:.2f} s", "rows": rows_target, "seconds": dt}


def gpu_baselines(x, w, n_out: int, iters: int, ours) -> dict:
    """Library baselines on the same GPU, same tensors: cuBLAS [M,2N] GEMM alone, plus eager
    and torch.compile'd ``silu(gu[:, N:]) * gu[:, :N]`` (the reference's B1/B2,
    ``bench_fused.py:52-62``).  Reported beside the kernel, never used by it.  The candidates
    are timed round-robin (three rounds, medians) together with this build's kernel, so that
    all of them see the same thermal / power-cap state."""
    import torch.nn.functional as F

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / iters

    def eager():
        gu = x @ w
        return F.silu(gu[:, n_out:]) * gu[:, :n_out]

    cands = {"this_build_ms": ours, "cublas_gemm_ms": lambda: x @ w,
             "cublas_plus_eager_act_ms": eager}
    out = {}
    try:
        act = torch.compile(lambda gu: F.silu(gu[:, n_out:]) * gu[:, :n_out])
        act(x @ w)                                   # compile outside the timing
        cands["cublas_plus_compiled_act_ms"] = lambda: act(x @ w)
    except Exception as e:  # inductor unavailable on this box
        out["cublas_plus_compiled_act_ms"] = None
        out["compile_error"] = repr(e)[:200]
    samples = {k: [] for k in cands}
    for _ in range(3):
        for k, fn in cands.items():
            samples[k].append(timed(fn))
    for k, v in samples.items():
        out[k] = sorted(v)[1]
    return out


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import swiglu_oracle as orc
    from swiglu_fused_b200.workloads import make_inputs

    torch.set_num_threads(threads)
    # Size a step at about 1.5 s of CPU work so that steps + warm-up end within minutes.
    probe = cpu_reference_rate(1.5, threads)
    rows = probe["rows"]
    w = make_inputs(8, K_DIM, N_OUT, form="fused_swiglu", seed=0)["w"]
    x = make_inputs(rows, K_DIM, 8, form="fused_swiglu", seed=1)["x"]
    for _ in range(min(args.warmup, 2)):
        orc.fused_swiglu(x, w)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.fused_swiglu(x, w)
    dt = (time.perf_counter() - t0) / args.steps
    flops = 2.0 * rows * K_DIM * 2 * N_OUT
    value = flops / dt / 1e12
    sample = (f"each step = {rows} of {M_TOTAL} rows of the c3 workload (full K, N), the reference's "
              f"fp32 check expression on CPU tensors, {threads} threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 2), "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "M": M_TOTAL, "K": K_DIM, "N": N_OUT,
                   "note": "CPU path of the reference (bench_fused.py:39-42 expression), bounded sample"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def run_ours(args) -> None:
    from swiglu_fused_b200 import _lib, matmul_fused_swiglu, matmul_silu_mul, sharding
    from swiglu_fused_b200.host_pipeline import HostPipeline
    from swiglu_fused_b200.workloads import make_inputs

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (sm_100a); there is no CPU fallback")
    rank, world, local_rank = sharding.init_from_env("nccl")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun "
                         f"--nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist

    m_total = args.rows or M_TOTAL
    rows = sharding.row_shard(m_total, world, rank)
    # Same global tensors on every rank (seeded CUDA generator); each keeps its rows.
    inp = make_inputs(m_total, K_DIM, N_OUT, form="fused_swiglu", seed=0, device=dev,
                      gen_device=str(dev))
    x_full, w = inp["x"], inp["w"]
    x = x_full[rows.begin:rows.end].clone() if world > 1 else x_full
    del x_full, inp
    h = torch.empty((rows.count, N_OUT), dtype=torch.bfloat16, device=dev)
    flops_total = 2.0 * m_total * K_DIM * 2 * N_OUT
    flops_local = 2.0 * rows.count * K_DIM * 2 * N_OUT

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.form == "silu_mul":
        # Profiling aid: time the reference's other operator instead (W_gate = right half of
        # the packed weight, up = x @ W_up precomputed outside the timed region).
        w_gate = w[:, N_OUT:].contiguous()
        up = x @ w[:, :N_OUT].contiguous()
        flops_total, flops_local = flops_total / 2, flops_local / 2

        def step():
            matmul_silu_mul(x, w_gate, up, out=h)
    else:
        def step():
            matmul_fused_swiglu(x, w, out=h)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    barrier()
    _lib.device_status()

    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    launches0 = _lib.kernel_launches()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    barrier()
    elapsed_ms = start.elapsed_time(stop)
    launches = _lib.kernel_launches() - launches0
    clocks = sampler.stop()
    _lib.device_status()

    t = torch.tensor([elapsed_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = t.item() / args.steps
    value = flops_total / (ms_per_step * 1e-3) / 1e12

    # ---- end to end: host buffers in, host buffer out, every step ----
    e2e = None
    if not args.no_e2e and args.form == "fused_swiglu":
        e2e_steps = max(2, min(args.steps, 8))
        pipe = HostPipeline(rows.count, K_DIM, N_OUT, device=dev)
        x_host = torch.empty((rows.count, K_DIM), dtype=torch.bfloat16).pin_memory()
        w_host = torch.empty((K_DIM, 2 * N_OUT), dtype=torch.bfloat16).pin_memory()
        h_host = torch.empty((rows.count, N_OUT), dtype=torch.bfloat16).pin_memory()
        x_host.copy_(x)
        w_host.copy_(w)
        for _ in range(2):
            pipe.run(x_host, w_host, h_host)
        e2e_launch0 = _lib.kernel_launches()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            pipe.run(x_host, w_host, h_host)
        torch.cuda.synchronize()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        e2e_launches = _lib.kernel_launches() - e2e_launch0
        te = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_same = bool(torch.equal(h_host.to(dev).view(torch.int16), h.view(torch.int16)))
        e2e = {"value": flops_total / te.item() / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": 2 * (x.numel() + w.numel()),
               "d2h_bytes_per_step": 2 * h.numel(), "ms_per_step": te.item() * 1e3,
               "steps": e2e_steps, "launches": e2e_launches, "matches_device_run": e2e_same,
               "note": "per rank: pinned host x and W copied in, h copied out, every step, by one "
                       "sgl_host_pipeline_run call (3 streams; the first rows are computed per "
                       "weight column window so the copy out starts while W is still arriving); "
                       "timed on the host clock around the calls, max over ranks"}
        pipe.close()
        del pipe, x_host, w_host, h_host

    peaks = load_peaks()
    achieved = flops_local / (elapsed_ms / args.steps * 1e-3) / 1e12   # this rank's kernel
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": (value / PUBLISHED_V4_TFLOPS)
        if (world == 1 and m_total == M_TOTAL and args.form == "fused_swiglu") else None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD if (m_total == M_TOTAL and args.form == "fused_swiglu") else
                   f"matmul_silu_mul {m_total}x{K_DIM}x{N_OUT} (profiling aid, not the headline)"
                   if args.form == "silu_mul" else
                   f"reduced-M case of c3 ({m_total} rows) for profiling, not a headline number",
                   "M": m_total, "K": K_DIM, "N": N_OUT,
                   "rows_per_gpu": rows.count, "parallelism": f"M-sharded x{world}, weights replicated, no collective",
                   "l2": "inputs+output larger than L2 (x+W+h per GPU = "
                         f"{(x.numel() + w.numel() + h.numel()) * 2 / 1e6:.0f} MB > 126 MB), no flush"},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops"],
                     "unit": "TFLOP/s", "frac": achieved / peaks["tflops"],
                     "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH if (world == 1 and m_total == M_TOTAL) else None,
                     "algorithmic_bytes": 2.0 * (rows.count * K_DIM + 2 * K_DIM * N_OUT + rows.count * N_OUT),
                     "peak_source": peaks["source"],
                     "frac_of_burst_peak": achieved / peaks["tflops_burst"],
                     "frac_of_nominal_2250": achieved / 2250.0},
        "clocks": clocks,
        "e2e": e2e,
        "gpu_launches": launches,
    }

    if world == 1 and m_total == M_TOTAL and args.form == "fused_swiglu":
        # The reference's other operator on the same shape, device-resident.
        inp3 = make_inputs(M_TOTAL, K_DIM, N_OUT, form="silu_mul", seed=0, device=dev,
                           gen_device=str(dev))
        up = inp3["x"] @ inp3["w_up"]
        h3 = torch.empty_like(up)
        for _ in range(3):
            matmul_silu_mul(inp3["x"], inp3["w_gate"], up, out=h3)
        torch.cuda.synchronize()
        s3, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n3 = max(3, args.steps // 2)
        s3.record()
        for _ in range(n3):
            matmul_silu_mul(inp3["x"], inp3["w_gate"], up, out=h3)
        e3.record()
        torch.cuda.synchronize()
        ms3 = s3.elapsed_time(e3) / n3
        line["silu_mul"] = {"workload": "c2_silu_mul 32768x3072x12288", "ms_per_call": ms3,
                            "tflops": 2.0 * M_TOTAL * K_DIM * N_OUT / (ms3 * 1e-3) / 1e12,
                            "published_ms": 2.281}
        del inp3, up, h3
        _lib.device_status()
        if not args.no_gpu_baselines:
            gb = gpu_baselines(x, w, N_OUT, max(5, args.steps // 2), step)
            b = gb.get("cublas_plus_compiled_act_ms") or gb.get("cublas_plus_eager_act_ms")
            gb["speedup_vs_cublas_plus_act"] = b / gb["this_build_ms"] if b else None
            gb["note"] = "round-robin timing, medians of 3 rounds; speedup uses this_build_ms"
            line["gpu_baselines"] = gb
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = {k: v for k, v in cpu_reference_rate(12.0, os.cpu_count() or 1).items()
                                    if k in ("value", "unit", "cores", "kind", "sample")}

    if rank == 0:
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def emit(line: dict) -> None:
    """Write the one JSON line to the process's real stdout."""
    os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())


# Libraries (NCCL prints its version banner) write to stdout too; keep fd 1 for the JSON
# line alone and send everything else to stderr.
_REAL_STDOUT = os.dup(1)


def main() -> None:
    sys.stdout.flush()
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true",
                    help="skip the CPU-baseline leg (it takes about 15 s)")
    ap.add_argument("--rows", type=int, default=0,
                    help="override M (profiling a reduced case under ncu); 0 = the full 32768")
    ap.add_argument("--form", choices=("fused_swiglu", "silu_mul"), default="fused_swiglu",
                    help="operator to time; silu_mul is a profiling aid, the headline is fused_swiglu")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-gpu-baselines", action="store_true",
                    help="skip the cuBLAS (+ eager / compiled activation) legs")
    args = ap.parse_args()
    if args.steps < 1:
        raise SystemExit("--steps must be >= 1")
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
