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
                timed region) against the measured cuBLAS bf16 peak of this pool
                (the burst figure while the timed region is shorter than a
                second, the sustained one beyond), with per-step event times;
  cpu_baseline  the reference's fp32 check expression (CPU oracle) timed on the
                host cores on a bounded row sample of the same workload;
  e2e           the same metric through the public operator with HOST buffers:
                pinned x and W copied in, h copied out, every step; at N > 1 every
                rank copies only its 1/N of W from the host and the ranks pass the
                pieces on over NVLink;
  silu_mul      the reference's other operator (`matmul_silu_mul`, configuration 2)
                on the same shape with its library comparators;
  gpu_baselines cuBLAS (+ eager / compiled activation) on the same tensors, timed
                in rotating order with this build's kernel;
  legs          the other configurations, each with parity flags computed inside
                the run: at N = 1 configuration 4 (16384 x 4096 x 14336) and its
                tile tail M = 64 / 256 / 1024; at N > 1 configuration 5
                (32768 x 8192 x 28672) column-parallel over the N ranks - compute
                only, with an NCCL all-gather, with the gather inside the kernel -
                and the row-parallel down projection with the reduce-scatter
                inside the GEMM.

``--impl reference`` times the reference's CPU path (its fp32 check expression,
restated in oracle/) on the host cores, rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import re
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
C4 = (16384, 4096, 14336)      # configuration 4: M, K, N (packed weight [4096, 28672], std 0.02)
C4_TAIL = (64, 256, 1024)
C5 = (32768, 8192, 28672)      # configuration 5 (packed weight [8192, 57344], std 0.02)
TRAFFIC_PROFILE = os.path.join(ROOT, "profiles", "swiglu_kernel_fused_c3_full_dram_traffic.md")


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"tflops_sustained": float(d["bf16_tflops_sustained"]),
                "tflops_burst": float(d["bf16_tflops"]), "hbm_gbs": float(d["hbm_gbs"]),
                "source": "measured (MEASURED_PEAKS.json)"}
    return {"tflops_sustained": 1400.0, "tflops_burst": 1590.0, "hbm_gbs": 6650.0,
            "source": "fallback (earlier measurement on this pool)"}


def profiled_traffic(form_name: str, M: int, N: int, K: int, cfg) -> float | None:
    """DRAM bytes per launch from the committed one-pass ncu summary, for exactly this problem
    and tile configuration; None when the summary has no line for it.  The summary carries
    machine-readable lines of the form
    ``traffic[fused_swiglu:32768x12288x3072 cta_group=2 block_k=128 group_m=16] = 2.27e9``."""
    if not os.path.exists(TRAFFIC_PROFILE):
        return None
    key = (f"{form_name}:{M}x{N}x{K} cta_group={cfg.cta_group} block_k={cfg.block_k} "
           f"group_m={cfg.group_m}" + (f" group_n={cfg.group_n}" if cfg.group_n else ""))
    with open(TRAFFIC_PROFILE) as f:
        for ln in f:
            m = re.match(r"\s*`?traffic\[(.+?)\]\s*=\s*([0-9.eE+]+)", ln)
            if m and m.group(1).strip() == key:
                return float(m.group(2))
    return None


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap",
        0x8: "hw_slowdown", 0x10: "sync_boost", 0x20: "sw_thermal_slowdown",
        0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, index: int, period_s: float = 0.002):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.max_mhz = [], None
        self._stop_evt = threading.Event()
        self.ready = threading.Event()      # NVML is up: samples from now on
        self.error = None

    def run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            self.ready.set()
            while not self._stop_evt.is_set():
                mhz = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
                mask = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
                self.samples.append((time.perf_counter(), mhz, mask))
                time.sleep(self.period)
        except Exception as e:  # NVML missing: report, do not fail the benchmark
            self.error = repr(e)
            self.ready.set()

    def begin(self) -> None:
        """Called right before the timed region: wait for NVML and note the time."""
        self.ready.wait(timeout=10)
        self.t_begin = time.perf_counter()

    def stop(self) -> dict:
        """Called right after the timed region.  Reports the samples taken inside it; a region
        shorter than one NVML query (several ranks querying at once take milliseconds each) may
        hold none, and then the samples next to it, taken while the same kernel ran as warm-up
        or just after, stand in and the record says so."""
        t_end = time.perf_counter()
        self._stop_evt.set()
        self.join(timeout=2)
        t0 = getattr(self, "t_begin", 0.0)
        inside = [v for v in self.samples if t0 <= v[0] <= t_end]
        used, where = inside, "inside the timed region"
        if not inside:
            before = [v for v in self.samples if v[0] < t0][-2:]
            after = [v for v in self.samples if v[0] > t_end][:1]
            used, where = before + after, "adjacent to the timed region (shorter than one query)"
        s = sorted(v[1] for v in used)
        mask = 0
        for v in used:
            mask |= v[2]
        reasons = [n for b, n in self.REASONS.items() if mask & b and n != "gpu_idle"]
        out = {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
               "sm_min_mhz": s[0] if s else None, "reasons": reasons, "samples": len(s),
               "sampled": where}
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


def spread(values) -> dict:
    v = sorted(values)
    return {"median": v[len(v) // 2], "min": v[0], "max": v[-1]}


def timed_calls(fn, iters: int) -> float:
    """Average device time of ``iters`` back-to-back calls (ms), CUDA events on the current
    stream."""
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    e.synchronize()
    return s.elapsed_time(e) / iters


def rotated_round_robin(cands: dict, rounds: int = 5, window_s: float = 0.3) -> dict:
    """Times every candidate ``rounds`` times in windows of about ``window_s`` seconds of
    back-to-back calls.  The order of the candidates is rotated by one place every round, so
    each candidate follows (and inherits the clocks and temperature left by) a different
    neighbour each time; reports median, min and max of the per-call time per candidate."""
    names = list(cands)
    iters = {}
    for n in names:                      # calibrate the window length, untimed
        cands[n]()
        torch.cuda.synchronize()
        t = max(timed_calls(cands[n], 3), 1e-3)
        iters[n] = max(3, min(20000, int(window_s * 1e3 / t)))
    samples = {n: [] for n in names}
    for r in range(rounds):
        order = names[r % len(names):] + names[:r % len(names)]
        for n in order:
            samples[n].append(timed_calls(cands[n], iters[n]))
    out = {n: dict(spread(samples[n]), iters_per_window=iters[n]) for n in names}
    out["order"] = "rotated"
    out["rounds"] = rounds
    out["window_s"] = window_s
    return out


def compiled_activation():
    """torch.compile'd ``silu(gu[:, N:]) * gu[:, :N]`` and ``silu(g) * up`` (the reference's
    fair baselines, bench_fused.py:52-62 and README.md:33), or (None, None, reason)."""
    import torch.nn.functional as F
    try:
        fused_act = torch.compile(lambda gu, n: F.silu(gu[:, n:]) * gu[:, :n], dynamic=False)
        silu_mul_act = torch.compile(lambda g, up: F.silu(g) * up, dynamic=False)
        return fused_act, silu_mul_act, None
    except Exception as e:  # inductor unavailable on this box
        return None, None, repr(e)[:200]


def fused_candidates(x, w, n_out: int, ours, act) -> dict:
    import torch.nn.functional as F

    def eager():
        gu = x @ w
        return F.silu(gu[:, n_out:]) * gu[:, :n_out]

    cands = {"this_build": ours, "cublas_gemm_only": lambda: x @ w, "cublas_plus_eager_act": eager}
    if act is not None:
        try:
            act(x @ w, n_out)                              # compile outside the timing
            cands["cublas_plus_compiled_act"] = lambda: act(x @ w, n_out)
        except Exception:
            pass
    return cands


def with_speedups(res: dict) -> dict:
    ours = res["this_build"]["median"]
    base = res.get("cublas_plus_compiled_act") or res.get("cublas_plus_eager_act")
    res["speedup_vs_cublas_plus_act"] = base["median"] / ours if base else None
    res["speedup_vs_cublas_gemm_only"] = res["cublas_gemm_only"]["median"] / ours
    res["unit"] = "ms per call"
    return res


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


def same_bits(a: torch.Tensor, b: torch.Tensor) -> bool:
    return bool(torch.equal(a.contiguous().view(torch.int16), b.contiguous().view(torch.int16)))


# --------------------------------------------------------------------------- legs, N = 1

def leg_silu_mul(dev, act_silu_mul) -> dict:
    """Configuration 2: ``matmul_silu_mul`` 32768 x 3072 x 12288 with ``up`` precomputed, beside
    the cuBLAS gate GEMM alone and followed by the eager / compiled ``silu(g) * up``
    (the reference's V1 / V2, bench.py:53-58 and README.md:32-33)."""
    import torch.nn.functional as F
    from swiglu_fused_b200 import _lib, matmul_silu_mul
    from swiglu_fused_b200.workloads import make_inputs

    inp = make_inputs(M_TOTAL, K_DIM, N_OUT, form="silu_mul", seed=0, device=dev, gen_device=str(dev))
    x, wg = inp["x"], inp["w_gate"]
    up = x @ inp["w_up"]
    h = torch.empty_like(up)
    cands = {"this_build": lambda: matmul_silu_mul(x, wg, up, out=h),
             "cublas_gemm_only": lambda: x @ wg,
             "cublas_plus_eager_act": lambda: F.silu(x @ wg) * up}
    if act_silu_mul is not None:
        try:
            act_silu_mul(x @ wg, up)
            cands["cublas_plus_compiled_act"] = lambda: act_silu_mul(x @ wg, up)
        except Exception:
            pass
    res = with_speedups(rotated_round_robin(cands))
    ms = res["this_build"]["median"]
    res.update({"workload": "c2_silu_mul 32768x3072x12288", "ms_per_call": ms,
                "tflops": 2.0 * M_TOTAL * K_DIM * N_OUT / (ms * 1e-3) / 1e12,
                "published_ms": 2.281})
    _lib.device_status()
    return res


def leg_c4(dev, act_fused, peaks) -> dict:
    """Configuration 4 (16384 x 4096 x 14336) and its tile tail, each beside cuBLAS and with a
    parity flag: sampled rows of the result against the CPU oracle for the main shape, the
    whole result for the tail shapes."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import swiglu_oracle as orc
    from swiglu_fused_b200 import _lib, matmul_fused_swiglu
    from swiglu_fused_b200.workloads import make_inputs

    M, K, N = C4
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=4, w_std=0.02, device=dev,
                      gen_device=str(dev))
    x_all, w = inp["x"], inp["w"]
    w_cpu = w.cpu()
    out = {}
    for m in (M,) + C4_TAIL:
        x = x_all[:m]
        h = torch.empty((m, N), dtype=torch.bfloat16, device=dev)
        res = with_speedups(rotated_round_robin(
            fused_candidates(x, w, N, lambda: matmul_fused_swiglu(x, w, out=h), act_fused),
            rounds=5, window_s=0.3 if m == M else 0.1))
        ms = res["this_build"]["median"]
        flops = 2.0 * m * K * 2 * N
        res["tflops"] = flops / (ms * 1e-3) / 1e12
        if m >= 1024:
            res["roofline"] = {"bound": "tensor", "achieved": res["tflops"],
                               "peak": peaks["tflops_burst"], "unit": "TFLOP/s",
                               "frac": res["tflops"] / peaks["tflops_burst"]}
        else:
            gbs = 2.0 * K * 2 * N / (ms * 1e-3) / 1e9      # the weight is streamed once
            res["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"],
                               "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                               "algorithmic_bytes": 2.0 * K * 2 * N}
        # parity inside the run
        matmul_fused_swiglu(x, w, out=h)
        torch.cuda.synchronize()
        rows = torch.arange(m) if m <= 256 else torch.linspace(0, m - 1, 96).long()
        xs = x[rows.to(dev)].cpu()
        ref64 = orc.fused_swiglu_exact(xs, w_cpu)          # K = 4096: measure against float64
        rep = orc.compare(h[rows.to(dev)].cpu(), ref64.to(torch.bfloat16), ref64, k_depth=K)
        rep32 = orc.compare(orc.fused_swiglu(xs, w_cpu), ref64.to(torch.bfloat16), ref64,
                            k_depth=K)
        res["parity_ok"] = bool(rep.ok)
        res["parity"] = (f"{len(rows)} rows x {N} columns vs the float64 CPU oracle: {rep}; the "
                         f"reference's own fp32 check expression against the same: {rep32}")
        out["c4_fused" if m == M else f"c4_tail_m{m}"] = res
    _lib.device_status()
    return out


def leg_neighbours(dev, peaks) -> dict:
    """The callers either side of the path (the rows after the hot path itself): the down
    projection at decode sizes (the plain entry point, which cuts K into ranges summed in
    thread-block clusters where that pays; the whole-K kernel; split-K with caller scratch;
    cuBLAS), the side-store
    training forward, the backward elementwise kernel and the two backward GEMMs at the
    headline shape, each beside its library counterpart on the same tensors."""
    from swiglu_fused_b200 import _lib, matmul_bf16, matmul_fused_swiglu
    from swiglu_fused_b200.ops import (matmul_bf16_splitk, matmul_fused_swiglu_save_factors,
                                       splitk_scratch_bytes, swiglu_grad_preact)

    out = {}
    g = torch.Generator(device=dev).manual_seed(9)
    # down projection at decode sizes: h[M, 14336] @ W_down[14336, 4096]
    Kd, Nd = 14336, 4096
    wd = torch.empty((Kd, Nd), dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=g)
    ha = torch.randn((256, Kd), dtype=torch.bfloat16, device=dev, generator=g)
    # The weight (117 MB) would fit the 126 MB L2 and stay there from call to call, which a
    # decode step that walks through all layers never sees: every call takes the next of three
    # copies (352 MB), so the weight always comes from HBM.  Same for every candidate.
    wds = [wd, wd.clone(), wd.clone()]
    turn = [0]

    def next_wd():
        turn[0] = (turn[0] + 1) % len(wds)
        return wds[turn[0]]

    dec = {"weights": "3 copies of W_down taken in turn (352 MB > L2): W always comes from HBM"}
    for m in (64, 256):
        a = ha[:m]
        c = torch.empty((m, Nd), dtype=torch.bfloat16, device=dev)
        scratch = torch.empty(splitk_scratch_bytes(m, Nd, Kd, 0), dtype=torch.uint8, device=dev)
        def whole_k():
            before = _lib.set_splitk_cluster_sum(False)
            matmul_bf16(a, next_wd(), out=c)
            _lib.set_splitk_cluster_sum(before)

        r = rotated_round_robin({
            "matmul_bf16": lambda: matmul_bf16(a, next_wd(), out=c),
            "unsplit": whole_k,
            "split_k": lambda: matmul_bf16_splitk(a, next_wd(), out=c, splits=0, scratch=scratch),
            "cublas": lambda: torch.matmul(a, next_wd(), out=c)}, rounds=5, window_s=0.05)
        want = a.float() @ wd.float()
        matmul_bf16_splitk(a, wd, out=c, splits=0, scratch=scratch)
        err = (c.float() - want).abs().max().item() / want.abs().max().item()
        r["max_err_over_scale"] = err
        r["hbm_frac"] = 2.0 * Kd * Nd / (r["split_k"]["median"] * 1e-3) / 1e9 / peaks["hbm_gbs"]
        dec[f"m{m}"] = r
    out["down_proj_decode_14336x4096"] = dec
    del wd, ha, wds

    # a narrow gate/up stage at decode size: few tiles, so the fused form cuts K into ranges
    # that run as thread-block clusters (beside its own whole-K tiles and the library pair)
    Mn, Kn, Nn = 64, 4096, 4096
    xn = torch.randn((Mn, Kn), dtype=torch.bfloat16, device=dev, generator=g)
    wn = torch.empty((Kn, 2 * Nn), dtype=torch.bfloat16, device=dev).normal_(0, Kn ** -0.5,
                                                                            generator=g)
    hn = torch.empty((Mn, Nn), dtype=torch.bfloat16, device=dev)
    wns = [wn] + [wn.clone() for _ in range(3)]     # 4 x 67 MB > L2, taken in turn (see above)
    turn_n = [0]

    def next_wn():
        turn_n[0] = (turn_n[0] + 1) % len(wns)
        return wns[turn_n[0]]

    def narrow_whole_k():
        before = _lib.set_splitk_cluster_sum(False)
        matmul_fused_swiglu(xn, next_wn(), out=hn)
        _lib.set_splitk_cluster_sum(before)

    def narrow_cublas():
        pre = xn @ next_wn()
        return torch.nn.functional.silu(pre[:, Nn:]) * pre[:, :Nn]

    r = rotated_round_robin({
        "this_build": lambda: matmul_fused_swiglu(xn, next_wn(), out=hn),
        "whole_k_tiles": narrow_whole_k,
        "cublas_plus_eager_act": narrow_cublas}, rounds=5, window_s=0.05)
    r["weights"] = "4 copies of W taken in turn (268 MB > L2): W always comes from HBM"
    matmul_fused_swiglu(xn, wn, out=hn)
    want = narrow_cublas().float()
    r["max_err_over_scale"] = ((hn.float() - want).abs().max() / want.abs().max()).item()
    r["hbm_frac"] = 2.0 * Kn * 2 * Nn / (r["this_build"]["median"] * 1e-3) / 1e9 / peaks["hbm_gbs"]
    out["fused_narrow_decode_64x4096x4096"] = r
    del xn, wn, hn, wns

    # training side at the headline shape
    import torch.nn.functional as F
    M, K, N = M_TOTAL, K_DIM, N_OUT
    x = torch.randn((M, K), dtype=torch.bfloat16, device=dev, generator=g)
    w = torch.empty((K, 2 * N), dtype=torch.bfloat16, device=dev).normal_(0, K ** -0.5, generator=g)
    h = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    factors = torch.empty((M, 2 * N), dtype=torch.bfloat16, device=dev)
    dy = torch.randn((M, N), dtype=torch.bfloat16, device=dev, generator=g)
    gp = torch.empty((M, 2 * N), dtype=torch.bfloat16, device=dev)
    gx = torch.empty((M, K), dtype=torch.bfloat16, device=dev)
    gw = torch.empty((K, 2 * N), dtype=torch.bfloat16, device=dev)
    matmul_fused_swiglu_save_factors(x, w, out=h, factors=factors)
    fwd = rotated_round_robin({
        "plain_forward": lambda: matmul_fused_swiglu(x, w, out=h),
        "save_factors_forward": lambda: matmul_fused_swiglu_save_factors(x, w, out=h,
                                                                         factors=factors)},
        rounds=3, window_s=0.2)
    out["save_factors_forward_c3"] = fwd
    ew = rotated_round_robin({
        "this_build": lambda: swiglu_grad_preact(dy, factors, out=gp),
        "torch_eager": lambda: torch.cat((dy * factors[:, :N], dy * factors[:, N:]), dim=1)},
        rounds=3, window_s=0.1)
    ew["hbm_frac"] = 10.0 * M * N / (ew["this_build"]["median"] * 1e-3) / 1e9 / peaks["hbm_gbs"]
    out["grad_preact_c3"] = ew
    swiglu_grad_preact(dy, factors, out=gp)
    bw = rotated_round_robin({
        "grad_x_this_build": lambda: matmul_bf16(gp, w, transpose_b=True, out=gx),
        "grad_x_cublas": lambda: torch.matmul(gp, w.t(), out=gx),
        "grad_w_this_build": lambda: matmul_bf16(x, gp, transpose_a=True, out=gw),
        "grad_w_cublas": lambda: torch.matmul(x.t(), gp, out=gw)}, rounds=3, window_s=0.2)
    out["backward_gemms_c3"] = bw
    torch.cuda.synchronize()
    _lib.device_status()
    return out


# --------------------------------------------------------------------------- legs, N > 1

def timed_ranks(fn, iters: int, dev, dist) -> float:
    """ms per call, device-timed between barriers, max over ranks."""
    for _ in range(3):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    ms = timed_calls(fn, iters)
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def all_true(flag: bool, dev, dist) -> bool:
    t = torch.tensor([int(bool(flag))], dtype=torch.int64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item())


def leg_c5(rank: int, world: int, dev, peaks) -> dict:
    """Configuration 5 (32768 x 8192 x 28672) column-parallel over the ranks, and the
    row-parallel down projection that consumes its output.  Every rank also computes the
    whole problem in ONE launch on its own GPU; the flags compare the sharded results with
    slices of that, bit for bit."""
    import torch.distributed as dist
    from swiglu_fused_b200 import _lib, matmul_bf16, matmul_fused_swiglu, sharding
    from swiglu_fused_b200.workloads import make_inputs

    M, K, N = C5
    iters = 10
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=5, w_std=0.02, device=dev,
                      gen_device=str(dev))
    x, w = inp["x"], inp["w"]
    del inp
    cols = sharding.col_shard(N, world, rank)
    single = matmul_fused_swiglu(x, w)                     # [M, N], one launch, this GPU only
    local = torch.empty((M, cols.count), dtype=torch.bfloat16, device=dev)
    full = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    sym = sharding.SymmetricOutput(M, N, dev)
    flops = 2.0 * M * K * 2 * N

    t_compute = timed_ranks(lambda: sharding.fused_swiglu_n_sharded(
        x, w, rank=rank, world=world, out=local), iters, dev, dist)
    t_nccl = timed_ranks(lambda: sharding.fused_swiglu_n_sharded(
        x, w, rank=rank, world=world, gather=True, out=full), iters, dev, dist)
    # the gather inside the kernel, three ways to move the tiles (see
    # sharding.fused_swiglu_n_sharded_fused_gather); each checked against the single launch
    ok_fused, t_modes = True, {}
    for mode in ("tma", "stores"):
        sym.tensor.zero_()
        t_modes[mode] = timed_ranks(lambda: sharding.fused_swiglu_n_sharded_fused_gather(
            x, w, sym, mode=mode), iters, dev, dist)
        torch.cuda.synchronize()
        ok_fused = ok_fused and same_bits(sym.tensor, single)
    ok_block = all_true(same_bits(local, single[:, cols.begin:cols.end]), dev, dist)
    ok_nccl = all_true(same_bits(full, single), dev, dist)
    ok_fused = all_true(ok_fused, dev, dist)
    if ok_fused and not os.environ.get("SWIGLU_B200_NO_MULTICAST"):
        # through the NVSwitch multicast mapping, where the fabric offers one; only after the
        # plain modes have passed on every rank
        del sym
        try:
            sym = sharding.SymmetricOutput(M, N, dev, multicast=True)
            have_mc = bool(sym.multicast_ptr)
        except Exception:   # a fabric or driver without multicast objects: the plain modes stand
            sym, have_mc = None, False
        if all_true(have_mc, dev, dist):
            sym.tensor.zero_()
            t_modes["multicast"] = timed_ranks(lambda: sharding.fused_swiglu_n_sharded_fused_gather(
                x, w, sym, mode="multicast"), iters, dev, dist)
            torch.cuda.synchronize()
            ok_fused = all_true(same_bits(sym.tensor, single), dev, dist)
    best = min(t_modes, key=t_modes.get)
    t_fused = t_modes[best]
    gather_bytes = 2.0 * M * (N - cols.count)              # received per GPU
    out = {
        "workload": f"c5: matmul_fused_swiglu {M}x{K}x{N}, {N // world} output columns per GPU, "
                    "x replicated, unsplit packed weight addressed through column windows",
        "world": world, "iters": iters,
        "compute_only_ms": t_compute, "compute_only_tflops": flops / (t_compute * 1e-3) / 1e12,
        "nccl_gather_ms": t_nccl, "fused_gather_ms": t_fused, "fused_gather_mode": best,
        "fused_gather_ms_by_mode": t_modes,
        "fused_gather_over_compute_only": t_fused / t_compute,
        "gather_bytes_in_per_gpu": gather_bytes,
        "nvlink_floor_ms": gather_bytes / 770e9 * 1e3,
        "roofline": {"bound": "tensor", "achieved": flops / world / (t_fused * 1e-3) / 1e12,
                     "peak": peaks["tflops_burst"], "unit": "TFLOP/s per GPU, gather included",
                     "frac": flops / world / (t_fused * 1e-3) / 1e12 / peaks["tflops_burst"]},
        "n_shard_block_bit_identical": ok_block,
        "n_shard_nccl_gather_bit_identical": ok_nccl,
        "n_shard_gather_bit_identical": ok_fused,
    }
    del full, sym, local

    # Row-parallel down projection: y[M, K] = h @ W_down, h column-sharded as the stage leaves
    # it, the partial products reduce-scattered by rows.
    h_loc = single[:, cols.begin:cols.end].contiguous()
    del single
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    wd_loc = torch.empty((cols.count, K), dtype=torch.bfloat16, device=dev).normal_(
        0, 0.02, generator=g)
    slots = sharding.RowParallelSlots(M, K, dev)
    rso16 = sharding.RowShardedOutput(M, K, dev, dtype=torch.bfloat16)
    y_own = torch.empty((slots.rows_per_rank, K), dtype=torch.bfloat16, device=dev)
    y_part = torch.empty((M, K), dtype=torch.bfloat16, device=dev)
    even = M % world == 0 and slots.rows_per_rank * world == M
    y_rs = torch.empty((M // world, K), dtype=torch.bfloat16, device=dev) if even else None

    def down_nccl():
        matmul_bf16(h_loc, wd_loc, out=y_part)
        dist.reduce_scatter_tensor(y_rs, y_part)

    t_local = timed_ranks(lambda: matmul_bf16(h_loc, wd_loc, out=y_part), iters, dev, dist)
    t_rs_nccl = timed_ranks(down_nccl, iters, dev, dist) if even else None
    t_rs_add = timed_ranks(lambda: sharding.down_proj_row_parallel(h_loc, wd_loc, rso16), iters,
                           dev, dist)
    t_rs_slots = timed_ranks(lambda: sharding.down_proj_row_parallel(
        h_loc, wd_loc, slots, out=y_own[:slots.my_rows]), iters, dev, dist)
    torch.cuda.synchronize()
    first = y_own[:slots.my_rows].clone()
    sharding.down_proj_row_parallel(h_loc, wd_loc, slots, out=y_own[:slots.my_rows])
    torch.cuda.synchronize()
    deterministic = all_true(same_bits(first, y_own[:slots.my_rows]), dev, dist)
    down = {
        "workload": f"h_local[{M}, {cols.count}] @ W_down[{cols.count}, {K}], result reduce-"
                    "scattered by rows",
        "local_gemm_only_ms": t_local, "gemm_plus_nccl_reduce_scatter_ms": t_rs_nccl,
        "fused_reduce_add_bf16_ms": t_rs_add, "fused_slots_fp32_sum_ms": t_rs_slots,
        "fused_slots_deterministic": deterministic,
    }
    if even:
        down_nccl()
        torch.cuda.synchronize()
        scale = y_rs.float().abs().max().item()
        err_slots = (first.float() - y_rs.float()).abs().max().item()
        err_add = (rso16.tensor[:rso16.my_rows].float() - y_rs.float()).abs().max().item()
        # every path rounds partial products to bf16 somewhere: agreement within a few bf16
        # ulps of the largest element
        tol = 4.0 * scale * 2.0 ** -8
        down.update({"max_abs_err_slots_vs_nccl": err_slots, "max_abs_err_add_vs_nccl": err_add,
                     "scale": scale, "tolerance": tol,
                     "down_proj_within_tolerance": all_true(err_slots <= tol and err_add <= tol,
                                                            dev, dist)})
    out["down_proj_row_parallel"] = down
    torch.cuda.synchronize()
    _lib.device_status()
    return out


# --------------------------------------------------------------------------- main arm

def run_ours(args) -> None:
    from swiglu_fused_b200 import (_lib, matmul_fused_swiglu, matmul_silu_mul, sharding,
                                   tile_table)
    from swiglu_fused_b200.host_pipeline import HostPipeline, SharedWeightHostPipeline
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

    m_total, k_dim, n_out = M_TOTAL, K_DIM, N_OUT
    if args.shape:
        m_total, k_dim, n_out = (int(v) for v in args.shape.lower().split("x"))
    if args.rows:
        m_total = args.rows
    headline = (m_total, k_dim, n_out) == (M_TOTAL, K_DIM, N_OUT) and \
        args.form == "fused_swiglu" and not args.tile_config
    rows = sharding.row_shard(m_total, world, rank)
    # Same global tensors on every rank (seeded CUDA generator); each keeps its rows.
    inp = make_inputs(m_total, k_dim, n_out, form="fused_swiglu", seed=0, device=dev,
                      gen_device=str(dev), w_std=None if headline or not args.shape else 0.02)
    x_full, w = inp["x"], inp["w"]
    x = x_full[rows.begin:rows.end].clone() if world > 1 else x_full
    h = torch.empty((rows.count, n_out), dtype=torch.bfloat16, device=dev)
    flops_total = 2.0 * m_total * k_dim * 2 * n_out
    flops_local = 2.0 * rows.count * k_dim * 2 * n_out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    m_shard_ok = None
    if world > 1 and headline and not args.no_legs:
        # the whole problem in one launch on this GPU; this rank's shard must be a slice of it
        h_single = matmul_fused_swiglu(x_full, w)
        matmul_fused_swiglu(x, w, out=h)
        torch.cuda.synchronize()
        m_shard_ok = all_true(same_bits(h, h_single[rows.begin:rows.end]), dev, dist)
        del h_single
    del x_full, inp

    pinned = None
    if args.tile_config:
        v = [int(t) for t in args.tile_config.split(",")]
        pinned = _lib.TileConfig(v[0], v[1], 0, v[2], 0, v[3] if len(v) > 3 else 0,
                                 v[4] if len(v) > 4 else 0)
    if args.form == "silu_mul":
        # Profiling aid: time the reference's other operator instead (W_gate = right half of
        # the packed weight, up = x @ W_up precomputed outside the timed region).
        w_gate = w[:, n_out:].contiguous()
        up = x @ w[:, :n_out].contiguous()
        flops_total, flops_local = flops_total / 2, flops_local / 2
        form_id, form_name = _lib.FORM_SILU_MUL, "silu_mul"

        def step():
            matmul_silu_mul(x, w_gate, up, out=h, config=pinned)
    else:
        form_id, form_name = _lib.FORM_FUSED_SWIGLU, "fused_swiglu"

        def step():
            matmul_fused_swiglu(x, w, out=h, config=pinned)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    barrier()
    _lib.device_status()

    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    launches0 = _lib.kernel_launches()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    sampler.begin()
    events[0].record()
    for i in range(args.steps):
        step()
        events[i + 1].record()
    barrier()
    elapsed_ms = events[0].elapsed_time(events[-1])
    step_ms = [events[i].elapsed_time(events[i + 1]) for i in range(args.steps)]
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
        if world > 1:
            pipe = SharedWeightHostPipeline(rows.count, k_dim, n_out, device=dev)
        else:
            pipe = HostPipeline(rows.count, k_dim, n_out, device=dev)
        x_host = torch.empty((rows.count, k_dim), dtype=torch.bfloat16).pin_memory()
        w_host = torch.empty((k_dim, 2 * n_out), dtype=torch.bfloat16).pin_memory()
        h_host = torch.empty((rows.count, n_out), dtype=torch.bfloat16).pin_memory()
        x_host.copy_(x)
        w_host.copy_(w)

        def e2e_time(copy_weight: bool):
            for _ in range(2):
                pipe.run(x_host, w_host, h_host, copy_weight=copy_weight)
            n0 = _lib.kernel_launches()
            barrier()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                pipe.run(x_host, w_host, h_host, copy_weight=copy_weight)
            torch.cuda.synchronize()
            dt = (time.perf_counter() - t0) / e2e_steps
            te = torch.tensor([dt], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(te, op=dist.ReduceOp.MAX)
            return te.item(), _lib.kernel_launches() - n0

        # what the host side of this box gives with every rank copying at once: bare pinned
        # copies of this rank's h (out) and x (in), the floor the pipeline works against
        def link_rate(dst, src):
            dst.copy_(src, non_blocking=True)
            barrier()
            t0 = time.perf_counter()
            for _ in range(3):
                dst.copy_(src, non_blocking=True)
            torch.cuda.synchronize()
            dt = torch.tensor([(time.perf_counter() - t0) / 3], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(dt, op=dist.ReduceOp.MAX)
            return src.numel() * 2 / dt.item() / 1e9

        d2h_gbs = link_rate(h_host, h)
        h2d_gbs = link_rate(x, x_host)
        h_host.zero_()
        e2e_s, e2e_launches = e2e_time(True)
        e2e_same = same_bits(h_host.to(dev), h)
        h_host.zero_()
        res_s, res_launches = e2e_time(False)
        res_same = same_bits(h_host.to(dev), h)
        if world > 1:
            e2e_same = all_true(e2e_same, dev, dist)
            res_same = all_true(res_same, dev, dist)
        e2e = {"value": flops_total / e2e_s / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": pipe.h2d_bytes, "d2h_bytes_per_step": pipe.d2h_bytes,
               "ms_per_step": e2e_s * 1e3, "steps": e2e_steps, "launches": e2e_launches,
               "matches_device_run": e2e_same,
               "host_link": {"d2h_gbs_per_gpu": d2h_gbs, "h2d_gbs_per_gpu": h2d_gbs,
                             "floor_ms": (pipe.d2h_bytes / d2h_gbs / 1e6),
                             "note": "bare pinned copies, one direction at a time, all ranks "
                                     "copying at once (slowest rank); floor_ms = this rank's h "
                                     "bytes at that device-to-host rate"},
               "host_bytes_per_step_all_ranks": world * (pipe.h2d_bytes + pipe.d2h_bytes)
               if world > 1 else pipe.h2d_bytes + pipe.d2h_bytes,
               "weight_resident": {
                   "value": flops_total / res_s / 1e12, "unit": UNIT, "ms_per_step": res_s * 1e3,
                   "h2d_bytes_per_step": pipe.h2d_bytes_no_weight,
                   "d2h_bytes_per_step": pipe.d2h_bytes, "launches": res_launches,
                   "matches_device_run": res_same,
                   "note": "same call with the weight left on the device from the run before "
                           "(weights are parameters, not per-step inputs): only x in, h out"},
               "note": "per rank, through one sgl_host_pipeline_run call (3+ streams): pinned host "
                       "x rows and W copied in, h copied out, every step; the first rows are "
                       "computed per weight column window so the copy out starts while W is still "
                       "arriving" + ("; each rank copies only its 1/N column slice of W from the "
                                     "host and pushes it to the other ranks' buffers over NVLink "
                                     "(peer copies + a flag per slice), so W crosses PCIe once "
                                     "per box, not N times" if world > 1 else "") +
                       "; timed on the host clock around the calls, max over ranks; byte counts "
                       "are per rank"}
        pipe.close()
        del pipe, x_host, w_host, h_host

    peaks = load_peaks()
    region_s = elapsed_ms * 1e-3
    burst = region_s < 1.0
    peak = peaks["tflops_burst"] if burst else peaks["tflops_sustained"]
    achieved = flops_local / (elapsed_ms / args.steps * 1e-3) / 1e12   # this rank's kernel
    cfg_used = pinned or tile_table.lookup(form_id, rows.count, n_out, k_dim) or \
        _lib.default_config(form_id, rows.count, n_out, k_dim)
    if headline:
        workload = WORKLOAD
    elif args.form == "silu_mul":
        workload = f"matmul_silu_mul {m_total}x{k_dim}x{n_out} (profiling aid, not the headline)"
    else:
        workload = (f"matmul_fused_swiglu {m_total}x{k_dim}x{n_out} (profiling aid, not the "
                    "headline number)")
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": (value / PUBLISHED_V4_TFLOPS) if (world == 1 and headline) else None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload, "M": m_total, "K": k_dim, "N": n_out,
                   "rows_per_gpu": rows.count,
                   "parallelism": f"M-sharded x{world}, weights replicated, no collective",
                   "tile_config": {"cta_group": cfg_used.cta_group, "block_k": cfg_used.block_k,
                                   "group_m": cfg_used.group_m, "l2_hints": cfg_used.l2_hints,
                                   "group_n": cfg_used.group_n},
                   "l2": "inputs+output larger than L2 (x+W+h per GPU = "
                         f"{(x.numel() + w.numel() + h.numel()) * 2 / 1e6:.0f} MB > 126 MB), no flush"},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak,
                     "unit": "TFLOP/s", "frac": achieved / peak,
                     "peak_kind": ("burst: the timed region lasts %.3f s, a kernel timed alone"
                                   % region_s) if burst else
                                  ("sustained: the timed region lasts %.1f s" % region_s),
                     "traffic": profiled_traffic(form_name, rows.count, n_out, k_dim, cfg_used),
                     "algorithmic_bytes": 2.0 * (rows.count * k_dim + 2 * k_dim * n_out
                                                 + rows.count * n_out),
                     "peak_source": peaks["source"],
                     "frac_of_burst_peak": achieved / peaks["tflops_burst"],
                     "frac_of_sustained_peak": achieved / peaks["tflops_sustained"],
                     "frac_of_nominal_2250": achieved / 2250.0,
                     "step_ms": dict(spread(step_ms), note="per-step CUDA-event times of this "
                                     "rank; multiply by clocks.sm_mhz to compare across clocks")},
        "clocks": clocks,
        "e2e": e2e,
        "gpu_launches": launches,
    }
    if m_shard_ok is not None:
        line["m_shard_bit_identical"] = m_shard_ok

    if headline and not args.no_legs:
        legs = {}
        if world == 1:
            act_fused, act_silu_mul, why = (None, None, "skipped") if args.no_gpu_baselines \
                else compiled_activation()
            if not args.no_gpu_baselines:
                gb = with_speedups(rotated_round_robin(fused_candidates(x, w, n_out, step, act_fused)))
                if why:
                    gb["compile_error"] = why
                line["gpu_baselines"] = gb
                line["silu_mul"] = leg_silu_mul(dev, act_silu_mul)
                del x, h
                torch.cuda.empty_cache()
                legs.update(leg_c4(dev, act_fused, peaks))
                torch.cuda.empty_cache()
                legs["neighbours"] = leg_neighbours(dev, peaks)
            if not args.no_cpu_baseline:
                line["cpu_baseline"] = {k: v for k, v in
                                        cpu_reference_rate(12.0, os.cpu_count() or 1).items()
                                        if k in ("value", "unit", "cores", "kind", "sample")}
        else:
            del x, h, w
            torch.cuda.empty_cache()
            legs["c5_n_shard"] = leg_c5(rank, world, dev, peaks)
        line["legs"] = legs

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
    ap.add_argument("--shape", default="",
                    help="MxKxN: time the operator on another shape (profiling aid, one GPU; "
                         "weights N(0, 0.02)); the JSON line then says so and carries no legs")
    ap.add_argument("--form", choices=("fused_swiglu", "silu_mul"), default="fused_swiglu",
                    help="operator to time; silu_mul is a profiling aid, the headline is fused_swiglu")
    ap.add_argument("--tile-config", default="",
                    help="cta_group,block_k,group_m,l2_hints,group_n: pin the tile configuration "
                         "of the timed operator (profiling aid; default = tile table / library)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-gpu-baselines", action="store_true",
                    help="skip the cuBLAS (+ eager / compiled activation) comparisons and the "
                         "configuration-2 and configuration-4 legs that are timed beside them")
    ap.add_argument("--no-legs", action="store_true",
                    help="headline only: skip configurations 2, 4 and 5 and the library baselines")
    args = ap.parse_args()
    if args.steps < 1:
        raise SystemExit("--steps must be >= 1")
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
