"""Seeded synthetic inputs with the shapes and value distributions of the five
benchmark configurations (no dataset is involved anywhere on this path).

The reference seeds the CUDA generator (``bench.py:32-35``, ``bench_fused.py:33-36``),
which cannot be reproduced without a GPU.  Here the values come from a CPU
``torch.Generator`` so the CPU oracle and the GPU see the same bytes: fp32
``randn`` -> scale -> cast to bf16; x first, then the weights.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    form: str        # "silu_mul" or "fused_swiglu"
    M: int
    K: int
    N: int           # output columns (the packed weight has 2N)
    w_std: float | None = None   # None -> 1/sqrt(K)

    @property
    def flops(self) -> float:
        """Algorithmic FLOPs: 2MNK (silu_mul) or 2MK(2N) (fused); activation not counted,
        as in the reference (``bench.py:22-23``, ``swiglu/matmul_fused_swiglu.py:143``)."""
        return 2.0 * self.M * self.N * self.K * (1 if self.form == "silu_mul" else 2)

    @property
    def bytes(self) -> float:
        """Algorithmic bytes, every operand once."""
        if self.form == "silu_mul":
            return 2.0 * (self.M * self.K + self.K * self.N + 2 * self.M * self.N)
        return 2.0 * (self.M * self.K + 2 * self.K * self.N + self.M * self.N)


WORKLOADS = {
    "c1_check": Workload("c1_check", "fused_swiglu", 512, 1024, 2048),
    "c1_check_silu_mul": Workload("c1_check_silu_mul", "silu_mul", 512, 1024, 2048),
    "c2_silu_mul": Workload("c2_silu_mul", "silu_mul", 32768, 3072, 12288),
    "c3_fused": Workload("c3_fused", "fused_swiglu", 32768, 3072, 12288),
    "c4_llama8b": Workload("c4_llama8b", "fused_swiglu", 16384, 4096, 14336, 0.02),
    "c4_tail_m64": Workload("c4_tail_m64", "fused_swiglu", 64, 4096, 14336, 0.02),
    "c4_tail_m256": Workload("c4_tail_m256", "fused_swiglu", 256, 4096, 14336, 0.02),
    "c4_tail_m1024": Workload("c4_tail_m1024", "fused_swiglu", 1024, 4096, 14336, 0.02),
    "c5_llama70b": Workload("c5_llama70b", "fused_swiglu", 32768, 8192, 28672, 0.02),
}


def _randn_bf16(rows: int, cols: int, std: float, gen: torch.Generator,
                device: torch.device | str) -> torch.Tensor:
    """N(0, std) in bf16, generated in row blocks to bound fp32 scratch."""
    out = torch.empty((rows, cols), dtype=torch.bfloat16, device=device)
    block = max(1, (64 << 20) // max(1, cols))
    for r0 in range(0, rows, block):
        r1 = min(rows, r0 + block)
        t = torch.randn((r1 - r0, cols), dtype=torch.float32, generator=gen,
                        device=gen.device)
        if std != 1.0:
            t.mul_(std)
        out[r0:r1].copy_(t.to(torch.bfloat16))
    return out


def make_inputs(M: int, K: int, N: int, *, form: str = "fused_swiglu", seed: int = 0,
                w_std: float | None = None, device: torch.device | str = "cpu",
                gen_device: str = "cpu") -> dict[str, torch.Tensor]:
    """Inputs for one problem.

    fused_swiglu: ``x`` [M,K], ``w`` [K,2N] = [W_up | W_gate].
    silu_mul:     ``x`` [M,K], ``w_gate`` [K,N], ``w_up`` [K,N] (the caller forms
                  ``up = x @ w_up`` with whatever GEMM it uses).
    ``gen_device="cuda"`` draws on the GPU instead (faster for the full-size
    benchmark shapes; values then differ from the CPU-seeded ones).
    """
    gen = torch.Generator(device=gen_device)
    gen.manual_seed(seed)
    std = w_std if w_std is not None else K ** -0.5
    x = _randn_bf16(M, K, 1.0, gen, device)
    if form == "fused_swiglu":
        w = _randn_bf16(K, 2 * N, std, gen, device)
        return {"x": x, "w": w}
    if form == "silu_mul":
        w_gate = _randn_bf16(K, N, std, gen, device)
        w_up = _randn_bf16(K, N, std, gen, device)
        return {"x": x, "w_gate": w_gate, "w_up": w_up}
    raise ValueError(f"unknown form {form!r}")


def make_workload_inputs(wl: Workload, **kw) -> dict[str, torch.Tensor]:
    return make_inputs(wl.M, wl.K, wl.N, form=wl.form, w_std=wl.w_std, **kw)
