"""CPU oracle for the fused SwiGLU gate/up stage.  TEST INFRASTRUCTURE ONLY.

Nothing in the product path (``swiglu_fused_b200``) imports this file; it is
used by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline legs
of ``bench.py`` as the checker / the timed CPU reference, never as a fallback.

It restates the reference's own fp32 check expressions on CPU tensors:

* silu_mul form, ``bench.py:39-40`` of the reference::

      gate_f32 = x.float() @ Wg.float()
      ref = F.silu(gate_f32) * up.float()

* fused form, ``bench_fused.py:39-42`` of the reference::

      gate_up_f32 = x.float() @ W.float()          # [M, 2N]
      C_ref = F.silu(gate_up_f32[:, N:]) * gate_up_f32[:, :N]

The result is rounded once to bf16 (round-to-nearest-even), which is what the
kernels store.  Parity status: PINNED to those expressions (executed with torch
on the CPU) and to the float64 golden vectors in ``tests/golden``; the
reference ships no golden vectors of its own, and its CUDA kernels cannot run
in a container without a GPU and without pycuda.

Error metrics follow the stated tolerance: <= 1 bf16 ulp on >= 99.9 % of the
elements and a floored relative error <= 1e-2, the floor being
``max(|ref|, 2**-7 * mean|ref|)`` (near-zero outputs are dominated by the
accumulation order, not by the kernel).  The floor grows with the depth of the
reduction beyond K = 1024, ``* sqrt(K / 1024)``, as the reference's own bound does
(``atol = max(1, sqrt(K) / 32)``, bench.py:43): an fp32 accumulator that takes
K products leaves absolute error proportional to the partial sums on outputs
that are themselves near zero.  Measured at K = 4096 (configuration 4) against
float64: with the K = 1024 floor the tcgen05 accumulation reaches 1.085e-2 on
two of 3.7 million elements, the CPU's fp32 sum 3.9e-3.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

ULP_FRACTION_REQUIRED = 0.999   # share of elements within 1 bf16 ulp
MAX_FLOORED_REL_ERR = 1e-2      # max |h - ref| / max(|ref|, 2^-7 mean|ref|)
REL_FLOOR_FACTOR = 2.0 ** -7


def silu_mul_f32(x: torch.Tensor, w_gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """fp32 ``silu(x @ w_gate) * up`` (reference ``bench.py:39-40``)."""
    gate_f32 = x.float() @ w_gate.float()
    return F.silu(gate_f32) * up.float()


def fused_swiglu_f32(x: torch.Tensor, w: torch.Tensor, up_col0: int | None = None,
                     gate_col0: int | None = None, n_out: int | None = None) -> torch.Tensor:
    """fp32 ``silu(gate) * up`` with ``[up | gate] = x @ w`` (reference ``bench_fused.py:39-42``).

    The optional window arguments select ``up = x @ w[:, up_col0:+n]`` and
    ``gate = x @ w[:, gate_col0:+n]`` for column-parallel shards.
    """
    if n_out is None:
        # exactly the reference's expression: one [M, 2N] fp32 GEMM, then the two halves
        n = w.shape[1] // 2
        gate_up_f32 = x.float() @ w.float()
        return F.silu(gate_up_f32[:, n:]) * gate_up_f32[:, :n]
    xf = x.float()
    up = xf @ w[:, up_col0:up_col0 + n_out].float()
    gate = xf @ w[:, gate_col0:gate_col0 + n_out].float()
    return F.silu(gate) * up


def matmul_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """fp32 ``a @ b`` of bf16 operands: the plain torch fp32 reference of the down projection
    (the reference project has no such product; this follows its fp32-check convention)."""
    return a.float() @ b.float()


def swiglu_factors_f32(x: torch.Tensor, w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``(h, factors)`` of the side-store forward, with the reference's expressions
    (``swiglu/triton/impls.py:455-468``): sig = sigmoid(gate); silu = gate * sig;
    silu_prime = sig + silu * (1 - sig); factors = [silu | left * silu_prime]; h = left * silu."""
    n = w.shape[1] // 2
    gu = x.float() @ w.float()
    left, gate = gu[:, :n], gu[:, n:]
    sig = torch.sigmoid(gate)
    silu = gate * sig
    silu_prime = sig + silu * (1.0 - sig)
    return left * silu, torch.cat([silu, left * silu_prime], dim=1)


def grad_preact_f32(dy: torch.Tensor, factors: torch.Tensor) -> torch.Tensor:
    """fp32 ``[dy * silu | dy * left * silu_prime]`` from the saved (bf16) factors."""
    n = dy.shape[1]
    f = factors.float()
    d = dy.float()
    return torch.cat([d * f[:, :n], d * f[:, n:]], dim=1)


def silu_mul(x, w_gate, up) -> torch.Tensor:
    """bf16 result of the silu_mul form."""
    return silu_mul_f32(x, w_gate, up).to(torch.bfloat16)


def fused_swiglu(x, w, up_col0=None, gate_col0=None, n_out=None) -> torch.Tensor:
    """bf16 result of the fused form."""
    return fused_swiglu_f32(x, w, up_col0, gate_col0, n_out).to(torch.bfloat16)


def fused_swiglu_exact(x, w) -> torch.Tensor:
    """The fused form evaluated in float64, NOT rounded: the value both an fp32-accumulating
    kernel and the reference's fp32 check approximate.  For deep reductions (K in the
    thousands) the fp32 check itself carries accumulation error of the size of the tolerance
    on near-zero outputs, so full-size comparisons measure against this instead."""
    n = w.shape[1] // 2
    gu = x.double() @ w.double()
    gate, up = gu[:, n:], gu[:, :n]
    return gate / (1.0 + torch.exp(-gate)) * up


def fused_swiglu_f64(x, w) -> torch.Tensor:
    """float64 evaluation, rounded to bf16: machine-independent golden values."""
    return fused_swiglu_exact(x, w).to(torch.bfloat16)


def silu_mul_f64(x, w_gate, up) -> torch.Tensor:
    gate = x.double() @ w_gate.double()
    return (gate / (1.0 + torch.exp(-gate)) * up.double()).to(torch.bfloat16)


# ----------------------------------------------------------------- error metrics

def bf16_ordinal(t: torch.Tensor) -> torch.Tensor:
    """Map bf16 values to integers that are monotone in the value (ulp distance = difference)."""
    assert t.dtype == torch.bfloat16
    bits = t.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
    neg = bits >= 0x8000
    return torch.where(neg, 0x8000 - bits, bits)


@dataclass
class ParityReport:
    n: int
    frac_exact: float
    frac_within_1ulp: float
    max_ulp: int
    max_floored_rel: float
    max_abs: float
    n_nonfinite: int

    @property
    def ok(self) -> bool:
        return (self.n_nonfinite == 0 and self.frac_within_1ulp >= ULP_FRACTION_REQUIRED
                and self.max_floored_rel <= MAX_FLOORED_REL_ERR)

    def __str__(self) -> str:
        return (f"n={self.n} exact={self.frac_exact:.6f} <=1ulp={self.frac_within_1ulp:.6f} "
                f"max_ulp={self.max_ulp} max_floored_rel={self.max_floored_rel:.3e} "
                f"max_abs={self.max_abs:.3e} nonfinite={self.n_nonfinite} ok={self.ok}")


def rel_floor_factor(k_depth: int | None) -> float:
    """Floor of the relative-error denominator as a fraction of mean|ref|."""
    if not k_depth or k_depth <= 1024:
        return REL_FLOOR_FACTOR
    return REL_FLOOR_FACTOR * (k_depth / 1024.0) ** 0.5


def compare(h: torch.Tensor, ref_bf16: torch.Tensor, ref_f32: torch.Tensor | None = None,
            k_depth: int | None = None) -> ParityReport:
    """Compare a kernel result with the oracle (both bf16, CPU or same device).  ``k_depth`` is
    the length of the reduction behind every element (None or <= 1024: the base floor)."""
    h = h.detach()
    ref_bf16 = ref_bf16.detach().to(h.device)
    assert h.shape == ref_bf16.shape, (h.shape, ref_bf16.shape)
    assert h.dtype == torch.bfloat16 and ref_bf16.dtype == torch.bfloat16
    ref = (ref_f32.detach().to(h.device) if ref_f32 is not None else ref_bf16.float())
    hf = h.float()
    nonfinite = int((~torch.isfinite(hf)).sum().item())
    d_ulp = (bf16_ordinal(h) - bf16_ordinal(ref_bf16)).abs()
    n = h.numel()
    floor = rel_floor_factor(k_depth) * ref.abs().mean()
    rel = (hf - ref).abs() / torch.maximum(ref.abs(), floor)
    rel = torch.nan_to_num(rel, nan=float("inf"))
    return ParityReport(
        n=n,
        frac_exact=float((d_ulp == 0).sum().item()) / n,
        frac_within_1ulp=float((d_ulp <= 1).sum().item()) / n,
        max_ulp=int(d_ulp.max().item()),
        max_floored_rel=float(rel.max().item()),
        max_abs=float(torch.nan_to_num((hf - ref).abs(), nan=float("inf")).max().item()),
        n_nonfinite=nonfinite,
    )
