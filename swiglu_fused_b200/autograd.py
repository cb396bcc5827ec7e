"""``torch.autograd`` wiring of the stage for training.

Forward: the side-store kernel (h + factors in one launch).  Backward: the elementwise
kernel for ``grad_preact``, then ``grad_x = grad_preact @ W^T`` and
``grad_W = x^T @ grad_preact`` on the GEMM form of the same kernel, each reading its
transposed operand in place.  The reference keeps its autograd Functions in its Triton
module (``swiglu/triton/impls.py:2913-3369``) and runs the two GEMMs through cuBLAS
(``:100-124``).
"""
from __future__ import annotations

import torch

from .ops import matmul_bf16, matmul_fused_swiglu_save_factors, swiglu_grad_preact


class FusedSwiGLUFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        h, factors = matmul_fused_swiglu_save_factors(x, w)
        ctx.save_for_backward(x, w, factors)
        return h

    @staticmethod
    def backward(ctx, grad_h: torch.Tensor):
        x, w, factors = ctx.saved_tensors
        # grad_preact overwrites the saved factors (no second [M, 2N] buffer).  The write goes
        # through a raw pointer, which autograd's version counter cannot see, so a second
        # backward over the same graph would silently multiply dy into factors that already
        # hold dy: refuse it instead.  (The reference writes grad_de to a new tensor and then
        # frees the saved ones, swiglu/triton/impls.py:3107-3116.)
        if getattr(ctx, "_factors_consumed", False):
            raise RuntimeError(
                "FusedSwiGLUFunction.backward ran twice over one forward: the saved factors "
                "were overwritten in place by the first backward (retain_graph=True is not "
                "supported; run the forward again)")
        ctx._factors_consumed = True
        grad_preact = swiglu_grad_preact(grad_h.contiguous(), factors, out=factors)  # in place
        grad_x = matmul_bf16(grad_preact, w, transpose_b=True) if ctx.needs_input_grad[0] else None
        grad_w = matmul_bf16(x, grad_preact, transpose_a=True) if ctx.needs_input_grad[1] else None
        return grad_x, grad_w


def fused_swiglu(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Differentiable ``silu(x @ W_gate) * (x @ W_up)`` with ``w = [W_up | W_gate]``."""
    return FusedSwiGLUFunction.apply(x, w)
