"""Weight layout helpers either side of the operator.

The operators take the reference's packed weight ``W[K, 2N] = [W_up | W_gate]``
(``swiglu/matmul_fused_swiglu.py:152-160``).  A checkpoint usually holds the same
parameters as an ``nn.Linear`` weight ``[2N, K]`` (output features first).  These helpers
convert between the two, under the names the reference uses
(``pack_swiglu_linear_weight`` / ``unpack_swiglu_linear_weight``,
``swiglu/triton/impls.py:1898-1917``).  Unlike the reference's Triton path there is no
chunk interleaving: the kernel reads the ``up`` and ``gate`` column windows of the plain
concatenation in place.  ``matmul_fused_swiglu(..., w_layout="nk")`` goes one step further
and consumes the ``[2N, K]`` checkpoint layout directly, with no conversion at all.
"""
from __future__ import annotations

import torch


def pack_swiglu_linear_weight(linear_weight: torch.Tensor) -> torch.Tensor:
    """``nn.Linear`` weight ``[2N, K]`` (rows: N up features, then N gate features)
    -> packed ``[K, 2N] = [W_up | W_gate]``, contiguous."""
    if linear_weight.dim() != 2 or linear_weight.shape[0] % 2:
        raise ValueError(f"expected a [2N, K] weight, got {tuple(linear_weight.shape)}")
    return linear_weight.t().contiguous()


def unpack_swiglu_linear_weight(packed_weight: torch.Tensor) -> torch.Tensor:
    """Packed ``[K, 2N]`` -> ``nn.Linear`` weight ``[2N, K]``, contiguous."""
    if packed_weight.dim() != 2 or packed_weight.shape[1] % 2:
        raise ValueError(f"expected a [K, 2N] weight, got {tuple(packed_weight.shape)}")
    return packed_weight.t().contiguous()


def pack_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """Separate ``W_gate[K, N]`` and ``W_up[K, N]`` -> packed ``[K, 2N] = [W_up | W_gate]``."""
    if w_gate.shape != w_up.shape or w_gate.dim() != 2:
        raise ValueError("w_gate and w_up must be [K, N] with equal shapes")
    return torch.cat([w_up, w_gate], dim=1).contiguous()


def split_packed(packed_weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Views ``(W_up, W_gate)`` of a packed ``[K, 2N]`` weight (no copy)."""
    n = packed_weight.shape[1] // 2
    return packed_weight[:, :n], packed_weight[:, n:]


def from_hf_llama(gate_proj: torch.Tensor, up_proj: torch.Tensor, layout: str = "kn") -> torch.Tensor:
    """Llama-style checkpoints store ``gate_proj.weight`` and ``up_proj.weight`` as ``[N, K]``.
    ``layout="kn"`` returns the packed ``[K, 2N]``; ``layout="nk"`` the ``[2N, K]`` stack
    ``[up_proj; gate_proj]`` for the direct checkpoint-layout path."""
    if gate_proj.shape != up_proj.shape or gate_proj.dim() != 2:
        raise ValueError("gate_proj and up_proj must be [N, K] with equal shapes")
    stacked = torch.cat([up_proj, gate_proj], dim=0)
    if layout == "nk":
        return stacked.contiguous()
    if layout == "kn":
        return stacked.t().contiguous()
    raise ValueError(f"unknown layout {layout!r}")
