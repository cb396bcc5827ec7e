"""``PackedSwiGLULinear``: the gate/up projection of a SwiGLU FFN as an ``nn.Module``.

Counterpart of the reference's module of the same name (``swiglu/triton/impls.py:3372-3596``),
with the same outside behaviour:

* the parameter ``weight`` is held as ``[in_features, 2 * hidden_features] = [W_up | W_gate]``
  (the reference's "normal" layout; its chunk-interleaved "packed" layout exists only to suit
  its Triton tiles and has no use here - the kernel reads the two column windows in place);
* the state dict carries the ``nn.Linear`` layout ``[2 * hidden_features, in_features]`` (rows:
  up features, then gate features), so existing checkpoints load and save unchanged, and a
  state dict in the internal layout is accepted as well;
* ``from_linear`` converts a bias-free ``nn.Linear`` whose output is ``[up | gate]``;
* ``forward`` accepts any leading dimensions and returns ``[..., hidden_features]``.

When gradients are needed the forward is the side-store kernel and the backward runs the
elementwise kernel and the two GEMMs of ``autograd.py``; otherwise the plain fused kernel
runs (no factor writes).
"""
from __future__ import annotations

import math
import warnings

import torch

from .autograd import fused_swiglu
from .ops import matmul_fused_swiglu
from .weights import pack_swiglu_linear_weight, unpack_swiglu_linear_weight


_BACKWARD_MODES = {"save_preact", "save_factors", "save_factors_normal", "save_factors_cute_bwd",
                   "onload_save_factors", "cublas_save_factors"}


class PackedSwiGLULinear(torch.nn.Module):
    """``block_n_half``, ``backward_mode`` and ``parameter_layout`` are the reference
    constructor's tuning switches (``swiglu/triton/impls.py:3388-3408``); they are accepted,
    checked against the same sets and otherwise unused: there is one native forward/backward
    path and one parameter layout here (asking for the ``"packed"`` layout warns and
    ``parameter_layout`` reads ``"normal"`` afterwards)."""

    def __init__(self, in_features: int, hidden_features: int, *, block_n_half=None,
                 backward_mode: str = "save_factors_normal", parameter_layout: str = "normal",
                 device=None, dtype=torch.bfloat16) -> None:
        super().__init__()
        if backward_mode not in _BACKWARD_MODES:
            raise ValueError(f"unknown backward_mode {backward_mode!r}")
        if parameter_layout not in ("packed", "normal"):
            raise ValueError(f"unknown parameter_layout {parameter_layout!r}")
        if parameter_layout == "packed":
            # the reference's chunk-interleaved internal layout does not exist here; say so
            # once instead of silently handing back a differently laid out `weight`
            warnings.warn(
                "PackedSwiGLULinear(parameter_layout='packed'): this implementation keeps "
                "`weight` as [in_features, 2 * hidden_features] = [W_up | W_gate] (the "
                "reference's 'normal' layout); state dicts are unaffected (nn.Linear layout "
                "either way)", stacklevel=2)
        self.block_n_half = block_n_half
        self.backward_mode = backward_mode
        self.parameter_layout = "normal"
        if in_features % 8 or hidden_features % 8:
            raise ValueError("in_features and hidden_features must be multiples of 8 "
                             f"(16-byte rows), got {in_features} and {hidden_features}")
        self.in_features = in_features
        self.hidden_features = hidden_features
        self.weight = torch.nn.Parameter(
            torch.empty(in_features, 2 * hidden_features, device=device, dtype=dtype))
        self.reset_parameters()

    @classmethod
    def from_linear(cls, linear: torch.nn.Linear, **kwargs) -> "PackedSwiGLULinear":
        if linear.bias is not None:
            raise ValueError("the projection has no bias term")
        if linear.out_features % 2:
            raise ValueError("out_features must be 2 * hidden_features")
        module = cls(linear.in_features, linear.out_features // 2, device=linear.weight.device,
                     dtype=linear.weight.dtype, **kwargs)
        module.load_linear_weight_(linear.weight)
        return module

    @torch.no_grad()
    def reset_parameters(self) -> None:
        # the reference's initialisation (swiglu/triton/impls.py:3449-3464): up rows
        # N(0, 1/in_features), gate rows Kaiming normal, drawn in the nn.Linear layout
        lw = torch.empty(2 * self.hidden_features, self.in_features, device=self.weight.device,
                         dtype=torch.float32)
        torch.nn.init.normal_(lw[: self.hidden_features], std=1.0 / math.sqrt(self.in_features))
        torch.nn.init.kaiming_normal_(lw[self.hidden_features:])
        self.load_linear_weight_(lw)

    @torch.no_grad()
    def load_linear_weight_(self, linear_weight: torch.Tensor) -> None:
        expected = (2 * self.hidden_features, self.in_features)
        if tuple(linear_weight.shape) != expected:
            raise ValueError(f"expected a weight of shape {expected}, got {tuple(linear_weight.shape)}")
        lw = linear_weight.detach().to(device=self.weight.device, dtype=self.weight.dtype)
        self.weight.copy_(pack_swiglu_linear_weight(lw))

    def linear_weight(self) -> torch.Tensor:
        """The parameters in the ``nn.Linear`` layout ``[2 * hidden_features, in_features]``."""
        with torch.no_grad():
            return unpack_swiglu_linear_weight(self.weight)

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        weight = self.linear_weight()
        destination[prefix + "weight"] = weight if keep_vars else weight.detach()

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys,
                              unexpected_keys, error_msgs) -> None:
        key = prefix + "weight"
        original = state_dict.get(key)
        if original is not None:
            linear_shape = (2 * self.hidden_features, self.in_features)
            internal_shape = (self.in_features, 2 * self.hidden_features)
            if tuple(original.shape) == linear_shape:
                # (a square weight is ambiguous by shape; the documented layout is nn.Linear's)
                state_dict[key] = pack_swiglu_linear_weight(original.detach())
            elif tuple(original.shape) != internal_shape:
                error_msgs.append(f"size mismatch for {key}: got {tuple(original.shape)}, expected "
                                  f"{linear_shape} (nn.Linear layout) or {internal_shape} (internal)")
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys,
                                      unexpected_keys, error_msgs)
        if original is not None:
            state_dict[key] = original          # leave the caller's dict as it was

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        needs_grad = torch.is_grad_enabled() and (x2.requires_grad or self.weight.requires_grad)
        out = fused_swiglu(x2, self.weight) if needs_grad else matmul_fused_swiglu(x2, self.weight)
        return out.view(*lead, self.hidden_features)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, hidden_features={self.hidden_features}"
