"""Names of ``swiglu/triton/impls.py`` that have a native counterpart in ``swiglu_fused_b200``.

Only the layout helpers (``:1898-1917``), the module (``:3372-3596``) and the differentiable
operator are provided.  The reference's Triton kernels (``fused_swiglu_wide_packed`` and the
rest) are not: importing them from here raises ``ImportError``, which the reference's own
benchmark treats as "variant unavailable" (``bench_fused.py:22-30``).
"""
from swiglu_fused_b200 import weights as _weights
from swiglu_fused_b200.autograd import fused_swiglu as fused_swiglu_autograd
from swiglu_fused_b200.module import PackedSwiGLULinear


def pack_swiglu_linear_weight(linear_weight, block_n_half=None):
    """``[2N, K]`` -> ``[K, 2N] = [W_up | W_gate]``.  ``block_n_half`` (the reference's chunk
    width for its interleaved layout) is accepted and unused: no interleaving is needed."""
    return _weights.pack_swiglu_linear_weight(linear_weight)


def unpack_swiglu_linear_weight(packed_weight, block_n_half=None):
    return _weights.unpack_swiglu_linear_weight(packed_weight)


__all__ = ["PackedSwiGLULinear", "pack_swiglu_linear_weight", "unpack_swiglu_linear_weight",
           "fused_swiglu_autograd"]
