"""B200-native fused SwiGLU gate/up stage (sm_100a, tcgen05 + TMA).

Public surface = the reference's two operators::

    from swiglu_fused_b200 import matmul_silu_mul, matmul_fused_swiglu

The same functions are importable under the reference's own module paths,
``swiglu.matmul_silu_mul`` and ``swiglu.matmul_fused_swiglu``.
"""
from ._lib import TileConfig, SglError
from .ops import (matmul_bf16, matmul_fused_swiglu, matmul_silu_mul, tune_matmul_fused_swiglu,
                  tune_matmul_silu_mul)

__all__ = [
    "matmul_silu_mul",
    "matmul_fused_swiglu",
    "matmul_bf16",
    "tune_matmul_silu_mul",
    "tune_matmul_fused_swiglu",
    "TileConfig",
    "SglError",
]
