"""Reference import path for ``matmul_fused_swiglu`` (reference: swiglu/matmul_fused_swiglu.py:152)."""
from swiglu_fused_b200.ops import matmul_fused_swiglu  # noqa: F401
