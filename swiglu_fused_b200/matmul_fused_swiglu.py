"""``matmul_fused_swiglu`` under its reference module name (swiglu/matmul_fused_swiglu.py)."""
from .ops import matmul_fused_swiglu, tune_matmul_fused_swiglu  # noqa: F401

BM = 128  # rows of x per CTA, as in the reference (swiglu/matmul_fused_swiglu.py:30)
