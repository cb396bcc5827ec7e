"""``matmul_silu_mul`` under its reference module name (swiglu/matmul_silu_mul.py)."""
from .ops import matmul_silu_mul, tune_matmul_silu_mul  # noqa: F401

BM = 128  # rows of x per CTA, as in the reference (swiglu/matmul_silu_mul.py:26)
