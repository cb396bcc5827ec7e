"""Reference import path for ``matmul_silu_mul`` (reference: swiglu/matmul_silu_mul.py:142)."""
from swiglu_fused_b200.ops import matmul_silu_mul  # noqa: F401
