"""Drop-in import path: ``swiglu.matmul_silu_mul`` / ``swiglu.matmul_fused_swiglu``
resolve to the B200-native operators of ``swiglu_fused_b200``, so the
reference's ``bench.py`` and ``bench_fused.py`` import lines work unchanged."""
