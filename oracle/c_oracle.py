"""ctypes wrapper of the plain-C oracle (``swiglu_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Rows are split across Python threads (the C calls release the GIL).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libswiglu_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "swiglu_oracle.c")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "-B" if force else "-s", "libswiglu_oracle.so"],
                       check=True, capture_output=True)
    return LIB


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        lib = C.CDLL(LIB)
        i64, vp = C.c_int64, C.c_void_p
        lib.oracle_silu_mul.restype = C.c_int
        lib.oracle_silu_mul.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, C.c_int]
        lib.oracle_fused_swiglu.restype = C.c_int
        lib.oracle_fused_swiglu.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i64,
                                            C.c_int]
        _lib = lib
    return _lib


def _row_blocks(M: int, threads: int):
    step = max(1, -(-M // threads))
    return [(r, min(M, r + step)) for r in range(0, M, step)]


def _check(t: torch.Tensor):
    assert t.dtype == torch.bfloat16 and t.device.type == "cpu" and t.is_contiguous()


def fused_swiglu(x, w, up_col0=None, gate_col0=None, n_out=None, acc64=False,
                 threads: int | None = None) -> torch.Tensor:
    _check(x)
    _check(w)
    M, K = x.shape
    if n_out is None:
        n_out = w.shape[1] // 2
        up_col0, gate_col0 = 0, n_out
    h = torch.empty((M, n_out), dtype=torch.bfloat16)
    lib = load()
    threads = threads or os.cpu_count() or 1

    def run(rows):
        r0, r1 = rows
        rc = lib.oracle_fused_swiglu(x.data_ptr() + r0 * K * 2, w.data_ptr(),
                                     h.data_ptr() + r0 * n_out * 2, r1 - r0, n_out, K, K,
                                     w.shape[1], n_out, up_col0, gate_col0, int(acc64))
        assert rc == 0

    with ThreadPoolExecutor(threads) as ex:
        list(ex.map(run, _row_blocks(M, threads)))
    return h


def silu_mul(x, w_gate, up, acc64=False, threads: int | None = None) -> torch.Tensor:
    _check(x)
    _check(w_gate)
    _check(up)
    M, K = x.shape
    N = w_gate.shape[1]
    h = torch.empty((M, N), dtype=torch.bfloat16)
    lib = load()
    threads = threads or os.cpu_count() or 1

    def run(rows):
        r0, r1 = rows
        rc = lib.oracle_silu_mul(x.data_ptr() + r0 * K * 2, w_gate.data_ptr(),
                                 up.data_ptr() + r0 * N * 2, h.data_ptr() + r0 * N * 2,
                                 r1 - r0, N, K, K, N, N, N, int(acc64))
        assert rc == 0

    with ThreadPoolExecutor(threads) as ex:
        list(ex.map(run, _row_blocks(M, threads)))
    return h
