"""Same-GPU comparator: launches the REFERENCE's own sm_100a kernels.  TEST INFRASTRUCTURE ONLY.

``make -C oracle ref`` compiles the reference's two ``.cu`` files, from where they lie,
into ``oracle/_ref/*.cubin`` (git-ignored build output).  This module loads those cubins
with the CUDA driver API through ctypes (the reference itself uses pycuda, which is not
installed) and launches them with the reference's own geometry:

* tensor maps as ``_setup`` builds them (``swiglu/matmul_silu_mul.py:65-75``,
  ``swiglu/_tma_utils.py:69-111``): bf16, rank 2, dims (cols, rows), box 64 x BM / 64 x BK,
  128-byte swizzle, no L2 promotion, no OOB fill;
* grid ``(M/128) * (N/BN)`` blocks of 256 threads, dynamic shared memory
  ``NS * (128 + BN/2) * BK * 2`` bytes, kernel names ``matmul_silu_mul_bm128_bn{BN}_bk{BK}_ns{NS}_gsm{GSM}``
  / ``matmul_fused_swiglu_bm128_...`` (``swiglu/matmul_silu_mul.py:46-47,57-58,78-95``,
  ``swiglu/matmul_fused_swiglu.py:46-53,85-103``).

The reference kernels only accept ``M % 256 == 0``, ``N % BN == 0``, ``K % BK == 0`` and
``K / BK >= NS`` (``swiglu/matmul_silu_mul.py:101-111``); ``check_legal`` enforces that
before anything is launched, because their waits are unbounded.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
CUBIN_V3 = os.path.join(REF_DIR, "matmul_silu_mul.cubin")
CUBIN_V4 = os.path.join(REF_DIR, "matmul_fused_swiglu.cubin")
BM = 128

_modules: dict[str, object] = {}


def available() -> bool:
    return os.path.exists(CUBIN_V3) and os.path.exists(CUBIN_V4)


_cuda = None


def _drv() -> C.CDLL:
    """libcuda through ctypes, as the reference's own helper does (``swiglu/_tma_utils.py:50``)."""
    global _cuda
    if _cuda is None:
        lib = C.CDLL("libcuda.so.1")
        lib.cuModuleLoadData.argtypes = [C.POINTER(C.c_void_p), C.c_char_p]
        lib.cuModuleGetFunction.argtypes = [C.POINTER(C.c_void_p), C.c_void_p, C.c_char_p]
        lib.cuFuncSetAttribute.argtypes = [C.c_void_p, C.c_int, C.c_int]
        lib.cuLaunchKernel.argtypes = [C.c_void_p] + [C.c_uint] * 7 + [C.c_void_p, C.c_void_p,
                                                                       C.c_void_p]
        lib.cuTensorMapEncodeTiled.argtypes = [
            C.c_void_p, C.c_int, C.c_uint32, C.c_void_p, C.POINTER(C.c_uint64),
            C.POINTER(C.c_uint64), C.POINTER(C.c_uint32), C.POINTER(C.c_uint32),
            C.c_int, C.c_int, C.c_int, C.c_int]
        for f in (lib.cuModuleLoadData, lib.cuModuleGetFunction, lib.cuFuncSetAttribute,
                  lib.cuLaunchKernel, lib.cuTensorMapEncodeTiled):
            f.restype = C.c_int
        _cuda = lib
    return _cuda


def _ck(err: int, what: str) -> None:
    if err != 0:
        raise RuntimeError(f"{what} failed with CUresult {err}")


def _function(cubin: str, name: str) -> C.c_void_p:
    d = _drv()
    torch.cuda.init()
    torch.zeros(1, device="cuda")          # make torch's primary context current
    mod = _modules.get(cubin)
    if mod is None:
        with open(cubin, "rb") as f:
            image = f.read()
        mod = C.c_void_p()
        _ck(d.cuModuleLoadData(C.byref(mod), image), "cuModuleLoadData")
        _modules[cubin] = mod
    fn = C.c_void_p()
    _ck(d.cuModuleGetFunction(C.byref(fn), mod, name.encode()), f"cuModuleGetFunction({name})")
    return fn


class _TensorMap:
    """128-byte CUtensorMap in a 64-byte aligned host buffer."""

    def __init__(self):
        self._raw = (C.c_uint8 * 256)()
        self.ptr = (C.addressof(self._raw) + 63) // 64 * 64


def _tmap_2d(t: torch.Tensor, box_rows: int, box_cols: int = 64) -> _TensorMap:
    """The reference's ``build_tma_2d`` for a dense row-major bf16 matrix."""
    d = _drv()
    rows, cols = t.shape
    assert t.is_contiguous() and t.dtype == torch.bfloat16
    m = _TensorMap()
    dims = (C.c_uint64 * 2)(cols, rows)
    strides = (C.c_uint64 * 1)(cols * 2)
    box = (C.c_uint32 * 2)(box_cols, box_rows)
    estr = (C.c_uint32 * 2)(1, 1)
    # bf16 = 9, interleave none = 0, swizzle 128B = 3, L2 promotion none = 0, OOB fill none = 0
    _ck(d.cuTensorMapEncodeTiled(m.ptr, 9, 2, t.data_ptr(), dims, strides, box, estr, 0, 3, 0, 0),
        "cuTensorMapEncodeTiled")
    return m


def check_legal(M: int, N: int, K: int, bn: int, bk: int, ns: int) -> None:
    ok = (M % BM == 0 and N % bn == 0 and K % bk == 0 and K // bk >= ns
          and ((M // BM) * (N // bn)) % 2 == 0 and (M // BM) % 2 == 0
          and ns * (BM + bn // 2) * bk * 2 <= 228 * 1024)
    if not ok:
        raise ValueError(f"shape {M}x{N}x{K} is not legal for the reference kernel "
                         f"(BN={bn}, BK={bk}, NS={ns})")


def _launch(fn, smem: int, grid: int, params: list) -> None:
    """params: ctypes objects (passed by address) or int addresses of by-value structs."""
    d = _drv()
    # CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES = 8
    _ck(d.cuFuncSetAttribute(fn, 8, smem), "cuFuncSetAttribute")
    ptrs = (C.c_void_p * len(params))()
    for i, p in enumerate(params):
        ptrs[i] = p if isinstance(p, int) else C.addressof(p)
    stream = torch.cuda.current_stream().cuda_stream
    _ck(d.cuLaunchKernel(fn, grid, 1, 1, 256, 1, 1, smem, stream, C.addressof(ptrs), None),
        "cuLaunchKernel")


def matmul_silu_mul(A, B_gate, up, bn=256, bk=64, ns=7, gsm=8):
    """The reference's V3 kernel: ``h = silu(A @ B_gate) * up``."""
    M, K = A.shape
    N = B_gate.shape[1]
    check_legal(M, N, K, bn, bk, ns)
    out = torch.empty((M, N), device=A.device, dtype=torch.bfloat16)
    ta, tb = _tmap_2d(A, BM), _tmap_2d(B_gate, bk)
    fn = _function(CUBIN_V3, f"matmul_silu_mul_bm{BM}_bn{bn}_bk{bk}_ns{ns}_gsm{gsm}")
    args = [ta.ptr, tb.ptr, C.c_void_p(out.data_ptr()), C.c_void_p(up.data_ptr()),
            C.c_int32(M), C.c_int32(N), C.c_int32(K)]
    _launch(fn, ns * (BM + bn // 2) * bk * 2, (M // BM) * (N // bn), args)
    return out


def matmul_fused_swiglu(A, W, bn=256, bk=64, ns=7, gsm=8):
    """The reference's V4 kernel: packed ``W = [W_up | W_gate]``."""
    M, K = A.shape
    N = W.shape[1] // 2
    check_legal(M, N, K, bn, bk, ns)
    out = torch.empty((M, N), device=A.device, dtype=torch.bfloat16)
    ta, tw = _tmap_2d(A, BM), _tmap_2d(W, bk)
    fn = _function(CUBIN_V4, f"matmul_fused_swiglu_bm{BM}_bn{bn}_bk{bk}_ns{ns}_gsm{gsm}")
    smem = max(ns * (BM + bn // 2) * bk * 2, BM * (bn + 8) * 2)
    args = [ta.ptr, tw.ptr, C.c_void_p(out.data_ptr()),
            C.c_int32(M), C.c_int32(N), C.c_int32(K)]
    _launch(fn, smem, (M // BM) * (N // bn), args)
    return out
