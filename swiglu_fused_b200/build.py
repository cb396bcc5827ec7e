"""Ahead-of-time build of ``libswiglu_b200.so`` (nvcc, sm_100a only).

Replaces the reference's per-process nvcc JIT + cubin cache
(``swiglu/_pycuda_loader.py:71-78,128-144``): the library is compiled once, in
tree, next to this file, and loaded with ``ctypes``.

Run ``python -m swiglu_fused_b200.build`` to (re)build.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC_DIR = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libswiglu_b200.so")
SOURCES = [os.path.join(CSRC_DIR, "swiglu_abi.cu")]
HEADERS = [
    os.path.join(CSRC_DIR, "swiglu_kernel.cuh"),
    os.path.join(CSRC_DIR, "swiglu_elementwise.cuh"),
    os.path.join(CSRC_DIR, "ptx_sm100.cuh"),
    os.path.join(CSRC_DIR, "swiglu_host_pipeline.cuh"),
    os.path.join(CSRC_DIR, "swiglu_mgpu.cuh"),
    os.path.join(os.path.dirname(PKG_DIR), "include", "swiglu_b200.h"),
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
]


def find_nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or add it to PATH")
    return cand


def is_stale() -> bool:
    """True if the library is missing or older than any of its sources."""
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(p) > built for p in SOURCES + HEADERS if os.path.exists(p))


DEBUG_LIB_PATH = os.path.join(PKG_DIR, "libswiglu_b200_debug.so")


def build_debug_library(force: bool = False) -> str:
    """The self-checking build (``-DSGL_DEBUG``): every TMA coordinate is checked before the
    copy is issued and every kernel role counts its work; violations are recorded in the
    status words, nothing traps.  Load it with ``SWIGLU_B200_LIB=<path>``."""
    srcs = [p for p in SOURCES + HEADERS if os.path.exists(p)]
    if not force and os.path.exists(DEBUG_LIB_PATH) and \
            all(os.path.getmtime(p) <= os.path.getmtime(DEBUG_LIB_PATH) for p in srcs):
        return DEBUG_LIB_PATH
    cmd = [find_nvcc(), *NVCC_FLAGS, "-DSGL_DEBUG", "-o", DEBUG_LIB_PATH, *SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    return DEBUG_LIB_PATH


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or stale; return its path."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [find_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", LIB_PATH, *SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        sys.stderr.write(proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force=True, verbose="-v" in sys.argv))
