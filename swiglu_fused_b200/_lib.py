"""ctypes binding of ``libswiglu_b200.so`` (the C ABI in ``include/swiglu_b200.h``).

There is no fallback: if the library is missing, or the device is not a B200,
the operators raise.  Nothing in this package computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
import functools
import os
import threading
from dataclasses import dataclass

from . import build as _build

FORM_SILU_MUL = 0
FORM_FUSED_SWIGLU = 1
FORM_MATMUL = 2
FORM_FUSED_SWIGLU_SAVE = 3

QUERY_SM_COUNT = 0
QUERY_MAX_SMEM_OPTIN = 1
QUERY_COMPUTE_CAPABILITY = 2
QUERY_KERNEL_LAUNCHES = 3

MGPU_M_SHARD = 0
MGPU_N_SHARD = 1
MGPU_N_SHARD_GATHER = 2

PIPE_H2D_BYTES = 0
PIPE_H2D_BYTES_NO_WEIGHT = 1
PIPE_D2H_BYTES = 2
PIPE_LAUNCHES = 3
PIPE_LAUNCHES_NO_WEIGHT = 4
PIPE_DEVICE_BYTES = 5
PIPE_PEER_BYTES = 6

# Every symbol include/swiglu_b200.h declares.
EXPORTED_SYMBOLS = (
    "sgl_matmul_silu_mul",
    "sgl_matmul_fused_swiglu",
    "sgl_matmul_fused_swiglu_nk",
    "sgl_matmul_fused_swiglu_save_factors",
    "sgl_swiglu_grad_preact",
    "sgl_matmul_fused_swiglu_multi_dst",
    "sgl_matmul_fused_swiglu_gather",
    "sgl_matmul_bf16",
    "sgl_matmul_bf16_ex",
    "sgl_matmul_bf16_splitk_scratch_bytes",
    "sgl_matmul_bf16_splitk",
    "sgl_matmul_bf16_splitk_static",
    "sgl_matmul_bf16_reduce_scatter",
    "sgl_sum_bf16_slots",
    "sgl_config_count",
    "sgl_config_get",
    "sgl_config_default",
    "sgl_config_smem_bytes",
    "sgl_tile_coord",
    "sgl_tile_coord_slabs",
    "sgl_query",
    "sgl_shard_range",
    "sgl_device_status",
    "sgl_selftest_wait_timeout",
    "sgl_set_wait_limit_ns",
    "sgl_set_splitk_cluster_sum",
    "sgl_splitk_cluster_plan",
    "sgl_host_pipeline_create",
    "sgl_host_pipeline_shared_bytes",
    "sgl_host_pipeline_plan",
    "sgl_host_pipeline_create_shared",
    "sgl_host_pipeline_run",
    "sgl_host_pipeline_query",
    "sgl_host_pipeline_destroy",
    "sgl_mgpu_create",
    "sgl_mgpu_fused_swiglu",
    "sgl_mgpu_size",
    "sgl_mgpu_destroy",
    "sgl_last_error",
    "sgl_version",
)


class SglConfig(C.Structure):
    """Mirror of ``struct sgl_config``."""

    _fields_ = [
        ("cta_group", C.c_int32),
        ("block_k", C.c_int32),
        ("stages", C.c_int32),
        ("group_m", C.c_int32),
        ("max_ctas", C.c_int32),
        ("l2_hints", C.c_int32),
        ("group_n", C.c_int32),
        ("wide", C.c_int32),
    ]


class SglPipeStep(C.Structure):
    """Mirror of ``struct sgl_pipe_step``."""

    _fields_ = [("row0", C.c_int64), ("row1", C.c_int64), ("col0", C.c_int64), ("col1", C.c_int64),
                ("copies_rows", C.c_int32), ("copies_weight_window", C.c_int32),
                ("waits_for_rank", C.c_int32), ("signals_peers", C.c_int32)]


@dataclass(frozen=True)
class TileConfig:
    """One tile-table entry: the (cta_group, block_k, stages, group_m) the kernel runs with.

    Counterpart of the reference's ``(BN, BK, NS, GSM)`` tuples
    (``swiglu/matmul_silu_mul.py:30-41``).
    """

    cta_group: int = 2
    block_k: int = 64
    stages: int = 0
    group_m: int = 8
    max_ctas: int = 0
    l2_hints: int = 0   # see sgl_config.l2_hints: 2 bits each for x, weight, h, up
    group_n: int = 0    # column slabs of the tile order, in tiles (0 = one slab)
    wide: int = 0       # 1 = 256-column tiles (fused form, cta_group 2, block_k 64)

    def to_c(self) -> SglConfig:
        """The C struct for this entry.  Cached per (immutable) entry: the library only reads
        it, and building a ctypes struct costs microseconds on a call path that takes a few."""
        return _config_struct(self)

    @staticmethod
    def from_c(c: SglConfig) -> "TileConfig":
        return TileConfig(c.cta_group, c.block_k, c.stages, c.group_m, c.max_ctas, c.l2_hints,
                          c.group_n, c.wide)


@functools.lru_cache(maxsize=256)
def _config_struct(cfg: "TileConfig") -> SglConfig:
    return SglConfig(cfg.cta_group, cfg.block_k, cfg.stages, cfg.group_m, cfg.max_ctas,
                     cfg.l2_hints, cfg.group_n, cfg.wide)


class SglError(RuntimeError):
    """A non-zero status from the library."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libswiglu_b200 status {code}: {message}")
        self.code = code
        self.message = message


_lock = threading.Lock()
_lib = None


def lib_path() -> str:
    return os.environ.get("SWIGLU_B200_LIB", _build.LIB_PATH)


def load() -> C.CDLL:
    """Load (once) and prototype the shared library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        if not os.path.exists(path) and path == _build.LIB_PATH:
            # A fresh checkout has sources only: compile once if a compiler is at hand.
            try:
                _build.build_library()
            except RuntimeError:
                pass
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python -m swiglu_fused_b200.build` "
                "(needs nvcc); there is no fallback path")
        lib = C.CDLL(path)
        i64, vp, ip = C.c_int64, C.c_void_p, C.c_int
        cfgp = C.POINTER(SglConfig)
        lib.sgl_matmul_silu_mul.restype = ip
        lib.sgl_matmul_silu_mul.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64,
                                            cfgp, vp]
        lib.sgl_matmul_fused_swiglu.restype = ip
        lib.sgl_matmul_fused_swiglu.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, i64,
                                                i64, cfgp, vp]
        lib.sgl_matmul_fused_swiglu_nk.restype = ip
        lib.sgl_matmul_fused_swiglu_nk.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, i64,
                                                   i64, cfgp, vp]
        lib.sgl_matmul_fused_swiglu_save_factors.restype = ip
        lib.sgl_matmul_fused_swiglu_save_factors.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64,
                                                             i64, i64, i64, i64, i64, cfgp, vp]
        lib.sgl_swiglu_grad_preact.restype = ip
        lib.sgl_swiglu_grad_preact.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, vp]
        lib.sgl_matmul_fused_swiglu_multi_dst.restype = ip
        lib.sgl_matmul_fused_swiglu_multi_dst.argtypes = [vp, vp, C.POINTER(vp), ip, i64, i64,
                                                          i64, i64, i64, i64, i64, i64, cfgp, vp]
        lib.sgl_matmul_fused_swiglu_gather.restype = ip
        lib.sgl_matmul_fused_swiglu_gather.argtypes = [vp, vp, vp, C.POINTER(vp), ip, vp, i64, i64,
                                                       i64, i64, i64, i64, i64, i64, cfgp, vp]
        lib.sgl_matmul_bf16.restype = ip
        lib.sgl_matmul_bf16.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, cfgp, vp]
        lib.sgl_matmul_bf16_ex.restype = ip
        lib.sgl_matmul_bf16_ex.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, ip, ip, cfgp,
                                           vp]
        lib.sgl_matmul_bf16_splitk_scratch_bytes.restype = i64
        lib.sgl_matmul_bf16_splitk_scratch_bytes.argtypes = [i64, i64, i64, ip]
        lib.sgl_matmul_bf16_splitk.restype = ip
        lib.sgl_matmul_bf16_splitk.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, ip, vp,
                                               i64, cfgp, vp]
        lib.sgl_matmul_bf16_splitk_static.restype = ip
        lib.sgl_matmul_bf16_splitk_static.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, ip,
                                                      cfgp, vp]
        lib.sgl_matmul_bf16_reduce_scatter.restype = ip
        lib.sgl_matmul_bf16_reduce_scatter.argtypes = [vp, vp, C.POINTER(vp), ip, i64, ip, ip, ip,
                                                       i64, i64, i64, i64, i64, i64, cfgp, vp]
        lib.sgl_sum_bf16_slots.restype = ip
        lib.sgl_sum_bf16_slots.argtypes = [vp, ip, i64, vp, i64, i64, i64, i64, vp]
        lib.sgl_config_count.restype = ip
        lib.sgl_config_count.argtypes = [ip]
        lib.sgl_config_get.restype = ip
        lib.sgl_config_get.argtypes = [ip, ip, cfgp]
        lib.sgl_config_default.restype = ip
        lib.sgl_config_default.argtypes = [ip, i64, i64, i64, cfgp]
        lib.sgl_config_smem_bytes.restype = ip
        lib.sgl_config_smem_bytes.argtypes = [ip, cfgp]
        lib.sgl_tile_coord.restype = ip
        lib.sgl_tile_coord.argtypes = [i64, i64, i64, i64, C.POINTER(i64), C.POINTER(i64)]
        lib.sgl_tile_coord_slabs.restype = ip
        lib.sgl_tile_coord_slabs.argtypes = [i64, i64, i64, i64, i64, C.POINTER(i64),
                                             C.POINTER(i64)]
        lib.sgl_query.restype = ip
        lib.sgl_query.argtypes = [ip, C.POINTER(i64)]
        lib.sgl_shard_range.restype = ip
        lib.sgl_shard_range.argtypes = [i64, i64, ip, ip, C.POINTER(i64), C.POINTER(i64)]
        lib.sgl_device_status.restype = ip
        lib.sgl_device_status.argtypes = [C.POINTER(C.c_uint32)]
        lib.sgl_selftest_wait_timeout.restype = ip
        lib.sgl_selftest_wait_timeout.argtypes = [C.c_uint64, vp]
        lib.sgl_set_wait_limit_ns.restype = ip
        lib.sgl_set_wait_limit_ns.argtypes = [C.c_uint64]
        lib.sgl_set_splitk_cluster_sum.restype = ip
        lib.sgl_set_splitk_cluster_sum.argtypes = [ip]
        lib.sgl_splitk_cluster_plan.restype = ip
        lib.sgl_splitk_cluster_plan.argtypes = [i64, i64, i64, C.POINTER(ip)] + [C.POINTER(ip)] * 3
        lib.sgl_host_pipeline_create.restype = ip
        lib.sgl_host_pipeline_create.argtypes = [ip, i64, i64, i64, i64, i64, ip, cfgp,
                                                 C.POINTER(vp)]
        lib.sgl_host_pipeline_shared_bytes.restype = i64
        lib.sgl_host_pipeline_shared_bytes.argtypes = [ip, i64, i64]
        lib.sgl_host_pipeline_plan.restype = ip
        lib.sgl_host_pipeline_plan.argtypes = [i64, i64, i64, i64, ip, ip, ip, ip, ip,
                                               C.POINTER(SglPipeStep)]
        lib.sgl_host_pipeline_create_shared.restype = ip
        lib.sgl_host_pipeline_create_shared.argtypes = [ip, i64, i64, i64, i64, i64, ip, cfgp, ip,
                                                        ip, C.POINTER(vp), C.POINTER(vp)]
        lib.sgl_host_pipeline_run.restype = ip
        lib.sgl_host_pipeline_run.argtypes = [vp, vp, i64, vp, i64, vp, i64, vp, i64, ip]
        lib.sgl_host_pipeline_query.restype = ip
        lib.sgl_host_pipeline_query.argtypes = [vp, ip, C.POINTER(i64)]
        lib.sgl_host_pipeline_destroy.restype = ip
        lib.sgl_host_pipeline_destroy.argtypes = [vp]
        lib.sgl_mgpu_create.restype = ip
        lib.sgl_mgpu_create.argtypes = [ip, C.POINTER(ip), C.POINTER(vp)]
        lib.sgl_mgpu_fused_swiglu.restype = ip
        lib.sgl_mgpu_fused_swiglu.argtypes = [vp, ip, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp),
                                              i64, i64, i64, i64, i64, i64, cfgp, C.POINTER(vp)]
        lib.sgl_mgpu_size.restype = ip
        lib.sgl_mgpu_size.argtypes = [vp]
        lib.sgl_mgpu_destroy.restype = ip
        lib.sgl_mgpu_destroy.argtypes = [vp]
        lib.sgl_last_error.restype = C.c_char_p
        lib.sgl_last_error.argtypes = []
        lib.sgl_version.restype = ip
        lib.sgl_version.argtypes = []
        _lib = lib
    return _lib


def check(code: int) -> int:
    """Raise on a non-zero status.  Invalid-argument codes become ValueError."""
    if code == 0:
        return 0
    msg = load().sgl_last_error().decode("utf-8", "replace")
    if -5 <= code <= -1 or code == -10:
        raise ValueError(f"libswiglu_b200 status {code}: {msg}")
    raise SglError(code, msg)


def query(what: int) -> int:
    out = C.c_int64(0)
    check(load().sgl_query(what, C.byref(out)))
    return out.value


def kernel_launches() -> int:
    """Kernels this process has launched through the library."""
    return query(QUERY_KERNEL_LAUNCHES)


def builtin_configs(form: int) -> list[TileConfig]:
    lib = load()
    n = lib.sgl_config_count(form)
    if n < 0:
        check(n)
    out = []
    for i in range(n):
        c = SglConfig()
        check(lib.sgl_config_get(form, i, C.byref(c)))
        out.append(TileConfig.from_c(c))
    return out


def default_config(form: int, M: int, N: int, K: int) -> TileConfig:
    c = SglConfig()
    check(load().sgl_config_default(form, M, N, K, C.byref(c)))
    return TileConfig.from_c(c)


def config_smem_bytes(form: int, cfg: TileConfig) -> int:
    c = cfg.to_c()
    n = load().sgl_config_smem_bytes(form, C.byref(c))
    if n < 0:
        check(n)
    return n


def tile_coord(t: int, tiles_m: int, tiles_n: int, group_m: int,
               group_n: int = 0) -> tuple[int, int]:
    m, n = C.c_int64(), C.c_int64()
    if group_n:
        check(load().sgl_tile_coord_slabs(t, tiles_m, tiles_n, group_m, group_n, C.byref(m),
                                          C.byref(n)))
        return m.value, n.value
    check(load().sgl_tile_coord(t, tiles_m, tiles_n, group_m, C.byref(m), C.byref(n)))
    return m.value, n.value


def shard_range(total: int, align: int, world: int, rank: int) -> tuple[int, int]:
    b, c = C.c_int64(), C.c_int64()
    check(load().sgl_shard_range(total, align, world, rank, C.byref(b), C.byref(c)))
    return b.value, c.value


def device_status() -> list[int]:
    """Synchronise, fetch and clear the kernels' error record; raise if one was set."""
    words = (C.c_uint32 * 8)()
    code = load().sgl_device_status(words)
    check(code)
    return list(words)


def set_wait_limit_ns(ns: int) -> None:
    check(load().sgl_set_wait_limit_ns(ns))


def set_splitk_cluster_sum(enabled: bool) -> bool:
    """Whether split-K problems whose K ranges can form thread-block clusters are summed inside
    the GEMM launch through distributed shared memory (default) or always through scratch
    memory and a second kernel.  Returns the previous setting."""
    return bool(load().sgl_set_splitk_cluster_sum(int(bool(enabled))))


B200_CLUSTERS_THAT_FIT = (0, 0, 74, 45, 33, 26, 22, 15, 15)   # GEMM kernel, clusters of n CTAs


def splitk_cluster_plan(M: int, N: int, K: int, clusters_that_fit=B200_CLUSTERS_THAT_FIT) -> dict:
    """The split-K plan for K ranges summed in thread-block clusters (no device needed):
    ``{"ctas", "tile_cols", "ranges", "k_per_range"}``, ``ctas == 0`` if there is none."""
    fit = (C.c_int * 9)(*clusters_that_fit)
    cols, ranges, per = C.c_int(0), C.c_int(0), C.c_int(0)
    n = load().sgl_splitk_cluster_plan(M, N, K, fit, C.byref(cols), C.byref(ranges), C.byref(per))
    if n < 0:
        check(n)
    return {"ctas": n, "tile_cols": cols.value, "ranges": ranges.value, "k_per_range": per.value}


def host_pipeline_plan(M: int, N: int, *, first_rows: int = 0, block_rows: int = 0,
                       windows: int = 0, world: int = 1, rank: int = 0,
                       copy_weight: bool = True) -> list[dict]:
    """The step list of the host-buffer pipeline for these sizes (no device needed)."""
    lib = load()
    n = lib.sgl_host_pipeline_plan(M, N, first_rows, block_rows, windows, world, rank,
                                   int(copy_weight), 0, None)
    if n < 0:
        check(n)
    arr = (SglPipeStep * max(n, 1))()
    check(min(0, lib.sgl_host_pipeline_plan(M, N, first_rows, block_rows, windows, world, rank,
                                            int(copy_weight), n, arr)))
    return [{f: getattr(arr[i], f) for f, _ in SglPipeStep._fields_} for i in range(n)]
