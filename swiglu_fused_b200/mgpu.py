"""Single-process multi-GPU launcher (``sgl_mgpu_*``): one Python process, several GPUs.

The package's other multi-GPU launchers (``sharding.py``) run one process per GPU under
``torch.distributed``; this one is for a host that keeps all its devices in one process, as the
reference's single-process launch layer would if it were extended beyond one GPU
(``swiglu/_pycuda_loader.py:47-55`` binds exactly one context).  The tensors of device ``r`` are
the ``r``-th entries of the lists; the work is enqueued on each device's current torch stream
and nothing waits on the host.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from . import _lib

MODES = {"m_shard": _lib.MGPU_M_SHARD, "n_shard": _lib.MGPU_N_SHARD,
         "n_shard_gather": _lib.MGPU_N_SHARD_GATHER}


class DeviceGroup:
    """``DeviceGroup([0, 1, ...])``: the GPUs of this process that share one launch."""

    def __init__(self, devices: Sequence[int]):
        self.devices = [int(d) for d in devices]
        self._lib = _lib.load()
        self._handle = C.c_void_p()
        arr = (C.c_int * len(self.devices))(*self.devices)
        _lib.check(self._lib.sgl_mgpu_create(len(self.devices), arr, C.byref(self._handle)))

    def __len__(self) -> int:
        return self._lib.sgl_mgpu_size(self._handle)

    def close(self) -> None:
        if self._handle:
            self._lib.sgl_mgpu_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def shard(self, total: int, align: int, rank: int) -> tuple[int, int]:
        """(begin, count) of shard ``rank``: rows with align 256, columns with align 128."""
        return _lib.shard_range(total, align, len(self.devices), rank)

    def fused_swiglu(self, mode: str, x: Sequence[torch.Tensor], w: Sequence[torch.Tensor],
                     h: Sequence[torch.Tensor], M: int, N: int, K: int, config=None) -> None:
        """Enqueue the fused form on every device of the group.

        ``m_shard``: ``x[r]`` = rows of shard r ``[rows_r, K]``, ``h[r]`` = ``[rows_r, N]``.
        ``n_shard``: ``x[r]`` = full ``[M, K]``, ``h[r]`` = ``[M, cols_r]`` (all with one pitch).
        ``n_shard_gather``: ``x[r]`` = full ``[M, K]``, ``h[r]`` = full ``[M, N]`` on every device.
        ``w[r]`` is always the unsplit packed ``[K, 2N]`` weight on device r.
        """
        if not self._handle:
            raise RuntimeError("device group is closed")
        if mode not in MODES:
            raise ValueError(f"mode must be one of {sorted(MODES)}, got {mode!r}")
        n = len(self.devices)
        if not (len(x) == len(w) == len(h) == n):
            raise ValueError(f"x, w and h must each have {n} entries")
        for r, (xr, wr, hr) in enumerate(zip(x, w, h)):
            for name, t in (("x", xr), ("w", wr), ("h", hr)):
                if t.device.type != "cuda" or t.device.index != self.devices[r]:
                    raise ValueError(f"{name}[{r}] is on {t.device}, expected cuda:{self.devices[r]}")
                if t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
                    raise ValueError(f"{name}[{r}] must be a 2-D bfloat16 tensor with unit "
                                     "stride along its rows")
            if tuple(wr.shape) != (K, 2 * N):
                raise ValueError(f"w[{r}] must be [{K}, {2 * N}], got {tuple(wr.shape)}")
            rows = self.shard(M, 256, r)[1] if mode == "m_shard" else M
            cols = self.shard(N, 128, r)[1] if mode == "n_shard" else N
            if tuple(xr.shape) != (rows, K):
                raise ValueError(f"x[{r}] must be [{rows}, {K}], got {tuple(xr.shape)}")
            if tuple(hr.shape) != (rows, cols):
                raise ValueError(f"h[{r}] must be [{rows}, {cols}], got {tuple(hr.shape)}")
        for name, ts in (("x", x), ("w", w), ("h", h)):
            if len({t.stride(0) for t in ts}) != 1:
                raise ValueError(f"all {name}[r] must have the same row pitch")
        vp = C.c_void_p * n
        streams = vp(*[torch.cuda.current_stream(d).cuda_stream for d in self.devices])
        cfg = C.byref(config.to_c()) if config is not None else None
        _lib.check(self._lib.sgl_mgpu_fused_swiglu(
            self._handle, MODES[mode], vp(*[t.data_ptr() for t in x]),
            vp(*[t.data_ptr() for t in w]), vp(*[t.data_ptr() for t in h]), M, N, K,
            x[0].stride(0), w[0].stride(0), h[0].stride(0), cfg, streams))
