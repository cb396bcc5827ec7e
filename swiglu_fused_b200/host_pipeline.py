"""End-to-end path for callers whose tensors live in HOST memory.

``HostPipeline.run(x_host, w_host, h_host)`` does what a caller of the operator with host
buffers has to do - copy x and W in, run the fused kernel, copy h out - through the library's
native pipeline (``sgl_host_pipeline_*``): copies in, launches and copies out overlap on three
streams, and the first rows are computed one weight column window at a time so that the copy
out of ``h`` (the longest leg) starts while the weight is still arriving.  Device buffers are
allocated once, at construction; ``run`` allocates nothing and returns when ``h_host`` is
complete.

The reference has no such path (its benchmark creates every tensor on the GPU,
``bench_fused.py:35-36``); this exists so the end-to-end cost, PCIe included, can be measured
through the same public operator.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib


def _check_host(t: torch.Tensor, name: str, rows: int, cols: int) -> None:
    if t.device.type != "cpu":
        raise ValueError(f"{name} must be a host tensor, got {t.device}")
    if t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be bfloat16, got {t.dtype}")
    if t.dim() != 2 or tuple(t.shape) != (rows, cols):
        raise ValueError(f"{name} must be [{rows}, {cols}], got {tuple(t.shape)}")
    if t.stride(1) != 1:
        raise ValueError(f"{name} must have unit stride along its rows")


class _NativePipeline:
    form = _lib.FORM_FUSED_SWIGLU

    def __init__(self, M: int, K: int, N: int, *, device="cuda:0", first_rows: int = 0,
                 block_rows: int = 0, windows: int = 0, config=None):
        self.M, self.K, self.N = M, K, N
        self.device = torch.device(device)
        self._lib = _lib.load()
        self._handle = C.c_void_p()
        cfg = C.byref(config.to_c()) if config is not None else None
        with torch.cuda.device(self.device):
            self._create(first_rows, block_rows, windows, cfg)
        self._read_counters()

    def _create(self, first_rows, block_rows, windows, cfg) -> None:
        _lib.check(self._lib.sgl_host_pipeline_create(
            self.form, self.M, self.N, self.K, first_rows, block_rows, windows, cfg,
            C.byref(self._handle)))

    def _read_counters(self) -> None:
        self.h2d_bytes = self._query(_lib.PIPE_H2D_BYTES)
        self.h2d_bytes_no_weight = self._query(_lib.PIPE_H2D_BYTES_NO_WEIGHT)
        self.d2h_bytes = self._query(_lib.PIPE_D2H_BYTES)
        self.launches_per_run = self._query(_lib.PIPE_LAUNCHES)
        self.launches_per_run_no_weight = self._query(_lib.PIPE_LAUNCHES_NO_WEIGHT)
        self.device_bytes = self._query(_lib.PIPE_DEVICE_BYTES)
        self.peer_bytes = self._query(_lib.PIPE_PEER_BYTES)

    def _query(self, what: int) -> int:
        out = C.c_int64()
        _lib.check(self._lib.sgl_host_pipeline_query(self._handle, what, C.byref(out)))
        return out.value

    def close(self) -> None:
        if self._handle:
            self._lib.sgl_host_pipeline_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _run(self, x_host, w_host, up_host, h_host, copy_weight: bool):
        if not self._handle:
            raise RuntimeError("pipeline is closed")
        _check_host(x_host, "x_host", self.M, self.K)
        _check_host(h_host, "h_host", self.M, self.N)
        w_cols = 2 * self.N if self.form == _lib.FORM_FUSED_SWIGLU else self.N
        if copy_weight:
            _check_host(w_host, "w_host", self.K, w_cols)
        if up_host is not None:
            _check_host(up_host, "up_host", self.M, self.N)
        _lib.check(self._lib.sgl_host_pipeline_run(
            self._handle, x_host.data_ptr(), x_host.stride(0),
            w_host.data_ptr() if copy_weight else None, w_host.stride(0) if copy_weight else 0,
            up_host.data_ptr() if up_host is not None else None,
            up_host.stride(0) if up_host is not None else 0,
            h_host.data_ptr(), h_host.stride(0), 1 if copy_weight else 0))
        return h_host


class HostPipeline(_NativePipeline):
    """Fused form: ``h_host = silu(x_host @ W_gate) * (x_host @ W_up)``, ``W = [W_up | W_gate]``."""

    form = _lib.FORM_FUSED_SWIGLU

    def run(self, x_host: torch.Tensor, w_host: torch.Tensor, h_host: torch.Tensor,
            copy_weight: bool = True) -> torch.Tensor:
        """One pass.  Host tensors should be pinned so the copies are asynchronous.
        Returns ``h_host`` after the last device->host copy has completed."""
        return self._run(x_host, w_host, None, h_host, copy_weight)


class SharedWeightHostPipeline(HostPipeline):
    """``HostPipeline`` for a process group whose ranks run the same weight on different rows
    (the M-sharded launch, one process per GPU).  Collective: every rank constructs it, with its
    own row count ``M``, and every rank calls ``run`` the same number of times.  Each rank copies
    only its 1/world column slice of ``w_host`` over PCIe; the slices travel on to the other
    ranks' weight buffers over NVLink (``sgl_host_pipeline_create_shared``), so the weight
    crosses the host link once per group.  The weight buffers are one symmetric-memory
    allocation per rank (``torch.distributed._symmetric_memory``, no multicast object)."""

    def __init__(self, M: int, K: int, N: int, *, device="cuda:0", group=None, **kw):
        import os

        import torch.distributed as dist
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        nbytes = _lib.load().sgl_host_pipeline_shared_bytes(self.form, N, K)
        if nbytes < 0:
            _lib.check(int(nbytes))
        self._region = symm_mem.empty(int(nbytes), dtype=torch.uint8, device=torch.device(device))
        self._region.zero_()
        self._symm = symm_mem.rendezvous(self._region, self.group)
        self.rank, self.world = self._symm.rank, self._symm.world_size
        self._ptrs = [int(p) for p in self._symm.buffer_ptrs]
        torch.cuda.synchronize(torch.device(device))
        dist.barrier(group=self.group)          # every region is zero before anybody signals
        super().__init__(M, K, N, device=device, **kw)
        dist.barrier(group=self.group)

    def _create(self, first_rows, block_rows, windows, cfg) -> None:
        arr = (C.c_void_p * self.world)(*self._ptrs)
        _lib.check(self._lib.sgl_host_pipeline_create_shared(
            self.form, self.M, self.N, self.K, first_rows, block_rows, windows, cfg,
            self.world, self.rank, arr, C.byref(self._handle)))

    def close(self, barrier: bool = True) -> None:
        """Collective (like the constructor): the ranks meet at a barrier first, because a
        region may only be released once no peer can still push a weight slice into it."""
        if self._handle and barrier:
            import torch.distributed as dist
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
        super().close()          # the native pipeline first: it borrows the regions
        self._region = None

    def __del__(self):
        try:
            self.close(barrier=False)    # no collective from a finaliser
        except Exception:
            pass


class HostPipelineSiluMul(_NativePipeline):
    """silu_mul form: ``h_host = silu(x_host @ W_gate) * up_host``."""

    form = _lib.FORM_SILU_MUL

    def run(self, x_host, w_gate_host, up_host, h_host, copy_weight: bool = True):
        return self._run(x_host, w_gate_host, up_host, h_host, copy_weight)


def _main() -> None:
    """``python -m swiglu_fused_b200.host_pipeline``: time the pipeline on the headline shape
    (or ``--rows/--k/--n``) for one or several schedules, next to the raw copy rates of the
    host link.  Prints one line per schedule; every result is checked, bit for bit, against the
    device-resident operator."""
    import argparse
    import time

    from .ops import matmul_fused_swiglu

    ap = argparse.ArgumentParser(description="time the host-buffer pipeline")
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--k", type=int, default=3072)
    ap.add_argument("--n", type=int, default=12288)
    ap.add_argument("--schedule", action="append", default=None, metavar="FIRST,BLOCK,WINDOWS",
                    help="first_rows,block_rows,windows (0 = default); may be repeated")
    ap.add_argument("--reps", type=int, default=6)
    args = ap.parse_args()
    M, K, N = args.rows, args.k, args.n
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn((M, K), device=dev, dtype=torch.bfloat16, generator=g)
    w = torch.empty((K, 2 * N), device=dev, dtype=torch.bfloat16).normal_(0, K ** -0.5, generator=g)
    want = matmul_fused_swiglu(x, w)
    xh = torch.empty((M, K), dtype=torch.bfloat16).pin_memory()
    wh = torch.empty((K, 2 * N), dtype=torch.bfloat16).pin_memory()
    hh = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    xh.copy_(x)
    wh.copy_(w)
    for name, dst, src in (("host->device (x)", x, xh), ("device->host (h)", hh, want)):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(3):
            dst.copy_(src, non_blocking=True)
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / 3
        print(f"{name}: {src.numel() * 2 / dt / 1e9:.1f} GB/s ({dt * 1e3:.2f} ms)")
    schedules = [tuple(int(v) for v in s.split(",")) for s in (args.schedule or ["0,0,0"])]
    for first, block, windows in schedules:
        pipe = HostPipeline(M, K, N, device=dev, first_rows=first, block_rows=block,
                            windows=windows)
        for _ in range(2):
            pipe.run(xh, wh, hh)
        same = torch.equal(hh.view(torch.int16), want.cpu().view(torch.int16))
        with_w, without_w = [], []
        for _ in range(args.reps):
            t0 = time.perf_counter()
            pipe.run(xh, wh, hh)
            with_w.append((time.perf_counter() - t0) * 1e3)
        for _ in range(args.reps):
            t0 = time.perf_counter()
            pipe.run(xh, None, hh, copy_weight=False)
            without_w.append((time.perf_counter() - t0) * 1e3)
        print(f"first_rows={first} block_rows={block} windows={windows}: "
              f"{sorted(with_w)[len(with_w) // 2]:.2f} ms per run "
              f"({pipe.launches_per_run} launches), weight resident "
              f"{sorted(without_w)[len(without_w) // 2]:.2f} ms, "
              f"bit-identical to the device run: {same}")
        pipe.close()


if __name__ == "__main__":
    _main()
