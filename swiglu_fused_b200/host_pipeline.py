"""End-to-end path for callers whose tensors live in HOST memory.

``HostPipeline.run(x_host, w_host, h_host)`` does what a caller of the operator
with host buffers has to do - copy x and W in, run the fused kernel, copy h out -
but in row blocks on three streams, so the host->device copy of block i+1, the
kernel of block i and the device->host copy of block i-1 overlap.  Device
buffers are allocated once, at construction; ``run`` allocates nothing.

The reference has no such path (its benchmark creates every tensor on the GPU,
``bench_fused.py:35-36``); this exists so the end-to-end cost, PCIe included, can
be measured through the same public operator.
"""
from __future__ import annotations

import torch

from .ops import matmul_fused_swiglu, matmul_silu_mul


class HostPipeline:
    """Fused form: ``h_host = silu(x_host @ W_gate) * (x_host @ W_up)``."""

    def __init__(self, M: int, K: int, N: int, *, device="cuda:0", blocks: int = 8,
                 row_align: int = 256, config=None):
        self.M, self.K, self.N = M, K, N
        self.device = torch.device(device)
        self.config = config
        rows = -(-M // blocks)
        rows = max(row_align, -(-rows // row_align) * row_align)
        self.bounds = [(r, min(M, r + rows)) for r in range(0, M, rows)]
        with torch.cuda.device(self.device):
            self.x_d = torch.empty((M, K), dtype=torch.bfloat16, device=self.device)
            self.w_d = torch.empty((K, 2 * N), dtype=torch.bfloat16, device=self.device)
            self.h_d = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
            self.s_in = torch.cuda.Stream(self.device)
            self.s_run = torch.cuda.Stream(self.device)
            self.s_out = torch.cuda.Stream(self.device)
            n = len(self.bounds)
            self.ev_w = torch.cuda.Event()
            self.ev_x = [torch.cuda.Event() for _ in range(n)]
            self.ev_h = [torch.cuda.Event() for _ in range(n)]
        self.h2d_bytes = 2 * (M * K + K * 2 * N)
        self.d2h_bytes = 2 * M * N
        self.launches_per_run = len(self.bounds)

    def run(self, x_host: torch.Tensor, w_host: torch.Tensor, h_host: torch.Tensor,
            copy_weight: bool = True) -> torch.Tensor:
        """One pass.  Host tensors should be pinned so the copies are asynchronous.
        Returns ``h_host`` after the last device->host copy has completed."""
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        with torch.cuda.stream(self.s_in):
            if copy_weight:
                self.w_d.copy_(w_host, non_blocking=True)
            self.ev_w.record(self.s_in)
            for i, (r0, r1) in enumerate(self.bounds):
                self.x_d[r0:r1].copy_(x_host[r0:r1], non_blocking=True)
                self.ev_x[i].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.ev_w)
            for i, (r0, r1) in enumerate(self.bounds):
                self.s_run.wait_event(self.ev_x[i])
                matmul_fused_swiglu(self.x_d[r0:r1], self.w_d, out=self.h_d[r0:r1],
                                    config=self.config)
                self.ev_h[i].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            for i, (r0, r1) in enumerate(self.bounds):
                self.s_out.wait_event(self.ev_h[i])
                h_host[r0:r1].copy_(self.h_d[r0:r1], non_blocking=True)
        self.s_out.synchronize()
        return h_host


class HostPipelineSiluMul:
    """silu_mul form: ``h_host = silu(x_host @ W_gate) * up_host`` in row blocks."""

    def __init__(self, M: int, K: int, N: int, *, device="cuda:0", blocks: int = 8,
                 row_align: int = 256, config=None):
        self.M, self.K, self.N = M, K, N
        self.device = torch.device(device)
        self.config = config
        rows = -(-M // blocks)
        rows = max(row_align, -(-rows // row_align) * row_align)
        self.bounds = [(r, min(M, r + rows)) for r in range(0, M, rows)]
        with torch.cuda.device(self.device):
            self.x_d = torch.empty((M, K), dtype=torch.bfloat16, device=self.device)
            self.w_d = torch.empty((K, N), dtype=torch.bfloat16, device=self.device)
            self.up_d = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
            self.h_d = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
            self.s_in = torch.cuda.Stream(self.device)
            self.s_run = torch.cuda.Stream(self.device)
            self.s_out = torch.cuda.Stream(self.device)
            n = len(self.bounds)
            self.ev_w = torch.cuda.Event()
            self.ev_x = [torch.cuda.Event() for _ in range(n)]
            self.ev_h = [torch.cuda.Event() for _ in range(n)]
        self.h2d_bytes = 2 * (M * K + K * N + M * N)
        self.d2h_bytes = 2 * M * N
        self.launches_per_run = len(self.bounds)

    def run(self, x_host, w_gate_host, up_host, h_host, copy_weight: bool = True):
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        with torch.cuda.stream(self.s_in):
            if copy_weight:
                self.w_d.copy_(w_gate_host, non_blocking=True)
            self.ev_w.record(self.s_in)
            for i, (r0, r1) in enumerate(self.bounds):
                self.x_d[r0:r1].copy_(x_host[r0:r1], non_blocking=True)
                self.up_d[r0:r1].copy_(up_host[r0:r1], non_blocking=True)
                self.ev_x[i].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.ev_w)
            for i, (r0, r1) in enumerate(self.bounds):
                self.s_run.wait_event(self.ev_x[i])
                matmul_silu_mul(self.x_d[r0:r1], self.w_d, self.up_d[r0:r1],
                                out=self.h_d[r0:r1], config=self.config)
                self.ev_h[i].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            for i, (r0, r1) in enumerate(self.bounds):
                self.s_out.wait_event(self.ev_h[i])
                h_host[r0:r1].copy_(self.h_d[r0:r1], non_blocking=True)
        self.s_out.synchronize()
        return h_host
