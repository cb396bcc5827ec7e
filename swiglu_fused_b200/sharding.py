"""Multi-GPU launchers: one process per GPU (``torch.distributed``), no collective
unless the caller asks for the gathered output.

The reference is single-GPU (every launch goes to one device's null stream,
``swiglu/matmul_silu_mul.py:91-94``); these launchers are the multi-GPU form of
its two operators:

* **M-sharded** (tokens): rank r owns rows ``[r0, r0+rows)`` of ``x`` and ``h``,
  the weight is replicated, nothing is exchanged.  ``h`` stays row-sharded, which
  is what the row-independent down-projection that follows wants.
* **N-sharded** (column-parallel): rank r owns output columns ``[c0, c0+cols)``
  and reads the matching ``up`` and ``gate`` column windows of the packed weight
  in place.  ``gather=True`` additionally all-gathers ``h`` over NCCL so every
  rank ends with the full ``[M, N]``.

All functions work with any initialised process group; the host-side logic is
exercised on CPU with the gloo backend (the kernels themselves need a B200).
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import _lib

ROW_ALIGN = 256   # a CTA pair's tile height: shard boundaries never split a pair tile
COL_ALIGN = 128   # the fused form's tile width


@dataclass(frozen=True)
class Shard:
    """Half-open range ``[begin, begin + count)`` owned by one rank."""

    begin: int
    count: int

    @property
    def end(self) -> int:
        return self.begin + self.count


def row_shard(M: int, world: int, rank: int, align: int = ROW_ALIGN) -> Shard:
    return Shard(*_lib.shard_range(M, align, world, rank))


def col_shard(N: int, world: int, rank: int, align: int = COL_ALIGN) -> Shard:
    return Shard(*_lib.shard_range(N, align, world, rank))


def init_from_env(backend: str | None = None) -> tuple[int, int, int]:
    """Join the process group described by RANK / WORLD_SIZE / MASTER_* (torchrun).

    Returns ``(rank, world, local_rank)``; with WORLD_SIZE unset or 1 nothing is
    initialised and ``(0, 1, 0)`` is returned.
    """
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1:
        return 0, 1, local_rank
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {}
        if backend == "nccl":
            torch.cuda.set_device(local_rank)
            kw["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend, rank=rank, world_size=world, **kw)
    return rank, world, local_rank


class SymmetricOutput:
    """A full-width ``[M, N]`` bf16 output buffer on every rank, each mapped into every
    other rank's address space (``torch.distributed._symmetric_memory``; multicast
    objects are not requested - peers are reached with plain stores).  Collective:
    every rank of ``group`` constructs it with the same shape."""

    def __init__(self, M: int, N: int, device, group=None, multicast: bool = False):
        """``multicast=True`` also asks for an NVSwitch multicast mapping of the buffers
        (``multicast_ptr``, 0 where the fabric offers none); the fused gather then sends every
        tile once and the switch replicates it."""
        import torch.distributed._symmetric_memory as symm_mem

        self.M, self.N = M, N
        self.group = group if group is not None else dist.group.WORLD
        before = os.environ.get("TORCH_SYMM_MEM_DISABLE_MULTICAST")
        os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "0" if multicast else "1"
        try:
            self.tensor = symm_mem.empty((M, N), dtype=torch.bfloat16, device=device)
            self.handle = symm_mem.rendezvous(self.tensor, self.group)
        finally:
            if before is None:
                os.environ.pop("TORCH_SYMM_MEM_DISABLE_MULTICAST", None)
            else:
                os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = before
        self.rank = self.handle.rank
        self.world = self.handle.world_size
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0) if multicast else 0

    def barrier(self) -> None:
        """Device-side barrier across the ranks on the current stream."""
        self.handle.barrier(channel=0)


def fused_swiglu_n_sharded_fused_gather(x: torch.Tensor, w: torch.Tensor, out: SymmetricOutput, *,
                                        n_total: int | None = None, stream=None, config=None,
                                        mode: str = "auto"):
    """Column-parallel fused SwiGLU with the all-gather of ``h`` inside the kernel.

    Every rank computes its column block and its epilogue delivers each finished tile into
    that column window of EVERY rank's ``out`` buffer, so the transfer overlaps the remaining
    tiles.  ``mode`` selects how the tiles travel:

    * ``"multicast"``: one ``multimem.st`` per 16 bytes to the NVSwitch multicast mapping of
      the buffers (``SymmetricOutput(..., multicast=True)``); the switch replicates, the
      sender's link carries each byte once;
    * ``"stores"``: the tile goes into this rank's buffer by TMA store and into each peer's by
      ordinary 16-byte stores over NVLink (the same epilogue code as multicast with plain
      addresses: what single-GPU tests can exercise);
    * ``"tma"``: one TMA store per destination (the stores share the SM's TMA queue with the
      operand loads, so a busy link slows the mainloop; kept for comparison);
    * ``"auto"``: multicast where ``out`` has a mapping, else tma (measured on 2, 4 and 8 GPUs:
      multicast < tma < stores).

    Two device-side barriers bracket the launch: nobody overwrites a buffer a peer may still
    be reading, and nobody reads before every peer's stores have landed.  Returns
    ``out.tensor`` (the full ``[M, N]``) on every rank; bit-identical in every mode.
    """
    from .ops import matmul_fused_swiglu_gather, matmul_fused_swiglu_multi_dst, stream_context

    if mode not in ("auto", "multicast", "stores", "tma"):
        raise ValueError(f"unknown gather mode {mode!r}")
    if mode == "auto":
        mode = "multicast" if out.multicast_ptr else "tma"
    if mode == "multicast" and not out.multicast_ptr:
        raise ValueError("this SymmetricOutput has no multicast mapping (construct it with "
                         "multicast=True on a fabric that offers one)")
    N = n_total if n_total is not None else w.shape[1] // 2
    rank, world = out.rank, out.world
    mine = col_shard(N, world, rank)
    ld = out.tensor.stride(0)
    # the two barriers run on torch's current stream: make that the launch stream
    with stream_context(stream, x.device):
        out.barrier()
        if mine.count > 0:
            # peers after this rank, nearest first: ranks start on different NVLink ports
            order = [(rank + i) % world for i in range(world)]
            kw = dict(up_col0=mine.begin, gate_col0=N + mine.begin, n_out=mine.count,
                      stream=stream, config=config)
            if mode == "tma":
                dsts = [out.ptrs[r] + 2 * mine.begin for r in order]
                matmul_fused_swiglu_multi_dst(x, w, dsts, ld, **kw)
            else:
                peers = [out.ptrs[r] + 2 * mine.begin for r in order[1:]]
                mc = out.multicast_ptr + 2 * mine.begin if mode == "multicast" else None
                matmul_fused_swiglu_gather(x, w, out.ptrs[rank] + 2 * mine.begin, peers, ld,
                                           multicast_ptr=mc, **kw)
        out.barrier()
    return out.tensor


class RowShardedOutput:
    """Per-rank ``[rows_per_rank, N]`` accumulation buffer (fp32 by default) in symmetric
    memory: rank r's buffer receives every rank's partial product for the rows r owns.
    Collective constructor, like ``SymmetricOutput``."""

    def __init__(self, M: int, N: int, device, group=None, dtype=torch.float32):
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("accumulation buffer must be fp32 or bf16")
        self.group = group if group is not None else dist.group.WORLD
        world = dist.get_world_size(self.group)
        self.M, self.N = M, N
        # equal row blocks, a multiple of the pair-tile height, the last one possibly ragged
        self.rows_per_rank = -(-(-(-M // world)) // ROW_ALIGN) * ROW_ALIGN
        self.tensor = symm_mem.empty((self.rows_per_rank, N), dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        self.rank, self.world = self.handle.rank, self.handle.world_size
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.my_rows = max(0, min(self.rows_per_rank, M - self.rank * self.rows_per_rank))

    def barrier(self) -> None:
        self.handle.barrier(channel=0)


class RowParallelSlots:
    """Receive buffers of the slot-based reduce-scatter: on every rank a bf16 tensor
    ``[world, rows_per_rank, N]`` in symmetric memory; slot s of rank o holds rank s's
    partial product for the rows o owns.  Collective constructor."""

    def __init__(self, M: int, N: int, device, group=None):
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        world = dist.get_world_size(self.group)
        self.M, self.N = M, N
        self.rows_per_rank = -(-(-(-M // world)) // ROW_ALIGN) * ROW_ALIGN
        self.tensor = symm_mem.empty((world, self.rows_per_rank, N), dtype=torch.bfloat16,
                                     device=device)
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        self.rank, self.world = self.handle.rank, self.handle.world_size
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.my_rows = max(0, min(self.rows_per_rank, M - self.rank * self.rows_per_rank))

    def barrier(self) -> None:
        self.handle.barrier(channel=0)


def down_proj_row_parallel(h_local: torch.Tensor, w_down_local: torch.Tensor, bufs, *,
                           out=None, stream=None, config=None) -> torch.Tensor:
    """``y = h @ W_down`` for a column-sharded ``h`` with the reduce-scatter fused into the
    GEMM, so ``h`` is never gathered.

    Rank r holds ``h_local = h[:, cols_r]`` (what the column-parallel gate/up stage leaves on
    it) and ``w_down_local = W_down[cols_r, :]``.  Returns the complete rows this rank owns.

    ``bufs`` selects the algorithm:

    * ``RowParallelSlots`` (default choice: deterministic, fp32 sums): every tile of the partial product is TMA-stored
      into the owner's slot for this rank while the GEMM runs; after a barrier each rank adds
      its ``world`` slots in fp32 (``sum_bf16_slots``).  Deterministic.  Returns bf16.
    * ``RowShardedOutput``: tiles are ADDED into one shared buffer per owner with TMA
      reduce operations (atomic per element).  Returns a view of that buffer (fp32 or bf16).
      Single pass and, with a bf16 buffer, the fastest form, but every contribution rounds to
      bf16 and the order of additions (hence the last bit) varies from run to run.
    """
    from .ops import matmul_bf16_reduce_scatter, stream_context, sum_bf16_slots

    # zero_() and the barriers run on torch's current stream: make that the launch stream, so
    # that they are ordered with the peer stores and additions of the kernel
    with stream_context(stream, h_local.device):
        if isinstance(bufs, RowParallelSlots):
            slot_bytes = bufs.rows_per_rank * bufs.N * 2
            dsts = [p + bufs.rank * slot_bytes for p in bufs.ptrs]
            bufs.barrier()                 # owners have finished reading the previous contents
            matmul_bf16_reduce_scatter(h_local, w_down_local, dsts, bufs.rows_per_rank, bufs.N,
                                       dst_f32=False, accumulate=False,
                                       first_dst=(bufs.rank + 1) % bufs.world, stream=stream,
                                       config=config)
            bufs.barrier()                 # every rank's tiles have landed
            return sum_bf16_slots(bufs.tensor, out, rows=bufs.my_rows, stream=stream)
        bufs.tensor.zero_()
        bufs.barrier()                     # every buffer is zero before anybody adds into it
        matmul_bf16_reduce_scatter(h_local, w_down_local, bufs.ptrs, bufs.rows_per_rank,
                                   bufs.tensor.stride(0),
                                   dst_f32=bufs.tensor.dtype == torch.float32, accumulate=True,
                                   first_dst=(bufs.rank + 1) % bufs.world, stream=stream,
                                   config=config)
        bufs.barrier()                     # every rank's additions have landed
    return bufs.tensor[:bufs.my_rows]


def fused_swiglu_m_sharded(x_local: torch.Tensor, w: torch.Tensor, *, out=None, stream=None,
                           config=None, op=None) -> torch.Tensor:
    """This rank's rows of ``h``: ``silu(x_local @ W_gate) * (x_local @ W_up)``.

    ``x_local`` is the rank's row block of x (see ``row_shard``), ``w`` the full
    packed weight, replicated on every rank.  No communication.
    """
    if op is None:
        from .ops import matmul_fused_swiglu as op
    return op(x_local, w, out=out, stream=stream, config=config)


def fused_swiglu_n_sharded(x: torch.Tensor, w: torch.Tensor, *, rank: int, world: int,
                           n_total: int | None = None, gather: bool = False,
                           group=None, out=None, stream=None, config=None,
                           op=None) -> torch.Tensor:
    """Column-parallel fused SwiGLU.

    ``x`` is replicated.  ``w`` is the unsplit packed weight ``[K, 2N]``; the rank
    computes its column block ``[c0, c0+cols)`` from the windows ``w[:, c0:...]``
    (up) and ``w[:, N+c0:...]`` (gate) without copying them.

    gather=False: returns the local block ``[M, cols]``.
    gather=True : returns the full ``[M, N]`` on every rank.  Each rank's kernel
                  writes its block into place in the full buffer, and the other
                  blocks arrive through one NCCL all-gather of column blocks.
    """
    if op is None:
        from .ops import matmul_fused_swiglu as op
    N = n_total if n_total is not None else w.shape[1] // 2
    M = x.shape[0]
    mine = col_shard(N, world, rank)
    if not gather:
        if mine.count == 0:
            return x.new_empty((M, 0))
        return op(x, w, up_col0=mine.begin, gate_col0=N + mine.begin, n_out=mine.count,
                  out=out, stream=stream, config=config)

    full = out if out is not None else x.new_empty((M, N))
    if mine.count > 0:
        op(x, w, up_col0=mine.begin, gate_col0=N + mine.begin, n_out=mine.count,
           out=full[:, mine.begin:mine.end], stream=stream, config=config)
    if world == 1:
        return full
    gather_column_blocks(full, N, rank, world, group=group)
    return full


def gather_column_blocks(full: torch.Tensor, N: int, rank: int, world: int, group=None) -> None:
    """In-place all-gather of column blocks of ``full`` ([M, N], row-major).

    Column blocks are strided in memory, so each block is broadcast from its
    owner through a contiguous staging copy; shards are equal-sized except for
    the ragged tail, which this handles too.
    """
    M = full.shape[0]
    shards = [col_shard(N, world, r) for r in range(world)]
    equal = len({s.count for s in shards}) == 1 and shards[0].count > 0
    if equal:
        cols = shards[0].count
        send = full[:, shards[rank].begin:shards[rank].end].contiguous()
        recv = full.new_empty((world, M, cols))
        dist.all_gather_into_tensor(recv.view(world * M, cols), send, group=group)
        for r, s in enumerate(shards):
            if r != rank:
                full[:, s.begin:s.end].copy_(recv[r])
        return
    for r, s in enumerate(shards):
        if s.count == 0:
            continue
        buf = full[:, s.begin:s.end].contiguous() if r == rank else full.new_empty((M, s.count))
        dist.broadcast(buf, src=r, group=group)
        if r != rank:
            full[:, s.begin:s.end].copy_(buf)
