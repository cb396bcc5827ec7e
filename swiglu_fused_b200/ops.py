"""The two operators, on the reference's Python surface.

``matmul_silu_mul(A, B_gate, up)``      mirrors ``swiglu/matmul_silu_mul.py:142-161``
``matmul_fused_swiglu(A, W)``           mirrors ``swiglu/matmul_fused_swiglu.py:152-172``

Same positional arguments, same result (a new ``[M, N]`` bf16 CUDA tensor).
Differences, all on purpose:

* inputs are validated (dtype, device, layout, alignment) and a bad call raises
  before anything is launched; the reference only asserts shapes;
* the launch goes to torch's current stream (or ``stream=``), not the null stream;
* ``out=`` lets the caller own the output (no allocation inside the call);
* ``config=`` pins a tile configuration; otherwise the persisted tile table,
  then the library default, decides;
* any ``M >= 1`` and any ``N``, ``K`` that are multiples of 8 are accepted;
* there is no CPU or eager fallback: without the CUDA library and a B200 the
  call raises.
"""
from __future__ import annotations

import contextlib
import ctypes as C
import os

import torch

from . import _lib, tile_table
from ._lib import TileConfig

DTYPE = torch.bfloat16


def _check_matrix(t: torch.Tensor, name: str, allow_empty_rows: bool = False) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor, got {type(t).__name__}")
    shape = t.shape
    if len(shape) != 2:
        raise ValueError(f"{name} must be 2-D, got shape {tuple(shape)}")
    if t.dtype != DTYPE:
        raise TypeError(f"{name} must be torch.bfloat16, got {t.dtype}")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this operator has no CPU path)")
    rows, cols = shape
    if cols < 1 or (rows < 1 and not allow_empty_rows):
        raise ValueError(f"{name} must not be empty, got shape {tuple(shape)}")
    if rows == 0:
        return
    s0, s1 = t.stride()
    if s1 != 1:
        raise ValueError(f"{name} must be row-major with unit column stride, "
                         f"got strides {(s0, s1)}")
    if rows > 1:
        if s0 < cols:
            raise ValueError(f"{name} has overlapping rows: strides {(s0, s1)}")
        if s0 % 8 != 0:
            raise ValueError(f"{name}: row stride {s0} must be a multiple of 8 elements")
    if t.data_ptr() % 16 != 0:
        raise ValueError(f"{name} must be 16-byte aligned")


class _OnDevice:
    """``with _on_device(dev):`` makes ``dev`` the current CUDA device for the library call and
    restores the previous one - but only when it is not current already, which on the usual
    single-device call path saves the several microseconds ``torch.cuda.device`` costs."""

    __slots__ = ("idx", "prev")

    def __init__(self, dev: torch.device):
        self.idx = dev.index if dev.index is not None else torch.cuda.current_device()
        self.prev = -1

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


_on_device = _OnDevice


def _ld(t: torch.Tensor) -> int:
    # A single-row tensor may report any stride; use the dense pitch (rounded to 8).
    if t.shape[0] == 1:
        return (t.shape[1] + 7) // 8 * 8
    return t.stride(0)


def _same_device(*named: tuple[str, torch.Tensor]) -> torch.device:
    dev = named[0][1].device
    for name, t in named[1:]:
        if t.device != dev:
            raise ValueError(f"{name} is on {t.device}, expected {dev}")
    return dev


# torch's raw-stream accessor (what its own compiled kernels use) is several times cheaper than
# building a torch.cuda.Stream object per call; fall back to the public API where it is absent.
_raw_current_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_handle(stream, device) -> int:
    if stream is None:
        if _raw_current_stream is not None and device.index is not None:
            return _raw_current_stream(device.index)
        return torch.cuda.current_stream(device).cuda_stream
    if isinstance(stream, torch.cuda.Stream):
        return stream.cuda_stream
    return int(stream)


def stream_context(stream, device):
    """Context manager that makes ``stream`` torch's current stream on ``device`` (a no-op for
    ``None``).  Work that torch itself enqueues around a launch - allocator bookkeeping of a
    temporary, ``zero_()``, a symmetric-memory barrier - is ordered with the launch only if it
    runs on the same stream, so callers that accept ``stream=`` wrap such work in this."""
    if stream is None:
        return contextlib.nullcontext()
    if not isinstance(stream, torch.cuda.Stream):
        stream = torch.cuda.ExternalStream(int(stream), device=device)
    return torch.cuda.stream(stream)


def _pick_config(form: int, config: TileConfig | None, M: int, N: int, K: int):
    if config is not None:
        return config
    return tile_table.lookup(form, M, N, K)


def _prep_out(out, M, N, device, name="out"):
    if out is None:
        return torch.empty((M, N), dtype=DTYPE, device=device)
    _check_matrix(out, name)
    if tuple(out.shape) != (M, N):
        raise ValueError(f"{name} shape {tuple(out.shape)} != {(M, N)}")
    if out.device != device:
        raise ValueError(f"{name} is on {out.device}, expected {device}")
    return out


def matmul_silu_mul(A, B_gate, up, *, out=None, stream=None, config: TileConfig | None = None):
    """h = silu(A @ B_gate) * up.

    A      : [M, K] bf16
    B_gate : [K, N] bf16
    up     : [M, N] bf16  (precomputed x @ W_up)
    returns: [M, N] bf16

    Without ``config``, narrow problems at decode sizes (up to 128 rows, K >= 4096, few tiles)
    take the cluster plan described for ``matmul_fused_swiglu``.
    """
    _check_matrix(A, "A", allow_empty_rows=True)
    _check_matrix(B_gate, "B_gate")
    _check_matrix(up, "up", allow_empty_rows=True)
    M, K = A.shape
    K2, N = B_gate.shape
    if K2 != K:
        raise ValueError(f"K mismatch: A.K={K} vs B_gate.K={K2}")
    if tuple(up.shape) != (M, N):
        raise ValueError(f"up shape {tuple(up.shape)} != {(M, N)}")
    if K % 8 or N % 8:
        raise ValueError(f"K={K} and N={N} must be multiples of 8")
    dev = _same_device(("A", A), ("B_gate", B_gate), ("up", up))
    if M == 0:   # no tokens: nothing to launch
        return out if out is not None else torch.empty((0, N), dtype=DTYPE, device=dev)
    h = _prep_out(out, M, N, dev)
    if os.environ.get("SWIGLU_B200_AUTOTUNE") == "1" and config is None \
            and tile_table.lookup(_lib.FORM_SILU_MUL, M, N, K) is None:
        tune_matmul_silu_mul(A, B_gate, up)
    cfg = _pick_config(_lib.FORM_SILU_MUL, config, M, N, K)
    cfg_c = cfg.to_c() if cfg is not None else None
    lib = _lib.load()
    with _on_device(dev):
        rc = lib.sgl_matmul_silu_mul(
            A.data_ptr(), B_gate.data_ptr(), up.data_ptr(), h.data_ptr(), M, N, K,
            _ld(A), _ld(B_gate), _ld(up), _ld(h),
            C.byref(cfg_c) if cfg_c is not None else None, _stream_handle(stream, dev))
    _lib.check(rc)
    return h


def matmul_fused_swiglu(A, W, *, out=None, stream=None, config: TileConfig | None = None,
                        up_col0: int | None = None, gate_col0: int | None = None,
                        n_out: int | None = None, w_layout: str = "kn"):
    """Single-kernel SwiGLU.  C = silu(gate) * up  where [up|gate] = A @ W.

    A : [M, K]  bf16
    W : [K, 2N] bf16 - left half = W_up, right half = W_gate
    returns: [M, N] bf16

    ``up_col0``/``gate_col0``/``n_out`` (all three together) select two column
    windows of a wider W instead: ``h = silu(A @ W[:, gate_col0:gate_col0+n_out])
    * (A @ W[:, up_col0:up_col0+n_out])`` - how a column-parallel shard addresses
    the unsplit packed weight.

    ``w_layout="nk"``: W is the checkpoint (``nn.Linear``) layout ``[2N, K]`` = ``[W_up^T ;
    W_gate^T]`` and is consumed as is (no transpose); the window arguments then count rows.

    Without ``config``, problems of up to 128 rows with K >= 4096 and few tiles (a narrow FFN at
    decode batch sizes) are cut along K into ranges that run as thread-block clusters; the CTAs
    of a cluster exchange their partial tiles through distributed shared memory and apply the
    activation to the columns they sum.  Deterministic; ``_lib.set_splitk_cluster_sum(False)``
    keeps whole-K tiles.
    """
    if w_layout not in ("kn", "nk"):
        raise ValueError(f"w_layout must be 'kn' or 'nk', got {w_layout!r}")
    _check_matrix(A, "A", allow_empty_rows=True)
    _check_matrix(W, "W")
    M, K = A.shape
    K2, N2 = W.shape if w_layout == "kn" else (W.shape[1], W.shape[0])
    if K != K2:
        raise ValueError(f"K mismatch: A.K={K} vs W.K={K2}")
    windowed = (up_col0 is not None, gate_col0 is not None, n_out is not None)
    if any(windowed) and not all(windowed):
        raise ValueError("up_col0, gate_col0 and n_out must be given together")
    if all(windowed):
        N = int(n_out)
        c_up, c_gate = int(up_col0), int(gate_col0)
        if N < 1 or c_up < 0 or c_gate < 0 or max(c_up, c_gate) + N > N2:
            raise ValueError(f"column windows [{c_up},+{N}) / [{c_gate},+{N}) outside W's {N2} columns")
    else:
        if N2 % 2 != 0:
            raise ValueError(f"W's 2nd dim ({N2}) must be even")
        N = N2 // 2
        c_up, c_gate = 0, N
    if K % 8 or N % 8 or c_up % 8 or c_gate % 8:
        raise ValueError(f"K={K}, N={N} and the column offsets must be multiples of 8")
    dev = _same_device(("A", A), ("W", W))
    if M == 0:   # no tokens: nothing to launch
        return out if out is not None else torch.empty((0, N), dtype=DTYPE, device=dev)
    h = _prep_out(out, M, N, dev)
    if os.environ.get("SWIGLU_B200_AUTOTUNE") == "1" and config is None and not any(windowed) \
            and tile_table.lookup(_lib.FORM_FUSED_SWIGLU, M, N, K) is None:
        tune_matmul_fused_swiglu(A, W)
    cfg = _pick_config(_lib.FORM_FUSED_SWIGLU, config, M, N, K)
    cfg_c = cfg.to_c() if cfg is not None else None
    lib = _lib.load()
    ldw = _ld(W) if W.shape[0] > 1 else max(_ld(W), (W.shape[1] + 7) // 8 * 8)
    entry = lib.sgl_matmul_fused_swiglu if w_layout == "kn" else lib.sgl_matmul_fused_swiglu_nk
    with _on_device(dev):
        rc = entry(
            A.data_ptr(), W.data_ptr(), h.data_ptr(), M, N, K, _ld(A), ldw, _ld(h),
            c_up, c_gate, C.byref(cfg_c) if cfg_c is not None else None,
            _stream_handle(stream, dev))
    _lib.check(rc)
    return h


def matmul_fused_swiglu_multi_dst(A, W, dst_ptrs, ldh: int, *, up_col0: int, gate_col0: int,
                                  n_out: int, stream=None, config: TileConfig | None = None):
    """Fused SwiGLU whose output block is written to several buffers at once.

    ``dst_ptrs[i]`` is the device address of element (0, 0) of this launch's
    ``[M, n_out]`` block inside destination ``i`` (row pitch ``ldh`` elements, bf16);
    destinations may be peer-GPU buffers mapped into this process.  Used by the
    column-parallel launcher to fuse the all-gather of ``h`` into the kernel.  The
    caller owns the buffers and the cross-rank synchronisation.
    """
    _check_matrix(A, "A")
    _check_matrix(W, "W")
    M, K = A.shape
    if W.shape[0] != K:
        raise ValueError(f"K mismatch: A.K={K} vs W.K={W.shape[0]}")
    N = int(n_out)
    if N < 1 or up_col0 < 0 or gate_col0 < 0 or max(up_col0, gate_col0) + N > W.shape[1]:
        raise ValueError("column windows outside W")
    if not 1 <= len(dst_ptrs) <= 8:
        raise ValueError(f"need 1..8 destinations, got {len(dst_ptrs)}")
    dev = _same_device(("A", A), ("W", W))
    cfg = _pick_config(_lib.FORM_FUSED_SWIGLU, config, M, N, K)
    cfg_c = cfg.to_c() if cfg is not None else None
    arr = (C.c_void_p * len(dst_ptrs))(*[int(p) for p in dst_ptrs])
    lib = _lib.load()
    with _on_device(dev):
        rc = lib.sgl_matmul_fused_swiglu_multi_dst(
            A.data_ptr(), W.data_ptr(), arr, len(dst_ptrs), M, N, K, _ld(A), _ld(W), int(ldh),
            int(up_col0), int(gate_col0), C.byref(cfg_c) if cfg_c is not None else None,
            _stream_handle(stream, dev))
    _lib.check(rc)


def matmul_fused_swiglu_gather(A, W, local_ptr: int, peer_ptrs, ldh: int, *, up_col0: int,
                               gate_col0: int, n_out: int, multicast_ptr: int | None = None,
                               stream=None, config: TileConfig | None = None):
    """Fused SwiGLU whose epilogue also hands every finished tile to other GPUs with ordinary
    stores (``peer_ptrs``: element (0, 0) of this launch's block in each peer's buffer), or,
    given ``multicast_ptr`` (that element in an NVSwitch multicast mapping of all the buffers),
    with one ``multimem.st`` per 16 bytes that the switch replicates to every member.
    ``local_ptr`` is the element in this GPU's own buffer.  The caller owns the buffers and the
    cross-rank synchronisation (``sharding.fused_swiglu_n_sharded_fused_gather`` does both)."""
    _check_matrix(A, "A")
    _check_matrix(W, "W")
    M, K = A.shape
    if W.shape[0] != K:
        raise ValueError(f"K mismatch: A.K={K} vs W.K={W.shape[0]}")
    N = int(n_out)
    if N < 1 or up_col0 < 0 or gate_col0 < 0 or max(up_col0, gate_col0) + N > W.shape[1]:
        raise ValueError("column windows outside W")
    if len(peer_ptrs) > 8:
        raise ValueError(f"at most 8 peer destinations, got {len(peer_ptrs)}")
    dev = _same_device(("A", A), ("W", W))
    cfg = _pick_config(_lib.FORM_FUSED_SWIGLU, config, M, N, K)
    cfg_c = cfg.to_c() if cfg is not None else None
    arr = (C.c_void_p * max(1, len(peer_ptrs)))(*[int(p) for p in peer_ptrs])
    with _on_device(dev):
        rc = _lib.load().sgl_matmul_fused_swiglu_gather(
            A.data_ptr(), W.data_ptr(), int(local_ptr), arr, len(peer_ptrs),
            int(multicast_ptr) if multicast_ptr else None, M, N, K, _ld(A), _ld(W), int(ldh),
            int(up_col0), int(gate_col0), C.byref(cfg_c) if cfg_c is not None else None,
            _stream_handle(stream, dev))
    _lib.check(rc)


def matmul_fused_swiglu_save_factors(A, W, *, out=None, factors=None, stream=None,
                                     config: TileConfig | None = None):
    """Training forward: returns ``(h, factors)`` with ``h`` as ``matmul_fused_swiglu`` and
    ``factors[M, 2N] = [silu(gate) | up * silu'(gate)]`` written by the same epilogue
    (reference: the Triton side-store forward, ``swiglu/triton/impls.py:384-468``)."""
    _check_matrix(A, "A")
    _check_matrix(W, "W")
    M, K = A.shape
    K2, N2 = W.shape
    if K != K2:
        raise ValueError(f"K mismatch: A.K={K} vs W.K={K2}")
    if N2 % 2:
        raise ValueError(f"W's 2nd dim ({N2}) must be even")
    N = N2 // 2
    if K % 8 or N % 8:
        raise ValueError(f"K={K} and N={N} must be multiples of 8")
    dev = _same_device(("A", A), ("W", W))
    h = _prep_out(out, M, N, dev)
    f = _prep_out(factors, M, 2 * N, dev, "factors")
    cfg = _pick_config(_lib.FORM_FUSED_SWIGLU_SAVE, config, M, N, K)
    cfg_c = cfg.to_c() if cfg is not None else None
    with _on_device(dev):
        rc = _lib.load().sgl_matmul_fused_swiglu_save_factors(
            A.data_ptr(), W.data_ptr(), h.data_ptr(), f.data_ptr(), M, N, K, _ld(A), _ld(W),
            _ld(h), _ld(f), 0, N, C.byref(cfg_c) if cfg_c is not None else None,
            _stream_handle(stream, dev))
    _lib.check(rc)
    return h, f


def swiglu_grad_preact(dy, factors, *, out=None, stream=None):
    """Backward elementwise step: ``[dy * factors[:, :N] | dy * factors[:, N:]]`` =
    ``[d/d(up) | d/d(gate)]``.  ``out=factors`` computes in place.  (Reference:
    ``_swiglu_grad_preact_normal_kernel``, ``swiglu/triton/impls.py:3947-3993``.)"""
    _check_matrix(dy, "dy")
    _check_matrix(factors, "factors")
    M, N = dy.shape
    if tuple(factors.shape) != (M, 2 * N):
        raise ValueError(f"factors shape {tuple(factors.shape)} != {(M, 2 * N)}")
    if N % 8:
        raise ValueError(f"N={N} must be a multiple of 8")
    dev = _same_device(("dy", dy), ("factors", factors))
    o = _prep_out(out, M, 2 * N, dev)
    with _on_device(dev):
        rc = _lib.load().sgl_swiglu_grad_preact(dy.data_ptr(), factors.data_ptr(), o.data_ptr(), M,
                                                N, _ld(dy), _ld(factors), _ld(o),
                                                _stream_handle(stream, dev))
    _lib.check(rc)
    return o


def matmul_bf16(A, B, *, out=None, stream=None, config: TileConfig | None = None,
                transpose_a: bool = False, transpose_b: bool = False):
    """``op(A) @ op(B)`` (bf16 in, fp32 accumulate, bf16 out) on the same TMA/tcgen05
    pipeline: the down projection ``y = h @ W_down`` that consumes the stage's output, and
    with the transpose flags the two GEMMs of the backward pass.

    A : [M, K] bf16, or [K, M] with ``transpose_a`` (read in place, no transpose copy)
    B : [K, N] bf16, or [N, K] with ``transpose_b``
    returns [M, N] bf16.

    Without ``config`` and transposes, problems of up to 256 rows and K >= 4096 (a down
    projection at decode batch sizes) are cut along K into ranges that run as thread-block
    clusters and sum themselves through distributed shared memory when that occupies clearly
    more SMs; the result is deterministic and differs from whole-K tiles only in the order of
    the fp32 additions (``_lib.set_splitk_cluster_sum(False)`` keeps whole-K tiles).
    """
    _check_matrix(A, "A", allow_empty_rows=not transpose_a)
    _check_matrix(B, "B")
    M, K = (A.shape[1], A.shape[0]) if transpose_a else A.shape
    K2, N = (B.shape[1], B.shape[0]) if transpose_b else B.shape
    if K2 != K:
        raise ValueError(f"K mismatch: op(A).K={K} vs op(B).K={K2}")
    # K is a contiguous extent (16-byte rows) unless both operands are stored [K, *], where it
    # only counts rows: the weight gradient x^T @ g then takes any token count.
    k_is_row_count = transpose_a and not transpose_b
    if (K % 8 and not k_is_row_count) or N % 8 or (transpose_a and M % 8):
        raise ValueError(f"K={K}, N={N} (and M={M} when A is transposed) must be multiples of 8")
    dev = _same_device(("A", A), ("B", B))
    if M == 0:
        return out if out is not None else torch.empty((0, N), dtype=DTYPE, device=dev)
    c = _prep_out(out, M, N, dev)
    cfg = _pick_config(_lib.FORM_MATMUL, config, M, N, K)
    cfg_c = cfg.to_c() if cfg is not None else None
    with _on_device(dev):
        rc = _lib.load().sgl_matmul_bf16_ex(
            A.data_ptr(), B.data_ptr(), c.data_ptr(), M, N, K, _ld(A), _ld(B), _ld(c),
            int(transpose_a), int(transpose_b), C.byref(cfg_c) if cfg_c is not None else None,
            _stream_handle(stream, dev))
    _lib.check(rc)
    return c


def splitk_scratch_bytes(M: int, N: int, K: int, splits: int = 0) -> int:
    """Bytes of device scratch ``matmul_bf16_splitk`` needs for this problem."""
    n = _lib.load().sgl_matmul_bf16_splitk_scratch_bytes(M, N, K, splits)
    if n < 0:
        _lib.check(int(n))
    return int(n)


def matmul_bf16_splitk(A, B, *, out=None, splits: int = 0, scratch=None, stream=None,
                       config: TileConfig | None = None):
    """``A @ B`` with K cut into ``splits`` ranges (0 = choose) - for short, deep problems
    such as the down projection at decode batch sizes, where one tile per CTA pair would
    leave most SMs idle.  Partial tiles go to ``scratch`` in fp32 and are then summed in fp32,
    in order.  ``scratch`` is a caller-owned uint8 CUDA tensor of at least
    ``splitk_scratch_bytes(M, N, K, splits)`` bytes (allocated here if omitted)."""
    _check_matrix(A, "A")
    _check_matrix(B, "B")
    M, K = A.shape
    K2, N = B.shape
    if K2 != K:
        raise ValueError(f"K mismatch: A.K={K} vs B.K={K2}")
    if K % 8 or N % 8:
        raise ValueError(f"K={K} and N={N} must be multiples of 8")
    dev = _same_device(("A", A), ("B", B))
    c = _prep_out(out, M, N, dev)
    need = splitk_scratch_bytes(M, N, K, splits)
    if scratch is None:
        # allocate on the launch stream: the caching allocator then hands the block to somebody
        # else only after the kernels queued on that stream have run
        with stream_context(stream, dev):
            scratch = torch.empty(need, dtype=torch.uint8, device=dev)
    if scratch.dtype != torch.uint8 or not scratch.is_cuda or scratch.device != dev \
            or not scratch.is_contiguous():
        raise ValueError("scratch must be a contiguous uint8 CUDA tensor on the operands' device")
    cfg = _pick_config(_lib.FORM_MATMUL, config, M, N, K)
    cfg_c = cfg.to_c() if cfg is not None else None
    with _on_device(dev):
        rc = _lib.load().sgl_matmul_bf16_splitk(
            A.data_ptr(), B.data_ptr(), c.data_ptr(), M, N, K, _ld(A), _ld(B), _ld(c), int(splits),
            scratch.data_ptr(), scratch.numel(), C.byref(cfg_c) if cfg_c is not None else None,
            _stream_handle(stream, dev))
    _lib.check(rc)
    return c


def matmul_bf16_reduce_scatter(A, B, dst_ptrs, rows_per_dst: int, ldc: int, *, dst_f32: bool,
                               accumulate: bool = True, first_dst: int = 0, stream=None,
                               config: TileConfig | None = None):
    """Sends ``A @ B`` to the row-block owners' buffers (GEMM + scatter in one kernel).

    ``dst_ptrs[d]`` is the device address of the ``[rows_per_dst, N]`` buffer (fp32 if
    ``dst_f32`` else bf16, row pitch ``ldc`` elements) on the rank that owns rows
    ``[d * rows_per_dst, (d+1) * rows_per_dst)``; peers' buffers are addressed through their
    mapping in this process.  ``accumulate=True`` adds into a buffer shared by all ranks (the
    caller zeroes it first); ``accumulate=False`` overwrites - the buffer is then this rank's
    private slot on the owner, summed afterwards with ``sum_bf16_slots``.  ``first_dst``
    rotates the tile order so it starts with that owner's rows (ranks pass different values
    to spread the traffic).  The caller synchronises the ranks.
    """
    _check_matrix(A, "A")
    _check_matrix(B, "B")
    M, K = A.shape
    K2, N = B.shape
    if K2 != K:
        raise ValueError(f"K mismatch: A.K={K} vs B.K={K2}")
    if not 1 <= len(dst_ptrs) <= 8:
        raise ValueError(f"need 1..8 destinations, got {len(dst_ptrs)}")
    dev = _same_device(("A", A), ("B", B))
    cfg = _pick_config(_lib.FORM_MATMUL, config, M, N, K)
    cfg_c = cfg.to_c() if cfg is not None else None
    arr = (C.c_void_p * len(dst_ptrs))(*[int(p) for p in dst_ptrs])
    with _on_device(dev):
        rc = _lib.load().sgl_matmul_bf16_reduce_scatter(
            A.data_ptr(), B.data_ptr(), arr, len(dst_ptrs), int(rows_per_dst), int(bool(dst_f32)),
            int(bool(accumulate)), int(first_dst), M, N, K, _ld(A), _ld(B), int(ldc), C.byref(cfg_c) if cfg_c is not None else None,
            _stream_handle(stream, dev))
    _lib.check(rc)


def sum_bf16_slots(slots, out=None, *, rows: int | None = None, stream=None):
    """``out[r, c] = bf16(sum_s slots[s, r, c])`` with fp32 accumulation in slot order.
    ``slots`` is ``[n_slots, R, C]`` bf16 (contiguous); ``rows`` limits the sum to the first
    rows of every slot."""
    if slots.dim() != 3 or slots.dtype != DTYPE or not slots.is_cuda or not slots.is_contiguous():
        raise ValueError("slots must be a contiguous [n_slots, rows, cols] bf16 CUDA tensor")
    n, R, Ccols = slots.shape
    r = R if rows is None else int(rows)
    if not 0 <= r <= R:
        raise ValueError(f"rows={r} outside [0, {R}]")
    if Ccols % 8:
        raise ValueError(f"cols={Ccols} must be a multiple of 8")
    dev = slots.device
    if r == 0:
        return out if out is not None else torch.empty((0, Ccols), dtype=DTYPE, device=dev)
    o = _prep_out(out, r, Ccols, dev)
    with _on_device(dev):
        rc = _lib.load().sgl_sum_bf16_slots(slots.data_ptr(), n, R * Ccols, o.data_ptr(), r, Ccols,
                                            Ccols, _ld(o), _stream_handle(stream, dev))
    _lib.check(rc)
    return o


def tune_matmul_silu_mul(A, B_gate, up, *, verbose=False, persist=False) -> TileConfig:
    """Sweep the tile table for this problem (reference: ``_tune``,
    ``swiglu/matmul_silu_mul.py:114-139``) and remember the winner."""
    M, K = A.shape
    N = B_gate.shape[1]
    out = torch.empty((M, N), dtype=DTYPE, device=A.device)
    return tile_table.autotune(
        _lib.FORM_SILU_MUL, lambda cfg: matmul_silu_mul(A, B_gate, up, out=out, config=cfg),
        M, N, K, verbose=verbose, persist=persist)


def tune_matmul_fused_swiglu(A, W, *, verbose=False, persist=False) -> TileConfig:
    """Sweep the tile table for this problem (reference: ``_tune``,
    ``swiglu/matmul_fused_swiglu.py:122-149``) and remember the winner."""
    M, K = A.shape
    N = W.shape[1] // 2
    out = torch.empty((M, N), dtype=DTYPE, device=A.device)
    return tile_table.autotune(
        _lib.FORM_FUSED_SWIGLU, lambda cfg: matmul_fused_swiglu(A, W, out=out, config=cfg),
        M, N, K, verbose=verbose, persist=persist)
