"""Cycle accounting of the kernel's roles (developer tool).

    python -m swiglu_fused_b200.role_cycles [--form fused_swiglu|fused_swiglu_save|silu_mul] [--rows M]
                                            [--block-k 64|128] [--group-m G] [--timeline] [--auto]
    torchrun --nproc-per-node W -m swiglu_fused_b200.role_cycles --k 8192 --cols 28672 \
             --gather none|tma|stores|multicast      # column-parallel over W GPUs, rank 0 reports

Builds a second copy of the library with ``-DSGL_PROFILE`` (``libswiglu_b200_prof.so``, next to
the normal one), in which every role of ``swiglu_kernel`` adds up, per CTA, the SM cycles it
spends waiting: the MMA issuer for a free accumulator and for operands, the TMA producer for a
free ring slot, the epilogue for an accumulator and for ``up``.  Prints the averages as a share
of the MMA loop, the cycles per 64-wide k-block against the 512-cycle tensor-core ideal, and the
spread between the fastest and the slowest CTA pair (what a dynamic tile scheduler could gain).
``--timeline`` prints instead when, after the launch reached the GPU, a CTA passed eight points
of its life (set-up done, first operands landed, last MMA committed, stores read, ...), which
is how the fixed cost of a short launch splits up.  The normal library carries none of this code.
"""
from __future__ import annotations

import argparse
import ctypes as C
import os
import subprocess

from . import build as _build

PROF_LIB = os.path.join(_build.PKG_DIR, "libswiglu_b200_prof.so")


def build_profile_library() -> str:
    srcs = _build.SOURCES + _build.HEADERS
    if os.path.exists(PROF_LIB) and all(os.path.getmtime(p) <= os.path.getmtime(PROF_LIB)
                                        for p in srcs if os.path.exists(p)):
        return PROF_LIB
    cmd = [_build.find_nvcc(), *_build.NVCC_FLAGS, "-DSGL_PROFILE", "-o", PROF_LIB,
           *_build.SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{proc.stderr}")
    return PROF_LIB


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--form", choices=("fused_swiglu", "fused_swiglu_save", "silu_mul", "grad_x", "grad_w",
                             "down", "down_splitk"),
                    default="fused_swiglu",
                    help="grad_x / grad_w: the backward GEMMs g @ W^T and x^T @ g of the same "
                         "problem (GEMM form, transposed operand read in place); down / "
                         "down_splitk: the plain product [rows, k] @ [k, cols], unsplit or with "
                         "K cut into ranges (then the cycles are those of the GEMM launch; the "
                         "time also covers the slot sum)")
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--k", type=int, default=3072)
    ap.add_argument("--n", "--cols", dest="n", type=int, default=12288)
    ap.add_argument("--block-k", type=int, default=0, help="0 = the default configuration")
    ap.add_argument("--group-m", type=int, default=0)
    ap.add_argument("--auto", action="store_true",
                    help="pass no configuration: the library chooses, which for short, deep "
                         "problems means K ranges summed in thread-block clusters (read the "
                         "timeline then; the per-k-block figures assume whole-K tiles)")
    ap.add_argument("--timeline", action="store_true",
                    help="also print where a CTA's time goes outside the K loop (set-up, first "
                         "operands, epilogue, teardown): %%globaltimer stamps of the last launch")
    ap.add_argument("--gather", choices=("none", "tma", "stores", "multicast"), default=None,
                    help="column-parallel launch over the ranks of a torchrun group: each rank "
                         "computes N / world columns; 'none' keeps them local, the others "
                         "gather h into every rank inside the kernel by that mode")
    args = ap.parse_args()

    os.environ["SWIGLU_B200_LIB"] = build_profile_library()
    import numpy as np
    import torch

    from . import _lib
    from .ops import (matmul_bf16, matmul_fused_swiglu, matmul_fused_swiglu_save_factors,
                      matmul_silu_mul)

    rank, world, sym = 0, 1, None
    dev = torch.device("cuda:0")
    if args.gather is not None:
        from . import sharding
        rank, world, local_rank = sharding.init_from_env("nccl")
        dev = torch.device("cuda", local_rank)
        torch.cuda.set_device(dev)
    M, K, N = args.rows, args.k, args.n
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn((M, K), device=dev, dtype=torch.bfloat16, generator=g)
    w = torch.empty((K, 2 * N), device=dev, dtype=torch.bfloat16).normal_(0, K ** -0.5, generator=g)
    out = torch.empty((M, N), device=dev, dtype=torch.bfloat16)
    form = {"fused_swiglu": _lib.FORM_FUSED_SWIGLU, "fused_swiglu_save": _lib.FORM_FUSED_SWIGLU_SAVE,
            "silu_mul": _lib.FORM_SILU_MUL}.get(args.form, _lib.FORM_MATMUL)
    depth = K                               # contraction depth of the launch that is profiled
    cfg = _lib.default_config(form, M, N, K)
    if args.form in ("down", "down_splitk"):
        w = w[:, :N]                        # [K, N], row pitch 2N
    if args.form == "grad_x":               # [M, 2N] @ [2N, K]
        depth, cfg = 2 * N, _lib.default_config(form, M, K, 2 * N)
    elif args.form == "grad_w":             # [K, M] @ [M, 2N]
        depth, cfg = M, _lib.default_config(form, K, 2 * N, M)
    if args.block_k or args.group_m:
        cfg = _lib.TileConfig(cfg.cta_group, args.block_k or cfg.block_k, 0,
                              args.group_m or cfg.group_m)
    if args.gather is not None:
        import torch.distributed as dist
        cols = sharding.col_shard(N, world, rank)
        cfg = _lib.default_config(form, M, cols.count, K)
        if args.gather == "none":
            local = torch.empty((M, cols.count), device=dev, dtype=torch.bfloat16)

            def run():
                sharding.fused_swiglu_n_sharded(x, w, rank=rank, world=world, out=local, config=cfg)
        else:
            sym = sharding.SymmetricOutput(M, N, dev, multicast=args.gather == "multicast")

            def run():
                sharding.fused_swiglu_n_sharded_fused_gather(x, w, sym, mode=args.gather, config=cfg)
    elif args.form == "fused_swiglu":
        def run():
            matmul_fused_swiglu(x, w, out=out, config=None if args.auto else cfg)
    elif args.form == "down":
        def run():
            matmul_bf16(x, w, out=out, config=None if args.auto else cfg)
    elif args.form == "down_splitk":
        from .ops import matmul_bf16_splitk, splitk_scratch_bytes
        scratch = torch.empty(splitk_scratch_bytes(M, N, K), dtype=torch.uint8, device=dev)

        def run():
            matmul_bf16_splitk(x, w, out=out, scratch=scratch, config=cfg)
    elif args.form in ("grad_x", "grad_w"):
        gp = torch.randn((M, 2 * N), device=dev, dtype=torch.bfloat16, generator=g)
        grad = torch.empty((M, K) if args.form == "grad_x" else (K, 2 * N), device=dev,
                           dtype=torch.bfloat16)
        if args.form == "grad_x":
            def run():
                matmul_bf16(gp, w, transpose_b=True, out=grad, config=cfg)
        else:
            def run():
                matmul_bf16(x, gp, transpose_a=True, out=grad, config=cfg)
    elif args.form == "fused_swiglu_save":
        factors = torch.empty((M, 2 * N), device=dev, dtype=torch.bfloat16)

        def run():
            matmul_fused_swiglu_save_factors(x, w, out=out, factors=factors, config=cfg)
    else:
        w_gate = w[:, N:].contiguous()
        up = x @ w[:, :N].contiguous()

        def run():
            matmul_silu_mul(x, w_gate, up, out=out, config=cfg)

    lib = _lib.load()
    lib.sgl_debug_profile.restype = C.c_int
    lib.sgl_debug_profile.argtypes = [C.POINTER(C.c_ulonglong)]
    for _ in range(20):
        run()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    run()
    t1.record()
    torch.cuda.synchronize()
    buf = (C.c_ulonglong * (512 * 8))()
    _lib.check(lib.sgl_debug_profile(buf))
    n_ctas = min(512, _lib.query(_lib.QUERY_SM_COUNT))
    p = np.frombuffer(buf, dtype=np.uint64).reshape(512, 8)[:n_ctas].astype(np.float64)
    lead = p[0::cfg.cta_group]              # the MMA issuer runs in the leader CTA of a pair
    lead = lead[lead[:, 2] > 0]             # a short problem does not occupy every SM
    p = p[p[:, 7] > 0] if (p[:, 7] > 0).any() else p
    loop = lead[:, 2]
    tiles = np.maximum(lead[:, 7], 1)
    kblocks = tiles * (-(-depth // 64))
    if rank != 0:
        dist.barrier()
        dist.destroy_process_group()
        return
    what = args.form if args.gather is None else \
        f"column-parallel x{world} (gather: {args.gather}), {N // world} columns per GPU,"
    ms = t0.elapsed_time(t1)
    print(f"{what} {M}x{K}x{N} {cfg}: {ms:.3f} ms")
    print(f"  MMA loop {loop.mean():.0f} clk per CTA = {loop.mean() / (ms * 1e3):.0f} MHz x the "
          f"launch time; {(loop / kblocks).mean():.0f} clk per 64-k block (tensor-core ideal 512)")
    print(f"  MMA issuer waits: free accumulator {100 * (lead[:, 0] / loop).mean():.1f} %, "
          f"operands {100 * (lead[:, 1] / loop).mean():.1f} %")
    print(f"  TMA producer waits for a ring slot {100 * p[:, 3].mean() / loop.mean():.1f} %")
    print(f"  epilogue: waits for an accumulator {100 * p[:, 4].mean() / loop.mean():.1f} %, "
          f"for up {100 * p[:, 5].mean() / loop.mean():.1f} %, busy "
          f"{100 * p[:, 6].mean() / loop.mean():.1f} %")
    print(f"  load balance: slowest / mean CTA = {loop.max() / loop.mean():.4f}, "
          f"tiles per CTA {int(tiles.min())}..{int(tiles.max())}")
    if args.timeline:
        lib.sgl_debug_timeline.restype = C.c_int
        lib.sgl_debug_timeline.argtypes = [C.POINTER(C.c_ulonglong)]
        tbuf = (C.c_ulonglong * (512 * 10))()
        _lib.check(lib.sgl_debug_timeline(tbuf))
        t = np.frombuffer(tbuf, dtype=np.uint64).reshape(512, 10).astype(np.int64)
        t = t[t[:, 0] > 0]                  # the CTAs of this process's launches
        t0 = t[:, 0].min()
        names = ("CTA start", "set-up done", "past the dependent-launch wait",
                 "first operands landed", "last MMA committed", "epilogue sees the accumulator",
                 "epilogue's stores have read", "teardown done")
        print("  timeline, ns after the first CTA started (mean / max over the CTAs):")
        order = list(range(8))
        if (t[:, 8] >= t0).all():           # split-K summed in thread-block clusters
            names += ("partial tile in shared memory", "all K ranges have reported")
            order = [0, 1, 2, 3, 4, 5, 8, 9, 6, 7]
        for i in order:
            print(f"    {names[i]:34s} {np.mean(t[:, i] - t0):9.0f} {np.max(t[:, i] - t0):9.0f}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
