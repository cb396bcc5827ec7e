"""Regenerates the golden fixtures in this directory.

    python tests/golden/make_golden.py

The reference ships no golden vectors, and its CUDA kernels cannot run without
a GPU and pycuda, so the fixtures pin the reference's *check expressions*
(``bench.py:39-40`` and ``bench_fused.py:39-42`` of the reference) evaluated in
float64 on seeded inputs and rounded once to bf16.  float64 makes the values
independent of the CPU's GEMM blocking, so the same files are valid on every
machine.  Small cases store inputs and outputs; the config-1 case (512x1024x2048)
stores a checksum of its seeded inputs and a strided sample of the output.
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import swiglu_oracle as orc  # noqa: E402
from swiglu_fused_b200.workloads import make_inputs  # noqa: E402

SMALL_CASES = [
    # name, form, M, K, N, seed
    ("fused_64x128x64", "fused_swiglu", 64, 128, 64, 1),
    ("fused_ragged_200x136x264", "fused_swiglu", 200, 136, 264, 2),
    ("silu_mul_64x128x64", "silu_mul", 64, 128, 64, 3),
    ("silu_mul_ragged_130x72x328", "silu_mul", 130, 72, 328, 4),
]
C1 = ("c1_512x1024x2048", 512, 1024, 2048, 0)
SAMPLE_STRIDE = 37


def u16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(u16(t).tobytes()).hexdigest()


def main() -> None:
    torch.set_num_threads(os.cpu_count() or 1)
    for name, form, M, K, N, seed in SMALL_CASES:
        inp = make_inputs(M, K, N, form=form, seed=seed)
        if form == "fused_swiglu":
            h = orc.fused_swiglu_f64(inp["x"], inp["w"])
            np.savez_compressed(os.path.join(HERE, name + ".npz"), form=form, x=u16(inp["x"]),
                                w=u16(inp["w"]), h=u16(h))
        else:
            up = (inp["x"].double() @ inp["w_up"].double()).to(torch.bfloat16)
            h = orc.silu_mul_f64(inp["x"], inp["w_gate"], up)
            np.savez_compressed(os.path.join(HERE, name + ".npz"), form=form, x=u16(inp["x"]),
                                w_gate=u16(inp["w_gate"]), up=u16(up), h=u16(h))
        print(name, "written")

    name, M, K, N, seed = C1
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=seed)
    h = orc.fused_swiglu_f64(inp["x"], inp["w"])
    # silu_mul view of the same problem: W_up = left half, W_gate = right half,
    # up = bf16(x @ W_up) is an input of that form.
    up = (inp["x"].double() @ inp["w"][:, :N].double()).to(torch.bfloat16)
    h3 = orc.silu_mul_f64(inp["x"], inp["w"][:, N:].contiguous(), up)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        x_sha256=sha(inp["x"]), w_sha256=sha(inp["w"]),
        h_fused_sample=u16(h).reshape(-1)[::SAMPLE_STRIDE],
        h_fused_sha256=sha(h),
        up_sample=u16(up).reshape(-1)[::SAMPLE_STRIDE],
        h_silu_mul_sample=u16(h3).reshape(-1)[::SAMPLE_STRIDE],
        h_silu_mul_sha256=sha(h3),
        sample_stride=SAMPLE_STRIDE, seed=seed, M=M, K=K, N=N)
    print(name, "written")


if __name__ == "__main__":
    main()
