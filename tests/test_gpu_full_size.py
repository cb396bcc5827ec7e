"""Full-size configurations (c3, c4, the c5 per-GPU column shard) checked through properties
that do not need a full CPU result: sampled rows against the oracle, exact linearity in
W_up, and row-permutation equivariance.  Inputs are generated on the GPU (seeded)."""
import pytest
import torch

import swiglu_oracle as orc
from swiglu_fused_b200 import _lib, matmul_fused_swiglu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

CASES = {
    # name: (M, K, N_total, w_std, (c0, n_out) column window or None)
    "c3": (32768, 3072, 12288, None, None),
    "c4": (16384, 4096, 14336, 0.02, None),
    "c5_shard3of8": (32768, 8192, 28672, 0.02, (3 * 3584, 3584)),
}


def bits(t):
    return t.contiguous().view(torch.int16)


@pytest.mark.parametrize("name", list(CASES))
def test_full_size_properties(name):
    M, K, N, std, window = CASES[name]
    g = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn((M, K), device=DEV, dtype=torch.bfloat16, generator=g)
    w = torch.empty((K, 2 * N), device=DEV, dtype=torch.bfloat16)
    w.normal_(0.0, std if std is not None else K ** -0.5, generator=g)
    if window is None:
        kw, c0, n = {}, 0, N
    else:
        c0, n = window
        kw = dict(up_col0=c0, gate_col0=N + c0, n_out=n)
    h = matmul_fused_swiglu(x, w, **kw)
    torch.cuda.synchronize()
    _lib.device_status()
    assert h.shape == (M, n) and bool(torch.isfinite(h.float()).all())

    # 1. sampled rows against the CPU oracle
    rows = torch.randint(0, M, (48,), generator=torch.Generator().manual_seed(1))
    rows = torch.cat([rows, torch.tensor([0, M - 1])])
    xs = x[rows.to(DEV)].cpu()
    w_up = w[:, c0:c0 + n].cpu()
    w_gate = w[:, N + c0:N + c0 + n].cpu()
    ref32 = torch.nn.functional.silu(xs.float() @ w_gate.float()) * (xs.float() @ w_up.float())
    rep = orc.compare(h[rows.to(DEV)].cpu(), ref32.to(torch.bfloat16), ref32, k_depth=K)
    assert rep.ok, f"{name}: {rep}"

    # 2. rows are independent: computing a row block alone gives the same bits
    r0, r1 = M // 2 - 256, M // 2 + 512
    part = matmul_fused_swiglu(x[r0:r1], w, **kw)
    assert torch.equal(bits(part), bits(h[r0:r1]))

    # 3. exact linearity in W_up: doubling W_up (exact in bf16) doubles h bit for bit
    w2 = w.clone()
    w2[:, c0:c0 + n] *= 2
    h2 = matmul_fused_swiglu(x[:4096], w2, **kw)
    want = (h[:4096].float() * 2).to(torch.bfloat16)
    big = h[:4096].float().abs() > 2.0 ** -100          # doubling is exact away from underflow
    assert torch.equal(bits(h2)[big], bits(want)[big])

    # 4. permuting the rows of x permutes the rows of h
    perm = torch.randperm(2048, generator=torch.Generator().manual_seed(2)).to(DEV)
    hp = matmul_fused_swiglu(x[:2048][perm].contiguous(), w, **kw)
    assert torch.equal(bits(hp), bits(h[:2048][perm]))
    torch.cuda.synchronize()
    _lib.device_status()


@pytest.mark.parametrize("M", [64, 256, 1024])
def test_c4_tile_tail_shapes_against_the_oracle(M):
    """Configuration 4's tile tail at its own K and N (M in {64, 256, 1024}, K = 4096,
    N = 14336, weights N(0, 0.02)): rows against the fp32 CPU oracle (all of them for M = 64,
    a spread of 64 otherwise, the first and the last included), and the tail result must be a
    bit-exact slice of the same rows computed inside a taller problem (a different tile
    schedule, the same per-element arithmetic).  The reference rejects M = 64
    (swiglu/matmul_silu_mul.py:101-111)."""
    K, N = 4096, 14336
    g = torch.Generator(device=DEV).manual_seed(4)
    x = torch.randn((2048, K), device=DEV, dtype=torch.bfloat16, generator=g)
    w = torch.empty((K, 2 * N), device=DEV, dtype=torch.bfloat16).normal_(0.0, 0.02, generator=g)
    h = matmul_fused_swiglu(x[:M], w)
    torch.cuda.synchronize()
    _lib.device_status()
    assert h.shape == (M, N) and bool(torch.isfinite(h.float()).all())
    rows = torch.arange(M) if M <= 64 else torch.unique(torch.linspace(0, M - 1, 64).long())
    xs = x[rows.to(DEV)].cpu()
    # K = 4096: against the float64 value (the fp32 check expression has accumulation error
    # of its own on near-zero outputs at this depth; it must itself sit within the tolerance)
    ref64 = orc.fused_swiglu_exact(xs, w.cpu())
    rep = orc.compare(h[rows.to(DEV)].cpu(), ref64.to(torch.bfloat16), ref64, k_depth=K)
    assert rep.ok, f"M={M}: {rep}"
    tall = matmul_fused_swiglu(x, w)
    assert torch.equal(bits(tall[:M]), bits(h))
    # guard band: an output buffer with extra rows and columns keeps its sentinel
    buf = torch.full((M + 32, N + 64), float("nan"), dtype=torch.bfloat16, device=DEV)
    matmul_fused_swiglu(x[:M], w, out=buf[:M, :N])
    assert torch.equal(bits(buf[:M, :N]), bits(h))
    assert bool(torch.isnan(buf[M:].float()).all()) and bool(torch.isnan(buf[:, N:].float()).all())
    torch.cuda.synchronize()
    _lib.device_status()
