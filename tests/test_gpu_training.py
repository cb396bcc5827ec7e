"""Side-store forward, backward elementwise kernel and the autograd wiring, against fp32
torch expressions (``swiglu_oracle.swiglu_factors_f32`` / ``grad_preact_f32``)."""
import pytest
import torch

import swiglu_oracle as orc
from swiglu_fused_b200 import TileConfig, _lib, matmul_bf16, matmul_fused_swiglu
from swiglu_fused_b200.autograd import fused_swiglu
from swiglu_fused_b200.ops import matmul_fused_swiglu_save_factors, swiglu_grad_preact
from swiglu_fused_b200.workloads import make_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(autouse=True)
def _device_status_clean():
    yield
    torch.cuda.synchronize()
    _lib.device_status()


@pytest.mark.parametrize("M,K,N", [(256, 128, 256), (512, 1024, 2048), (200, 136, 264),
                                    (1024, 512, 384), (64, 256, 128), (1, 8, 8)])
def test_save_factors_forward(M, K, N):
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=M + K)
    x, w = inp["x"].to(DEV), inp["w"].to(DEV)
    h32, f32 = orc.swiglu_factors_f32(inp["x"], inp["w"])
    plain = matmul_fused_swiglu(x, w)
    for cg, bk in [(1, 64), (1, 128), (2, 64), (2, 128)]:
        hbuf = torch.full((M + 2, N + 16), float("nan"), dtype=torch.bfloat16, device=DEV)
        fbuf = torch.full((M + 2, 2 * N + 16), float("nan"), dtype=torch.bfloat16, device=DEV)
        h, f = matmul_fused_swiglu_save_factors(x, w, out=hbuf[1:M + 1, 8:8 + N],
                                                factors=fbuf[1:M + 1, 8:8 + 2 * N],
                                                config=TileConfig(cg, bk, 0, 8))
        # h is the same computation as the plain fused kernel
        assert torch.equal(h.contiguous().view(torch.int16), plain.view(torch.int16)), (cg, bk)
        rep_s = orc.compare(f[:, :N].contiguous().cpu(), f32[:, :N].to(torch.bfloat16).contiguous(),
                            f32[:, :N].contiguous())
        rep_d = orc.compare(f[:, N:].contiguous().cpu(), f32[:, N:].to(torch.bfloat16).contiguous(),
                            f32[:, N:].contiguous())
        assert rep_s.ok, f"silu factor {(cg, bk)}: {rep_s}"
        assert rep_d.ok, f"gate factor {(cg, bk)}: {rep_d}"
        for buf, r, c in ((hbuf, M, N), (fbuf, M, 2 * N)):
            guard = buf.clone()
            guard[1:r + 1, 8:8 + c] = float("nan")
            assert torch.isnan(guard).all(), "wrote outside the outputs"


@pytest.mark.parametrize("M,N", [(128, 128), (300, 264), (1024, 2048), (1, 8)])
def test_grad_preact_kernel(M, N):
    g = torch.Generator().manual_seed(M + N)
    dy = torch.randn((M, N), generator=g).to(torch.bfloat16)
    factors = torch.randn((M, 2 * N), generator=g).to(torch.bfloat16)
    ref32 = orc.grad_preact_f32(dy, factors)
    got = swiglu_grad_preact(dy.to(DEV), factors.to(DEV))
    # one fp32 multiply rounded once: bit exact
    assert torch.equal(got.cpu().view(torch.int16), ref32.to(torch.bfloat16).view(torch.int16))
    fd = factors.to(DEV)
    same = swiglu_grad_preact(dy.to(DEV), fd, out=fd)       # in place
    assert same is fd and torch.equal(fd.view(torch.int16), got.view(torch.int16))


def test_autograd_matches_fp32_autograd():
    M, K, N = 512, 256, 384
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=5)
    x = inp["x"].to(DEV).requires_grad_(True)
    w = inp["w"].to(DEV).requires_grad_(True)
    gen = torch.Generator().manual_seed(6)
    dy = torch.randn((M, N), generator=gen).to(torch.bfloat16).to(DEV)
    h = fused_swiglu(x, w)
    h.backward(dy)
    xf = inp["x"].float().to(DEV).requires_grad_(True)
    wf = inp["w"].float().to(DEV).requires_grad_(True)
    gu = xf @ wf
    ref = torch.nn.functional.silu(gu[:, N:]) * gu[:, :N]
    ref.backward(dy.float())
    for got, want, name in ((x.grad, xf.grad, "grad_x"), (w.grad, wf.grad, "grad_w")):
        err = (got.float() - want).abs().max().item()
        scale = want.abs().max().item()
        assert err <= 2e-2 * scale, f"{name}: max err {err} vs scale {scale}"


def test_autograd_with_a_ragged_token_count():
    """M = 200 tokens: the weight gradient x^T @ grad_preact has K = 200, which only counts
    rows of both operands and need not be a multiple of 8."""
    M, K, N = 200, 256, 384
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=15)
    x = inp["x"].to(DEV).requires_grad_(True)
    w = inp["w"].to(DEV).requires_grad_(True)
    gen = torch.Generator().manual_seed(16)
    dy = torch.randn((M, N), generator=gen).to(torch.bfloat16).to(DEV)
    fused_swiglu(x, w).backward(dy)
    torch.cuda.synchronize()
    _lib.device_status()
    xf = inp["x"].float().to(DEV).requires_grad_(True)
    wf = inp["w"].float().to(DEV).requires_grad_(True)
    gu = xf @ wf
    (torch.nn.functional.silu(gu[:, N:]) * gu[:, :N]).backward(dy.float())
    for got, want, name in ((x.grad, xf.grad, "grad_x"), (w.grad, wf.grad, "grad_w")):
        err = (got.float() - want).abs().max().item()
        scale = want.abs().max().item()
        assert err <= 2e-2 * scale, f"{name}: max err {err} vs scale {scale}"
    # and an odd row count straight through the GEMM entry point
    a = torch.randn((203, 264), generator=gen).to(torch.bfloat16).to(DEV)     # stored [K, M]
    b = torch.randn((203, 136), generator=gen).to(torch.bfloat16).to(DEV)     # stored [K, N]
    got = matmul_bf16(a, b, transpose_a=True)
    ref32 = a.float().t() @ b.float()
    assert orc.compare(got.cpu(), ref32.to(torch.bfloat16).cpu(), ref32.cpu()).ok
    with pytest.raises(ValueError):           # every other layout keeps the 16-byte rule
        matmul_bf16(a.t().contiguous(), b)


def test_second_backward_over_one_forward_is_refused():
    """The backward overwrites the saved factors in place; a second pass over the same graph
    would use factors that already hold dy, so it raises instead of returning wrong numbers."""
    M, K, N = 256, 128, 256
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=25)
    x = inp["x"].to(DEV).requires_grad_(True)
    w = inp["w"].to(DEV).requires_grad_(True)
    dy = torch.ones((M, N), dtype=torch.bfloat16, device=DEV)
    h = fused_swiglu(x, w)
    h.backward(dy, retain_graph=True)
    first = x.grad.clone()
    with pytest.raises(RuntimeError, match="ran twice"):
        h.backward(dy)
    assert torch.equal(x.grad.view(torch.int16), first.view(torch.int16))
    # a fresh forward is fine
    x.grad = None
    fused_swiglu(x, w).backward(dy)
    assert torch.equal(x.grad.view(torch.int16), first.view(torch.int16))


def test_module_forward_and_training_step():
    """``PackedSwiGLULinear`` (reference: ``swiglu/triton/impls.py:3372-3596``): loads an
    ``nn.Linear`` checkpoint, the inference forward equals the operator bit for bit, and one
    SGD step moves the parameters as the fp32 torch model does."""
    from swiglu_fused_b200.module import PackedSwiGLULinear

    torch.manual_seed(7)
    B, S, K, N = 4, 96, 256, 384
    lin = torch.nn.Linear(K, 2 * N, bias=False, dtype=torch.bfloat16)
    mod = PackedSwiGLULinear.from_linear(lin).to(DEV)
    x = torch.randn((B, S, K)).to(torch.bfloat16).to(DEV)
    with torch.no_grad():
        y = mod(x)
    assert tuple(y.shape) == (B, S, N)
    want = matmul_fused_swiglu(x.reshape(-1, K), mod.weight.detach())
    assert torch.equal(y.reshape(-1, N).view(torch.int16), want.view(torch.int16))
    ref32 = orc.fused_swiglu_f32(x.reshape(-1, K).cpu(), lin.weight.detach().t().contiguous())
    assert orc.compare(want.cpu(), ref32.to(torch.bfloat16), ref32).ok

    # training forward (side-store kernel) gives the same h; the backward reaches the parameter
    x.requires_grad_(True)
    y2 = mod(x)
    assert torch.equal(y2.detach().view(torch.int16), y.view(torch.int16))
    dy = torch.randn((B, S, N)).to(torch.bfloat16).to(DEV)
    y2.backward(dy)
    wf = lin.weight.detach().float().t().contiguous().to(DEV).requires_grad_(True)   # [K, 2N]
    xf = x.detach().float().reshape(-1, K).requires_grad_(True)
    gu = xf @ wf
    (torch.nn.functional.silu(gu[:, N:]) * gu[:, :N]).backward(dy.float().reshape(-1, N))
    for got, ref, name in ((x.grad.reshape(-1, K), xf.grad, "grad_x"),
                           (mod.weight.grad, wf.grad, "grad_w")):
        err = (got.float() - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item(), name
    # the state dict after the step is still in the nn.Linear layout
    opt = torch.optim.SGD(mod.parameters(), lr=1e-2)
    opt.step()
    sd = mod.state_dict()
    assert tuple(sd["weight"].shape) == (2 * N, K)
    assert not torch.equal(sd["weight"].cpu(), lin.weight.detach())
