"""Weight layout helpers (CPU) and the checkpoint-layout path of the kernel (GPU)."""
import pytest
import torch

import swiglu_oracle as orc
from swiglu_fused_b200 import weights
from swiglu_fused_b200.workloads import make_inputs


def test_pack_unpack_roundtrip_and_split():
    K, N = 48, 40
    lin = torch.arange(2 * N * K, dtype=torch.float32).reshape(2 * N, K).to(torch.bfloat16)
    packed = weights.pack_swiglu_linear_weight(lin)
    assert packed.shape == (K, 2 * N) and packed.is_contiguous()
    assert torch.equal(weights.unpack_swiglu_linear_weight(packed), lin)
    w_up, w_gate = weights.split_packed(packed)
    assert torch.equal(w_up, lin[:N].t()) and torch.equal(w_gate, lin[N:].t())
    assert torch.equal(weights.pack_gate_up(w_gate.contiguous(), w_up.contiguous()), packed)
    with pytest.raises(ValueError):
        weights.pack_swiglu_linear_weight(torch.zeros(3, 4))


def test_from_hf_llama_matches_the_packed_convention():
    N, K = 24, 16
    g = torch.Generator().manual_seed(0)
    gate_proj = torch.randn((N, K), generator=g).to(torch.bfloat16)
    up_proj = torch.randn((N, K), generator=g).to(torch.bfloat16)
    x = torch.randn((8, K), generator=g).to(torch.bfloat16)
    kn = weights.from_hf_llama(gate_proj, up_proj, "kn")
    nk = weights.from_hf_llama(gate_proj, up_proj, "nk")
    assert kn.shape == (K, 2 * N) and nk.shape == (2 * N, K)
    assert torch.equal(nk.t(), kn)
    want = torch.nn.functional.silu(x.float() @ gate_proj.float().t()) * (x.float() @ up_proj.float().t())
    assert torch.allclose(orc.fused_swiglu_f32(x, kn), want, rtol=1e-5, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,N", [(256, 128, 256), (512, 1024, 2048), (200, 136, 264),
                                    (1024, 512, 384), (64, 4096, 512), (1, 8, 8)])
def test_checkpoint_layout_equals_packed_layout(M, K, N):
    from swiglu_fused_b200 import TileConfig, _lib, matmul_fused_swiglu

    dev = "cuda:0"
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=M + N)
    x, w = inp["x"].to(dev), inp["w"].to(dev)
    w_nk = weights.unpack_swiglu_linear_weight(w)          # [2N, K], rows: up then gate
    ref32 = orc.fused_swiglu_f32(inp["x"], inp["w"])
    for cg, bk in [(1, 64), (1, 128), (2, 64), (2, 128)]:
        cfg = TileConfig(cg, bk, 0, 8)
        a = matmul_fused_swiglu(x, w, config=cfg)
        b = matmul_fused_swiglu(x, w_nk, w_layout="nk", config=cfg)
        # same products accumulated in the same order: identical results
        assert torch.equal(a.view(torch.int16), b.view(torch.int16)), (cg, bk)
        assert orc.compare(b.cpu(), ref32.to(torch.bfloat16), ref32).ok
    # row windows of the checkpoint layout = column windows of the packed layout
    if N >= 256:
        win = matmul_fused_swiglu(x, w_nk, w_layout="nk", up_col0=128, gate_col0=N + 128, n_out=128)
        assert torch.equal(win.view(torch.int16), a[:, 128:256].contiguous().view(torch.int16))
    torch.cuda.synchronize()
    _lib.device_status()
