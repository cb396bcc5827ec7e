"""``PackedSwiGLULinear`` host logic: parameter layout, ``nn.Linear``-layout state dict,
conversion from ``nn.Linear`` (reference module: ``swiglu/triton/impls.py:3372-3596``).
No kernel runs here; the forward and backward are covered by the GPU tests."""
import pytest
import torch

from swiglu_fused_b200.module import PackedSwiGLULinear


def test_parameter_is_up_then_gate_columns_and_state_dict_is_linear_layout():
    torch.manual_seed(0)
    m = PackedSwiGLULinear(64, 24, device="cpu")
    assert tuple(m.weight.shape) == (64, 48) and m.weight.dtype == torch.bfloat16
    sd = m.state_dict()
    assert list(sd) == ["weight"] and tuple(sd["weight"].shape) == (48, 64)
    assert torch.equal(sd["weight"], m.weight.detach().t())
    # rows [0, N) of the nn.Linear weight are the up features = left columns of the parameter
    assert torch.equal(sd["weight"][:24].t(), m.weight.detach()[:, :24])
    # initialisation scales: up ~ N(0, 1/K), gate ~ Kaiming (std sqrt(2/K))
    up_std = m.weight.detach()[:, :24].float().std().item()
    gate_std = m.weight.detach()[:, 24:].float().std().item()
    assert 0.8 * 64 ** -0.5 < up_std < 1.2 * 64 ** -0.5
    assert 0.8 * (2 / 64) ** 0.5 < gate_std < 1.2 * (2 / 64) ** 0.5


def test_state_dict_round_trip_and_internal_layout_is_accepted():
    torch.manual_seed(1)
    a = PackedSwiGLULinear(40, 16, device="cpu")
    b = PackedSwiGLULinear(40, 16, device="cpu")
    sd = a.state_dict()
    keep = sd["weight"].clone()
    b.load_state_dict(sd)
    assert torch.equal(b.weight, a.weight)
    assert torch.equal(sd["weight"], keep), "the caller's state dict must not be modified"
    c = PackedSwiGLULinear(40, 16, device="cpu")
    c.load_state_dict({"weight": a.weight.detach().clone()})        # internal [K, 2N] layout
    assert torch.equal(c.weight, a.weight)
    with pytest.raises(RuntimeError):
        c.load_state_dict({"weight": torch.zeros(8, 8, dtype=torch.bfloat16)})


def test_from_linear_and_back():
    torch.manual_seed(2)
    lin = torch.nn.Linear(40, 32, bias=False, dtype=torch.bfloat16)
    m = PackedSwiGLULinear.from_linear(lin)
    assert (m.in_features, m.hidden_features) == (40, 16)
    assert torch.equal(m.linear_weight(), lin.weight.detach())
    assert torch.equal(m.weight.detach()[:, 16:], lin.weight.detach()[16:].t())   # gate columns
    with pytest.raises(ValueError):
        PackedSwiGLULinear.from_linear(torch.nn.Linear(40, 32, bias=True))
    with pytest.raises(ValueError):
        PackedSwiGLULinear(36, 16, device="cpu")            # rows must be multiples of 16 bytes
    with pytest.raises(ValueError):
        m.load_linear_weight_(torch.zeros(16, 40))
    # plugging into a container keeps the nn.Linear layout under the usual key
    seq = torch.nn.Sequential(m)
    assert tuple(seq.state_dict()["0.weight"].shape) == (32, 40)


def test_reference_import_path_and_constructor_switches():
    from swiglu.triton.impls import (PackedSwiGLULinear as P, pack_swiglu_linear_weight,
                                     unpack_swiglu_linear_weight)
    assert P is PackedSwiGLULinear
    with pytest.warns(UserWarning, match="parameter_layout='packed'"):
        m = P(64, 32, block_n_half=64, backward_mode="save_factors", parameter_layout="packed",
              device="cpu")
    assert m.parameter_layout == "normal" and m.backward_mode == "save_factors"
    lw = m.linear_weight()
    assert torch.equal(pack_swiglu_linear_weight(lw, 64), m.weight.detach())
    assert torch.equal(unpack_swiglu_linear_weight(m.weight.detach(), 64), lw)
    with pytest.raises(ValueError):
        P(64, 32, backward_mode="nope", device="cpu")
    with pytest.raises(ValueError):
        P(64, 32, parameter_layout="nope", device="cpu")
    with pytest.raises(ImportError):
        from swiglu.triton.impls import fused_swiglu_wide_packed  # noqa: F401
