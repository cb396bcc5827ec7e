"""The CPU oracle against the committed golden vectors and against the plain-C restatement."""
import hashlib
import os

import numpy as np
import pytest
import torch

import c_oracle
import swiglu_oracle as orc
from swiglu_fused_b200.workloads import make_inputs

SMALL = ["fused_64x128x64", "fused_ragged_200x136x264", "silu_mul_64x128x64",
         "silu_mul_ragged_130x72x328"]


def bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.int16).numpy().tobytes()).hexdigest()


@pytest.mark.parametrize("name", SMALL)
def test_oracle_matches_golden(golden_dir, name):
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    x, h_gold = bf16(g["x"]), bf16(g["h"])
    if str(g["form"]) == "fused_swiglu":
        w = bf16(g["w"])
        h32 = orc.fused_swiglu(x, w)
        h64 = orc.fused_swiglu_f64(x, w)
        hc32 = c_oracle.fused_swiglu(x, w, acc64=False)
        hc64 = c_oracle.fused_swiglu(x, w, acc64=True)
    else:
        wg, up = bf16(g["w_gate"]), bf16(g["up"])
        h32 = orc.silu_mul(x, wg, up)
        h64 = orc.silu_mul_f64(x, wg, up)
        hc32 = c_oracle.silu_mul(x, wg, up, acc64=False)
        hc64 = c_oracle.silu_mul(x, wg, up, acc64=True)
    # float64 evaluations reproduce the stored values exactly (torch and plain C).
    assert torch.equal(h64.view(torch.int16), h_gold.view(torch.int16))
    assert orc.compare(hc64, h_gold).max_ulp <= 1
    assert orc.compare(hc64, h_gold).frac_exact >= 0.9999
    # the fp32 oracle (what the kernels are judged against) is within the stated tolerance
    for h in (h32, hc32):
        rep = orc.compare(h, h_gold)
        assert rep.ok, str(rep)
        assert rep.frac_within_1ulp >= 0.9999, str(rep)


def test_c1_inputs_and_oracle_match_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "c1_512x1024x2048.npz"))
    M, K, N, seed, stride = (int(g[k]) for k in ("M", "K", "N", "seed", "sample_stride"))
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=seed)
    assert sha(inp["x"]) == str(g["x_sha256"]), "seeded x changed: regenerate or fix the generator"
    assert sha(inp["w"]) == str(g["w_sha256"])
    h = orc.fused_swiglu(inp["x"], inp["w"])
    gold = bf16(g["h_fused_sample"])
    rep = orc.compare(h.reshape(-1)[::stride].contiguous(), gold)
    assert rep.ok and rep.frac_within_1ulp >= 0.9999, str(rep)
    # silu_mul view of the same problem
    up = (inp["x"].float() @ inp["w"][:, :N].float()).to(torch.bfloat16)
    up_gold = bf16(g["up_sample"])
    assert orc.compare(up.reshape(-1)[::stride].contiguous(), up_gold).frac_within_1ulp >= 0.9999
    h3 = orc.silu_mul(inp["x"], inp["w"][:, N:].contiguous(), up)
    rep3 = orc.compare(h3.reshape(-1)[::stride].contiguous(), bf16(g["h_silu_mul_sample"]))
    # `up` is an input of this form; a 1-ulp difference in it moves h by up to 1 ulp too
    assert rep3.frac_within_1ulp >= 0.999, str(rep3)


def test_fused_window_arguments_equal_sliced_weight():
    inp = make_inputs(48, 64, 96, form="fused_swiglu", seed=5)
    x, w = inp["x"], inp["w"]  # [64, 192]
    full = orc.fused_swiglu(x, w)
    part = orc.fused_swiglu(x, w, up_col0=32, gate_col0=96 + 32, n_out=32)
    assert torch.equal(part.view(torch.int16), full[:, 32:64].contiguous().view(torch.int16))
    cpart = c_oracle.fused_swiglu(x, w, up_col0=32, gate_col0=128, n_out=32)
    assert orc.compare(cpart, part).ok


def test_bf16_ordinal_is_monotone_and_counts_ulps():
    vals = torch.tensor([-2.0, -1.0, -0.0, 0.0, 2.0 ** -126, 1.0, 1.0078125, 3.0],
                        dtype=torch.bfloat16)
    o = orc.bf16_ordinal(vals)
    assert o[2] == o[3] == 0           # -0 and +0 coincide
    assert torch.all(o[1:] >= o[:-1])  # monotone
    assert o[6] - o[5] == 1            # 1.0 -> next bf16 is one ulp away


def test_compare_flags_errors():
    ref = torch.linspace(-3, 3, 4096).to(torch.bfloat16)
    assert orc.compare(ref.clone(), ref).ok
    bad = ref.clone()
    bad[:64] = (bad[:64].float() * 1.5).to(torch.bfloat16)  # 1.6 % of elements far off
    assert not orc.compare(bad, ref).ok
    nan = ref.clone()
    nan[7] = float("nan")
    assert not orc.compare(nan, ref).ok


def test_relative_error_floor_grows_with_the_reduction_depth():
    assert orc.rel_floor_factor(None) == 2.0 ** -7
    assert orc.rel_floor_factor(1024) == 2.0 ** -7
    assert orc.rel_floor_factor(4096) == 2.0 ** -6
    # a deviation of 1.2 % of the base floor on a zero output: outside at K = 1024, inside at 4096
    ref = torch.full((64, 64), 1.0)
    ref[0, 0] = 0.0
    h = ref.clone()
    h[0, 0] = 0.012 * 2.0 ** -7 * float(ref.mean())
    hb, rb = h.to(torch.bfloat16), ref.to(torch.bfloat16)
    assert not orc.compare(hb, rb, ref).ok
    assert orc.compare(hb, rb, ref, k_depth=4096).ok
