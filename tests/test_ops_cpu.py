"""The Python operators reject bad calls before launching, and never fall back to the CPU."""
import pytest
import torch

import swiglu.matmul_fused_swiglu as ref_path_fused
import swiglu.matmul_silu_mul as ref_path_v3
from swiglu_fused_b200 import matmul_fused_swiglu, matmul_silu_mul, tile_table, _lib
from swiglu_fused_b200.workloads import WORKLOADS, make_inputs


def test_reference_import_paths_resolve_to_the_same_operators():
    assert ref_path_v3.matmul_silu_mul is matmul_silu_mul
    assert ref_path_fused.matmul_fused_swiglu is matmul_fused_swiglu


def test_cpu_tensors_are_rejected_not_computed():
    x = torch.zeros(8, 16, dtype=torch.bfloat16)
    w = torch.zeros(16, 32, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="no CPU path"):
        matmul_fused_swiglu(x, w)
    with pytest.raises(ValueError, match="no CPU path"):
        matmul_silu_mul(x, w[:, :16].contiguous(), torch.zeros(8, 16, dtype=torch.bfloat16))


def test_dtype_and_rank_checks():
    with pytest.raises(TypeError):
        matmul_fused_swiglu(torch.zeros(8, 16), torch.zeros(16, 32))
    with pytest.raises(ValueError, match="2-D"):
        matmul_fused_swiglu(torch.zeros(2, 8, 16, dtype=torch.bfloat16),
                            torch.zeros(16, 32, dtype=torch.bfloat16))
    with pytest.raises(TypeError):
        matmul_fused_swiglu([[1.0]], torch.zeros(16, 32, dtype=torch.bfloat16))


def test_workload_table_matches_the_benchmark_configurations():
    c3 = WORKLOADS["c3_fused"]
    assert (c3.M, c3.K, c3.N) == (32768, 3072, 12288)
    assert c3.flops == 2 * 32768 * 3072 * 2 * 12288
    assert abs(c3.bytes - 1.1576e9) < 1e6
    c2 = WORKLOADS["c2_silu_mul"]
    assert c2.flops == 2 * 32768 * 3072 * 12288
    assert abs(c2.bytes - 1.8874e9) < 1e6
    assert WORKLOADS["c5_llama70b"].w_std == 0.02


def test_seeded_inputs_are_reproducible_and_scaled():
    a = make_inputs(64, 256, 32, seed=3)
    b = make_inputs(64, 256, 32, seed=3)
    assert torch.equal(a["x"], b["x"]) and torch.equal(a["w"], b["w"])
    assert a["w"].shape == (256, 64)
    assert abs(a["x"].float().std().item() - 1.0) < 0.05
    assert abs(a["w"].float().std().item() - 256 ** -0.5) < 0.01
    c = make_inputs(64, 256, 32, seed=3, form="silu_mul", w_std=0.02)
    assert set(c) == {"x", "w_gate", "w_up"}
    assert abs(c["w_up"].float().std().item() - 0.02) < 0.002


def test_tile_table_roundtrip(tmp_path, monkeypatch):
    monkeypatch.setattr(tile_table, "_table", None)
    monkeypatch.setenv("SWIGLU_B200_TILE_TABLE", str(tmp_path / "t.json"))
    assert tile_table.lookup(_lib.FORM_FUSED_SWIGLU, 1, 2, 3) is None
    cfg = _lib.TileConfig(2, 64, 6, 16)
    tile_table.remember(_lib.FORM_FUSED_SWIGLU, 32768, 12288, 3072, cfg)
    tile_table.save()
    monkeypatch.setattr(tile_table, "_table", None)
    got = tile_table.lookup(_lib.FORM_FUSED_SWIGLU, 32768, 12288, 3072)
    assert (got.cta_group, got.block_k, got.stages, got.group_m) == (2, 64, 6, 16)
    monkeypatch.setattr(tile_table, "_table", None)


def test_candidate_configs_drop_pairs_for_a_single_row_tile():
    small = tile_table.legal_configs(_lib.FORM_FUSED_SWIGLU, 64, 14336, 4096)
    assert small and all(c.cta_group == 1 for c in small)
    big = tile_table.legal_configs(_lib.FORM_FUSED_SWIGLU, 32768, 12288, 3072)
    assert any(c.cta_group == 2 for c in big) and any(c.cta_group == 1 for c in big)


def test_shipped_tile_table_entries_are_valid_configurations():
    import json
    import os

    path = tile_table.TABLE_PATH
    assert os.path.exists(path)
    raw = json.load(open(path))
    names = {v: k for k, v in tile_table.FORM_NAMES.items()}
    assert raw["entries"], "the shipped table should carry the tuned benchmark shapes"
    for key, v in raw["entries"].items():
        form_name, shape = key.split(":")
        M, N, K = (int(t) for t in shape.split("x"))
        form = names[form_name]
        cfg = _lib.TileConfig(v["cta_group"], v["block_k"], v["stages"], v["group_m"], 0,
                              v.get("l2_hints", 0))
        assert 0 < _lib.config_smem_bytes(form, cfg) <= 227 * 1024, key
        assert M >= 1 and N % 8 == 0 and K % 8 == 0
    # the headline shape is tuned
    assert tile_table.lookup(_lib.FORM_FUSED_SWIGLU, 32768, 12288, 3072) is not None


def test_gather_mode_is_validated_before_anything_is_launched():
    """`fused_swiglu_n_sharded_fused_gather` rejects an unknown mode, and the multicast mode
    without a multicast mapping, before it touches a barrier or a kernel."""
    import types

    import torch

    from swiglu_fused_b200 import sharding

    calls = []
    out = types.SimpleNamespace(rank=0, world=2, multicast_ptr=0, ptrs=[0, 0],
                                tensor=torch.zeros((4, 8), dtype=torch.bfloat16),
                                barrier=lambda: calls.append("barrier"))
    x = torch.zeros((4, 8), dtype=torch.bfloat16)
    w = torch.zeros((8, 16), dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="unknown gather mode"):
        sharding.fused_swiglu_n_sharded_fused_gather(x, w, out, mode="bogus")
    with pytest.raises(ValueError, match="no multicast mapping"):
        sharding.fused_swiglu_n_sharded_fused_gather(x, w, out, mode="multicast")
    assert calls == []
