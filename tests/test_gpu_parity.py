"""Parity of the CUDA kernels (called through the C ABI) with the CPU oracle.

Tolerance (stated by the task, checked by ``swiglu_oracle.compare``): at least
99.9 % of the elements within 1 bf16 ulp of the oracle and a floored relative
error <= 1e-2, the floor being ``max(|ref|, 2**-7 * mean|ref|)``.
Where two kernel results must be identical (determinism, row/column shards,
schedules that only reorder tiles) the comparison is bit-exact.
"""
import os

import numpy as np
import pytest
import torch

import swiglu_oracle as orc
from swiglu_fused_b200 import TileConfig, _lib, matmul_fused_swiglu, matmul_silu_mul
from swiglu_fused_b200.workloads import make_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# Every kernel variant: (cta_group, block_k).
VARIANTS_FUSED = [(1, 64), (1, 128), (2, 64), (2, 128)]
VARIANTS_SILU_MUL = [(1, 64), (1, 128), (2, 64), (2, 128)]


def bits(t):
    return t.contiguous().view(torch.int16)


def bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


@pytest.fixture(autouse=True)
def _device_status_clean():
    yield
    torch.cuda.synchronize()
    _lib.device_status()   # raises if any kernel wait timed out


def silu_mul_problem(M, K, N, seed):
    inp = make_inputs(M, K, N, form="silu_mul", seed=seed)
    up = (inp["x"].float() @ inp["w_up"].float()).to(torch.bfloat16)
    return inp["x"], inp["w_gate"], up


# ---------------------------------------------------------------- golden fixtures

@pytest.mark.parametrize("name", ["fused_64x128x64", "fused_ragged_200x136x264"])
def test_fused_matches_golden_vectors(golden_dir, name):
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    x, w, gold = bf16(g["x"]), bf16(g["w"]), bf16(g["h"])
    for cg, bk in VARIANTS_FUSED:
        h = matmul_fused_swiglu(x.to(DEV), w.to(DEV), config=TileConfig(cg, bk, 0, 8))
        rep = orc.compare(h.cpu(), gold)
        assert rep.ok, f"cta_group={cg} block_k={bk}: {rep}"


@pytest.mark.parametrize("name", ["silu_mul_64x128x64", "silu_mul_ragged_130x72x328"])
def test_silu_mul_matches_golden_vectors(golden_dir, name):
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    x, wg, up, gold = bf16(g["x"]), bf16(g["w_gate"]), bf16(g["up"]), bf16(g["h"])
    for cg, bk in VARIANTS_SILU_MUL:
        h = matmul_silu_mul(x.to(DEV), wg.to(DEV), up.to(DEV), config=TileConfig(cg, bk, 0, 8))
        rep = orc.compare(h.cpu(), gold)
        assert rep.ok, f"cta_group={cg} block_k={bk}: {rep}"


def test_config1_both_forms_match_oracle_and_golden_sample(golden_dir):
    g = np.load(os.path.join(golden_dir, "c1_512x1024x2048.npz"))
    M, K, N, stride = 512, 1024, 2048, int(g["sample_stride"])
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=0)
    x, w = inp["x"], inp["w"]
    ref32 = orc.fused_swiglu_f32(x, w)
    h = matmul_fused_swiglu(x.to(DEV), w.to(DEV)).cpu()
    rep = orc.compare(h, ref32.to(torch.bfloat16), ref32)
    assert rep.ok, str(rep)
    rep_g = orc.compare(h.reshape(-1)[::stride].contiguous(), bf16(g["h_fused_sample"]))
    assert rep_g.ok, str(rep_g)

    w_up, w_gate = w[:, :N].contiguous(), w[:, N:].contiguous()
    up = (x.float() @ w_up.float()).to(torch.bfloat16)
    ref32 = orc.silu_mul_f32(x, w_gate, up)
    h3 = matmul_silu_mul(x.to(DEV), w_gate.to(DEV), up.to(DEV)).cpu()
    rep3 = orc.compare(h3, ref32.to(torch.bfloat16), ref32)
    assert rep3.ok, str(rep3)


# ---------------------------------------------------------------- shape ladder

LADDER = [(M, K, N) for M in (64, 128, 192, 256, 1024) for N in (128, 256, 384)
          for K in (64, 128, 1024)]
ODD = [(1, 8, 8), (7, 72, 40), (129, 200, 136), (257, 64, 520), (300, 1032, 264), (513, 136, 8)]


@pytest.mark.parametrize("M,K,N", LADDER + ODD)
def test_fused_shape_ladder(M, K, N):
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=M * 7 + K * 3 + N)
    x, w = inp["x"], inp["w"]
    ref32 = orc.fused_swiglu_f32(x, w)
    ref = ref32.to(torch.bfloat16)
    xd, wd = x.to(DEV), w.to(DEV)
    # guard band: one row above/below and 8 columns left/right stay NaN
    big = torch.full((M + 2, N + 16), float("nan"), dtype=torch.bfloat16, device=DEV)
    for cg, bk in VARIANTS_FUSED:
        out = big[1:M + 1, 8:8 + N]
        matmul_fused_swiglu(xd, wd, out=out, config=TileConfig(cg, bk, 0, 8))
        rep = orc.compare(out.cpu(), ref, ref32)
        assert rep.ok, f"{(M, K, N)} cta_group={cg} block_k={bk}: {rep}"
        guard = big.clone()
        guard[1:M + 1, 8:8 + N] = float("nan")
        assert torch.isnan(guard).all(), f"{(M, K, N)} cg={cg} bk={bk}: wrote outside h"
        big.fill_(float("nan"))


@pytest.mark.parametrize("M,K,N", LADDER + ODD)
def test_silu_mul_shape_ladder(M, K, N):
    x, wg, up = silu_mul_problem(M, K, N, seed=M * 5 + K * 11 + N)
    ref32 = orc.silu_mul_f32(x, wg, up)
    ref = ref32.to(torch.bfloat16)
    xd, wd, ud = x.to(DEV), wg.to(DEV), up.to(DEV)
    big = torch.full((M + 2, N + 16), float("nan"), dtype=torch.bfloat16, device=DEV)
    for cg, bk in VARIANTS_SILU_MUL:
        out = big[1:M + 1, 8:8 + N]
        matmul_silu_mul(xd, wd, ud, out=out, config=TileConfig(cg, bk, 0, 8))
        rep = orc.compare(out.cpu(), ref, ref32)
        assert rep.ok, f"{(M, K, N)} cta_group={cg} block_k={bk}: {rep}"
        guard = big.clone()
        guard[1:M + 1, 8:8 + N] = float("nan")
        assert torch.isnan(guard).all(), f"{(M, K, N)} cg={cg} bk={bk}: wrote outside h"
        big.fill_(float("nan"))


# ---------------------------------------------------------------- layouts and schedules

def test_strided_inputs_equal_dense_inputs():
    M, K, N = 384, 264, 392
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=11)
    x, w = inp["x"].to(DEV), inp["w"].to(DEV)
    dense = matmul_fused_swiglu(x, w)
    xs = torch.zeros((M, K + 24), dtype=torch.bfloat16, device=DEV)[:, :K]
    ws = torch.zeros((K, 2 * N + 40), dtype=torch.bfloat16, device=DEV)[:, :2 * N]
    xs.copy_(x)
    ws.copy_(w)
    assert torch.equal(bits(matmul_fused_swiglu(xs, ws)), bits(dense))

    x3, wg, up = (t.to(DEV) for t in silu_mul_problem(M, K, N, seed=12))
    dense3 = matmul_silu_mul(x3, wg, up)
    ups = torch.zeros((M, N + 8), dtype=torch.bfloat16, device=DEV)[:, :N]
    ups.copy_(up)
    assert torch.equal(bits(matmul_silu_mul(x3, wg, ups)), bits(dense3))


def test_results_do_not_depend_on_schedule_or_ring_depth():
    M, K, N = 1024, 512, 1024
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=21)
    x, w = inp["x"].to(DEV), inp["w"].to(DEV)
    base = matmul_fused_swiglu(x, w, config=TileConfig(2, 64, 0, 8))
    for cfg in (TileConfig(2, 64, 2, 1, max_ctas=4),    # 32 tiles on 2 CTA pairs, shallow ring
                TileConfig(2, 64, 3, 3, max_ctas=6),
                TileConfig(2, 64, 0, 32),
                TileConfig(1, 64, 2, 5, max_ctas=3)):
        assert torch.equal(bits(matmul_fused_swiglu(x, w, config=cfg)), bits(base)), cfg
    x3, wg, up = (t.to(DEV) for t in silu_mul_problem(M, K, N, seed=22))
    base3 = matmul_silu_mul(x3, wg, up, config=TileConfig(2, 64, 0, 8))
    for cfg in (TileConfig(2, 64, 2, 1, max_ctas=2), TileConfig(1, 64, 2, 4, max_ctas=5),
                TileConfig(2, 64, 0, 16)):
        assert torch.equal(bits(matmul_silu_mul(x3, wg, up, config=cfg)), bits(base3)), cfg


def test_run_to_run_determinism():
    inp = make_inputs(768, 1024, 640, form="fused_swiglu", seed=31)
    x, w = inp["x"].to(DEV), inp["w"].to(DEV)
    a = matmul_fused_swiglu(x, w)
    for _ in range(5):
        assert torch.equal(bits(matmul_fused_swiglu(x, w)), bits(a))


def test_row_shards_and_column_windows_equal_slices_of_the_full_result():
    M, K, N = 1024, 256, 768
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=41)
    x, w = inp["x"].to(DEV), inp["w"].to(DEV)
    full = matmul_fused_swiglu(x, w)
    world = 4
    for r in range(world):
        r0, rows = _lib.shard_range(M, 256, world, r)
        part = matmul_fused_swiglu(x[r0:r0 + rows], w)
        assert torch.equal(bits(part), bits(full[r0:r0 + rows]))
        c0, cols = _lib.shard_range(N, 128, world, r)
        win = matmul_fused_swiglu(x, w, up_col0=c0, gate_col0=N + c0, n_out=cols)
        assert torch.equal(bits(win), bits(full[:, c0:c0 + cols]))
        # shard writing straight into its column block of the full output
        dst = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
        matmul_fused_swiglu(x, w, up_col0=c0, gate_col0=N + c0, n_out=cols,
                            out=dst[:, c0:c0 + cols])
        assert torch.equal(bits(dst[:, c0:c0 + cols]), bits(full[:, c0:c0 + cols]))


def test_both_forms_agree_when_up_is_exact():
    # With up = fp32-exact small integers the silu_mul form (bf16 `up` input) and the
    # fused form (fp32 `up` accumulator) see the same factors.
    M, K, N = 256, 64, 256
    g = torch.Generator().manual_seed(5)
    x = torch.randint(-2, 3, (M, K), generator=g).to(torch.bfloat16)
    w_up = torch.randint(-1, 2, (K, N), generator=g).to(torch.bfloat16)
    w_gate = (torch.randn((K, N), generator=g) * 0.125).to(torch.bfloat16)
    up = (x.float() @ w_up.float())
    assert up.abs().max() <= 256           # exactly representable in bf16
    up = up.to(torch.bfloat16)
    w = torch.cat([w_up, w_gate], dim=1).contiguous()
    a = matmul_fused_swiglu(x.to(DEV), w.to(DEV))
    b = matmul_silu_mul(x.to(DEV), w_gate.to(DEV), up.to(DEV))
    assert torch.equal(bits(a), bits(b))


def test_out_and_stream_arguments_and_no_hidden_allocation():
    M, K, N = 512, 256, 512
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=51)
    x, w = inp["x"].to(DEV), inp["w"].to(DEV)
    ref = matmul_fused_swiglu(x, w)
    out = torch.empty_like(ref)
    side = torch.cuda.Stream()
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    before = torch.cuda.memory_allocated()
    n0 = _lib.kernel_launches()
    with torch.cuda.stream(side):
        got = matmul_fused_swiglu(x, w, out=out)
    side.synchronize()
    assert got is out
    assert _lib.kernel_launches() - n0 == 1
    assert torch.cuda.max_memory_allocated() == before, "the call allocated device memory"
    assert torch.equal(bits(out), bits(ref))
    out.zero_()
    matmul_fused_swiglu(x, w, out=out, stream=side)
    side.synchronize()
    assert torch.equal(bits(out), bits(ref))


def test_bad_calls_raise_before_launch():
    x = torch.zeros((64, 64), dtype=torch.bfloat16, device=DEV)
    w = torch.zeros((64, 128), dtype=torch.bfloat16, device=DEV)
    n0 = _lib.kernel_launches()
    with pytest.raises(ValueError):
        matmul_fused_swiglu(x, w[:32])                      # K mismatch
    with pytest.raises(ValueError):
        matmul_fused_swiglu(x, w, out=torch.empty((64, 32), dtype=torch.bfloat16, device=DEV))
    with pytest.raises(ValueError):
        matmul_fused_swiglu(x.t(), w)                       # not row-major
    with pytest.raises(TypeError):
        matmul_fused_swiglu(x.float(), w)
    with pytest.raises(ValueError):
        matmul_fused_swiglu(x, w, config=TileConfig(2, 64, 9, 8))
    with pytest.raises(ValueError):
        matmul_silu_mul(x, w[:, :64].contiguous(),
                        torch.zeros((32, 64), dtype=torch.bfloat16, device=DEV))
    with pytest.raises(ValueError):
        matmul_fused_swiglu(x, w, up_col0=0, gate_col0=100, n_out=32)   # window outside W
    assert _lib.kernel_launches() == n0


def test_extreme_gate_values_saturate_cleanly():
    # silu(+big) = big, silu(-big) = -0: no NaN/Inf from the exp/rcp path.  Results whose
    # magnitude is below 2**-100 may flush to zero (the approximate reciprocal flushes
    # subnormals), so those are compared by absolute value only.
    M, K, N = 128, 64, 128
    x = torch.zeros((M, K), dtype=torch.bfloat16)
    x[:, 0] = 1.0
    w_gate = torch.zeros((K, N), dtype=torch.bfloat16)
    w_gate[0, :] = torch.linspace(-300, 300, N).to(torch.bfloat16)
    up = torch.ones((M, N), dtype=torch.bfloat16)
    h = matmul_silu_mul(x.to(DEV), w_gate.to(DEV), up.to(DEV)).cpu()
    ref32 = orc.silu_mul_f32(x, w_gate, up)
    assert torch.isfinite(h.float()).all()
    tiny = ref32.abs() < 2.0 ** -100
    assert (h.float()[tiny].abs() < 2.0 ** -99).all()
    keep = ~tiny[0]
    rep = orc.compare(h[:, keep].contiguous(), ref32[:, keep].to(torch.bfloat16).contiguous(),
                      ref32[:, keep].contiguous())
    assert rep.ok, str(rep)
    xd = x.to(DEV)
    w = torch.cat([torch.ones((K, N), dtype=torch.bfloat16) * x[0:1, :].t(), w_gate], dim=1)
    hf = matmul_fused_swiglu(xd, w.contiguous().to(DEV)).cpu()   # up = 1 through the GEMM
    assert torch.equal(bits(hf), bits(h))


def test_empty_batch_returns_empty_without_launching():
    n0 = _lib.kernel_launches()
    x = torch.empty((0, 64), dtype=torch.bfloat16, device=DEV)
    w = torch.zeros((64, 256), dtype=torch.bfloat16, device=DEV)
    h = matmul_fused_swiglu(x, w)
    assert h.shape == (0, 128) and h.dtype == torch.bfloat16
    h3 = matmul_silu_mul(x, w[:, :128].contiguous(),
                         torch.empty((0, 128), dtype=torch.bfloat16, device=DEV))
    assert h3.shape == (0, 128)
    assert _lib.kernel_launches() == n0


def test_autotune_picks_a_working_entry_and_remembers_it(monkeypatch, tmp_path):
    from swiglu_fused_b200 import tile_table, tune_matmul_fused_swiglu, tune_matmul_silu_mul

    monkeypatch.setattr(tile_table, "_table", None)
    monkeypatch.setenv("SWIGLU_B200_TILE_TABLE", str(tmp_path / "tuned.json"))
    M, K, N = 1024, 512, 768
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=61)
    x, w = inp["x"].to(DEV), inp["w"].to(DEV)
    best = tune_matmul_fused_swiglu(x, w, persist=True)
    assert best in tile_table.legal_configs(_lib.FORM_FUSED_SWIGLU, M, N, K)
    assert tile_table.lookup(_lib.FORM_FUSED_SWIGLU, M, N, K) == best
    monkeypatch.setattr(tile_table, "_table", None)          # reload from the file
    again = tile_table.lookup(_lib.FORM_FUSED_SWIGLU, M, N, K)
    assert (again.cta_group, again.block_k, again.group_m) == \
        (best.cta_group, best.block_k, best.group_m)
    ref32 = orc.fused_swiglu_f32(inp["x"], inp["w"])
    assert orc.compare(matmul_fused_swiglu(x, w).cpu(), ref32.to(torch.bfloat16), ref32).ok

    x3, wg, up = (t.to(DEV) for t in silu_mul_problem(M, K, N, seed=62))
    best3 = tune_matmul_silu_mul(x3, wg, up)
    assert best3 in tile_table.legal_configs(_lib.FORM_SILU_MUL, M, N, K)
    monkeypatch.setattr(tile_table, "_table", None)


def test_launch_is_capturable_in_a_cuda_graph():
    M, K, N = 512, 256, 512
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=71)
    x, w = inp["x"].to(DEV), inp["w"].to(DEV)
    ref = matmul_fused_swiglu(x, w)
    out = torch.zeros_like(ref)
    matmul_fused_swiglu(x, w, out=out)            # first call sets function attributes
    out.zero_()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        with torch.cuda.graph(graph, stream=s):
            matmul_fused_swiglu(x, w, out=out)
    torch.cuda.synchronize()
    assert not torch.equal(bits(out), bits(ref))  # capture does not execute
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(bits(out), bits(ref))


def test_concurrent_launches_from_two_host_threads():
    import threading

    M, K, N = 1024, 512, 512
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=81)
    x, w = inp["x"].to(DEV), inp["w"].to(DEV)
    ref = matmul_fused_swiglu(x, w)
    outs = [torch.zeros_like(ref) for _ in range(2)]
    errors = []

    def worker(i):
        try:
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                for _ in range(20):
                    matmul_fused_swiglu(x, w, out=outs[i])
            st.synchronize()
        except Exception as e:  # surfaced below
            errors.append(e)

    torch.cuda.synchronize()
    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for o in outs:
        assert torch.equal(bits(o), bits(ref))


def test_a_wait_that_runs_out_is_reported_and_the_context_survives():
    """Failure detection without a fault: a wait nobody satisfies times out after 2 ms, the
    kernel records it and exits, the host sees the status, and the next launch works."""
    import time

    lib = _lib.load()
    torch.cuda.synchronize()
    _lib.device_status()                                   # clean before
    t0 = time.perf_counter()
    assert lib.sgl_selftest_wait_timeout(2_000_000, None) == 0
    with pytest.raises(_lib.SglError) as err:
        _lib.device_status()                               # synchronises, reads, clears
    elapsed = time.perf_counter() - t0
    assert err.value.code == -9 and "0x1ff" in err.value.message
    assert elapsed < 1.0, f"the bounded wait took {elapsed:.3f} s for a 2 ms limit"
    assert _lib.device_status()[0] == 0                    # record was cleared
    inp = make_inputs(256, 128, 256, form="fused_swiglu", seed=91)
    ref32 = orc.fused_swiglu_f32(inp["x"], inp["w"])
    h = matmul_fused_swiglu(inp["x"].to(DEV), inp["w"].to(DEV))
    assert orc.compare(h.cpu(), ref32.to(torch.bfloat16), ref32).ok


@pytest.mark.parametrize("M,K,N,window", [(512, 256, 1024, (256, 384)), (200, 136, 264, (64, 136)),
                                          (1000, 264, 1160, (384, 392))])
def test_gather_epilogues_write_every_destination(M, K, N, window):
    """The column-parallel gather on one GPU: the "peers" are further buffers of this GPU.
    Every destination (TMA stores to each, or TMA store + ordinary 16-byte stores) must hold
    the column block, bit for bit, in its window of a full-width buffer, and nothing else may
    be touched (NaN sentinels around the window stay)."""
    from swiglu_fused_b200.ops import matmul_fused_swiglu_gather, matmul_fused_swiglu_multi_dst

    c0, n = window
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=M + N)
    x, w = inp["x"].to(DEV), inp["w"].to(DEV)
    want = matmul_fused_swiglu(x, w, up_col0=c0, gate_col0=N + c0, n_out=n)
    for mode in ("tma", "stores"):
        bufs = [torch.full((M + 8, N), float("nan"), dtype=torch.bfloat16, device=DEV)
                for _ in range(4)]
        ptrs = [b.data_ptr() + 2 * c0 for b in bufs]
        kw = dict(up_col0=c0, gate_col0=N + c0, n_out=n)
        if mode == "tma":
            matmul_fused_swiglu_multi_dst(x, w, ptrs, N, **kw)
        else:
            matmul_fused_swiglu_gather(x, w, ptrs[0], ptrs[1:], N, **kw)
        torch.cuda.synchronize()
        _lib.device_status()
        for i, b in enumerate(bufs):
            assert torch.equal(b[:M, c0:c0 + n].contiguous().view(torch.int16),
                               want.view(torch.int16)), (mode, i)
            rest = b.clone()
            rest[:M, c0:c0 + n] = float("nan")
            assert bool(torch.isnan(rest.float()).all()), (mode, i)


@pytest.mark.parametrize("M,K,N", [(256, 128, 512), (200, 136, 264), (1000, 264, 1160),
                                   (512, 1024, 2048), (2048, 512, 640), (300, 4096, 1408)])
def test_wide_tiles_give_the_same_bits(M, K, N):
    """Tiles of 256 output columns (two MMAs per k-step into one accumulator stage) against
    the 128-column tiles: same per-element arithmetic in the same order, so identical bits, on
    aligned and ragged shapes, several tiles per CTA pair included (max_ctas = 8), with column
    windows, and with the gather epilogue."""
    from swiglu_fused_b200.ops import matmul_fused_swiglu_gather

    inp = make_inputs(M, K, N, form="fused_swiglu", seed=M + K)
    x, w = inp["x"].to(DEV), inp["w"].to(DEV)
    want = matmul_fused_swiglu(x, w, config=TileConfig(2, 64, 0, 8))
    for cfg in (TileConfig(2, 64, 0, 8, 0, 0, 0, 1), TileConfig(2, 64, 2, 4, 8, 18, 0, 1),
                TileConfig(2, 64, 0, 1, 4, 0, 2, 1)):
        got = matmul_fused_swiglu(x, w, config=cfg)
        torch.cuda.synchronize()
        _lib.device_status()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), cfg
    ref32 = orc.fused_swiglu_f32(inp["x"], inp["w"])
    assert orc.compare(want.cpu(), ref32.to(torch.bfloat16), ref32).ok
    # a column window, delivered to two buffers by the store epilogue
    c0, n = 128, min(N - 128, 264)
    win = matmul_fused_swiglu(x, w, up_col0=c0, gate_col0=N + c0, n_out=n,
                              config=TileConfig(2, 64, 0, 8))
    bufs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    matmul_fused_swiglu_gather(x, w, bufs[0].data_ptr() + 2 * c0, [bufs[1].data_ptr() + 2 * c0], N,
                               up_col0=c0, gate_col0=N + c0, n_out=n,
                               config=TileConfig(2, 64, 0, 8, 0, 0, 0, 1))
    torch.cuda.synchronize()
    _lib.device_status()
    for b in bufs:
        assert torch.equal(b[:, c0:c0 + n].contiguous().view(torch.int16), win.view(torch.int16))
    with pytest.raises(ValueError):       # wide tiles exist for CTA pairs with BLOCK_K 64 only
        matmul_fused_swiglu(x, w, config=TileConfig(2, 128, 0, 8, 0, 0, 0, 1))


@pytest.mark.parametrize("M,K,N", [(64, 4096, 4096), (16, 4096, 5632), (100, 8192, 1000), (128, 4096, 256),
                                    (8, 16384, 520)])
def test_narrow_fused_problems_cut_k_into_clusters(M, K, N):
    """A gate/up stage with few tiles at decode sizes (up to 128 rows, K >= 4096, the library's
    own configuration): K is cut into ranges that run as thread-block clusters; each CTA sums
    its share of the tile over the ranges and applies silu(gate) * up.  One launch, the fp32
    reference's value (the sum order differs from the whole-K kernel's, the per-element
    arithmetic after it does not), and nothing outside the output is touched; column windows
    and strided outputs included."""
    inp = make_inputs(M, K, N, form="fused_swiglu", seed=M + K + N)
    x, w = inp["x"].to(DEV), inp["w"].to(DEV)
    big = torch.full((M + 2, N + 16), float("nan"), dtype=torch.bfloat16, device=DEV)
    out = big[1:M + 1, 8:8 + N]
    n0 = _lib.kernel_launches()
    for _ in range(3):
        matmul_fused_swiglu(x, w, out=out)
    torch.cuda.synchronize()
    assert _lib.kernel_launches() - n0 == 3
    _lib.device_status()
    before = _lib.set_splitk_cluster_sum(False)
    try:
        whole = matmul_fused_swiglu(x, w)
    finally:
        _lib.set_splitk_cluster_sum(before)
    got = out.contiguous()
    ref64 = orc.fused_swiglu_exact(inp["x"], inp["w"])
    rep = orc.compare(got.cpu(), ref64.to(torch.bfloat16), ref64, k_depth=K)
    assert rep.ok, str(rep)
    # two kernels that each sit within one ulp of the exact value can be two apart
    both = orc.compare(got, whole, k_depth=K)
    assert both.n_nonfinite == 0 and both.frac_within_1ulp >= 0.99 and \
        both.max_floored_rel <= 2 * orc.MAX_FLOORED_REL_ERR, str(both)
    assert not torch.equal(got, whole), "the whole-K kernel ran: no cluster plan was taken"
    guard = big.clone()
    guard[1:M + 1, 8:8 + N] = float("nan")
    assert torch.isnan(guard).all(), "wrote outside the output"
    # a column window of the packed weight (what a column-parallel rank computes)
    if N >= 512:
        c0, n = 128, 264
        win = matmul_fused_swiglu(x, w, up_col0=c0, gate_col0=N + c0, n_out=n)
        # (fewer tiles, so possibly more K ranges than the full width got: same value, not
        # necessarily the same bits)
        rep = orc.compare(win, got[:, c0:c0 + n].contiguous(), k_depth=K)
        assert rep.n_nonfinite == 0 and rep.frac_within_1ulp >= 0.99 and \
            rep.max_floored_rel <= 2 * orc.MAX_FLOORED_REL_ERR, str(rep)
    # an explicit configuration is taken literally: whole-K tiles
    lit = matmul_fused_swiglu(x, w, config=TileConfig(1, 64, 0, 8))
    assert torch.equal(lit.view(torch.int16), whole.view(torch.int16))
    _lib.device_status()


@pytest.mark.parametrize("M,K,N", [(64, 4096, 4096), (16, 8192, 1000), (128, 4096, 520), (72, 16384, 256)])
def test_narrow_silu_mul_problems_cut_k_into_clusters(M, K, N):
    """The same plan in the silu_mul form: the K ranges of a 256-column tile run as a thread-block
    cluster, the gate pre-activation is summed over them and the CTA that sums a group of
    columns reads `up` for it from global memory and applies silu(gate) * up."""
    x, wg, up = silu_mul_problem(M, K, N, seed=M + K + N)
    xd, wd, ud = x.to(DEV), wg.to(DEV), up.to(DEV)
    big = torch.full((M + 2, N + 16), float("nan"), dtype=torch.bfloat16, device=DEV)
    out = big[1:M + 1, 8:8 + N]
    upbig = torch.zeros((M, N + 24), dtype=torch.bfloat16, device=DEV)   # a strided `up`
    upbig[:, 8:8 + N] = ud
    n0 = _lib.kernel_launches()
    for _ in range(3):
        matmul_silu_mul(xd, wd, upbig[:, 8:8 + N], out=out)
    torch.cuda.synchronize()
    assert _lib.kernel_launches() - n0 == 3
    _lib.device_status()
    before = _lib.set_splitk_cluster_sum(False)
    try:
        whole = matmul_silu_mul(xd, wd, ud)
    finally:
        _lib.set_splitk_cluster_sum(before)
    got = out.contiguous()
    ref32 = orc.silu_mul_f32(x, wg, up)
    rep = orc.compare(got.cpu(), ref32.to(torch.bfloat16), ref32, k_depth=K)
    assert rep.ok, str(rep)
    both = orc.compare(got, whole, k_depth=K)
    assert both.n_nonfinite == 0 and both.frac_within_1ulp >= 0.99 and \
        both.max_floored_rel <= 2 * orc.MAX_FLOORED_REL_ERR, str(both)
    assert not torch.equal(got, whole), "the whole-K kernel ran: no cluster plan was taken"
    guard = big.clone()
    guard[1:M + 1, 8:8 + N] = float("nan")
    assert torch.isnan(guard).all(), "wrote outside the output"
    lit = matmul_silu_mul(xd, wd, ud, config=TileConfig(1, 64, 0, 8))
    assert torch.equal(lit.view(torch.int16), whole.view(torch.int16))
    _lib.device_status()
