"""The plain bf16 GEMM form (down projection) and its fused reduce-scatter, against the torch
fp32 reference (``swiglu_oracle.matmul_f32``).  Same tolerance as the activation kernels:
>= 99.9 % of elements within 1 bf16 ulp, floored relative error <= 1e-2."""
import pytest
import torch

import swiglu_oracle as orc
from swiglu_fused_b200 import TileConfig, _lib, matmul_bf16
from swiglu_fused_b200.ops import matmul_bf16_reduce_scatter

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
VARIANTS = [(1, 64), (1, 128), (2, 64), (2, 128)]


@pytest.fixture(autouse=True)
def _device_status_clean():
    yield
    torch.cuda.synchronize()
    _lib.device_status()


def problem(M, K, N, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn((M, K), generator=g).to(torch.bfloat16)
    b = (torch.randn((K, N), generator=g) * K ** -0.5).to(torch.bfloat16)
    return a, b


@pytest.mark.parametrize("M,K,N", [(128, 64, 256), (256, 256, 256), (512, 1024, 2048),
                                    (200, 136, 264), (1024, 512, 1024), (1, 8, 8),
                                    (300, 1032, 520), (64, 4096, 512)])
def test_matmul_matches_fp32_reference(M, K, N):
    a, b = problem(M, K, N, seed=M + K + N)
    ref32 = orc.matmul_f32(a, b)
    ref = ref32.to(torch.bfloat16)
    ad, bd = a.to(DEV), b.to(DEV)
    big = torch.full((M + 2, N + 16), float("nan"), dtype=torch.bfloat16, device=DEV)
    for cg, bk in VARIANTS:
        out = big[1:M + 1, 8:8 + N]
        matmul_bf16(ad, bd, out=out, config=TileConfig(cg, bk, 0, 8))
        rep = orc.compare(out.cpu(), ref, ref32)
        assert rep.ok, f"{(M, K, N)} cta_group={cg} block_k={bk}: {rep}"
        guard = big.clone()
        guard[1:M + 1, 8:8 + N] = float("nan")
        assert torch.isnan(guard).all(), "wrote outside the output"
        big.fill_(float("nan"))


@pytest.mark.parametrize("M,K,N", [(256, 128, 256), (512, 1024, 768), (200, 136, 264),
                                    (1024, 520, 384), (64, 2048, 128)])
@pytest.mark.parametrize("ta,tb", [(False, True), (True, False), (True, True)])
def test_transposed_operands_are_read_in_place(M, K, N, ta, tb):
    a, b = problem(M, K, N, seed=M * 3 + K + N)
    ref32 = orc.matmul_f32(a, b)
    ad = (a.t().contiguous() if ta else a).to(DEV)        # stored [K, M] when ta
    bd = (b.t().contiguous() if tb else b).to(DEV)        # stored [N, K] when tb
    plain = matmul_bf16(a.to(DEV), b.to(DEV))
    for cg, bk in VARIANTS:
        got = matmul_bf16(ad, bd, transpose_a=ta, transpose_b=tb, config=TileConfig(cg, bk, 0, 8))
        rep = orc.compare(got.cpu(), ref32.to(torch.bfloat16), ref32)
        assert rep.ok, f"{(M, K, N)} ta={ta} tb={tb} cg={cg} bk={bk}: {rep}"
    # same products, same accumulation order: identical to the untransposed call
    assert torch.equal(matmul_bf16(ad, bd, transpose_a=ta, transpose_b=tb).view(torch.int16),
                       plain.view(torch.int16))


def test_matmul_equals_cublas_on_exact_data():
    # small integers: every product and partial sum is exact, so any correct GEMM agrees bit for bit
    g = torch.Generator().manual_seed(1)
    a = torch.randint(-3, 4, (512, 256), generator=g).to(torch.bfloat16).to(DEV)
    b = torch.randint(-2, 3, (256, 768), generator=g).to(torch.bfloat16).to(DEV)
    assert torch.equal(matmul_bf16(a, b).view(torch.int16), (a @ b).view(torch.int16))


@pytest.mark.parametrize("dst_f32", [True, False])
def test_reduce_scatter_epilogue_on_one_gpu(dst_f32):
    """Two row-block owners, both buffers on this GPU; two launches (two 'ranks') add their
    partial products of a K-split problem.  The sum must equal the unsplit product."""
    M, K, N = 1024, 512, 768
    a, b = problem(M, K, N, seed=9)
    ad, bd = a.to(DEV), b.to(DEV)
    rows = 512
    dt = torch.float32 if dst_f32 else torch.bfloat16
    bufs = [torch.zeros((rows, N), dtype=dt, device=DEV) for _ in range(2)]
    ptrs = [t.data_ptr() for t in bufs]
    for r in range(2):                                   # rank r holds K-slice r
        ks = slice(r * K // 2, (r + 1) * K // 2)
        matmul_bf16_reduce_scatter(ad[:, ks], bd[ks].contiguous(), ptrs, rows, N, dst_f32=dst_f32,
                                   first_dst=r)          # each 'rank' starts at a different owner
    torch.cuda.synchronize()
    got = torch.cat(bufs, dim=0)
    ref32 = orc.matmul_f32(a, b)
    if dst_f32:
        assert torch.allclose(got.cpu(), ref32, rtol=1e-5, atol=1e-4)
        rep = orc.compare(got.to(torch.bfloat16).cpu(), ref32.to(torch.bfloat16), ref32)
        assert rep.ok, str(rep)
    else:
        # bf16 accumulation rounds after each rank's contribution, relative to the size of the
        # PARTIAL sums (which can cancel), so the bound is absolute: one bf16 ulp of the
        # largest partial sum.  The fp32 destination is the accurate one.
        rep = orc.compare(got.cpu(), ref32.to(torch.bfloat16), ref32)
        part = orc.matmul_f32(a[:, :K // 2], b[:K // 2]).abs().max().item()
        assert rep.max_abs <= part * 2.0 ** -7 and rep.frac_within_1ulp >= 0.9, str(rep)


def test_slot_scatter_and_slot_sum_on_one_gpu():
    """Two 'ranks' (K halves) write their partial products into their own slots of two owners'
    buffers (both on this GPU); each owner then sums its slots."""
    from swiglu_fused_b200.ops import sum_bf16_slots

    M, K, N = 1024, 512, 640
    a, b = problem(M, K, N, seed=19)
    ad, bd = a.to(DEV), b.to(DEV)
    rows, world = 512, 2
    owners = [torch.full((world, rows, N), float("nan"), dtype=torch.bfloat16, device=DEV)
              for _ in range(world)]
    for r in range(world):
        ks = slice(r * K // 2, (r + 1) * K // 2)
        dsts = [o.data_ptr() + r * rows * N * 2 for o in owners]
        matmul_bf16_reduce_scatter(ad[:, ks], bd[ks].contiguous(), dsts, rows, N, dst_f32=False,
                                   accumulate=False, first_dst=(r + 1) % world)
    torch.cuda.synchronize()
    got = torch.cat([sum_bf16_slots(o) for o in owners], dim=0)
    parts = [orc.matmul_f32(a[:, r * K // 2:(r + 1) * K // 2], b[r * K // 2:(r + 1) * K // 2])
             .to(torch.bfloat16).float() for r in range(world)]
    want = (parts[0] + parts[1]).to(torch.bfloat16)
    rep = orc.compare(got.cpu(), want)
    # the kernel's partial products can differ from the CPU's by one bf16 ulp of the PARTIAL,
    # which after cancellation is several ulps of the sum: bound the error by the partials
    part = max(p.abs().max().item() for p in parts)
    assert rep.frac_within_1ulp >= 0.99 and rep.max_abs <= part * 2.0 ** -7, str(rep)
    # a limited row count and an explicit output
    out = torch.empty((100, N), dtype=torch.bfloat16, device=DEV)
    sum_bf16_slots(owners[0], out, rows=100)
    assert torch.equal(out.view(torch.int16), got[:100].contiguous().view(torch.int16))


@pytest.mark.parametrize("M,K,N,splits", [(64, 4096, 512, 0), (64, 14336, 4096, 8), (128, 2048, 256, 4),
                                           (200, 1032, 264, 3), (16, 512, 128, 2), (256, 1024, 256, 1),
                                           (300, 8192, 520, 16)])
def test_splitk_matches_fp32_reference_and_unsplit_kernel(M, K, N, splits):
    from swiglu_fused_b200.ops import matmul_bf16_splitk, splitk_scratch_bytes

    a, b = problem(M, K, N, seed=M + K + N + splits)
    ad, bd = a.to(DEV), b.to(DEV)
    ref32 = orc.matmul_f32(a, b)
    need = splitk_scratch_bytes(M, N, K, splits)
    scratch = torch.full((need + 256,), 0xFF, dtype=torch.uint8, device=DEV)   # NaN-ish fill + canary
    big = torch.full((M + 2, N + 16), float("nan"), dtype=torch.bfloat16, device=DEV)
    out = big[1:M + 1, 8:8 + N]
    for cfg in (None, TileConfig(1, 64, 0, 8), TileConfig(2, 128, 0, 8)):
        matmul_bf16_splitk(ad, bd, out=out, splits=splits, scratch=scratch[:need], config=cfg)
        rep = orc.compare(out.cpu(), ref32.to(torch.bfloat16), ref32)
        assert rep.ok, f"{(M, K, N, splits)} {cfg}: {rep}"
        # fp32 partial sums: agrees with the unsplit kernel except where the fp32 summation
        # order moves a value across a bf16 rounding boundary
        one = matmul_bf16(ad, bd, config=cfg)
        both = orc.compare(out.contiguous(), one)
        assert both.ok and both.frac_exact >= 0.99, str(both)
        assert bool((scratch[need:] == 0xFF).all()), "wrote past the scratch it asked for"
        guard = big.clone()
        guard[1:M + 1, 8:8 + N] = float("nan")
        assert torch.isnan(guard).all(), "wrote outside the output"
    with pytest.raises(ValueError):
        matmul_bf16_splitk(ad, bd, splits=splits, scratch=scratch[:need - 64])


@pytest.mark.parametrize("M,K,N,splits", [(64, 14336, 4096, 8), (64, 14336, 4096, 0), (33, 4096, 264, 4),
                                           (128, 2048, 512, 8), (8, 1024, 4096, 2), (100, 8192, 1000, 3),
                                           (16, 512, 128, 2), (64, 8192, 2048, 16)])
def test_splitk_summed_in_the_cluster_gives_the_bits_of_the_two_kernel_form(M, K, N, splits):
    """Where the K ranges of a tile run as one thread-block cluster the partial tiles never
    leave the SMs: one launch instead of two kernels and no scratch traffic.  Same fp32
    additions in the same order: the result must be the two-kernel form's bit for bit, and the
    scratch (still passed, for the problems that need it) must stay untouched."""
    from swiglu_fused_b200.ops import matmul_bf16_splitk, splitk_scratch_bytes

    a, b = problem(M, K, N, seed=7 * M + K + N + splits)
    ad, bd = a.to(DEV), b.to(DEV)
    need = splitk_scratch_bytes(M, N, K, splits)
    scratch = torch.full((need + 256,), 0xFF, dtype=torch.uint8, device=DEV)
    before = _lib.set_splitk_cluster_sum(False)
    try:
        n0 = _lib.kernel_launches()
        two = matmul_bf16_splitk(ad, bd, splits=splits, scratch=scratch[:need])
        torch.cuda.synchronize()
        assert _lib.kernel_launches() - n0 == 2
    finally:
        _lib.set_splitk_cluster_sum(before)
    _lib.set_splitk_cluster_sum(True)
    scratch.fill_(0xFF)
    big = torch.full((M + 2, N + 16), float("nan"), dtype=torch.bfloat16, device=DEV)
    out = big[1:M + 1, 8:8 + N]
    n0 = _lib.kernel_launches()
    for _ in range(3):           # back to back: a launch must not disturb its successor
        matmul_bf16_splitk(ad, bd, out=out, splits=splits, scratch=scratch[:need])
    torch.cuda.synchronize()
    launches = (_lib.kernel_launches() - n0) // 3
    tiles = -(-N // 256)
    if splits == 0:
        # left to choose, the library takes a plan whose clusters all fit at once (narrower
        # tiles, fewer ranges): one launch, and other K ranges than the two-kernel choice, so
        # the fp32 additions differ in order
        assert launches == 1
        both = orc.compare(out.contiguous(), two)
        assert both.ok and both.frac_exact >= 0.99, str(both)
    else:
        # clusters are placed whole: 15 of 8 CTAs fit a B200, so 16 tiles x 8 ranges stay on
        # the two-kernel form; a handful of tiles always fits
        assert launches == 1 if tiles <= 4 else launches in (1, 2), (launches, tiles)
        assert torch.equal(out.contiguous().view(torch.int16), two.view(torch.int16))
    if launches == 1:
        assert bool((scratch == 0xFF).all()), "the cluster sum touched the scratch"
    guard = big.clone()
    guard[1:M + 1, 8:8 + N] = float("nan")
    assert torch.isnan(guard).all(), "wrote outside the output"
    ref32 = orc.matmul_f32(a, b)
    assert orc.compare(out.cpu(), ref32.to(torch.bfloat16), ref32).ok
    _lib.device_status()


def test_plain_matmul_cuts_k_into_clusters_where_that_fills_the_gpu():
    """The plain entry point needs no scratch for K ranges that sum themselves in thread-block
    clusters, so with the library's own configuration it takes that plan for short, deep
    problems (the down projection at decode sizes) and only there: same bits as the split-K
    entry point left to choose, the whole-K kernel's bits where the whole-K grid already fills
    the GPU, and the fp32 reference's value either way."""
    from swiglu_fused_b200.ops import matmul_bf16_splitk

    a, b = problem(64, 14336, 4096, seed=77)
    ad, bd = a.to(DEV), b.to(DEV)
    n0 = _lib.kernel_launches()
    got = matmul_bf16(ad, bd)
    assert _lib.kernel_launches() - n0 == 1
    assert torch.equal(got.view(torch.int16), matmul_bf16_splitk(ad, bd).view(torch.int16))
    before = _lib.set_splitk_cluster_sum(False)
    try:
        whole = matmul_bf16(ad, bd)
    finally:
        _lib.set_splitk_cluster_sum(before)
    both = orc.compare(got, whole)
    assert both.ok and both.frac_exact >= 0.99 and not torch.equal(got, whole), str(both)
    ref32 = orc.matmul_f32(a, b)
    assert orc.compare(got.cpu(), ref32.to(torch.bfloat16), ref32).ok
    # an explicit configuration is taken literally: whole-K tiles
    assert torch.equal(matmul_bf16(ad, bd, config=TileConfig(1, 64, 0, 8)).view(torch.int16),
                       whole.view(torch.int16))
    # 112 whole-K tiles already occupy as many SMs as any cluster plan would: nothing changes
    a2, b2 = problem(64, 4096, 14336, seed=78)
    a2d, b2d = a2.to(DEV), b2.to(DEV)
    got2 = matmul_bf16(a2d, b2d)
    before = _lib.set_splitk_cluster_sum(False)
    try:
        whole2 = matmul_bf16(a2d, b2d)
    finally:
        _lib.set_splitk_cluster_sum(before)
    assert torch.equal(got2.view(torch.int16), whole2.view(torch.int16))
    # 129 to 256 rows: two rows of single-CTA tiles in clusters instead of one row of CTA pairs
    for (M3, K3, N3) in ((256, 14336, 4096), (136, 8192, 2056)):
        a3, b3 = problem(M3, K3, N3, seed=M3)
        a3d, b3d = a3.to(DEV), b3.to(DEV)
        big = torch.full((M3 + 2, N3 + 16), float("nan"), dtype=torch.bfloat16, device=DEV)
        out3 = big[1:M3 + 1, 8:8 + N3]
        matmul_bf16(a3d, b3d, out=out3)
        before = _lib.set_splitk_cluster_sum(False)
        try:
            whole3 = matmul_bf16(a3d, b3d)
        finally:
            _lib.set_splitk_cluster_sum(before)
        both = orc.compare(out3.contiguous(), whole3)
        assert both.ok and both.frac_exact >= 0.99, str(both)
        assert not torch.equal(out3.contiguous(), whole3)        # it did take the other plan
        ref32 = orc.matmul_f32(a3, b3)
        assert orc.compare(out3.cpu(), ref32.to(torch.bfloat16), ref32).ok
        guard = big.clone()
        guard[1:M3 + 1, 8:8 + N3] = float("nan")
        assert torch.isnan(guard).all(), "wrote outside the output"
    _lib.device_status()


def test_reduce_scatter_rejects_bad_row_blocks():
    a = torch.zeros((256, 64), dtype=torch.bfloat16, device=DEV)
    b = torch.zeros((64, 64), dtype=torch.bfloat16, device=DEV)
    buf = torch.zeros((256, 64), dtype=torch.float32, device=DEV)
    with pytest.raises(ValueError):
        matmul_bf16_reduce_scatter(a, b, [buf.data_ptr()], 100, 64, dst_f32=True)   # not % 32
    with pytest.raises(ValueError):
        matmul_bf16_reduce_scatter(a, b, [buf.data_ptr()], 128, 64, dst_f32=True)   # does not cover M


@pytest.mark.parametrize("M,K,N", [(64, 14336, 4096), (16, 4096, 1024), (128, 2048, 520),
                                    (100, 1024, 200), (128, 512, 8192)])
def test_short_problems_use_narrow_tiles_and_stay_exact(M, K, N):
    """Up to 128 rows the default configuration runs single-CTA tiles, and when 256-column
    tiles would leave most SMs idle the launcher narrows them (down to 64 columns).  The result
    must not depend on the tile width: same accumulation order per element, so the CTA-pair
    kernel (always 256 wide) gives the same bits."""
    a, b = problem(M, K, N, seed=M + K + N + 1)
    ref32 = orc.matmul_f32(a, b)
    ad, bd = a.to(DEV), b.to(DEV)
    big = torch.full((M + 2, N + 16), float("nan"), dtype=torch.bfloat16, device=DEV)
    out = big[1:M + 1, 8:8 + N]
    # (whole-K tiles are what this test is about: keep the deep shapes off the cluster plan)
    before = _lib.set_splitk_cluster_sum(False)
    try:
        matmul_bf16(ad, bd, out=out)                   # default: cta_group 1, narrowed tiles
    finally:
        _lib.set_splitk_cluster_sum(before)
    rep = orc.compare(out.cpu(), ref32.to(torch.bfloat16), ref32)
    assert rep.ok, str(rep)
    wide = matmul_bf16(ad, bd, config=TileConfig(2, 64, 0, 8))
    assert torch.equal(out.contiguous().view(torch.int16), wide.view(torch.int16))
    guard = big.clone()
    guard[1:M + 1, 8:8 + N] = float("nan")
    assert torch.isnan(guard).all(), "wrote outside the output"
