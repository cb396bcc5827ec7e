"""Host-buffer pipeline (``sgl_host_pipeline_*``): host tensors in, host tensor out, through the
C ABI.  The result must be bit-identical to the device-resident operator on the same inputs
(the pipeline only reorders the work into column windows and row blocks, and both of those are
bit-exact re-tilings of the same per-element arithmetic), and within the stated tolerance of
the fp32 oracle."""
import pytest
import torch

import swiglu_oracle as orc
from swiglu_fused_b200 import _lib, matmul_fused_swiglu, matmul_silu_mul
from swiglu_fused_b200.host_pipeline import HostPipeline, HostPipelineSiluMul

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(autouse=True)
def _device_status_clean():
    yield
    torch.cuda.synchronize()
    _lib.device_status()


def fused_problem(M, K, N, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((M, K), generator=g).to(torch.bfloat16)
    w = (torch.randn((K, 2 * N), generator=g) * K ** -0.5).to(torch.bfloat16)
    return x, w


def same_bits(a, b):
    return torch.equal(a.view(torch.int16), b.view(torch.int16))


@pytest.mark.parametrize("M,K,N,kw", [
    (4096, 512, 2048, {}),                                   # defaults: 8 windows of 256
    (5000, 264, 1288, {}),                                   # ragged rows and last window
    (3000, 128, 512, {"first_rows": 1000, "block_rows": 1024, "windows": 2}),
    (300, 64, 136, {}),                                      # smaller than one block
    (2048, 256, 1024, {"first_rows": 2048}),                 # phase 1 only
    (2048, 256, 1024, {"windows": 1}),                       # whole weight, then rows
])
def test_fused_pipeline_matches_device_operator(M, K, N, kw):
    x, w = fused_problem(M, K, N, seed=M + N)
    want = matmul_fused_swiglu(x.to(DEV), w.to(DEV)).cpu()
    rep = orc.compare(want, orc.fused_swiglu_f32(x, w).to(torch.bfloat16),
                      orc.fused_swiglu_f32(x, w))
    assert rep.ok, rep
    pipe = HostPipeline(M, K, N, device=DEV, **kw)
    xh, wh = x.pin_memory(), w.pin_memory()
    hh = torch.full((M, N), float("nan"), dtype=torch.bfloat16).pin_memory()
    n0 = _lib.kernel_launches()
    pipe.run(xh, wh, hh)
    assert _lib.kernel_launches() - n0 == pipe.launches_per_run
    assert same_bits(hh, want)
    # second pass on the resident weight: row blocks only
    hh.fill_(float("nan"))
    n0 = _lib.kernel_launches()
    pipe.run(xh, None, hh, copy_weight=False)
    assert _lib.kernel_launches() - n0 == pipe.launches_per_run_no_weight
    assert same_bits(hh, want)
    assert pipe.h2d_bytes == 2 * (M * K + 2 * K * N)
    assert pipe.h2d_bytes_no_weight == 2 * M * K
    assert pipe.d2h_bytes == 2 * M * N
    assert pipe.device_bytes == 2 * (M * K + 2 * K * N + M * N)
    pipe.close()


def test_fused_pipeline_pitched_and_pageable_host_buffers():
    M, K, N = 1536, 136, 520
    x, w = fused_problem(M, K, N, seed=3)
    want = matmul_fused_swiglu(x.to(DEV), w.to(DEV)).cpu()
    # rows wider than the data: the pitch is honoured on the way in and on the way out
    xb = torch.zeros((M, K + 24), dtype=torch.bfloat16)
    wb = torch.zeros((K, 2 * N + 8), dtype=torch.bfloat16)
    hb = torch.full((M, N + 16), 7.0, dtype=torch.bfloat16)
    xb[:, :K] = x
    wb[:, :2 * N] = w
    pipe = HostPipeline(M, K, N, device=DEV)
    pipe.run(xb[:, :K], wb[:, :2 * N], hb[:, :N])          # pageable memory: slower, still right
    assert same_bits(hb[:, :N].contiguous(), want)
    assert (hb[:, N:] == 7.0).all(), "wrote beyond the N columns of a pitched host row"


@pytest.mark.parametrize("M,K,N", [(4096, 256, 2048), (2500, 72, 776)])
def test_silu_mul_pipeline_matches_device_operator(M, K, N):
    g = torch.Generator().manual_seed(M)
    x = torch.randn((M, K), generator=g).to(torch.bfloat16)
    wg = (torch.randn((K, N), generator=g) * K ** -0.5).to(torch.bfloat16)
    up = torch.randn((M, N), generator=g).to(torch.bfloat16)
    want = matmul_silu_mul(x.to(DEV), wg.to(DEV), up.to(DEV)).cpu()
    ref32 = orc.silu_mul_f32(x, wg, up)
    assert orc.compare(want, ref32.to(torch.bfloat16), ref32).ok
    pipe = HostPipelineSiluMul(M, K, N, device=DEV)
    hh = torch.full((M, N), float("nan"), dtype=torch.bfloat16).pin_memory()
    pipe.run(x.pin_memory(), wg.pin_memory(), up.pin_memory(), hh)
    assert same_bits(hh, want)
    hh.fill_(float("nan"))
    pipe.run(x.pin_memory(), None, up.pin_memory(), hh, copy_weight=False)
    assert same_bits(hh, want)
    assert pipe.h2d_bytes == 2 * (M * K + K * N + M * N)


def test_pipeline_argument_errors():
    with pytest.raises(ValueError):
        HostPipeline(0, 64, 64, device=DEV)
    with pytest.raises(ValueError):
        HostPipeline(256, 64, 68, device=DEV)               # N not a multiple of 8
    with pytest.raises(ValueError):
        HostPipeline(256, 64, 64, device=DEV, windows=65)
    pipe = HostPipeline(256, 64, 64, device=DEV)
    x = torch.zeros((256, 64), dtype=torch.bfloat16)
    w = torch.zeros((64, 128), dtype=torch.bfloat16)
    h = torch.zeros((256, 64), dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        pipe.run(x.to(DEV), w, h)                           # device tensor where host is expected
    with pytest.raises(ValueError):
        pipe.run(x, w[:, :64], h)                           # wrong weight shape
    with pytest.raises(ValueError):
        pipe.run(x.float(), w, h)
    pipe.close()
    with pytest.raises(RuntimeError):
        pipe.run(x, w, h)


def test_shared_weight_pipeline_with_a_group_of_one():
    """The shared-weight form with world = 1: the region is caller memory (here a torch tensor
    standing in for a symmetric allocation), the double-buffered weight alternates between runs,
    nothing is pushed or waited for, and the result is the device operator's, bit for bit."""
    import ctypes as C

    M, K, N = 3000, 264, 1288
    x, w = fused_problem(M, K, N, seed=77)
    want = matmul_fused_swiglu(x.to(DEV), w.to(DEV)).cpu()
    lib = _lib.load()
    nbytes = lib.sgl_host_pipeline_shared_bytes(_lib.FORM_FUSED_SWIGLU, N, K)
    assert nbytes >= 2 * (2 * K * 2 * N)
    region = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    handle = C.c_void_p()
    ptrs = (C.c_void_p * 1)(region.data_ptr())
    _lib.check(lib.sgl_host_pipeline_create_shared(_lib.FORM_FUSED_SWIGLU, M, N, K, 0, 0, 0, None,
                                                   1, 0, ptrs, C.byref(handle)))
    xh, wh = x.pin_memory(), w.pin_memory()
    hh = torch.full((M, N), float("nan"), dtype=torch.bfloat16).pin_memory()
    try:
        # copy_weight = 0 before any weight was copied is refused
        rc = lib.sgl_host_pipeline_run(handle, xh.data_ptr(), K, None, 0, None, 0, hh.data_ptr(),
                                       N, 0)
        assert rc == -10, lib.sgl_last_error()
        for i in range(3):                       # parities 0, 1, 0
            hh.fill_(float("nan"))
            _lib.check(lib.sgl_host_pipeline_run(handle, xh.data_ptr(), K, wh.data_ptr(), 2 * N,
                                                 None, 0, hh.data_ptr(), N, 1))
            assert same_bits(hh, want), i
        hh.fill_(float("nan"))
        _lib.check(lib.sgl_host_pipeline_run(handle, xh.data_ptr(), K, None, 0, None, 0,
                                             hh.data_ptr(), N, 0))
        assert same_bits(hh, want)
    finally:
        lib.sgl_host_pipeline_destroy(handle)


def test_pipeline_calls_leave_the_current_device_alone():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs to tell the devices apart")
    M, K, N = 1024, 128, 256
    x, w = fused_problem(M, K, N, seed=5)
    pipe = HostPipeline(M, K, N, device="cuda:1")
    hh = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    torch.cuda.set_device(0)
    pipe.run(x.pin_memory(), w.pin_memory(), hh)
    assert torch.cuda.current_device() == 0
    pipe.close()
    assert torch.cuda.current_device() == 0


def test_shared_weight_pipeline_reports_a_peer_that_never_sends():
    """Two ranks' regions on one GPU, but only rank 0 ever runs: its launch over rank 1's slice
    waits for a flag that nobody raises.  With the wait limit set to 50 ms the one-thread wait
    kernel gives up, `run` returns a device-status error naming the missing rank - nothing
    hangs - and the context keeps computing correct results afterwards."""
    import ctypes as C

    M, K, N = 1024, 128, 512
    x, w = fused_problem(M, K, N, seed=91)
    lib = _lib.load()
    nbytes = lib.sgl_host_pipeline_shared_bytes(_lib.FORM_FUSED_SWIGLU, N, K)
    regions = [torch.zeros(nbytes, dtype=torch.uint8, device=DEV) for _ in range(2)]
    ptrs = (C.c_void_p * 2)(*[r.data_ptr() for r in regions])
    handle = C.c_void_p()
    _lib.check(lib.sgl_host_pipeline_create_shared(_lib.FORM_FUSED_SWIGLU, M, N, K, 0, 0, 0, None,
                                                   2, 0, ptrs, C.byref(handle)))
    xh, wh = x.pin_memory(), w.pin_memory()
    hh = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    _lib.set_wait_limit_ns(50_000_000)
    try:
        rc = lib.sgl_host_pipeline_run(handle, xh.data_ptr(), K, wh.data_ptr(), 2 * N, None, 0,
                                       hh.data_ptr(), N, 1)
        assert rc == -9, (rc, lib.sgl_last_error())           # SGL_ERR_DEVICE_STATUS
        msg = lib.sgl_last_error().decode()
        assert "rank 1" in msg and "did not arrive" in msg
        # rank 0's own slice did reach the "peer": its flag is raised in rank 1's region
        flags = regions[1][-1024:].view(torch.int32)
        assert int(flags[0]) == 1
    finally:
        _lib.set_wait_limit_ns(2_000_000_000)
        lib.sgl_host_pipeline_destroy(handle)
    torch.cuda.synchronize()
    _lib.device_status()                                      # the record was cleared by run
    want = matmul_fused_swiglu(x.to(DEV), w.to(DEV))
    ref32 = orc.fused_swiglu_f32(x, w)
    assert orc.compare(want.cpu(), ref32.to(torch.bfloat16), ref32).ok
