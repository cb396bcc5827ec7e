"""The allocation-free split-K entry point, ``sgl_matmul_bf16_splitk_static``.

Some users of this library cannot give it scratch memory: a plug-in inside a server that has
already handed the whole GPU to its own pool, or a decode loop where ``cudaMalloc`` is banned
because it stalls the device.  For them the partial tiles of the split-K down projection live
in a fixed 8 MiB array inside the library.  This file calls that entry point directly through
the C ABI (ctypes, raw pointers) and checks it against ``sgl_matmul_bf16_splitk`` fed with
caller-owned scratch: same arithmetic, so the outputs must agree bit for bit, which is well
inside the usual tolerance (>= 99.9 % of elements within 1 bf16 ulp).  Two different problems
are run back to back to show that what the first call leaves in the shared array does not leak
into the second.  The file sorts last on purpose, and it works the same whether it runs alone
in a fresh process or after every other test.
"""
import ctypes as C

import pytest
import torch

import swiglu_oracle as orc
from swiglu_fused_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
STATIC_BYTES = 8 << 20


def _problem(M, K, N, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn((M, K), generator=g).to(torch.bfloat16)
    b = (torch.randn((K, N), generator=g) * K ** -0.5).to(torch.bfloat16)
    return a, b


def _call_static(lib, a, b, c, splits):
    M, K = a.shape
    N = b.shape[1]
    return lib.sgl_matmul_bf16_splitk_static(
        a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, a.stride(0), b.stride(0), c.stride(0),
        splits, None, torch.cuda.current_stream().cuda_stream)


def _call_with_scratch(lib, a, b, c, splits):
    M, K = a.shape
    N = b.shape[1]
    need = lib.sgl_matmul_bf16_splitk_scratch_bytes(M, N, K, splits)
    assert 0 < need <= STATIC_BYTES
    scratch = torch.empty(need, dtype=torch.uint8, device=a.device)
    rc = lib.sgl_matmul_bf16_splitk(
        a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, a.stride(0), b.stride(0), c.stride(0),
        splits, scratch.data_ptr(), need, None, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()          # scratch stays alive until the kernels are done
    return rc


def test_static_scratch_entry_point_matches_caller_scratch_twice_in_a_row():
    lib = _lib.load()
    # first problem fills the whole 8 MiB (8 ranges x 64 rows x 4096 columns x 4 bytes);
    # the second is smaller and uses a different number of ranges
    cases = [(64, 14336, 4096, 8, 101), (48, 2048, 1024, 4, 202)]
    for M, K, N, splits, seed in cases:
        a_h, b_h = _problem(M, K, N, seed)
        a, b = a_h.to(DEV), b_h.to(DEV)
        want = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
        assert _call_with_scratch(lib, a, b, want, splits) == 0, lib.sgl_last_error()

        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = _call_static(lib, a, b, got, splits)
        assert rc == 0, lib.sgl_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before      # torch's allocator was not touched
        rep = orc.compare(got, want)
        assert rep.ok and rep.frac_within_1ulp >= 0.999, str(rep)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        # and both are the product: against the fp32 reference
        ref32 = orc.matmul_f32(a_h, b_h)
        assert orc.compare(got.cpu(), ref32.to(torch.bfloat16), ref32).ok
    _lib.device_status()


def test_automatic_split_count_gives_way_to_the_fixed_scratch():
    """splits = 0 lets the library choose.  For 128 x 4096 x 14336 the wave-filling choice is
    9 ranges (18.9 MB of partial tiles), which the 8 MiB array cannot hold: the automatic
    choice must come down to the 4 ranges that fit exactly, and give the same bits as the
    caller-scratch entry point told to use 4.  The driver's view of device memory must not
    move either (a cudaMalloc inside the library would not show in torch's own counters)."""
    lib = _lib.load()
    # (with the K ranges summed in thread-block clusters the library would not touch the scratch
    # at all for this problem and would choose its ranges differently; this test is about the
    # two-kernel form, which every problem whose clusters do not fit still takes)
    before = _lib.set_splitk_cluster_sum(False)
    try:
        _automatic_split_count_gives_way(lib)
    finally:
        _lib.set_splitk_cluster_sum(before)


def _automatic_split_count_gives_way(lib):
    M, K, N = 128, 14336, 4096
    assert lib.sgl_matmul_bf16_splitk_scratch_bytes(M, N, K, 0) > STATIC_BYTES   # unconstrained
    assert lib.sgl_matmul_bf16_splitk_scratch_bytes(M, N, K, 4) == STATIC_BYTES
    a_h, b_h = _problem(M, K, N, 303)
    a, b = a_h.to(DEV), b_h.to(DEV)
    want = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
    assert _call_with_scratch(lib, a, b, want, 4) == 0, lib.sgl_last_error()
    got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    _call_static(lib, a, b, got, 0)          # first use resolves the array's address
    torch.cuda.synchronize()
    got.fill_(float("nan"))
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    rc = _call_static(lib, a, b, got, 0)
    assert rc == 0, lib.sgl_last_error()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    ref32 = orc.matmul_f32(a_h, b_h)
    assert orc.compare(got.cpu(), ref32.to(torch.bfloat16), ref32).ok
    _lib.device_status()


def test_static_scratch_entry_point_rejects_what_does_not_fit():
    lib = _lib.load()
    M, K, N, splits = 256, 4096, 4096, 8          # 8 x 256 x 4096 x 4 = 32 MiB > 8 MiB
    a = torch.zeros((M, K), dtype=torch.bfloat16, device=DEV)
    b = torch.zeros((K, N), dtype=torch.bfloat16, device=DEV)
    c = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
    n0 = _lib.kernel_launches()
    rc = _call_static(lib, a, b, c, splits)
    assert rc == -10
    msg = lib.sgl_last_error().decode()
    assert "8388608" in msg and "scratch" in msg
    assert _lib.kernel_launches() == n0            # nothing was launched
    torch.cuda.synchronize()
    assert bool((c == 7.0).all())                  # and the output was left alone


def test_static_entry_point_with_the_cluster_sum_allocates_nothing_either():
    """Left to choose its K ranges, the static entry point sums them in thread-block clusters
    where they fit: no scratch traffic, still no allocation, and the product within the
    tolerance of the fp32 reference."""
    lib = _lib.load()
    _lib.set_splitk_cluster_sum(True)
    M, K, N = 128, 14336, 4096
    a_h, b_h = _problem(M, K, N, 404)
    a, b = a_h.to(DEV), b_h.to(DEV)
    got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert _call_static(lib, a, b, got, 0) == 0, lib.sgl_last_error()
    torch.cuda.synchronize()
    got.fill_(float("nan"))
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    n0 = _lib.kernel_launches()
    assert _call_static(lib, a, b, got, 0) == 0, lib.sgl_last_error()
    torch.cuda.synchronize()
    assert _lib.kernel_launches() - n0 == 1
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    ref32 = orc.matmul_f32(a_h, b_h)
    assert orc.compare(got.cpu(), ref32.to(torch.bfloat16), ref32).ok
    _lib.device_status()
