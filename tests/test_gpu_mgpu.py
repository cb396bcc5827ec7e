"""Single-process multi-GPU launcher (``sgl_mgpu_*``) through the C ABI.

Every mode must reproduce, bit for bit, what one launch over the whole problem gives: row
shards and column windows re-tile the same per-element arithmetic.  A device may be listed
twice in a group, so the sharding logic is exercised on one GPU as well; with two or more GPUs
the same tests run across real devices (peer stores included)."""
import pytest
import torch

import swiglu_oracle as orc
from swiglu_fused_b200 import _lib, matmul_fused_swiglu
from swiglu_fused_b200.mgpu import DeviceGroup

pytestmark = pytest.mark.gpu


def groups():
    out = [[0], [0, 0], [0, 0, 0]]
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if n >= 2:
        out.append(list(range(min(n, 8))))
        out.append([1, 0])
    return out


@pytest.fixture(autouse=True)
def _device_status_clean():
    yield
    for d in range(torch.cuda.device_count()):
        with torch.cuda.device(d):
            torch.cuda.synchronize()
            _lib.device_status()


def problem(M, K, N, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((M, K), generator=g).to(torch.bfloat16)
    w = (torch.randn((K, 2 * N), generator=g) * K ** -0.5).to(torch.bfloat16)
    return x, w


def same_bits(a, b):
    return torch.equal(a.cpu().view(torch.int16), b.cpu().view(torch.int16))


def sync_all(devs):
    for d in set(devs):
        torch.cuda.synchronize(d)


@pytest.mark.parametrize("devs", groups())
@pytest.mark.parametrize("M,K,N", [(1024, 256, 512), (1300, 136, 776), (200, 64, 128)])
def test_all_modes_match_one_launch(devs, M, K, N):
    x, w = problem(M, K, N, seed=M + N + len(devs))
    want = matmul_fused_swiglu(x.to("cuda:0"), w.to("cuda:0"))
    ref32 = orc.fused_swiglu_f32(x, w)
    assert orc.compare(want.cpu(), ref32.to(torch.bfloat16), ref32).ok
    grp = DeviceGroup(devs)
    n = len(devs)
    assert len(grp) == n
    ws = [w.to(f"cuda:{d}") for d in devs]

    # rows
    xs, hs, ranges = [], [], []
    for r, d in enumerate(devs):
        b, c = grp.shard(M, 256, r)
        ranges.append((b, c))
        xs.append(x[b:b + c].to(f"cuda:{d}"))
        hs.append(torch.full((c, N), float("nan"), dtype=torch.bfloat16, device=f"cuda:{d}"))
    grp.fused_swiglu("m_shard", xs, ws, hs, M, N, K)
    sync_all(devs)
    for (b, c), hr in zip(ranges, hs):
        assert same_bits(hr, want[b:b + c])

    # columns, local blocks (one pitch for all devices: views of equally wide buffers)
    xf = [x.to(f"cuda:{d}") for d in devs]
    width = max(grp.shard(N, 128, r)[1] for r in range(n))
    hs, ranges = [], []
    for r, d in enumerate(devs):
        b, c = grp.shard(N, 128, r)
        ranges.append((b, c))
        buf = torch.full((M, max(width, 8)), float("nan"), dtype=torch.bfloat16, device=f"cuda:{d}")
        hs.append(buf[:, :c])
    grp.fused_swiglu("n_shard", xf, ws, hs, M, N, K)
    sync_all(devs)
    for (b, c), hr in zip(ranges, hs):
        assert same_bits(hr, want[:, b:b + c])

    # columns, gathered into a full h on every device by the kernels' epilogues
    hs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=f"cuda:{d}") for d in devs]
    n0 = _lib.kernel_launches()
    grp.fused_swiglu("n_shard_gather", xf, ws, hs, M, N, K)
    launched = _lib.kernel_launches() - n0
    sync_all(devs)
    assert launched == sum(1 for r in range(n) if grp.shard(N, 128, r)[1] > 0)
    for hr in hs:
        assert same_bits(hr, want)
    grp.close()


def test_gather_twice_in_a_row_on_side_streams():
    devs = groups()[-1] if torch.cuda.device_count() >= 2 else [0, 0]
    M, K, N = 2048, 512, 1024
    x, w = problem(M, K, N, seed=11)
    want = matmul_fused_swiglu(x.to("cuda:0"), w.to("cuda:0"))
    grp = DeviceGroup(devs)
    xf = [x.to(f"cuda:{d}") for d in devs]
    ws = [w.to(f"cuda:{d}") for d in devs]
    hs = [torch.zeros((M, N), dtype=torch.bfloat16, device=f"cuda:{d}") for d in devs]
    sync_all(devs)
    streams = {d: torch.cuda.Stream(d) for d in set(devs)}
    for _ in range(2):
        for d, s in streams.items():
            torch.cuda.set_stream(s)
        try:
            grp.fused_swiglu("n_shard_gather", xf, ws, hs, M, N, K)
            # stream order alone must make the whole h visible on every stream
            outs = []
            for d, hr in zip(devs, hs):
                with torch.cuda.stream(streams[d]):
                    outs.append(hr.clone())
        finally:
            for d in streams:
                torch.cuda.set_stream(torch.cuda.default_stream(d))
        sync_all(devs)
        for o in outs:
            assert same_bits(o, want)
        for hr in hs:
            hr.zero_()
        sync_all(devs)
    grp.close()


def test_argument_errors():
    with pytest.raises(ValueError):
        DeviceGroup([])
    with pytest.raises(ValueError):
        DeviceGroup([0] * 9)
    with pytest.raises(ValueError):
        DeviceGroup([torch.cuda.device_count()])
    grp = DeviceGroup([0, 0])
    x, w = problem(512, 64, 256, seed=1)
    xd, wd = x.to("cuda:0"), w.to("cuda:0")
    h = torch.empty((512, 256), dtype=torch.bfloat16, device="cuda:0")
    with pytest.raises(ValueError):
        grp.fused_swiglu("rows", [xd, xd], [wd, wd], [h, h], 512, 256, 64)
    with pytest.raises(ValueError):
        grp.fused_swiglu("n_shard_gather", [xd], [wd], [h], 512, 256, 64)
    with pytest.raises(ValueError):
        grp.fused_swiglu("n_shard_gather", [xd, xd], [wd, wd], [h, h.cpu()], 512, 256, 64)
    with pytest.raises(ValueError):
        grp.fused_swiglu("m_shard", [xd, xd], [wd, wd], [h, h], 512, 256, 64)   # x is not a shard
    grp.close()
    with pytest.raises(RuntimeError):
        grp.fused_swiglu("n_shard_gather", [xd, xd], [wd, wd], [h, h], 512, 256, 64)
