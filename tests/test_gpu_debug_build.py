"""The self-checking build of the library (``-DSGL_DEBUG``), used where compute-sanitizer is not
available: every TMA coordinate is checked against the 16-byte rule and the tensor's extent
before the copy is issued, and the kernel's roles count their work.  A violation would be
RECORDED in the status words (nothing traps or faults); here no launch of the shape ladder may
record one, the role counters must balance (k-blocks produced = k-blocks consumed = what the
schedule says, tiles finished by the epilogue = tiles of the schedule), and the results must
equal the normal library's bit for bit.  Runs in a child process because a process loads one
copy of the library.
"""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu

CHILD = textwrap.dedent('''
    import ctypes as C, sys
    import numpy as np, torch
    from swiglu_fused_b200 import _lib, matmul_bf16, matmul_fused_swiglu, matmul_silu_mul, TileConfig
    from swiglu_fused_b200.workloads import make_inputs
    lib = _lib.load()
    has_counts = hasattr(lib, "sgl_debug_counts")
    if has_counts:
        lib.sgl_debug_counts.restype = C.c_int
        lib.sgl_debug_counts.argtypes = [C.POINTER(C.c_ulonglong)]
    dev = "cuda:0"
    sms = _lib.query(_lib.QUERY_SM_COUNT)
    out = {}
    shapes = [(64, 64, 128), (200, 136, 264), (1000, 264, 1160), (512, 1024, 2048), (2048, 512, 640)]
    for (M, K, N) in shapes:
        for cg, bk, wide in ((1, 64, 0), (2, 128, 0), (2, 64, 0), (1, 128, 0), (2, 64, 1)):
            if cg == 2 and M <= 128:
                continue
            cfg = TileConfig(cg, bk, 0, 4, 0, 0, 0, wide)
            inp = make_inputs(M, K, N, form="fused_swiglu", seed=M + N)
            x, w = inp["x"].to(dev), inp["w"].to(dev)
            h = matmul_fused_swiglu(x, w, config=cfg)
            torch.cuda.synchronize()
            _lib.device_status()              # raises if a coordinate check (or a wait) failed
            if has_counts:
                buf = (C.c_ulonglong * (512 * 4))()
                _lib.check(lib.sgl_debug_counts(buf))
                c = np.frombuffer(buf, dtype=np.uint64).reshape(512, 4)
                tiles = -(-M // (128 * cg)) * -(-N // (256 if wide else 128))
                clusters = min(sms // cg, tiles)
                kb = -(-K // bk)
                for cl in range(clusters):
                    mine = len(range(cl, tiles, clusters))
                    lead = cl * cg
                    assert c[lead, 1] == mine * kb, ("consumed", M, K, N, cg, bk, cl, c[lead])
                    for r in range(cg):
                        assert c[lead + r, 0] == mine * kb, ("produced", M, K, N, cg, bk, cl, r)
                        assert c[lead + r, 2] == mine, ("tiles", M, K, N, cg, bk, cl, r)
            out[(M, K, N, cg, bk, wide)] = h.cpu()
        inp = make_inputs(M, K, N, form="silu_mul", seed=M)
        x, wg = inp["x"].to(dev), inp["w_gate"].to(dev)
        up = (x @ inp["w_up"].to(dev))
        out[(M, K, N, "silu_mul")] = matmul_silu_mul(x, wg, up).cpu()
        out[(M, K, N, "gemm")] = matmul_bf16(x, wg).cpu()
        torch.cuda.synchronize()
        _lib.device_status()
    # split-K with the K ranges summed in thread-block clusters (explicit and chosen ranges)
    from swiglu_fused_b200.ops import matmul_bf16_splitk
    g = torch.Generator().manual_seed(5)
    a = torch.randn((72, 2048), generator=g).to(torch.bfloat16).to(dev)
    b = (torch.randn((2048, 520), generator=g) * 2048 ** -0.5).to(torch.bfloat16).to(dev)
    for splits in (4, 0):
        n0 = _lib.kernel_launches()
        out[("splitk", splits)] = matmul_bf16_splitk(a, b, splits=splits).cpu()
        assert _lib.kernel_launches() - n0 == 1, "the K ranges were not summed in their clusters"
        _lib.device_status()
    if hasattr(lib, "sgl_debug_cluster_sum_missing_arrivals"):
        # the cluster sum's bounded wait: its barrier is told to expect one arrival that never
        # comes, every CTA's wait runs out after 20 ms, the launch returns, the status names
        # the wait, and the next launch computes the right product again
        lib.sgl_debug_cluster_sum_missing_arrivals.restype = C.c_int
        lib.sgl_debug_cluster_sum_missing_arrivals.argtypes = [C.c_int]
        _lib.set_wait_limit_ns(20_000_000)
        _lib.check(lib.sgl_debug_cluster_sum_missing_arrivals(1))
        matmul_bf16_splitk(a, b, splits=4)
        torch.cuda.synchronize()
        try:
            _lib.device_status()
            raise SystemExit("the missing arrival went unnoticed")
        except _lib.SglError as e:
            assert "106" in str(e), str(e)
        _lib.check(lib.sgl_debug_cluster_sum_missing_arrivals(0))
        _lib.set_wait_limit_ns(2_000_000_000)
        again = matmul_bf16_splitk(a, b, splits=4).cpu()
        _lib.device_status()
        assert torch.equal(again.view(torch.int16), out[("splitk", 4)].view(torch.int16))
        print("cluster-sum wait timed out as told")
    torch.save(out, sys.argv[1])
    print("counts" if has_counts else "plain", len(out))
''')


def _run(lib_path, out_path):
    env = dict(os.environ)
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    if lib_path:
        env["SWIGLU_B200_LIB"] = lib_path
    else:
        env.pop("SWIGLU_B200_LIB", None)
    proc = subprocess.run([sys.executable, "-c", CHILD, out_path], env=env, capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-1500:] + proc.stderr[-3000:]
    return proc.stdout


def test_debug_build_records_nothing_and_matches_the_normal_library(tmp_path):
    import torch

    from swiglu_fused_b200 import build

    debug_lib = build.DEBUG_LIB_PATH
    if not os.path.exists(debug_lib):
        try:
            build.build_debug_library()
        except RuntimeError as e:
            pytest.skip(f"debug library not built and no compiler here: {e}")
    a, b = str(tmp_path / "debug.pt"), str(tmp_path / "normal.pt")
    said = _run(debug_lib, a)
    assert "cluster-sum wait timed out as told" in said and "counts" in said, said
    assert _run(None, b).startswith("plain")
    da, db = torch.load(a), torch.load(b)
    assert da.keys() == db.keys() and len(da) > 20
    for k in da:
        assert torch.equal(da[k].view(torch.int16), db[k].view(torch.int16)), k


def test_launch_tracing_is_off_by_default_and_on_by_environment():
    """SGL_LOG=1 writes one line per kernel launch to stderr (form, shape, tile entry, grid);
    SGL_NVTX=1 wraps the launches in NVTX ranges (harmless without a profiler); by default the
    library prints nothing."""
    code = textwrap.dedent('''
        import torch
        from swiglu_fused_b200 import matmul_fused_swiglu, _lib
        x = torch.randn((300, 128), device="cuda:0").to(torch.bfloat16)
        w = torch.randn((128, 512), device="cuda:0").to(torch.bfloat16)
        matmul_fused_swiglu(x, w)
        torch.cuda.synchronize()
        _lib.device_status()
        print("done")
    ''')
    env = dict(os.environ)
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    for extra, expect in (({}, False), ({"SGL_LOG": "1", "SGL_NVTX": "1"}, True)):
        e = dict(env)
        e.pop("SGL_LOG", None)
        e.pop("SGL_NVTX", None)
        e.update(extra)
        proc = subprocess.run([sys.executable, "-c", code], env=e, capture_output=True, text=True,
                              timeout=300)
        assert proc.returncode == 0 and "done" in proc.stdout, proc.stderr[-2000:]
        lines = [ln for ln in proc.stderr.splitlines() if ln.startswith("[libswiglu_b200] launch")]
        assert bool(lines) == expect, proc.stderr[-2000:]
        if expect:
            assert "fused_swiglu 300x256x128" in lines[0] and "grid=" in lines[0], lines[0]
