"""Host-side helpers of ``bench.py`` that need no GPU: the rotating candidate order, the reader
of the committed DRAM-traffic summary, and the choice of clock samples around a timed region."""
import importlib.util
import os
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    argv, sys.argv = sys.argv, ["bench.py"]
    try:
        spec.loader.exec_module(mod)
    finally:
        sys.argv = argv
    return mod


def test_traffic_summary_is_keyed_by_problem_and_tile_entry(bench):
    from swiglu_fused_b200 import TileConfig

    got = bench.profiled_traffic("fused_swiglu", 32768, 12288, 3072, TileConfig(2, 128, 0, 16, 0, 26))
    assert got is not None and 2.0e9 < got < 2.5e9
    slabs = bench.profiled_traffic("fused_swiglu", 32768, 12288, 3072,
                                   TileConfig(2, 128, 0, 16, 0, 26, 48))
    assert slabs is not None and slabs > got                 # the slab order reads more, not less
    # another tile entry, another shape or another form: no figure rather than a wrong one
    assert bench.profiled_traffic("fused_swiglu", 32768, 12288, 3072, TileConfig(2, 64, 0, 16)) is None
    assert bench.profiled_traffic("fused_swiglu", 4096, 12288, 3072, TileConfig(2, 128, 0, 16)) is None
    assert bench.profiled_traffic("silu_mul", 32768, 12288, 3072, TileConfig(2, 128, 0, 16)) is None


def test_spread_reports_median_min_max(bench):
    assert bench.spread([3.0, 1.0, 2.0]) == {"median": 2.0, "min": 1.0, "max": 3.0}


def test_clock_sampler_uses_samples_inside_the_region_or_says_which_it_used(bench):
    s = bench.ClockSampler(0)
    now = time.perf_counter()
    s.max_mhz = 1965
    s.t_begin = now - 0.010
    s.samples = [(now - 0.020, 1500, 0x4), (now - 0.008, 1400, 0x4), (now - 0.004, 1300, 0x0)]
    s.ready.set()
    s.join = lambda timeout=None: None            # the thread was never started
    out = s.stop()
    assert out["samples"] == 2 and out["sm_mhz"] in (1300, 1400) and out["sm_min_mhz"] == 1300
    assert out["reasons"] == ["sw_power_cap"] and out["sampled"].startswith("inside")
    # a region shorter than one query: the neighbours stand in, and the record says so
    s2 = bench.ClockSampler(0)
    now = time.perf_counter()
    s2.max_mhz = 1965
    s2.t_begin = now - 0.001
    s2.samples = [(now - 0.030, 1965, 0), (now - 0.020, 1950, 0), (now - 0.010, 1940, 0)]
    s2.join = lambda timeout=None: None
    out2 = s2.stop()
    assert out2["samples"] == 2 and out2["sm_mhz"] in (1940, 1950)
    assert out2["sampled"].startswith("adjacent")
    s3 = bench.ClockSampler(0)
    s3.join = lambda timeout=None: None
    assert s3.stop()["sm_mhz"] is None


def test_peaks_come_from_the_measured_file_or_the_stated_fallback(bench):
    p = bench.load_peaks()
    assert p["tflops_burst"] >= p["tflops_sustained"] > 1000 and p["hbm_gbs"] > 5000
    assert p["source"].startswith(("measured", "fallback"))
