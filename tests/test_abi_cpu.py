"""Host-side checks of the C ABI that need no GPU: the library loads, exports
every symbol the header declares, validates arguments before touching a device,
and its host logic (tile table, tile order, shard ranges) is right."""
import ctypes as C
import os
import re

import pytest

from swiglu_fused_b200 import _lib
from swiglu_fused_b200._lib import SglConfig, TileConfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "swiglu_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sgl_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_functions()
    assert len(names) >= 13
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert sorted(_lib.EXPORTED_SYMBOLS) == names
    assert lib.sgl_version() >= 100


def test_missing_library_is_a_loud_error(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setenv("SWIGLU_B200_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()
    monkeypatch.delenv("SWIGLU_B200_LIB")
    monkeypatch.setattr(_lib, "_lib", None)
    _lib.load()


# Arguments are validated before any CUDA call, so these work without a device.
BUF = (C.c_uint8 * 4096)()
P = (C.addressof(BUF) + 15) // 16 * 16


@pytest.mark.parametrize("kwargs,code,needle", [
    (dict(x=0), -1, "x is NULL"),
    (dict(h=P + 2), -4, "16-byte"),
    (dict(M=0), -2, ">= 1"),
    (dict(K=12), -2, "multiples of 8"),
    (dict(ldx=8), -3, "smaller"),
    (dict(ldh=68), -3, "multiple of 8"),
    (dict(gate_col0=60), -4, "multiples of 8"),
    (dict(up_col0=-8), -10, ">= 0"),
    (dict(ldw=64), -3, "smaller"),
    (dict(cfg=SglConfig(3, 64, 0, 8, 0)), -5, "unsupported"),
    (dict(cfg=SglConfig(2, 64, 7, 8, 0)), -5, "stages"),
    (dict(cfg=SglConfig(2, 64, 0, 0, 0)), -5, "unsupported"),
])
def test_fused_argument_validation(kwargs, code, needle):
    lib = _lib.load()
    a = dict(x=P, w=P, h=P, M=64, N=64, K=64, ldx=64, ldw=128, ldh=64, up_col0=0, gate_col0=64,
             cfg=None, stream=None)
    a.update(kwargs)
    cfg = C.byref(a["cfg"]) if a["cfg"] is not None else None
    rc = lib.sgl_matmul_fused_swiglu(a["x"], a["w"], a["h"], a["M"], a["N"], a["K"], a["ldx"],
                                     a["ldw"], a["ldh"], a["up_col0"], a["gate_col0"], cfg,
                                     a["stream"])
    assert rc == code, lib.sgl_last_error()
    assert needle in lib.sgl_last_error().decode()
    with pytest.raises((ValueError, _lib.SglError)):
        _lib.check(rc)


@pytest.mark.parametrize("kwargs,code", [
    (dict(up=0), -1), (dict(w=P + 8), -4), (dict(N=0), -2), (dict(ldup=32), -3),
    (dict(ldw=60), -3),
])
def test_silu_mul_argument_validation(kwargs, code):
    lib = _lib.load()
    a = dict(x=P, w=P, up=P, h=P, M=64, N=64, K=64, ldx=64, ldw=64, ldup=64, ldh=64)
    a.update(kwargs)
    rc = lib.sgl_matmul_silu_mul(a["x"], a["w"], a["up"], a["h"], a["M"], a["N"], a["K"],
                                 a["ldx"], a["ldw"], a["ldup"], a["ldh"], None, None)
    assert rc == code, lib.sgl_last_error()


def test_tile_table_fits_shared_memory():
    for form in (_lib.FORM_SILU_MUL, _lib.FORM_FUSED_SWIGLU):
        cfgs = _lib.builtin_configs(form)
        assert len(cfgs) >= 8
        for c in cfgs:
            assert c.stages >= 2
            smem = _lib.config_smem_bytes(form, c)
            assert 0 < smem <= 227 * 1024, (form, c, smem)
            # one more stage must not fit, i.e. `stages` is the deepest ring
            if c.stages < 8:
                too_deep = TileConfig(c.cta_group, c.block_k, c.stages + 1, c.group_m)
                with pytest.raises(ValueError):
                    _lib.config_smem_bytes(form, too_deep)
    # the pair kernels at BLOCK_K=64 keep at least 5 stages in flight
    assert _lib.builtin_configs(_lib.FORM_FUSED_SWIGLU)[0].stages >= 5
    assert _lib.builtin_configs(_lib.FORM_SILU_MUL)[0].stages >= 5


def test_default_config_uses_pairs_only_when_there_are_two_row_tiles():
    assert _lib.default_config(_lib.FORM_FUSED_SWIGLU, 64, 14336, 4096).cta_group == 1
    assert _lib.default_config(_lib.FORM_FUSED_SWIGLU, 128, 14336, 4096).cta_group == 1
    assert _lib.default_config(_lib.FORM_FUSED_SWIGLU, 32768, 12288, 3072).cta_group == 2
    with pytest.raises(ValueError):
        _lib.default_config(_lib.FORM_FUSED_SWIGLU, 32768, 12290, 3072)


def test_default_config_by_problem_height():
    f = _lib.FORM_FUSED_SWIGLU
    one_row = _lib.default_config(f, 256, 14336, 4096)        # one pair-tile row: wide tiles
    assert (one_row.cta_group, one_row.block_k, one_row.wide) == (2, 64, 1)
    few = _lib.default_config(f, 512, 14336, 4096)            # a few tile rows: BLOCK_K 128
    assert (few.cta_group, few.block_k, few.wide) == (2, 128, 0)
    tall = _lib.default_config(f, 32768, 12288, 3072)
    assert (tall.cta_group, tall.block_k, tall.group_m, tall.wide) == (2, 128, 16, 0)
    assert tall.l2_hints == (2 | 2 << 2 | 1 << 4)             # x, W evict-last; h evict-first
    assert _lib.default_config(_lib.FORM_SILU_MUL, 256, 14336, 4096).wide == 0
    # wide tiles exist for the fused form on CTA pairs with BLOCK_K 64 only
    assert _lib.config_smem_bytes(f, _lib.TileConfig(2, 64, 0, 8, 0, 0, 0, 1)) <= 227 * 1024
    with pytest.raises(ValueError):
        _lib.config_smem_bytes(f, _lib.TileConfig(2, 128, 0, 8, 0, 0, 0, 1))
    with pytest.raises(ValueError):
        _lib.config_smem_bytes(_lib.FORM_MATMUL, _lib.TileConfig(2, 64, 0, 8, 0, 0, 0, 1))


def test_shared_weight_pipeline_region_size():
    lib = _lib.load()
    K, N = 3072, 12288
    n = lib.sgl_host_pipeline_shared_bytes(_lib.FORM_FUSED_SWIGLU, N, K)
    assert n == 2 * (2 * K * 2 * N) + 1024                    # two weight copies + the flag words
    assert lib.sgl_host_pipeline_shared_bytes(_lib.FORM_SILU_MUL, N, K) == 2 * (2 * K * N) + 1024
    assert lib.sgl_host_pipeline_shared_bytes(_lib.FORM_MATMUL, N, K) < 0
    assert lib.sgl_host_pipeline_shared_bytes(_lib.FORM_FUSED_SWIGLU, N + 4, K) < 0


def model_tile_coord(t, tiles_m, tiles_n, group_m):
    """Independent Python model of the GROUP_SIZE_M order."""
    per_band = group_m * tiles_n
    band = t // per_band
    first = band * group_m
    rows = min(group_m, tiles_m - first)
    r = t % per_band
    return first + r % rows, r // rows


@pytest.mark.parametrize("tiles_m,tiles_n,group_m", [
    (1, 1, 8), (1, 112, 8), (128, 96, 8), (7, 5, 4), (9, 3, 16), (10, 7, 3), (64, 48, 1),
    (33, 2, 32), (5, 1, 2),
])
def test_tile_order_is_a_bijection_and_matches_the_model(tiles_m, tiles_n, group_m):
    seen = set()
    for t in range(tiles_m * tiles_n):
        mn = _lib.tile_coord(t, tiles_m, tiles_n, group_m)
        assert mn == model_tile_coord(t, tiles_m, tiles_n, group_m)
        assert 0 <= mn[0] < tiles_m and 0 <= mn[1] < tiles_n
        seen.add(mn)
    assert len(seen) == tiles_m * tiles_n
    with pytest.raises(ValueError):
        _lib.tile_coord(tiles_m * tiles_n, tiles_m, tiles_n, group_m)


def model_tile_coord_slabs(t, tiles_m, tiles_n, group_m, group_n):
    """Independent model of the slab order: column slabs outermost, then row bands."""
    order = []
    for n0 in range(0, tiles_n, group_n):
        cols = range(n0, min(tiles_n, n0 + group_n))
        for m0 in range(0, tiles_m, group_m):
            rows = range(m0, min(tiles_m, m0 + group_m))
            order += [(m, n) for n in cols for m in rows]
    return order[t]


@pytest.mark.parametrize("tiles_m,tiles_n,group_m,group_n", [
    (128, 96, 16, 48), (128, 96, 16, 32), (7, 5, 4, 2), (9, 3, 16, 2), (10, 7, 3, 3), (5, 1, 2, 1),
    (4, 9, 2, 9), (4, 9, 2, 20),
])
def test_slab_tile_order_is_a_bijection_and_matches_the_model(tiles_m, tiles_n, group_m, group_n):
    seen = set()
    for t in range(tiles_m * tiles_n):
        mn = _lib.tile_coord(t, tiles_m, tiles_n, group_m, group_n)
        assert mn == model_tile_coord_slabs(t, tiles_m, tiles_n, group_m, min(group_n, tiles_n))
        seen.add(mn)
    assert len(seen) == tiles_m * tiles_n


def test_tile_order_keeps_a_band_of_rows_together():
    # the first group_m*tiles_n tiles touch only the first group_m tile rows
    tiles_m, tiles_n, g = 128, 96, 8
    rows = {_lib.tile_coord(t, tiles_m, tiles_n, g)[0] for t in range(g * tiles_n)}
    assert rows == set(range(g))


@pytest.mark.parametrize("total,align,world", [
    (32768, 256, 8), (32768, 256, 1), (28672, 128, 8), (1000, 256, 4), (64, 256, 8),
    (14336, 128, 3), (0, 8, 2), (4104, 8, 5),
])
def test_shard_ranges_partition_the_items(total, align, world):
    pos = 0
    sizes = []
    for r in range(world):
        b, c = _lib.shard_range(total, align, world, r)
        assert b == pos and c >= 0
        if b + c < total:
            assert (b + c) % align == 0
        pos = b + c
        sizes.append(c)
    assert pos == total
    whole = [s for s in sizes if s % align == 0 and s > 0]
    if whole:
        assert max(whole) - min(whole) <= align
    with pytest.raises(ValueError):
        _lib.shard_range(total, align, world, world)


def test_query_without_device_reports_cuda_error_not_crash():
    import torch
    if torch.cuda.is_available():
        assert _lib.query(_lib.QUERY_SM_COUNT) > 0
    else:
        with pytest.raises(_lib.SglError):
            _lib.query(_lib.QUERY_SM_COUNT)
    assert _lib.kernel_launches() >= 0


def test_splitk_scratch_plan():
    lib = _lib.load()
    f = lib.sgl_matmul_bf16_splitk_scratch_bytes
    # 8 ranges x 64 rows x 4096 columns x 4 bytes: exactly the built-in scratch size
    assert f(64, 4096, 14336, 8) == 8 << 20
    # rows are padded to whole 32-row store boxes
    assert f(33, 4096, 14336, 8) == 8 * 64 * 4096 * 4
    # K ranges are multiples of 128 and never empty: 1000 / 8 -> ranges of 128 -> 8 ranges
    assert f(64, 256, 1000, 8) == 8 * 64 * 256 * 4
    # more ranges than 128-wide pieces of K: clipped (K = 256 has only 2)
    assert f(64, 256, 256, 8) == 2 * 64 * 256 * 4
    # automatic choice: one tile of output, 14336 deep -> many ranges; many tiles -> one range
    assert f(64, 256, 14336, 0) == 16 * 64 * 256 * 4
    assert f(8192, 8192, 4096, 0) == 1 * 8192 * 8192 * 4
    # decode-size down projection: 16 column tiles, one CTA each -> 9 ranges fill 144 of 148 SMs
    assert f(64, 4096, 14336, 0) == 9 * 64 * 4096 * 4
    # above 128 rows CTA pairs work on 256-row tiles: 74 pairs / 16 tiles -> 4 ranges, one wave
    assert f(256, 4096, 14336, 0) == 4 * 256 * 4096 * 4
    assert f(64, 4096, 14332, 8) == -2       # K not a multiple of 8
    assert f(0, 4096, 14336, 8) == -2
    assert f(64, 4096, 14336, 65) == -10     # too many ranges


def test_host_pipeline_rejects_bad_arguments_before_touching_a_device():
    import ctypes as C
    lib = _lib.load()
    handle = C.c_void_p()
    create = lib.sgl_host_pipeline_create
    assert create(_lib.FORM_MATMUL, 256, 256, 64, 0, 0, 0, None, C.byref(handle)) == -10
    assert create(_lib.FORM_FUSED_SWIGLU, 256, 260, 64, 0, 0, 0, None, C.byref(handle)) == -2
    assert create(_lib.FORM_FUSED_SWIGLU, 256, 256, 64, -1, 0, 0, None, C.byref(handle)) == -10
    assert create(_lib.FORM_FUSED_SWIGLU, 256, 256, 64, 0, 0, 65, None, C.byref(handle)) == -10
    assert create(_lib.FORM_FUSED_SWIGLU, 256, 256, 64, 0, 0, 0, None, None) == -1
    assert not handle.value
    out = C.c_int64()
    assert lib.sgl_host_pipeline_query(None, _lib.PIPE_D2H_BYTES, C.byref(out)) == -1
    assert lib.sgl_host_pipeline_run(None, None, 0, None, 0, None, 0, None, 0, 1) == -1
    assert lib.sgl_host_pipeline_destroy(None) == 0
    import torch
    if not torch.cuda.is_available():
        # no device: a CUDA error code and a message, not a crash
        rc = create(_lib.FORM_FUSED_SWIGLU, 256, 256, 64, 0, 0, 0, None, C.byref(handle))
        assert rc > 0 and lib.sgl_last_error()


def test_mgpu_rejects_bad_arguments_before_touching_a_device():
    import ctypes as C
    lib = _lib.load()
    handle = C.c_void_p()
    one = (C.c_int * 1)(0)
    nine = (C.c_int * 9)(*([0] * 9))
    assert lib.sgl_mgpu_create(1, one, None) == -1
    assert lib.sgl_mgpu_create(1, None, C.byref(handle)) == -1
    assert lib.sgl_mgpu_create(0, one, C.byref(handle)) == -10
    assert lib.sgl_mgpu_create(9, nine, C.byref(handle)) == -10
    assert not handle.value
    assert lib.sgl_mgpu_size(None) == 0
    assert lib.sgl_mgpu_destroy(None) == 0
    assert lib.sgl_mgpu_fused_swiglu(None, 0, None, None, None, 256, 256, 64, 64, 512, 256, None,
                                     None) == -1
    import torch
    if not torch.cuda.is_available():
        rc = lib.sgl_mgpu_create(1, one, C.byref(handle))
        assert rc != 0 and lib.sgl_last_error()
        assert not handle.value


def test_header_is_plain_c_and_a_c_program_links_against_the_library(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 (no C++, no torch types) and a C
    program must link against the library and call it."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    lib_file = _lib.lib_path()
    src = tmp_path / "use_abi.c"
    src.write_text(r'''
#include <stdio.h>
#include <string.h>
#include "swiglu_b200.h"
int main(void) {
  sgl_config cfg;
  int64_t b = 0, c = 0, tm = 0, tn = 0;
  if (sgl_version() < 100) return 1;
  if (sgl_config_count(SGL_FORM_FUSED_SWIGLU) < 1) return 2;
  if (sgl_config_default(SGL_FORM_FUSED_SWIGLU, 32768, 12288, 3072, &cfg) != SGL_OK) return 3;
  if (sgl_config_smem_bytes(SGL_FORM_FUSED_SWIGLU, &cfg) <= 0) return 4;
  if (sgl_shard_range(32768, 256, 8, 3, &b, &c) != SGL_OK || b != 3 * 4096 || c != 4096) return 5;
  if (sgl_tile_coord(0, 4, 4, 2, &tm, &tn) != SGL_OK) return 6;
  if (sgl_matmul_fused_swiglu(NULL, NULL, NULL, 1, 8, 8, 8, 16, 8, 0, 8, NULL, NULL)
      != SGL_ERR_NULL_POINTER) return 7;
  if (strlen(sgl_last_error()) == 0) return 8;
  printf("cta_group=%d block_k=%d\n", cfg.cta_group, cfg.block_k);
  return 0;
}
''')
    exe = tmp_path / "use_abi"
    inc = os.path.dirname(HEADER)
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", f"-I{inc}",
                    str(src), "-o", str(exe), lib_file,
                    f"-Wl,-rpath,{os.path.dirname(lib_file)}"], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, (out.returncode, out.stdout, out.stderr)
    assert "cta_group=2 block_k=128" in out.stdout


def test_ctypes_prototypes_match_the_header():
    """Every declared function has a ctypes prototype with the same number of parameters, and
    pointer / 64-bit / int parameters are bound as such (an ABI drift between the header and the
    binding would otherwise only show up as corrupted arguments on the GPU)."""
    import ctypes as C
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    decls = re.findall(r"\b(?:int|int64_t|const char\*)\s+(sgl_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", text)
    assert len(decls) == len(_lib.EXPORTED_SYMBOLS)
    lib = _lib.load()
    for name, params in decls:
        params = params.strip()
        plist = [] if params in ("", "void") else [p.strip() for p in params.split(",")]
        fn = getattr(lib, name)
        assert fn.argtypes is not None, f"{name} has no ctypes prototype"
        assert len(fn.argtypes) == len(plist), (name, plist, fn.argtypes)
        for decl, ctype in zip(plist, fn.argtypes):
            if "*" in decl:
                assert ctype is C.c_void_p or issubclass(ctype, C._Pointer) or ctype is C.c_char_p, \
                    (name, decl, ctype)
            elif decl.startswith("int64_t"):
                assert ctype is C.c_int64, (name, decl, ctype)
            elif decl.startswith("uint64_t"):
                assert ctype is C.c_uint64, (name, decl, ctype)
            elif decl.startswith("int "):
                assert ctype is C.c_int, (name, decl, ctype)


def test_splitk_cluster_plan_choice():
    """Which tile width and how many K ranges the library picks when the ranges are to run as
    thread-block clusters, for a given table of how many clusters fit (a B200's by default)."""
    plan = _lib.splitk_cluster_plan
    # decode down projection: 16 tiles of 256 columns would need 16 clusters of 8 (15 fit);
    # 22 tiles of 192 columns x 6 ranges load 2432 x (64 + 192) operand elements per CTA, less
    # than 128 columns x 4 ranges (3584 x 192) and 64 columns x 2 ranges (7168 x 128)
    assert plan(64, 4096, 14336) == {"ctas": 132, "tile_cols": 192, "ranges": 6, "k_per_range": 2432}
    # two rows of tiles double the tile count: 32 tiles of 256 columns x 4 ranges load
    # 3584 x (128 + 256) operand elements per CTA, 44 tiles of 192 columns x 3 ranges (more
    # CTAs) 4864 x (128 + 192): the lighter CTA wins
    assert plan(256, 4096, 14336) == {"ctas": 128, "tile_cols": 256, "ranges": 4, "k_per_range": 3584}
    # one tile's worth of columns: narrow tiles, as many ranges as fit
    assert plan(64, 256, 14336) == {"ctas": 32, "tile_cols": 64, "ranges": 8, "k_per_range": 1792}
    assert plan(16, 512, 1024)["ranges"] == 2 and plan(16, 512, 1024)["k_per_range"] == 512
    # K too short for two ranges of 512, or more tiles than clusters of two: no plan
    assert plan(64, 4096, 768)["ctas"] == 0
    assert plan(64, 28672, 8192)["ctas"] == 0
    # a GPU that holds no clusters at all
    assert plan(64, 4096, 14336, clusters_that_fit=(0,) * 9)["ctas"] == 0
    # ranges are multiples of 128 and none is empty
    for K in (1024, 1500 // 8 * 8, 4096, 5000 // 8 * 8, 14336):
        p = plan(64, 1024, K)
        if p["ctas"]:
            assert p["k_per_range"] % 128 == 0 and p["k_per_range"] >= 512
            assert (p["ranges"] - 1) * p["k_per_range"] < K <= p["ranges"] * p["k_per_range"]
    with pytest.raises(ValueError):
        plan(300, 4096, 14336)


def test_cluster_sum_switch_returns_the_previous_setting():
    was = _lib.set_splitk_cluster_sum(False)
    try:
        assert _lib.set_splitk_cluster_sum(True) is False
        assert _lib.set_splitk_cluster_sum(True) is True
    finally:
        _lib.set_splitk_cluster_sum(was)
