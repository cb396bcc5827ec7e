"""Persisted tile table and autotuner.

The reference tunes on the first call for every ``(M, N, K)`` and forgets the
result when the process exits (``_tune`` / ``_best``,
``swiglu/matmul_silu_mul.py:98,114-139``; ``swiglu/matmul_fused_swiglu.py:106,122-149``).
Here the winners live in ``tile_table.json`` next to this file, keyed by form
and shape, and a shape without an entry uses the library's built-in default.
``autotune`` re-measures and (optionally) writes the file back.  Set
``SWIGLU_B200_AUTOTUNE=1`` to tune on first use the way the reference does.
"""
from __future__ import annotations

import json
import os
import threading

from . import _lib
from ._lib import TileConfig

TABLE_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tile_table.json")
FORM_NAMES = {_lib.FORM_SILU_MUL: "silu_mul", _lib.FORM_FUSED_SWIGLU: "fused_swiglu",
              _lib.FORM_MATMUL: "matmul", _lib.FORM_FUSED_SWIGLU_SAVE: "fused_swiglu_save"}

_lock = threading.Lock()
_table: dict[str, TileConfig] | None = None


def _key(form: int, M: int, N: int, K: int) -> str:
    return f"{FORM_NAMES[form]}:{M}x{N}x{K}"


def _load() -> dict[str, TileConfig]:
    global _table
    if _table is not None:          # hot path of every operator call: no lock once loaded
        return _table
    with _lock:
        if _table is None:
            _table = {}
            path = os.environ.get("SWIGLU_B200_TILE_TABLE", TABLE_PATH)
            if os.path.exists(path):
                with open(path) as f:
                    raw = json.load(f)
                for k, v in raw.get("entries", {}).items():
                    _table[k] = TileConfig(int(v["cta_group"]), int(v["block_k"]),
                                           int(v.get("stages", 0)), int(v["group_m"]), 0,
                                           int(v.get("l2_hints", 0)), int(v.get("group_n", 0)),
                                           int(v.get("wide", 0)))
        return _table


def lookup(form: int, M: int, N: int, K: int) -> TileConfig | None:
    """Tuned entry for this exact problem, or None (the library default applies)."""
    return _load().get(_key(form, M, N, K))


def remember(form: int, M: int, N: int, K: int, cfg: TileConfig) -> None:
    _load()[_key(form, M, N, K)] = cfg


def save(path: str | None = None) -> str:
    """Write the in-memory table to disk (atomically)."""
    path = path or os.environ.get("SWIGLU_B200_TILE_TABLE", TABLE_PATH)
    entries = {
        k: {"cta_group": c.cta_group, "block_k": c.block_k, "stages": c.stages,
            "group_m": c.group_m, "l2_hints": c.l2_hints, "group_n": c.group_n,
            "wide": c.wide}
        for k, c in sorted(_load().items())
    }
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        json.dump({"version": 1, "entries": entries}, f, indent=1, sort_keys=True)
        f.write("\n")
    os.replace(tmp, path)
    return path


def legal_configs(form: int, M: int, N: int, K: int) -> list[TileConfig]:
    """Built-in configurations worth timing for this problem.

    Every configuration is *correct* for every shape (ragged tiles are
    zero-filled and clipped), unlike the reference, whose legality rules reject
    shapes outright (``_legal_for_problem``, ``swiglu/matmul_silu_mul.py:101-111``).
    This only drops entries that cannot win: CTA pairs when there is a single
    128-row tile, and duplicate tile orders when the band covers all rows.
    """
    out = []
    seen = set()
    for c in _lib.builtin_configs(form):
        if c.cta_group == 2 and M <= 128:
            continue
        rows = 128 * c.cta_group
        tiles_m = -(-M // rows)
        eff_group = min(c.group_m, tiles_m)
        sig = (c.cta_group, c.block_k, c.stages, eff_group, c.l2_hints, c.group_n, c.wide)
        if sig in seen:
            continue
        seen.add(sig)
        out.append(c)
    return out


def time_call(fn, warmup: int = 3, iters: int = 10) -> float:
    """Median device time of ``fn()`` in milliseconds (CUDA events, current stream)."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        stop.synchronize()
        times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]


def autotune(form: int, run, M: int, N: int, K: int, *, verbose: bool = False,
             persist: bool = False, warmup: int = 3, iters: int = 10) -> TileConfig:
    """Time every candidate with ``run(cfg)`` and remember the fastest.

    ``run`` launches the operator once with the given TileConfig on the current
    stream.  Returns the winner; with ``persist`` also rewrites the table file.
    """
    best, best_ms = None, float("inf")
    for cfg in legal_configs(form, M, N, K):
        try:
            ms = time_call(lambda: run(cfg), warmup, iters)
        except (ValueError, RuntimeError) as e:  # a config that does not fit this device
            if verbose:
                print(f"  {cfg}: failed: {e}")
            continue
        if verbose:
            print(f"  {cfg}: {ms:.4f} ms")
        if ms < best_ms:
            best, best_ms = cfg, ms
    if best is None:
        raise RuntimeError("no tile configuration ran")
    remember(form, M, N, K, best)
    if persist:
        save()
    return best
