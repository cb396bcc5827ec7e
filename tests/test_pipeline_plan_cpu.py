"""The schedule of the host-buffer pipeline (``sgl_host_pipeline_plan``), checked without a GPU.

One run must produce every element of this rank's ``h`` exactly once, copy every row of x and
(with ``copy_weight``) every column of this rank's weight slice exactly once before it is used,
and in the shared-weight form wait for every other rank's slice before touching its columns -
for every rank of the group, for even and ragged sizes.  The slices of the ranks must partition
the weight's columns (they are what each rank copies from the host), and the order in which a
rank consumes its peers' slices must be the order in which they are pushed to it.
"""
import numpy as np
import pytest

from swiglu_fused_b200 import _lib

CASES = [
    # M (rows of this rank), N, world, kwargs
    (32768, 12288, 1, {}),
    (4096, 12288, 8, {}),
    (16384, 12288, 2, {}),
    (1000, 1160, 4, {}),                       # ragged rows and a ragged last slice
    (300, 136, 3, {}),                         # fewer 256-column blocks than ranks
    (5000, 1288, 2, {"first_rows": 1000, "block_rows": 1024, "windows": 4}),
    (2048, 1024, 1, {"windows": 1}),
]


@pytest.mark.parametrize("M,N,world,kw", CASES)
def test_every_rank_schedule_covers_h_once_and_orders_its_inputs(M, N, world, kw):
    slices = [_lib.shard_range(N, 256, world, r) for r in range(world)]
    assert sum(c for _, c in slices) == N                      # the slices partition the weight
    for rank in range(world):
        plan = _lib.host_pipeline_plan(M, N, world=world, rank=rank, **kw)
        cover = np.zeros((M, N), dtype=np.int16)
        rows_in = np.zeros(M, dtype=np.int16)
        cols_in = np.zeros(N, dtype=np.int16)
        arrived = {rank} if world > 1 else set(range(world))
        signalled = 0
        waits = []
        for st in plan:
            r0, r1, c0, c1 = st["row0"], st["row1"], st["col0"], st["col1"]
            assert 0 <= r0 < r1 <= M and 0 <= c0 <= c1 <= N
            if st["copies_rows"]:
                rows_in[r0:r1] += 1
            if st["copies_weight_window"]:
                cols_in[c0:c1] += 1
                own0, ownn = slices[rank] if world > 1 else (0, N)
                assert own0 <= c0 and c1 <= own0 + ownn        # only its own slice comes from the host
            if st["waits_for_rank"] >= 0:
                q = st["waits_for_rank"]
                assert q != rank and (c0, c1 - c0) == slices[q]
                arrived.add(q)
                waits.append(q)
            signalled += st["signals_peers"]
            # everything the step reads is there: its rows of x and its columns of the weight
            assert (rows_in[r0:r1] == 1).all()
            if world > 1:
                for q, (q0, qn) in enumerate(slices):
                    if qn and c0 < q0 + qn and q0 < c1:
                        assert q in arrived, (rank, st, q)
                        if q == rank:
                            assert (cols_in[max(c0, q0):min(c1, q0 + qn)] == 1).all()
            else:
                assert (cols_in[c0:c1] == 1).all()
            cover[r0:r1, c0:c1] += 1
        assert (cover == 1).all()
        assert (rows_in == 1).all()
        if world > 1:
            assert signalled == 1
            own0, ownn = slices[rank]
            assert (cols_in[own0:own0 + ownn] == 1).all() and cols_in.sum() == ownn
            # peers' slices are consumed in the order they are pushed: rank r pushes to r+1
            # first, so rank-1's slice lands first, then rank-2's, ...
            want = [(rank - d) % world for d in range(1, world) if slices[(rank - d) % world][1]]
            assert waits == want
        else:
            assert (cols_in == 1).all()
        # the weight-resident schedule: row blocks only, same coverage, no weight traffic
        res = _lib.host_pipeline_plan(M, N, world=world, rank=rank, copy_weight=False, **kw)
        cover[:] = 0
        for st in res:
            assert not st["copies_weight_window"] and st["waits_for_rank"] == -1
            assert (st["col0"], st["col1"]) == (0, N) and st["copies_rows"]
            cover[st["row0"]:st["row1"]] += 1
        assert (cover == 1).all()


def test_bad_plan_requests_are_rejected():
    lib = _lib.load()
    assert lib.sgl_host_pipeline_plan(0, 128, 0, 0, 0, 1, 0, 1, 0, None) < 0
    assert lib.sgl_host_pipeline_plan(128, 130, 0, 0, 0, 1, 0, 1, 0, None) < 0
    assert lib.sgl_host_pipeline_plan(128, 128, 0, 0, 0, 2, 2, 1, 0, None) < 0
    assert lib.sgl_host_pipeline_plan(128, 128, 0, 0, 0, 2, 1, 1, 4, None) < 0
