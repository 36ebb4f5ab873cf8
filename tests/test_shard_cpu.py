"""N-row sharding: the plan's arithmetic, and the gather of slices over world_size-2 gloo ranks on the CPU.

The slices themselves come from the oracle here (there is no GPU): what is under test is that sharding by rows, computing
each slice on its own and joining the slices gives the unsharded result bit for bit, on even and odd row counts.
"""
import os
import sys

import numpy as np
import pytest

from qiyas_b200 import blocks as B
from qiyas_b200.shard import ShardPlan

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_plan_covers_rows_once():
    for rows in (0, 1, 7, 28669, 28672, 11003):
        for world in (1, 2, 4, 8):
            plan = ShardPlan(rows, world)
            seen = []
            for r in range(world):
                lo, hi = plan.range(r)
                assert 0 <= lo <= hi <= rows and hi - lo <= plan.per_rank
                seen += list(range(lo, hi))
            assert seen == list(range(rows))


def test_c_abi_range_is_the_plan():
    # qb200_shard_range needs no device: the same arithmetic as ShardPlan, uneven and empty shards included
    import ctypes as C

    from qiyas_b200 import _lib
    lib = _lib.load()
    for rows in (0, 1, 7, 28669, 28672, 11003):
        for world in (1, 2, 3, 8):
            plan = ShardPlan(rows, world)
            for r in range(world):
                first, count = C.c_int(-1), C.c_int(-1)
                assert lib.qb200_shard_range(rows, world, r, C.byref(first), C.byref(count)) == 0
                assert (first.value, first.value + count.value) == plan.range(r)
    assert lib.qb200_shard_range(10, 0, 0, None, None) == -2 and lib.qb200_shard_range(10, 2, 2, None, None) == -2


def test_plan_bytes_and_views():
    plan = ShardPlan(28669, 8)
    assert plan.per_rank == 3584 and plan.count(7) == 28669 - 7 * 3584
    lo, hi = plan.byte_range(7, "q4_0", 8160)
    assert lo == 7 * 3584 * 255 * 18 and hi == 28669 * 255 * 18
    w = B.make_weights(B.Q8_0, 37, 64, 1)
    parts = [ShardPlan(37, 4).slice_weights(r, "q8_0", 64, w) for r in range(4)]
    assert np.array_equal(np.concatenate(parts), w)
    with pytest.raises(ValueError):
        plan.range(8)


def _worker(rank, world, port, rows, cols, m, out):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from oracle import qiyas_oracle as O
    from qiyas_b200.shard import ShardPlan, all_gather_columns, all_gather_rows
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = B.make_weights(B.Q4_0, rows, cols, 5)
        x = B.make_activations(cols, 6)
        plan = ShardPlan(rows, world)
        n = plan.count(rank)
        mine = plan.slice_weights(rank, B.Q4_0, cols, w)
        y_slice = O.gemv_blocks(B.Q4_0, B.F32, mine, x, n, cols, order=1) if n else np.zeros(0, np.float32)
        y = all_gather_rows(plan, rank, torch.from_numpy(y_slice)).numpy()
        a = O.encode(B.Q8_0, B.make_activations(m * cols, 7))
        c_slice = O.matmul_blocks(B.Q8_0, B.Q4_0, a, mine, m, n, cols, order=1) if n else np.zeros((m, 0), np.float32)
        c = all_gather_columns(plan, rank, torch.from_numpy(np.ascontiguousarray(c_slice)), m).numpy()
        if rank == 0:
            np.save(out + ".y.npy", y)
            np.save(out + ".c.npy", c)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("rows,cols", [(64, 256), (61, 96)])
def test_gather_of_slices_equals_unsharded(oracle, tmp_path, rows, cols):
    import torch.multiprocessing as mp
    m, world = 5, 2
    out = str(tmp_path / "gathered")
    port = 29600 + (os.getpid() % 300) + rows
    mp.spawn(_worker, args=(world, port, rows, cols, m, out), nprocs=world, join=True)
    w = B.make_weights(B.Q4_0, rows, cols, 5)
    x = B.make_activations(cols, 6)
    want_y = oracle.gemv_blocks(B.Q4_0, B.F32, w, x, rows, cols, order=1)
    a = oracle.encode(B.Q8_0, B.make_activations(m * cols, 7))
    want_c = oracle.matmul_blocks(B.Q8_0, B.Q4_0, a, w, m, rows, cols, order=1)
    assert np.array_equal(np.load(out + ".y.npy").view(np.uint32), want_y.view(np.uint32))
    assert np.array_equal(np.load(out + ".c.npy").view(np.uint32), want_c.view(np.uint32))
