"""N-row sharding on real GPUs: two ranks, NCCL all-gather of the slices, against the unsharded oracle result.

Needs two GPUs; on a one-GPU box it is skipped (the gather logic is covered by the gloo test on the CPU)."""
import os
import sys

import numpy as np
import pytest

from qiyas_b200 import blocks as B

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, rows, cols, m, out):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from oracle import qiyas_oracle as O
    from qiyas_b200.ops import GpuOps
    from qiyas_b200.shard import ShardedGemv, ShardedMatMul, ShardPlan
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    try:
        dev = f"cuda:{rank}"
        ops = GpuOps(device=rank)
        w = B.make_weights(B.Q4_0, rows, cols, 5)
        x = torch.from_numpy(B.make_activations(cols, 6)).to(dev)
        plan = ShardPlan(rows, world)
        shard = torch.from_numpy(plan.slice_weights(rank, B.Q4_0, cols, w)).to(dev)
        gemv = ShardedGemv(ops, plan, rank, B.Q4_0, cols, shard)
        y = gemv.full(x, torch.empty(max(gemv.rows, 1), dtype=torch.float32, device=dev), fmt_x=B.F32)
        a = torch.from_numpy(O.encode(B.Q8_0, B.make_activations(m * cols, 7))).to(dev)
        mm = ShardedMatMul(ops, plan, rank, B.Q4_0, cols, shard)
        c = mm.full(B.Q8_0, a, torch.empty(max(m * mm.n, 1), dtype=torch.float32, device=dev), m)
        assert ops.gpu.status() == 0
        if rank == 0:
            np.save(out + ".y.npy", y.cpu().numpy())
            np.save(out + ".c.npy", c.cpu().numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("rows,cols", [(4096, 8192), (4093, 8160)])
def test_two_ranks_equal_unsharded(oracle, tmp_path, rows, cols):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    m, world = 33, 2
    out = str(tmp_path / "gathered")
    port = 29900 + (os.getpid() % 90) + rows % 7
    mp.spawn(_worker, args=(world, port, rows, cols, m, out), nprocs=world, join=True)
    w = B.make_weights(B.Q4_0, rows, cols, 5)
    x = B.make_activations(cols, 6)
    want_y = oracle.gemv_blocks(B.Q4_0, B.F32, w, x, rows, cols, order=1)
    mag = np.abs(want_y).max()
    assert np.max(np.abs(np.load(out + ".y.npy") - want_y)) <= 1e-5 * mag
    a = oracle.encode(B.Q8_0, B.make_activations(m * cols, 7))
    want_c = oracle.matmul_blocks(B.Q8_0, B.Q4_0, a, w, m, rows, cols, order=1)
    assert np.array_equal(np.load(out + ".c.npy").view(np.uint32), want_c.view(np.uint32))
