"""N-row sharding on real GPUs against the unsharded oracle result.

Two ranks on two GPUs: the NCCL all-gather of the slices, and the exchange fused into the gemv kernel (stores into the
peer's copy of y through CUDA IPC, flags, bounded wait).  Those need two GPUs and are skipped on a one-GPU box, where the
exchange's kernels are still exercised: two ranks' launches run one after the other on the one GPU into two buffers
(no kernel ever waits for one that has not been launched before it), and a wait on a flag that nothing sets runs out
and reports it."""
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
        # the same y by the exchange inside the gemv kernel, three epochs with three different x
        from qiyas_b200.shard import PeerExchange
        ex = PeerExchange(ops, rows, rank, world)
        try:
            for epoch in range(3):
                xe = torch.from_numpy(B.make_activations(cols, 60 + epoch)).to(dev)
                got = gemv.exchange(xe, ex, fmt_x=B.F32)
                torch.cuda.synchronize()
                assert ops.gpu.status() == 0
                np.save(f"{out}.x{epoch}.r{rank}.npy", got.cpu().numpy())
                dist.barrier()                 # the peers have read their y before the next epoch overwrites it
        finally:
            torch.cuda.synchronize()
            dist.barrier()
            ex.close()
        # a chain of products, each reading the whole output of the one before it from the exchange it was published to:
        # the kernels wait for the flags themselves, two exchanges alternate, one wait at the end
        if chained_case(rows, cols):
            wc = B.make_weights(B.Q4_0, rows, rows, 9)
            sc = torch.from_numpy(plan.slice_weights(rank, B.Q4_0, rows, wc)).to(dev)
            gc = ShardedGemv(ops, plan, rank, B.Q4_0, rows, sc)
            ea, eb = PeerExchange(ops, rows, rank, world), PeerExchange(ops, rows, rank, world)
            try:
                v = torch.from_numpy(B.make_activations(rows, 70)).to(dev)
                yv = gc.exchange(v, ea, fmt_x=B.F32, wait=False)
                for step in range(1, CHAIN):
                    src, dst = (ea, eb) if step % 2 else (eb, ea)
                    yv = gc.exchange(yv, dst, fmt_x=B.F32, after=src, wait=step == CHAIN - 1)
                torch.cuda.synchronize()
                assert ops.gpu.status() == 0
                np.save(f"{out}.chain.r{rank}.npy", yv.cpu().numpy())
            finally:
                torch.cuda.synchronize()
                dist.barrier()
                ea.close()
                eb.close()
        # the same C by the exchange inside the product kernel's epilogue, twice (m rows, then fewer: another kernel)
        # (a third time with more than 64 rows: the 128-row-tile kernel)
        a_tall = torch.from_numpy(O.encode(B.Q8_0, B.make_activations(M_TALL * cols, 8))).to(dev)
        ec = PeerExchange(ops, M_TALL * rows, rank, world)
        try:
            for epoch, rows_a in enumerate((m, 5, M_TALL)):
                got = mm.exchange(B.Q8_0, a_tall if rows_a == M_TALL else a, rows_a, ec)
                torch.cuda.synchronize()
                assert ops.gpu.status() == 0
                np.save(f"{out}.cx{epoch}.r{rank}.npy", got.reshape(-1)[:rows_a * rows].cpu().numpy())
                dist.barrier()
        finally:
            torch.cuda.synchronize()
            dist.barrier()
            ec.close()
        if rank == 0:
            np.save(out + ".y.npy", y.cpu().numpy())
            np.save(out + ".c.npy", c.cpu().numpy())
    finally:
        dist.destroy_process_group()


CHAIN = 4
M_TALL = 130


def chained_case(rows, cols):
    """The chained products (a square matrix of `rows`: every y is the next x) ride on one of the shapes only."""
    return rows == 4096 and cols == 8192


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
    a_tall = oracle.encode(B.Q8_0, B.make_activations(M_TALL * cols, 8))
    want_tall = oracle.matmul_blocks(B.Q8_0, B.Q4_0, a_tall, w, M_TALL, rows, cols, order=1)
    for epoch, rows_a in enumerate((m, 5, M_TALL)):
        for rank in range(world):
            got = np.load(f"{out}.cx{epoch}.r{rank}.npy")
            want = want_tall if rows_a == M_TALL else want_c[:rows_a]
            assert np.array_equal(got.view(np.uint32), want.reshape(-1).view(np.uint32)), (epoch, rank)
    for epoch in range(3):
        want = oracle.gemv_blocks(B.Q4_0, B.F32, w, B.make_activations(cols, 60 + epoch), rows, cols, order=1)
        for rank in range(world):
            got = np.load(f"{out}.x{epoch}.r{rank}.npy")
            assert np.max(np.abs(got - want)) <= 1e-5 * np.abs(want).max(), (epoch, rank)
    if chained_case(rows, cols):
        # the chain on the CPU: every rank must hold the same whole vector, and it must be the oracle's chain (each step
        # re-encodes its x to Q8_0, where a last-bit difference of an element can move a code: hence the looser bound)
        wc = B.make_weights(B.Q4_0, rows, rows, 9)
        v = B.make_activations(rows, 70)
        for _ in range(CHAIN):
            v = oracle.gemv_blocks(B.Q4_0, B.F32, wc, v, rows, rows, order=1)
        got = [np.load(f"{out}.chain.r{rank}.npy") for rank in range(world)]
        assert np.array_equal(got[0].view(np.uint32), got[1].view(np.uint32))
        assert np.max(np.abs(got[0] - v)) <= 2e-3 * np.abs(v).max()


def _peers(lib, world, rank, ys, flags):
    from qiyas_b200 import _lib
    p = _lib.ShardPeers()
    p.world, p.rank = world, rank
    for w in range(world):
        p.out[w], p.flags[w] = ys[w].data_ptr(), flags[w].data_ptr()
    return p


@pytest.mark.parametrize("counted", [False, True])
@pytest.mark.parametrize("rows,world", [(4096, 2), (4093, 4), (5, 8)])
def test_exchange_kernels_on_one_gpu(oracle, rows, world, counted):
    # every rank's launches in turn on the one GPU, each with its own copy of y and its own flags; then every rank's wait
    import ctypes as C
    import torch

    from . import helpers as H
    from qiyas_b200.shard import ShardPlan
    o = H.ops()
    cols = 2048
    w = B.make_weights(B.Q4_0, rows, cols, 15)
    plan = ShardPlan(rows, world)
    shards = [H.dev(plan.slice_weights(r, B.Q4_0, cols, w)) if plan.count(r) else None for r in range(world)]
    ys = [torch.full((rows + 8,), float("nan"), dtype=torch.float32, device="cuda:0") for _ in range(world)]
    flags = [torch.zeros(16, dtype=torch.int32, device="cuda:0") for _ in range(world)]
    for epoch in (1, 2):
        xf = B.make_activations(cols, 16 + epoch)
        x = H.dev(xf)
        for r in range(world):
            p = _peers(o.lib, world, r, ys, flags)
            a = shards[r].data_ptr() if shards[r] is not None else None
            assert o.lib.qb200_shard_gemv(B.Q4_0, B.F32, a, x.data_ptr(), rows, cols, C.byref(p), 0 if counted else epoch, None) == 0, o.gpu.error()
        for r in range(world):
            p = _peers(o.lib, world, r, ys, flags)
            assert o.lib.qb200_shard_wait(C.byref(p), 0 if counted else epoch, 0, None) == 0      # 0: epochs counted on the device
        assert o.gpu.status() == 0
        want = oracle.gemv_blocks(B.Q4_0, B.F32, w, xf, rows, cols, order=1)
        for r in range(world):
            got = ys[r].cpu().numpy()
            assert np.max(np.abs(got[:rows] - want)) <= 1e-5 * np.abs(want).max(), (epoch, r)
            assert np.isnan(got[rows:]).all()                       # nothing stored past the vector
            assert (flags[r].cpu().numpy()[:world] == epoch).all()


@pytest.mark.parametrize("m,n,k,world,fmt_b,prepacked", [(37, 300, 512, 2, B.Q8_0, False), (130, 517, 256, 4, B.Q8_0, False),
                                                         (200, 256, 320, 2, B.Q4_0, True), (8, 1000, 256, 2, B.Q4_K, False),
                                                         (64, 640, 256, 3, B.Q4_0, True), (5, 3, 64, 8, B.Q8_0, False)])
def test_product_exchange_kernels_on_one_gpu(oracle, m, n, k, world, fmt_b, prepacked):
    # the sharded A.B^T: every rank's product in turn on the one GPU, each storing its column block into every rank's copy
    # of C (each copy with its own flags); then every rank's wait.  Bit for bit the unsharded oracle product in every copy.
    import ctypes as C
    import torch

    from . import helpers as H
    from qiyas_b200.shard import ShardPlan
    o = H.ops()
    b = B.make_weights(fmt_b, n, k, 25)
    a_raw = oracle.encode(B.Q8_0, B.make_activations(m * k, 26))
    a = H.dev(a_raw)
    plan = ShardPlan(n, world)
    shards = [H.dev(plan.slice_weights(r, fmt_b, k, b)) if plan.count(r) else None for r in range(world)]
    packed = [o.Prepack(fmt_b, s, plan.count(r), k) if prepacked and s is not None else None for r, s in enumerate(shards)]
    cs = [torch.full((m * n + 8,), float("nan"), dtype=torch.float32, device="cuda:0") for _ in range(world)]
    flags = [torch.zeros(16, dtype=torch.int32, device="cuda:0") for _ in range(world)]
    if fmt_b == B.Q4_K:
        want = oracle.matmul_q4_k(B.Q8_0, a_raw, b, m, n, k).reshape(-1)
    else:
        want = oracle.matmul_blocks(B.Q8_0, fmt_b, a_raw, b, m, n, k, order=1).reshape(-1)
    for epoch in (1, 2):
        for c in cs:
            c.fill_(float("nan"))
        for r in range(world):
            p = _peers(o.lib, world, r, cs, flags)
            raw = shards[r].data_ptr() if shards[r] is not None and packed[r] is None else None
            pk = packed[r].data_ptr() if packed[r] is not None else None
            assert o.lib.qb200_shard_matmul(B.Q8_0, fmt_b, a.data_ptr(), raw, pk, m, n, k, C.byref(p), epoch, None, 0, None) == 0, o.gpu.error()
        for r in range(world):
            p = _peers(o.lib, world, r, cs, flags)
            assert o.lib.qb200_shard_wait(C.byref(p), epoch, 0, None) == 0
        assert o.gpu.status() == 0
        for r in range(world):
            got = cs[r].cpu().numpy()
            assert np.array_equal(got[:m * n].view(np.uint32), want.view(np.uint32)), (epoch, r)
            assert np.isnan(got[m * n:]).all()                      # nothing stored past the matrix
            assert (flags[r].cpu().numpy()[:world] == epoch).all()


def test_a_wait_nobody_answers_runs_out():
    # a flag that nothing sets: the wait gives up after its limit, reports bit 2 and the context stays usable
    import ctypes as C
    import torch

    from . import helpers as H
    o = H.ops()
    ys = [torch.zeros(64, dtype=torch.float32, device="cuda:0") for _ in range(2)]
    flags = [torch.zeros(16, dtype=torch.int32, device="cuda:0") for _ in range(2)]
    p = _peers(o.lib, 2, 0, ys, flags)
    assert o.gpu.status() == 0
    assert o.lib.qb200_shard_wait(C.byref(p), 1, 2_000_000, None) == 0           # about a millisecond
    assert o.gpu.status() == 4
    assert o.gpu.status() == 0                                                  # read and cleared
    flags[0][:2] = 1
    assert o.lib.qb200_shard_wait(C.byref(p), 1, 2_000_000, None) == 0
    assert o.gpu.status() == 0


@pytest.mark.parametrize("counted", [False, True])
def test_chained_exchange_kernels_on_one_gpu(oracle, counted):
    # the chain's kernels (the wait inside the gemv) with every rank's launches in turn on the one GPU: a product's launches
    # all precede the next product's, so no kernel waits for one that has not been launched
    import ctypes as C
    import torch

    from . import helpers as H
    from qiyas_b200.shard import ShardPlan
    o = H.ops()
    rows, world, steps = 1024, 4, 4
    w = B.make_weights(B.Q4_0, rows, rows, 25)
    plan = ShardPlan(rows, world)
    shards = [H.dev(plan.slice_weights(r, B.Q4_0, rows, w)) for r in range(world)]
    ys = [[torch.zeros(rows, dtype=torch.float32, device="cuda:0") for _ in range(world)] for _ in range(2)]
    flags = [[torch.zeros(16, dtype=torch.int32, device="cuda:0") for _ in range(world)] for _ in range(2)]
    x0 = B.make_activations(rows, 26)
    x = H.dev(x0)
    epochs = [0, 0]
    for step in range(steps):
        dst, src = step % 2, (step + 1) % 2
        epochs[dst] += 1
        for r in range(world):
            pd = _peers(o.lib, world, r, ys[dst], flags[dst])
            if step == 0:
                rc = o.lib.qb200_shard_gemv(B.Q4_0, B.F32, shards[r].data_ptr(), x.data_ptr(), rows, rows, C.byref(pd), 0 if counted else epochs[dst], None)
            else:
                ps = _peers(o.lib, world, r, ys[src], flags[src])
                rc = o.lib.qb200_shard_gemv_after(B.Q4_0, B.F32, shards[r].data_ptr(), ys[src][r].data_ptr(), rows, rows, C.byref(pd),
                                                  0 if counted else epochs[dst], C.byref(ps), 0 if counted else epochs[src], 0, None)
            assert rc == 0, o.gpu.error()
    for r in range(world):
        pd = _peers(o.lib, world, r, ys[(steps - 1) % 2], flags[(steps - 1) % 2])
        assert o.lib.qb200_shard_wait(C.byref(pd), 0 if counted else epochs[(steps - 1) % 2], 0, None) == 0
    assert o.gpu.status() == 0
    v = x0
    for _ in range(steps):
        v = oracle.gemv_blocks(B.Q4_0, B.F32, w, v, rows, rows, order=1)
    for r in range(world):
        got = ys[(steps - 1) % 2][r].cpu().numpy()
        assert np.max(np.abs(got - v)) <= 2e-3 * np.abs(v).max(), r
        assert np.array_equal(got.view(np.uint32), ys[(steps - 1) % 2][0].cpu().numpy().view(np.uint32))


def test_a_wait_inside_the_gemv_runs_out():
    # the exchange x is said to come from never raised its flags: the kernel's own wait gives up after its limit, reports
    # bit 2, computes on what is there, and the context stays usable
    import ctypes as C
    import torch

    from . import helpers as H
    o = H.ops()
    rows = 256
    w = H.dev(B.make_weights(B.Q4_0, rows, rows, 27))
    ys = [[torch.zeros(rows, dtype=torch.float32, device="cuda:0")] for _ in range(2)]
    flags = [[torch.zeros(16, dtype=torch.int32, device="cuda:0")] for _ in range(2)]
    pd, ps = _peers(o.lib, 1, 0, ys[0], flags[0]), _peers(o.lib, 1, 0, ys[1], flags[1])
    assert o.gpu.status() == 0
    assert o.lib.qb200_shard_gemv_after(B.Q4_0, B.F32, w.data_ptr(), ys[1][0].data_ptr(), rows, rows, C.byref(pd), 1, C.byref(ps), 7, 2_000_000, None) == 0
    assert o.gpu.status() == 4
    assert o.gpu.status() == 0
    flags[1][0][0] = 7
    assert o.lib.qb200_shard_gemv_after(B.Q4_0, B.F32, w.data_ptr(), ys[1][0].data_ptr(), rows, rows, C.byref(pd), 2, C.byref(ps), 7, 2_000_000, None) == 0
    assert o.gpu.status() == 0
