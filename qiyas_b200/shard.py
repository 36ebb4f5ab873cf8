"""N-row sharding of a weight matrix across the GPUs of one box, and the gather of the output slices.

The reference is single-device (src/Gpu.cs:94: ordinal 0 always); this is the one parallel strategy the path needs:
output rows are independent (gemv: one dot a row; A.B^T: column j of C needs row j of B only), so rank r keeps rows
[r*ceil(N/g), ...) of the weights, computes its slice with the ordinary single-GPU kernels, and nothing crosses
NVLink unless a full output vector is wanted, in which case the f32 slices are joined by one all-gather
(`torch.distributed`: NCCL on GPUs, gloo in the CPU tests).  x / A are replicated (they are small).

For the gemv, whose slices are a few kilobytes, the all-gather's launch latency is several times the product's own
time.  `PeerExchange` is the alternative on one box: every rank maps every other rank's output vector (CUDA IPC) and
the gemv kernel itself stores its rows into all of them, followed by a flag a rank; `ShardedGemv.exchange` is that call
plus the bounded wait for the peers' flags (qb200_shard_gemv / qb200_shard_wait).  `ShardedMatMul.exchange` does the same
for A.B^T: the product kernel stores its column block of C into every rank's copy of C (qb200_shard_matmul).
"""
from dataclasses import dataclass

from .blocks import fmt_id, row_bytes


@dataclass(frozen=True)
class ShardPlan:
    """Contiguous row slices of an N-row matrix over `world` ranks: ceil(N/world) rows each, the last ones shorter or empty."""
    rows: int
    world: int

    def __post_init__(self):
        if self.rows < 0 or self.world < 1:
            raise ValueError("rows >= 0 and world >= 1")

    @property
    def per_rank(self):
        return (self.rows + self.world - 1) // self.world

    def range(self, rank):
        """[first, last) rows of `rank`."""
        if not 0 <= rank < self.world:
            raise ValueError(f"rank {rank} of {self.world}")
        first = min(self.rows, rank * self.per_rank)
        return first, min(self.rows, first + self.per_rank)

    def count(self, rank):
        first, last = self.range(rank)
        return last - first

    def byte_range(self, rank, fmt, cols):
        """[first, last) bytes of `rank`'s rows in a row-major block matrix with `cols` columns."""
        rb = row_bytes(fmt_id(fmt), cols)
        first, last = self.range(rank)
        return first * rb, last * rb

    def slice_weights(self, rank, fmt, cols, weights):
        """`rank`'s rows of a flat uint8 weight array (numpy or torch): a view, no copy."""
        lo, hi = self.byte_range(rank, fmt, cols)
        return weights[lo:hi]


def all_gather_rows(plan, rank, y_slice, group=None, out=None):
    """The full output vector from every rank's slice of it (gemv): f32[rows].

    When the rows divide evenly the slices are gathered in place into `out` (allocated here when not given): one
    collective, no copy.  Otherwise slices are padded to ceil(N/g) so that one equal-count all-gather serves the uneven
    last shard.
    """
    import torch
    import torch.distributed as dist
    per = plan.per_rank
    if per * plan.world == plan.rows and y_slice.numel() == per:
        if out is None:
            out = torch.empty(plan.rows, dtype=y_slice.dtype, device=y_slice.device)
        if plan.world == 1:
            out.copy_(y_slice)
        else:
            dist.all_gather_into_tensor(out, y_slice, group=group)
        return out
    mine = torch.zeros(per, dtype=y_slice.dtype, device=y_slice.device)
    mine[:plan.count(rank)] = y_slice[:plan.count(rank)]
    out = torch.empty(per * plan.world, dtype=y_slice.dtype, device=y_slice.device)
    if plan.world == 1:
        out.copy_(mine)
    else:
        dist.all_gather_into_tensor(out, mine, group=group)
    return out[:plan.rows] if per * plan.world == plan.rows else torch.cat(
        [out[r * per:r * per + plan.count(r)] for r in range(plan.world)])


def all_gather_columns(plan, rank, c_slice, m, group=None):
    """The full C (m x N) from every rank's column block C[:, first:last] (A.B^T with B sharded by rows)."""
    import torch
    import torch.distributed as dist
    per = plan.per_rank
    mine = torch.zeros((m, per), dtype=c_slice.dtype, device=c_slice.device)
    n_mine = plan.count(rank)
    mine[:, :n_mine] = c_slice.reshape(m, -1)[:, :n_mine]
    out = torch.empty((plan.world, m, per), dtype=c_slice.dtype, device=c_slice.device)
    if plan.world == 1:
        out[0].copy_(mine)
    else:
        dist.all_gather_into_tensor(out.view(-1), mine.view(-1), group=group)
    return torch.cat([out[r, :, :plan.count(r)] for r in range(plan.world)], dim=1).contiguous()


class ShardedGemv:
    """One rank's part of y = W.x with W sharded by rows: the local kernel call, and the optional gather."""

    def __init__(self, ops, plan, rank, fmt, cols, w_shard):
        self.ops, self.plan, self.rank, self.fmt, self.cols, self.w = ops, plan, rank, fmt_id(fmt), cols, w_shard
        self.rows = plan.count(rank)

    def local(self, x, y_slice, fmt_x=None, stream=None):
        """This rank's slice of y (no communication)."""
        return self.ops.GemvBlocks(self.fmt, self.w, x, y_slice, self.rows, self.cols, fmt_x=fmt_x, stream=stream)

    def full(self, x, y_slice, fmt_x=None, group=None, out=None):
        """The whole y on every rank: the local slice, then the all-gather over NVLink."""
        self.local(x, y_slice, fmt_x=fmt_x)
        return all_gather_rows(self.plan, self.rank, y_slice, group=group, out=out)


class ShardedMatMul:
    """One rank's part of C = A.B^T with B sharded by rows (C by columns)."""

    def __init__(self, ops, plan, rank, fmt_b, k, b_shard):
        self.ops, self.plan, self.rank, self.fmt_b, self.k, self.b = ops, plan, rank, fmt_id(fmt_b), k, b_shard
        self.n = plan.count(rank)

    def local(self, fmt_a, a, c_slice, m, stream=None):
        """C[:, first:last] as a contiguous m x n_local block."""
        if self.n == 0:
            return None
        return self.ops.MatMulBlocks(fmt_a, a, self.b, c_slice, m, self.n, self.k, fmt_b=self.fmt_b, stream=stream)

    def full(self, fmt_a, a, c_slice, m, group=None):
        self.local(fmt_a, a, c_slice, m)
        return all_gather_columns(self.plan, self.rank, c_slice, m, group=group)


class _DeviceArray:
    """A raw device allocation as something torch can wrap (`torch.as_tensor(obj, device=...)`), without owning it."""

    def __init__(self, ptr, count, typestr):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": typestr, "data": (ptr, False), "version": 2}


class PeerExchange:
    """Every rank's copy of the whole output vector and its flag array, as this process addresses them.

    Each rank allocates its own (plain cudaMalloc through the library, so that the allocation can be exported), hands the
    others a CUDA IPC handle over `torch.distributed` (any backend: the handles are 64 bytes of host data), and opens
    theirs.  With world 1 nothing is exchanged.  `close()` unmaps and frees; the object must outlive every call that uses it.
    """

    def __init__(self, ops, rows_total, rank, world, group=None):
        import ctypes as C

        from . import _lib
        if not 1 <= world <= _lib.SHARD_MAX:
            raise ValueError(f"at most {_lib.SHARD_MAX} ranks")
        self.ops, self.lib, self.rows_total, self.rank, self.world = ops, ops.lib, int(rows_total), rank, world
        self._own, self._opened = [], []
        y, flags = C.c_void_p(), C.c_void_p()
        y_bytes = max(256, (self.rows_total * 4 + 255) // 256 * 256)
        ops.gpu.check(self.lib.qb200_malloc(C.byref(y), y_bytes), "malloc y")
        self._own.append(y.value)
        ops.gpu.check(self.lib.qb200_malloc(C.byref(flags), 256), "malloc flags")
        self._own.append(flags.value)
        ops.gpu.check(self.lib.qb200_memset(y, 0, y_bytes, None), "memset")
        ops.gpu.check(self.lib.qb200_memset(flags, 0, 256, None), "memset")
        ops.gpu.Synchronize()
        out, fl = [None] * world, [None] * world
        out[rank], fl[rank] = y.value, flags.value
        if world > 1:
            import torch.distributed as dist
            mine = (C.create_string_buffer(64), C.create_string_buffer(64))
            ops.gpu.check(self.lib.qb200_ipc_export(y, mine[0]), "ipc export")
            ops.gpu.check(self.lib.qb200_ipc_export(flags, mine[1]), "ipc export")
            handles = [None] * world
            dist.all_gather_object(handles, (mine[0].raw, mine[1].raw), group=group)
            for w in range(world):
                if w == rank:
                    continue
                for which, store in ((0, out), (1, fl)):
                    ptr = C.c_void_p()
                    ops.gpu.check(self.lib.qb200_ipc_import(C.create_string_buffer(handles[w][which], 64), C.byref(ptr)), "ipc import")
                    self._opened.append(ptr.value)
                    store[w] = ptr.value
            dist.barrier(group=group)          # everyone has opened everything before anyone stores
        self.peers = _lib.ShardPeers()
        self.peers.world, self.peers.rank = world, rank
        for w in range(world):
            self.peers.out[w], self.peers.flags[w] = out[w], fl[w]
        self.y_ptr = y.value
        self.epoch = 0

    def y(self):
        """This rank's copy of the whole output vector as a torch tensor (a view of the allocation, not a copy)."""
        import torch
        return torch.as_tensor(_DeviceArray(self.y_ptr, self.rows_total, "<f4"), device=f"cuda:{self.ops.gpu.device}")

    def close(self):
        for ptr in self._opened:
            self.lib.qb200_ipc_close(ptr)
        for ptr in self._own:
            self.lib.qb200_free(ptr)
        self._opened, self._own = [], []


def _exchange(self, x, exchange, fmt_x=None, stream=None, limit_cycles=0, after=None, wait=True):
    """This rank's slice into every rank's copy of y (stores from inside the gemv kernel), then the bounded wait for the
    peers' slices: after it, work on `stream` sees the whole y in `exchange.y()`.

    A chain of products (each x the whole y of the one before): pass `after` = the exchange whose y this x is and
    `wait=False` on all but the last; the kernel then waits for that exchange's flags itself, with its weights' copies
    already running, and no wait kernel stands between the products.  Alternate two exchanges along the chain."""
    import ctypes as C

    from .ops import _ptr, _stream
    exchange.epoch += 1
    fx = self.fmt if fmt_x is None else fmt_id(fmt_x)
    if after is None:
        rc = self.ops.lib.qb200_shard_gemv(self.fmt, fx, _ptr(self.w), _ptr(x), self.plan.rows, self.cols, C.byref(exchange.peers), exchange.epoch,
                                           _stream(stream))
    else:
        rc = self.ops.lib.qb200_shard_gemv_after(self.fmt, fx, _ptr(self.w), _ptr(x), self.plan.rows, self.cols, C.byref(exchange.peers),
                                                 exchange.epoch, C.byref(after.peers), after.epoch, int(limit_cycles), _stream(stream))
    self.ops.gpu.check(rc, "shard_gemv")
    if wait:
        self.ops.gpu.check(self.ops.lib.qb200_shard_wait(C.byref(exchange.peers), exchange.epoch, int(limit_cycles), _stream(stream)), "shard_wait")
    return exchange.y()


ShardedGemv.exchange = _exchange


def _exchange_columns(self, fmt_a, a, m, exchange, b_packed=None, stream=None, limit_cycles=0, wait=True):
    """This rank's column block into every rank's copy of C (stores from inside the product kernel's epilogue), then the
    bounded wait for the peers' blocks: after it, work on `stream` sees the whole m x n C in `exchange.y()`
    (`exchange` = a PeerExchange over m * n values).  `b_packed`: the shard as `Prepack` left it, instead of the raw rows."""
    import ctypes as C

    from .ops import _ptr, _stream
    exchange.epoch += 1
    rc = self.ops.lib.qb200_shard_matmul(fmt_id(fmt_a), self.fmt_b, _ptr(a), None if b_packed is not None else _ptr(self.b),
                                         None if b_packed is None else _ptr(b_packed), int(m), self.plan.rows, self.k, C.byref(exchange.peers),
                                         exchange.epoch, None, 0, _stream(stream))
    self.ops.gpu.check(rc, "shard_matmul")
    if wait:
        self.ops.gpu.check(self.ops.lib.qb200_shard_wait(C.byref(exchange.peers), exchange.epoch, int(limit_cycles), _stream(stream)), "shard_wait")
    return exchange.y()[:int(m) * self.plan.rows].view(int(m), self.plan.rows)


ShardedMatMul.exchange = _exchange_columns
