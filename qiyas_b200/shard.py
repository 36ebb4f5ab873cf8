"""N-row sharding of a weight matrix across the GPUs of one box, and the gather of the output slices.

The reference is single-device (src/Gpu.cs:94: ordinal 0 always); this is the one parallel strategy the path needs:
output rows are independent (gemv: one dot a row; A.B^T: column j of C needs row j of B only), so rank r keeps rows
[r*ceil(N/g), ...) of the weights, computes its slice with the ordinary single-GPU kernels, and nothing crosses
NVLink unless a full output vector is wanted, in which case the f32 slices are joined by one all-gather
(`torch.distributed`: NCCL on GPUs, gloo in the CPU tests).  x / A are replicated (they are small).
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
