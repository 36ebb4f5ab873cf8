"""Shared pieces of the GPU parity tests: device buffers through torch, the operators through the C ABI."""
import numpy as np

from qiyas_b200 import blocks as B

_ops = None


def ops():
    global _ops
    if _ops is None:
        from qiyas_b200.ops import GpuOps
        _ops = GpuOps(device=0)
    return _ops


def dev(array, offset=0):
    """A host array on the device; `offset` bytes of padding in front give an operand of chosen misalignment."""
    import torch
    raw = np.ascontiguousarray(array).view(np.uint8).reshape(-1)
    buf = torch.empty(raw.size + offset + 64, dtype=torch.uint8, device="cuda:0")
    view = buf[offset:offset + raw.size]
    view.copy_(torch.from_numpy(raw))
    return view


def empty(count, dtype):
    import torch
    return torch.empty(count, dtype=dtype, device="cuda:0")


def x_for(fmt_x, oracle, xf):
    """x in the requested form: f32 as drawn, or the reference encoder's blocks of it."""
    if fmt_x == B.F32:
        return xf
    return oracle.encode(fmt_x, xf)


def x_values(fmt_x, oracle, x, cols):
    """The stored values of x as f32 (what a float64 reference reads)."""
    if fmt_x == B.F32:
        return oracle.decode(B.Q8_0, oracle.encode(B.Q8_0, x), cols)
    return oracle.decode(fmt_x, x, cols)


def gemv_gpu(fmt_a, fmt_x, a, x, rows, cols, want_sums=False, offset_a=0):
    import torch
    o = ops()
    da, dx = dev(a, offset_a), dev(x)
    y = empty(max(rows, 1), torch.float32)
    y.fill_(float("nan"))
    if want_sums:
        sums = empty(max(rows * (cols // 32), 1), torch.int32)
        lane = o.GemvBlockSums(fmt_a, da, dx, y, sums, rows, cols, fmt_x=fmt_x)
    else:
        lane = o.GemvBlocks(fmt_a, da, dx, y, rows, cols, fmt_x=fmt_x)
    assert o.gpu.status() == 0
    out = y.cpu().numpy()[:rows]
    if want_sums:
        return out, sums.cpu().numpy()[:rows * (cols // 32)].reshape(rows, cols // 32), lane
    return out, lane
