"""Host-side mirror of the reference's operator surface for the block-scaled products.

``GpuOps`` keeps the names, argument meaning and error behaviour of the reference's C# class for
this path (src/BlockProducts.cs:175-187, src/MatMulBlocks.cs:389-443, src/GpuOps.cs:277-285) and
forwards every call through the C ABI of ``libqiyas_b200.so``.  Operands are device pointers
(ints, as the reference's ``ulong``) or CUDA ``torch`` tensors, whose ``data_ptr()`` is taken:
torch is used for device memory and streams only.

Errors follow the reference: a format or shape the block product does not take raises
``NotImplementedError`` (the reference's NotSupportedException); a CUDA failure raises
``RuntimeError`` (its InvalidOperationException).  Nothing here computes on the CPU.
"""
import ctypes as C
from dataclasses import dataclass

from . import _lib
from .blocks import BLOCK_VALUES, F32, NAMES, Q4_0, Q8_0, fmt_id, nbytes

OP_GEMV, OP_MATMUL = 0, 1


@dataclass(frozen=True)
class ProductView:
    """A product on views (src/Products.cs:15): C = op(A).op(B); the block product takes A.B^T, batch 1."""
    M: int
    N: int
    K: int
    TransA: bool = False
    TransB: bool = True
    Batch: int = 1
    StrideA: int = 0
    StrideB: int = 0
    StrideC: int = 0

    @property
    def ValuesC(self):
        """src/Products.cs:30: the values C spans over all the batch's products."""
        return self.M * self.N + (self.Batch - 1) * (self.StrideC if self.Batch > 1 else 0)


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return x.data_ptr()


def _stream(stream):
    if stream is None:
        return None
    if isinstance(stream, int):
        return stream or None
    return stream.cuda_stream or None


class Gpu:
    """The device binding for this path (stands where src/Gpu.cs stands in the reference): one device, bound once."""

    def __init__(self, device=0):
        self.lib = _lib.load()
        rc = self.lib.qb200_init(int(device))
        if rc:
            raise RuntimeError(f"qb200_init({device}): {self.error()}")
        self.device = int(device)
        caps = _lib.Caps()
        self.check(self.lib.qb200_caps(C.byref(caps)), "qb200_caps")
        self.caps = caps

    def error(self):
        return self.lib.qb200_last_error().decode()

    def check(self, rc, what):
        """Maps a return code as a C# shim would: format / shape / limit errors are the reference's NotSupportedException,
        other negative codes an argument error, positive codes a CUDA failure (its InvalidOperationException)."""
        if rc == 0:
            return
        if rc in (-1, -2, -6):
            raise NotImplementedError(self.error())
        if rc < 0:
            raise ValueError(self.error())
        raise RuntimeError(f"{what}: {self.error()}")

    def Synchronize(self):
        self.check(self.lib.qb200_synchronize(), "synchronize")

    def status(self):
        """Device status word (0 = every bounded wait inside the kernels completed); synchronizes."""
        value = C.c_int(0)
        self.check(self.lib.qb200_device_status(C.byref(value)), "device_status")
        return value.value


class GpuOps:
    """GemvBlocks / MatMulBlocks / Gemv / MatMulViewBlocks / MatMulView on block formats, as the reference names them."""

    def __init__(self, gpu=None, device=0):
        self.gpu = gpu if gpu is not None else Gpu(device)
        self.lib = self.gpu.lib
        self.BlockProducts = None          # the gate's override (src/MatMulBlocks.cs:406): True forces the block product
        self._scratch = {}

    # -- availability -------------------------------------------------------------------------
    @property
    def BlockProductAvailable(self):
        return bool(self.lib.qb200_block_product_available())

    def lane_name(self, op, fmt):
        return self.lib.qb200_lane_name(op, fmt_id(fmt)).decode()

    # -- gemv ----------------------------------------------------------------------------------
    def GemvBlocks(self, fmt, a, x, y, rows, cols, fmt_x=None, stream=None):
        """y (f32 lanes) = A.x; `fmt` names A's block type; x is in the same format unless `fmt_x` says otherwise."""
        fa = fmt_id(fmt)
        fx = fa if fmt_x is None else fmt_id(fmt_x)
        rc = self.lib.qb200_gemv_blocks(fa, fx, _ptr(a), _ptr(x), _ptr(y), int(rows), int(cols), _stream(stream))
        self.gpu.check(rc, "GemvBlocks")
        return self.lane_name(OP_GEMV, fa)

    def GemvBlockSums(self, fmt, a, x, y, sums, rows, cols, fmt_x=None, stream=None):
        fa = fmt_id(fmt)
        fx = fa if fmt_x is None else fmt_id(fmt_x)
        rc = self.lib.qb200_gemv_block_sums(fa, fx, _ptr(a), _ptr(x), _ptr(y), _ptr(sums), int(rows), int(cols), _stream(stream))
        self.gpu.check(rc, "GemvBlockSums")
        return self.lane_name(OP_GEMV, fa)

    def Gemv(self, fmt, a, x, y, rows, cols, transposed=False, stream=None):
        """The public gemv's block branch (src/GpuOps.cs:277-285): f32 lanes, then `Back` into y's block format."""
        fa = fmt_id(fmt)
        if fa not in (Q8_0, Q4_0) or transposed or cols % 32:
            raise NotImplementedError(f"{NAMES.get(fa, fa)}: only the block-scaled branch of Gemv is built here")
        lanes = self._rent(rows * 4)
        return self.GemvBlocksBack(fa, a, x, lanes, fa, y, rows, cols, stream=stream)

    def GemvBlocksBack(self, fmt, a, x, y_lanes, fmt_y, y_blocks, rows, cols, fmt_x=None, stream=None):
        """GemvBlocks and the `Back` of its result (src/GpuOps.cs:283-284) in one launch: f32 lanes and Q8_0 / Q4_0 blocks."""
        fa = fmt_id(fmt)
        fx = fa if fmt_x is None else fmt_id(fmt_x)
        rc = self.lib.qb200_gemv_blocks_back(fa, fx, _ptr(a), _ptr(x), _ptr(y_lanes), fmt_id(fmt_y), _ptr(y_blocks), int(rows),
                                             int(cols), _stream(stream))
        self.gpu.check(rc, "GemvBlocksBack")
        return self.lane_name(OP_GEMV, fa)

    # -- A.B^T ---------------------------------------------------------------------------------
    def MatMulBlocks(self, fmt, a, b, c_lanes, m, n, k, fmt_b=None, workspace=None, workspace_bytes=0, stream=None):
        """C (f32 lanes, m x n) = A.B^T; `fmt` names A's block type and B's unless `fmt_b` is given."""
        fa = fmt_id(fmt)
        fb = fa if fmt_b is None else fmt_id(fmt_b)
        rc = self.lib.qb200_matmul_blocks(fa, fb, _ptr(a), _ptr(b), _ptr(c_lanes), int(m), int(n), int(k), _ptr(workspace),
                                          int(workspace_bytes), _stream(stream))
        self.gpu.check(rc, "MatMulBlocks")
        return self.lane_name(OP_MATMUL, fa)

    def MatMulBlockSums(self, fmt, a, b, c_lanes, sums, m, n, k, fmt_b=None, stream=None):
        fa = fmt_id(fmt)
        fb = fa if fmt_b is None else fmt_id(fmt_b)
        rc = self.lib.qb200_matmul_block_sums(fa, fb, _ptr(a), _ptr(b), _ptr(c_lanes), _ptr(sums), int(m), int(n), int(k), _stream(stream))
        self.gpu.check(rc, "MatMulBlockSums")
        return self.lane_name(OP_MATMUL, fa)

    def workspace_bytes(self, fmt, m, n, k, fmt_b=None):
        fa = fmt_id(fmt)
        return int(self.lib.qb200_matmul_workspace_bytes(fa, fa if fmt_b is None else fmt_id(fmt_b), int(m), int(n), int(k)))

    def MatMulBlocksBack(self, fmt, a, b, c_lanes, fmt_c, c_blocks, m, n, k, fmt_b=None, workspace=None, workspace_bytes=0, stream=None):
        """MatMulBlocks and the `Back` of its result (src/MatMulBlocks.cs:418-421) in one call: f32 lanes and Q8_0 / Q4_0 blocks."""
        fa = fmt_id(fmt)
        fb = fa if fmt_b is None else fmt_id(fmt_b)
        rc = self.lib.qb200_matmul_blocks_back(fa, fb, _ptr(a), _ptr(b), _ptr(c_lanes), fmt_id(fmt_c), _ptr(c_blocks), int(m), int(n), int(k),
                                               _ptr(workspace), int(workspace_bytes), _stream(stream))
        self.gpu.check(rc, "MatMulBlocksBack")
        return self.lane_name(OP_MATMUL, fa)

    def Prepack(self, fmt_b, b, n, k, stream=None):
        """The weights re-laid once for the tensor cores: a device buffer that MatMulBlocksPrepacked takes in place of b."""
        import torch
        fb = fmt_id(fmt_b)
        need = int(self.lib.qb200_matmul_prepacked_bytes(fb, int(n), int(k)))
        if need == 0:
            raise NotImplementedError("the block product takes k in whole blocks of B")
        packed = torch.empty(need, dtype=torch.uint8, device=f"cuda:{self.gpu.device}")       # torch allocations are 256-byte aligned
        self.gpu.check(self.lib.qb200_matmul_prepack(fb, _ptr(b), int(n), int(k), packed.data_ptr(), need, _stream(stream)), "Prepack")
        return packed

    def MatMulBlocksPrepacked(self, fmt, a, b_packed, c_lanes, m, n, k, fmt_b=None, workspace=None, workspace_bytes=0, stream=None):
        fa = fmt_id(fmt)
        fb = fa if fmt_b is None else fmt_id(fmt_b)
        rc = self.lib.qb200_matmul_blocks_prepacked(fa, fb, _ptr(a), _ptr(b_packed), _ptr(c_lanes), int(m), int(n), int(k), _ptr(workspace),
                                                    int(workspace_bytes), _stream(stream))
        self.gpu.check(rc, "MatMulBlocksPrepacked")
        return self.lane_name(OP_MATMUL, fa)

    def MatMulBlocksBatched(self, fmt, a, b, c_lanes, m, n, k, batch, stride_a, stride_b, stride_c, fmt_b=None, stream=None):
        """`batch` products in one launch; strides in values as ProductView gives them (0 broadcasts an operand)."""
        fa = fmt_id(fmt)
        fb = fa if fmt_b is None else fmt_id(fmt_b)
        rc = self.lib.qb200_matmul_blocks_batched(fa, fb, _ptr(a), _ptr(b), _ptr(c_lanes), int(m), int(n), int(k), int(batch), int(stride_a),
                                                  int(stride_b), int(stride_c), None, 0, _stream(stream))
        self.gpu.check(rc, "MatMulBlocksBatched")
        return self.lane_name(OP_MATMUL, fa)

    def BlockView(self, fmt, v):
        """src/MatMulBlocks.cs:410-411, widened to batches whose operands start on whole blocks (the reference sends every
        batch to its decoded route)."""
        if not (fmt_id(fmt) in (Q8_0, Q4_0) and not v.TransA and v.TransB and v.K % 32 == 0 and self.BlockProductAvailable):
            return False
        if v.Batch == 1:
            return True
        return v.StrideA % 32 == 0 and v.StrideB % 32 == 0 and v.StrideC % 32 == 0 and v.StrideC >= v.M * v.N

    def MatMulViewBlocks(self, fmt, v, a, b, c, stream=None):
        """The block product for the view, C encoded to the type by blocks (src/MatMulBlocks.cs:414-424)."""
        if v.Batch == 1:
            lanes = self._rent(v.M * v.N * 4)
            return self.MatMulBlocksBack(fmt, a, b, lanes, fmt, c, v.M, v.N, v.K, stream=stream)
        lanes = self._rent(v.ValuesC * 4)
        if v.StrideC > v.M * v.N:             # values between two products' results belong to no product: they encode as zeros
            self.gpu.check(self.lib.qb200_memset(_ptr(lanes), 0, int(v.ValuesC * 4), _stream(stream)), "memset")
        lane = self.MatMulBlocksBatched(fmt, a, b, lanes, v.M, v.N, v.K, v.Batch, v.StrideA, v.StrideB, v.StrideC, stream=stream)
        self.Back(fmt, lanes, c, v.ValuesC, stream=stream)
        return lane

    def MatMulView(self, fmt, v, a, b, c, stream=None):
        """src/GpuOps.Products.cs:15-19: the block product where the view allows it.  The decoded route is not part of
        this library, so a view outside the block path, or `BlockProducts = False`, is not supported."""
        if self.BlockView(fmt, v) and self.UseBlocks(fmt, v):
            return self.MatMulViewBlocks(fmt, v, a, b, c, stream=stream)
        raise NotImplementedError("only A.B^T of two Q8_0 / Q4_0 operands with k in whole blocks is built here")

    def UseBlocks(self, fmt, v):
        """src/MatMulBlocks.cs:428-442 chooses between the block product and the decoded route by timing both once a
        shape; with one route built the choice is the gate's override alone: False refuses, True or None take the blocks."""
        return self.BlockProducts is not False

    def MatMulBackward(self, fmt, a, b, dc, da, db, m, n, k, stream=None):
        """src/GpuOps.Products.cs:101-106: dA = dC.B^T is the view (m, k, n, TransB) and takes the block product when n is
        whole blocks; dB = A^T.dC is a transposed-A view, which only the decoded route serves: pass db=None."""
        if db is not None:
            raise NotImplementedError("dB = A^T.dC is a view of the decoded route, which is not part of this library")
        return self.MatMulView(fmt, ProductView(m, k, n, False, True), dc, b, da, stream=stream)

    # -- codecs --------------------------------------------------------------------------------
    def Back(self, fmt, lanes, stored, count, stream=None):
        """f32 lanes -> blocks (src/GpuOps.cs:964-975)."""
        self.gpu.check(self.lib.qb200_encode(fmt_id(fmt), _ptr(lanes), _ptr(stored), int(count), _stream(stream)), "Back")

    def Lanes(self, fmt, stored, lanes, count, stream=None):
        """blocks -> f32 lanes, the Widen kernel (src/GpuOps.cs:948-962)."""
        self.gpu.check(self.lib.qb200_decode(fmt_id(fmt), _ptr(stored), _ptr(lanes), int(count), _stream(stream)), "Lanes")

    # -- host-buffer form (upload, product, download), for callers that hold numpy arrays ---------
    def GemvBlocksHost(self, fmt, a, x, y, rows, cols, fmt_x=None):
        fa = fmt_id(fmt)
        fx = fa if fmt_x is None else fmt_id(fmt_x)
        rc = self.lib.qb200_gemv_blocks_host(fa, fx, a.ctypes.data, x.ctypes.data, y.ctypes.data, int(rows), int(cols))
        self.gpu.check(rc, "GemvBlocksHost")
        return self.lane_name(OP_GEMV, fa)

    # -- the reference's Rent: a kept f32 lane buffer per size class -------------------------------
    def _rent(self, nbytes_):
        import torch
        size = max(256, (int(nbytes_) + 255) // 256 * 256)
        buf = self._scratch.get("lanes")
        if buf is None or buf.numel() < size:
            buf = torch.empty(size, dtype=torch.uint8, device=f"cuda:{self.gpu.device}")
            self._scratch["lanes"] = buf
        return buf


__all__ = ["Gpu", "GpuOps", "ProductView", "OP_GEMV", "OP_MATMUL", "BLOCK_VALUES", "F32", "nbytes"]
