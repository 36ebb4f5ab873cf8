"""qiyas_b200: the block-scaled quantized products of Qiyas (gemv and A.B^T over Q8_0, Q4_0, Q4_K, Q6_K) as
hand-written sm_100a CUDA kernels behind a C ABI (libqiyas_b200.so), with a host mirror of the reference's operators."""
from . import blocks
from .blocks import F32, Q4_0, Q4_K, Q6_K, Q8_0

__all__ = ["blocks", "Q8_0", "Q4_0", "Q4_K", "Q6_K", "F32", "GpuOps", "Gpu", "ProductView"]


def __getattr__(name):
    # the operators bind the CUDA library on first use; importing the package alone needs no GPU
    if name in ("GpuOps", "Gpu", "ProductView"):
        from . import ops
        return getattr(ops, name)
    raise AttributeError(name)
