"""ctypes binding of libqiyas_b200.so: exactly the entry points of include/qiyas_b200.h.

There is no Python or CPU fallback behind any of them: a missing library raises here, and a
machine without an sm_100 device makes qb200_init fail.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY = os.path.join(HERE, "libqiyas_b200.so")


SHARD_MAX = 8


class ShardPeers(C.Structure):
    """qb200_shard_peers_t: every rank's output vector and flag array as this process addresses them."""
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("out", C.c_void_p * SHARD_MAX), ("flags", C.c_void_p * SHARD_MAX)]


class Caps(C.Structure):
    _fields_ = [("device", C.c_int), ("sm_major", C.c_int), ("sm_minor", C.c_int), ("sm_count", C.c_int),
                ("tcgen05", C.c_int), ("max_shared_bytes", C.c_int), ("l2_bytes", C.c_int64), ("global_bytes", C.c_int64)]


_P, _I, _Z, _L = C.c_void_p, C.c_int, C.c_size_t, C.c_int64

SIGNATURES = {
    "qb200_init": (_I, [_I]),
    "qb200_caps": (_I, [C.POINTER(Caps)]),
    "qb200_last_error": (C.c_char_p, []),
    "qb200_block_product_available": (_I, []),
    "qb200_lane_name": (C.c_char_p, [_I, _I]),
    "qb200_device_status": (_I, [C.POINTER(_I)]),
    "qb200_gemv_blocks": (_I, [_I, _I, _P, _P, _P, _I, _I, _P]),
    "qb200_gemv_blocks_back": (_I, [_I, _I, _P, _P, _P, _I, _P, _I, _I, _P]),
    "qb200_gemv_block_sums": (_I, [_I, _I, _P, _P, _P, _P, _I, _I, _P]),
    "qb200_gemv_blocks_host": (_I, [_I, _I, _P, _P, _P, _I, _I]),
    "qb200_gemv_blocks_noalloc": (_I, [_I, _I, _P, _P, _P, _I, _I, _P]),
    "qb200_gemv_noalloc_status": (_I, [C.POINTER(_I)]),
    "qb200_matmul_workspace_bytes": (_Z, [_I, _I, _I, _I, _I]),
    "qb200_matmul_blocks": (_I, [_I, _I, _P, _P, _P, _I, _I, _I, _P, _Z, _P]),
    "qb200_matmul_blocks_back": (_I, [_I, _I, _P, _P, _P, _I, _P, _I, _I, _I, _P, _Z, _P]),
    "qb200_matmul_prepacked_bytes": (_Z, [_I, _I, _I]),
    "qb200_matmul_prepack": (_I, [_I, _P, _I, _I, _P, _Z, _P]),
    "qb200_matmul_prepacked_workspace_bytes": (_Z, [_I, _I, _I, _I]),
    "qb200_matmul_blocks_prepacked": (_I, [_I, _I, _P, _P, _P, _I, _I, _I, _P, _Z, _P]),
    "qb200_matmul_batched_workspace_bytes": (_Z, [_I, _I, _I, _I, _I, _I, _L, _L]),
    "qb200_matmul_blocks_batched": (_I, [_I, _I, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _P, _Z, _P]),
    "qb200_matmul_block_sums": (_I, [_I, _I, _P, _P, _P, _P, _I, _I, _I, _P]),
    "qb200_shard_range": (_I, [_I, _I, _I, C.POINTER(_I), C.POINTER(_I)]),
    "qb200_shard_gemv": (_I, [_I, _I, _P, _P, _I, _I, C.POINTER(ShardPeers), C.c_uint, _P]),
    "qb200_shard_matmul": (_I, [_I, _I, _P, _P, _P, _I, _I, _I, C.POINTER(ShardPeers), C.c_uint, _P, _Z, _P]),
    "qb200_shard_wait": (_I, [C.POINTER(ShardPeers), C.c_uint, C.c_longlong, _P]),
    "qb200_shard_gemv_after": (_I, [_I, _I, _P, _P, _I, _I, C.POINTER(ShardPeers), C.c_uint, C.POINTER(ShardPeers), C.c_uint, C.c_longlong, _P]),
    "qb200_ipc_export": (_I, [_P, _P]),
    "qb200_ipc_import": (_I, [_P, C.POINTER(_P)]),
    "qb200_ipc_close": (_I, [_P]),
    "qb200_tensor_rate": (_I, [C.POINTER(C.c_double)]),
    "qb200_encode": (_I, [_I, _P, _P, _L, _P]),
    "qb200_decode": (_I, [_I, _P, _P, _L, _P]),
    "qb200_malloc": (_I, [C.POINTER(_P), _Z]),
    "qb200_free": (_I, [_P]),
    "qb200_malloc_host": (_I, [C.POINTER(_P), _Z]),
    "qb200_free_host": (_I, [_P]),
    "qb200_memcpy_h2d": (_I, [_P, _P, _Z, _P]),
    "qb200_memcpy_d2h": (_I, [_P, _P, _Z, _P]),
    "qb200_memset": (_I, [_P, _I, _Z, _P]),
    "qb200_synchronize": (_I, []),
}

_lib = None


def load():
    """The loaded library with typed entry points; raises when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIBRARY):
            raise ImportError(f"{LIBRARY} is missing: run `python -m qiyas_b200.build` (nvcc, sm_100a); there is no fallback path")
        lib = C.CDLL(LIBRARY)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
