"""numpy front end of the C oracle (``qiyas_oracle.c``): test infrastructure only.

Each function hands numpy buffers to the C restatement of the reference's CPU arithmetic and
returns numpy arrays.  Formats are the integers of ``include/qiyas_b200.h``.
"""
import ctypes as C
import os

import numpy as np

Q8_0, Q4_0, Q4_K, Q6_K, F32 = 0, 1, 2, 3, 100
BLOCK_VALUES = {Q8_0: 32, Q4_0: 32, Q4_K: 256, Q6_K: 256}
BLOCK_BYTES = {Q8_0: 34, Q4_0: 18, Q4_K: 144, Q6_K: 210}

_lib = None


def lib():
    global _lib
    if _lib is None:
        from . import build as _build
        path = _build.LIBRARY
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(_build.SOURCE):
            path = _build.build()
        _lib = C.CDLL(path)
        _lib.qo_half_to_float.restype = C.c_float
        _lib.qo_half_to_float.argtypes = [C.c_uint16]
        _lib.qo_float_to_half.restype = C.c_uint16
        _lib.qo_float_to_half.argtypes = [C.c_float]
        _lib.qo_bytes.restype = C.c_int64
        _lib.qo_bytes.argtypes = [C.c_int, C.c_int64]
        _lib.qo_now.restype = C.c_double
        _lib.qo_time_gemv_blocks.restype = C.c_double
        _lib.qo_time_gemv_blocks.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        _lib.qo_set_dot_variant.argtypes = [C.c_int]
        _lib.qo_dot_variant_available.argtypes = [C.c_int]
        _lib.qo_decode.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_void_p]
        _lib.qo_encode.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_void_p, C.c_int]
        _lib.qo_gemv_blocks.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                        C.c_void_p, C.c_void_p]
        _lib.qo_k_block_sums.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        _lib.qo_gemv_f64.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        _lib.qo_gemv_decoded_f32.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        _lib.qo_matmul_blocks.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                          C.c_int, C.c_void_p]
        _lib.qo_matmul_f64.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        _lib.qo_matmul_q4_k.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        _lib.qo_matmul_q6_k.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _bytes(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(-1)


def nbytes(fmt, values):
    return int(lib().qo_bytes(fmt, values))


def threads():
    return int(lib().qo_team_size())


def set_dot_variant(variant):
    """The CPU gemv's integer dot: 0 the plain loop (the reference's "s32 blocks" lane), 1 AVX2 widening multiply-adds
    (standing in for its "s8dp blocks" vector lane).  Same results bit for bit; returns False when the host lacks AVX2."""
    if not lib().qo_dot_variant_available(int(variant)):
        return False
    lib().qo_set_dot_variant(int(variant))
    return True


def half_to_float(h):
    return float(lib().qo_half_to_float(int(h)))


def float_to_half(f):
    return int(lib().qo_float_to_half(float(f)))


def decode(fmt, blocks, count):
    blocks = _bytes(blocks)
    out = np.empty(count, np.float32)
    if lib().qo_decode(fmt, _ptr(blocks), count, _ptr(out)):
        raise ValueError("decode: not a block format")
    return out


def encode(fmt, values, device_rounding=False):
    values = np.ascontiguousarray(values, np.float32).reshape(-1)
    out = np.zeros(nbytes(fmt, values.size), np.uint8)
    if lib().qo_encode(fmt, _ptr(values), values.size, _ptr(out), 1 if device_rounding else 0):
        raise ValueError("encode: not a block format")
    return out


def gemv_blocks(fmt_a, fmt_x, a, x, rows, cols, order=1, want_sums=False, want_abs=False):
    """y (f32) for A in Q8_0/Q4_0 and x in Q8_0/Q4_0/f32; order 0 = CPU rounding order, 1 = device order."""
    a = _bytes(a)
    x = np.ascontiguousarray(x, np.float32) if fmt_x == F32 else _bytes(x)
    y = np.empty(rows, np.float32)
    sums = np.empty((rows, cols // 32), np.int32) if want_sums else None
    mag = np.empty(rows, np.float64) if want_abs else None
    if lib().qo_gemv_blocks(fmt_a, fmt_x, _ptr(a), _ptr(x), _ptr(y), rows, cols, order, _ptr(sums), _ptr(mag)):
        raise ValueError("gemv_blocks: the block product takes Q8_0 or Q4_0 with columns in whole blocks")
    out = [y]
    if want_sums:
        out.append(sums)
    if want_abs:
        out.append(mag)
    return out[0] if len(out) == 1 else tuple(out)


def k_block_sums(fmt_a, a, xq, rows, cols):
    a = _bytes(a)
    xq = np.ascontiguousarray(xq, np.int8)
    sums = np.empty((rows, cols // 32), np.int32)
    if lib().qo_k_block_sums(fmt_a, _ptr(a), _ptr(xq), rows, cols, _ptr(sums)):
        raise ValueError("k_block_sums: Q4_K or Q6_K with columns in whole super-blocks")
    return sums


def gemv_f64(fmt_a, a, x, rows, cols):
    a = _bytes(a)
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty(rows, np.float64)
    if lib().qo_gemv_f64(fmt_a, _ptr(a), _ptr(x), _ptr(y), rows, cols):
        raise ValueError("gemv_f64: columns in whole blocks")
    return y


def gemv_decoded_f32(fmt_a, a, x, rows, cols):
    a = _bytes(a)
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty(rows, np.float32)
    if lib().qo_gemv_decoded_f32(fmt_a, _ptr(a), _ptr(x), _ptr(y), rows, cols):
        raise ValueError("gemv_decoded_f32: columns in whole blocks")
    return y


def matmul_blocks(fmt_a, fmt_b, a, b, m, n, k, order=1, want_sums=False):
    a, b = _bytes(a), _bytes(b)
    c = np.empty((m, n), np.float32)
    sums = np.empty((m, n, k // 32), np.int32) if want_sums else None
    if lib().qo_matmul_blocks(fmt_a, fmt_b, _ptr(a), _ptr(b), _ptr(c), m, n, k, order, _ptr(sums)):
        raise ValueError("matmul_blocks: the block product takes Q8_0 or Q4_0 with k in whole blocks")
    return (c, sums) if want_sums else c


def matmul_q4_k(fmt_a, a, b, m, n, k, want_sums=False):
    """C (f32) = A.B^T for A in Q8_0 / Q4_0 and B in Q4_K, in the order this repo's device kernel defines (see the C file)."""
    a, b = _bytes(a), _bytes(b)
    c = np.empty((m, n), np.float32)
    sums = np.empty((m, n, k // 32), np.int32) if want_sums else None
    if lib().qo_matmul_q4_k(fmt_a, _ptr(a), _ptr(b), _ptr(c), m, n, k, _ptr(sums)):
        raise ValueError("matmul_q4_k: A in Q8_0 or Q4_0, k in whole super-blocks of 256")
    return (c, sums) if want_sums else c


def matmul_q6_k(fmt_a, a, b, m, n, k, want_sums=False):
    """C (f32) = A.B^T for A in Q8_0 / Q4_0 and B in Q6_K, in the order this repo's device kernel defines (see the C file)."""
    a, b = _bytes(a), _bytes(b)
    c = np.empty((m, n), np.float32)
    sums = np.empty((m, n, k // 16), np.int32) if want_sums else None
    if lib().qo_matmul_q6_k(fmt_a, _ptr(a), _ptr(b), _ptr(c), m, n, k, _ptr(sums)):
        raise ValueError("matmul_q6_k: A in Q8_0 or Q4_0, k in whole super-blocks of 256")
    return (c, sums) if want_sums else c


def matmul_f64(fmt_a, fmt_b, a, b, m, n, k):
    a, b = _bytes(a), _bytes(b)
    c = np.empty((m, n), np.float64)
    if lib().qo_matmul_f64(fmt_a, fmt_b, _ptr(a), _ptr(b), _ptr(c), m, n, k):
        raise ValueError("matmul_f64: k in whole blocks")
    return c


def time_gemv_blocks(fmt_a, fmt_x, a, x, rows, cols, reps):
    """Seconds per call of the CPU block gemv on the thread team (the bench's CPU baseline)."""
    a = _bytes(a)
    x = np.ascontiguousarray(x, np.float32) if fmt_x == F32 else _bytes(x)
    y = np.empty(rows, np.float32)
    return float(lib().qo_time_gemv_blocks(fmt_a, fmt_x, _ptr(a), _ptr(x), _ptr(y), rows, cols, reps))
