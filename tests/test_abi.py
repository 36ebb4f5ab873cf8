"""The C-ABI library loads and exports every symbol include/qiyas_b200.h declares (no GPU needed)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def library():
    from qiyas_b200 import build
    return ctypes.CDLL(build.build())


def declared_functions():
    text = open(os.path.join(ROOT, "include", "qiyas_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qb200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_surface():
    names = declared_functions()
    for must in ("qb200_init", "qb200_gemv_blocks", "qb200_matmul_blocks", "qb200_encode", "qb200_decode", "qb200_last_error"):
        assert must in names


def test_every_declared_symbol_is_exported(library):
    for name in declared_functions():
        assert hasattr(library, name), name


def test_binding_matches_header():
    from qiyas_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_calls_fail_loudly_without_a_device(library):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    library.qb200_last_error.restype = ctypes.c_char_p
    assert library.qb200_init(0) != 0
    assert library.qb200_last_error()
    # nothing runs on the CPU instead: the product entry points refuse
    assert library.qb200_gemv_blocks(0, 0, None, None, None, 4, 32, None) == -5
    assert library.qb200_matmul_blocks(0, 0, None, None, None, 4, 4, 32, None, 0, None) == -5
    # ... and so do the sharded ones, before they look at their peers
    from qiyas_b200 import _lib
    peers = _lib.ShardPeers()
    peers.world, peers.rank = 2, 0
    assert library.qb200_shard_gemv(0, 0, None, None, 8, 32, ctypes.byref(peers), 1, None) == -5
    assert library.qb200_shard_matmul(0, 0, None, None, None, 4, 8, 32, ctypes.byref(peers), 1, None, 0, None) == -5
    assert library.qb200_shard_wait(ctypes.byref(peers), 1, 0, None) == -5
    assert library.qb200_block_product_available() == 0


def test_packed_sizes_follow_the_layouts(library):
    # host arithmetic only: weights with f16 scales are packed in slabs of a 128-row tile and eight k-blocks (eight times
    # 4 KB of codes and 2 KB of scale rows); a call's workspace has room for A in its few-rows form as well
    import ctypes as C
    lib = library
    lib.qb200_matmul_prepacked_bytes.restype = C.c_size_t
    lib.qb200_matmul_prepacked_bytes.argtypes = [C.c_int, C.c_int, C.c_int]
    lib.qb200_matmul_prepacked_workspace_bytes.restype = C.c_size_t
    lib.qb200_matmul_prepacked_workspace_bytes.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int]
    for fmt in (0, 1):
        for n, k in ((11008, 4096), (129, 64), (1, 32), (300, 8160)):
            tiles, groups = (n + 127) // 128, (k // 32 + 7) // 8
            assert lib.qb200_matmul_prepacked_bytes(fmt, n, k) == (tiles * groups * 34816 + 255) // 256 * 256
    for m, k in ((1, 32), (16, 64), (64, 64), (33, 4096)):
        bn = 16 if m <= 16 else 32 if m <= 32 else 64
        few = (k // 32 + 7) // 8 * (8 * bn * 32 + 8 * bn * 16)
        assert lib.qb200_matmul_prepacked_workspace_bytes(0, 0, m, k) >= few
