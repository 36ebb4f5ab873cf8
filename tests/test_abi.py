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
    assert library.qb200_block_product_available() == 0
