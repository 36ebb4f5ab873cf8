"""The products of the reference's known-answer blocks, in closed form (tests/golden/kat_products.json).

The reference pins its codecs with hand-laid blocks (src/Checks.cs:264-355) but holds no product vector; the golden file
carries the products those blocks give by plain integer arithmetic (tests/golden/make_kat_products.py).  Every expected
value is exact in f32, so the CPU restatement (both summation orders), the integer sums and the CUDA kernels must all
reproduce them bit for bit.
"""
import json
import os

import numpy as np
import pytest

from qiyas_b200 import blocks as B

from . import helpers as H

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = json.load(open(os.path.join(HERE, "golden", "kat_products.json")))["cases"]
GEMV = [c for c in CASES if c["op"] == "gemv"]
MATMUL = [c for c in CASES if c["op"] == "matmul"]


def ident(c):
    return f"{c['op']}-{B.NAMES[c.get('fmt_b', c.get('fmt_a'))]}-{c.get('rows', c.get('m'))}x{c.get('cols', c.get('k'))}"


def raw(hexed):
    return np.frombuffer(bytes.fromhex(hexed), np.uint8).copy()


def test_the_golden_file_is_what_its_script_writes(tmp_path):
    # the committed vectors are reproducible from the committed derivation
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_kat_products", os.path.join(HERE, "golden", "make_kat_products.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    first = mod.gemv_case(B.Q8_0, 1, 32)
    assert first == GEMV[0] and first["sums"] == [[2736]] and first["y"] == [684.0]       # 0.25 * sum (i - 16)^2
    assert mod.matmul_case(B.Q4_K, 3, 5, 256) == [c for c in MATMUL if c["fmt_b"] == B.Q4_K][0]


@pytest.mark.parametrize("case", GEMV, ids=ident)
def test_oracle_gemv_reproduces_the_known_answers(oracle, case):
    fmt, rows, cols = case["fmt_a"], case["rows"], case["cols"]
    a, x = raw(case["a"]), raw(case["x"])
    want = np.array(case["y"], np.float32)
    sums = np.array(case["sums"], np.int32)
    xv = oracle.decode(B.Q8_0, x, cols)
    assert np.array_equal(oracle.gemv_f64(fmt, a, xv, rows, cols), want.astype(np.float64))
    if fmt in (B.Q8_0, B.Q4_0):
        for order in (0, 1):                 # the CPU's rounding order and the device kernel's
            y, s = oracle.gemv_blocks(fmt, B.Q8_0, a, x, rows, cols, order=order, want_sums=True)
            assert np.array_equal(s, sums)
            assert np.array_equal(y.view(np.uint32), want.view(np.uint32))
    else:
        xq = x.reshape(-1, 34)[:, 2:].reshape(-1).view(np.int8)
        assert np.array_equal(oracle.k_block_sums(fmt, a, xq, rows, cols), sums)
        assert np.array_equal(oracle.gemv_decoded_f32(fmt, a, xv, rows, cols).view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("case", MATMUL, ids=ident)
def test_oracle_matmul_reproduces_the_known_answers(oracle, case):
    fmt_b, m, n, k = case["fmt_b"], case["m"], case["n"], case["k"]
    a, b = raw(case["a"]), raw(case["b"])
    want = np.array(case["c"], np.float32)
    sums = np.array(case["sums"], np.int32)
    assert np.array_equal(oracle.matmul_f64(B.Q8_0, fmt_b, a, b, m, n, k), want.astype(np.float64))
    if fmt_b in (B.Q8_0, B.Q4_0):
        for order in (0, 1):
            got = oracle.matmul_blocks(B.Q8_0, fmt_b, a, b, m, n, k, order=order, want_sums=order == 1)
            c = got[0] if order == 1 else got
            assert np.array_equal(c.view(np.uint32), want.view(np.uint32))
            if order == 1:
                assert np.array_equal(got[1], sums)
    else:
        fn = oracle.matmul_q4_k if fmt_b == B.Q4_K else oracle.matmul_q6_k
        c, s = fn(B.Q8_0, a, b, m, n, k, want_sums=True)
        assert np.array_equal(s, sums)
        assert np.array_equal(c.view(np.uint32), want.view(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("case", GEMV, ids=ident)
def test_gpu_gemv_reproduces_the_known_answers(case):
    fmt, rows, cols = case["fmt_a"], case["rows"], case["cols"]
    a, x = raw(case["a"]), raw(case["x"])
    want = np.array(case["y"], np.float32)
    y, sums, _ = H.gemv_gpu(fmt, B.Q8_0, a, x, rows, cols, want_sums=True)
    assert np.array_equal(sums, np.array(case["sums"], np.int32))
    assert np.array_equal(y.view(np.uint32), want.view(np.uint32))
    y, _ = H.gemv_gpu(fmt, B.Q8_0, a, x, rows, cols)
    assert np.array_equal(y.view(np.uint32), want.view(np.uint32))
    # x as f32: the in-kernel encoder must recover the same Q8_0 blocks (values d q with d = 0.5 are exact in the encoding)


@pytest.mark.gpu
@pytest.mark.parametrize("case", MATMUL, ids=ident)
def test_gpu_matmul_reproduces_the_known_answers(case):
    import torch
    fmt_b, m, n, k = case["fmt_b"], case["m"], case["n"], case["k"]
    a, b = raw(case["a"]), raw(case["b"])
    want = np.array(case["c"], np.float32)
    sums = np.array(case["sums"], np.int32)
    o = H.ops()
    da, db = H.dev(a), H.dev(b)
    c = H.empty(m * n, torch.float32)
    got_sums = H.empty(sums.size, torch.int32)
    o.MatMulBlockSums(B.Q8_0, da, db, c, got_sums, m, n, k, fmt_b=fmt_b)
    assert o.gpu.status() == 0
    assert np.array_equal(got_sums.cpu().numpy().reshape(sums.shape), sums)
    assert np.array_equal(c.cpu().numpy().reshape(m, n).view(np.uint32), want.view(np.uint32))
    c.fill_(float("nan"))
    o.MatMulBlocks(B.Q8_0, da, db, c, m, n, k, fmt_b=fmt_b)
    assert o.gpu.status() == 0
    assert np.array_equal(c.cpu().numpy().reshape(m, n).view(np.uint32), want.view(np.uint32))
