"""The reference's own acceptance gate for this path, restated: `Close` on the public operators.

`Checks.BlockProducts` (src/Checks.cs:1224-1266) forces the block product, runs MatMulView at 37 x 29 x {64, 320} and the
gemv at 37 x 64 for q8_0 and q4_0 on values uniform in [-1, 1], and compares the STORED output (after `Back`) with the
float64 reference encoded to the type, within `Close` (src/Checks.cs:1870-1930): two steps of the block (the block's
largest reference magnitude times 2^-mantissa, mantissas 6 and 2, src/Bench/Registry.cs:150-154) plus four lane ulps.
The repository's own bars are tighter (bit-exact lanes); this is the gate a maintainer of the reference would run.
.NET's Random(seed) streams are not reproducible here, so the inputs come from numpy generators over the same range.
"""
import numpy as np
import pytest

from qiyas_b200 import blocks as B

from . import helpers as H



MANTISSA = {B.Q8_0: 6, B.Q4_0: 2}            # src/Bench/Registry.cs:150-154


def close(oracle, fmt, output, reference, n):
    """src/Checks.cs:1870-1930 for a block format: worst excess over the tolerance in block steps (0 = passes)."""
    expected = oracle.decode(fmt, oracle.encode(fmt, reference.astype(np.float32)), n).astype(np.float64)
    got = oracle.decode(fmt, output, n).astype(np.float64)
    pad = (-n) % 32
    block_max = np.abs(np.concatenate([reference, np.zeros(pad)])).reshape(-1, 32).max(axis=1)
    block_max = np.repeat(np.where(block_max == 0, 1.0, block_max), 32)[:n]
    bstep = block_max * 2.0 ** -MANTISSA[fmt]
    tol = 2 * bstep + 4 * np.abs(reference) * 2.0 ** -23
    over = np.abs(got - expected) > tol
    return float(np.max(np.where(over, np.abs(got - expected) / bstep, 0.0)))


def make(oracle, fmt, count, seed):
    """Registry.Make(type, count, seed, -1, 1): floats uniform in [-1, 1] stored by the type."""
    return oracle.encode(fmt, np.random.default_rng(seed).uniform(-1, 1, count).astype(np.float32))


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", [B.Q8_0, B.Q4_0])
@pytest.mark.parametrize("k", [64, 320])
def test_block_product_gate(oracle, fmt, k):
    import torch
    from qiyas_b200.ops import ProductView
    o = H.ops()
    m, n = 37, 29
    a, b = make(oracle, fmt, m * k, 34), make(oracle, fmt, n * k, 35)
    v = ProductView(m, n, k, False, True)
    c = H.empty(B.nbytes(fmt, m * n), torch.uint8)
    o.BlockProducts = True                   # the gate forces the block product
    try:
        lane = o.MatMulView(B.NAMES[fmt], v, H.dev(a), H.dev(b), c)
    finally:
        o.BlockProducts = None
    assert lane == "s8 tcgen05 blocks" and o.gpu.status() == 0
    want = oracle.matmul_f64(fmt, fmt, a, b, m, n, k).reshape(-1)
    assert close(oracle, fmt, c.cpu().numpy(), want, m * n) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", [B.Q8_0, B.Q4_0])
def test_block_gemv_gate(oracle, fmt):
    import torch
    o = H.ops()
    m, k = 37, 64
    a, x = make(oracle, fmt, m * k, 44), make(oracle, fmt, k, 45)
    y = H.empty(B.nbytes(fmt, m), torch.uint8)
    lane = o.Gemv(B.NAMES[fmt], H.dev(a), H.dev(x), y, m, k)
    assert lane == "s8dp blocks" and o.gpu.status() == 0
    want = oracle.gemv_f64(fmt, a, oracle.decode(fmt, x, k), m, k)
    assert close(oracle, fmt, y.cpu().numpy(), want, m) == 0.0


def test_close_rejects_what_the_reference_would():
    # the tolerance function itself: three block steps off in one value is a failure, one step is not
    from oracle import qiyas_oracle as O
    ref = np.linspace(-1, 1, 64)
    stored = O.encode(B.Q8_0, ref.astype(np.float32))
    assert close(O, B.Q8_0, stored, ref, 64) == 0.0
    bad = stored.copy()
    bad[2 + 5] = np.uint8((int(np.int8(bad[2 + 5])) + 6) & 255)         # six codes = about three of the gate's steps (mantissa 6 against 7 bits of code)
    assert close(O, B.Q8_0, bad, ref, 64) > 2.0
