"""Device codecs against the C oracle: decode bit for bit, encode byte for byte (the reference's own gate between its
device and CPU codecs, src/Checks.cs:231-254)."""
import numpy as np
import pytest

from qiyas_b200 import blocks as B

from . import helpers as H

pytestmark = pytest.mark.gpu

FORMATS = [B.Q8_0, B.Q4_0, B.Q4_K, B.Q6_K]


def gate_values(n, seed):
    rng = np.random.default_rng(seed)
    return ((rng.random(n) * 8 - 4) * np.where(np.arange(n) % 7 == 0, 0.01, 1.0)).astype(np.float32)


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("n", [1, 31, 32, 256, 1001, 70000])
def test_encode_equals_cpu_encoder(oracle, fmt, n):
    import torch
    values = gate_values(n, 99 + n)
    want = oracle.encode(fmt, values, device_rounding=True)
    out = H.empty(want.size, torch.uint8)
    H.ops().Back(fmt, H.dev(values), out, n)
    assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("fmt", FORMATS)
def test_encode_special_blocks(oracle, fmt):
    import torch
    bv = B.BLOCK_VALUES[fmt]
    values = np.zeros(bv * 4, np.float32)
    values[bv:2 * bv] = 1e-7                       # scales that underflow f16
    values[2 * bv:3 * bv] = np.linspace(-3, 3, bv)
    values[3 * bv] = -65000.0
    want = oracle.encode(fmt, values, device_rounding=True)
    out = H.empty(want.size, torch.uint8)
    H.ops().Back(fmt, H.dev(values), out, values.size)
    assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("n", [1, 255, 1001, 65536 + 17])
def test_decode_equals_cpu_decoder(oracle, fmt, n):
    import torch
    rows = (n + B.BLOCK_VALUES[fmt] - 1) // B.BLOCK_VALUES[fmt]
    stored = B.make_weights(fmt, rows, B.BLOCK_VALUES[fmt], 5 + n)
    want = oracle.decode(fmt, stored, n)
    lanes = H.empty(n, torch.float32)
    H.ops().Lanes(fmt, H.dev(stored), lanes, n)
    assert np.array_equal(lanes.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("fmt", FORMATS)
def test_round_trip_on_device(oracle, fmt):
    import torch
    n = 1001
    values = gate_values(n, 99)
    stored = H.empty(B.nbytes(fmt, n), torch.uint8)
    lanes = H.empty(n, torch.float32)
    o = H.ops()
    o.Back(fmt, H.dev(values), stored, n)
    o.Lanes(fmt, stored, lanes, n)
    back = lanes.cpu().numpy()
    mant = {B.Q8_0: 6, B.Q4_0: 2, B.Q4_K: 2, B.Q6_K: 4}[fmt]
    bv = B.BLOCK_VALUES[fmt]
    for i in range(n):
        lo = i // bv * bv
        step = np.max(np.abs(values[lo:min(n, lo + bv)])) * 2.0 ** -mant + 1e-30
        assert abs(float(back[i]) - float(values[i])) <= 1.5 * step
