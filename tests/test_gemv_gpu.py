"""Parity of the CUDA gemv with the C oracle, through the C ABI.

Gates, in the order the task states them: every block's s32 sum bit-exact; f32 outputs within 1e-5
(relative to the row's sum of |terms| and, norm-wise, to max|y|) of the reference's device-order
block product (src/BlockProducts.cs:158-161) and of its CPU order (src/BlockProducts.cs:50); and an
error against float64 on the stored values (Program.cs:946-952) no larger than the reference's.
"""
import numpy as np
import pytest

from qiyas_b200 import blocks as B

from . import helpers as H

pytestmark = pytest.mark.gpu

REL = 1e-5     # the tolerance the task states for f32 lanes


def check_q(oracle, fmt_a, fmt_x, rows, cols, seed, offset_a=0, strict_f64=True):
    a = B.make_weights(fmt_a, rows, cols, seed)
    xf = B.make_activations(cols, seed + 1)
    x = H.x_for(fmt_x, oracle, xf)
    y, sums, lane = H.gemv_gpu(fmt_a, fmt_x, a, x, rows, cols, want_sums=True, offset_a=offset_a)
    y_plain, _ = H.gemv_gpu(fmt_a, fmt_x, a, x, rows, cols, offset_a=offset_a)
    assert lane == "s8dp blocks"
    assert np.array_equal(y.view(np.uint32), y_plain.view(np.uint32))      # the sums variant changes nothing in y
    ref_dev, ref_sums, mag = oracle.gemv_blocks(fmt_a, fmt_x, a, x, rows, cols, order=1, want_sums=True, want_abs=True)
    ref_cpu = oracle.gemv_blocks(fmt_a, fmt_x, a, x, rows, cols, order=0)
    assert np.array_equal(sums, ref_sums)
    for ref in (ref_dev, ref_cpu):
        assert np.all(np.abs(y.astype(np.float64) - ref) <= REL * mag + 1e-30)
        assert np.max(np.abs(y.astype(np.float64) - ref)) <= REL * np.max(np.abs(ref))
    y64 = oracle.gemv_f64(fmt_a, a, H.x_values(fmt_x, oracle, x, cols), rows, cols)
    err_gpu, err_ref = np.abs(y - y64), np.abs(ref_dev - y64)
    if strict_f64 and rows * cols >= 1 << 20:
        assert np.sqrt(np.mean(err_gpu ** 2)) <= np.sqrt(np.mean(err_ref ** 2))
        assert np.max(err_gpu) <= np.max(err_ref)
    else:
        assert np.max(err_gpu) <= max(np.max(err_ref), REL * np.max(np.abs(y64)))


@pytest.mark.parametrize("fmt_a", [B.Q8_0, B.Q4_0])
@pytest.mark.parametrize("fmt_x", ["same", B.Q8_0, B.F32])
def test_gate_shape_37x64(oracle, fmt_a, fmt_x):
    # the reference's own gemv gate shape (src/Checks.cs:1251-1256)
    check_q(oracle, fmt_a, fmt_a if fmt_x == "same" else fmt_x, 37, 64, 44)


@pytest.mark.parametrize("fmt_a", [B.Q8_0, B.Q4_0])
@pytest.mark.parametrize("rows,cols", [(1, 32), (3, 64), (2, 96), (37, 320), (61, 2080), (131, 4064), (257, 8160), (64, 11008), (5, 65536)])
def test_small_and_ragged_shapes(oracle, fmt_a, rows, cols):
    check_q(oracle, fmt_a, B.F32, rows, cols, 7 + rows)


@pytest.mark.parametrize("offset", [2, 6, 14, 18])
@pytest.mark.parametrize("fmt_a", [B.Q8_0, B.Q4_0])
def test_operand_alignment_of_two_bytes(oracle, fmt_a, offset):
    check_q(oracle, fmt_a, B.F32, 67, 1056, 21, offset_a=offset)


def test_config_q8_0_4096(oracle):
    check_q(oracle, B.Q8_0, B.F32, 4096, 4096, 100)


def test_config_q8_0_odd_4093x4064(oracle):
    check_q(oracle, B.Q8_0, B.F32, 4093, 4064, 101)


def test_config_q4_0_8192(oracle):
    check_q(oracle, B.Q4_0, B.F32, 8192, 8192, 102)


def test_config_q4_0_odd_8191x8160(oracle):
    check_q(oracle, B.Q4_0, B.F32, 8191, 8160, 103)


def test_many_chunks_per_block_back_to_back(oracle):
    # 28672 x 8192 (the sharded configuration's matrix): every block's ring slots are reused many times, and three
    # launches in a row that share y make each kernel a dependent of the one before
    import torch
    rows, cols = 28672, 8192
    a = B.make_weights(B.Q4_0, rows, cols, 400)
    xf = B.make_activations(cols, 401)
    o = H.ops()
    da, dx = H.dev(a), H.dev(xf)
    y = H.empty(rows, torch.float32)
    for _ in range(3):
        o.GemvBlocks(B.Q4_0, da, dx, y, rows, cols, fmt_x=B.F32)
    assert o.gpu.status() == 0
    ref, mag = oracle.gemv_blocks(B.Q4_0, B.F32, a, xf, rows, cols, order=1, want_abs=True)
    assert np.all(np.abs(y.cpu().numpy().astype(np.float64) - ref) <= REL * mag)


@pytest.mark.parametrize("fmt_a,rows,cols", [
    (B.Q8_0, 4096, 4096), (B.Q8_0, 1021, 4064), (B.Q4_0, 8192, 8192), (B.Q4_0, 2049, 8160), (B.Q4_0, 300, 16384),
    (B.Q4_0, 64, 32768), (B.Q4_K, 4096, 4096), (B.Q4_K, 1030, 11008), (B.Q6_K, 4096, 4096), (B.Q6_K, 1030, 11008),
    (B.Q6_K, 515, 2304), (B.Q4_0, 28672, 8192)])
def test_independent_calls_in_a_row(oracle, fmt_a, rows, cols):
    # six calls that share no output: from the second on each is independent of the launch before it and takes the
    # variant of four small blocks an SM, whose blocks run beside those of the neighbouring launches; then three calls
    # into one y, which go back to the whole-SM variant.  Every output is checked.
    import torch
    n = 6
    ws = [B.make_weights(fmt_a, rows, cols, 900 + i) for i in range(2)]
    xf = B.make_activations(cols, 910)
    o = H.ops()
    dws, dx = [H.dev(w) for w in ws], H.dev(xf)
    ys = [H.empty(rows, torch.float32) for _ in range(n)]
    for i in range(n):
        o.GemvBlocks(fmt_a, dws[i % 2], dx, ys[i], rows, cols, fmt_x=B.F32)
    for i in range(3):
        o.GemvBlocks(fmt_a, dws[i % 2], dx, ys[0], rows, cols, fmt_x=B.F32)
    assert o.gpu.status() == 0
    if fmt_a in (B.Q8_0, B.Q4_0):
        refs = [oracle.gemv_blocks(fmt_a, B.F32, w, xf, rows, cols, order=1, want_abs=True) for w in ws]
    else:                      # K-quant rows: float64 on the stored values of the matrix and of x as Q8_0
        xv = H.x_values(B.F32, oracle, xf, cols)
        refs = []
        for w in ws:
            y64 = oracle.gemv_f64(fmt_a, w, xv, rows, cols)
            refs.append((y64, np.max(np.abs(y64))))
    for i in range(n):
        ref, mag = refs[i % 2]
        assert np.all(np.abs(ys[i].cpu().numpy().astype(np.float64) - ref) <= REL * mag), i
    assert np.array_equal(ys[2].cpu().numpy(), ys[4].cpu().numpy())


def test_reference_signature_same_format(oracle):
    # GemvBlocks<TN>(a, x, y, rows, cols): x in a's format (src/BlockProducts.cs:178)
    for fmt in (B.Q8_0, B.Q4_0):
        check_q(oracle, fmt, fmt, 515, 2048, 55)


def test_zero_rows_and_errors():
    import torch
    o = H.ops()
    y = H.empty(4, torch.float32)
    a = H.empty(64, torch.uint8)
    assert o.GemvBlocks("q8_0", a, a, y, 0, 32) == "s8dp blocks"
    with pytest.raises(NotImplementedError):
        o.GemvBlocks("q8_0", a, a, y, 1, 33)                # columns not in whole blocks
    with pytest.raises(NotImplementedError):
        o.GemvBlocks("f32", a, a, y, 1, 32)                 # not a block format
    with pytest.raises(NotImplementedError):
        o.GemvBlocks("q4_k", a, a, y, 1, 256, fmt_x="q4_0")  # K-quant rows take Q8_0 or f32 x


def test_repeatable_bit_for_bit(oracle):
    a = B.make_weights(B.Q4_0, 1000, 4096, 9)
    x = B.make_activations(4096, 10)
    first, _ = H.gemv_gpu(B.Q4_0, B.F32, a, x, 1000, 4096)
    for _ in range(5):
        again, _ = H.gemv_gpu(B.Q4_0, B.F32, a, x, 1000, 4096)
        assert np.array_equal(first.view(np.uint32), again.view(np.uint32))


# ---- Q4_K / Q6_K: no block product in the reference (its gemv decodes them, src/GpuOps.cs:287-300) ----

def check_k(oracle, fmt_a, rows, cols, seed, fmt_x=B.F32):
    a = B.make_weights(fmt_a, rows, cols, seed)
    xf = B.make_activations(cols, seed + 1)
    x = H.x_for(fmt_x, oracle, xf)
    y, sums, _ = H.gemv_gpu(fmt_a, fmt_x, a, x, rows, cols, want_sums=True)
    xq_blocks = oracle.encode(B.Q8_0, xf).reshape(-1, 34)
    xq = xq_blocks[:, 2:].copy().view(np.int8).reshape(-1)
    assert np.array_equal(sums, oracle.k_block_sums(fmt_a, a, xq, rows, cols))
    xv = H.x_values(fmt_x, oracle, x, cols)
    y64 = oracle.gemv_f64(fmt_a, a, xv, rows, cols)
    decoded = oracle.gemv_decoded_f32(fmt_a, a, xv, rows, cols)          # the reference's route on the same stored values
    scale = np.max(np.abs(y64))
    assert np.max(np.abs(y - y64)) <= REL * scale
    assert np.max(np.abs(y - decoded)) <= REL * scale
    if rows * cols >= 1 << 20:
        assert np.max(np.abs(y - y64)) <= np.max(np.abs(decoded - y64)) * 1.0 + 0.0


@pytest.mark.parametrize("fmt_a", [B.Q4_K, B.Q6_K])
@pytest.mark.parametrize("rows,cols", [(1, 256), (5, 512), (37, 1280), (129, 2304), (33, 11008)])
def test_k_quants_small(oracle, fmt_a, rows, cols):
    check_k(oracle, fmt_a, rows, cols, 31 + rows)


@pytest.mark.parametrize("fmt_a", [B.Q4_K, B.Q6_K])
@pytest.mark.parametrize("rows,cols", [(4096, 4096), (11008, 4096), (4096, 11008)])
def test_k_quants_layer_shapes(oracle, fmt_a, rows, cols):
    check_k(oracle, fmt_a, rows, cols, 200)


def test_k_quants_take_q8_0_x(oracle):
    check_k(oracle, B.Q4_K, 65, 1024, 77, fmt_x=B.Q8_0)
    check_k(oracle, B.Q6_K, 65, 1024, 78, fmt_x=B.Q8_0)


@pytest.mark.parametrize("fmt_y", [B.Q8_0, B.Q4_0])
@pytest.mark.parametrize("fmt_a,rows,cols", [
    (B.Q8_0, 37, 64), (B.Q4_0, 32, 96), (B.Q8_0, 1000, 4096), (B.Q4_0, 8192, 8192), (B.Q4_0, 4099, 8160),
    (B.Q4_K, 4096, 4096), (B.Q6_K, 1030, 11008), (B.Q4_0, 28669, 8160)])
def test_back_in_the_same_launch(oracle, fmt_a, rows, cols, fmt_y):
    # Gemv<TN>'s block branch (src/GpuOps.cs:277-285): the blocks written by the gemv's own blocks must be, byte for
    # byte, the encoder's output on the f32 lanes of the same call (gate BlockFormats, src/Checks.cs:241-254), and
    # the lanes must be the plain call's, for a call that waits for its predecessor and for calls that do not
    import torch
    a = B.make_weights(fmt_a, rows, cols, 70)
    xf = B.make_activations(cols, 71)
    o = H.ops()
    da, dx = H.dev(a), H.dev(xf)
    plain = H.empty(rows, torch.float32)
    o.GemvBlocks(fmt_a, da, dx, plain, rows, cols, fmt_x=B.F32)
    nbytes = B.nbytes(fmt_y, (rows + 31) // 32 * 32)
    outs = []
    for i in range(4):                       # four calls that share no output: independent of one another
        lanes = H.empty(rows, torch.float32)
        blocks = H.empty(nbytes, torch.uint8)
        blocks.fill_(0xAB)
        o.GemvBlocksBack(fmt_a, da, dx, lanes, fmt_y, blocks, rows, cols, fmt_x=B.F32)
        outs.append((lanes, blocks))
    lanes2 = outs[0][0]
    o.GemvBlocksBack(fmt_a, da, dx, lanes2, fmt_y, outs[0][1], rows, cols, fmt_x=B.F32)      # same outputs again: a dependent call
    assert o.gpu.status() == 0
    want_lanes = plain.cpu().numpy()
    for lanes, blocks in outs:
        got = lanes.cpu().numpy()
        assert np.allclose(got, want_lanes, rtol=0, atol=REL * np.max(np.abs(want_lanes)))
        assert np.array_equal(blocks.cpu().numpy(), oracle.encode(fmt_y, got, device_rounding=True))


@pytest.mark.parametrize("rounds", [1, 6])
def test_order_against_a_launch_two_back(oracle, rounds):
    # A writes v; B shares nothing with A (so it does not wait for A and runs beside it); C reads v as its x.  C is
    # independent of its direct predecessor B, but not of A, which may still be running: C must order itself after A.
    # v is poisoned before every round, so a C that starts early reads NaN.
    import torch
    n = 8192
    wa = B.make_weights(B.Q4_0, n, n, 31)
    wb = B.make_weights(B.Q8_0, 512, 2048, 32)
    wc = B.make_weights(B.Q4_0, 1024, n, 33)
    xa = B.make_activations(n, 34)
    xb = B.make_activations(2048, 35)
    o = H.ops()
    dwa, dwb, dwc, dxa, dxb = H.dev(wa), H.dev(wb), H.dev(wc), H.dev(xa), H.dev(xb)
    v = H.empty(n, torch.float32)
    yb = H.empty(512, torch.float32)
    yc = H.empty(1024, torch.float32)
    warm = H.empty(n, torch.float32)
    for _ in range(rounds):
        v.fill_(float("nan"))
        o.GemvBlocks(B.Q4_0, dwa, dxa, warm, n, n, fmt_x=B.F32)            # something to run beside
        o.GemvBlocks(B.Q4_0, dwa, dxa, v, n, n, fmt_x=B.F32)               # A
        o.GemvBlocks(B.Q8_0, dwb, dxb, yb, 512, 2048, fmt_x=B.F32)         # B
        o.GemvBlocks(B.Q4_0, dwc, v, yc, 1024, n, fmt_x=B.F32)             # C
        assert o.gpu.status() == 0
        got_v = v.cpu().numpy()
        assert np.isfinite(got_v).all()
        ref, mag = oracle.gemv_blocks(B.Q4_0, B.F32, wc, got_v, 1024, n, order=1, want_abs=True)
        got = yc.cpu().numpy().astype(np.float64)
        assert np.isfinite(got).all()
        assert np.all(np.abs(got - ref) <= REL * mag)


@pytest.mark.parametrize("rounds", [6])
def test_order_against_the_predecessor_of_a_call_that_waited(oracle, rounds):
    # A (few rows: its blocks leave most multiprocessors free) writes v; B reads v, so it waits for A; C also reads v but
    # shares nothing with B.  C is scheduled as B's dependent: were B to release its dependents before its own wait for A
    # has passed, C would read v while A is still writing it.  v is poisoned before every round, so an early C reads NaN.
    import torch
    k, rows_a = 8192, 256
    wa = B.make_weights(B.Q4_0, rows_a, k, 41)
    wb = B.make_weights(B.Q8_0, 2048, rows_a, 42)
    wc = B.make_weights(B.Q4_0, 1024, rows_a, 43)
    xa = B.make_activations(k, 44)
    o = H.ops()
    dwa, dwb, dwc, dxa = H.dev(wa), H.dev(wb), H.dev(wc), H.dev(xa)
    v = H.empty(rows_a, torch.float32)
    yb = H.empty(2048, torch.float32)
    yc = H.empty(1024, torch.float32)
    for _ in range(rounds):
        v.fill_(float("nan"))
        yb.fill_(float("nan"))
        yc.fill_(float("nan"))
        o.GemvBlocks(B.Q4_0, dwa, dxa, v, rows_a, k, fmt_x=B.F32)          # A
        o.GemvBlocks(B.Q8_0, dwb, v, yb, 2048, rows_a, fmt_x=B.F32)        # B = f(v)
        o.GemvBlocks(B.Q4_0, dwc, v, yc, 1024, rows_a, fmt_x=B.F32)        # C = g(v), outputs disjoint from B's
        assert o.gpu.status() == 0
        got_v = v.cpu().numpy()
        assert np.isfinite(got_v).all()
        for fmt, w, y, rows in ((B.Q8_0, wb, yb, 2048), (B.Q4_0, wc, yc, 1024)):
            ref, mag = oracle.gemv_blocks(fmt, B.F32, w, got_v, rows, rows_a, order=1, want_abs=True)
            got = y.cpu().numpy().astype(np.float64)
            assert np.isfinite(got).all()
            assert np.all(np.abs(got - ref) <= REL * mag)


def test_long_run_of_independent_calls(oracle):
    # more independent calls in a row than the library remembers (64): the run is cut by a call that orders itself after
    # everything before it, and every output is still right; the same again after the library's own synchronize
    import torch
    rows, cols, n = 515, 2304, 70
    w = B.make_weights(B.Q8_0, rows, cols, 61)
    xf = B.make_activations(cols, 62)
    o = H.ops()
    dw, dx = H.dev(w), H.dev(xf)
    ref, mag = oracle.gemv_blocks(B.Q8_0, B.F32, w, xf, rows, cols, order=1, want_abs=True)
    for _ in range(2):
        ys = [H.empty(rows, torch.float32) for _ in range(n)]
        for y in ys:
            y.fill_(float("nan"))
        for y in ys:
            o.GemvBlocks(B.Q8_0, dw, dx, y, rows, cols, fmt_x=B.F32)
        o.gpu.Synchronize()
        assert o.gpu.status() == 0
        for y in ys:
            assert np.all(np.abs(y.cpu().numpy().astype(np.float64) - ref) <= REL * mag)


@pytest.mark.parametrize("fmt_a", [B.Q8_0, B.Q4_K])
def test_x_encoded_in_the_kernel_at_extreme_magnitudes(oracle, fmt_a):
    # blocks of x whose scale lands among the f16 subnormals (there amax / d can pass 127.5 and the encoder's clamp to
    # +-127 acts), zero blocks, and large ones: f32 x encoded inside the kernel must give what the encoder's blocks give
    rows, cols = 67, 4096
    rng = np.random.default_rng(5)
    xf = rng.standard_normal(cols).astype(np.float32)
    mags = [0.0, 1e-8, 6e-8, 9e-8, 3e-7, 2e-6, 1e-5, 7e-5, 1e-3, 1.0, 3e4]
    for b in range(cols // 32):
        xf[b * 32:(b + 1) * 32] *= np.float32(mags[b % len(mags)])
    a = B.make_weights(fmt_a, rows, cols, 17)
    xq = oracle.encode(B.Q8_0, xf, device_rounding=True)
    y_f, sums_f, _ = H.gemv_gpu(fmt_a, B.F32, a, xf, rows, cols, want_sums=True)
    y_q, sums_q, _ = H.gemv_gpu(fmt_a, B.Q8_0, a, xq, rows, cols, want_sums=True)
    assert np.array_equal(sums_f, sums_q)
    assert np.array_equal(y_f.view(np.uint32), y_q.view(np.uint32))
    plain_f, _ = H.gemv_gpu(fmt_a, B.F32, a, xf, rows, cols)
    plain_q, _ = H.gemv_gpu(fmt_a, B.Q8_0, a, xq, rows, cols)
    assert np.array_equal(plain_f.view(np.uint32), plain_q.view(np.uint32))
