"""Parity of the tcgen05 A.B^T with the C oracle, through the C ABI.

The kernel keeps the reference device kernel's arithmetic (src/MatMulBlocks.cs:339-347: per k-block
acc = fma(float(D), sA*sB, acc), ascending), so C must equal the oracle's device-order product bit for bit;
every k-block's s32 sum must be exact; against the reference's CPU order (src/MatMulBlocks.cs:130-148) the
tolerance is 1e-5; and the error against the double-double float64 reference (Program.cs:995-1019) must not
exceed the reference's own.
"""
import numpy as np
import pytest

from qiyas_b200 import blocks as B

from . import helpers as H

pytestmark = pytest.mark.gpu


def operands(oracle, fmt_a, fmt_b, m, n, k, seed, quantized_a=True):
    rng = np.random.default_rng(seed)
    if quantized_a:       # activations drawn then row-quantized by the reference's encoder
        a = oracle.encode(fmt_a, rng.standard_normal(m * k).astype(np.float32), device_rounding=True)
    else:
        a = B.make_weights(fmt_a, m, k, seed + 7)
    b = B.make_weights(fmt_b, n, k, seed + 1)
    return a, b


def matmul_gpu(fmt_a, fmt_b, a, b, m, n, k, want_sums=False, workspace=False):
    import torch
    o = H.ops()
    da, db = H.dev(a), H.dev(b)
    c = H.empty(m * n, torch.float32)
    c.fill_(float("nan"))
    if want_sums:
        sums = H.empty(m * n * (k // 32), torch.int32)
        lane = o.MatMulBlockSums(fmt_a, da, db, c, sums, m, n, k, fmt_b=fmt_b)
    elif workspace:
        need = o.workspace_bytes(fmt_a, m, n, k, fmt_b=fmt_b)
        ws = torch.empty(need + 256, dtype=torch.uint8, device="cuda:0")
        off = (-ws.data_ptr()) % 256
        lane = o.MatMulBlocks(fmt_a, da, db, c, m, n, k, fmt_b=fmt_b, workspace=ws.data_ptr() + off, workspace_bytes=need)
    else:
        lane = o.MatMulBlocks(fmt_a, da, db, c, m, n, k, fmt_b=fmt_b)
    assert o.gpu.status() == 0
    assert lane == "s8 tcgen05 blocks"
    out = c.cpu().numpy().reshape(m, n)
    if want_sums:
        return out, sums.cpu().numpy().reshape(m, n, k // 32)
    return out


def check(oracle, fmt_a, fmt_b, m, n, k, seed, f64=True):
    a, b = operands(oracle, fmt_a, fmt_b, m, n, k, seed)
    c, sums = matmul_gpu(fmt_a, fmt_b, a, b, m, n, k, want_sums=True)
    ref, ref_sums = oracle.matmul_blocks(fmt_a, fmt_b, a, b, m, n, k, order=1, want_sums=True)
    assert np.array_equal(sums, ref_sums)
    assert np.array_equal(c.view(np.uint32), ref.view(np.uint32))
    plain = matmul_gpu(fmt_a, fmt_b, a, b, m, n, k)
    assert np.array_equal(plain.view(np.uint32), ref.view(np.uint32))
    cpu = oracle.matmul_blocks(fmt_a, fmt_b, a, b, m, n, k, order=0)
    assert np.max(np.abs(c - cpu)) <= 1e-5 * np.max(np.abs(cpu))
    if f64:
        c64 = oracle.matmul_f64(fmt_a, fmt_b, a, b, m, n, k)
        assert np.max(np.abs(c - c64)) <= np.max(np.abs(ref - c64))


@pytest.mark.parametrize("fmt", [B.Q8_0, B.Q4_0])
@pytest.mark.parametrize("k", [64, 320])
def test_gate_shapes_37x29(oracle, fmt, k):
    # the reference's block product gate: M 37, N 29, K 64 and 320 (src/Checks.cs:1234-1249)
    check(oracle, fmt, fmt, 37, 29, k, 34)


@pytest.mark.parametrize("fmt_a,fmt_b", [(B.Q8_0, B.Q4_0), (B.Q4_0, B.Q8_0)])
def test_mixed_formats(oracle, fmt_a, fmt_b):
    check(oracle, fmt_a, fmt_b, 45, 131, 96, 5)


@pytest.mark.parametrize("m,n,k", [(1, 1, 32), (1, 129, 32), (128, 128, 32), (129, 127, 160), (16, 257, 4096), (257, 384, 1056), (3, 5, 8160)])
def test_edges(oracle, m, n, k):
    check(oracle, B.Q8_0, B.Q8_0, m, n, k, 9 + m, f64=m * n * k < 1 << 24)


@pytest.mark.parametrize("fmt_a,fmt_b", [(B.Q8_0, B.Q8_0), (B.Q4_0, B.Q4_0), (B.Q8_0, B.Q4_0), (B.Q4_0, B.Q8_0)])
@pytest.mark.parametrize("m,n,k", [(1, 1, 32), (5, 3, 96), (16, 257, 4096), (8, 1021, 8160), (13, 130, 1056), (16, 16, 8192), (2, 4099, 64),
                                   (17, 300, 160), (32, 129, 2080), (33, 260, 1024), (64, 515, 4096), (48, 128, 7 * 32), (65, 140, 320)])
def test_few_rows_of_a(oracle, fmt_a, fmt_b, m, n, k):
    # m <= 64 takes the kernel with the operands' sides exchanged (B's rows on the lanes of tensor memory, 16 / 32 / 64
    # columns for A's rows, several k-blocks a commit): the same bits; k-block counts that leave a ragged last batch and stage
    a, b = operands(oracle, fmt_a, fmt_b, m, n, k, 900 + m + n)
    c = matmul_gpu(fmt_a, fmt_b, a, b, m, n, k)
    ref = oracle.matmul_blocks(fmt_a, fmt_b, a, b, m, n, k, order=1)
    assert np.array_equal(c.view(np.uint32), ref.view(np.uint32))
    # and the 128-row-tile kernel gives them too (the checking entry point always takes it)
    c2, _ = matmul_gpu(fmt_a, fmt_b, a, b, m, n, k, want_sums=True) if m * n * (k // 32) <= 1 << 24 else (c, None)
    assert np.array_equal(c2.view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("fmt_b", [B.Q8_0, B.Q4_0])
@pytest.mark.parametrize("m,n,k,offset", [(8, 300, 512, 0), (8, 300, 512, 2), (32, 129, 256, 0), (19, 1000, 2048, 16), (3, 128, 256, 6), (64, 257, 1024, 0),
                                            (40, 1000, 4096, 32), (8, 100, 256, 0), (50, 5, 512, 0)])
def test_raw_weights_in_the_product_kernel(oracle, fmt_b, m, n, k, offset):
    # at most 64 rows of A, k in whole groups of eight blocks: the kernel converts the raw rows of B itself when B lies on a
    # 16-byte boundary, and falls back to the packing pass when it does not; the same bits either way
    import torch
    o = H.ops()
    a, b = operands(oracle, B.Q8_0, fmt_b, m, n, k, 700 + m + offset)
    buf = torch.zeros(b.size + 64, dtype=torch.uint8, device="cuda:0")
    base = buf.data_ptr() + (-buf.data_ptr()) % 16 + offset
    view = buf[base - buf.data_ptr():][:b.size]
    view.copy_(torch.from_numpy(b))
    c = H.empty(m * n, torch.float32)
    c.fill_(float("nan"))
    o.MatMulBlocks(B.Q8_0, H.dev(a), base, c, m, n, k, fmt_b=fmt_b)
    assert o.gpu.status() == 0
    ref = oracle.matmul_blocks(B.Q8_0, fmt_b, a, b, m, n, k, order=1)
    assert np.array_equal(c.cpu().numpy().reshape(m, n).view(np.uint32), ref.view(np.uint32))


def test_caller_workspace(oracle):
    m, n, k = 70, 300, 512
    a, b = operands(oracle, B.Q8_0, B.Q8_0, m, n, k, 3)
    c = matmul_gpu(B.Q8_0, B.Q8_0, a, b, m, n, k, workspace=True)
    ref = oracle.matmul_blocks(B.Q8_0, B.Q8_0, a, b, m, n, k, order=1)
    assert np.array_equal(c.view(np.uint32), ref.view(np.uint32))


def tile_rows(m, seed, extra=4):
    """Rows of A to check at a full-size shape: the first and last row, one row of every 128-row tile, a few at random."""
    rng = np.random.default_rng(seed)
    per_tile = [t * 128 + int(rng.integers(0, min(128, m - t * 128))) for t in range((m + 127) // 128)]
    return np.unique(np.concatenate([[0, m - 1], per_tile, rng.integers(0, m, extra)])).astype(np.int64)


def sampled_rows_check(oracle, fmt_a, fmt_b, m, n, k, seed, prepacked=False):
    """Full-size shapes: C on the GPU; a sample of A's rows through the oracle (a row of C needs that row of A only)."""
    import torch
    a, b = operands(oracle, fmt_a, fmt_b, m, n, k, seed)
    if prepacked:
        o = H.ops()
        da, db = H.dev(a), H.dev(b)
        c_dev = H.empty(m * n, torch.float32)
        c_dev.fill_(float("nan"))
        packed = o.Prepack(fmt_b, db, n, k)
        o.MatMulBlocksPrepacked(fmt_a, da, packed, c_dev, m, n, k, fmt_b=fmt_b)
        assert o.gpu.status() == 0
        c = c_dev.cpu().numpy().reshape(m, n)
    else:
        c = matmul_gpu(fmt_a, fmt_b, a, b, m, n, k)
    pick = tile_rows(m, seed)
    rb = B.row_bytes(fmt_a, k)
    a_rows = a.reshape(m, rb)[pick].reshape(-1)
    ref = oracle.matmul_blocks(fmt_a, fmt_b, a_rows, b, len(pick), n, k, order=1)
    assert np.array_equal(c[pick].view(np.uint32), ref.view(np.uint32))
    assert np.isfinite(c).all()


@pytest.mark.parametrize("m", [1, 16, 128, 512, 2048])
def test_prefill_config_q8_0(oracle, m):
    sampled_rows_check(oracle, B.Q8_0, B.Q8_0, m, 11008, 4096, 300 + m)


def test_prefill_config_odd(oracle):
    sampled_rows_check(oracle, B.Q8_0, B.Q8_0, 509, 11003, 4096, 77)


@pytest.mark.parametrize("m", [1, 8, 64, 512, 2048])
def test_sharded_config_q4_0_weights_q8_0_activations(oracle, m):
    # BASELINE configs[4] on one GPU: Q8_0 activations against the whole 28672 x 8192 Q4_0 matrix, weights prepacked
    sampled_rows_check(oracle, B.Q8_0, B.Q4_0, m, 28672, 8192, 700 + m, prepacked=True)


def test_sharded_config_odd(oracle):
    sampled_rows_check(oracle, B.Q8_0, B.Q4_0, 67, 28669, 8160, 79)
    sampled_rows_check(oracle, B.Q8_0, B.Q4_0, 33, 1021, 8160, 80)


def test_prepacked_weights_give_the_same_bits(oracle):
    import torch
    o = H.ops()
    for fmt_b, (m, n, k) in [(B.Q8_0, (70, 300, 512)), (B.Q4_0, (129, 257, 1056)), (B.Q4_K, (37, 61, 512)), (B.Q6_K, (37, 61, 512))]:
        a, b = operands(oracle, B.Q8_0, fmt_b, m, n, k, 21)
        want = matmul_gpu(B.Q8_0, fmt_b, a, b, m, n, k) if fmt_b in (B.Q8_0, B.Q4_0) else matmul_gpu_k(B.Q8_0, fmt_b, a, b, m, n, k)
        da, db = H.dev(a), H.dev(b)
        packed = o.Prepack(fmt_b, db, n, k)
        db.fill_(0)                                          # the packed form is all the product reads
        for _ in range(2):                                   # the packed weights serve call after call
            c = H.empty(m * n, torch.float32)
            c.fill_(float("nan"))
            o.MatMulBlocksPrepacked(B.Q8_0, da, packed, c, m, n, k, fmt_b=fmt_b)
            assert o.gpu.status() == 0
            assert np.array_equal(c.cpu().numpy().reshape(m, n).view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("fmt", [B.Q8_0, B.Q4_0])
@pytest.mark.parametrize("m,n,k", [(37, 64, 320), (130, 352, 96), (37, 29, 64), (512, 1024, 256)])
def test_back_in_the_product_launch(oracle, fmt, m, n, k):
    # MatMulViewBlocks: lanes, then Back (src/MatMulBlocks.cs:414-424); blocks byte for byte the encoder's on the same lanes
    import torch
    o = H.ops()
    a, b = operands(oracle, fmt, fmt, m, n, k, 55)
    da, db = H.dev(a), H.dev(b)
    lanes = H.empty(m * n, torch.float32)
    lanes.fill_(float("nan"))
    blocks = H.empty(B.nbytes(fmt, m * n), torch.uint8)
    blocks.fill_(0xEE)
    o.MatMulBlocksBack(fmt, da, db, lanes, fmt, blocks, m, n, k)
    assert o.gpu.status() == 0
    ref = oracle.matmul_blocks(fmt, fmt, a, b, m, n, k, order=1)
    assert np.array_equal(lanes.cpu().numpy().reshape(m, n).view(np.uint32), ref.view(np.uint32))
    assert np.array_equal(blocks.cpu().numpy(), oracle.encode(fmt, ref.reshape(-1), device_rounding=True))


def test_batched_products(oracle):
    # ProductView with Batch > 1 (src/Products.cs:15-22): strides in values, 0 broadcasts an operand
    import torch
    from qiyas_b200.ops import ProductView
    o = H.ops()
    m, n, k, batch = 45, 70, 160, 3
    sa, sb, sc = m * k + 64, n * k + 96, (m * n + 31) // 32 * 32 + 32     # gaps between the batch's operands and results, whole blocks
    rng = np.random.default_rng(8)
    a = oracle.encode(B.Q8_0, rng.uniform(-1, 1, sa * batch).astype(np.float32), device_rounding=True)
    b = oracle.encode(B.Q8_0, rng.uniform(-1, 1, sb * batch).astype(np.float32), device_rounding=True)
    da, db = H.dev(a), H.dev(b)
    for stride_a, stride_b in [(sa, sb), (0, sb), (sa, 0)]:
        c = H.empty(sc * batch, torch.float32)
        c.fill_(float("nan"))
        o.MatMulBlocksBatched(B.Q8_0, da, db, c, m, n, k, batch, stride_a, stride_b, sc)
        assert o.gpu.status() == 0
        got = c.cpu().numpy()
        for i in range(batch):
            ai = a[stride_a * i // 32 * 34:][:m * k // 32 * 34]
            bi = b[stride_b * i // 32 * 34:][:n * k // 32 * 34]
            ref = oracle.matmul_blocks(B.Q8_0, B.Q8_0, ai, bi, m, n, k, order=1)
            assert np.array_equal(got[i * sc:i * sc + m * n].view(np.uint32), ref.reshape(-1).view(np.uint32)), (stride_a, stride_b, i)
    # through the view: C encoded to blocks over the whole batch
    v = ProductView(m, n, k, False, True, batch, sa, sb, sc)
    assert o.BlockView("q8_0", v)
    out = H.empty(B.nbytes(B.Q8_0, v.ValuesC), torch.uint8)
    assert o.MatMulView("q8_0", v, da, db, out) == "s8 tcgen05 blocks"
    full = np.zeros(v.ValuesC, np.float32)
    for i in range(batch):
        ref = oracle.matmul_blocks(B.Q8_0, B.Q8_0, a[sa * i // 32 * 34:][:m * k // 32 * 34], b[sb * i // 32 * 34:][:n * k // 32 * 34], m, n, k, order=1)
        full[i * sc:i * sc + m * n] = ref.reshape(-1)
    assert np.array_equal(out.cpu().numpy(), oracle.encode(B.Q8_0, full, device_rounding=True))


def test_backward_da_takes_the_block_product(oracle):
    # MatMulBackward (src/GpuOps.Products.cs:101-106): dA = dC.B^T is the view (m, k, n, TransB) on dC (m x n) and B (k x n)
    import torch
    o = H.ops()
    m, n, k = 33, 96, 50                       # C = A.B with A m x k, B k x n: the product for dA contracts over n
    rng = np.random.default_rng(12)
    dc = oracle.encode(B.Q8_0, rng.uniform(-1, 1, m * n).astype(np.float32), device_rounding=True)
    b = oracle.encode(B.Q8_0, rng.uniform(-1, 1, k * n).astype(np.float32), device_rounding=True)
    da = H.empty(B.nbytes(B.Q8_0, m * k), torch.uint8)
    assert o.MatMulBackward("q8_0", None, H.dev(b), H.dev(dc), da, None, m, n, k) == "s8 tcgen05 blocks"
    lanes = oracle.matmul_blocks(B.Q8_0, B.Q8_0, dc, b, m, k, n, order=1).reshape(-1)
    assert np.array_equal(da.cpu().numpy(), oracle.encode(B.Q8_0, lanes, device_rounding=True))
    with pytest.raises(NotImplementedError):
        o.MatMulBackward("q8_0", None, H.dev(b), H.dev(dc), da, da, m, n, k)


def test_view_surface(oracle):
    import torch
    from qiyas_b200.ops import ProductView
    o = H.ops()
    m, n, k = 37, 29, 320
    a, b = operands(oracle, B.Q8_0, B.Q8_0, m, n, k, 34)
    v = ProductView(m, n, k, False, True)
    assert o.BlockProductAvailable and o.BlockView("q8_0", v)
    out = H.empty(B.nbytes(B.Q8_0, m * n), torch.uint8)
    assert o.MatMulView("q8_0", v, H.dev(a), H.dev(b), out) == "s8 tcgen05 blocks"
    lanes = oracle.matmul_blocks(B.Q8_0, B.Q8_0, a, b, m, n, k, order=1).reshape(-1)
    assert np.array_equal(out.cpu().numpy(), oracle.encode(B.Q8_0, lanes, device_rounding=True))
    with pytest.raises(NotImplementedError):
        o.MatMulView("q8_0", ProductView(m, n, k, True, True), H.dev(a), H.dev(b), out)
    o.BlockProducts = False                  # the gate's override: never the block product
    with pytest.raises(NotImplementedError):
        o.MatMulView("q8_0", v, H.dev(a), H.dev(b), out)
    o.BlockProducts = None
    with pytest.raises(NotImplementedError):
        o.MatMulBlocks("q8_0", H.dev(a), H.dev(b), out, m, n, 33)
    with pytest.raises(NotImplementedError):
        o.MatMulBlocks("q4_k", H.dev(a), H.dev(b), out, m, n, 256)                    # A is never a K-quant
    with pytest.raises(NotImplementedError):
        o.MatMulBlocks("q8_0", H.dev(a), H.dev(b), out, m, n, 320, fmt_b="q4_k")      # k in whole super-blocks of B
    with pytest.raises(NotImplementedError):
        o.MatMulBlocks("q8_0", H.dev(a), H.dev(b), out, m, n, 288, fmt_b="q6_k")


# ---- B in Q4_K / Q6_K (no counterpart kernel in the reference, whose K-quant products decode to f32 first:
# src/GpuOps.Products.cs:28-42).  Gates: every sub-block's s32 sum exact (32 values for Q4_K, 16 for Q6_K), C bit for
# bit the oracle's restatement of the kernel's order, and within 1e-5 (relative to max|C|) of float64 on the stored values.

def matmul_gpu_k(fmt_a, fmt_b, a, b, m, n, k, want_sums=False):
    import torch
    o = H.ops()
    da, db = H.dev(a), H.dev(b)
    c = H.empty(m * n, torch.float32)
    c.fill_(float("nan"))
    per = 32 if fmt_b == B.Q4_K else 16
    if want_sums:
        sums = H.empty(m * n * (k // per), torch.int32)
        o.MatMulBlockSums(fmt_a, da, db, c, sums, m, n, k, fmt_b=fmt_b)
    else:
        o.MatMulBlocks(fmt_a, da, db, c, m, n, k, fmt_b=fmt_b)
    assert o.gpu.status() == 0
    out = c.cpu().numpy().reshape(m, n)
    return (out, sums.cpu().numpy().reshape(m, n, k // per)) if want_sums else out


def oracle_k(oracle, fmt_b):
    return oracle.matmul_q4_k if fmt_b == B.Q4_K else oracle.matmul_q6_k


def check_k(oracle, fmt_a, fmt_b, m, n, k, seed):
    a, b = operands(oracle, fmt_a, fmt_b, m, n, k, seed)
    ref, ref_sums = oracle_k(oracle, fmt_b)(fmt_a, a, b, m, n, k, want_sums=True)
    c, got_sums = matmul_gpu_k(fmt_a, fmt_b, a, b, m, n, k, want_sums=True)
    assert np.array_equal(got_sums, ref_sums)
    assert np.array_equal(c.view(np.uint32), ref.view(np.uint32))
    plain = matmul_gpu_k(fmt_a, fmt_b, a, b, m, n, k)
    assert np.array_equal(plain.view(np.uint32), ref.view(np.uint32))
    if m * n * k < 1 << 24:
        c64 = oracle.matmul_f64(fmt_a, fmt_b, a, b, m, n, k)
        assert np.max(np.abs(plain - c64)) <= 1e-5 * np.max(np.abs(c64))


@pytest.mark.parametrize("fmt_b", [B.Q4_K, B.Q6_K])
@pytest.mark.parametrize("fmt_a", [B.Q8_0, B.Q4_0])
@pytest.mark.parametrize("m,n,k", [(1, 1, 256), (37, 29, 512), (129, 127, 1280), (16, 257, 4096), (24, 300, 1024), (32, 129, 768), (5, 1000, 2304)])
def test_k_quant_weights(oracle, fmt_a, fmt_b, m, n, k):
    check_k(oracle, fmt_a, fmt_b, m, n, k, 500 + m)


@pytest.mark.parametrize("fmt_b", [B.Q4_K, B.Q6_K])
def test_k_quant_weights_prefill_shape(oracle, fmt_b):
    # M 512 against an 11008 x 4096 K-quant matrix: a sample of A's rows through the oracle
    m, n, k = 512, 11008, 4096
    a, b = operands(oracle, B.Q8_0, fmt_b, m, n, k, 611)
    c = matmul_gpu_k(B.Q8_0, fmt_b, a, b, m, n, k)
    pick = np.array([0, 127, 128, 300, 511])
    a_rows = a.reshape(m, B.row_bytes(B.Q8_0, k))[pick].reshape(-1)
    ref = oracle_k(oracle, fmt_b)(B.Q8_0, a_rows, b, len(pick), n, k)
    assert np.array_equal(c[pick].view(np.uint32), ref.view(np.uint32))
    assert np.isfinite(c).all()


def test_a_gemv_after_a_product_reads_its_output(oracle):
    # the gemv's record of launches in flight knows gemv launches only: a product (or a codec) between two gemvs must make
    # the second one order itself after everything, or it could start beside the product whose C it reads as x
    import torch
    o = H.ops()
    n, k, rows = 2048, 1024, 96
    b = B.make_weights(B.Q8_0, n, k, 31)
    a_raw = oracle.encode(B.Q8_0, B.make_activations(k, 32))
    w = B.make_weights(B.Q8_0, rows, n, 33)
    bd, ad, wd, x0 = H.dev(b), H.dev(a_raw), H.dev(w), H.dev(B.make_activations(n, 34))
    c = torch.empty(n, dtype=torch.float32, device="cuda:0")
    y0, y = torch.empty(rows, dtype=torch.float32, device="cuda:0"), torch.empty(rows, dtype=torch.float32, device="cuda:0")
    want_c = oracle.matmul_blocks(B.Q8_0, B.Q8_0, a_raw, b, 1, n, k, order=1).reshape(-1)
    want_y = oracle.gemv_blocks(B.Q8_0, B.F32, w, want_c, rows, n, order=1)
    for _ in range(3):
        c.fill_(float("nan"))
        y.fill_(float("nan"))
        o.GemvBlocks(B.Q8_0, wd, x0, y0, rows, n, fmt_x=B.F32)         # a launch the record knows, unrelated to what follows
        o.MatMulBlocks(B.Q8_0, ad, bd, c, 1, n, k)
        o.GemvBlocks(B.Q8_0, wd, c, y, rows, n, fmt_x=B.F32)
        torch.cuda.synchronize()
        assert o.gpu.status() == 0
        assert np.array_equal(c.cpu().numpy().view(np.uint32), want_c.view(np.uint32))
        assert np.max(np.abs(y.cpu().numpy() - want_y)) <= 1e-5 * np.abs(want_y).max()
