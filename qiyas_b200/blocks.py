"""Block formats of the path: byte layouts, storage sizes and seeded synthetic tensors.

The four GGUF layouts as the reference stores them (src/Blocks.cs:10-17, type structs :261-331):

=====  ======  =====  ==========================================================================
name   values  bytes  layout
=====  ======  =====  ==========================================================================
q8_0   32      34     f16 d @0, 32 int8 q @2; value = d*q
q4_0   32      18     f16 d @0, 16 nibble bytes @2 (low nibble = value i, high = value i+16);
                      value = d*(q-8)
q4_k   256     144    f16 d @0, f16 dmin @2, 12 bytes of 6-bit scales/mins @4, 128 nibble bytes @16
q6_k   256     210    128 bytes ql @0, 64 bytes qh @128, 16 int8 scales @192, f16 d @208
=====  ======  =====  ==========================================================================

The generators build tensors directly as bytes with the value laws of the benchmark
configurations (scales |N(0,1)|*c + eps rounded to f16, codes uniform over their range); they
stand in for model weights, which are not available offline.
"""
import numpy as np

Q8_0, Q4_0, Q4_K, Q6_K, F32 = 0, 1, 2, 3, 100
NAMES = {Q8_0: "q8_0", Q4_0: "q4_0", Q4_K: "q4_k", Q6_K: "q6_k", F32: "f32"}
IDS = {v: k for k, v in NAMES.items()}
BLOCK_VALUES = {Q8_0: 32, Q4_0: 32, Q4_K: 256, Q6_K: 256}
BLOCK_BYTES = {Q8_0: 34, Q4_0: 18, Q4_K: 144, Q6_K: 210}


def fmt_id(fmt):
    """Format id from an id or a reference type name ("q8_0", ...)."""
    if isinstance(fmt, str):
        if fmt not in IDS:
            raise NotImplementedError(f"{fmt}: not a block format of this path")
        return IDS[fmt]
    return int(fmt)


def nbytes(fmt, values):
    """TN.Bytes(values): whole blocks (src/Blocks.cs:269)."""
    fmt = fmt_id(fmt)
    bv = BLOCK_VALUES[fmt]
    return (int(values) + bv - 1) // bv * BLOCK_BYTES[fmt]


def row_bytes(fmt, cols):
    fmt = fmt_id(fmt)
    if cols % BLOCK_VALUES[fmt]:
        raise ValueError(f"{NAMES[fmt]}: {cols} columns are not whole blocks of {BLOCK_VALUES[fmt]}")
    return cols // BLOCK_VALUES[fmt] * BLOCK_BYTES[fmt]


def _f16_bytes(values):
    return np.asarray(values, np.float32).astype(np.float16).view(np.uint8).reshape(values.shape + (2,))


def make_q8_0(rng, rows, cols, scale=0.02, eps=1e-3):
    """rows x cols in Q8_0: d = |N(0,1)|*scale + eps (f16), codes uniform in [-127, 127]."""
    nb = rows * (cols // 32)
    out = np.empty((nb, 34), np.uint8)
    out[:, 0:2] = _f16_bytes(np.abs(rng.standard_normal(nb, dtype=np.float32)) * scale + eps)
    out[:, 2:] = rng.integers(-127, 128, size=(nb, 32), dtype=np.int8).view(np.uint8)
    return out.reshape(-1)


def make_q4_0(rng, rows, cols, scale=0.02, eps=1e-3):
    """rows x cols in Q4_0: d as Q8_0's, 16 bytes of nibbles uniform in 0..15."""
    nb = rows * (cols // 32)
    out = np.empty((nb, 18), np.uint8)
    out[:, 0:2] = _f16_bytes(np.abs(rng.standard_normal(nb, dtype=np.float32)) * scale + eps)
    out[:, 2:] = rng.integers(0, 256, size=(nb, 16), dtype=np.uint8)
    return out.reshape(-1)


def pack_q4_k_scales(ls, lm):
    """8 six-bit scales and 8 six-bit mins into the 12-byte field (inverse of ScaleMin, src/Blocks.cs:73-77)."""
    ls = np.asarray(ls, np.uint8)
    lm = np.asarray(lm, np.uint8)
    sc = np.zeros(ls.shape[:-1] + (12,), np.uint8)
    sc[..., 0:4] = (ls[..., 0:4] & 63) | ((ls[..., 4:8] >> 4) << 6)
    sc[..., 4:8] = (lm[..., 0:4] & 63) | ((lm[..., 4:8] >> 4) << 6)
    sc[..., 8:12] = (ls[..., 4:8] & 15) | ((lm[..., 4:8] & 15) << 4)
    return sc


def make_q4_k(rng, rows, cols, scale=0.01):
    """rows x cols in Q4_K: d, dmin = |N(0,1)|*scale (f16); scales, mins uniform 0..63; nibbles uniform."""
    nb = rows * (cols // 256)
    out = np.empty((nb, 144), np.uint8)
    out[:, 0:2] = _f16_bytes(np.abs(rng.standard_normal(nb, dtype=np.float32)) * scale)
    out[:, 2:4] = _f16_bytes(np.abs(rng.standard_normal(nb, dtype=np.float32)) * scale)
    out[:, 4:16] = pack_q4_k_scales(rng.integers(0, 64, size=(nb, 8), dtype=np.uint8),
                                    rng.integers(0, 64, size=(nb, 8), dtype=np.uint8))
    out[:, 16:] = rng.integers(0, 256, size=(nb, 128), dtype=np.uint8)
    return out.reshape(-1)


def pack_q6_k_codes(q):
    """256 six-bit codes (0..63, value order) into ql (128 bytes) and qh (64 bytes), src/Blocks.cs:204-214."""
    q = np.asarray(q, np.uint8).reshape(q.shape[:-1] + (2, 4, 32))         # half, group of 32, l
    q1, q2, q3, q4 = q[..., 0, :], q[..., 1, :], q[..., 2, :], q[..., 3, :]
    ql = np.concatenate([(q1 & 15) | ((q3 & 15) << 4), (q2 & 15) | ((q4 & 15) << 4)], axis=-1)   # half, 64
    qh = ((q1 >> 4) & 3) | (((q2 >> 4) & 3) << 2) | (((q3 >> 4) & 3) << 4) | (((q4 >> 4) & 3) << 6)
    lead = q.shape[:-3]
    return ql.reshape(lead + (128,)), qh.reshape(lead + (64,))


def make_q6_k(rng, rows, cols, scale=0.001):
    """rows x cols in Q6_K: codes uniform 0..63, 16 int8 sub-scales uniform [-127, 127], d = |N(0,1)|*scale."""
    nb = rows * (cols // 256)
    out = np.empty((nb, 210), np.uint8)
    ql, qh = pack_q6_k_codes(rng.integers(0, 64, size=(nb, 256), dtype=np.uint8))
    out[:, 0:128] = ql
    out[:, 128:192] = qh
    out[:, 192:208] = rng.integers(-127, 128, size=(nb, 16), dtype=np.int8).view(np.uint8)
    out[:, 208:210] = _f16_bytes(np.abs(rng.standard_normal(nb, dtype=np.float32)) * scale)
    return out.reshape(-1)


_MAKERS = {Q8_0: make_q8_0, Q4_0: make_q4_0, Q4_K: make_q4_k, Q6_K: make_q6_k}


def make_weights(fmt, rows, cols, seed):
    """A seeded rows x cols weight matrix in `fmt`, as a flat uint8 array of whole-block rows."""
    fmt = fmt_id(fmt)
    row_bytes(fmt, cols)
    return _MAKERS[fmt](np.random.default_rng(seed), rows, cols)


def make_activations(count, seed):
    """f32 activations ~ N(0,1)."""
    return np.random.default_rng(seed).standard_normal(count, dtype=np.float32)
