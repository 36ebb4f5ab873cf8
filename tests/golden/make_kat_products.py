"""Generates tests/golden/kat_products.json: block products whose answers follow in closed form from the reference's
own known-answer blocks.

The reference pins its four codecs with hand-laid blocks (`BlockSpecifications`, src/Checks.cs:264-355): formulas over
the index, no random data.  This script lays the same blocks out from those formulas (and variants of them rotated by
the row number, so that rows differ), multiplies them as exact integers and rationals in plain Python, and stores
operands, every block's integer sum and the products.  Nothing here calls the oracle or the CUDA library: the file is
the independent answer both are held to.  All scales are powers of two and all sums are small integers, so every
expected value is exact in f32 whatever the order of the additions: the same vectors pin the reference's CPU order,
its device order and the kernels' orders bit for bit.

    python tests/golden/make_kat_products.py        # rewrites kat_products.json beside it

The blocks (value i of a block, r = the row's number, all index arithmetic as in src/Checks.cs):
  Q8_0 (:269-281)  d = 0.5,   q_i = ((i + r) mod 32) - 16                       value = d q
  Q4_0 (:283-293)  d = 0.25,  byte j = n_j | (15 - n_j) << 4, n_j = (j + r) & 15  value = d (q - 8)
  Q4_K (:295-321)  d = 1, dmin = 0.5, scales 1..8, mins 0..7, q_(j,i) = (i + j + r) & 15, value = d sc_j q - dmin m_j
  Q6_K (:323-351)  d = 0.125, sc_j = j - 8, q_(j,i) = (3 i + j + r) & 63,        value = d sc_j (q - 32)
r = 0 gives exactly the reference's blocks.
"""
import json
import os
import struct
from fractions import Fraction

HERE = os.path.dirname(os.path.abspath(__file__))
Q8_0, Q4_0, Q4_K, Q6_K = 0, 1, 2, 3


def half(v):
    return struct.pack("<e", v)


def q8_0_block(r):
    q = [((i + r) % 32) - 16 for i in range(32)]
    return half(0.5) + bytes((v & 255) for v in q), Fraction(1, 2), q


def q4_0_block(r):
    n = [(j + r) & 15 for j in range(16)]
    raw = bytes(n[j] | ((15 - n[j]) << 4) for j in range(16))
    q = [n[j] - 8 for j in range(16)] + [15 - n[j] - 8 for j in range(16)]      # value j in the low nibble, j + 16 in the high
    return half(0.25) + raw, Fraction(1, 4), q


def q4_k_block(r):
    ls, lm = [1, 2, 3, 4, 5, 6, 7, 8], [0, 1, 2, 3, 4, 5, 6, 7]
    sc = [0] * 12
    for j in range(8):
        if j < 4:
            sc[j] |= ls[j]
            sc[j + 4] |= lm[j]
        else:
            sc[j + 4] = (ls[j] & 0xF) | ((lm[j] & 0xF) << 4)
            sc[j - 4] |= (ls[j] >> 4) << 6
            sc[j] |= (lm[j] >> 4) << 6
    qs = [0] * 128
    q = [[(i + j + r) & 15 for i in range(32)] for j in range(8)]
    for j in range(8):
        for i in range(32):
            at = j // 2 * 32 + i
            qs[at] = (qs[at] & 0xF0) | q[j][i] if j % 2 == 0 else (qs[at] & 0x0F) | (q[j][i] << 4)
    return half(1.0) + half(0.5) + bytes(sc) + bytes(qs), (Fraction(1), Fraction(1, 2), ls, lm), q


def q6_k_block(r):
    q = [[(3 * i + j + r) & 63 for i in range(16)] for j in range(16)]
    flat = [q[j][i] for j in range(16) for i in range(16)]
    ql, qh = [0] * 128, [0] * 64
    for hf in range(2):
        lb, hb, vb = hf * 64, hf * 32, hf * 128
        for l in range(32):
            q1, q2, q3, q4 = flat[vb + l], flat[vb + l + 32], flat[vb + l + 64], flat[vb + l + 96]
            ql[lb + l] = (q1 & 0xF) | ((q3 & 0xF) << 4)
            ql[lb + l + 32] = (q2 & 0xF) | ((q4 & 0xF) << 4)
            qh[hb + l] = ((q1 >> 4) & 3) | (((q2 >> 4) & 3) << 2) | (((q3 >> 4) & 3) << 4) | (((q4 >> 4) & 3) << 6)
    scales = [j - 8 for j in range(16)]
    return bytes(ql) + bytes(qh) + bytes((s & 255) for s in scales) + half(0.125), (Fraction(1, 8), scales), q


def x_values(cols, r=0):
    """x (or a row of A) as Q8_0 blocks of the first kind: bytes, scale, codes per block."""
    blocks = [q8_0_block(r + b) for b in range(cols // 32)]
    return b"".join(b[0] for b in blocks), [b[1] for b in blocks], [b[2] for b in blocks]


def row_against(fmt, r, cols, xd, xq):
    """One row of `fmt` (blocks built with row number r, r + 1, ... along the row) against x: (bytes, sums, value).

    `sums` are the integers the kernels' checking entry points report for every 32 values (src/BlockProducts.cs:158 for
    Q8_0 / Q4_0: sum qA qX with Q4_0's q - 8; Q4_K: sum q qX of the sub-block; Q6_K: sc_a sum16 + sc_b sum16 with q - 32);
    `fine` are the per-16-value sums of Q6_K (what the A.B^T checking entry point reports for Q6_K rows)."""
    raw, sums, fine, total = b"", [], [], Fraction(0)
    if fmt in (Q8_0, Q4_0):
        for b in range(cols // 32):
            blk, d, q = (q8_0_block if fmt == Q8_0 else q4_0_block)(r + b)
            dot = sum(q[i] * xq[b][i] for i in range(32))
            raw += blk
            sums.append(dot)
            total += d * xd[b] * dot
    elif fmt == Q4_K:
        for sb in range(cols // 256):
            blk, (d, dmin, ls, lm), q = q4_k_block(r + sb)
            raw += blk
            for j in range(8):
                b = sb * 8 + j
                dot = sum(q[j][i] * xq[b][i] for i in range(32))
                sums.append(dot)
                total += d * ls[j] * xd[b] * dot - dmin * lm[j] * xd[b] * sum(xq[b])
    else:
        for sb in range(cols // 256):
            blk, (d, scales), q = q6_k_block(r + sb)
            raw += blk
            for b32 in range(8):
                b = sb * 8 + b32
                pair = []
                for hf in range(2):
                    j = 2 * b32 + hf
                    dot = sum((q[j][i] - 32) * xq[b][16 * hf + i] for i in range(16))
                    pair.append(scales[j] * dot)
                    fine.append(dot)
                    total += d * scales[j] * xd[b] * dot
                sums.append(pair[0] + pair[1])
    return raw, sums, fine, total


def exact_f32(v):
    f = float(v)
    assert Fraction(f) == v and struct.unpack("<f", struct.pack("<f", f))[0] == f, v
    return f


def gemv_case(fmt, rows, cols):
    xb, xd, xq = x_values(cols)
    a, sums, y = b"", [], []
    for r in range(rows):
        raw, s, _, total = row_against(fmt, r, cols, xd, xq)
        a += raw
        sums.append(s)
        y.append(exact_f32(total))
    return {"op": "gemv", "fmt_a": fmt, "fmt_x": Q8_0, "rows": rows, "cols": cols, "a": a.hex(), "x": xb.hex(), "sums": sums, "y": y}


def matmul_case(fmt_b, m, n, k):
    a, c, sums = b"", [], []
    rows_b = None
    for i in range(m):
        ab, ad, aq = x_values(k, 3 * i)                        # row i of A: Q8_0 blocks of the first kind, rotated by 3 i
        a += ab
        ci, si, bb = [], [], b""
        for j in range(n):
            raw, s, fine, total = row_against(fmt_b, j, k, ad, aq)
            bb += raw
            ci.append(exact_f32(total))
            si.append(fine if fmt_b == Q6_K else s)
        rows_b = bb
        c.append(ci)
        sums.append(si)
    return {"op": "matmul", "fmt_a": Q8_0, "fmt_b": fmt_b, "m": m, "n": n, "k": k, "a": a.hex(), "b": rows_b.hex(), "sums": sums, "c": c}


def main():
    cases = []
    # the reference's own blocks, one block a row (r = 0): the products the verdict of the formulas gives by hand
    cases.append(gemv_case(Q8_0, 1, 32))        # 0.25 * sum (i - 16)^2 = 0.25 * 2736
    cases.append(gemv_case(Q4_0, 1, 32))
    cases.append(gemv_case(Q4_K, 1, 256))
    cases.append(gemv_case(Q6_K, 1, 256))
    assert cases[0]["sums"] == [[2736]] and cases[0]["y"] == [684.0]
    # several rows and blocks
    for fmt, cols in ((Q8_0, 96), (Q4_0, 160), (Q4_K, 512), (Q6_K, 768)):
        cases.append(gemv_case(fmt, 5, cols))
    for fmt_b, k in ((Q8_0, 64), (Q4_0, 96), (Q4_K, 256), (Q6_K, 512)):
        cases.append(matmul_case(fmt_b, 3, 5, k))
    with open(os.path.join(HERE, "kat_products.json"), "w") as f:
        json.dump({"source": "src/Checks.cs:264-355 (BlockSpecifications), products in closed form", "cases": cases}, f, separators=(",", ":"))
        f.write("\n")
    print(len(cases), "cases")


if __name__ == "__main__":
    main()
