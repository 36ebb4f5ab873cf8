// Block-scaled gemv for sm_100a: y = A.x with A in Q8_0 / Q4_0 / Q4_K / Q6_K rows and x in blocks or f32.
//
// Replaces Ptx.GemvBlocks (reference src/BlockProducts.cs:78-172), which walks one row per thread with 2-byte loads.
// Here the matrix is one flat byte stream: a producer warp moves whole groups of rows ("units") into a ring of
// shared-memory slots with untiled TMA bulk copies (16-byte aligned middle part; the ragged head and tail bytes by
// plain 2-byte loads), and consumer warps unpack the raw block bytes in registers, take each block's integer dot with
// dp4a in s32, apply the f16 block scales in f32 and reduce each row with warp shuffles.  x is turned once per block of
// threads into int8 values + f32 scales (+ per-block sums) in shared memory, in the reference's Q8_0 encoding when it
// arrives as f32 (src/Ptx.Blocks.cs:52-73).
//
// Per block the arithmetic is the reference kernel's: scale = dA*dX (rounded), acc = fma(scale, float(dot), acc)
// (src/BlockProducts.cs:158-161).  The order in which a row's blocks are added differs (lanes, then a shuffle tree,
// then column segments in ascending order); it is fixed for a given shape, so results are reproducible run to run.
#include "common.cuh"
#include "launch.h"

namespace qb {

struct GemvArgs {
    const uint8_t *a;
    const void *x;
    float *y;
    int32_t *sums;
    int *status;         // device word for STATUS_* bits
    int rows, cols, fmt_x;
    uint32_t row_bytes;
    int nw;              // consumer warps; the producer is warp nw
    int cs, rg;          // column segments x row groups = nw
    int stage_rows;      // rows per unit = rg * RW
    int units;           // ceil(rows / stage_rows)
    int stages;          // ring depth
    uint32_t stage_stride;
    uint32_t off_xq, off_xm, off_part, off_ring;   // shared-memory offsets
};

constexpr int MAX_STAGES = 16;
constexpr uint32_t SMEM_HEADER = 512;   // full[16], empty[16], red[16] barriers and the abort word

__device__ __forceinline__ int dp4a_u8s8(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_s8s8(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------------------------- x -> int8 + scales in shared memory

// One block of 32 activations as the reference's Q8_0 encoder stores them (src/Blocks.cs:37-45, device twin
// src/Ptx.Blocks.cs:54-73): d = amax/127 through f16 and back, id = 1/d (0 when d is 0), q = clamp(rni(v*id), -127, 127).
__device__ __forceinline__ void quantize32(const float (&v)[32], uint32_t (&w)[8], float &d_out, int &sum_out)
{
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(v[i]));
    float d = __half2float(__float2half_rn(__fdiv_rn(amax, 127.f)));
    float id = d == 0.f ? 0.f : __fdiv_rn(1.f, d);
    int sum = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int q = __float2int_rn(__fmul_rn(v[i * 4 + j], id));
            q = max(-127, min(127, q));
            sum += q;
            word |= (uint32_t)(q & 255) << (8 * j);
        }
        w[i] = word;
    }
    d_out = d;
    sum_out = sum;
}

// Block b of x (any of its three forms) as 8 words of int8, its scale and the sum of its values.
__device__ __forceinline__ void load_x_block(const void *x, int fmt_x, int b, uint32_t (&w)[8], float &d, int &sum)
{
    if (fmt_x == QB200_F32) {
        const float *p = (const float *)x + (size_t)b * 32;
        float v[32];
        if (((uintptr_t)p & 15) == 0) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                float4 t = __ldg((const float4 *)p + i);
                v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = __ldg(p + i);
        }
        quantize32(v, w, d, sum);
        return;
    }
    if (fmt_x == QB200_Q8_0) {
        const uint16_t *p = (const uint16_t *)((const uint8_t *)x + (size_t)b * 34);
        d = half_bits_to_float(__ldg(p));
        sum = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            w[i] = (uint32_t)__ldg(p + 1 + 2 * i) | (uint32_t)__ldg(p + 2 + 2 * i) << 16;
            sum = dp4a_s8s8(w[i], 0x01010101u, sum);
        }
        return;
    }
    // Q4_0: value i in the low nibble of byte i, value i + 16 in the high nibble; each minus 8 (src/BlockProducts.cs:34)
    const uint16_t *p = (const uint16_t *)((const uint8_t *)x + (size_t)b * 18);
    d = half_bits_to_float(__ldg(p));
    sum = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t n = (uint32_t)__ldg(p + 1 + 2 * i) | (uint32_t)__ldg(p + 2 + 2 * i) << 16;
        w[i] = __vsub4(n & 0x0F0F0F0Fu, 0x08080808u);
        w[i + 4] = __vsub4((n >> 4) & 0x0F0F0F0Fu, 0x08080808u);
    }
#pragma unroll
    for (int i = 0; i < 8; i++) sum = dp4a_s8s8(w[i], 0x01010101u, sum);
}

// PAIRED layout (Q8_0 / Q4_0 rows): a lane of the consumer handles blocks 2l and 2l+1 of every run of 64 blocks, so
// the 64 bytes of a pair are stored as four 16-byte pieces at [(run*4 + piece)*32 + lane] (consecutive lanes read
// consecutive 16 bytes), and a pair's {d0, d1, sum0, sum1} as one 16-byte record at [pair].
// NATURAL layout (Q4_K / Q6_K rows): int8 values in order, then per block a {d, sum} record.
template <bool PAIRED>
__device__ __forceinline__ void stage_x(const GemvArgs &p, uint8_t *smem, int tid, int threads)
{
    const int blocks = p.cols / 32;
    uint4 *xq = (uint4 *)(smem + p.off_xq);
    for (int b = tid; b < blocks; b += threads) {
        uint32_t w[8];
        float d;
        int sum;
        load_x_block(p.x, p.fmt_x, b, w, d, sum);
        if (PAIRED) {
            int run = b >> 6, lane = (b & 63) >> 1, half = b & 1;
            xq[(run * 4 + half * 2) * 32 + lane] = make_uint4(w[0], w[1], w[2], w[3]);
            xq[(run * 4 + half * 2 + 1) * 32 + lane] = make_uint4(w[4], w[5], w[6], w[7]);
            uint32_t *m = (uint32_t *)(smem + p.off_xm) + (b >> 1) * 4;
            m[half] = __float_as_uint(d);
            m[2 + half] = (uint32_t)sum;
        } else {
            xq[b * 2] = make_uint4(w[0], w[1], w[2], w[3]);
            xq[b * 2 + 1] = make_uint4(w[4], w[5], w[6], w[7]);
            uint2 *m = (uint2 *)(smem + p.off_xm);
            m[b] = make_uint2(__float_as_uint(d), (uint32_t)sum);
        }
    }
    if (PAIRED && (blocks & 1) && tid == 0) {           // the missing partner of a last odd block reads as zero
        uint32_t *m = (uint32_t *)(smem + p.off_xm) + (blocks >> 1) * 4;
        m[1] = 0;
        m[3] = 0;
    }
}

// ---------------------------------------------------------------------------------- raw blocks out of shared memory

// NWORDS code words of the block at q (2-byte aligned) and its f16 scale bits.  Whether q is 4-byte aligned is the
// same for every lane of a warp (lanes are a multiple of 4 bytes apart), so the branch does not diverge.
template <int NWORDS>
__device__ __forceinline__ void load_block(const uint8_t *q, uint32_t (&w)[NWORDS], uint32_t &hscale)
{
    if (((uint32_t)(uintptr_t)q & 2u) == 0) {
        const uint32_t *t = (const uint32_t *)q;
        uint32_t prev = t[0];
        hscale = prev & 0xFFFFu;
#pragma unroll
        for (int i = 0; i < NWORDS; i++) {
            uint32_t next = t[i + 1];
            w[i] = __funnelshift_r(prev, next, 16);
            prev = next;
        }
    } else {
        hscale = *(const uint16_t *)q;
        const uint32_t *t = (const uint32_t *)(q + 2);
#pragma unroll
        for (int i = 0; i < NWORDS; i++) w[i] = t[i];
    }
}

// 32 bits at a 2-byte aligned shared address.
__device__ __forceinline__ uint32_t ld32_a2(const uint8_t *q)
{
    const uint32_t *t = (const uint32_t *)((uintptr_t)q & ~(uintptr_t)3);
    uint32_t sh = ((uint32_t)(uintptr_t)q & 2u) * 8u;
    return __funnelshift_r(t[0], t[1], sh);
}

// ---------------------------------------------------------------------------------- consumers, one per format

// Q8_0 / Q4_0: RW rows at once over this warp's column runs; a lane takes blocks 2l, 2l+1 of each run of 64.
template <int FMT, int RW, bool SUMS>
__device__ __forceinline__ void consume_q(const GemvArgs &p, const uint8_t *smem, const uint8_t *rows, int nvalid, int row0,
                                          int seg, int lane, float (&acc)[RW])
{
    constexpr int BB = block_bytes(FMT), NWORDS = FMT == QB200_Q8_0 ? 8 : 4;
    const int blocks = p.cols / 32;
    const uint4 *xq = (const uint4 *)(smem + p.off_xq);
    const uint4 *xm = (const uint4 *)(smem + p.off_xm);
    for (int run = seg; run * 64 < blocks; run += p.cs) {
        const int b0 = run * 64 + lane * 2;
        if (b0 >= blocks) continue;
        const bool two = b0 + 1 < blocks;
        uint4 x0 = xq[(run * 4 + 0) * 32 + lane], x1 = xq[(run * 4 + 1) * 32 + lane];
        uint4 x2 = xq[(run * 4 + 2) * 32 + lane], x3 = xq[(run * 4 + 3) * 32 + lane];
        uint4 meta = xm[b0 >> 1];
        const float dx0 = __uint_as_float(meta.x), dx1 = __uint_as_float(meta.y);
        const uint32_t xa[8] = { x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w };
        const uint32_t xb[8] = { x2.x, x2.y, x2.z, x2.w, x3.x, x3.y, x3.z, x3.w };
#pragma unroll
        for (int r = 0; r < RW; r++) {
            if (r >= nvalid) break;
            const uint8_t *q = rows + (size_t)r * p.row_bytes + (size_t)b0 * BB;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                if (h == 1 && !two) break;
                uint32_t w[NWORDS], hs;
                load_block<NWORDS>(q + h * BB, w, hs);
                const uint32_t *xw = h ? xb : xa;
                int dot;
                if (FMT == QB200_Q8_0) {
                    dot = 0;
#pragma unroll
                    for (int i = 0; i < 8; i++) dot = dp4a_s8s8(w[i], xw[i], dot);
                } else {
                    // sum (q-8)*x = sum q*x - 8*sum x; the high nibbles are taken in place (16q), exact after >> 4
                    int lo = 0, hi = 0;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        lo = dp4a_u8s8(w[i] & 0x0F0F0F0Fu, xw[i], lo);
                        hi = dp4a_u8s8(w[i] & 0xF0F0F0F0u, xw[i + 4], hi);
                    }
                    dot = lo + (hi >> 4) - 8 * (int)(h ? meta.w : meta.z);
                }
                const float scale = __fmul_rn(half_bits_to_float(hs), h ? dx1 : dx0);
                acc[r] = __fmaf_rn(scale, (float)dot, acc[r]);
                if (SUMS) p.sums[(size_t)(row0 + r) * blocks + b0 + h] = dot;
            }
        }
    }
}

// Q4_K: eight lanes a super-block; a lane takes 16 bytes of nibbles = half of sub-block 2p (low nibbles) and half of
// sub-block 2p+1 (high nibbles).  value = (d*sc)*q - dmin*m (src/Blocks.cs:79-96), so against x = dx*qx a sub-block gives
// (d*sc)*dx*sum(q*qx) - (dmin*m)*dx*sum(qx).  The 6-bit fields are unpacked as ScaleMin does (src/Blocks.cs:73-77), four at a time.
template <int RW, bool SUMS>
__device__ __forceinline__ void consume_q4k(const GemvArgs &p, const uint8_t *smem, const uint8_t *rows, int nvalid, int row0,
                                            int seg, int lane, float (&acc)[RW])
{
    const int sbs = p.cols / 256;
    const uint8_t *xq = smem + p.off_xq;
    const uint2 *xm = (const uint2 *)(smem + p.off_xm);
    const int part = lane & 7, pr = part >> 1, hsel = part & 1;
    for (int run = seg; run * 4 < sbs; run += p.cs) {
        const int sb = run * 4 + (lane >> 3);
        if (sb >= sbs) continue;
        const int xb = sb * 8 + pr * 2;                                    // x block of sub-block 2p
        const uint4 xlo = *(const uint4 *)(xq + (size_t)xb * 32 + hsel * 16);
        const uint4 xhi = *(const uint4 *)(xq + (size_t)xb * 32 + 32 + hsel * 16);
        const uint2 ma = xm[xb], mb = xm[xb + 1];
        const float dxa = __uint_as_float(ma.x), dxb = __uint_as_float(mb.x);
#pragma unroll
        for (int r = 0; r < RW; r++) {
            if (r >= nvalid) break;
            const uint8_t *blk = rows + (size_t)r * p.row_bytes + (size_t)sb * 144;
            uint32_t h0, s0, s1, s2, n[4];
            if (((uint32_t)(uintptr_t)blk & 15u) == 0) {
                const uint4 hdr = *(const uint4 *)blk;
                const uint4 nb = *(const uint4 *)(blk + 16 + pr * 32 + hsel * 16);
                h0 = hdr.x; s0 = hdr.y; s1 = hdr.z; s2 = hdr.w;
                n[0] = nb.x; n[1] = nb.y; n[2] = nb.z; n[3] = nb.w;
            } else {
                h0 = ld32_a2(blk); s0 = ld32_a2(blk + 4); s1 = ld32_a2(blk + 8); s2 = ld32_a2(blk + 12);
#pragma unroll
                for (int i = 0; i < 4; i++) n[i] = ld32_a2(blk + 16 + pr * 32 + hsel * 16 + 4 * i);
            }
            const float d = half_bits_to_float(h0 & 0xFFFFu), dmin = half_bits_to_float(h0 >> 16);
            // scales of sub-blocks 0..3 | 4..7 and their mins, a byte each
            const uint32_t sc_lo = s0 & 0x3F3F3F3Fu, sc_hi = (s2 & 0x0F0F0F0Fu) | (((s0 >> 6) & 0x03030303u) << 4);
            const uint32_t mn_lo = s1 & 0x3F3F3F3Fu, mn_hi = ((s2 >> 4) & 0x0F0F0F0Fu) | (((s1 >> 6) & 0x03030303u) << 4);
            const uint32_t scw = (pr < 2 ? sc_lo : sc_hi) >> ((pr & 1) * 16), mnw = (pr < 2 ? mn_lo : mn_hi) >> ((pr & 1) * 16);
            const int sca = scw & 255, scb = (scw >> 8) & 255, mna = mnw & 255, mnb = (mnw >> 8) & 255;
            int lo = 0, hi = 0;
            const uint32_t xl[4] = { xlo.x, xlo.y, xlo.z, xlo.w }, xh[4] = { xhi.x, xhi.y, xhi.z, xhi.w };
#pragma unroll
            for (int i = 0; i < 4; i++) {
                lo = dp4a_u8s8(n[i] & 0x0F0F0F0Fu, xl[i], lo);
                hi = dp4a_u8s8(n[i] & 0xF0F0F0F0u, xh[i], hi);
            }
            hi >>= 4;
            float a = acc[r];
            a = __fmaf_rn(__fmul_rn(__fmul_rn(d, (float)sca), dxa), (float)lo, a);
            a = __fmaf_rn(__fmul_rn(__fmul_rn(d, (float)scb), dxb), (float)hi, a);
            if (hsel == 0) {
                a = __fmaf_rn(-__fmul_rn(__fmul_rn(dmin, (float)mna), dxa), (float)(int)ma.y, a);
                a = __fmaf_rn(-__fmul_rn(__fmul_rn(dmin, (float)mnb), dxb), (float)(int)mb.y, a);
            }
            acc[r] = a;
            if (SUMS) {
                lo += __shfl_xor_sync(__activemask(), lo, 1);
                hi += __shfl_xor_sync(__activemask(), hi, 1);
                if (hsel == 0) {
                    int32_t *o = p.sums + (size_t)(row0 + r) * (p.cols / 32) + xb;
                    o[0] = lo;
                    o[1] = hi;
                }
            }
        }
    }
}

// Q6_K: sixteen lanes a super-block; a lane takes one word of each of ql[64h..], ql[64h+32..] and qh[32h..]: four
// values of each of four runs of 32 (src/Blocks.cs:157-171).  value = d*sc*(q-32); per 16-value sub-block the integer
// sum is sc * (sum q*qx - 32*sum qx).
template <int RW, bool SUMS>
__device__ __forceinline__ void consume_q6k(const GemvArgs &p, const uint8_t *smem, const uint8_t *rows, int nvalid, int row0,
                                            int seg, int lane, float (&acc)[RW])
{
    const int sbs = p.cols / 256;
    const uint8_t *xq = smem + p.off_xq;
    const uint2 *xm = (const uint2 *)(smem + p.off_xm);
    const int half = (lane >> 3) & 1, t = lane & 7;
    for (int run = seg; run * 2 < sbs; run += p.cs) {
        const int sb = run * 2 + (lane >> 4);
        if (sb >= sbs) continue;
        uint32_t xw[4];
        float dx[4];
        int ones[4];
#pragma unroll
        for (int g = 0; g < 4; g++) {
            xw[g] = *(const uint32_t *)(xq + (size_t)sb * 256 + half * 128 + g * 32 + t * 4);
            dx[g] = __uint_as_float(xm[sb * 8 + half * 4 + g].x);
            ones[g] = dp4a_s8s8(xw[g], 0x01010101u, 0);
        }
#pragma unroll
        for (int r = 0; r < RW; r++) {
            if (r >= nvalid) break;
            const uint8_t *blk = rows + (size_t)r * p.row_bytes + (size_t)sb * 210;
            const uint32_t A = ld32_a2(blk + half * 64 + t * 4), B = ld32_a2(blk + half * 64 + 32 + t * 4);
            const uint32_t H = ld32_a2(blk + 128 + half * 32 + t * 4);
            const float d = half_bits_to_float(*(const uint16_t *)(blk + 208));
            const int8_t *sc = (const int8_t *)(blk + 192 + half * 8 + (t >> 2));
            uint32_t q[4];
            q[0] = (A & 0x0F0F0F0Fu) | ((H << 4) & 0x30303030u);
            q[1] = (B & 0x0F0F0F0Fu) | ((H << 2) & 0x30303030u);
            q[2] = ((A >> 4) & 0x0F0F0F0Fu) | (H & 0x30303030u);
            q[3] = ((B >> 4) & 0x0F0F0F0Fu) | ((H >> 2) & 0x30303030u);
            float a = acc[r];
#pragma unroll
            for (int g = 0; g < 4; g++) {
                int isum = (int)sc[2 * g] * (dp4a_u8s8(q[g], xw[g], 0) - 32 * ones[g]);
                a = __fmaf_rn(__fmul_rn(d, dx[g]), (float)isum, a);
                if (SUMS) {
                    isum += __shfl_xor_sync(__activemask(), isum, 1);
                    isum += __shfl_xor_sync(__activemask(), isum, 2);
                    isum += __shfl_xor_sync(__activemask(), isum, 4);
                    if (t == 0) p.sums[(size_t)(row0 + r) * (p.cols / 32) + sb * 8 + half * 4 + g] = isum;
                }
            }
            acc[r] = a;
        }
    }
}

// ---------------------------------------------------------------------------------- the kernel

template <int FMT, int RW, bool SUMS>
__global__ void __launch_bounds__(544, 1) gemv_kernel(const GemvArgs p)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = (uint64_t *)smem;
    volatile int *abort_flag = (volatile int *)(smem + 3 * MAX_STAGES * 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + MAX_STAGES * 8, red0 = full0 + 2 * MAX_STAGES * 8;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, p.nw);
            mbar_init(red0 + 8 * s, p.nw);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();

    uint8_t *ring = smem + p.off_ring;

    if (warp == p.nw) {
        // ---- producer: one untiled bulk copy a unit, plus the bytes outside its 16-byte aligned middle
        int issued = 0;
        for (int i = 0;; i++) {
            const int u = blockIdx.x + i * gridDim.x;
            if (u >= p.units) break;
            const int s = i % p.stages;
            const uint32_t phase = (uint32_t)(i / p.stages) & 1u;
            if (i >= p.stages && !mbar_wait(empty0 + 8 * s, phase ^ 1u, abort_flag, p.status, STATUS_GEMV_WAIT)) break;
            const int row0 = u * p.stage_rows, nrows = min(p.stage_rows, p.rows - row0);
            const uint8_t *g0 = p.a + (size_t)row0 * p.row_bytes, *g1 = g0 + (size_t)nrows * p.row_bytes;
            const uint32_t mis = (uint32_t)(uintptr_t)g0 & 15u;
            const uint8_t *b0 = (const uint8_t *)(((uintptr_t)g0 + 15) & ~(uintptr_t)15);
            const uint8_t *b1 = (const uint8_t *)((uintptr_t)g1 & ~(uintptr_t)15);
            uint8_t *slot = ring + (size_t)s * p.stage_stride + mis;      // g0's byte lands here
            const uint8_t *head_end, *tail_begin;
            if (b1 > b0) {
                if (lane == 0) {
                    mbar_expect_tx(full0 + 8 * s, (uint32_t)(b1 - b0));
                    bulk_g2s(smem_u32(slot + (b0 - g0)), b0, (uint32_t)(b1 - b0), full0 + 8 * s);
                }
                head_end = b0;
                tail_begin = b1;
            } else {
                head_end = g1;
                tail_begin = g1;
            }
            // at most 15 halfwords on either side
            if (lane < 16) {
                const uint8_t *src = g0 + 2 * lane;
                if (src < head_end) *(uint16_t *)(slot + 2 * lane) = __ldg((const uint16_t *)src);
            } else {
                const uint8_t *src = tail_begin + 2 * (lane - 16);
                if (src < g1) *(uint16_t *)(slot + (src - g0)) = __ldg((const uint16_t *)src);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(full0 + 8 * s);
            issued = i + 1;
        }
        // after a wait that gave up: let the copies still in flight land before the block exits
        if (*abort_flag && lane == 0) {
            for (int i = max(0, issued - p.stages); i < issued; i++) {
                const uint32_t bar = full0 + 8 * (i % p.stages), phase = (uint32_t)(i / p.stages) & 1u;
                long long start = clock64();
                while (!mbar_try_wait(bar, phase) && clock64() - start < WAIT_CYCLES) { }
            }
        }
        return;
    }

    // ---- consumers
    const int threads = p.nw * 32;
    if (FMT == QB200_Q8_0 || FMT == QB200_Q4_0) stage_x<true>(p, smem, threadIdx.x, threads);
    else stage_x<false>(p, smem, threadIdx.x, threads);
    named_bar_sync(1, threads);

    const int seg = warp % p.cs, rgi = warp / p.cs;
    float *part = (float *)(smem + p.off_part);
    for (int i = 0;; i++) {
        const int u = blockIdx.x + i * gridDim.x;
        if (u >= p.units) break;
        const int s = i % p.stages;
        const uint32_t phase = (uint32_t)(i / p.stages) & 1u;
        if (!mbar_wait(full0 + 8 * s, phase, abort_flag, p.status, STATUS_GEMV_WAIT)) break;
        const int row0 = u * p.stage_rows, nrows = min(p.stage_rows, p.rows - row0);
        const uint32_t mis = (uint32_t)(uintptr_t)(p.a + (size_t)row0 * p.row_bytes) & 15u;
        const int lr0 = rgi * RW;
        const uint8_t *rows = ring + (size_t)s * p.stage_stride + mis + (size_t)lr0 * p.row_bytes;
        const int nvalid = max(0, min(RW, nrows - lr0));
        float acc[RW];
#pragma unroll
        for (int r = 0; r < RW; r++) acc[r] = 0.f;
        if (FMT == QB200_Q4_K) consume_q4k<RW, SUMS>(p, smem, rows, nvalid, row0 + lr0, seg, lane, acc);
        else if (FMT == QB200_Q6_K) consume_q6k<RW, SUMS>(p, smem, rows, nvalid, row0 + lr0, seg, lane, acc);
        else consume_q<FMT, RW, SUMS>(p, smem, rows, nvalid, row0 + lr0, seg, lane, acc);
#pragma unroll
        for (int r = 0; r < RW; r++) acc[r] = warp_sum(acc[r]);     // every lane has read its last byte of the slot
        if (p.cs == 1) {
            if (lane == 0) mbar_arrive(empty0 + 8 * s);
#pragma unroll
            for (int r = 0; r < RW; r++) if (lane == r && r < nvalid) p.y[row0 + lr0 + r] = acc[r];
        } else {
            float *mine = part + (size_t)s * p.stage_rows * p.cs;
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < RW; r++) mine[(lr0 + r) * p.cs + seg] = acc[r];
                mbar_arrive(red0 + 8 * s);
                if (warp != 0) mbar_arrive(empty0 + 8 * s);
            }
            if (warp == 0) {
                // the unit's rows (at most 32): segments added in ascending order
                if (!mbar_wait(red0 + 8 * s, phase, abort_flag, p.status, STATUS_GEMV_WAIT)) break;
                if (lane < nrows) {
                    float sum = mine[lane * p.cs];
                    for (int c = 1; c < p.cs; c++) sum += mine[lane * p.cs + c];
                    p.y[row0 + lane] = sum;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * s);
            }
        }
    }
}

// ---------------------------------------------------------------------------------- host side: shape -> configuration

static int g_sm_count = 0, g_max_smem = 0;
static int *g_status = nullptr;

struct GemvPlan {
    int rw, nw, cs, rg, stages, grid;
    uint32_t stage_stride, smem_bytes;
    GemvArgs args;
};

static int env_int(const char *name, int fallback)
{
    const char *v = getenv(name);
    return v && *v ? atoi(v) : fallback;
}

static int cols_per_run(int fmt) { return fmt == QB200_Q4_K ? 1024 : fmt == QB200_Q6_K ? 512 : 2048; }

// Splits the consumer warps into column segments x row groups and sizes the ring.
static int plan_gemv(int fmt_a, int rows, int cols, GemvPlan &pl)
{
    const uint32_t row_bytes = (uint32_t)(cols / block_values(fmt_a) * block_bytes(fmt_a));
    const int runs = (cols + cols_per_run(fmt_a) - 1) / cols_per_run(fmt_a);
    int nw = env_int("QB200_GEMV_WARPS", 8);
    if (nw != 4 && nw != 8 && nw != 16) nw = 8;
    const uint32_t budget = (uint32_t)g_max_smem - 1024;
    const uint32_t xq_bytes = ((uint32_t)cols + 2047u) / 2048u * 2048u;      // whole runs of 64 blocks in the paired layout
    const uint32_t x_bytes = xq_bytes + (uint32_t)(cols / 32 + 2) * 8u + 64u;
    const uint32_t target = (uint32_t)env_int("QB200_GEMV_STAGE_BYTES", 20480);
    // candidates: the fewest idle run slots first, then a unit closest to the target size
    int best_cs = 1, best_rw = 1;
    double best_score = 1e30;
    for (int cs = 1; cs <= nw; cs *= 2) {
        const int per = (runs + cs - 1) / cs;
        const double waste = (double)(per * cs) / runs;
        for (int rw = 4; rw >= 1; rw /= 2) {
            const int stage_rows = nw / cs * rw;
            if (cs > 1 && stage_rows > 32) continue;
            const double bytes = (double)stage_rows * row_bytes;
            if (bytes + 256 > (budget - x_bytes - SMEM_HEADER) / 2) continue;
            double size_pen = bytes > target ? bytes / target : target / bytes;
            double score = waste * 4.0 + size_pen + (rw == 1 ? 0.5 : 0.0);
            if (score < best_score) { best_score = score; best_cs = cs; best_rw = rw; }
        }
    }
    if (best_score > 1e29) return QB200_E_LIMIT;
    const int force_rw = env_int("QB200_GEMV_RW", 0), force_cs = env_int("QB200_GEMV_CS", 0);
    if (force_rw == 1 || force_rw == 2 || force_rw == 4) best_rw = force_rw;
    if (force_cs >= 1 && force_cs <= nw && (nw % force_cs) == 0) best_cs = force_cs;
    pl.rw = best_rw; pl.nw = nw; pl.cs = best_cs; pl.rg = nw / best_cs;
    const int stage_rows = pl.rg * pl.rw;
    if (best_cs > 1 && stage_rows > 32) return QB200_E_LIMIT;
    pl.stage_stride = ((uint32_t)stage_rows * row_bytes + 48u + 127u) / 128u * 128u;
    GemvArgs &a = pl.args;
    a.row_bytes = row_bytes;
    a.nw = nw; a.cs = pl.cs; a.rg = pl.rg; a.stage_rows = stage_rows;
    a.units = (rows + stage_rows - 1) / stage_rows;
    a.off_xq = SMEM_HEADER;
    a.off_xm = a.off_xq + xq_bytes;
    a.off_part = a.off_xm + ((uint32_t)(cols / 32 + 2) * 8u + 15u) / 16u * 16u;
    const uint32_t part_one = (uint32_t)stage_rows * pl.cs * 4u;
    // ring depth: what fits, at most MAX_STAGES, no more than this block's share of the units needs
    uint32_t fixed = a.off_part;
    int stages = MAX_STAGES;
    while (stages > 1 && fixed + (uint32_t)stages * part_one + 128u + (uint32_t)stages * pl.stage_stride > budget) stages--;
    const int force_stages = env_int("QB200_GEMV_STAGES", 0);
    if (force_stages >= 1 && force_stages < stages) stages = force_stages;
    if (fixed + (uint32_t)stages * part_one + 128u + (uint32_t)stages * pl.stage_stride > budget) return QB200_E_LIMIT;
    pl.grid = a.units < g_sm_count ? a.units : g_sm_count;
    const int per_block = (a.units + pl.grid - 1) / pl.grid;
    if (stages > per_block) stages = per_block;
    pl.stages = stages;
    a.stages = stages;
    a.stage_stride = pl.stage_stride;
    a.off_ring = (fixed + (uint32_t)stages * part_one + 127u) / 128u * 128u;
    pl.smem_bytes = a.off_ring + (uint32_t)stages * pl.stage_stride;
    return 0;
}

template <int FMT, bool SUMS>
static cudaError_t launch_fmt(const GemvPlan &pl, cudaStream_t stream)
{
    const dim3 grid(pl.grid), block((pl.nw + 1) * 32);
    switch (pl.rw) {
    case 4: gemv_kernel<FMT, 4, SUMS><<<grid, block, pl.smem_bytes, stream>>>(pl.args); break;
    case 2: gemv_kernel<FMT, 2, SUMS><<<grid, block, pl.smem_bytes, stream>>>(pl.args); break;
    default: gemv_kernel<FMT, 1, SUMS><<<grid, block, pl.smem_bytes, stream>>>(pl.args); break;
    }
    return cudaGetLastError();
}

template <int FMT, bool SUMS>
static cudaError_t set_attr(int bytes)
{
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(gemv_kernel<FMT, 4, SUMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes))) return e;
    if ((e = cudaFuncSetAttribute(gemv_kernel<FMT, 2, SUMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes))) return e;
    return cudaFuncSetAttribute(gemv_kernel<FMT, 1, SUMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

cudaError_t gemv_init(int sm_count, int max_smem, int *status)
{
    g_sm_count = sm_count;
    g_max_smem = max_smem;
    g_status = status;
    cudaError_t e;
    if ((e = set_attr<QB200_Q8_0, false>(max_smem))) return e;
    if ((e = set_attr<QB200_Q4_0, false>(max_smem))) return e;
    if ((e = set_attr<QB200_Q4_K, false>(max_smem))) return e;
    if ((e = set_attr<QB200_Q6_K, false>(max_smem))) return e;
    if ((e = set_attr<QB200_Q8_0, true>(max_smem))) return e;
    if ((e = set_attr<QB200_Q4_0, true>(max_smem))) return e;
    if ((e = set_attr<QB200_Q4_K, true>(max_smem))) return e;
    return set_attr<QB200_Q6_K, true>(max_smem);
}

// Returns 0, a negative QB200_E_* or a positive cudaError_t.  Arguments are already validated.
int gemv_launch(int fmt_a, int fmt_x, const void *a, const void *x, float *y, int32_t *sums, int rows, int cols, cudaStream_t stream)
{
    if (rows == 0) return 0;
    GemvPlan pl;
    int rc = plan_gemv(fmt_a, rows, cols, pl);
    if (rc) return rc;
    pl.args.a = (const uint8_t *)a;
    pl.args.x = x;
    pl.args.y = y;
    pl.args.sums = sums;
    pl.args.status = g_status;
    pl.args.rows = rows;
    pl.args.cols = cols;
    pl.args.fmt_x = fmt_x;
    cudaError_t e;
    if (sums) {
        switch (fmt_a) {
        case QB200_Q8_0: e = launch_fmt<QB200_Q8_0, true>(pl, stream); break;
        case QB200_Q4_0: e = launch_fmt<QB200_Q4_0, true>(pl, stream); break;
        case QB200_Q4_K: e = launch_fmt<QB200_Q4_K, true>(pl, stream); break;
        default: e = launch_fmt<QB200_Q6_K, true>(pl, stream); break;
        }
    } else {
        switch (fmt_a) {
        case QB200_Q8_0: e = launch_fmt<QB200_Q8_0, false>(pl, stream); break;
        case QB200_Q4_0: e = launch_fmt<QB200_Q4_0, false>(pl, stream); break;
        case QB200_Q4_K: e = launch_fmt<QB200_Q4_K, false>(pl, stream); break;
        default: e = launch_fmt<QB200_Q6_K, false>(pl, stream); break;
        }
    }
    return (int)e;
}

// The plan for a shape, for the bench's report and the tests of the host logic (no device needed once sizes are set).
void gemv_describe(int fmt_a, int rows, int cols, int *out8)
{
    GemvPlan pl;
    memset(&pl, 0, sizeof pl);
    int rc = plan_gemv(fmt_a, rows, cols, pl);
    out8[0] = rc; out8[1] = pl.nw; out8[2] = pl.cs; out8[3] = pl.rw; out8[4] = pl.stages; out8[5] = pl.grid;
    out8[6] = (int)pl.stage_stride; out8[7] = (int)pl.smem_bytes;
}

void gemv_set_device_limits(int sm_count, int max_smem) { g_sm_count = sm_count; g_max_smem = max_smem; }

}  // namespace qb
