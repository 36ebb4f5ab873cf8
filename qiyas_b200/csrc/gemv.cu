// Block-scaled gemv for sm_100a: y = A.x with A in Q8_0 / Q4_0 / Q4_K / Q6_K rows and x in blocks or f32.
//
// Replaces Ptx.GemvBlocks (reference src/BlockProducts.cs:78-172), which walks one row per thread with 2-byte loads.
// Here the matrix is one flat byte stream: a producer warp moves whole groups of rows ("chunks") into a ring of
// shared-memory slots with untiled TMA bulk copies (16-byte aligned middle part; the ragged head and tail bytes by
// plain 2-byte loads), and consumer warps unpack the raw block bytes in registers, take each block's integer dot with
// dp4a in s32, apply the f16 block scales in f32 and reduce each row with warp shuffles.
//
// x is prepared inside the same kernel: the consumer threads of every block turn it into int8 values + f32 scales +
// per-block sums in shared memory (f32 x is encoded to Q8_0 operation for operation as the reference's lanes_to_q8_0
// does, src/Ptx.Blocks.cs:52-73; Q8_0 / Q4_0 x is unpacked), laid out so that every lane fetches the blocks it meets in
// every row with a few 16-byte loads and keeps them in registers for the whole kernel.  (The entry point that must not
// allocate prepares x with a small kernel of its own into a static device array instead: see the end of the file.)
//
// A consumer warp owns a fixed column segment of every row (runs of 64 blocks); the warps of a row group split a row
// between them, write one partial sum per row and segment to shared memory, and the block adds the segments in
// ascending order (no barrier per chunk).
//
// Per block the arithmetic is the reference kernel's: scale = dA*dX (rounded), acc = fma(scale, float(dot), acc)
// (src/BlockProducts.cs:158-161).  The order in which a row's blocks are added differs (lanes, then a shuffle tree,
// then column segments in ascending order); it is fixed for a given shape, so results are reproducible run to run.
//
// Launch order: calls are launched as programmatic dependents (PDL) of whatever precedes them in the stream.  A call
// whose buffers none of the gemv launches still in flight touches skips griddepcontrol.wait and runs beside them; every
// other call waits (gemv_launch).
#include "common.cuh"
#include "encode_blocks.cuh"
#include "launch.h"

#include <mutex>

namespace qb {

struct GemvArgs {
    const uint8_t *a;
    const uint8_t *xprep; // x as prepare_x_kernel lays it out (used when x is null)
    const void *x;        // x as the caller gave it: prepared inside the kernel, in shared memory at off_x
    int fmt_x;
    float *y;
    uint8_t *yb;         // optional: y again as Q8_0 / Q4_0 blocks (fmt_y), encoded by the block that computed the rows
    int fmt_y;
    int chunk_align;     // block boundaries fall on multiples of this many chunks (32 rows when yb is set, else 1 chunk)
    int32_t *sums;
    GemvPublish publish;          // where the rows this launch wrote go besides y (the sharded gemv's exchange); world 0: nowhere
    int *status;         // device word for STATUS_* bits
    int rows, cols;
    uint32_t row_bytes;
    int nw;              // consumer warps; the producer is warp nw
    int cs, rg;          // column segments x row groups = nw
    int stage_rows;      // rows per unit = rg * RW
    int units;           // ceil(rows / stage_rows)
    int chunks;          // ceil(rows / RW)
    int slots;           // ring depth in chunks (a chunk = the RW rows of one row group): a multiple of rg, slots/rg a row group
    int independent;     // 1: nothing this call reads or writes is touched by the launch before it, so no wait on that launch
    int prefetch;        // chunks a block requests before x has been asked for (the rest wait, so x's reads meet idle queues)
    int flush_units;     // units whose partial sums fit the partials area before they are added up
    uint32_t slot_stride;
    uint32_t row_flip;   // 1 when a row is 2 (mod 4) bytes long: rows alternate between the two 4-byte alignments
    uint32_t off_x, off_part, off_ring;   // shared-memory offsets
};

constexpr int MAX_SLOTS = 60;
constexpr uint32_t SMEM_HEADER = 1024;  // full[60] and empty[60] barriers, the x barrier and the abort word

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

// Four row sums at once: halves of the warp trade two values, quarters one, then three plain steps.  Afterwards every
// lane of the eight-lane group g (lanes 8g .. 8g+7) holds the whole sum of row g.  6 shuffles instead of 20.
__device__ __forceinline__ float warp_sum4(const float (&a)[4], int lane)
{
    const bool up = lane & 16;
    const float b0 = (up ? a[2] : a[0]) + __shfl_xor_sync(0xffffffffu, up ? a[0] : a[2], 16);
    const float b1 = (up ? a[3] : a[1]) + __shfl_xor_sync(0xffffffffu, up ? a[1] : a[3], 16);
    const bool odd = lane & 8;
    float c = (odd ? b1 : b0) + __shfl_xor_sync(0xffffffffu, odd ? b0 : b1, 8);
    c += __shfl_xor_sync(0xffffffffu, c, 4);
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    return c;
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

// Prepared x.  PAIRED (Q8_0 / Q4_0 rows): a lane of the gemv handles blocks 2l and 2l+1 of every run of 64 blocks, so the
// 64 bytes of a pair are stored as four 16-byte pieces at [(run*4 + piece)*32 + lane] (consecutive lanes, consecutive 16
// bytes), followed by one 16-byte record {d0, d1, sum0, sum1} a pair.  NATURAL (Q4_K / Q6_K rows): the int8 values in
// order, followed by one 8-byte record {d, sum} a block.  `codes_bytes` is where the records start.
__host__ __device__ inline uint32_t xprep_codes_bytes(int cols) { return ((uint32_t)cols + 2047u) / 2048u * 2048u; }
__host__ __device__ inline uint32_t xprep_bytes(int cols) { return xprep_codes_bytes(cols) + ((uint32_t)(cols / 32 + 2) * 8u + 255u) / 256u * 256u; }

template <bool PAIRED>
__global__ void __launch_bounds__(128) prepare_x_kernel(const void *x, int fmt_x, int cols, uint8_t *out, int independent)
{
    // the gemv that follows may start now: it waits for this grid's end only where it first reads `out`
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // x may be the output of the kernel before this one: wait for it, unless the host has established that it is not.
    // (`out` is free in either case: the gemv before this one lets its dependents start only once all its threads
    // have x in registers.)
    if (!independent) asm volatile("griddepcontrol.wait;" ::: "memory");
    const int blocks = cols / 32, b = blockIdx.x * blockDim.x + threadIdx.x;
    uint8_t *meta = out + xprep_codes_bytes(cols);
    if (b >= blocks) {
        if (PAIRED && b == blocks && (blocks & 1)) {      // the missing partner of a last odd block reads as zero
            uint32_t *m = (uint32_t *)meta + (size_t)(b >> 1) * 4;
            m[1] = 0;
            m[3] = 0;
        }
        return;
    }
    uint32_t w[8];
    float d;
    int sum;
    load_x_block(x, fmt_x, b, w, d, sum);
    uint4 *xq = (uint4 *)out;
    if (PAIRED) {
        const int run = b >> 6, lane = (b & 63) >> 1, half = b & 1;
        xq[(run * 4 + half * 2) * 32 + lane] = make_uint4(w[0], w[1], w[2], w[3]);
        xq[(run * 4 + half * 2 + 1) * 32 + lane] = make_uint4(w[4], w[5], w[6], w[7]);
        uint32_t *m = (uint32_t *)meta + (size_t)(b >> 1) * 4;
        m[half] = __float_as_uint(d);
        m[2 + half] = (uint32_t)sum;
    } else {
        xq[b * 2] = make_uint4(w[0], w[1], w[2], w[3]);
        xq[b * 2 + 1] = make_uint4(w[4], w[5], w[6], w[7]);
        ((uint2 *)meta)[b] = make_uint2(__float_as_uint(d), (uint32_t)sum);
    }
}

// The same preparation inside the gemv kernel, by all its consumer threads, into shared memory.  f32 x: four threads a
// block of 32 values (eight values each, coalesced 32-byte reads); the block's max and sum meet by two shuffles.
// The arithmetic is quantize32's, value for value.
template <bool PAIRED>
__device__ __forceinline__ void prepare_x_in_block(const void *x, int fmt_x, int cols, uint8_t *out, int tid, int threads, uint32_t xbar)
{
    const int blocks = cols / 32;
    uint8_t *meta = out + xprep_codes_bytes(cols);
    constexpr int XU = 4;
    bool told = false;
    if (fmt_x == QB200_F32 && ((uintptr_t)x & 15) == 0) {
        const int items = blocks * 4;
        // up to XU items a thread and pass: all reads are issued before any is used (a read takes about a
        // microsecond while the matrix streams, a second pass would wait that long again)
        for (int base = 0; base < items; base += XU * threads) {
            float v[XU][8];
            bool valid[XU];
#pragma unroll
            for (int u = 0; u < XU; u++) {
                const int it = base + u * threads + tid;
                valid[u] = it < items;
                float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
                if (valid[u]) {
                    lo = __ldg((const float4 *)x + (size_t)it * 2);
                    hi = __ldg((const float4 *)x + (size_t)it * 2 + 1);
                }
                v[u][0] = lo.x; v[u][1] = lo.y; v[u][2] = lo.z; v[u][3] = lo.w; v[u][4] = hi.x; v[u][5] = hi.y; v[u][6] = hi.z; v[u][7] = hi.w;
            }
            if (!told) {            // x's first reads are on their way: the producer may ask for the rest of the matrix
                told = true;
                if ((tid & 31) == 0) mbar_arrive(xbar);
            }
#pragma unroll
            for (int u = 0; u < XU; u++) {
                if (!__any_sync(0xffffffffu, valid[u])) continue;
                const int it = base + u * threads + tid, b = it >> 2, part = it & 3;
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[u][i]));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                const float d = __half2float(__float2half_rn(__fdiv_rn(amax, 127.f)));
                const float id = d == 0.f ? 0.f : __fdiv_rn(1.f, d);
                uint32_t w0 = 0, w1 = 0;
                int sum = 0;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int q0 = max(-127, min(127, __float2int_rn(__fmul_rn(v[u][j], id))));
                    const int q1 = max(-127, min(127, __float2int_rn(__fmul_rn(v[u][4 + j], id))));
                    sum += q0 + q1;
                    w0 |= (uint32_t)(q0 & 255) << (8 * j);
                    w1 |= (uint32_t)(q1 & 255) << (8 * j);
                }
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                if (!valid[u]) continue;
                if (PAIRED) {
                    const int run = b >> 6, lane = (b & 63) >> 1, half = b & 1;
                    *(uint2 *)(out + ((size_t)((run * 4 + half * 2 + (part >> 1)) * 32 + lane)) * 16 + (part & 1) * 8) = make_uint2(w0, w1);
                    if (part == 0) {
                        uint32_t *m = (uint32_t *)meta + (size_t)(b >> 1) * 4;
                        m[half] = __float_as_uint(d);
                        m[2 + half] = (uint32_t)sum;
                    }
                } else {
                    *(uint2 *)(out + (size_t)b * 32 + part * 8) = make_uint2(w0, w1);
                    if (part == 0) ((uint2 *)meta)[b] = make_uint2(__float_as_uint(d), (uint32_t)sum);
                }
            }
        }
    } else {
        for (int b = tid; b < blocks; b += threads) {
            uint32_t w[8];
            float d;
            int sum;
            load_x_block(x, fmt_x, b, w, d, sum);
            uint4 *xq = (uint4 *)out;
            if (PAIRED) {
                const int run = b >> 6, lane = (b & 63) >> 1, half = b & 1;
                xq[(run * 4 + half * 2) * 32 + lane] = make_uint4(w[0], w[1], w[2], w[3]);
                xq[(run * 4 + half * 2 + 1) * 32 + lane] = make_uint4(w[4], w[5], w[6], w[7]);
                uint32_t *m = (uint32_t *)meta + (size_t)(b >> 1) * 4;
                m[half] = __float_as_uint(d);
                m[2 + half] = (uint32_t)sum;
            } else {
                xq[b * 2] = make_uint4(w[0], w[1], w[2], w[3]);
                xq[b * 2 + 1] = make_uint4(w[4], w[5], w[6], w[7]);
                ((uint2 *)meta)[b] = make_uint2(__float_as_uint(d), (uint32_t)sum);
            }
        }
    }
    if (PAIRED && (blocks & 1) && tid == 0) {
        uint32_t *m = (uint32_t *)meta + (size_t)(blocks >> 1) * 4;
        m[1] = 0;
        m[3] = 0;
    }
    if (!told && (tid & 31) == 0) mbar_arrive(xbar);
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

// The same with the alignment known at compile time: Q4 = the block starts on a 4-byte boundary (its codes do not).
template <int NWORDS, bool Q4>
__device__ __forceinline__ void load_block_at(const uint8_t *q, uint32_t (&w)[NWORDS], uint32_t &hscale)
{
    if (Q4) {
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

// ---------------------------------------------------------------------------------- a warp's share of x, in registers

// Q8_0 / Q4_0 rows: per run of 64 blocks a lane holds blocks 2l and 2l+1 of x.
struct XPair {
    uint32_t a[8], b[8];     // int8 values of the two blocks
    float d0, d1;            // their scales
    int s0, s1;              // the sums of their values (for Q4_0 rows: sum (q-8)*x = sum q*x - 8*sum x)
    int count;               // how many of the two blocks exist (a row can end inside a run)
    int first;               // index of block 2l of this run
};

__device__ __forceinline__ void load_x(XPair &x, const GemvArgs &p, const uint8_t *xp, int run, int lane)
{
    const int blocks = p.cols / 32;
    x.first = run * 64 + lane * 2;
    x.count = max(0, min(2, blocks - x.first));
    x.d0 = x.d1 = 0.f;
    x.s0 = x.s1 = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) x.a[i] = x.b[i] = 0;
    if (x.count == 0) return;
    const uint4 *xq = (const uint4 *)xp;
    const uint4 x0 = xq[(run * 4 + 0) * 32 + lane], x1 = xq[(run * 4 + 1) * 32 + lane];
    const uint4 x2 = xq[(run * 4 + 2) * 32 + lane], x3 = xq[(run * 4 + 3) * 32 + lane];
    const uint4 meta = ((const uint4 *)(xp + xprep_codes_bytes(p.cols)))[x.first >> 1];
    x.a[0] = x0.x; x.a[1] = x0.y; x.a[2] = x0.z; x.a[3] = x0.w; x.a[4] = x1.x; x.a[5] = x1.y; x.a[6] = x1.z; x.a[7] = x1.w;
    x.b[0] = x2.x; x.b[1] = x2.y; x.b[2] = x2.z; x.b[3] = x2.w; x.b[4] = x3.x; x.b[5] = x3.y; x.b[6] = x3.z; x.b[7] = x3.w;
    x.d0 = __uint_as_float(meta.x); x.d1 = __uint_as_float(meta.y);
    x.s0 = (int)meta.z; x.s1 = (int)meta.w;
}

// Q4_K rows: four lanes a super-block, eight super-blocks a run; a lane holds sub-blocks 2p and 2p+1 of x (its pair's 32
// bytes of nibbles carry the first in the low halves and the second in the high halves).
struct XK4 {
    uint32_t lo[8], hi[8];
    float da, db;
    int sa, sb;              // sums of the two sub-blocks' x values (the min term)
    int xb;                  // x block of sub-block 2p
    bool valid;
};

__device__ __forceinline__ void load_x(XK4 &x, const GemvArgs &p, const uint8_t *xp, int run, int lane)
{
    const int sb = run * 8 + (lane >> 2), pr = lane & 3;
    x.valid = sb < p.cols / 256;
    x.xb = sb * 8 + pr * 2;
    x.da = x.db = 0.f;
    x.sa = x.sb = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) x.lo[i] = x.hi[i] = 0;
    if (!x.valid) return;
    const uint4 *xq = (const uint4 *)(xp + (size_t)x.xb * 32);
    const uint4 l0 = xq[0], l1 = xq[1], h0 = xq[2], h1 = xq[3];
    const uint2 *meta = (const uint2 *)(xp + xprep_codes_bytes(p.cols));
    const uint2 ma = meta[x.xb], mb = meta[x.xb + 1];
    x.lo[0] = l0.x; x.lo[1] = l0.y; x.lo[2] = l0.z; x.lo[3] = l0.w; x.lo[4] = l1.x; x.lo[5] = l1.y; x.lo[6] = l1.z; x.lo[7] = l1.w;
    x.hi[0] = h0.x; x.hi[1] = h0.y; x.hi[2] = h0.z; x.hi[3] = h0.w; x.hi[4] = h1.x; x.hi[5] = h1.y; x.hi[6] = h1.z; x.hi[7] = h1.w;
    x.da = __uint_as_float(ma.x); x.db = __uint_as_float(mb.x);
    x.sa = (int)ma.y; x.sb = (int)mb.y;
}

// Q6_K rows: eight lanes a super-block, four super-blocks a run.  Runs pair up over eight super-blocks, the even run
// taking the even ones and the odd run the odd ones: blocks are 210 bytes, so whether a lane's block starts on 4 bytes
// is then the same for the whole warp.  A lane (h, ab, lr) holds bytes 16lr.. of x blocks 4h+ab and 4h+ab+2.
struct XK6 {
    uint32_t lo[4], hi[4];
    float dlo, dhi;
    int olo, ohi;            // sums of those 16 values (the -32 offset)
    int sb;
    bool valid;
};

__device__ __forceinline__ int k6_run_block(int run, int lane) { return 8 * (run >> 1) + 2 * (lane >> 3) + (run & 1); }

__device__ __forceinline__ void load_x(XK6 &x, const GemvArgs &p, const uint8_t *xp, int run, int lane)
{
    x.sb = k6_run_block(run, lane);
    x.valid = x.sb < p.cols / 256;
    x.dlo = x.dhi = 0.f;
    x.olo = x.ohi = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) x.lo[i] = x.hi[i] = 0;
    if (!x.valid) return;
    const int xb = x.sb * 8 + ((lane >> 2) & 1) * 4 + ((lane >> 1) & 1), lr = lane & 1;
    const uint4 a = *(const uint4 *)(xp + (size_t)xb * 32 + lr * 16), b = *(const uint4 *)(xp + (size_t)(xb + 2) * 32 + lr * 16);
    const uint2 *meta = (const uint2 *)(xp + xprep_codes_bytes(p.cols));
    x.lo[0] = a.x; x.lo[1] = a.y; x.lo[2] = a.z; x.lo[3] = a.w;
    x.hi[0] = b.x; x.hi[1] = b.y; x.hi[2] = b.z; x.hi[3] = b.w;
    x.dlo = __uint_as_float(meta[xb].x);
    x.dhi = __uint_as_float(meta[xb + 2].x);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        x.olo = dp4a_s8s8(x.lo[i], 0x01010101u, x.olo);
        x.ohi = dp4a_s8s8(x.hi[i], 0x01010101u, x.ohi);
    }
}

template <int FMT> struct XOf { typedef XPair type; };
template <> struct XOf<QB200_Q4_K> { typedef XK4 type; };
template <> struct XOf<QB200_Q6_K> { typedef XK6 type; };

// ---------------------------------------------------------------------------------- one row against one run of x

// Q8_0 / Q4_0: the lane's two blocks of this run.
template <int FMT, bool SUMS>
__device__ __forceinline__ float row_dot(const XPair &x, const uint8_t *row, int lane, int32_t *sums_row, float acc)
{
    constexpr int BB = block_bytes(FMT), NWORDS = FMT == QB200_Q8_0 ? 8 : 4;
    if (x.count == 0) return acc;
    const uint8_t *q = row + (size_t)x.first * BB;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        if (h == 1 && x.count < 2) break;
        uint32_t w[NWORDS], hs;
        load_block<NWORDS>(q + h * BB, w, hs);
        const uint32_t *xw = h ? x.b : x.a;
        int dot;
        if (FMT == QB200_Q8_0) {
            int e = 0, o = 0;
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
                e = dp4a_s8s8(w[i], xw[i], e);
                o = dp4a_s8s8(w[i + 1], xw[i + 1], o);
            }
            dot = e + o;
        } else {
            // sum (q-8)*x = sum q*x - 8*sum x; the high nibbles are taken in place (16q), exact after >> 4
            int lo = 0, hi = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                lo = dp4a_u8s8(w[i] & 0x0F0F0F0Fu, xw[i], lo);
                hi = dp4a_u8s8(w[i] & 0xF0F0F0F0u, xw[i + 4], hi);
            }
            dot = lo + (hi >> 4) - 8 * (h ? x.s1 : x.s0);
        }
        const float scale = __fmul_rn(half_bits_to_float(hs), h ? x.d1 : x.d0);
        acc = __fmaf_rn(scale, (float)dot, acc);
        if (SUMS) sums_row[x.first + h] = dot;
    }
    (void)lane;
    return acc;
}

// The same for a lane whose two blocks both exist, with the first block's alignment known at compile time (the second
// block, 34 or 18 bytes on, has the other alignment): no branches, so the loads of several rows can be in flight at once.
// MASK: the row may end inside this lane's pair or before it.  A lane without blocks does nothing; a lane with one reads
// its missing partner all the same (the bytes after the row: the next row or the slot's padding) and takes its scale as 0.
template <int FMT, bool Q4, bool MASK>
__device__ __forceinline__ float row_dot_fast(const XPair &x, const uint8_t *row, float acc)
{
    constexpr int BB = block_bytes(FMT), NWORDS = FMT == QB200_Q8_0 ? 8 : 4;
    if (MASK && x.count == 0) return acc;
    const uint8_t *q = row + (size_t)x.first * BB;
    uint32_t w0[NWORDS], w1[NWORDS], h0, h1;
    load_block_at<NWORDS, Q4>(q, w0, h0);
    load_block_at<NWORDS, !Q4>(q + BB, w1, h1);
    if (MASK && x.count < 2) h1 = 0;
    int dot0, dot1;
    if (FMT == QB200_Q8_0) {
        int e0 = 0, o0 = 0, e1 = 0, o1 = 0;
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            e0 = dp4a_s8s8(w0[i], x.a[i], e0);
            o0 = dp4a_s8s8(w0[i + 1], x.a[i + 1], o0);
            e1 = dp4a_s8s8(w1[i], x.b[i], e1);
            o1 = dp4a_s8s8(w1[i + 1], x.b[i + 1], o1);
        }
        dot0 = e0 + o0;
        dot1 = e1 + o1;
    } else {
        int lo0 = 0, hi0 = 0, lo1 = 0, hi1 = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            lo0 = dp4a_u8s8(w0[i] & 0x0F0F0F0Fu, x.a[i], lo0);
            hi0 = dp4a_u8s8(w0[i] & 0xF0F0F0F0u, x.a[i + 4], hi0);
            lo1 = dp4a_u8s8(w1[i] & 0x0F0F0F0Fu, x.b[i], lo1);
            hi1 = dp4a_u8s8(w1[i] & 0xF0F0F0F0u, x.b[i + 4], hi1);
        }
        dot0 = lo0 + (hi0 >> 4) - 8 * x.s0;
        dot1 = lo1 + (hi1 >> 4) - 8 * x.s1;
    }
    acc = __fmaf_rn(__fmul_rn(half_bits_to_float(h0), x.d0), (float)dot0, acc);
    acc = __fmaf_rn(__fmul_rn(half_bits_to_float(h1), x.d1), (float)dot1, acc);
    return acc;
}

// RW whole rows of a unit against this warp's runs of x; row r's first block has alignment Q4E (even r) or Q4O (odd r).
template <int FMT, int RW, int RUNS, bool Q4E, bool Q4O, bool MASK>
__device__ __forceinline__ void rows_fast(const XPair (&xr)[RUNS], const uint8_t *rows, uint32_t row_bytes, float (&acc)[RW])
{
#pragma unroll
    for (int j = 0; j < RUNS; j++) {
#pragma unroll
        for (int r = 0; r < RW; r++) {
            if (r & 1) acc[r] = row_dot_fast<FMT, Q4O, MASK>(xr[j], rows + (size_t)r * row_bytes, acc[r]);
            else acc[r] = row_dot_fast<FMT, Q4E, MASK>(xr[j], rows + (size_t)r * row_bytes, acc[r]);
        }
    }
}

// The four alignment cases of a chunk: whether its first row's first block of this lane starts on 4 bytes, and whether
// the next row has the other alignment (rows of an odd number of halfwords).
template <int FMT, int RW, int RUNS, bool MASK>
__device__ __forceinline__ void rows_fast_any(const XPair (&xr)[RUNS], const uint8_t *rows, uint32_t row_bytes, bool q4, bool flip, float (&acc)[RW])
{
    if (!flip) {
        if (q4) rows_fast<FMT, RW, RUNS, true, true, MASK>(xr, rows, row_bytes, acc);
        else rows_fast<FMT, RW, RUNS, false, false, MASK>(xr, rows, row_bytes, acc);
    } else {
        if (q4) rows_fast<FMT, RW, RUNS, true, false, MASK>(xr, rows, row_bytes, acc);
        else rows_fast<FMT, RW, RUNS, false, true, MASK>(xr, rows, row_bytes, acc);
    }
}

// Q4_K: value = (d*sc)*q - dmin*m (src/Blocks.cs:79-96), so against x = dx*qx a sub-block gives
// (d*sc)*dx*sum(q*qx) - (dmin*m)*dx*sum(qx).  The 6-bit fields are unpacked as ScaleMin does (src/Blocks.cs:73-77), four at a time.
// A16 = the super-blocks start on 16 bytes (then three 16-byte loads fetch header and nibbles).
template <bool SUMS, bool A16>
__device__ __forceinline__ float row_dot_k4(const XK4 &x, const uint8_t *row, int lane, int32_t *sums_row, float acc)
{
    const int pr = lane & 3;
    const uint8_t *blk = row + (size_t)(x.xb >> 3) * 144;
    uint32_t h0, s0, s1, s2, n[8];
    if (A16) {
        const uint4 hdr = *(const uint4 *)blk;
        const uint4 na = *(const uint4 *)(blk + 16 + pr * 32), nb = *(const uint4 *)(blk + 32 + pr * 32);
        h0 = hdr.x; s0 = hdr.y; s1 = hdr.z; s2 = hdr.w;
        n[0] = na.x; n[1] = na.y; n[2] = na.z; n[3] = na.w; n[4] = nb.x; n[5] = nb.y; n[6] = nb.z; n[7] = nb.w;
    } else {
        h0 = ld32_a2(blk); s0 = ld32_a2(blk + 4); s1 = ld32_a2(blk + 8); s2 = ld32_a2(blk + 12);
#pragma unroll
        for (int i = 0; i < 8; i++) n[i] = ld32_a2(blk + 16 + pr * 32 + 4 * i);
    }
    const float d = half_bits_to_float(h0 & 0xFFFFu), dmin = half_bits_to_float(h0 >> 16);
    // scales of sub-blocks 0..3 | 4..7 and their mins, a byte each
    const uint32_t sc_lo = s0 & 0x3F3F3F3Fu, sc_hi = (s2 & 0x0F0F0F0Fu) | (((s0 >> 6) & 0x03030303u) << 4);
    const uint32_t mn_lo = s1 & 0x3F3F3F3Fu, mn_hi = ((s2 >> 4) & 0x0F0F0F0Fu) | (((s1 >> 6) & 0x03030303u) << 4);
    const uint32_t scw = (pr < 2 ? sc_lo : sc_hi) >> ((pr & 1) * 16), mnw = (pr < 2 ? mn_lo : mn_hi) >> ((pr & 1) * 16);
    const int sca = scw & 255, scb = (scw >> 8) & 255, mna = mnw & 255, mnb = (mnw >> 8) & 255;
    int lo0 = 0, lo1 = 0, hi0 = 0, hi1 = 0;
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
        lo0 = dp4a_u8s8(n[i] & 0x0F0F0F0Fu, x.lo[i], lo0);
        hi0 = dp4a_u8s8(n[i] & 0xF0F0F0F0u, x.hi[i], hi0);
        lo1 = dp4a_u8s8(n[i + 1] & 0x0F0F0F0Fu, x.lo[i + 1], lo1);
        hi1 = dp4a_u8s8(n[i + 1] & 0xF0F0F0F0u, x.hi[i + 1], hi1);
    }
    const int lo = lo0 + lo1, hi = (hi0 + hi1) >> 4;
    acc = __fmaf_rn(__fmul_rn(__fmul_rn(d, (float)sca), x.da), (float)lo, acc);
    acc = __fmaf_rn(__fmul_rn(__fmul_rn(d, (float)scb), x.db), (float)hi, acc);
    acc = __fmaf_rn(-__fmul_rn(__fmul_rn(dmin, (float)mna), x.da), (float)x.sa, acc);
    acc = __fmaf_rn(-__fmul_rn(__fmul_rn(dmin, (float)mnb), x.db), (float)x.sb, acc);
    if (SUMS) {
        sums_row[x.xb] = lo;
        sums_row[x.xb + 1] = hi;
    }
    return acc;
}

template <int FMT, bool SUMS>
__device__ __forceinline__ float row_dot(const XK4 &x, const uint8_t *row, int lane, int32_t *sums_row, float acc)
{
    if (!x.valid) return acc;
    if (((uint32_t)(uintptr_t)row & 15u) == 0) return row_dot_k4<SUMS, true>(x, row, lane, sums_row, acc);
    return row_dot_k4<SUMS, false>(x, row, lane, sums_row, acc);
}

// RW whole rows on 16 bytes against this warp's runs: one test a run (a row can end inside the last one).
template <int RW, int RUNS>
__device__ __forceinline__ void rows_fast(const XK4 (&xr)[RUNS], const uint8_t *rows, uint32_t row_bytes, int lane, float (&acc)[RW])
{
#pragma unroll
    for (int j = 0; j < RUNS; j++) {
        if (!xr[j].valid) continue;
#pragma unroll
        for (int r = 0; r < RW; r++) acc[r] = row_dot_k4<false, true>(xr[j], rows + (size_t)r * row_bytes, lane, nullptr, acc[r]);
    }
}

// Q6_K (src/Blocks.cs:157-171): value = d*sc*(q-32) with q = a nibble of ql and two bits of qh.  A lane takes 16 bytes
// of ql[64h + 32ab ..] and of qh[32h ..]: the low nibbles are 16 values of run 4h+ab, the high nibbles of run 4h+ab+2,
// each one 16-value sub-block, whose integer sum is sc * (sum q*qx - 32*sum qx).  A4 = the block starts on 4 bytes.
template <bool A4>
__device__ __forceinline__ void load_words4(const uint8_t *q, uint32_t (&w)[4])
{
    if (A4) {
        const uint32_t *t = (const uint32_t *)q;
#pragma unroll
        for (int i = 0; i < 4; i++) w[i] = t[i];
    } else {
        const uint32_t *t = (const uint32_t *)(q - 2);
        uint32_t prev = t[0];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t next = t[i + 1];
            w[i] = __funnelshift_r(prev, next, 16);
            prev = next;
        }
    }
}

template <bool SUMS, bool A4>
__device__ __forceinline__ float row_dot_k6(const XK6 &x, const uint8_t *blk, int lane, int32_t *sums_row, float acc)
{
    const int h = (lane >> 2) & 1, ab = (lane >> 1) & 1, lr = lane & 1;
    uint32_t W[4], H[4];
    load_words4<A4>(blk + h * 64 + ab * 32 + lr * 16, W);
    load_words4<A4>(blk + 128 + h * 32 + lr * 16, H);
    const float d = half_bits_to_float(*(const uint16_t *)(blk + 208));
    const int8_t *sc = (const int8_t *)(blk + 192 + h * 8 + ab * 2 + lr);
    const int sc_lo = sc[0], sc_hi = sc[4];
    const int up = 4 - 2 * ab, down = 2 * ab;
    int dlo = 0, dhi = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t qlo = (W[i] & 0x0F0F0F0Fu) | ((H[i] << up) & 0x30303030u);
        const uint32_t qhi = ((W[i] >> 4) & 0x0F0F0F0Fu) | ((H[i] >> down) & 0x30303030u);
        dlo = dp4a_u8s8(qlo, x.lo[i], dlo);
        dhi = dp4a_u8s8(qhi, x.hi[i], dhi);
    }
    int ilo = sc_lo * (dlo - 32 * x.olo), ihi = sc_hi * (dhi - 32 * x.ohi);
    acc = __fmaf_rn(__fmul_rn(d, x.dlo), (float)ilo, acc);
    acc = __fmaf_rn(__fmul_rn(d, x.dhi), (float)ihi, acc);
    if (SUMS) {             // an entry of the check output is a whole x block: this lane's half and its neighbour's
        ilo += __shfl_xor_sync(__activemask(), ilo, 1);
        ihi += __shfl_xor_sync(__activemask(), ihi, 1);
        if (lr == 0) {
            const int xb = x.sb * 8 + h * 4 + ab;
            sums_row[xb] = ilo;
            sums_row[xb + 2] = ihi;
        }
    }
    return acc;
}

template <int FMT, bool SUMS>
__device__ __forceinline__ float row_dot(const XK6 &x, const uint8_t *row, int lane, int32_t *sums_row, float acc)
{
    if (!x.valid) return acc;
    const uint8_t *blk = row + (size_t)x.sb * 210;
    if (((uint32_t)(uintptr_t)blk & 2u) == 0) return row_dot_k6<SUMS, true>(x, blk, lane, sums_row, acc);
    return row_dot_k6<SUMS, false>(x, blk, lane, sums_row, acc);
}

// RW whole rows against this warp's runs: one test a run (a row can end inside the last one).  The alignment branch is
// uniform over the lanes that have a block.
template <int RW, int RUNS>
__device__ __forceinline__ void rows_fast(const XK6 (&xr)[RUNS], const uint8_t *rows, uint32_t row_bytes, int lane, float (&acc)[RW])
{
#pragma unroll
    for (int j = 0; j < RUNS; j++) {
        if (!xr[j].valid) continue;
        const uint8_t *blk0 = rows + (size_t)xr[j].sb * 210;
#pragma unroll
        for (int r = 0; r < RW; r++) {
            const uint8_t *blk = blk0 + (size_t)r * row_bytes;
            if (((uint32_t)(uintptr_t)blk & 2u) == 0) acc[r] = row_dot_k6<false, true>(xr[j], blk, lane, nullptr, acc[r]);
            else acc[r] = row_dot_k6<false, false>(xr[j], blk, lane, nullptr, acc[r]);
        }
    }
}

// The reference's `Back` step (src/GpuOps.cs:964-975) for the rows [row_lo, row_hi) that one block of the gemv wrote
// (row_lo a multiple of 32): the f32 results again as Q8_0 / Q4_0 blocks, a thread a block of 32; values past the
// last row are zero.
__device__ __forceinline__ void back_rows(const float *y, uint8_t *yb, int fmt_y, int rows, int row_lo, int row_hi, int tid, int threads)
{
    const int count = (row_hi - row_lo + 31) / 32;
    for (int b = tid; b < count; b += threads) {
        const int r0 = row_lo + b * 32;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; i++) v[i] = r0 + i < rows ? __ldcg(y + r0 + i) : 0.f;
        if (fmt_y == QB200_Q8_0) encode_q8_0_block(v, yb + (size_t)(r0 >> 5) * 34);
        else encode_q4_0_block(v, yb + (size_t)(r0 >> 5) * 18);
    }
}

// ---------------------------------------------------------------------------------- the kernel

// The ring holds `slots` chunks; a chunk is RW consecutive rows, fetched by one bulk copy with its own pair of barriers
// and consumed by the cs warps of one row group.  Block b takes the contiguous chunks [b*C/grid, (b+1)*C/grid) of the
// C chunks of the matrix (so blocks differ by at most one chunk); its j-th chunk goes to row group j % rg, and the rg
// chunks dealt in one round are a unit.  RUNS = runs of x a warp holds (its column segment: runs seg, seg + cs, ...).
// NW = the most consumer warps a block of this variant has: 16 (one block an SM) or 4 (four blocks an SM, normally of
// four successive launches: while one block prepares x or drains, the others keep the memory system busy).
// TAIL = what a block does with the rows it wrote once they are in y (variants of their own, so that the plain gemv
// carries none of it): TAIL_BACK encodes them as blocks (the reference's `Back`); TAIL_PUBLISH stores them into the
// other GPUs' copies of the output vector and, from the grid's last block, raises this rank's flag on every GPU.
enum { TAIL_NONE = 0, TAIL_BACK = 1, TAIL_PUBLISH = 2 };
template <int FMT, int RW, int RUNS, bool SUMS, int NW, int TAIL = TAIL_NONE>
__global__ void __launch_bounds__((NW + 1) * 32, 16 / NW) gemv_kernel(const GemvArgs p)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = (uint64_t *)smem;
    volatile int *abort_flag = (volatile int *)(smem + 2 * MAX_SLOTS * 8 + 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + MAX_SLOTS * 8, xbar = empty0 + MAX_SLOTS * 8;

    if (threadIdx.x == 0) {
        mbar_init(xbar, p.nw);
        for (int s = 0; s < p.slots; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, p.cs);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();

    uint8_t *ring = smem + p.off_ring;
    // block b takes the chunks [C*b/grid, C*(b+1)/grid); with TAIL_BACK, whole groups of chunk_align chunks (32 rows)
    int chunk0, chunk1;
    if constexpr (TAIL != TAIL_BACK) {
        chunk0 = (int)((long long)p.chunks * blockIdx.x / gridDim.x);
        chunk1 = (int)((long long)p.chunks * (blockIdx.x + 1) / gridDim.x);
    } else {
        const int groups = (p.chunks + p.chunk_align - 1) / p.chunk_align;
        chunk0 = min(p.chunks, (int)((long long)groups * blockIdx.x / gridDim.x) * p.chunk_align);
        chunk1 = min(p.chunks, (int)((long long)groups * (blockIdx.x + 1) / gridDim.x) * p.chunk_align);
    }
    const int my_units = (chunk1 - chunk0 + p.rg - 1) / p.rg;

    if (warp == p.nw) {
        // ---- producer: one untiled bulk copy a chunk, plus the bytes outside its 16-byte aligned middle.  The weights
        // are read-only for the whole call, so the copies start before the kernel that prepares x has ended.
        // Every lane issues its own chunk's copy (a lone thread needs some hundreds of cycles a copy for the address
        // arithmetic and the barrier calls, which would pace the whole kernel): a pass of the warp issues `step`
        // consecutive chunks, never more than there are slots, so no lane of a pass waits on another lane of it.
        // (with x in a buffer shared between calls the consumers decide when the next call may be scheduled)
        // The trigger comes before this call's own wait (if it has one) has passed, so the next call can start while
        // this call's predecessors are still running: the host's record of launches in flight keeps them for that
        // reason (gemv_launch).  (Making the trigger conditional on the call not waiting cost 1-8 % of every launch.)
        if (p.x) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        // A slot belongs to one row group for the whole kernel (spg slots a group): the warps that wait on a slot's
        // barrier are then always the ones that released its previous use, so a phase parity can never be mistaken for the
        // parity two phases back.
        const int total = my_units * p.rg, step = min(32, p.slots), spg = p.slots / p.rg;
        int issued = 0;
        bool alive = true, x_asked = false;
        for (int base = 0; base < total && alive; base += step) {
            const int k = base + lane;                       // this lane's chunk, counted within the block
            bool ok = true;
            if (lane < step && k < total) {
                const int g = k % p.rg, i = k / p.rg, s = g * spg + i % spg;
                const uint32_t use = (uint32_t)(i / spg);
                // the matrix beyond the first `prefetch` chunks is asked for only once the consumers have asked for x
                if (k >= p.prefetch && !x_asked) ok = mbar_wait(xbar, 0u, abort_flag, p.status, STATUS_GEMV_WAIT);
                if (ok && use > 0) ok = mbar_wait(empty0 + 8 * s, (use - 1u) & 1u, abort_flag, p.status, STATUS_GEMV_WAIT);
                if (ok) {
                    const int chunk = chunk0 + k;
                    const int row0 = chunk * RW, nrows = chunk < chunk1 ? max(0, min(RW, p.rows - row0)) : 0;
                    const uint8_t *g0 = p.a + (size_t)row0 * p.row_bytes, *g1 = g0 + (size_t)nrows * p.row_bytes;
                    const uint32_t mis = (uint32_t)(uintptr_t)g0 & 15u;
                    const uint8_t *b0 = (const uint8_t *)(((uintptr_t)g0 + 15) & ~(uintptr_t)15);
                    const uint8_t *b1 = (const uint8_t *)((uintptr_t)g1 & ~(uintptr_t)15);
                    uint8_t *slot = ring + (size_t)s * p.slot_stride + mis;      // g0's byte lands here
                    const uint8_t *head_end = g1, *tail_begin = g1;
                    if (b1 > b0) {
                        mbar_expect_tx(full0 + 8 * s, (uint32_t)(b1 - b0));
                        bulk_g2s(smem_u32(slot + (b0 - g0)), b0, (uint32_t)(b1 - b0), full0 + 8 * s);
                        head_end = b0;
                        tail_begin = b1;
                    }
                    // at most 7 halfwords on either side (none when the chunk starts and ends on 16 bytes); all reads
                    // are issued before the first is stored.  (A chunk shorter than 16 bytes has no middle: slow loop.)
                    if (head_end - g0 <= 14 && g1 - tail_begin <= 14) {
                        uint16_t hv[7], tv[7];
#pragma unroll
                        for (int i = 0; i < 7; i++) {
                            hv[i] = g0 + 2 * i < head_end ? __ldg((const uint16_t *)(g0 + 2 * i)) : (uint16_t)0;
                            tv[i] = tail_begin + 2 * i < g1 ? __ldg((const uint16_t *)(tail_begin + 2 * i)) : (uint16_t)0;
                        }
#pragma unroll
                        for (int i = 0; i < 7; i++) {
                            if (g0 + 2 * i < head_end) *(uint16_t *)(slot + 2 * i) = hv[i];
                            if (tail_begin + 2 * i < g1) *(uint16_t *)(slot + (tail_begin - g0) + 2 * i) = tv[i];
                        }
                    } else {
                        for (const uint8_t *src = g0; src < head_end; src += 2) *(uint16_t *)(slot + (src - g0)) = __ldg((const uint16_t *)src);
                        for (const uint8_t *src = tail_begin; src < g1; src += 2) *(uint16_t *)(slot + (src - g0)) = __ldg((const uint16_t *)src);
                    }
                    mbar_arrive(full0 + 8 * s);
                }
            }
            alive = __all_sync(0xffffffffu, ok);
            if (base + step > p.prefetch) x_asked = true;    // every lane beyond the prefetch has seen the x barrier complete
            issued = min(total, base + step);
        }
        // after a wait that gave up: let the copies still in flight land before the block exits
        if (*abort_flag && lane == 0) {
            for (int k = max(0, issued - p.slots); k < issued; k++) {
                const int g = k % p.rg, i = k / p.rg;
                const uint32_t bar = full0 + 8 * (g * spg + i % spg), ph = (uint32_t)(i / spg) & 1u;
                long long start = clock64();
                while (!mbar_try_wait(bar, ph) && clock64() - start < WAIT_CYCLES) { }
            }
        }
        return;
    }

    // ---- consumers: each warp's column segment of the prepared x into registers
    const int threads = p.nw * 32;
    const int seg = warp % p.cs, rgi = warp / p.cs;
    typename XOf<FMT>::type xr[RUNS];
    // whatever wrote x (or prepared it) has ended and its writes are visible; skipped when the host has established that
    // the launch before this one (the only one that can still be running) shares no buffer with this call
    if (!p.independent || !p.x) asm volatile("griddepcontrol.wait;" ::: "memory");
    if constexpr (TAIL == TAIL_PUBLISH) {
        // x is the output of an earlier exchange: thread w waits (bounded) until rank w's word of this rank's flag array
        // of that exchange has reached its epoch -- the peers' rows of x have then arrived (the acquire pairs with the
        // publishers' release; the barrier hands it to the block's other threads).  The launch before this one has
        // completed (the wait above), so with counted epochs the count of published calls is that exchange's last epoch.
        // The weights' copies have been running all along.
        if (p.publish.wait_flags) {
            if ((int)threadIdx.x < p.publish.world) {
                const unsigned int *flags = p.publish.wait_flags;
                const unsigned int epoch = p.publish.wait_epoch ? p.publish.wait_epoch : __ldcg(flags + QB200_SHARD_MAX);
                if (epoch) {
                    const long long start = clock64();
                    for (;;) {
                        unsigned int v;
                        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + threadIdx.x) : "memory");
                        if ((int)(v - epoch) >= 0) break;
                        if (clock64() - start > p.publish.wait_limit) {
                            atomicOr(p.status, STATUS_SHARD_WAIT);
                            break;
                        }
                        __nanosleep(50);
                    }
                    // the exchange's count of waits follows its count of published calls (one block counts)
                    if (blockIdx.x == 0 && threadIdx.x == 0 && !p.publish.wait_epoch) atomicAdd((unsigned int *)flags + QB200_SHARD_MAX + 1, 1u);
                }
            }
            named_bar_sync(1, threads);
        }
    }
    const uint8_t *xp = p.xprep;
    if (p.x) {
        if (FMT == QB200_Q8_0 || FMT == QB200_Q4_0) prepare_x_in_block<true>(p.x, p.fmt_x, p.cols, smem + p.off_x, threadIdx.x, threads, xbar);
        else prepare_x_in_block<false>(p.x, p.fmt_x, p.cols, smem + p.off_x, threadIdx.x, threads, xbar);
            named_bar_sync(1, threads);
        xp = smem + p.off_x;
    }
#pragma unroll
    for (int j = 0; j < RUNS; j++) load_x(xr[j], p, xp, seg + j * p.cs, lane);
    if (!p.x) {
        // x came from a buffer that the next call's preparing kernel rewrites: every warp of the block has its part in
        // registers before any of them lets that kernel be scheduled
        if (lane == 0) mbar_arrive(xbar);
        named_bar_sync(1, threads);
    }
    // x is in registers: the next call's kernels may be scheduled as this grid's blocks retire
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // whether every lane of this warp has both blocks of every run (then whole chunks take the branch-free path)
    bool whole_runs = false;
    if (FMT == QB200_Q8_0 || FMT == QB200_Q4_0) whole_runs = (seg + (RUNS - 1) * p.cs + 1) * 64 <= p.cols / 32;

    float *part = (float *)(smem + p.off_part);
    const int blocks32 = p.cols / 32;
    const uint32_t first_off = (FMT == QB200_Q8_0 || FMT == QB200_Q4_0) ? (uint32_t)(seg * 64 + lane * 2) * (uint32_t)block_bytes(FMT) : 0u;
    bool alive = true;
    const int spg = p.slots / p.rg;                  // this row group's own slots: rgi*spg .. rgi*spg + spg - 1
    int sl = 0, flush_i = 0;
    uint32_t phase = 0;
    for (int i = 0; i < my_units; i++) {
        const int chunk = chunk0 + i * p.rg + rgi, s = rgi * spg + sl;
        const int row0 = chunk * RW;
        const int nvalid = chunk < chunk1 ? max(0, min(RW, p.rows - row0)) : 0;
        if (alive) alive = mbar_wait_warp(full0 + 8 * s, phase, abort_flag, p.status, STATUS_GEMV_WAIT);
        if (alive) {
            const uint32_t mis = (uint32_t)(uintptr_t)(p.a + (size_t)row0 * p.row_bytes) & 15u;
            const uint8_t *rows = ring + (size_t)s * p.slot_stride + mis;
            float acc[RW];
#pragma unroll
            for (int r = 0; r < RW; r++) acc[r] = 0.f;
            bool done = false;
            if constexpr ((FMT == QB200_Q8_0 || FMT == QB200_Q4_0) && !SUMS) {
                if (!done && nvalid == RW) {
                    const bool q4 = (((uint32_t)(uintptr_t)rows + first_off) & 2u) == 0;
                    if (whole_runs) rows_fast_any<FMT, RW, RUNS, false>(xr, rows, p.row_bytes, q4, p.row_flip != 0, acc);
                    else rows_fast_any<FMT, RW, RUNS, true>(xr, rows, p.row_bytes, q4, p.row_flip != 0, acc);
                    done = true;
                }
            }
            if constexpr (FMT == QB200_Q6_K && !SUMS) {
                if (!done && nvalid == RW) {
                    rows_fast<RW, RUNS>(xr, rows, p.row_bytes, lane, acc);
                    done = true;
                }
            }
            if constexpr (FMT == QB200_Q4_K && !SUMS) {
                if (!done && nvalid == RW && (((uint32_t)(uintptr_t)rows | p.row_bytes) & 15u) == 0) {
                    rows_fast<RW, RUNS>(xr, rows, p.row_bytes, lane, acc);
                    done = true;
                }
            }
            if (!done) {
#pragma unroll
                for (int j = 0; j < RUNS; j++) {
#pragma unroll
                    for (int r = 0; r < RW; r++) {
                        if (r < nvalid)
                            acc[r] = row_dot<FMT, SUMS>(xr[j], rows + (size_t)r * p.row_bytes, lane,
                                                        SUMS ? p.sums + (size_t)(row0 + r) * blocks32 : nullptr, acc[r]);
                    }
                }
            }
            // the row sums (every lane has read its last byte of the slot once these shuffles are done)
            if constexpr (RW == 4) {
                const float total = warp_sum4(acc, lane);           // lanes 8r .. 8r+7 hold row r
                if (lane == 0) mbar_arrive(empty0 + 8 * s);
                const int r = lane >> 3;
                if ((lane & 7) == 0) {
                    if (p.cs == 1) { if (r < nvalid) p.y[row0 + r] = total; }
                    else part[((size_t)flush_i * p.stage_rows + rgi * RW + r) * p.cs + seg] = total;
                }
            } else {
#pragma unroll
                for (int r = 0; r < RW; r++) acc[r] = warp_sum(acc[r]);
                if (lane == 0) mbar_arrive(empty0 + 8 * s);
                if (p.cs == 1) {
#pragma unroll
                    for (int r = 0; r < RW; r++) if (lane == r && r < nvalid) p.y[row0 + r] = acc[r];
                } else if (lane == 0) {
                    float *mine = part + ((size_t)flush_i * p.stage_rows + rgi * RW) * p.cs + seg;
#pragma unroll
                    for (int r = 0; r < RW; r++) mine[r * p.cs] = acc[r];
                }
            }
        }
        if (++sl == spg) { sl = 0; phase ^= 1u; }
        // the partial sums of the last flush_units units: segments added in ascending order
        if (p.cs > 1 && (++flush_i == p.flush_units || i + 1 == my_units)) {
            named_bar_sync(1, threads);
            const int first = i + 1 - flush_i, count = flush_i * p.stage_rows;
            for (int idx = threadIdx.x; idx < count; idx += threads) {
                const int k = idx / p.stage_rows, lr = idx - k * p.stage_rows;
                const int ch = chunk0 + (first + k) * p.rg + lr / RW, row = ch * RW + lr % RW;
                if (ch < chunk1 && row < p.rows) {
                    const float *src = part + (size_t)idx * p.cs;
                    float sum = src[0];
                    for (int c = 1; c < p.cs; c++) sum += src[c];
                    p.y[row] = sum;
                }
            }
            flush_i = 0;
            if (i + 1 < my_units) named_bar_sync(1, threads);
        }
    }
    if constexpr (TAIL == TAIL_BACK) {
        named_bar_sync(1, threads);
        if (!*abort_flag) back_rows(p.y, p.yb, p.fmt_y, p.rows, chunk0 * RW, min(p.rows, chunk1 * RW), threadIdx.x, threads);
    }
    if constexpr (TAIL == TAIL_PUBLISH) {
        // The block's rows are in y (this GPU's copy of the output vector): plain stores carry them into every other
        // GPU's copy, a fence orders them before the block's count, and the block that counts last raises the flags.
        // A block that gave up on a wait publishes nothing and does not count: the flags then never show this epoch
        // and the readers' bounded waits report it.
        // (the barrier also tells every thread whether anyone has given up: all publish, or none does)
        if (named_bar_and(1, threads, !*abort_flag)) {
            const GemvPublish *pub = &p.publish;
            const int r0 = chunk0 * RW, r1 = min(p.rows, chunk1 * RW), world = pub->world;
            for (int idx = r0 + (int)threadIdx.x; idx < r1; idx += threads) {
                const float v = __ldcg(p.y + idx);
                for (int w = 0; w < world; w++) {
                    float *dst = pub->out[w];
                    if (dst) dst[idx] = v;
                }
            }
            // The block's stores are ordered before its count by one fence: the barrier makes them thread 0's to order.
            // Device scope is enough here (the count is read on this GPU); the block that counts last adds the
            // system-scope fence before the flags, and causality carries the other blocks' stores along with it.
            named_bar_sync(1, threads);
            if (threadIdx.x == 0) {
                __threadfence();
                const unsigned int before = atomicAdd(pub->counter, 1u);
                if (before == gridDim.x - 1) {
                    *pub->counter = 0u;
                    __threadfence_system();
                    // epoch 0: the call's number is counted on the device (a captured graph replays the same arguments)
                    const unsigned int epoch = pub->epoch ? pub->epoch : atomicAdd(pub->epoch_counter, 1u) + 1u;
                    for (int w = 0; w < world; w++) {
                        unsigned int *f = pub->flag[w];
                        // (the fence above is the release: the flags themselves are plain system-scope stores, one a peer)
                        if (f) asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------- host side: shape -> configuration

static int g_sm_count = 0, g_max_smem = 0;
static int g_epoch = 0;          // counts the library's bindings to a device: plans made under an earlier one are void
static int *g_status = nullptr;

struct GemvPlan {
    int rw, runs_per_warp, nw, nwmax, cs, rg, stages, grid;
    bool deep;
    bool serial;            // launch without the programmatic attribute: after everything earlier in the stream
    uint32_t stage_stride, smem_bytes;
    GemvArgs args;
};

// bytes of a chunk the plan aims at: rows a warp takes at once are halved until a chunk is at most this
constexpr uint32_t CHUNK_BYTES = 24576;

// Runs of x that cover a row: 2048 columns each, but Q6_K runs are four super-blocks of one parity out of eight.
static int runs_of(int fmt, int cols)
{
    if (fmt != QB200_Q6_K) return (cols + 2047) / 2048;
    const int sb = cols / 256, rem = sb % 8;
    return sb / 8 * 2 + (rem == 0 ? 0 : rem == 1 ? 1 : 2);
}
static int max_runs_per_warp(int fmt) { return fmt == QB200_Q6_K ? 4 : 2; }
static constexpr uint32_t PART_BYTES = 16384;

// Splits the consumer warps of a block of at most `nwmax` warps (16 / nwmax such blocks share an SM) into column
// segments x row groups and sizes the ring.  `rw_first` = the most rows a warp takes at once.
static int plan_blocks(int fmt_a, int rows, int cols, int nwmax, int rw_first, bool back, GemvPlan &pl)
{
    const uint32_t row_bytes = (uint32_t)(cols / block_values(fmt_a) * block_bytes(fmt_a));
    const int runs = runs_of(fmt_a, cols);
    int nw = nwmax;
    const int ctas = 16 / nwmax;                                 // blocks meant to share an SM
    const uint32_t budget = ctas > 1 ? (uint32_t)(g_max_smem + 1024) / ctas - 2048 : (uint32_t)g_max_smem - 1024;
    // column segments: c segments leave nw / c row groups, each taking a chunk in ceil(runs / c) run times; the most
    // rows per run time wins (warps that do not fill a row group stay out), then the most segments (few registers of x)
    int cs = 0;
    double best = 0.0;
    for (int c = 1; c <= nw; c++) {
        const int per = (runs + c - 1) / c;
        if (per > max_runs_per_warp(fmt_a)) continue;
        const double rate = (double)(nw / c) / per;
        if (rate > best * (1.0 + 1e-9) || (rate > best * (1.0 - 1e-9) && c > cs)) { best = rate; cs = c; }
    }
    if (cs == 0) return QB200_E_LIMIT;
    const int per = (runs + cs - 1) / cs, rg = nw / cs;
    nw = rg * cs;
    // rows a warp takes at once: a chunk near the target size, at least one row
    int rw = rw_first;
    while (rw > 1 && (uint64_t)rw * row_bytes > (uint64_t)CHUNK_BYTES) rw /= 2;
    pl.rw = rw; pl.runs_per_warp = per; pl.nw = nw; pl.nwmax = nwmax; pl.cs = cs; pl.rg = rg;
    const int stage_rows = rg * rw;
    pl.stage_stride = ((uint32_t)rw * row_bytes + 64u + 127u) / 128u * 128u;       // one chunk, up to 15 bytes of misalignment before it and a block's length of slack after it
    GemvArgs &a = pl.args;
    a.row_bytes = row_bytes;
    a.nw = nw; a.cs = cs; a.rg = rg; a.stage_rows = stage_rows;
    a.units = (rows + stage_rows - 1) / stage_rows;
    a.chunks = (rows + rw - 1) / rw;
    a.chunk_align = back ? 32 / rw : 1;
    a.row_flip = (row_bytes & 2u) ? 1u : 0u;
    a.off_x = SMEM_HEADER;
    a.off_part = a.off_x + xprep_bytes(cols);
    // partial sums: room for every round of a block when that is small, else PART_BYTES with flushes in between
    const uint32_t round_bytes = (uint32_t)stage_rows * cs * 4u;
    // blocks of one grid an SM: one, so that the blocks sharing an SM belong to successive launches
    const int gctas = 1;
    const int grid_guess = g_sm_count < 1 ? 1 : g_sm_count * gctas;
    const uint32_t rounds = (uint32_t)(((a.chunks + grid_guess - 1) / grid_guess + rg - 1) / rg) + 1u;
    const uint32_t part_cap = ctas > 1 ? PART_BYTES / 4 : PART_BYTES;
    const uint32_t part_bytes = rounds * round_bytes < part_cap ? (rounds * round_bytes + 127u) / 128u * 128u : part_cap;
    a.off_ring = (a.off_part + part_bytes + 127u) / 128u * 128u;
    a.flush_units = (int)(part_bytes / round_bytes);
    if (a.flush_units < 1) return QB200_E_LIMIT;
    if (a.off_ring + (uint64_t)rg * pl.stage_stride > budget) return QB200_E_LIMIT;
    pl.grid = a.chunks < g_sm_count * gctas ? a.chunks : g_sm_count * gctas;
    int slots = (int)((budget - a.off_ring) / pl.stage_stride);
    if (slots > MAX_SLOTS) slots = MAX_SLOTS;
    const int per_block = ((a.chunks + pl.grid - 1) / pl.grid + a.chunk_align - 1 + rg - 1) / rg;      // rounds of rg chunks a block takes at most
    if (slots > per_block * rg) slots = per_block * rg;
    slots = slots / rg * rg;                     // every row group owns the same number of slots
    if (slots < rg) return QB200_E_LIMIT;
    pl.stages = slots;
    pl.deep = slots >= 2 * rg || slots >= per_block * rg;        // a row group can compute on one chunk while the next arrives
    a.slots = slots;
    // the whole-SM variant holds half its ring back until x has been asked for (x's reads then meet idle queues); the
    // small blocks, with two to four slots, ask for all of them at once (no measurable difference either way)
    a.prefetch = nwmax == 4 ? slots : (slots + 1) / 2;
    a.slot_stride = pl.stage_stride;
    pl.smem_bytes = a.off_ring + (uint32_t)slots * pl.stage_stride;
    return 0;
}

// The plan of a call.  `overlapped` = the call is expected to run beside its neighbours in the stream (it shares no
// buffer with the launches that may still be running, or the launch before it was such a call): then blocks of 4
// consumer warps, one an SM, so that four successive launches are
// resident together and one's start and end hide behind the others' streaming; the chunk shrinks until a row group has
// two slots.  A call in a chain of calls that wait for one another gets the whole SM instead: blocks of 16 warps.  The
// checking variant (per-block sums) always takes the latter, a row at a time, and so does a call that also encodes
// its output (that variant exists for the whole-SM blocks only).
static int plan_gemv(int fmt_a, int rows, int cols, bool sums, bool overlapped, bool back, GemvPlan &pl)
{
    const int rw_first = sums ? 1 : 4;
    if (!sums && !back && overlapped) {      // (a publishing call is never `overlapped`)
        for (int rw = rw_first; rw >= 1; rw /= 2)
            if (plan_blocks(fmt_a, rows, cols, 4, rw, back, pl) == 0 && pl.deep) return 0;
    }
    return plan_blocks(fmt_a, rows, cols, 16, rw_first, back, pl);
}

template <int FMT, int RW, int RUNS, bool SUMS, int NW, int TAIL>
static cudaError_t launch_one(const GemvPlan &pl, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(pl.grid);
    cfg.blockDim = dim3((pl.nw + 1) * 32);
    cfg.dynamicSmemBytes = pl.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = pl.serial ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, gemv_kernel<FMT, RW, RUNS, SUMS, NW, TAIL>, pl.args);
}

template <int FMT, int RW, bool SUMS, int NW, int TAIL>
static cudaError_t launch_runs(const GemvPlan &pl, cudaStream_t stream)
{
    if (pl.runs_per_warp == 1) return launch_one<FMT, RW, 1, SUMS, NW, TAIL>(pl, stream);
    if (pl.runs_per_warp == 2 || FMT != QB200_Q6_K) return launch_one<FMT, RW, 2, SUMS, NW, TAIL>(pl, stream);
    if (pl.runs_per_warp == 3) return launch_one<FMT, RW, FMT == QB200_Q6_K ? 3 : 2, SUMS, NW, TAIL>(pl, stream);
    return launch_one<FMT, RW, FMT == QB200_Q6_K ? 4 : 2, SUMS, NW, TAIL>(pl, stream);
}

template <int FMT, int NW, int TAIL>
static cudaError_t launch_rows(const GemvPlan &pl, cudaStream_t stream)
{
    switch (pl.rw) {
    case 4: return launch_runs<FMT, 4, false, NW, TAIL>(pl, stream);
    case 2: return launch_runs<FMT, 2, false, NW, TAIL>(pl, stream);
    default: return launch_runs<FMT, 1, false, NW, TAIL>(pl, stream);
    }
}

template <int FMT>
static cudaError_t launch_fmt(const GemvPlan &pl, bool sums, cudaStream_t stream)
{
    if (sums) return launch_runs<FMT, 1, true, 16, TAIL_NONE>(pl, stream);      // the checking variant: a row at a time
    if (pl.args.yb) return launch_rows<FMT, 16, TAIL_BACK>(pl, stream);         // with `Back`: always whole-SM blocks
    if (pl.args.publish.world > 0) return launch_rows<FMT, 16, TAIL_PUBLISH>(pl, stream); // with the exchange: whole-SM blocks too
    return pl.nwmax == 4 ? launch_rows<FMT, 4, TAIL_NONE>(pl, stream) : launch_rows<FMT, 16, TAIL_NONE>(pl, stream);
}

template <int FMT, int RW, bool SUMS, int NW, int TAIL>
static cudaError_t set_attr_runs(int bytes)
{
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(gemv_kernel<FMT, RW, 1, SUMS, NW, TAIL>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes))) return e;
    if ((e = cudaFuncSetAttribute(gemv_kernel<FMT, RW, 2, SUMS, NW, TAIL>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes))) return e;
    if (FMT == QB200_Q6_K) {
        if ((e = cudaFuncSetAttribute(gemv_kernel<FMT, RW, FMT == QB200_Q6_K ? 3 : 2, SUMS, NW, TAIL>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes))) return e;
        e = cudaFuncSetAttribute(gemv_kernel<FMT, RW, FMT == QB200_Q6_K ? 4 : 2, SUMS, NW, TAIL>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    }
    return e;
}

template <int FMT>
static cudaError_t set_attr(int bytes)
{
    cudaError_t e;
    const int small = (bytes + 1024) / 4 - 2048;                 // what a block of the four-an-SM variant may ask for
    if ((e = set_attr_runs<FMT, 1, true, 16, TAIL_NONE>(bytes))) return e;
    if ((e = set_attr_runs<FMT, 1, false, 16, TAIL_NONE>(bytes))) return e;
    if ((e = set_attr_runs<FMT, 2, false, 16, TAIL_NONE>(bytes))) return e;
    if ((e = set_attr_runs<FMT, 4, false, 16, TAIL_NONE>(bytes))) return e;
    if ((e = set_attr_runs<FMT, 1, false, 16, TAIL_BACK>(bytes))) return e;
    if ((e = set_attr_runs<FMT, 2, false, 16, TAIL_BACK>(bytes))) return e;
    if ((e = set_attr_runs<FMT, 4, false, 16, TAIL_BACK>(bytes))) return e;
    if ((e = set_attr_runs<FMT, 1, false, 16, TAIL_PUBLISH>(bytes))) return e;
    if ((e = set_attr_runs<FMT, 2, false, 16, TAIL_PUBLISH>(bytes))) return e;
    if ((e = set_attr_runs<FMT, 4, false, 16, TAIL_PUBLISH>(bytes))) return e;
    if ((e = set_attr_runs<FMT, 1, false, 4, TAIL_NONE>(small))) return e;
    if ((e = set_attr_runs<FMT, 2, false, 4, TAIL_NONE>(small))) return e;
    return set_attr_runs<FMT, 4, false, 4, TAIL_NONE>(small);
}

cudaError_t gemv_init(int sm_count, int max_smem, int *status)
{
    g_epoch++;                   // plans and launch histories made for the device bound before are void
    gemv_forget_history();
    g_sm_count = sm_count;
    g_max_smem = max_smem;
    g_status = status;
    cudaError_t e;
    if ((e = set_attr<QB200_Q8_0>(max_smem))) return e;
    if ((e = set_attr<QB200_Q4_0>(max_smem))) return e;
    if ((e = set_attr<QB200_Q4_K>(max_smem))) return e;
    return set_attr<QB200_Q6_K>(max_smem);
}

// Returns 0, a negative QB200_E_* or a positive cudaError_t.  Arguments are already validated.

// Ordering against earlier gemv launches of this thread.  A gemv is normally launched as a programmatic dependent of
// whatever precedes it in the stream, and may skip griddepcontrol.wait; every launch lets its successor be scheduled
// at its very start, before its own wait (if any) has passed, so any launch since the last point of full order may still
// be running when a new one starts.  The history holds what those launches read and wrote.  A new call that touches
// none of it (its inputs are not their outputs, its outputs are not their inputs or outputs) is "independent": no
// wait.  A call that conflicts waits.  griddepcontrol.wait orders it after its direct predecessor's completion, which is
// enough when that predecessor itself waited for everything before it (`settled`: waiting for the newest entry is then
// waiting for all of them); the call joins the history, which stays: its own successor may start while any of them
// still runs.  Otherwise (launches running side by side, or nothing known) the call is launched without the
// programmatic attribute, which orders it after everything earlier in the stream, and the history restarts with it.
// Other work in the stream (kernels, copies) is launched without the attribute and only adds order.
struct Touched { const uint8_t *p; size_t n; };
struct Launched { Touched a, x, y, yb; bool everything; };
constexpr int HISTORY = 64;
static thread_local struct {
    cudaStream_t stream;
    int count;              // 0: nothing known about the stream (first call, another stream, a call outside this record)
    bool settled;           // the newest entry waited for everything before it: to wait for it is to wait for them all
    Launched at[HISTORY];
} t_hist = { nullptr, 0, false, {} };

void gemv_forget_history() { t_hist.count = 0; }

void gemv_history_everything(cudaStream_t stream)
{
    memset(&t_hist.at[0], 0, sizeof t_hist.at[0]);
    t_hist.at[0].everything = true;
    t_hist.stream = stream;
    t_hist.count = 1;
    t_hist.settled = true;
}

// The host thread's cached plans belong to the device they were made for: dropped when the library binds another one.
static thread_local int t_plans_cached = 0, t_plans_next = 0, t_plans_epoch = 0;

static bool overlap(const Touched &u, const Touched &v)
{
    return u.n && v.n && u.p < v.p + v.n && v.p < u.p + u.n;
}

// does the new call read what `old` wrote, or write what `old` read or wrote?
static bool conflicts(const Launched &now, const Launched &old)
{
    if (old.everything) return true;
    const Touched *outs[2] = { &now.y, &now.yb }, *old_outs[2] = { &old.y, &old.yb };
    for (int i = 0; i < 2; i++) {
        if (overlap(now.x, *old_outs[i]) || overlap(now.a, *old_outs[i])) return true;
        if (overlap(*outs[i], old.x) || overlap(*outs[i], old.a)) return true;
        for (int j = 0; j < 2; j++) if (overlap(*outs[i], *old_outs[j])) return true;
    }
    return false;
}

int gemv_launch(int fmt_a, int fmt_x, const void *a, const void *x, float *y, int32_t *sums, int fmt_y, void *y_blocks, int rows,
                int cols, cudaStream_t stream, const void *publish)
{
    if (rows == 0) return 0;
    const size_t row_bytes = (size_t)(cols / block_values(fmt_a)) * block_bytes(fmt_a);
    Launched now;
    now.a = { (const uint8_t *)a, (size_t)rows * row_bytes };
    now.x = { (const uint8_t *)x, fmt_x == QB200_F32 ? (size_t)cols * 4 : (size_t)(cols / 32) * block_bytes(fmt_x) };
    now.y = { (const uint8_t *)y, (size_t)rows * 4 };
    now.yb = { (const uint8_t *)y_blocks, y_blocks ? (size_t)((rows + 31) / 32) * block_bytes(fmt_y) : 0 };
    now.everything = false;
    const bool known = t_hist.count > 0 && t_hist.stream == stream;
    // a publishing launch writes memory this record does not describe (the other GPUs' copies): it waits, and so does its successor
    bool conflict = !known || sums || publish || t_hist.count == HISTORY;
    bool weights_written = false;           // the producer reads A before any wait: nothing in flight may write it
    if (known) {
        for (int i = 0; i < t_hist.count; i++) {
            conflict = conflict || conflicts(now, t_hist.at[i]);
            weights_written = weights_written || overlap(now.a, t_hist.at[i].y) || overlap(now.a, t_hist.at[i].yb);
        }
    }
    const bool independent = !conflict;
    // the launch before this one ran beside its neighbours: expect the same of this one and of the next, whether or
    // not this one has to wait first (the choice of block variant below)
    const bool in_a_burst = known && !t_hist.settled;
    // full order by the launch itself: nothing known, the weights themselves in flight (the producer reads them before
    // any wait), launches side by side that a wait on the newest would not cover, or a history that has no room left
    const bool serial = conflict && (!known || weights_written || !t_hist.settled || t_hist.count == HISTORY);
    if (publish) {
        // it writes memory this record does not describe, and has itself waited for everything before it (by its launch
        // or by griddepcontrol.wait after a settled history): the next call waits for it, by griddepcontrol.wait alone
        memset(&t_hist.at[0], 0, sizeof t_hist.at[0]);
        t_hist.at[0].everything = true;
        t_hist.stream = stream;
        t_hist.count = 1;
        t_hist.settled = true;
    } else if (independent) {
        t_hist.at[t_hist.count++] = now;
        t_hist.settled = false;
    } else if (serial) {
        t_hist.stream = stream;
        t_hist.at[0] = now;
        t_hist.count = 1;
        t_hist.settled = true;
    } else {
        // waited by griddepcontrol.wait: everything before it is covered by waiting for it, but may still be running
        // when the next call is scheduled
        t_hist.at[t_hist.count++] = now;
        t_hist.settled = true;
    }
    // the last few shapes' plans are kept: a decode loop calls the same shapes over and over
    static thread_local struct { int fmt, rows, cols, kind; GemvPlan plan; } cache[8];
    int &cached = t_plans_cached, &next = t_plans_next;
    if (t_plans_epoch != g_epoch) { cached = next = 0; t_plans_epoch = g_epoch; }
    GemvPlan pl;
    bool hit = false;
    const bool overlapped = (independent || in_a_burst) && !sums && !publish;
    const int kind = (sums ? 2 : overlapped ? 1 : 0) | (y_blocks ? 4 : 0) | (publish ? 8 : 0);
    for (int i = 0; i < cached && !hit; i++)
        if (cache[i].fmt == fmt_a && cache[i].rows == rows && cache[i].cols == cols && cache[i].kind == kind) { pl = cache[i].plan; hit = true; }
    if (!hit) {
        int rc = plan_gemv(fmt_a, rows, cols, sums != nullptr, overlapped, y_blocks != nullptr, pl);
        if (rc) return rc;
        cache[next].fmt = fmt_a; cache[next].rows = rows; cache[next].cols = cols; cache[next].kind = kind; cache[next].plan = pl;
        next = (next + 1) % 8;
        if (cached < 8) cached++;
    }
    pl.args.a = (const uint8_t *)a;
    pl.args.xprep = nullptr;
    pl.args.x = x;
    pl.args.fmt_x = fmt_x;
    pl.args.independent = independent ? 1 : 0;
    pl.serial = serial;
    pl.args.y = y;
    pl.args.yb = (uint8_t *)y_blocks;
    pl.args.fmt_y = fmt_y;
    pl.args.sums = sums;
    if (publish) pl.args.publish = *(const GemvPublish *)publish;
    else memset(&pl.args.publish, 0, sizeof pl.args.publish);
    pl.args.status = g_status;
    pl.args.rows = rows;
    pl.args.cols = cols;
    cudaError_t e;
    switch (fmt_a) {
    case QB200_Q8_0: e = launch_fmt<QB200_Q8_0>(pl, sums != nullptr, stream); break;
    case QB200_Q4_0: e = launch_fmt<QB200_Q4_0>(pl, sums != nullptr, stream); break;
    case QB200_Q4_K: e = launch_fmt<QB200_Q4_K>(pl, sums != nullptr, stream); break;
    default: e = launch_fmt<QB200_Q6_K>(pl, sums != nullptr, stream); break;
    }
    return (int)e;
}

// ---------------------------------------------------------------------------------- the variant that allocates nothing

// Scratch of the no-allocation entry point: x in the gemv's own layout (prepare_x_kernel) for up to
// QB200_NOALLOC_MAX_COLS columns, and a status word.  Both live in every device's image of this library from load to
// exit.  In host code these names are only handles: the device address comes from cudaGetSymbolAddress.
constexpr int NOALLOC_MAX_COLS = QB200_NOALLOC_MAX_COLS;
constexpr uint32_t NOALLOC_SCRATCH_BYTES = (NOALLOC_MAX_COLS + 2047) / 2048 * 2048 + ((NOALLOC_MAX_COLS / 32 + 2) * 8 + 255) / 256 * 256;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];
static __device__ int g_noalloc_status;

struct NoAllocDevice {
    void *scratch;
    int *status;
};
static NoAllocDevice g_noalloc[64];
static std::mutex g_noalloc_lock;           // first use on a device may come from any host thread

// First use on the current device: resolves the two symbols' device addresses and gives the kernels their
// shared-memory attribute on this device.  Allocates nothing.
static int noalloc_setup(int device, NoAllocDevice **out)
{
    if (device < 0 || device >= 64) return QB200_E_DEVICE;
    std::lock_guard<std::mutex> guard(g_noalloc_lock);
    NoAllocDevice &d = g_noalloc[device];
    if (!d.scratch) {
        cudaError_t e;
        int major = 0, sms = 0, smem = 0;
        if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device))) return (int)e;
        if (major != 10) return QB200_E_DEVICE;
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device))) return (int)e;
        if ((e = cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device))) return (int)e;
        void *scratch = nullptr, *status = nullptr;
        if ((e = cudaGetSymbolAddress(&scratch, g_noalloc_scratch))) return (int)e;
        if ((e = cudaGetSymbolAddress(&status, g_noalloc_status))) return (int)e;
        if (g_sm_count == 0) { g_sm_count = sms; g_max_smem = smem; }
        if ((e = set_attr<QB200_Q8_0>(smem)) || (e = set_attr<QB200_Q4_0>(smem)) || (e = set_attr<QB200_Q4_K>(smem)) || (e = set_attr<QB200_Q6_K>(smem)))
            return (int)e;
        d.status = (int *)status;
        d.scratch = scratch;
    }
    *out = &d;
    return 0;
}

// y = A.x as gemv_launch computes it, with x prepared in the static array instead of shared memory.  Nothing in the
// array has to start at zero: the preparing kernel rewrites every byte the gemv reads.  The status word is zero when the
// module loads and is only ever OR-ed into by the kernels; gemv_noalloc_status reads and clears it, so a bounded wait
// that gave up in any call since the last reading is reported, not just one in the latest call.
int gemv_launch_noalloc(int fmt_a, int fmt_x, const void *a, const void *x, float *y, int rows, int cols, cudaStream_t stream)
{
    if (cols > NOALLOC_MAX_COLS) return QB200_E_LIMIT;
    if (rows == 0) return 0;
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e) return (int)e;
    NoAllocDevice *dev = nullptr;
    int rc = noalloc_setup(device, &dev);
    if (rc) return rc;
    GemvPlan pl;
    if ((rc = plan_gemv(fmt_a, rows, cols, false, false, false, pl))) return rc;
    pl.args.a = (const uint8_t *)a;
    pl.args.xprep = (const uint8_t *)dev->scratch;
    pl.args.x = nullptr;
    pl.args.fmt_x = fmt_x;
    pl.args.independent = 0;
    t_hist.count = 0;
    pl.serial = false;
    pl.args.y = y;
    pl.args.yb = nullptr;
    pl.args.fmt_y = 0;
    pl.args.sums = nullptr;
    memset(&pl.args.publish, 0, sizeof pl.args.publish);
    pl.args.status = dev->status;
    pl.args.rows = rows;
    pl.args.cols = cols;
    const int blocks = cols / 32, threads = 128, grid = (blocks + 1 + threads - 1) / threads;
    if (fmt_a == QB200_Q8_0 || fmt_a == QB200_Q4_0) prepare_x_kernel<true><<<grid, threads, 0, stream>>>(x, fmt_x, cols, (uint8_t *)dev->scratch, 0);
    else prepare_x_kernel<false><<<grid, threads, 0, stream>>>(x, fmt_x, cols, (uint8_t *)dev->scratch, 0);
    if ((e = cudaGetLastError())) return (int)e;
    switch (fmt_a) {
    case QB200_Q8_0: e = launch_fmt<QB200_Q8_0>(pl, false, stream); break;
    case QB200_Q4_0: e = launch_fmt<QB200_Q4_0>(pl, false, stream); break;
    case QB200_Q4_K: e = launch_fmt<QB200_Q4_K>(pl, false, stream); break;
    default: e = launch_fmt<QB200_Q6_K>(pl, false, stream); break;
    }
    return (int)e;
}

// Reads and clears the static status word of the current device (0 = no bounded wait gave up since the last reading);
// synchronizes the device.
int gemv_noalloc_status(int *value)
{
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e) return (int)e;
    if (device < 0 || device >= 64 || !g_noalloc[device].status) { *value = 0; return 0; }
    if ((e = cudaDeviceSynchronize())) return (int)e;
    if ((e = cudaMemcpy(value, g_noalloc[device].status, sizeof(int), cudaMemcpyDeviceToHost))) return (int)e;
    if (*value) {
        const int zero = 0;
        if ((e = cudaMemcpy(g_noalloc[device].status, &zero, sizeof zero, cudaMemcpyHostToDevice))) return (int)e;
    }
    return 0;
}

}  // namespace qb
