// Block-scaled A.B^T for sm_100a: C (m x n, f32) = A (m x k) . B (n x k)^T with A and B in Q8_0 / Q4_0 rows.
//
// Replaces Ptx.MatMulBlocks (reference src/MatMulBlocks.cs:178-386: 64 x 64 tiles, mma.sync m16n8k32, operands staged
// by 16-bit loads).  The arithmetic is that kernel's: per k-block of 32 the exact s32 product sum D, then
//     acc = fma(float(D), sA*sB, acc)        (src/MatMulBlocks.cs:339-347), k-blocks in ascending order,
// so the f32 result equals the reference's device result bit for bit.
//
// Two steps:
//  1. pack_rows_kernel re-lays each operand in scratch memory for the tensor cores: the scales are stripped out of the
//     34- / 18-byte blocks into an f32 plane, Q4_0 nibbles are widened to int8 (q - 8), and the int8 codes are stored
//     tile by tile in the canonical K-major, unswizzled shared-memory layout of tcgen05 (8-row x 16-byte core matrices),
//     so that a whole (128 rows x several k-blocks) slab is one contiguous run of bytes.
//  2. matmul_kernel: one 128 x 128 tile of C a block.  A producer warp brings slabs of codes and scales into a ring of
//     shared-memory stages with untiled TMA bulk copies; one thread issues a tcgen05.mma (kind::i8, M 128, N 128, K 32)
//     per k-block into one of four 128-column accumulators in tensor memory, with accumulation off, and commits it to
//     an mbarrier; sixteen epilogue warps read the s32 sums back with tcgen05.ld, scale them in f32 (packed f32x2
//     instructions) and add them to register accumulators while the next k-blocks' products run.
#include "common.cuh"
#include "launch.h"

namespace qb {

#ifndef QB_MM_WAIT
#define QB_MM_WAIT mbar_wait_lanes
#endif

// The probes inside the kernel are tuning aids: compiled in only with -DQB_MM_TUNING.
#ifdef QB_MM_TUNING
#define MM_PROBE(p) ((p).probe)
#else
#define MM_PROBE(p) 0
#endif

constexpr int TILE = 128;            // rows of A and of B per block tile
constexpr int KS = 4;                // k-blocks per shared-memory stage (even: pairs of k-blocks never straddle stages)
constexpr int MM_STAGES = 5;
constexpr int TMEM_STAGES = 4;       // 4 x 128 columns = all 512 columns of tensor memory
constexpr int SLAB = TILE * 32;      // bytes of codes per tile and k-block
constexpr int EPI_WARPS = 16;
constexpr int MM_THREADS = 32 * (2 + EPI_WARPS);   // warp 0 producer, warp 1 MMA, the rest epilogue
constexpr uint32_t STAGE_BYTES = KS * (2 * SLAB + 4 * TILE * 4);   // codes of A and B, scales of A and B, A's scaled sums, B's mins
constexpr uint32_t MM_HEADER = 1024;
constexpr uint32_t MM_ZEROS = MM_HEADER + MM_STAGES * STAGE_BYTES;    // 2 KB of zeros: the absent second half of a 16-value k-block
constexpr uint32_t MM_SMEM = MM_ZEROS + SLAB / 2;

struct PackedOperand {
    const uint8_t *codes;    // [tile][kb][2][16][8][16]
    const float *scales;     // [tile][kb][128]
    const float *extra;      // [tile][kb][128]: A: scale * sum of the block's codes; B (Q4_K): dmin * m.  Null when unused.
};

struct MatmulArgs {
    PackedOperand a, b;
    float *c;
    int32_t *sums;
    int *status;
    int m, n, kb;
    int probe;       // tuning aid: 1 = no arithmetic, 2 = no tensor-memory reads; 0 in normal use
};

// ---------------------------------------------------------------------------------- step 1: operands for the tensor cores

// A block of 256 threads re-lays 32 rows x 8 k-blocks.  The rows' bytes (8 consecutive blocks of a row are contiguous
// in the raw operand, 2-byte aligned) are first copied to shared memory with coalesced loads (16 bytes wide when the
// rows lie on 16-byte boundaries, else 2); then a thread a
// block assembles its 32 int8 values and its scale.  Row r of tile t lands at byte
// (t*kb + b)*4096 + j*2048 + (r/8)*128 + (r%8)*16 for its bytes 16j..16j+15, and its scale at ((t*kb + b)*128 + r).
// Rows past `rows` (the padding of the last tile) are written as zeros.
// SPLIT (against Q6_K rows, whose scales change every 16 values): a block becomes two k-blocks of 16 values each, 2 KB
// of codes a tile (the other 16 values of the tensor instruction's 32 are zeros that are never stored), same scale.
template <int FMT, bool SPLIT>
__global__ void __launch_bounds__(256) pack_rows_kernel(const uint8_t *raw, int rows, int kb, uint8_t *codes, float *scales, float *usums)
{
    // halfwords a row segment; the pitch is an odd number of 32-bit words, so the 32 rows start in 32 different banks
    constexpr int BB = block_bytes(FMT), HALVES = 8 * BB / 2, PITCH = HALVES + 2, VECS = 8 * BB / 16;
    __shared__ __align__(16) uint16_t seg[32 * PITCH];
    const int r0 = blockIdx.x * 32, b0 = blockIdx.y * 8;
    const int nb = min(8, kb - b0), halves = nb * BB / 2;
    const size_t row_bytes = (size_t)kb * BB;
    if (nb == 8 && (((uintptr_t)raw | row_bytes) & 15) == 0) {
        // whole segments on 16-byte boundaries (8 blocks are 272 or 144 bytes): 16-byte loads
        for (int idx = threadIdx.x; idx < 32 * VECS; idx += 256) {
            const int rr = idx / VECS, c = idx - rr * VECS;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r0 + rr < rows) v = __ldg((const uint4 *)(raw + (size_t)(r0 + rr) * row_bytes + (size_t)b0 * BB) + c);
            uint32_t *dst = (uint32_t *)(seg + rr * PITCH) + c * 4;
            dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
        }
    } else {
        for (int idx = threadIdx.x; idx < 32 * HALVES; idx += 256) {
            const int rr = idx / HALVES, h = idx - rr * HALVES;
            uint16_t v = 0;
            if (r0 + rr < rows && h < halves) v = __ldg((const uint16_t *)(raw + ((size_t)(r0 + rr) * kb + b0) * BB) + h);
            seg[rr * PITCH + h] = v;
        }
    }
    __syncthreads();
    const int rl = threadIdx.x & 31, bl = threadIdx.x >> 5, r = r0 + rl, b = b0 + bl;
    if (b >= kb) return;
    const uint16_t *p = seg + rl * PITCH + bl * (BB / 2);
    const float d = half_bits_to_float(p[0]);           // zero rows read as scale 0, codes 0 (Q4_0: see below)
    uint32_t w[8];
    if (FMT == QB200_Q8_0) {
#pragma unroll
        for (int i = 0; i < 8; i++) w[i] = (uint32_t)p[1 + 2 * i] | (uint32_t)p[2 + 2 * i] << 16;
    } else {
        // value i in the low nibble of byte i, value i + 16 in the high nibble, each minus 8 (src/MatMulBlocks.cs:282-299)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t n = (uint32_t)p[1 + 2 * i] | (uint32_t)p[2 + 2 * i] << 16;
            w[i] = __vsub4(n & 0x0F0F0F0Fu, 0x08080808u);
            w[i + 4] = __vsub4((n >> 4) & 0x0F0F0F0Fu, 0x08080808u);
        }
        if (r >= rows) {
#pragma unroll
            for (int i = 0; i < 8; i++) w[i] = 0;
        }
    }
    const int t = r / TILE, rr = r % TILE;
    uint8_t *slab = codes + ((size_t)t * kb + b) * SLAB + (rr >> 3) * 128 + (rr & 7) * 16;
    *(uint4 *)slab = make_uint4(w[0], w[1], w[2], w[3]);
    *(uint4 *)(slab + SLAB / 2) = make_uint4(w[4], w[5], w[6], w[7]);       // SPLIT: this is the next k-block's slab
    if (SPLIT) {
        scales[((size_t)t * kb + b) * 2 * TILE + rr] = d;
        scales[((size_t)t * kb + b) * 2 * TILE + TILE + rr] = d;
        return;
    }
    scales[((size_t)t * kb + b) * TILE + rr] = d;
    if (usums) {            // against a format with mins: scale * (sum of the codes), the factor of the other operand's min
        int sum = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) asm("dp4a.s32.s32 %0, %1, %2, %0;" : "+r"(sum) : "r"(w[i]), "r"(0x01010101));
        usums[((size_t)t * kb + b) * TILE + rr] = __fmul_rn(d, (float)sum);
    }
}

// Q4_K rows as an operand: a block of 256 threads re-lays 32 rows x one super-block (144 bytes, src/Blocks.cs:79-96) into
// eight k-blocks.  Sub-block j (32 values): codes q = the low (j even) or high nibbles of qs[32 (j/2) ..], kept as int8
// 0..15; scale d * sc and min dmin * m, each rounded to f32 as DecodeQ4_K rounds them, with sc and m unpacked as ScaleMin
// does (src/Blocks.cs:73-77).  value = (d*sc)*q - dmin*m, so a k-block contributes sA*(d*sc)*sum(qA*q) - (dmin*m)*sA*sum(qA).
__global__ void __launch_bounds__(256) pack_q4_k_kernel(const uint8_t *raw, int rows, int kb, uint8_t *codes, float *scales, float *mins)
{
    constexpr int PITCH = 37;                           // words a row of 144 bytes (36 words): odd, so rows start in different banks
    __shared__ uint32_t seg[32 * PITCH];
    const int r0 = blockIdx.x * 32, sb = blockIdx.y;
    const size_t row_bytes = (size_t)(kb / 8) * 144;
    if ((((uintptr_t)raw | row_bytes) & 15) == 0) {
        for (int idx = threadIdx.x; idx < 32 * 9; idx += 256) {
            const int rr = idx / 9, c = idx - rr * 9;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r0 + rr < rows) v = __ldg((const uint4 *)(raw + (size_t)(r0 + rr) * row_bytes + (size_t)sb * 144) + c);
            uint32_t *dst = seg + rr * PITCH + c * 4;
            dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
        }
    } else {
        for (int idx = threadIdx.x; idx < 32 * 72; idx += 256) {
            const int rr = idx / 72, h = idx - rr * 72;
            uint16_t v = 0;
            if (r0 + rr < rows) v = __ldg((const uint16_t *)(raw + (size_t)(r0 + rr) * row_bytes + (size_t)sb * 144) + h);
            ((uint16_t *)(seg + rr * PITCH))[h] = v;
        }
    }
    __syncthreads();
    const int rl = threadIdx.x & 31, j = threadIdx.x >> 5, r = r0 + rl, b = sb * 8 + j;
    const uint32_t *row = seg + rl * PITCH;
    const uint8_t *sc12 = (const uint8_t *)(row + 1);
    const float d = half_bits_to_float(row[0] & 0xFFFFu), dmin = half_bits_to_float(row[0] >> 16);
    int sc, m;
    if (j < 4) { sc = sc12[j] & 63; m = sc12[j + 4] & 63; }
    else { sc = (sc12[j + 4] & 0xF) | ((sc12[j - 4] >> 6) << 4); m = (sc12[j + 4] >> 4) | ((sc12[j] >> 6) << 4); }
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t n = row[4 + (j >> 1) * 8 + i];
        w[i] = (j & 1) ? (n >> 4) & 0x0F0F0F0Fu : n & 0x0F0F0F0Fu;
    }
    const int t = r / TILE, rr = r % TILE;
    uint8_t *slab = codes + ((size_t)t * kb + b) * SLAB + (rr >> 3) * 128 + (rr & 7) * 16;
    *(uint4 *)slab = make_uint4(w[0], w[1], w[2], w[3]);
    *(uint4 *)(slab + SLAB / 2) = make_uint4(w[4], w[5], w[6], w[7]);
    scales[((size_t)t * kb + b) * TILE + rr] = __fmul_rn(d, (float)sc);       // rows past the end read as zeros throughout
    mins[((size_t)t * kb + b) * TILE + rr] = __fmul_rn(dmin, (float)m);
}

// Q6_K rows as an operand: a block of 256 threads re-lays 32 rows x one super-block (210 bytes, src/Blocks.cs:157-171)
// into sixteen k-blocks of 16 values (2 KB of codes a tile each).  Sub-block s = 8 half + 2 g + (l / 16) holds the values
// 128 half + 32 g + l: code = nibble of ql[64 half + 32 (g & 1) + l] (high nibble for g >= 2) | two bits of
// qh[32 half + l] at 2 g, minus 32; scale d * sc[s] rounded to f32, as DecodeQ6_K's d * sc * q evaluates left to right.
__global__ void __launch_bounds__(256) pack_q6_k_kernel(const uint8_t *raw, int rows, int kb16, uint8_t *codes, float *scales)
{
    constexpr int PITCH = 107;                          // halfwords a row of 210 bytes (105): an odd number of words + 1
    __shared__ __align__(4) uint16_t seg[32 * PITCH];
    const int r0 = blockIdx.x * 32, sb = blockIdx.y;
    const size_t row_bytes = (size_t)(kb16 / 16) * 210;
    for (int idx = threadIdx.x; idx < 32 * 105; idx += 256) {
        const int rr = idx / 105, h = idx - rr * 105;
        uint16_t v = 0;
        if (r0 + rr < rows) v = __ldg((const uint16_t *)(raw + (size_t)(r0 + rr) * row_bytes + (size_t)sb * 210) + h);
        seg[rr * PITCH + h] = v;
    }
    __syncthreads();
    const int rl = threadIdx.x & 31, pairw = threadIdx.x >> 5, r = r0 + rl;
    const uint8_t *row = (const uint8_t *)(seg + rl * PITCH);
    const float d = half_bits_to_float(seg[rl * PITCH + 104]);
    const int t = r / TILE, rr = r % TILE;
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const int s = pairw * 2 + e, half = s >> 3, g = (s >> 1) & 3, l0 = (s & 1) * 16;
        const uint8_t *ql = row + 64 * half + 32 * (g & 1) + l0, *qh = row + 128 + 32 * half + l0;
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t word = 0;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int l = 4 * i + c;
                const int nib = g >= 2 ? ql[l] >> 4 : ql[l] & 15;
                const int q = (nib | (((qh[l] >> (2 * g)) & 3) << 4)) - 32;
                word |= (uint32_t)(q & 255) << (8 * c);
            }
            w[i] = word;
        }
        const size_t kbi = (size_t)t * kb16 + (size_t)sb * 16 + s;
        *(uint4 *)(codes + kbi * (SLAB / 2) + (rr >> 3) * 128 + (rr & 7) * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        scales[kbi * TILE + rr] = __fmul_rn(d, (float)(int8_t)row[192 + s]);
    }
}

// ---------------------------------------------------------------------------------- tcgen05 in inline PTX

__device__ __forceinline__ void tmem_alloc(uint32_t holder_smem, uint32_t columns)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major, no swizzle.  Core matrices are 8 rows x 16 bytes, stored contiguously
// (128 bytes); LBO = bytes between the two 16-byte k-chunks of a row, SBO = bytes between 8-row groups.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo)
{
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (uint64_t)(lbo >> 4) << 16 | (uint64_t)(sbo >> 4) << 32 | (uint64_t)1 << 46;
}

// Instruction descriptor of kind::i8: D s32, A and B signed 8-bit, both K-major, dense, M x N.
__host__ __device__ constexpr uint32_t idesc_s8(int m, int n)
{
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// D[tmem] = A.B^T for one k-block (K = 32 bytes of int8), accumulation off: each k-block needs its own scale.
__device__ __forceinline__ void mma_s8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(0u)
        : "memory");
}

// The mbarrier gets one arrival when every tcgen05.mma this thread issued so far has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 columns of 32-bit accumulators: thread l of the warp gets row (lane base + l), columns c .. c+31.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, int32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------- step 2: the product

// Packed f32 pairs (sm_100): one instruction rounds two independent products / fused multiply-adds, each exactly as
// mul.rn.f32 / fma.rn.f32 would.
__device__ __forceinline__ uint64_t pack2(float lo, float hi)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b)
{
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c)
{
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b)
{
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

// Two s32 block sums as two floats, exactly, without the conversion unit: |D| <= 32*127*127 < 2^22, so the integer
// D + 0x4B400000 is the bit pattern of the float 12582912 + D (1.5 * 2^23 has a unit in the last place of 1 and D stays
// inside its binade), and subtracting 12582912 leaves float(D) with no rounding anywhere.
__device__ __forceinline__ uint64_t to_float2(int32_t d0, int32_t d1)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(d0 + 0x4B400000), "r"(d1 + 0x4B400000));
    return add2(r, pack2(-12582912.f, -12582912.f));
}

// 32 columns of one k-block into the accumulators: acc = fma(float(D), sA*sB, acc) (src/MatMulBlocks.cs:344-346).
__device__ __forceinline__ void scale_add(const int32_t (&v)[32], float sa, const float *sb, uint64_t (&acc)[16])
{
#ifdef QB_MM_SCALAR
#pragma unroll
    for (int c4 = 0; c4 < 8; c4++) {
        const float4 s = *(const float4 *)(sb + 4 * c4);
        float a0, a1, a2, a3;
        unpack2(acc[2 * c4], a0, a1);
        unpack2(acc[2 * c4 + 1], a2, a3);
        a0 = __fmaf_rn((float)v[4 * c4], __fmul_rn(sa, s.x), a0);
        a1 = __fmaf_rn((float)v[4 * c4 + 1], __fmul_rn(sa, s.y), a1);
        a2 = __fmaf_rn((float)v[4 * c4 + 2], __fmul_rn(sa, s.z), a2);
        a3 = __fmaf_rn((float)v[4 * c4 + 3], __fmul_rn(sa, s.w), a3);
        acc[2 * c4] = pack2(a0, a1);
        acc[2 * c4 + 1] = pack2(a2, a3);
    }
    return;
#endif
    const uint64_t sa2 = pack2(sa, sa);
#pragma unroll
    for (int c4 = 0; c4 < 8; c4++) {
        const ulonglong2 s = *(const ulonglong2 *)(sb + 4 * c4);
        acc[2 * c4] = fma2(pack2((float)v[4 * c4], (float)v[4 * c4 + 1]), mul2(sa2, s.x), acc[2 * c4]);
        acc[2 * c4 + 1] = fma2(pack2((float)v[4 * c4 + 2], (float)v[4 * c4 + 3]), mul2(sa2, s.y), acc[2 * c4 + 1]);
    }
}

// The min term of one k-block for 32 columns: acc = fma(-(dmin*m), sA*sum(qA), acc); `nu` is -(sA*sum(qA)).
__device__ __forceinline__ void min_add(float nu, const float *wb, uint64_t (&acc)[16])
{
    const uint64_t nu2 = pack2(nu, nu);
#pragma unroll
    for (int c4 = 0; c4 < 8; c4++) {
        const ulonglong2 w = *(const ulonglong2 *)(wb + 4 * c4);
        acc[2 * c4] = fma2(w.x, nu2, acc[2 * c4]);
        acc[2 * c4 + 1] = fma2(w.y, nu2, acc[2 * c4 + 1]);
    }
}

// MINS: B is Q4_K; every k-block also has the min term, from two more planes a stage.
// HALF: B is Q6_K; a k-block is 16 values (2 KB of codes an operand), and the tensor instruction's other 16 are read,
// through the descriptor's leading-dimension offset, from a patch of zeros in shared memory.
template <bool SUMS, bool MINS, bool HALF>
__global__ void __launch_bounds__(MM_THREADS, 1) matmul_kernel(const MatmulArgs p)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = smem_u32(smem);
    const uint32_t full0 = base, empty0 = base + 8 * MM_STAGES, tfull0 = base + 16 * MM_STAGES, tempty0 = tfull0 + 8 * TMEM_STAGES;
    const uint32_t holder = tempty0 + 8 * TMEM_STAGES;
    volatile int *abort_flag = (volatile int *)(smem + 512);
    volatile uint32_t *holder_ptr = (volatile uint32_t *)(smem + (holder - base));

    if (threadIdx.x == 0) {
        for (int s = 0; s < MM_STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1 + EPI_WARPS);      // the MMA thread's commit and the epilogue warps
        }
        for (int s = 0; s < TMEM_STAGES; s++) {
            mbar_init(tfull0 + 8 * s, 1);            // only the first two of each are used: one a pair of accumulators
            mbar_init(tempty0 + 8 * s, EPI_WARPS);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (HALF) {
        for (int i = threadIdx.x; i < SLAB / 2 / 16; i += MM_THREADS) *(uint4 *)(smem + MM_ZEROS + i * 16) = make_uint4(0, 0, 0, 0);
        fence_proxy_async();            // the tensor cores read the patch through the async proxy
    }
    if (warp == 1) tmem_alloc(holder, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *holder_ptr;

    const int tn = blockIdx.x, tm = blockIdx.y;
    constexpr uint32_t CB = HALF ? SLAB / 2 : SLAB;       // bytes of codes a k-block and operand
    const int stages_total = (p.kb + KS - 1) / KS;
    uint8_t *ring = smem + MM_HEADER;

    if (warp == 0) {
        // ---- producer: four contiguous slabs a stage (A codes, B codes, A scales, B scales)
        if (lane == 0) {
            int issued = 0;
            for (int it = 0; it < stages_total; it++) {
                const int s = it % MM_STAGES;
                const uint32_t phase = (uint32_t)(it / MM_STAGES) & 1u;
                if (it >= MM_STAGES && !mbar_wait(empty0 + 8 * s, phase ^ 1u, abort_flag, p.status, STATUS_MATMUL_WAIT)) break;
                const int kb0 = it * KS, nkb = min(KS, p.kb - kb0);
                const uint32_t dst = smem_u32(ring + (size_t)s * STAGE_BYTES), bar = full0 + 8 * s;
                const uint32_t code_bytes = (uint32_t)nkb * CB, scale_bytes = (uint32_t)nkb * TILE * 4;
                mbar_arrive_expect_tx(bar, 2 * code_bytes + (MINS ? 4 : 2) * scale_bytes);
                bulk_g2s(dst, p.a.codes + ((size_t)tm * p.kb + kb0) * CB, code_bytes, bar);
                bulk_g2s(dst + KS * SLAB, p.b.codes + ((size_t)tn * p.kb + kb0) * CB, code_bytes, bar);
                bulk_g2s(dst + 2 * KS * SLAB, p.a.scales + ((size_t)tm * p.kb + kb0) * TILE, scale_bytes, bar);
                bulk_g2s(dst + 2 * KS * SLAB + KS * TILE * 4, p.b.scales + ((size_t)tn * p.kb + kb0) * TILE, scale_bytes, bar);
                if (MINS) {
                    bulk_g2s(dst + 2 * KS * SLAB + 2 * KS * TILE * 4, p.a.extra + ((size_t)tm * p.kb + kb0) * TILE, scale_bytes, bar);
                    bulk_g2s(dst + 2 * KS * SLAB + 3 * KS * TILE * 4, p.b.extra + ((size_t)tn * p.kb + kb0) * TILE, scale_bytes, bar);
                }
                issued = it + 1;
            }
            if (*abort_flag) {          // let the copies still in flight land before the block exits
                for (int it = max(0, issued - MM_STAGES); it < issued; it++) {
                    long long start = clock64();
                    while (!mbar_try_wait(full0 + 8 * (it % MM_STAGES), (uint32_t)(it / MM_STAGES) & 1u) && clock64() - start < WAIT_CYCLES) { }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue: one thread.  The four accumulators form two pairs; a pair of k-blocks is issued into a pair of
        // accumulators and committed to one barrier, so the barrier traffic is per two k-blocks on both sides.
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_s8(TILE, TILE);
            // descriptors differ from k-block to k-block only in the start address (16-byte units)
            const uint64_t desc_hi = smem_desc(0, SLAB / 2, 128);
            int np = 0;                            // pairs issued so far
            bool alive = true;
            for (int it = 0; it < stages_total && alive; it++) {
                const int s = it % MM_STAGES;
                if (!mbar_wait(full0 + 8 * s, (uint32_t)(it / MM_STAGES) & 1u, abort_flag, p.status, STATUS_MATMUL_WAIT)) break;
                tc_fence_after();
                const uint32_t a_smem = smem_u32(ring + (size_t)s * STAGE_BYTES), b_smem = a_smem + KS * SLAB;
                const int nkb = min(KS, p.kb - it * KS);
                for (int kk = 0; kk < nkb; kk += 2, np++) {
                    const int pair = np & 1, use = np >> 1;
                    if (use > 0) {
                        if (!mbar_wait(tempty0 + 8 * pair, (uint32_t)(use - 1) & 1u, abort_flag, p.status, STATUS_MATMUL_WAIT)) { alive = false; break; }
                        tc_fence_after();
                    }
                    // HALF: the second 16-byte k-chunk of every row is the zero patch (for A; B's may be anything finite)
                    auto desc = [&](uint32_t addr, bool zeros) {
                        if (HALF) return smem_desc(addr, zeros ? base + MM_ZEROS - addr : SLAB / 2, 128);
                        return desc_hi | (uint64_t)((addr & 0x3FFFFu) >> 4);
                    };
                    mma_s8(tmem + (uint32_t)(2 * pair) * TILE, desc(a_smem + kk * CB, true), desc(b_smem + kk * CB, true), idesc);
                    if (kk + 1 < nkb)
                        mma_s8(tmem + (uint32_t)(2 * pair + 1) * TILE, desc(a_smem + (kk + 1) * CB, true), desc(b_smem + (kk + 1) * CB, true), idesc);
                    mma_commit(tfull0 + 8 * pair);
                }
                mma_commit(empty0 + 8 * s);      // the stage's codes are free once these products have run
            }
        }
    } else {
        // ---- epilogue: a warp owns 32 rows (tensor-memory lanes 32*(warp%4) ..) x 32 columns of every accumulator;
        // four warps a scheduler cover each other's tensor-memory reads.  Two k-blocks a barrier round.
        const int q = warp & 3, cg = (warp - 2) >> 2;
        const int row = tm * TILE + q * 32 + lane, col0 = tn * TILE + cg * 32;
        const uint32_t tlane = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(cg * 32);
        uint64_t acc[16];
#pragma unroll
        for (int c = 0; c < 16; c++) acc[c] = 0ull;
        bool alive = true;
        int s = 0, kk = 0, np = 0;
        uint32_t sphase = 0;
        for (int i = 0; i < p.kb; i += 2, np++) {
            const int pair = np & 1, cnt = min(2, p.kb - i);
            if (!QB_MM_WAIT(tfull0 + 8 * pair, (uint32_t)(np >> 1) & 1u, abort_flag, p.status, STATUS_MATMUL_WAIT)) { alive = false; break; }
            tc_fence_after();
            int32_t v[32];
            if (!(MM_PROBE(p) & 2)) tmem_ld32(tlane + (uint32_t)(2 * pair) * TILE, v);
            if (kk == 0 && !QB_MM_WAIT(full0 + 8 * s, sphase, abort_flag, p.status, STATUS_MATMUL_WAIT)) { alive = false; break; }
            const float *sa_s = (const float *)(ring + (size_t)s * STAGE_BYTES + 2 * KS * SLAB) + kk * TILE;
            const float *sb_s = sa_s + KS * TILE + cg * 32;
            const float sa0 = sa_s[q * 32 + lane], sa1 = sa_s[TILE + q * 32 + lane];
            float nu0 = 0.f, nu1 = 0.f;
            if (MINS) {
                nu0 = -sa_s[2 * KS * TILE + q * 32 + lane];
                nu1 = -sa_s[2 * KS * TILE + TILE + q * 32 + lane];
            }
            tmem_ld_wait();
            if (!(MM_PROBE(p) & 1)) {
                scale_add(v, sa0, sb_s, acc);
                if (MINS) min_add(nu0, sb_s + 2 * KS * TILE, acc);
            }
            if (SUMS && row < p.m) {
#pragma unroll
                for (int c = 0; c < 32; c++)
                    if (col0 + c < p.n) p.sums[((size_t)row * p.n + col0 + c) * p.kb + i] = v[c];
            }
            if (cnt == 2) {
                if (!(MM_PROBE(p) & 2)) tmem_ld32(tlane + (uint32_t)(2 * pair + 1) * TILE, v);
                tmem_ld_wait();
            }
            tc_fence_before();
            if (lane == 0) mbar_arrive(tempty0 + 8 * pair);      // both accumulators have been read (warp-wide reads)
            if (cnt == 2) {
                if (!(MM_PROBE(p) & 1)) {
                    scale_add(v, sa1, sb_s + TILE, acc);
                    if (MINS) min_add(nu1, sb_s + 2 * KS * TILE + TILE, acc);
                }
                if (SUMS && row < p.m) {
#pragma unroll
                    for (int c = 0; c < 32; c++)
                        if (col0 + c < p.n) p.sums[((size_t)row * p.n + col0 + c) * p.kb + i + 1] = v[c];
                }
            }
            kk += 2;
            if (kk >= KS || i + cnt >= p.kb) {
                if (lane == 0) mbar_arrive(empty0 + 8 * s);      // this warp has read the stage's scales
                kk = 0;
                if (++s == MM_STAGES) { s = 0; sphase ^= 1u; }
            }
        }
        if (alive && row < p.m) {
            float *out = p.c + (size_t)row * p.n + col0;
            float f[32];
#pragma unroll
            for (int c = 0; c < 16; c++) unpack2(acc[c], f[2 * c], f[2 * c + 1]);
            if ((p.n & 3) == 0 && col0 + 32 <= p.n && ((uintptr_t)p.c & 15) == 0) {
#pragma unroll
                for (int c4 = 0; c4 < 8; c4++) *(float4 *)(out + 4 * c4) = make_float4(f[4 * c4], f[4 * c4 + 1], f[4 * c4 + 2], f[4 * c4 + 3]);
            } else {
#pragma unroll
                for (int c = 0; c < 32; c++) if (col0 + c < p.n) out[c] = f[c];
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------------- host side

static int *g_mm_status = nullptr;
static int g_mm_probe = 0;

void matmul_set_probe(int mode) { g_mm_probe = mode; }

template <bool SUMS>
static cudaError_t set_mm_attr()
{
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(matmul_kernel<SUMS, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MM_SMEM))) return e;
    if ((e = cudaFuncSetAttribute(matmul_kernel<SUMS, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MM_SMEM))) return e;
    return cudaFuncSetAttribute(matmul_kernel<SUMS, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MM_SMEM);
}

cudaError_t matmul_init(int, int max_smem, int *status)
{
    g_mm_status = status;
    if ((int)MM_SMEM > max_smem) return cudaErrorInvalidValue;
    cudaError_t e;
    if ((e = set_mm_attr<false>())) return e;
    return set_mm_attr<true>();
}

// k-blocks of the product: 32 values each, 16 against Q6_K rows
static int k_blocks(int fmt_b, int k) { return fmt_b == QB200_Q6_K ? k / 16 : k / 32; }
static size_t packed_codes_bytes(int rows, int k) { return (size_t)((rows + TILE - 1) / TILE) * (k / 32) * SLAB; }
static size_t packed_scales_bytes(int rows, int kbs) { return (size_t)((rows + TILE - 1) / TILE) * kbs * TILE * 4; }
static size_t align256(size_t v) { return (v + 255) / 256 * 256; }

// Scratch for both packed operands: codes, scales and the extra plane of A, then the same of B, each on a 256-byte
// boundary (the extra planes are only written when B is Q4_K, but always have their place).
size_t matmul_workspace_bytes(int, int fmt_b, int m, int n, int k)
{
    const int kbs = k_blocks(fmt_b, k);
    return align256(packed_codes_bytes(m, k)) + 2 * align256(packed_scales_bytes(m, kbs)) + align256(packed_codes_bytes(n, k)) +
           2 * align256(packed_scales_bytes(n, kbs));
}

static cudaError_t pack(int fmt, const void *raw, int rows, int k, uint8_t *codes, float *scales, float *extra, bool want_extra,
                        bool split, cudaStream_t stream)
{
    const int kb = k / 32, padded = (rows + TILE - 1) / TILE * TILE;
    if (fmt == QB200_Q4_K) {
        pack_q4_k_kernel<<<dim3(padded / 32, kb / 8), 256, 0, stream>>>((const uint8_t *)raw, rows, kb, codes, scales, extra);
        return cudaGetLastError();
    }
    if (fmt == QB200_Q6_K) {
        pack_q6_k_kernel<<<dim3(padded / 32, k / 256), 256, 0, stream>>>((const uint8_t *)raw, rows, k / 16, codes, scales);
        return cudaGetLastError();
    }
    const dim3 grid(padded / 32, (kb + 7) / 8);
    float *usums = want_extra ? extra : nullptr;
    const uint8_t *r = (const uint8_t *)raw;
    if (fmt == QB200_Q8_0) {
        if (split) pack_rows_kernel<QB200_Q8_0, true><<<grid, 256, 0, stream>>>(r, rows, kb, codes, scales, usums);
        else pack_rows_kernel<QB200_Q8_0, false><<<grid, 256, 0, stream>>>(r, rows, kb, codes, scales, usums);
    } else {
        if (split) pack_rows_kernel<QB200_Q4_0, true><<<grid, 256, 0, stream>>>(r, rows, kb, codes, scales, usums);
        else pack_rows_kernel<QB200_Q4_0, false><<<grid, 256, 0, stream>>>(r, rows, kb, codes, scales, usums);
    }
    return cudaGetLastError();
}

template <bool SUMS>
static void launch_product(bool mins, bool half, dim3 grid, const MatmulArgs &args, cudaStream_t stream)
{
    if (mins) matmul_kernel<SUMS, true, false><<<grid, MM_THREADS, MM_SMEM, stream>>>(args);
    else if (half) matmul_kernel<SUMS, false, true><<<grid, MM_THREADS, MM_SMEM, stream>>>(args);
    else matmul_kernel<SUMS, false, false><<<grid, MM_THREADS, MM_SMEM, stream>>>(args);
}

// fmt_a: Q8_0 / Q4_0; fmt_b: Q8_0 / Q4_0 / Q4_K / Q6_K (k then in whole super-blocks of 256).
int matmul_launch(int fmt_a, int fmt_b, const void *a, const void *b, float *c, int32_t *sums, int m, int n, int k, void *workspace,
                  cudaStream_t stream)
{
    const bool mins = fmt_b == QB200_Q4_K, half = fmt_b == QB200_Q6_K;
    const int kbs = k_blocks(fmt_b, k);
    uint8_t *w = (uint8_t *)workspace;
    uint8_t *a_codes = w;
    float *a_scales = (float *)(w += align256(packed_codes_bytes(m, k)));
    float *a_extra = (float *)(w += align256(packed_scales_bytes(m, kbs)));
    uint8_t *b_codes = (w += align256(packed_scales_bytes(m, kbs)));
    float *b_scales = (float *)(w += align256(packed_codes_bytes(n, k)));
    float *b_extra = (float *)(w += align256(packed_scales_bytes(n, kbs)));
    cudaError_t e;
    if (!(g_mm_probe & 8)) {                // (tuning aid: 8 = operands as packed by an earlier call, 4 = no product)
        if ((e = pack(fmt_a, a, m, k, a_codes, a_scales, a_extra, mins, half, stream))) return (int)e;
        if ((e = pack(fmt_b, b, n, k, b_codes, b_scales, b_extra, false, false, stream))) return (int)e;
    }
    if (g_mm_probe & 4) return 0;
    MatmulArgs args;
    args.a.codes = a_codes; args.a.scales = a_scales; args.a.extra = mins ? a_extra : nullptr;
    args.b.codes = b_codes; args.b.scales = b_scales; args.b.extra = mins ? b_extra : nullptr;
    args.c = c; args.sums = sums; args.status = g_mm_status;
    args.m = m; args.n = n; args.kb = kbs; args.probe = g_mm_probe;
    const dim3 grid((n + TILE - 1) / TILE, (m + TILE - 1) / TILE);
    if (sums) launch_product<true>(mins, half, grid, args, stream);
    else launch_product<false>(mins, half, grid, args, stream);
    return (int)cudaGetLastError();
}

}  // namespace qb
