// Block-scaled A.B^T for sm_100a: C (m x n, f32) = A (m x k) . B (n x k)^T with A in Q8_0 / Q4_0 rows and B in
// Q8_0 / Q4_0 / Q4_K / Q6_K rows.
//
// Replaces Ptx.MatMulBlocks (reference src/MatMulBlocks.cs:178-386: 64 x 64 tiles, mma.sync m16n8k32, operands staged
// by 16-bit loads).  The arithmetic is that kernel's: per k-block of 32 the exact product sum D, then
//     acc = fma(float(D), sA*sB, acc)        (src/MatMulBlocks.cs:339-347), k-blocks in ascending order,
// so the f32 result equals the reference's device result bit for bit.
//
// Two steps:
//  1. pack kernels re-lay an operand for the tensor cores: the scales are stripped out of the raw blocks into an f32
//     plane, nibbles are widened, and the codes are stored as 8-row x 16-byte core matrices (the canonical K-major,
//     unswizzled shared-memory layout of tcgen05), so that the rows a tile needs for one k-block are one contiguous run
//     of bytes.  A (activations) is packed on every call, tile-major; B (weights) is packed k-block-major and can be
//     packed once and kept by the caller (matmul_prepack_b): the layout does not depend on m.
//  2. matmul_kernel (more than 64 rows of A): a persistent grid, one block a multiprocessor.  The output is cut into
//     units of 32 columns of one 128-row tile of A; block b takes a contiguous, equal share of the units and walks it in
//     pieces of up to BNMAX columns.  A producer warp brings codes and scales into a ring of shared-memory stages with
//     untiled TMA bulk copies; two threads issue the tcgen05.mma of the k-blocks (M 128, N = the piece's width or its
//     half, accumulation off) into accumulators in tensor memory and commit each to an mbarrier; the epilogue warps
//     (eight of 64 columns with the scale products on the tensor cores, sixteen of 32 otherwise) read the sums back
//     with tcgen05.ld, scale them in f32 and add them to register accumulators while the products of the next k-blocks
//     run.  Optional tails: C again as blocks (`Back`), or C into the other GPUs' copies (the sharded product: a
//     publisher warp).
//  3. fewrows_kernel / fewq_kernel (at most 64 rows of A): the operands change sides, B's 128 rows on the lanes of tensor
//     memory and A's rows as N = 16 / 32 / 64; fewrows_kernel can also take Q8_0 / Q4_0 weights as raw blocks, fetched
//     by 2-D TMA tile copies and re-laid by converter warps inside the kernel.
//
// Where both operands carry plain f16 block scales (Q8_0 / Q4_0 against Q8_0 / Q4_0) the scale products sA*sB are taken
// by the tensor cores as well (TCS): a second instruction a k-block, kind::f16 with K = 16, multiplies the 128 x 1 column
// of A's scales by the 1 x N row of B's (each stored as a row [d, 0, ..., 0] of eight f16; the other eight of K come
// from a patch of zeros) into a second accumulator.  A product of two f16 values has at most 22 significant bits, so
// the f32 it leaves in tensor memory is exactly mul.rn.f32(sA, sB), and the epilogue is two tensor-memory reads and one
// packed fma an element pair: no shared-memory reads, no scale product on the CUDA cores.  Q4_K / Q6_K scales are
// products d*sc rounded to f32 (17 or more significant bits): they stay on the CUDA-core path.
//
// KIND selects the tensor instruction: 0 = kind::i8 (codes as int8, s32 sums, converted to f32 in the epilogue),
// 1 = kind::f16 (codes as f16: every product and every sum of 32 products is an integer below 2^24, so the f32 sums
// are exact and need no conversion; twice the operand bytes).
#include <cuda.h>                 // CUtensorMap (types only: the encoder is fetched through the runtime)
#include "common.cuh"
#include "encode_blocks.cuh"
#include "launch.h"

namespace qb {

constexpr int TILE = 128;            // rows of A a tile = lanes of tensor memory
constexpr int BNMAX = 128;           // columns of the widest piece = columns of one accumulator in tensor memory
constexpr int EPI_WARPS = 16;
constexpr int GROUP = 8;             // k-blocks a group of B with f16 scales = f16 a 16-byte scale row
// With the scale products on the tensor cores an epilogue warp takes 64 columns instead of 32 (MM_FAT): eight warps,
// two a scheduler (one of each set of 64 columns), 168 registers a thread; four warps instead of eight have to have read
// an accumulator before it is released (measured: equal at M 512, 3-4 % faster at M 2048 and on the 28672 x 8192 shape).
#ifndef MM_FAT
#define MM_FAT 1
#endif
__host__ __device__ constexpr int epi_warps(bool tcs) { return tcs && MM_FAT ? 8 : EPI_WARPS; }
__host__ __device__ constexpr int mm_threads(bool tcs) { return 32 * (3 + epi_warps(tcs)); }     // warp 0 producer, warp 1 and the last warp MMA issue, the rest epilogue
constexpr uint32_t MM_HEADER = 1024;
constexpr uint32_t MM_SMEM_MAX = 232448;           // 227 KB of shared memory a block

// Probes for tuning runs, compiled in only with -DQB_MM_TUNING: bit 0 no epilogue arithmetic, bit 1 no tensor-memory
// reads, bit 2 no accumulator handshake, bits 4-5 the form of the barrier wait.
#ifdef QB_MM_TUNING
#define MM_PROBE(p) ((p).probe)
#define MM_TRACE(p, slot, value) do { if ((p).trace && blockIdx.x == 0) (p).trace[slot] = (value); } while (0)
#define MM_CLOCK() clock64()
#else
#define MM_PROBE(p) 0
#define MM_TRACE(p, slot, value) do { } while (0)
#define MM_CLOCK() 0ll
#endif

// Sizes that follow from the tensor kind, the operand B's format (MINS: Q4_K, HALF: Q6_K with k-blocks of 16 values) and
// where the scale products are taken (TCS: on the tensor cores).
template <int KIND, bool MINS, bool HALF, bool TCS>
struct Cfg {
    static_assert(!TCS || (!MINS && !HALF), "only plain f16 block scales multiply exactly on the tensor cores");
    static constexpr int ESZ = KIND ? 2 : 1;             // bytes a code
    static constexpr int KV = HALF ? 16 : 32;            // values a k-block
    static constexpr int KC = KV * ESZ / 16;             // 16-byte k-chunks a row and k-block
    static constexpr int KS = (KIND ? 64 : 128) / KV;    // k-blocks a shared-memory stage
    static constexpr int SW = TCS ? 16 : 4;              // bytes a scale: an f32, or a row [d, 0 x 7] of f16 for the tensor cores
    static constexpr int TCOLS = TCS ? 2 * BNMAX : BNMAX;   // tensor-memory columns a k-block: the sums, and the scale products
    static constexpr int NT = 512 / TCOLS;               // k-blocks in flight in tensor memory
    static constexpr uint32_t A_KB = TILE * KC * 16, B_KB = BNMAX * KC * 16;      // bytes of codes a k-block
    // TCS: B's scale rows hold eight k-blocks each, one set of rows serves the whole stage
    static constexpr uint32_t A_CODES = KS * A_KB, B_CODES = KS * B_KB, A_SC = KS * TILE * SW, B_SC = (TCS ? 1 : KS) * BNMAX * SW;
    static constexpr uint32_t O_B = A_CODES, O_SA = O_B + B_CODES, O_SB = O_SA + A_SC, O_UA = O_SB + B_SC, O_MB = O_UA + A_SC;
    static constexpr uint32_t STAGE = A_CODES + B_CODES + (MINS ? 2 : 1) * (A_SC + B_SC);
    static constexpr uint32_t PATCH = ((KIND == 0 && HALF) || TCS) ? 2048 : 0;    // zeros: the half of K an instruction reads but the operand does not have
    static constexpr int S_FIT = (int)((MM_SMEM_MAX - MM_HEADER - PATCH) / STAGE);
    static constexpr int S = S_FIT > 6 ? 6 : S_FIT;
    static constexpr uint32_t O_PATCH = MM_HEADER + S * STAGE;
    static constexpr uint32_t SMEM = O_PATCH + PATCH;
    static_assert(S >= 2, "the ring needs two stages");
    static_assert(2 * S + 2 * NT + 2 <= 64, "barriers fit the header");
    static_assert(!TCS || GROUP % KS == 0, "a stage lies inside one group of k-blocks");
};

struct PackedA {             // tile-major: [tile][k-block][16 row groups][KC][8 rows][16 bytes], scales [tile][k-block][128]
    const uint8_t *codes;
    const float *scales;     // f32 each, or 16-byte rows for the tensor cores (TCS); the few-rows kernel's A is `codes` alone (LAY_FEW)
    const float *extra;      // scale * sum of the block's codes (the factor of B's min); null unless B is Q4_K
};
struct PackedB {             // LAY_KBLOCK (codes, scales, extra) or LAY_GROUPED (codes only: the slabs hold the scale rows)
    const uint8_t *codes;
    const float *scales;
    const float *extra;      // Q4_K: dmin * m
    int rows_pad;
    int groups;              // LAY_GROUPED: groups of eight k-blocks a tile
};

// (tuning builds compile the sharded product's exchange out with -DMM_PUBLISH=0)
#ifndef MM_PUBLISH
#define MM_PUBLISH 1
#endif
#define MM_WORLD(p) (MM_PUBLISH ? (p).pub.world : 0)

struct MatmulArgs {
    PackedA a;
    PackedB b;
    float *c;
    int32_t *sums;
    uint8_t *cb;             // optional: C again as blocks of fmt_c (the reference's `Back`), encoded by the block that wrote the lanes
    int fmt_c;
    int *status;
    int m, n, kb;            // kb = k-blocks of the product
    int unit;                // columns a unit: 16, or 32 when cb is set (a block of C lies inside one piece)
    int units;               // ceil(n / unit)
    int mtiles;
    int probe;               // tuning build only (see MM_PROBE)
    long long *trace;        // tuning build only: clock stamps of block 0
    const uint8_t *b_raw;    // few rows of A on raw weights: B's rows as the caller holds them (k in whole groups of eight blocks, 16-byte aligned)
    int ldc;                 // values from a row of C to the next (n, unless C is a column block of a wider matrix: the sharded product)
    GemvPublish pub;         // the sharded product's exchange: where C's column block goes besides c (world 0: nowhere), and the flags
    int batch;               // products: operand sets a_stride / b_stride bytes apart in their packed form (0: the same for all), results c_stride values apart
    size_t a_stride, b_stride, c_stride;
};

// ---------------------------------------------------------------------------------- step 1: operands for the tensor cores

// Layouts of a packed operand.
//  LAY_TILE: A of the 128-row-tile kernel.  Codes [tile][k-block][16 row groups][kc][8 rows][16 bytes]; scales
//            [tile][k-block][128], f32 each or (tcs) a 16-byte row of eight f16 with the scale at position k-block % 8.
//  LAY_KBLOCK: B whose scale products are taken on the CUDA cores (Q4_K, Q6_K).  Codes [k-block][rows_pad / 8 row
//            groups][kc][8][16]; f32 planes [k-block][rows_pad].
//  LAY_GROUPED: B with plain f16 block scales (Q8_0, Q4_0).  One slab a 128-row tile and group of eight k-blocks: the
//            eight k-blocks' codes (each [16 row groups][kc][8][16]) and then 128 scale rows of eight f16, the scale of
//            k-block 8 g + j at position j (zero past the last k-block).  A row of B and a row of A whose only non-zero
//            is at position j multiply to exactly sB * sA of that k-block.
//  LAY_FEW: A of the few-rows kernel, bn rows.  One slab a group of eight k-blocks: the eight k-blocks' codes (each
//            [bn / 8 row groups][kc][8][16]), then 8 x bn scale rows: row j * bn + r has row r's scale of k-block
//            8 g + j at position j and zeros elsewhere, so that one instruction over the rows of several k-blocks
//            leaves every k-block's scale products side by side.
enum { LAY_TILE = 0, LAY_KBLOCK = 1, LAY_GROUPED = 2, LAY_FEW = 3 };

struct PackTarget {
    uint8_t *codes;
    float *scales;
    float *extra;
    int layout;
    int tcs;                 // LAY_TILE: scales as 16-byte rows for the tensor cores' scale product instead of f32
    int rows_pad;
    int kbs;                 // k-blocks a row in the packed operand
    int kc;                  // k-chunks a k-block
    int kind;
    int bn;                  // LAY_FEW: rows kept
};

__host__ __device__ inline size_t grouped_slab(int kc) { return (size_t)GROUP * TILE * kc * 16 + TILE * 16; }
__host__ __device__ inline size_t few_slab(int bn, int kc) { return (size_t)GROUP * bn * kc * 16 + (size_t)GROUP * bn * 16; }
// the few-rows form of A against weights whose scale products stay on the CUDA cores (Q4_K): codes, then f32 scales
// [8][bn], then the scaled sums of the codes [8][bn]
__host__ __device__ inline size_t fewq_slab(int bn, int kc) { return (size_t)GROUP * bn * kc * 16 + 2 * (size_t)GROUP * bn * 4; }
__host__ __device__ inline int groups_of(int kbs) { return (kbs + GROUP - 1) / GROUP; }

// Byte offset of k-chunk `kci` (counted along the whole row) of row r.
__device__ __forceinline__ size_t chunk_offset(const PackTarget &t, int r, int kci)
{
    const int kblock = kci / t.kc, kc = kci - kblock * t.kc;
    if (t.layout == LAY_GROUPED) {
        const size_t slab = ((size_t)(r / TILE) * groups_of(t.kbs) + kblock / GROUP) * grouped_slab(t.kc);
        return slab + (size_t)(kblock % GROUP) * (TILE * t.kc * 16) + (size_t)(((r % TILE) / 8) * t.kc + kc) * 128 + (size_t)(r & 7) * 16;
    }
    if (t.layout == LAY_FEW) {
        const size_t slab = (size_t)(kblock / GROUP) * (t.tcs ? few_slab(t.bn, t.kc) : fewq_slab(t.bn, t.kc));
        return slab + (size_t)(kblock % GROUP) * (t.bn * t.kc * 16) + (size_t)((r / 8) * t.kc + kc) * 128 + (size_t)(r & 7) * 16;
    }
    size_t group;
    if (t.layout == LAY_TILE) group = ((size_t)(r / TILE) * t.kbs + kblock) * (TILE / 8) + (r % TILE) / 8;
    else group = (size_t)kblock * (t.rows_pad / 8) + r / 8;
    return (group * t.kc + kc) * 128 + (size_t)(r & 7) * 16;
}
// Index of (row, k-block) in a plane of LAY_TILE / LAY_KBLOCK.
__device__ __forceinline__ size_t scale_offset(const PackTarget &t, int r, int kblock)
{
    if (t.layout == LAY_TILE) return ((size_t)(r / TILE) * t.kbs + kblock) * TILE + r % TILE;
    return (size_t)kblock * t.rows_pad + r;
}
// A 16-byte row of eight f16: `bits` at position j, zeros elsewhere.
__device__ __forceinline__ uint4 scale_row(uint32_t bits, int j)
{
    const uint32_t w = (bits & 0xFFFFu) << (16 * (j & 1));
    return make_uint4(j >> 1 == 0 ? w : 0u, j >> 1 == 1 ? w : 0u, j >> 1 == 2 ? w : 0u, j >> 1 == 3 ? w : 0u);
}
// The scale of (row, k-block): d as an f32, or its f16 bits where the layout feeds the tensor cores' scale product.
__device__ __forceinline__ void store_scale(const PackTarget &t, int r, int kblock, float d, uint32_t d_bits)
{
    const int j = kblock % GROUP;
    if (t.layout == LAY_GROUPED) {
        const size_t slab = ((size_t)(r / TILE) * groups_of(t.kbs) + kblock / GROUP) * grouped_slab(t.kc);
        uint16_t *row = (uint16_t *)(t.codes + slab + (size_t)GROUP * TILE * t.kc * 16 + (size_t)(r % TILE) * 16);
        row[j] = (uint16_t)d_bits;
        if (kblock == t.kbs - 1) for (int z = j + 1; z < GROUP; z++) row[z] = 0;      // positions past the last k-block multiply as zeros
    } else if (t.layout == LAY_FEW) {
        if (r >= t.bn) return;
        if (!t.tcs) {
            const size_t slab = (size_t)(kblock / GROUP) * fewq_slab(t.bn, t.kc);
            *(float *)(t.codes + slab + (size_t)GROUP * t.bn * t.kc * 16 + (size_t)(j * t.bn + r) * 4) = d;
            return;
        }
        const size_t slab = (size_t)(kblock / GROUP) * few_slab(t.bn, t.kc);
        *(uint4 *)(t.codes + slab + (size_t)GROUP * t.bn * t.kc * 16 + (size_t)(j * t.bn + r) * 16) = scale_row(d_bits, j);
    } else if (t.tcs) ((uint4 *)t.scales)[scale_offset(t, r, kblock)] = scale_row(d_bits, j);
    else t.scales[scale_offset(t, r, kblock)] = d;
}

// The extra value of (row, k-block): scale * (sum of the block's codes), the factor of the other operand's min.
__device__ __forceinline__ void store_extra(const PackTarget &t, int r, int kblock, float value)
{
    if (t.layout == LAY_FEW) {
        if (r >= t.bn) return;
        const size_t slab = (size_t)(kblock / GROUP) * fewq_slab(t.bn, t.kc);
        *(float *)(t.codes + slab + (size_t)GROUP * t.bn * t.kc * 16 + (size_t)GROUP * t.bn * 4 + (size_t)((kblock % GROUP) * t.bn + r) * 4) = value;
    } else t.extra[scale_offset(t, r, kblock)] = value;
}

// 16 int8 values (four words) as one k-chunk (int8) or two (f16), starting at k-chunk kci0 of row r.
__device__ __forceinline__ void store_codes16(const PackTarget &t, int r, int kci0, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3)
{
    if (t.layout == LAY_FEW && r >= t.bn) return;
    if (t.kind == 0) {
        *(uint4 *)(t.codes + chunk_offset(t, r, kci0)) = make_uint4(w0, w1, w2, w3);
        return;
    }
    const uint32_t w[4] = { w0, w1, w2, w3 };
#pragma unroll
    for (int h = 0; h < 2; h++) {
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t word = w[2 * h + (i >> 1)] >> (16 * (i & 1));
            const __half2 v = __halves2half2(__int2half_rn((int)(int8_t)(word & 255)), __int2half_rn((int)(int8_t)((word >> 8) & 255)));
            o[i] = *(const uint32_t *)&v;
        }
        *(uint4 *)(t.codes + chunk_offset(t, r, kci0 + h)) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// Q8_0 / Q4_0 rows.  A block of 256 threads re-lays 32 rows x 8 blocks: the rows' bytes (8 consecutive blocks of a row
// are contiguous in the raw operand, 2-byte aligned) go to shared memory with coalesced loads (16 bytes wide when the
// rows lie on 16-byte boundaries, else 2); then a thread a block assembles its 32 int8 values and its scale.
// Rows past `rows` (the padding up to rows_pad) are written as zeros.
// SPLIT (against Q6_K rows, whose scales change every 16 values): a block becomes two k-blocks of 16 values, same scale.
// PACK_ROWS rows a block: 128 for a large operand (more loads in flight a thread: the weights' packing is a quarter to a
// third faster than with 32), 32 for a small one (the activations: more blocks than multiprocessors first)
template <int FMT, bool SPLIT, int PACK_ROWS>
__global__ void __launch_bounds__(256) pack_rows_kernel(const uint8_t *raw, int rows, int kb32, PackTarget t, int want_usums)
{
    // halfwords a row segment; the pitch is an odd number of 32-bit words, so the 32 rows start in 32 different banks
    constexpr int BB = block_bytes(FMT), HALVES = 8 * BB / 2, PITCH = HALVES + 2, VECS = 8 * BB / 16;
    __shared__ __align__(16) uint16_t seg[PACK_ROWS * PITCH];
    // a product launched as a programmatic dependent may start its prologue now (it waits for this grid before it reads A)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int r0 = blockIdx.x * PACK_ROWS, b0 = blockIdx.y * 8;
    const int nb = min(8, kb32 - b0), halves = nb * BB / 2;
    const size_t row_bytes = (size_t)kb32 * BB;
    if (nb == 8 && (((uintptr_t)raw | row_bytes) & 15) == 0) {
#pragma unroll 4
        for (int idx = threadIdx.x; idx < PACK_ROWS * VECS; idx += 256) {
            const int rr = idx / VECS, c = idx - rr * VECS;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r0 + rr < rows) v = __ldg((const uint4 *)(raw + (size_t)(r0 + rr) * row_bytes + (size_t)b0 * BB) + c);
            uint32_t *dst = (uint32_t *)(seg + rr * PITCH) + c * 4;
            dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
        }
    } else {
        for (int idx = threadIdx.x; idx < PACK_ROWS * HALVES; idx += 256) {
            const int rr = idx / HALVES, h = idx - rr * HALVES;
            uint16_t v = 0;
            if (r0 + rr < rows && h < halves) v = __ldg((const uint16_t *)(raw + ((size_t)(r0 + rr) * kb32 + b0) * BB) + h);
            seg[rr * PITCH + h] = v;
        }
    }
    __syncthreads();
    const int bl = threadIdx.x >> 5, b = b0 + bl;
    if (b >= kb32) return;
#pragma unroll
    for (int rh = 0; rh < PACK_ROWS / 32; rh++) {
    const int rl = (threadIdx.x & 31) + 32 * rh, r = r0 + rl;
    if (r >= t.rows_pad) break;
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
    const int per16 = t.kind ? 2 : 1;                   // k-chunks 16 values take
    store_codes16(t, r, 2 * b * per16, w[0], w[1], w[2], w[3]);
    store_codes16(t, r, (2 * b + 1) * per16, w[4], w[5], w[6], w[7]);
    if (SPLIT) {
        store_scale(t, r, 2 * b, d, p[0]);
        store_scale(t, r, 2 * b + 1, d, p[0]);
        continue;
    }
    store_scale(t, r, b, d, p[0]);
    if (want_usums) {       // against a format with mins: scale * (sum of the codes), the factor of the other operand's min
        int sum = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) asm("dp4a.s32.s32 %0, %1, %2, %0;" : "+r"(sum) : "r"(w[i]), "r"(0x01010101));
        store_extra(t, r, b, __fmul_rn(d, (float)sum));
    }
    }
}

// Q4_K rows as an operand: a block of 256 threads re-lays 32 rows x one super-block (144 bytes, src/Blocks.cs:79-96) into
// eight k-blocks.  Sub-block j (32 values): codes q = the low (j even) or high nibbles of qs[32 (j/2) ..], kept as
// 0..15; scale d * sc and min dmin * m, each rounded to f32 as DecodeQ4_K rounds them, with sc and m unpacked as ScaleMin
// does (src/Blocks.cs:73-77).  value = (d*sc)*q - dmin*m, so a k-block contributes sA*(d*sc)*sum(qA*q) - (dmin*m)*sA*sum(qA).
template <int PR>       // rows a block: 128 for a whole weight matrix (more loads in flight a thread), 32 for a small one
__global__ void __launch_bounds__(256) pack_q4_k_kernel(const uint8_t *raw, int rows, int kb32, PackTarget t)
{
    constexpr int PITCH = 37;                           // words a row of 144 bytes (36 words): odd, so rows start in different banks
    __shared__ uint32_t seg[PR * PITCH];
    const int r0 = blockIdx.x * PR, sb = blockIdx.y;
    const size_t row_bytes = (size_t)(kb32 / 8) * 144;
    if ((((uintptr_t)raw | row_bytes) & 15) == 0) {
#pragma unroll 4
        for (int idx = threadIdx.x; idx < PR * 9; idx += 256) {
            const int rr = idx / 9, c = idx - rr * 9;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r0 + rr < rows) v = __ldg((const uint4 *)(raw + (size_t)(r0 + rr) * row_bytes + (size_t)sb * 144) + c);
            uint32_t *dst = seg + rr * PITCH + c * 4;
            dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
        }
    } else {
        for (int idx = threadIdx.x; idx < PR * 72; idx += 256) {
            const int rr = idx / 72, h = idx - rr * 72;
            uint16_t v = 0;
            if (r0 + rr < rows) v = __ldg((const uint16_t *)(raw + (size_t)(r0 + rr) * row_bytes + (size_t)sb * 144) + h);
            ((uint16_t *)(seg + rr * PITCH))[h] = v;
        }
    }
    __syncthreads();
#pragma unroll
    for (int rh = 0; rh < PR / 32; rh++) {
    const int rl = (threadIdx.x & 31) + 32 * rh, j = threadIdx.x >> 5, r = r0 + rl, b = sb * 8 + j;
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
    const int per16 = t.kind ? 2 : 1;
    store_codes16(t, r, 2 * b * per16, w[0], w[1], w[2], w[3]);
    store_codes16(t, r, (2 * b + 1) * per16, w[4], w[5], w[6], w[7]);
    t.scales[scale_offset(t, r, b)] = __fmul_rn(d, (float)sc);       // rows past the end read as zeros throughout
    t.extra[scale_offset(t, r, b)] = __fmul_rn(dmin, (float)m);
    }
}

// Q6_K rows as an operand: a block of 256 threads re-lays 32 rows x one super-block (210 bytes, src/Blocks.cs:157-171)
// into sixteen k-blocks of 16 values.  Sub-block s = 8 half + 2 g + (l / 16) holds the values
// 128 half + 32 g + l: code = nibble of ql[64 half + 32 (g & 1) + l] (high nibble for g >= 2) | two bits of
// qh[32 half + l] at 2 g, minus 32; scale d * sc[s] rounded to f32, as DecodeQ6_K's d * sc * q evaluates left to right.
__global__ void __launch_bounds__(256) pack_q6_k_kernel(const uint8_t *raw, int rows, int kb16, PackTarget t)
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
    const int per16 = t.kind ? 2 : 1;
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
        const int kblock = sb * 16 + s;
        store_codes16(t, r, kblock * per16, w[0], w[1], w[2], w[3]);
        t.scales[scale_offset(t, r, kblock)] = __fmul_rn(d, (float)(int8_t)row[192 + s]);
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
// (128 bytes); LBO = bytes between the 16-byte k-chunks of a row, SBO = bytes between 8-row groups.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo)
{
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (uint64_t)((lbo >> 4) & 0x3FFFu) << 16 | (uint64_t)((sbo >> 4) & 0x3FFFu) << 32 | (uint64_t)1 << 46;
}

// Instruction descriptors, both operands K-major, dense, M x N.  kind::i8: D s32, A and B signed 8-bit;
// kind::f16: D f32, A and B f16.
__host__ __device__ constexpr uint32_t idesc_of(int kind, int m, int n)
{
    return (kind == 0 ? (2u << 4) | (1u << 7) | (1u << 10) : (1u << 4)) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// D[tmem] (+)= A.B^T over 32 bytes of K (32 int8 or 16 f16 values a row).
template <int KIND>
__device__ __forceinline__ void mma_issue(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    if (KIND == 0) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// The mbarrier gets one arrival when every tcgen05.mma this thread issued so far has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 8 columns of 32-bit accumulators: thread l of the warp gets row (lane base + l), columns c .. c+7.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                   "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32])
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
// Nothing is emitted: the registers pass through the statement, so that what uses them stays below the wait before it.
// The sharded product's exchange.  Every block stores its part of C into the other GPUs' copies beside its own (plain
// stores through peer-mapped pointers); at its end, after the barrier that makes the block's stores thread 0's to order,
// thread 0 fences and counts the block in, and the block that counts last fences at system scope and raises this rank's
// flag in every rank's flag array.  When a bounded wait gave up in any block the flags are not raised: they then never
// show this epoch and the readers' own bounded waits report it.
__device__ __forceinline__ bool peers_aligned(const GemvPublish &pub)
{
    uintptr_t bits = 0;
    for (int w = 0; w < pub.world; w++) bits |= (uintptr_t)pub.out[w];
    return (bits & 15) == 0;
}
__device__ __noinline__ void publish_count(const GemvPublish &pub, bool ok)
{
    // (a block that gave up counts all the same, with a mark in the upper half of the word, so that the counter returns to
    // zero for the next call)
    __threadfence();
    const unsigned int before = atomicAdd(pub.counter, ok ? 1u : 0x10001u);
    if ((before & 0xffffu) != gridDim.x - 1) return;
    *pub.counter = 0u;
    if (!ok || (before >> 16)) return;
    __threadfence_system();
    // epoch 0: the call's number is counted on the device (a captured graph replays the same arguments)
    const unsigned int epoch = pub.epoch ? pub.epoch : atomicAdd(pub.epoch_counter, 1u) + 1u;
    for (int w = 0; w < pub.world; w++) {
        unsigned int *f = pub.flag[w];
        if (f) asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
    }
}

__device__ __forceinline__ void pin16(uint32_t *v)
{
    asm volatile("" : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]),
                      "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]) :: "memory");
}
// The reads issued so far have landed, and nothing that uses v is scheduled above this point (the registers pass through
// the statement, so their uses depend on it).
__device__ __forceinline__ void tmem_ld_landed16(uint32_t (&v)[16])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]),
                   "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
                 :
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_landed16x2(uint32_t (&v)[16], uint32_t (&x)[16])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]),
                   "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
                   "+r"(x[0]), "+r"(x[1]), "+r"(x[2]), "+r"(x[3]), "+r"(x[4]), "+r"(x[5]), "+r"(x[6]), "+r"(x[7]), "+r"(x[8]), "+r"(x[9]),
                   "+r"(x[10]), "+r"(x[11]), "+r"(x[12]), "+r"(x[13]), "+r"(x[14]), "+r"(x[15])
                 :
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_landed32(uint32_t (&v)[32])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]),
                   "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]), "+r"(v[16]), "+r"(v[17]), "+r"(v[18]),
                   "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]), "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]),
                   "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
                 :
                 : "memory");
}

// ---------------------------------------------------------------------------------- step 2: the product

// Barrier waits of this kernel.  WAIT_MODE 0: mbarrier.try_wait with a long suspend hint; 1: try_wait with the default
// time limit; 2: test_wait in a plain spin.  All give up like mbar_wait (bounded, abort word, status bit).
// With the scale products on the tensor cores: 1 = the 128 columns of a piece are two sets of 64, each with its own issuing
// thread, its own two accumulators (64 of sums + 64 of scale products) and its own eight epilogue warps, so that the two
// halves of the block run out of step with one another instead of all sixteen warps waiting and computing together
// (measured: 1 to 3.5 % faster, M 512 to 2048 at N 11008, K 4096).
#ifndef MM_SPLIT2
#define MM_SPLIT2 1
#endif
#ifndef MM_WAIT_MODE
#define MM_WAIT_MODE 1
#endif
__device__ __forceinline__ bool mm_poll(uint32_t bar, uint32_t parity, int mode)
{
    uint32_t done;
    if (mode == 0) return mbar_try_wait(bar, parity);
    if (mode == 1)
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ bool mm_wait(uint32_t bar, uint32_t parity, volatile int *abort, int *status, int mode)
{
    if (mm_poll(bar, parity, mode & 3)) return true;
    const long long start = clock64();
    for (int spins = 0;; spins++) {
        if (mm_poll(bar, parity, mode & 3)) return true;
        if (mode & 16) __nanosleep(40);
        if ((spins & 63) != 63) continue;       // the give-up conditions are looked at every 64th poll
        if (*abort) return false;
        if (clock64() - start > WAIT_CYCLES) {
            *abort = 1;
            atomicOr(status, STATUS_MATMUL_WAIT);
            return false;
        }
    }
}
// Every lane polls; all lanes see the same barrier, so they leave together except in the give-up case, where the
// abort word makes the stragglers follow within a few polls.
__device__ __forceinline__ bool mm_wait_lanes(uint32_t bar, uint32_t parity, volatile int *abort, int *status, int mode)
{
    if (mode & 8) {             // lane 0 polls, the others get its answer
        int ok = 1;
        if ((threadIdx.x & 31) == 0) ok = mm_wait(bar, parity, abort, status, mode) ? 1 : 0;
        return __shfl_sync(0xffffffffu, ok, 0) != 0;
    }
    const bool ok = mm_wait(bar, parity, abort, status, mode);
    return __all_sync(0xffffffffu, ok);
}

// Packed f32 pairs (sm_100): one instruction rounds two independent products / fused multiply-adds, each exactly as
// mul.rn.f32 / fma.rn.f32 would.
__device__ __forceinline__ uint64_t pack2(float lo, float hi)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ uint64_t pack2u(uint32_t lo, uint32_t hi)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
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

// Two block sums as a pair of floats: converted (kind::i8) or as they are (kind::f16 leaves exact f32 sums).
template <int KIND>
__device__ __forceinline__ uint64_t sums2(uint32_t d0, uint32_t d1)
{
    if (KIND == 0) return pack2((float)(int32_t)d0, (float)(int32_t)d1);
    return pack2u(d0, d1);
}
template <int KIND>
__device__ __forceinline__ float sum_as_float(uint32_t d) { return KIND == 0 ? (float)(int32_t)d : __uint_as_float(d); }
template <int KIND>
__device__ __forceinline__ int32_t sum_as_int(uint32_t d) { return KIND == 0 ? (int32_t)d : __float2int_rn(__uint_as_float(d)); }

// Eight columns of one k-block into the accumulators: acc = fma(float(D), sA*sB, acc) (src/MatMulBlocks.cs:344-346).
template <int KIND>
__device__ __forceinline__ void scale_add8(const uint32_t (&v)[8], uint64_t sa2, const float *sb, uint64_t (&acc)[4])
{
    const ulonglong2 s0 = *(const ulonglong2 *)sb, s1 = *(const ulonglong2 *)(sb + 4);
    acc[0] = fma2(sums2<KIND>(v[0], v[1]), mul2(sa2, s0.x), acc[0]);
    acc[1] = fma2(sums2<KIND>(v[2], v[3]), mul2(sa2, s0.y), acc[1]);
    acc[2] = fma2(sums2<KIND>(v[4], v[5]), mul2(sa2, s1.x), acc[2]);
    acc[3] = fma2(sums2<KIND>(v[6], v[7]), mul2(sa2, s1.y), acc[3]);
}

// The min term of one k-block for eight columns: acc = fma(dmin*m, -(sA*sum(qA)), acc); `nu2` is -(sA*sum(qA)) twice.
__device__ __forceinline__ void min_add8(uint64_t nu2, const float *wb, uint64_t (&acc)[4])
{
    const ulonglong2 w0 = *(const ulonglong2 *)wb, w1 = *(const ulonglong2 *)(wb + 4);
    acc[0] = fma2(w0.x, nu2, acc[0]);
    acc[1] = fma2(w0.y, nu2, acc[1]);
    acc[2] = fma2(w1.x, nu2, acc[2]);
    acc[3] = fma2(w1.y, nu2, acc[3]);
}

// The share of block `b` of `grid`: units [lo, hi) of the batch * mtiles * units of the call, cut into pieces that stay
// inside one tile of A (`tile` counts the tiles of all the batch's products) and are at most `wmax` units wide (as even
// as the count allows).  Every role of the block walks the same pieces in the same order.
struct Pieces {
    long long at, hi;
    int units, wmax;
    __device__ Pieces(const MatmulArgs &p, int wmax_) : units(p.units), wmax(wmax_)
    {
        const long long total = (long long)p.batch * p.mtiles * p.units;
        at = total * blockIdx.x / gridDim.x;
        hi = total * (blockIdx.x + 1) / gridDim.x;
    }
    __device__ bool next(int &tile, int &u0, int &w)
    {
        if (at >= hi) return false;
        tile = (int)(at / units);
        const long long end = min(hi, (long long)(tile + 1) * units);
        const int len = (int)(end - at), np = (len + wmax - 1) / wmax;
        w = (len + np - 1) / np;
        u0 = (int)(at - (long long)tile * units);
        at += w;
        return true;
    }
};

// VAR: how a k-block's sums are scaled.  PLAIN: f32 scales from shared memory, product and fma on the CUDA cores;
// MINS: the same with Q4_K's min term; HALF: Q6_K's k-blocks of 16 values; TCS: scale products from the tensor cores.
enum { VAR_PLAIN = 0, VAR_MINS = 1, VAR_HALF = 2, VAR_TCS = 3 };

template <int KIND, int OUT, int VAR>
__global__ void __launch_bounds__(mm_threads(VAR == VAR_TCS) + (OUT == 2 ? 32 : 0), 1) matmul_kernel(const __grid_constant__ MatmulArgs p)
{
    // OUT: 0 lanes, 1 lanes and the blocks' integer sums, 2 lanes into the other GPUs' copies of C as well (the sharded product)
    constexpr bool SUMS = OUT == 1, PUB = OUT == 2;
    constexpr bool MINS = VAR == VAR_MINS, HALF = VAR == VAR_HALF, TCS = VAR == VAR_TCS;
    using G = Cfg<KIND, MINS, HALF, TCS>;
    constexpr int EW = epi_warps(TCS), MMA2_WARP = 2 + EW, PUB_WARP = MMA2_WARP + 1, EC = 128 / (EW / 4);      // epilogue warps, the second issuer's warp, columns a warp
    constexpr int S = G::S, KS = G::KS, KC = G::KC, NT = G::NT, TCOLS = G::TCOLS, THREADS = mm_threads(TCS);
    extern __shared__ __align__(1024) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = smem_u32(smem);
    constexpr bool SPLIT2 = TCS && MM_SPLIT2;
    constexpr int NTB = SPLIT2 ? 2 * NT : NT;                // accumulator barriers: a set of NT for each half when split
    const uint32_t full0 = base, empty0 = base + 8 * S, tfull0 = base + 16 * S, tempty0 = tfull0 + 8 * NTB;
    const uint32_t holder = tempty0 + 8 * NTB;
    static_assert(2 * S + 2 * NTB + 2 <= 64, "barriers fit the header");
    volatile int *abort_flag = (volatile int *)(smem + 768);
    volatile uint32_t *holder_ptr = (volatile uint32_t *)(smem + (holder - base));

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, TCS ? 2 : 2 + EW);      // the two issuers' commits, and the epilogue warps where they read the scales
        }
        for (int t = 0; t < NTB; t++) {
            mbar_init(tfull0 + 8 * t, 1);
            mbar_init(tempty0 + 8 * t, SPLIT2 ? EW / 2 : EW);
        }
        *abort_flag = 0;
        for (int i = 0; i < EW; i++) *(volatile int *)(smem + 772 + 4 * i) = 0;          // pieces each epilogue warp has stored (the sharded product)
        mbar_fence_init();
    }
    if (G::PATCH) {
        for (int i = threadIdx.x; i < (int)G::PATCH / 16; i += THREADS) *(uint4 *)(smem + G::O_PATCH + i * 16) = make_uint4(0, 0, 0, 0);
        fence_proxy_async();            // the tensor cores read the patch through the async proxy
    }
    if (warp == 1) tmem_alloc(holder, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *holder_ptr;
    uint8_t *ring = smem + MM_HEADER;
    const int wmax = BNMAX / p.unit;
#ifdef QB_MM_TUNING
    const int wmode = ((p.probe >> 4) & 3) | ((p.probe >> 7) & 1) << 3 | ((p.probe >> 8) & 1) << 4;
#else
    constexpr int wmode = MM_WAIT_MODE;
#endif

    if (warp == 0) {
        // ---- producer: a stage is KS k-blocks; A's codes, scales (and scaled sums) are one copy each a stage (tile-major),
        // B's one copy each a k-block.  Lane 0 posts the byte count, then every lane issues its own copy.
        Pieces pieces(p, wmax);
        int tile, u0, w, sc = 0;
        bool alive = true;
        long long w_empty = 0, t_begin = MM_CLOCK();
        asm volatile("griddepcontrol.wait;" ::: "memory");       // the kernel before this one packed A
        while (alive && pieces.next(tile, u0, w)) {
            const int n0 = u0 * p.unit, bn = w * p.unit, bi = tile / p.mtiles, mt = tile - bi * p.mtiles;
            const uint8_t *a_codes = p.a.codes + bi * p.a_stride, *b_codes = p.b.codes + bi * p.b_stride;
            const uint8_t *a_scales = (const uint8_t *)p.a.scales + bi * p.a_stride, *a_extra = (const uint8_t *)p.a.extra + bi * p.a_stride;
            const uint8_t *b_scales = (const uint8_t *)p.b.scales + bi * p.b_stride, *b_extra = (const uint8_t *)p.b.extra + bi * p.b_stride;
            for (int kb0 = 0; kb0 < p.kb && alive; kb0 += KS, sc++) {
                const int s = sc % S, nkb = min(KS, p.kb - kb0);
                int ok = 1;
                const long long w0 = MM_CLOCK();
                if (lane == 0 && sc >= S) ok = mm_wait(empty0 + 8 * s, (uint32_t)(sc / S - 1) & 1u, abort_flag, p.status, wmode) ? 1 : 0;
                w_empty += MM_CLOCK() - w0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { alive = false; break; }
                const uint32_t dst = smem_u32(ring + (size_t)s * G::STAGE), bar = full0 + 8 * s;
                const uint32_t a_code_bytes = (uint32_t)nkb * G::A_KB, a_sc_bytes = (uint32_t)nkb * TILE * G::SW;
                uint32_t b_code_bytes = (uint32_t)bn * KC * 16, b_sc_bytes = (uint32_t)bn * G::SW;
                if (MM_PROBE(p) & 4) b_code_bytes = 0;          // tuning: no copies of B's codes
                if (MM_PROBE(p) & 64) b_sc_bytes = 0;           // tuning: no copies of B's scales
                if (lane == 0)
                    mbar_arrive_expect_tx(bar, a_code_bytes + (MINS ? 2 : 1) * a_sc_bytes + (uint32_t)nkb * b_code_bytes +
                                                   (TCS ? 1u : (uint32_t)nkb * (MINS ? 2 : 1)) * b_sc_bytes);
                __syncwarp();
                const size_t a_at = (size_t)mt * p.kb + kb0;
                if (lane == 0) bulk_g2s(dst, a_codes + a_at * G::A_KB, a_code_bytes, bar);
                else if (lane == 1) bulk_g2s(dst + G::O_SA, a_scales + a_at * TILE * G::SW, a_sc_bytes, bar);
                else if (lane == 2) { if (MINS) bulk_g2s(dst + G::O_UA, a_extra + a_at * TILE * G::SW, a_sc_bytes, bar); }
                else if (TCS) {
                    // B's slabs (a 128-row tile and group of eight k-blocks each): a piece's rows lie in one slab, or in two
                    // when it crosses a multiple of 128 (lanes 16.. copy the second part); codes a k-block, scale rows a stage
                    const int part = lane >> 4, job = (lane & 15) - 3, kk = job >> 1, what = job & 1;
                    const int first = min(bn, TILE - n0 % TILE);                 // rows in the first slab
                    const int rows_here = part ? bn - first : first, row0 = part ? 0 : n0 % TILE, done = part ? first : 0;
                    if (job >= 0 && kk < nkb && rows_here > 0 && !(what == 0 ? b_code_bytes == 0 : b_sc_bytes == 0)) {
                        const size_t kb = (size_t)(kb0 + kk);
                        const uint8_t *slab = b_codes + ((size_t)(n0 / TILE + part) * p.b.groups + kb / GROUP) * grouped_slab(KC);
                        if (what == 0)
                            bulk_g2s(dst + G::O_B + kk * G::B_KB + done * (KC * 16), slab + (kb % GROUP) * (size_t)(TILE * KC * 16) + (size_t)(row0 / 8) * (KC * 128),
                                     (uint32_t)rows_here * KC * 16, bar);
                        else if (kk == 0)
                            bulk_g2s(dst + G::O_SB + done * 16, slab + (size_t)GROUP * TILE * KC * 16 + (size_t)row0 * 16, (uint32_t)rows_here * 16, bar);
                    }
                } else {
                    constexpr int NC = MINS ? 3 : 2;
                    const int job = lane - 3, kk = job / NC, what = job - kk * NC;
                    if (kk < nkb) {
                        const size_t kb = (size_t)(kb0 + kk);
                        if ((what == 0 && b_code_bytes == 0) || (what != 0 && b_sc_bytes == 0)) { }
                        else if (what == 0)
                            bulk_g2s(dst + G::O_B + kk * G::B_KB, b_codes + (kb * (p.b.rows_pad / 8) + n0 / 8) * (KC * 128), b_code_bytes, bar);
                        else if (what == 1)
                            bulk_g2s(dst + G::O_SB + kk * BNMAX * G::SW, b_scales + (kb * p.b.rows_pad + n0) * G::SW, b_sc_bytes, bar);
                        else
                            bulk_g2s(dst + G::O_MB + kk * BNMAX * G::SW, b_extra + (kb * p.b.rows_pad + n0) * G::SW, b_sc_bytes, bar);
                    }
                }
            }
        }
        if (lane == 0) { MM_TRACE(p, 0, w_empty); MM_TRACE(p, 1, MM_CLOCK() - t_begin); MM_TRACE(p, 2, (long long)sc); }
        if (*abort_flag && lane == 0) {          // let the copies still in flight land before the block exits
            for (int it = max(0, sc - S); it < sc; it++) {
                long long start = clock64();
                while (!mbar_try_wait(full0 + 8 * (it % S), (uint32_t)(it / S) & 1u) && clock64() - start < WAIT_CYCLES) { }
            }
        }
    } else if (warp == 1 || warp == MMA2_WARP) {
        // ---- MMA issue: two threads (an instruction costs its issuer about 60 cycles and a commit about 50, a lone thread
        // issues a dependent instruction every few cycles: one thread's own instruction stream was what paced the kernel).
        // Thread `role` takes the k-blocks of its parity, i.e. always the same accumulators of tensor memory, and commits
        // each to its barrier; both wait for every stage and both commit its release.  Descriptors are formed by adding
        // constants; the waits are a single poll when the barrier is ready.
        if (lane == 0) {
            Pieces pieces(p, wmax);
            const int role = warp == 1 ? 0 : 1;
            int tile, u0, w, sc = 0, tc0 = 0, tcs = 0;
            bool alive = true;
            long long w_full = 0, w_tempty = 0, c_mma = 0, c_commit = 0, t_begin = MM_CLOCK();
            constexpr uint32_t SBO = KC * 128;
            // the descriptor without its start address: LBO 128, SBO, version
            constexpr uint64_t DESC_HI = (uint64_t)(128u >> 4) << 16 | (uint64_t)(SBO >> 4) << 32 | (uint64_t)1 << 46;
            const uint32_t patch = base + G::O_PATCH;
            static_assert(NT % 2 == 0, "each issuer owns the accumulators of its parity");
            while (alive && pieces.next(tile, u0, w)) {
                // split: this thread's set of 64 columns, its width in this piece (none: the thread only keeps the stages moving)
                const int set_bn = !SPLIT2 ? w * p.unit : role == 0 ? min(64, w * p.unit) : w * p.unit - 64;
                const uint32_t idesc = idesc_of(KIND, TILE, set_bn > 0 ? set_bn : 16), idesc_s = idesc_of(1, TILE, set_bn > 0 ? set_bn : 16);
                for (int kb0 = 0; kb0 < p.kb && alive; kb0 += KS, sc++) {
                    const int s = sc % S, nkb = min(KS, p.kb - kb0);
                    const long long w0 = MM_CLOCK();
                    if (!mm_poll(full0 + 8 * s, (uint32_t)(sc / S) & 1u, wmode & 3) &&
                        !mm_wait(full0 + 8 * s, (uint32_t)(sc / S) & 1u, abort_flag, p.status, wmode)) { alive = false; break; }
                    w_full += MM_CLOCK() - w0;
                    tc_fence_after();
                    const uint32_t a_smem = smem_u32(ring + (size_t)s * G::STAGE);
                    const uint32_t b_rows = SPLIT2 ? (uint32_t)role * 64u : 0u;       // the set's first row of B in the stage
                    const uint64_t a_desc = DESC_HI | (uint64_t)(a_smem >> 4), b_desc = DESC_HI | (uint64_t)((a_smem + G::O_B + b_rows / 8 * SBO) >> 4);
                    // scale rows: the second half of K is the patch of zeros, LBO bytes past the start; a k-block on, A's start is
                    // one slab further and the patch that much nearer; B's rows hold the group's eight scales, the same for all
                    const uint64_t sa_desc = smem_desc(a_smem + G::O_SA, patch - (a_smem + G::O_SA), 128), sb_desc = smem_desc(a_smem + G::O_SB + b_rows * 16, patch - (a_smem + G::O_SB + b_rows * 16), 128);
                    constexpr uint64_t SA_STEP = (uint64_t)((TILE * 16) >> 4) - ((uint64_t)((TILE * 16) >> 4) << 16);
#pragma unroll
                    for (int kk = 0; kk < KS; kk++) {
                        // not split: the k-blocks of this thread's parity, accumulator tc % NT; split: every k-block of a piece
                        // its set has columns in, the set's own count and accumulators
                        const int tc = SPLIT2 ? tcs + kk : tc0 + kb0 + kk;
                        if (kk < nkb && (SPLIT2 ? set_bn > 0 : (tc & 1) == role)) {
                            const int t = tc % NT, tb = SPLIT2 ? role * NT + t : t;
                            if (tc >= NT) {
                                const uint32_t par = (uint32_t)(tc / NT - 1) & 1u;
                                const long long w1 = MM_CLOCK();
                                if (!mm_poll(tempty0 + 8 * tb, par, wmode & 3) && !mm_wait(tempty0 + 8 * tb, par, abort_flag, p.status, wmode)) { alive = false; break; }
                                w_tempty += MM_CLOCK() - w1;
                                tc_fence_after();
                            }
                            const uint32_t d = tmem + (uint32_t)(SPLIT2 ? role * 256 + t * 128 : t * TCOLS);
                            const long long c0 = MM_CLOCK();
                            if (MM_PROBE(p) & 8) { }            // tuning: no products, commits only
                            else if (KIND == 0 && HALF) {
                                // the second 16-byte k-chunk of every row of A is the patch of zeros; B's may then be anything
                                const uint32_t a_at = a_smem + kk * G::A_KB, b_at = a_smem + G::O_B + kk * G::B_KB;
                                mma_issue<KIND>(d, smem_desc(a_at, patch - a_at, 128), smem_desc(b_at, 128, 128), idesc, 0u);
                            } else {
                                mma_issue<KIND>(d, a_desc + (uint64_t)kk * (G::A_KB >> 4), b_desc + (uint64_t)kk * (G::B_KB >> 4), idesc, 0u);
                                if (KC == 4) mma_issue<KIND>(d, a_desc + (uint64_t)kk * (G::A_KB >> 4) + (256 >> 4), b_desc + (uint64_t)kk * (G::B_KB >> 4) + (256 >> 4), idesc, 1u);
                            }
                            // the scale products: A's rows [0 .., d at k-block % 8, .. 0], B's rows of eight scales, the other half of K zeros
                            if (TCS && !(MM_PROBE(p) & 8)) mma_issue<1>(d + (SPLIT2 ? 64 : BNMAX), sa_desc + (uint64_t)kk * SA_STEP, sb_desc, idesc_s, 0u);
                            const long long c1 = MM_CLOCK();
                            mma_commit(tfull0 + 8 * tb);
                            c_commit += MM_CLOCK() - c1;
                            c_mma += c1 - c0;
                        }
                    }
                    if (alive) mma_commit(empty0 + 8 * s);      // the stage is free once both issuers' products have run
                    if (SPLIT2 && set_bn > 0) tcs += nkb;
                }
                tc0 += p.kb;
            }
            if (role == 0) { MM_TRACE(p, 8, w_full); MM_TRACE(p, 9, w_tempty); MM_TRACE(p, 10, MM_CLOCK() - t_begin); MM_TRACE(p, 11, (long long)tc0); MM_TRACE(p, 12, c_mma); MM_TRACE(p, 13, c_commit); }
        }
    } else if (PUB && warp == PUB_WARP) {
        // ---- the sharded product's publisher (PUB: one more warp): it carries the finished pieces of C into the other GPUs'
        // copies.  Once the epilogue warps have all stored a piece (their words), the piece is re-read row by row from this
        // GPU's C (still in the L2) and stored to the peers, a warp a row's contiguous bytes: the peer stores cross NVLink as
        // whole lines, and where they wait for the link only this warp waits with them.
        Pieces pub_pieces(p, wmax);
        int pub_tile = 0, pub_u0 = 0, pub_w = 0, pub_count = 0, pub_off = 0;
        bool pub_has = false, pub_stored = false, pub_end = !(PUB && MM_WORLD(p) > 0);
        auto publish_some = [&](int rounds) {
            constexpr int UNR = 8;
            while (rounds-- > 0 && !pub_end) {
                if (!pub_has) {
                    if (!pub_pieces.next(pub_tile, pub_u0, pub_w)) { pub_end = true; return; }
                    if (pub_pieces.at >= pub_pieces.hi) { pub_end = true; return; }      // the block's last piece is the epilogue warps' own
                    pub_has = true; pub_stored = false; pub_off = 0;
                }
                if (!pub_stored) {
                    const int ready = lane >= EW || *(volatile int *)(smem + 772 + 4 * lane) > pub_count;
                    if (!__all_sync(0xffffffffu, ready)) return;
                    __threadfence();
                    pub_stored = true;
                }
                const int n0 = pub_u0 * p.unit, mt = pub_tile % p.mtiles;
                const int rows_here = min(TILE, p.m - mt * TILE), wcols = min(p.n, n0 + pub_w * p.unit) - n0;
                const size_t origin = (size_t)(mt * TILE) * p.ldc + n0;
                const bool vec = (p.ldc & 3) == 0 && ((uintptr_t)p.c & 15) == 0 && peers_aligned(p.pub) && (wcols & 3) == 0;
                const int upr = vec ? wcols >> 2 : wcols, total = rows_here * upr;         // units (float4 or float) a row, and in the piece
                float4 x[UNR];
                size_t off[UNR];
#pragma unroll
                for (int u = 0; u < UNR; u++) {
                    const int idx = pub_off + u * 32 + lane, rr = idx / upr, c = idx - rr * upr;
                    off[u] = origin + (size_t)rr * p.ldc + (vec ? 4 * c : c);
                    if (idx < total) {
                        if (vec) x[u] = __ldcg((const float4 *)(p.c + off[u]));
                        else x[u].x = __ldcg(p.c + off[u]);
                    }
                }
                for (int pw = 0; pw < p.pub.world; pw++) {
                    float *peer = p.pub.out[pw];
                    if (!peer) continue;
#pragma unroll
                    for (int u = 0; u < UNR; u++) {
                        if (pub_off + u * 32 + lane < total) {
                            if (vec) *(float4 *)(peer + off[u]) = x[u];
                            else peer[off[u]] = x[u].x;
                        }
                    }
                }
                pub_off += UNR * 32;
                if (pub_off >= total) { pub_has = false; pub_count++; }
            }
        };
        const long long start = clock64();
        while (!pub_end) {
            publish_some(1 << 20);
            if (pub_end) break;
            int stop = *abort_flag != 0;
            if (!stop && clock64() - start > 4 * WAIT_CYCLES) {           // (the whole kernel's time, not one handshake's)
                *abort_flag = 1;
                atomicOr(p.status, STATUS_MATMUL_WAIT);
                stop = 1;
            }
            if (__any_sync(0xffffffffu, stop)) break;
            __nanosleep(500);
        }
    } else {
        // ---- epilogue: warp (q, g) owns rows 32 q .. 32 q + 31 of the tile (the tensor-memory lanes a warp may read) and
        // columns 32 g .. 32 g + 31 of the piece (none when the piece is narrower); the four warps of a q share a scheduler.
        // A k-block costs a warp one poll of its barrier, one or two wide tensor-memory reads, one wait for them, and
        // the arithmetic: the instruction count of this loop is what bounds the kernel.
        const int q = warp & 3, g = (warp - 2) >> 2;
        // split: the warp's set of 64 columns (its half of tensor memory, its barriers) and its 32 columns inside it
        const int set = SPLIT2 ? g * EC / 64 : 0;
        constexpr int SLOT = SPLIT2 ? 128 : TCOLS, S_OFF = SPLIT2 ? 64 : BNMAX;
        const uint32_t tlane = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(SPLIT2 ? set * 256 + (g * EC) % 64 : g * EC);
        const uint32_t tfull_w = tfull0 + 8 * (set * NT), tempty_w = tempty0 + 8 * (set * NT);
        Pieces pieces(p, wmax);
        int tile, u0, w, sc = 0, tc = 0, pieces_done = 0;
        bool alive = true;
        long long w_tfull = 0, t_store = 0, t_begin = MM_CLOCK();
        while (alive && pieces.next(tile, u0, w)) {
            const int n0 = u0 * p.unit, bi = tile / p.mtiles, mt = tile - bi * p.mtiles;
            const bool active = g * EC < w * p.unit;                    // this warp has columns in the piece
            const int row = mt * TILE + q * 32 + lane;
            float *c_out = p.c + bi * p.c_stride;
            int32_t *sums_out = SUMS ? p.sums + (size_t)bi * p.m * p.n * p.kb : nullptr;
            // 32 f32 accumulators: as 16 pairs for the packed instructions of the CUDA-core scale path, as 32 scalars for TCS
            uint64_t acc[TCS ? 1 : 16];
            float accf[TCS ? EC : 1];
#pragma unroll
            for (int j = 0; j < (TCS ? 1 : 16); j++) acc[j] = 0ull;
#pragma unroll
            for (int j = 0; j < (TCS ? EC : 1); j++) accf[j] = 0.f;
            int kk = 0;
            // split: a piece the warp's set has no columns in goes by without a wait
            const bool set_active = !SPLIT2 || set * 64 < w * p.unit;
            for (int i = 0; i < p.kb && alive && set_active; i++, tc++) {
                const int t = tc % NT, s = sc % S;
                {
                    const uint32_t bar = tfull_w + 8 * t, par = (uint32_t)(tc / NT) & 1u;
                    const long long w0 = MM_CLOCK();
                    if (!((wmode & 8) ? false : mm_poll(bar, par, wmode & 3)) && !mm_wait_lanes(bar, par, abort_flag, p.status, wmode)) { alive = false; break; }
                    w_tfull += MM_CLOCK() - w0;
                }
                tc_fence_after();
                const uint32_t at = tlane + (uint32_t)(t * SLOT);
                if (TCS) {
                    // chunks of 16 columns, HG of them a wait: sums and scale products side by side in registers
                    constexpr int HG = EC / 32;
#pragma unroll
                    for (int h = 0; h < EC / 16; h += HG) {
                        uint32_t v[HG][16], x[HG][16];
#pragma unroll
                        for (int hh = 0; hh < HG; hh++) {
                            if (active && !(MM_PROBE(p) & 2)) {
                                tmem_ld16(at + 16 * (h + hh), v[hh]);
                                tmem_ld16(at + S_OFF + 16 * (h + hh), x[hh]);
                            }
                        }
                        tmem_ld_wait();
#pragma unroll
                        for (int hh = 0; hh < HG; hh++) { pin16(v[hh]); pin16(x[hh]); }
                        if (h + HG == EC / 16) {
                            tc_fence_before();
                            if (lane == 0) mbar_arrive(tempty_w + 8 * t);        // the accumulator has been read (warp-wide reads)
                        }
#pragma unroll
                        for (int hh = 0; hh < HG; hh++) {
                            if (active && !(MM_PROBE(p) & 1)) {
                                // scalar fma on the registers the reads filled: forming f32x2 pairs would cost a move or two a pair
#pragma unroll
                                for (int c = 0; c < 16; c++)
                                    accf[16 * (h + hh) + c] = __fmaf_rn(sum_as_float<KIND>(v[hh][c]), __uint_as_float(x[hh][c]), accf[16 * (h + hh) + c]);
                            }
                            if (SUMS && active && row < p.m) {
#pragma unroll
                                for (int c = 0; c < 16; c++) {
                                    const int cc = g * EC + 16 * (h + hh) + c, col = n0 + cc;
                                    if (col < p.n && cc < w * p.unit) sums_out[((size_t)row * p.n + col) * p.kb + i] = sum_as_int<KIND>(v[hh][c]);
                                }
                            }
                        }
                    }
                } else {
                    uint32_t v[32];
                    if (active && !(MM_PROBE(p) & 2)) tmem_ld32(at, v);
                    // the stage's scales (complete long since: the product that filled the accumulator read the same stage)
                    if (kk == 0 && !mm_poll(full0 + 8 * s, (uint32_t)(sc / S) & 1u, wmode & 3) &&
                        !mm_wait_lanes(full0 + 8 * s, (uint32_t)(sc / S) & 1u, abort_flag, p.status, wmode)) { alive = false; }
                    const uint8_t *stage = ring + (size_t)s * G::STAGE;
                    const float sa = ((const float *)(stage + G::O_SA))[kk * TILE + q * 32 + lane];
                    const uint64_t sa2 = pack2(sa, sa);
                    uint64_t nu2 = 0ull;
                    if (MINS) {
                        const float nu = -((const float *)(stage + G::O_UA))[kk * TILE + q * 32 + lane];
                        nu2 = pack2(nu, nu);
                    }
                    const float *sb = (const float *)(stage + G::O_SB) + kk * BNMAX + g * 32;
                    tmem_ld_landed32(v);
                    tc_fence_before();
                    if (lane == 0) mbar_arrive(tempty0 + 8 * t);         // the accumulator has been read (warp-wide reads)
                    if (!alive) break;
                    if (active && !(MM_PROBE(p) & 1)) {
#pragma unroll
                        for (int c4 = 0; c4 < 8; c4++) {
                            const ulonglong2 sc2 = *(const ulonglong2 *)(sb + 4 * c4);
                            acc[2 * c4] = fma2(sums2<KIND>(v[4 * c4], v[4 * c4 + 1]), mul2(sa2, sc2.x), acc[2 * c4]);
                            acc[2 * c4 + 1] = fma2(sums2<KIND>(v[4 * c4 + 2], v[4 * c4 + 3]), mul2(sa2, sc2.y), acc[2 * c4 + 1]);
                        }
                        if (MINS) {
                            const float *wb = sb + (G::O_MB - G::O_SB) / 4;
#pragma unroll
                            for (int c4 = 0; c4 < 8; c4++) {
                                const ulonglong2 m2 = *(const ulonglong2 *)(wb + 4 * c4);
                                acc[2 * c4] = fma2(m2.x, nu2, acc[2 * c4]);
                                acc[2 * c4 + 1] = fma2(m2.y, nu2, acc[2 * c4 + 1]);
                            }
                        }
                    }
                    if (SUMS && active && row < p.m) {
#pragma unroll
                        for (int c = 0; c < 32; c++) {
                            const int col = n0 + g * 32 + c;
                            if (col < p.n) sums_out[((size_t)row * p.n + col) * p.kb + i] = sum_as_int<KIND>(v[c]);
                        }
                    }
                }
                if (++kk == KS || i + 1 == p.kb) {
                    if (!TCS) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(empty0 + 8 * s);      // this warp has read the stage's scales
                    }
                    kk = 0;
                    sc++;
                }
            }
            tmem_ld_wait();
            const long long s0 = MM_CLOCK();
            if (alive && active && row < p.m) {
                const bool vec = (p.ldc & 3) == 0 && ((uintptr_t)c_out & 15) == 0;
                const int col0 = n0 + g * EC, col_end = min(p.n, n0 + w * p.unit);        // (a warp of 64 columns may reach past the piece)
                const size_t at = (size_t)row * p.ldc + col0;
                float *out = c_out + at;
#pragma unroll
                for (int c4 = 0; c4 < EC / 4; c4++) {
                    float f[4];
                    if (TCS) {
#pragma unroll
                        for (int c = 0; c < 4; c++) f[c] = accf[(TCS ? 4 * c4 : 0) + (TCS ? c : 0)];
                    } else {
                        unpack2(acc[TCS ? 0 : (2 * c4) % 16], f[0], f[1]);
                        unpack2(acc[TCS ? 0 : (2 * c4 + 1) % 16], f[2], f[3]);
                    }
                    if (vec && col0 + 4 * c4 + 4 <= col_end) *(float4 *)(out + 4 * c4) = make_float4(f[0], f[1], f[2], f[3]);
                    else {
#pragma unroll
                        for (int c = 0; c < 4; c++) if (col0 + 4 * c4 + c < col_end) out[4 * c4 + c] = f[c];
                    }
                }
            }
            t_store += MM_CLOCK() - s0;
            if (PUB && MM_WORLD(p) > 0) {
                // the sharded product: this warp's lanes of the piece are in this GPU's C; it says so in its own word (the
                // pieces it has finished), which the publisher warp reads: a warp without columns in a narrow piece may be a
                // piece ahead of the others, so the words are kept apart
                if (pieces.at < pieces.hi) {
                    __syncwarp();
                    if (lane == 0) {
                        __threadfence();
                        *(volatile int *)(smem + 772 + 4 * (warp - 2)) = ++pieces_done;
                    }
                } else {
                    // the block's last piece: no arithmetic is left to hide its transfer behind, so all the epilogue warps carry
                    // it, the same way (once every warp has stored its lanes: the barrier, which also tells every thread
                    // whether all of them are still going)
                    if (!named_bar_and(2, EW * 32, alive && !*abort_flag)) { alive = false; break; }
                    constexpr int T = EW * 32, UNR = 2;
                    const int tid = threadIdx.x - 64, rows_here = min(TILE, p.m - mt * TILE), wcols = min(p.n, n0 + w * p.unit) - n0;
                    const size_t origin = (size_t)(mt * TILE) * p.ldc + n0;
                    const bool vec4 = (p.ldc & 3) == 0 && ((uintptr_t)p.c & 15) == 0 && peers_aligned(p.pub) && (wcols & 3) == 0;
                    const int upr = vec4 ? wcols >> 2 : wcols, total = rows_here * upr;
                    for (int i0 = tid; i0 < total; i0 += UNR * T) {
                        float4 x[UNR];
                        size_t off[UNR];
#pragma unroll
                        for (int u = 0; u < UNR; u++) {
                            const int idx = i0 + u * T, rr = idx / upr, c = idx - rr * upr;
                            off[u] = origin + (size_t)rr * p.ldc + (vec4 ? 4 * c : c);
                            if (idx < total) {
                                if (vec4) x[u] = __ldcg((const float4 *)(p.c + off[u]));
                                else x[u].x = __ldcg(p.c + off[u]);
                            }
                        }
                        for (int pw = 0; pw < p.pub.world; pw++) {
                            float *peer = p.pub.out[pw];
                            if (!peer) continue;
#pragma unroll
                            for (int u = 0; u < UNR; u++) {
                                if (i0 + u * T < total) {
                                    if (vec4) *(float4 *)(peer + off[u]) = x[u];
                                    else peer[off[u]] = x[u].x;
                                }
                            }
                        }
                    }
                }
            }
            if (p.cb) {
                // `Back` for the piece (src/MatMulBlocks.cs:421 -> Ptx.LanesToBlock): once every epilogue warp has stored its
                // lanes, the epilogue threads encode the piece's blocks of 32 consecutive values (n % 32 == 0, unit 32: a block
                // lies in one row of one piece).  All warps come here whether or not a wait gave up; the barrier also tells every
                // thread whether all of them are still going, so that they leave together or not at all.
                if (!named_bar_and(2, EW * 32, alive && !*abort_flag)) { alive = false; break; }
                const int bw = w * p.unit / 32, tid = threadIdx.x - 64;
                const int rows_here = min(TILE, p.m - mt * TILE);
                for (int idx = tid; idx < rows_here * bw; idx += EW * 32) {
                    const int rr = idx / bw, bc = idx - rr * bw;
                    const size_t first = bi * p.c_stride + (size_t)(mt * TILE + rr) * p.n + n0 + bc * 32;      // c_stride is whole blocks (ldc = n with `Back`)
                    float f[32];
#pragma unroll
                    for (int c = 0; c < 8; c++) {
                        const float4 x = __ldcg((const float4 *)(p.c + first) + c);
                        f[4 * c] = x.x; f[4 * c + 1] = x.y; f[4 * c + 2] = x.z; f[4 * c + 3] = x.w;
                    }
                    if (p.fmt_c == QB200_Q8_0) encode_q8_0_block(f, p.cb + (first >> 5) * 34);
                    else encode_q4_0_block(f, p.cb + (first >> 5) * 18);
                }
            }
        }
        if (lane == 0 && warp < 6) { MM_TRACE(p, 16 + 4 * (warp - 2), w_tfull); MM_TRACE(p, 17 + 4 * (warp - 2), MM_CLOCK() - t_begin); MM_TRACE(p, 18 + 4 * (warp - 2), t_store); }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
    if (PUB && MM_WORLD(p) > 0 && threadIdx.x == 0) publish_count(p.pub, !*abort_flag);
}

// ---------------------------------------------------------------------------------- few rows of A: the operands change sides

// With few rows of A (m <= 64: a decoding batch) a 128-row tile of A is mostly padding, and the kernel above still pays
// a full accumulator and a full handshake a k-block.  Here the operands change sides: the 128 rows of a tile of B are the
// tensor instruction's M (the lanes of tensor memory), the rows of A its N = BN (16, 32 or 64).  The sums are the same
// integers and the scale product commutes exactly, so acc = fma(float(D), sB*sA, acc) is the same f32 as above.
// A k-block's sums now take BN columns of tensor memory, so BATCH = 64 / BN k-blocks form a batch of 64 + 64 columns:
// BATCH instructions for the sums, ONE for the scale products of all of them (B's scale rows hold the group's eight
// scales; A's rows for k-block j are zero except at position j: LAY_FEW), one commit, one barrier round trip, one wait of
// the epilogue; NB batches are in flight.  Thread (q, lane) of the four epilogue warps owns row n0 + 32 q + lane of B,
// i.e. column n of C, and keeps its BN accumulators in registers; a warp's stores of one row of C are 32 consecutive
// floats.  A shared-memory stage is one group of eight k-blocks: B's slab in one copy (read once from HBM), A's in another.
// RAW: 0 = B comes prepacked (LAY_GROUPED slabs, one copy a stage); 1 + format = B comes as raw Q8_0 / Q4_0 rows and eight
// converter warps re-lay a tile's group of k-blocks into the stage themselves: coalesced 16-byte loads of the rows' bytes
// into registers (the next stage's while the current one is converted), through a staging buffer in shared memory, then
// a thread a (row, block) writes the int8 codes as core matrices and the f16 scale into the scale rows, as the pack
// kernels would have written them to memory.  The weights are then read once, in their raw form (Q4_0: 4 bits a value),
// and a call on raw operands needs no packing pass over B.
template <int BN, int RAW = 0>
struct FewCfg {
    static constexpr int KS = GROUP;                               // k-blocks a shared-memory stage
    // RAW 3, 4: as 1, 2 with the rows' bytes fetched by the TMA unit (one 2-D tile copy a stage from a tensor map over B's
    // rows, into a ring of RAWS raw stages) instead of by the converters' own loads
    static constexpr bool TMA = RAW >= 3;
    static constexpr int RFMT = TMA ? RAW - 2 : RAW;
    static constexpr int RAW_BB = RFMT == 2 ? 18 : 34;              // bytes a raw block
    static constexpr int RAW_HALVES = GROUP * RAW_BB / 2, RAW_PITCH = RAW_HALVES + 2;      // halfwords a row's group; an odd number of words a row
    static constexpr int RAWS = TMA ? 3 : 0;
    static constexpr uint32_t RAW_ROW = GROUP * RAW_BB, RAW_STAGE = TILE * RAW_ROW;
    static constexpr uint32_t STAGING = TMA ? RAWS * RAW_STAGE : RAW ? TILE * RAW_PITCH * 2 : 0;
    static constexpr int BATCH = 64 / BN;                          // k-blocks a batch in tensor memory
    static constexpr int BCOLS = 128;                              // its columns: 64 of sums, 64 of scale products
    static constexpr int NB = 512 / BCOLS;                         // batches in flight
    static constexpr uint32_t B_KB = TILE * 32, A_KB = BN * 32;    // bytes of codes a k-block
    static constexpr uint32_t B_SLAB = GROUP * B_KB + TILE * 16, A_SLAB = GROUP * A_KB + GROUP * BN * 16;
    static constexpr uint32_t O_BS = GROUP * B_KB, O_A = B_SLAB, O_AS = O_A + GROUP * A_KB;
    static constexpr uint32_t STAGE = B_SLAB + A_SLAB;
    static constexpr uint32_t PATCH = 2048;
    static constexpr int S_FIT = (int)((MM_SMEM_MAX - MM_HEADER - PATCH - STAGING) / STAGE);
    static constexpr int S = S_FIT > 8 ? 8 : S_FIT;
    static constexpr uint32_t O_PATCH = MM_HEADER + S * STAGE;
    static constexpr uint32_t O_STAGING = O_PATCH + PATCH;
    static constexpr uint32_t SMEM = O_STAGING + STAGING;
    static_assert(BN == 16 || BN == 32 || BN == 64, "the batch is 64 columns of sums");
    static_assert(S >= 2 && 2 * S + 2 * NB + 2 * RAWS + 2 <= 64, "barriers fit the header");
};
// Warps of the few-rows kernel: 0 producer, 1 and 2 issue the tensor instructions of the even and the odd batches (one
// thread each: an instruction costs its issuer about 60 cycles, whatever its shape, and this kernel's are small), 3 idle,
// 4 .. the epilogue: four warps (one a quarter of the lanes) for every 32 columns of sums.
#ifndef FEW_CW
#define FEW_CW 16
#endif
constexpr int CONV_WARPS = 8;               // RAW: the warps after the epilogue's
template <int BN, int RAW = 0> __host__ __device__ constexpr int few_threads() { return 32 * (4 + 4 * (BN / FEW_CW) + (RAW ? CONV_WARPS : 0)); }

template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&v)[N])
{
    static_assert(N % 16 == 0, "whole reads of 16 columns");
#pragma unroll
    for (int c = 0; c < N; c += 16) tmem_ld16(taddr + c, *(uint32_t(*)[16])(v + c));
}

template <int BN, int RAW>
__global__ void __launch_bounds__((few_threads<BN, RAW>()), 1) fewrows_kernel(const __grid_constant__ MatmulArgs p, const __grid_constant__ CUtensorMap bmap)
{
    using G = FewCfg<BN, RAW>;
    constexpr bool TMA = G::TMA;
    constexpr int RFMT = G::RFMT, RAWS = G::RAWS;
    constexpr int S = G::S, KS = G::KS, BATCH = G::BATCH, NB = G::NB, BPS = KS / BATCH;
    constexpr int CG = BN / FEW_CW, CW = FEW_CW;                    // column groups of the epilogue, columns a warp
    constexpr int THREADS = few_threads<BN, RAW>(), CONV0 = 4 + 4 * CG;      // the first converter warp
    // k-blocks of a batch the epilogue reads at once (64 registers of sums and scale products a thread)
    constexpr int SUB = RAW && BATCH > 2 ? 2 : BATCH;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = smem_u32(smem);
    const uint32_t full0 = base, empty0 = base + 8 * S, tfull0 = base + 16 * S, tempty0 = tfull0 + 8 * NB;
    const uint32_t rawfull0 = tempty0 + 8 * NB, rawempty0 = rawfull0 + 8 * RAWS;         // the raw stages' barriers (TMA)
    const uint32_t holder = rawempty0 + 8 * RAWS;
    volatile int *abort_flag = (volatile int *)(smem + 768);
    volatile uint32_t *holder_ptr = (volatile uint32_t *)(smem + (holder - base));
    constexpr int wmode = MM_WAIT_MODE;
    static_assert((NB & (NB - 1)) == 0, "batches in flight: a power of two");

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(full0 + 8 * s, RAW ? 1 + CONV_WARPS : 1);     // the producer's copies, and the converter warps
            mbar_init(empty0 + 8 * s, 2);                // both issuers' commits
        }
        for (int t = 0; t < NB; t++) {
            mbar_init(tfull0 + 8 * t, 1);
            mbar_init(tempty0 + 8 * t, 4 * CG);
        }
        for (int r = 0; r < RAWS; r++) {
            mbar_init(rawfull0 + 8 * r, 1);
            mbar_init(rawempty0 + 8 * r, CONV_WARPS);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    for (int i = threadIdx.x; i < (int)G::PATCH / 16; i += THREADS) *(uint4 *)(smem + G::O_PATCH + i * 16) = make_uint4(0, 0, 0, 0);
    fence_proxy_async();
    if (warp == 1) tmem_alloc(holder, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *holder_ptr;
    uint8_t *ring = smem + MM_HEADER;
    // a tile: 128 rows of B of one product; this block takes tiles blockIdx.x, + gridDim.x, ...; a stage: one group of a tile
    const int ntiles = p.b.rows_pad / TILE, tiles = p.batch * ntiles, groups = p.b.groups;
    const int my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0, stages = my_tiles * groups;
    const int bpt = (p.kb + BATCH - 1) / BATCH;                        // batches a tile

    if (warp == 0) {
        // ---- producer (one thread): per stage the slab of the tile of B (codes and scale rows, one copy) and A's slab of
        // the group (another).  B does not depend on the kernel before this one (A's packing), so the first stages' copies
        // of B are issued before griddepcontrol.wait lets A's follow.
        if (lane == 0) {
            long long w_empty = 0;
            const long long t_begin = MM_CLOCK();
            const bool with_a = !(MM_PROBE(p) & 1);
            auto b_src = [&](int sc) {
                const int tile = blockIdx.x + (sc / groups) * gridDim.x, bi = tile / ntiles, nt = tile - bi * ntiles;
                return p.b.codes + bi * p.b_stride + ((size_t)nt * groups + sc % groups) * G::B_SLAB;
            };
            auto a_src = [&](int sc) {
                const int tile = blockIdx.x + (sc / groups) * gridDim.x, bi = tile / ntiles;
                return p.a.codes + bi * p.a_stride + (size_t)(sc % groups) * G::A_SLAB;
            };
            const int pre = min(S, stages);
            for (int sc = 0; sc < pre; sc++) {
                mbar_arrive_expect_tx(full0 + 8 * sc, (RAW ? 0u : G::B_SLAB) + (with_a ? G::A_SLAB : 0u));
                if (!RAW) bulk_g2s(smem_u32(ring + (size_t)sc * G::STAGE), b_src(sc), G::B_SLAB, full0 + 8 * sc);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int sc = 0; sc < pre && with_a; sc++) bulk_g2s(smem_u32(ring + (size_t)sc * G::STAGE) + G::O_A, a_src(sc), G::A_SLAB, full0 + 8 * sc);
            int sc = pre;
            for (; sc < stages; sc++) {
                const int s = sc % S;
                const long long w0 = MM_CLOCK();
                if (!mm_wait(empty0 + 8 * s, (uint32_t)(sc / S - 1) & 1u, abort_flag, p.status, wmode)) break;
                w_empty += MM_CLOCK() - w0;
                const uint32_t dst = smem_u32(ring + (size_t)s * G::STAGE), bar = full0 + 8 * s;
                mbar_arrive_expect_tx(bar, (RAW ? 0u : G::B_SLAB) + (with_a ? G::A_SLAB : 0u));
                if (!RAW) bulk_g2s(dst, b_src(sc), G::B_SLAB, bar);
                if (with_a) bulk_g2s(dst + G::O_A, a_src(sc), G::A_SLAB, bar);
            }
            MM_TRACE(p, 0, w_empty); MM_TRACE(p, 1, MM_CLOCK() - t_begin); MM_TRACE(p, 2, (long long)sc);
            if (*abort_flag) {          // let the copies still in flight land before the block exits
                for (int it = max(0, sc - S); it < sc; it++) {
                    long long start = clock64();
                    while (!mbar_try_wait(full0 + 8 * (it % S), (uint32_t)(it / S) & 1u) && clock64() - start < WAIT_CYCLES) { }
                }
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ---- MMA issue, the batches of this warp's parity (the epilogue takes batches in order, so neither issuer gets a
        // whole round of the NB accumulators ahead of the other): per k-block the sums (kind::i8, M 128, N BN, K 32); per
        // batch the scale products of its k-blocks (kind::f16, N 64, K 16: the 16-byte scale rows, the other half of K
        // from the patch of zeros) and one commit.  Batch b of stage sc is batch (sc / groups) * bpt + (sc % groups) * BPS + b
        // of the block.  Both issuers commit a stage's release.
        if (lane == 0) {
            bool alive = true;
            long long w_full = 0, w_tempty = 0;
            const long long t_begin = MM_CLOCK();
            const int role = warp - 1;
            constexpr uint64_t DESC_HI = (uint64_t)(128u >> 4) << 16 | (uint64_t)(256u >> 4) << 32 | (uint64_t)1 << 46;
            const uint32_t patch = base + G::O_PATCH;
            constexpr uint32_t idesc = idesc_of(0, TILE, BN), idesc_s = idesc_of(1, TILE, 64);
            for (int sc = 0; sc < stages && alive; sc++) {
                const int s = sc % S, g = sc % groups, nkb = min(KS, p.kb - g * KS);
                const int tc0 = (sc / groups) * bpt + g * BPS;
                const long long w0 = MM_CLOCK();
                if (!mm_poll(full0 + 8 * s, (uint32_t)(sc / S) & 1u, wmode & 3) &&
                    !mm_wait(full0 + 8 * s, (uint32_t)(sc / S) & 1u, abort_flag, p.status, wmode)) { alive = false; break; }
                w_full += MM_CLOCK() - w0;
                tc_fence_after();
                // B's scale rows are the same for the whole group, A's move a batch of rows on (and the patch that much nearer)
                const uint32_t st = smem_u32(ring + (size_t)s * G::STAGE);
                const uint64_t bc = DESC_HI | (uint64_t)(st >> 4), ac = DESC_HI | (uint64_t)((st + G::O_A) >> 4);
                const uint64_t bs = smem_desc(st + G::O_BS, patch - (st + G::O_BS), 128);
                const uint64_t as = smem_desc(st + G::O_AS, patch - (st + G::O_AS), 128);
                constexpr uint64_t AS_STEP = (uint64_t)((64 * 16) >> 4) - ((uint64_t)((64 * 16) >> 4) << 16);
#pragma unroll
                for (int b = 0; b < BPS; b++) {
                    const int tc = tc0 + b;
                    if (b * BATCH < nkb && (tc & 1) == role) {
                        const int slot = tc & (NB - 1);
                        if (tc >= NB) {
                            const uint32_t par = (uint32_t)(tc / NB - 1) & 1u;
                            const long long w1 = MM_CLOCK();
                            if (!mm_poll(tempty0 + 8 * slot, par, wmode & 3) && !mm_wait(tempty0 + 8 * slot, par, abort_flag, p.status, wmode)) { alive = false; break; }
                            w_tempty += MM_CLOCK() - w1;
                            tc_fence_after();
                        }
                        const uint32_t d = tmem + (uint32_t)(slot * G::BCOLS);
#pragma unroll
                        for (int j = 0; j < BATCH; j++) {
                            const int kk = b * BATCH + j;
                            if (kk < nkb) mma_issue<0>(d + j * BN, bc + (uint64_t)kk * (G::B_KB >> 4), ac + (uint64_t)kk * (G::A_KB >> 4), idesc, 0u);
                        }
                        // the rows of a k-block the group does not have give columns nobody reads
                        if (!(MM_PROBE(p) & 8)) mma_issue<1>(d + 64, bs, as + (uint64_t)b * AS_STEP, idesc_s, 0u);
                        mma_commit(tfull0 + 8 * slot);
                    }
                }
                if (alive) mma_commit(empty0 + 8 * s);      // the stage is free once both issuers' products have run
            }
            MM_TRACE(p, 8 + 4 * (warp - 1), w_full); MM_TRACE(p, 9 + 4 * (warp - 1), w_tempty); MM_TRACE(p, 10 + 4 * (warp - 1), MM_CLOCK() - t_begin);
        }
    } else if (TMA && warp == 3) {
        // ---- the raw rows' producer (one thread): per stage one 2-D tile copy, the tile's 128 rows x the group's bytes, into
        // the ring of raw stages (rows past the matrix come as zeros).  B does not depend on the kernel before this one.
        if (lane == 0) {
            for (int sc = 0; sc < stages; sc++) {
                const int r = sc % RAWS, tile = blockIdx.x + (sc / groups) * gridDim.x, n0 = (tile % ntiles) * TILE;
                if (sc >= RAWS && !mm_wait(rawempty0 + 8 * r, (uint32_t)(sc / RAWS - 1) & 1u, abort_flag, p.status, wmode)) break;
                mbar_arrive_expect_tx(rawfull0 + 8 * r, G::RAW_STAGE);
                const uint32_t dst = base + G::O_STAGING + (uint32_t)r * G::RAW_STAGE;
                const int x = (sc % groups) * (int)(G::RAW_ROW / 2);            // in 16-bit elements: a multiple of 16 bytes
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                             :: "r"(dst), "l"((uint64_t)&bmap), "r"(x), "r"(n0), "r"(rawfull0 + 8 * r) : "memory");
            }
            if (*abort_flag) {          // let the copies still in flight land before the block exits
                for (int r = 0; r < RAWS; r++) {
                    long long start = clock64();
                    while (!mbar_try_wait(rawfull0 + 8 * r, 0u) && !mbar_try_wait(rawfull0 + 8 * r, 1u) && clock64() - start < WAIT_CYCLES / 64) { }
                }
            }
        }
    } else if (warp >= 4 && warp < CONV0) {
        // ---- epilogue: warp (q, cg) reads lanes 32 q .. 32 q + 31 and columns cg * CW .. of every k-block's sums
        const int q = warp & 3, cg = (warp - 4) >> 2;
        const uint32_t tlane = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(cg * CW);
        int tc = 0;
        bool alive = true;
        long long w_tfull = 0, w_ld = 0;
        const long long t_begin = MM_CLOCK();
        for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
            const int bi = tile / ntiles, n0 = (tile - bi * ntiles) * TILE;
            float acc[CW];
#pragma unroll
            for (int c = 0; c < CW; c++) acc[c] = 0.f;
            for (int i = 0; i < p.kb && alive; i += BATCH, tc++) {
                const int t = tc & (NB - 1), nb = min(BATCH, p.kb - i);
                const uint32_t bar = tfull0 + 8 * t, par = (uint32_t)(tc / NB) & 1u;
                const long long w0 = MM_CLOCK();
                if (!mm_poll(bar, par, wmode & 3) && !mm_wait_lanes(bar, par, abort_flag, p.status, wmode)) { alive = false; break; }
                const long long w1 = MM_CLOCK();
                w_tfull += w1 - w0;
                tc_fence_after();
                const uint32_t at = tlane + (uint32_t)(t * G::BCOLS);
#pragma unroll
                for (int j0 = 0; j0 < BATCH; j0 += SUB) {
                    uint32_t v[SUB][CW], x[SUB][CW];
#pragma unroll
                    for (int j = 0; j < SUB; j++) {
                        tmem_ld_cols<CW>(at + (j0 + j) * BN, v[j]);
                        tmem_ld_cols<CW>(at + 64 + (j0 + j) * BN, x[j]);
                    }
                    tmem_ld_wait();
                    if (j0 == 0) w_ld += MM_CLOCK() - w1;
#pragma unroll
                    for (int j = 0; j < SUB; j++) {
#pragma unroll
                        for (int c = 0; c < CW; c += 16) { pin16(v[j] + c); pin16(x[j] + c); }
                    }
                    if (j0 + SUB >= BATCH) {
                        tc_fence_before();
                        if (lane == 0) mbar_arrive(tempty0 + 8 * t);         // the batch has been read (warp-wide reads)
                    }
#pragma unroll
                    for (int j = 0; j < SUB; j++) {
                        if (j0 + j < nb && !(MM_PROBE(p) & 4)) {
#pragma unroll
                            for (int c = 0; c < CW; c++) acc[c] = __fmaf_rn((float)(int32_t)v[j][c], __uint_as_float(x[j][c]), acc[c]);
                        }
                    }
                }
            }
            const int col = n0 + q * 32 + lane;
            float *c_out = p.c + bi * p.c_stride;
            if (alive && col < p.n) {
#pragma unroll
                for (int r = 0; r < CW; r++) if (cg * CW + r < p.m) c_out[(size_t)(cg * CW + r) * p.ldc + col] = acc[r];
                for (int pw = 0; pw < MM_WORLD(p); pw++) {          // the sharded product: into the other GPUs' copies of C
                    float *peer = p.pub.out[pw];
                    if (!peer) continue;
#pragma unroll
                    for (int r = 0; r < CW; r++) if (cg * CW + r < p.m) peer[(size_t)(cg * CW + r) * p.ldc + col] = acc[r];
                }
            }
            if (p.cb) {
                // `Back` for the tile: once the epilogue warps have stored their lanes, their threads encode the tile's blocks of
                // 32 consecutive values of a row of C (n % 32 == 0: a block lies inside one warp's columns)
                // (the barrier also tells every thread whether all of them are still going: they leave together or not at all)
                if (!named_bar_and(2, 128 * CG, alive && !*abort_flag)) { alive = false; break; }
                const int bw = min(TILE, p.n - n0) / 32, tid = threadIdx.x - 128;
                for (int idx = tid; idx < p.m * bw; idx += 128 * CG) {
                    const int rr = idx / bw, bc = idx - rr * bw;
                    const size_t first = bi * p.c_stride + (size_t)rr * p.n + n0 + bc * 32;
                    float f[32];
#pragma unroll
                    for (int c = 0; c < 8; c++) {
                        const float4 x4 = __ldcg((const float4 *)(p.c + first) + c);
                        f[4 * c] = x4.x; f[4 * c + 1] = x4.y; f[4 * c + 2] = x4.z; f[4 * c + 3] = x4.w;
                    }
                    if (p.fmt_c == QB200_Q8_0) encode_q8_0_block(f, p.cb + (first >> 5) * 34);
                    else encode_q4_0_block(f, p.cb + (first >> 5) * 18);
                }
            }
        }
        if (lane == 0 && warp < 8) { MM_TRACE(p, 16 + 4 * (warp - 4), w_tfull); MM_TRACE(p, 17 + 4 * (warp - 4), MM_CLOCK() - t_begin); MM_TRACE(p, 18 + 4 * (warp - 4), w_ld); }
    } else if (TMA && warp >= CONV0) {
        // ---- converters on raw stages the TMA unit filled: lane = 8 rows x 4 blocks (rows 272 or 144 bytes apart: eight rows
        // start in eight different banks; reads of different blocks then collide two ways at most, and the eight lanes of a
        // 16-byte store write one core matrix's 128 contiguous bytes); a warp takes four (row group, half of the blocks) pairs
        constexpr int BB = G::RAW_BB;
        const int cw = warp - CONV0, rsub = lane & 7, jsub = lane >> 3;
        for (int sc = 0; sc < stages; sc++) {
            const int r = sc % RAWS, s = sc % S;
            if (!mm_wait(rawfull0 + 8 * r, (uint32_t)(sc / RAWS) & 1u, abort_flag, p.status, wmode)) break;
            if (sc >= S && !mm_wait(empty0 + 8 * s, (uint32_t)(sc / S - 1) & 1u, abort_flag, p.status, wmode)) break;
            const uint8_t *raw = smem + G::O_STAGING + (size_t)r * G::RAW_STAGE;
            uint8_t *stage = ring + (size_t)s * G::STAGE;
#pragma unroll
            for (int i4 = 0; i4 < 4; i4++) {
                const int pair = cw * 4 + i4, rg = pair >> 1, j = (pair & 1) * 4 + jsub, row = rg * 8 + rsub;
                const uint32_t *w32 = (const uint32_t *)(raw + (size_t)row * G::RAW_ROW) + (j * BB) / 4;
                const uint32_t shift = (j & 1) ? 32u : 16u;             // an odd block starts two bytes past a word boundary
                uint32_t w[8], d_bits;
                if (RFMT == 1) {
                    uint32_t v[9];
#pragma unroll
                    for (int i = 0; i < 9; i++) v[i] = w32[i];
                    d_bits = (j & 1) ? v[0] >> 16 : v[0] & 0xFFFFu;
#pragma unroll
                    for (int i = 0; i < 8; i++) w[i] = __funnelshift_rc(v[i], v[i + 1], shift);
                } else {
                    // value i in the low nibble of byte i, value i + 16 in the high nibble, each minus 8 (src/MatMulBlocks.cs:282-299)
                    uint32_t v[5];
#pragma unroll
                    for (int i = 0; i < 5; i++) v[i] = w32[i];
                    d_bits = (j & 1) ? v[0] >> 16 : v[0] & 0xFFFFu;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const uint32_t nib = __funnelshift_rc(v[i], v[i + 1], shift);
                        w[i] = __vsub4(nib & 0x0F0F0F0Fu, 0x08080808u);
                        w[i + 4] = __vsub4((nib >> 4) & 0x0F0F0F0Fu, 0x08080808u);
                    }
                }
                uint8_t *codes = stage + j * G::B_KB + rg * 256 + rsub * 16;
                *(uint4 *)codes = make_uint4(w[0], w[1], w[2], w[3]);
                *(uint4 *)(codes + 128) = make_uint4(w[4], w[5], w[6], w[7]);
                *(uint16_t *)(stage + G::O_BS + row * 16 + j * 2) = (uint16_t)d_bits;
            }
            fence_proxy_async();                         // the tensor cores read the stage through the async proxy
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(full0 + 8 * s);
                mbar_arrive(rawempty0 + 8 * r);          // the raw stage has been read
            }
        }
    } else if (RAW && warp >= CONV0) {
        // ---- converters (RAW): the tile's rows of the group, raw, become the stage's codes and scale rows
        constexpr int BB = G::RAW_BB, VECS = GROUP * BB / 16, PITCH = G::RAW_PITCH, CT = CONV_WARPS * 32, PER = (TILE * VECS + CT - 1) / CT;
        const int ct = threadIdx.x - CONV0 * 32;
        uint16_t *staging = (uint16_t *)(smem + G::O_STAGING);
        const size_t row_bytes = (size_t)p.kb * BB;
        // 16-byte pieces of the 128 row segments, consecutive threads on consecutive pieces (coalesced); rows past the end
        // read as zeros.  The next stage's bytes are on their way (in registers) while one is converted; a second stage
        // ahead changed nothing (the loads of one stage already fill the multiprocessor's queue of pending requests: this
        // path is bound by that queue and by the conversion's own shared-memory traffic, not by the tensor cores).
        auto load = [&](int sc, uint4 (&held)[PER]) {
            if (sc >= stages) return;
            const int tile = blockIdx.x + (sc / groups) * gridDim.x, n0 = (tile % ntiles) * TILE;
            const uint8_t *src = p.b_raw + (size_t)(sc % groups) * (GROUP * BB);
#pragma unroll
            for (int i = 0; i < PER; i++) {
                const int idx = ct + i * CT, rr = idx / VECS, c = idx - rr * VECS;
                held[i] = make_uint4(0, 0, 0, 0);
                if (idx < TILE * VECS && n0 + rr < p.n) held[i] = __ldg((const uint4 *)(src + (size_t)(n0 + rr) * row_bytes) + c);
            }
        };
        // one stage: its bytes from registers to the staging buffer, the registers refilled with the next stage's, the
        // conversion into the ring; false when the block gives up
        const bool load_first = (warp & 1) == 0;
        long long c_sts = 0, c_bar = 0, c_wait = 0, c_conv = 0, c_and = 0, c_fence = 0, c_load = 0;
        const long long c_begin = MM_CLOCK();
        auto step = [&](int sc, uint4 (&held)[PER]) -> bool {
            const long long q0 = MM_CLOCK();
#pragma unroll
            for (int i = 0; i < PER; i++) {
                const int idx = ct + i * CT, rr = idx / VECS, c = idx - rr * VECS;
                if (idx < TILE * VECS) {
                    uint32_t *dst = (uint32_t *)(staging + rr * PITCH) + c * 4;
                    dst[0] = held[i].x; dst[1] = held[i].y; dst[2] = held[i].z; dst[3] = held[i].w;
                }
            }
            const long long q1 = MM_CLOCK();
            named_bar_sync(3, CT);                       // the staging buffer holds the stage's raw bytes
            const long long q2 = MM_CLOCK();
            // half the warps ask for the next stage's bytes before they convert, the other half after: the loads' issue (the
            // queue of pending requests) and the conversion (shared memory, integer pipe) then overlap across warps
            if (load_first) load(sc + 1, held);
            c_load += MM_CLOCK() - q2;
            const int s = sc % S;
            bool ok = true;
            if (sc >= S) ok = mm_wait(empty0 + 8 * s, (uint32_t)(sc / S - 1) & 1u, abort_flag, p.status, wmode);
            const long long q3 = MM_CLOCK();
            c_sts += q1 - q0; c_bar += q2 - q1; c_wait += q3 - q2;
            if (ok) {
                uint8_t *stage = ring + (size_t)s * G::STAGE;
                const int rl = ct & (TILE - 1), half = ct >> 7;
#pragma unroll
                for (int jj = 0; jj < GROUP / 2; jj++) {
                    const int j = half * (GROUP / 2) + jj;
                    // the block's bytes as 32-bit words: a block starts on a word boundary when j is even (34 j and 18 j are
                    // then multiples of 4), two bytes past one when j is odd; jj has j's parity (half * 4 is even)
                    const uint32_t *w32 = (const uint32_t *)(staging + rl * PITCH) + (j * BB) / 4;
                    uint32_t w[8], d_bits;
                    if (RFMT == 1) {
                        uint32_t r[9];
#pragma unroll
                        for (int i = 0; i < 9; i++) r[i] = w32[i];
                        if (jj & 1) {
                            d_bits = r[0] >> 16;
#pragma unroll
                            for (int i = 0; i < 8; i++) w[i] = r[i + 1];
                        } else {
                            d_bits = r[0] & 0xFFFFu;
#pragma unroll
                            for (int i = 0; i < 8; i++) w[i] = __funnelshift_r(r[i], r[i + 1], 16);
                        }
                    } else {
                        // value i in the low nibble of byte i, value i + 16 in the high nibble, each minus 8 (src/MatMulBlocks.cs:282-299)
                        uint32_t r[5];
#pragma unroll
                        for (int i = 0; i < 5; i++) r[i] = w32[i];
                        d_bits = (jj & 1) ? r[0] >> 16 : r[0] & 0xFFFFu;
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const uint32_t nib = (jj & 1) ? r[i + 1] : __funnelshift_r(r[i], r[i + 1], 16);
                            w[i] = __vsub4(nib & 0x0F0F0F0Fu, 0x08080808u);
                            w[i + 4] = __vsub4((nib >> 4) & 0x0F0F0F0Fu, 0x08080808u);
                        }
                    }
                    uint8_t *codes = stage + j * G::B_KB + (rl / 8) * 256 + (rl & 7) * 16;
                    *(uint4 *)codes = make_uint4(w[0], w[1], w[2], w[3]);
                    *(uint4 *)(codes + 128) = make_uint4(w[4], w[5], w[6], w[7]);
                    *(uint16_t *)(stage + G::O_BS + rl * 16 + j * 2) = (uint16_t)d_bits;
                }
                const long long q5 = MM_CLOCK();
                fence_proxy_async();                     // the tensor cores read the stage through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(full0 + 8 * s);
                c_fence += MM_CLOCK() - q5;
            }
            if (!load_first) load(sc + 1, held);
            // everybody has read the staging buffer; and everybody goes on, or nobody does
            const long long q4 = MM_CLOCK();
            const bool go = named_bar_and(3, CT, ok && !*abort_flag);
            c_conv += q4 - q3; c_and += MM_CLOCK() - q4;
            return go;
        };
        uint4 held0[PER];
        load(0, held0);
        for (int sc = 0; sc < stages; sc++) {
            if (!step(sc, held0)) break;
        }
        if (ct == 0) { MM_TRACE(p, 32, c_sts); MM_TRACE(p, 33, c_bar); MM_TRACE(p, 34, c_wait); MM_TRACE(p, 35, c_conv); MM_TRACE(p, 36, c_and); MM_TRACE(p, 37, MM_CLOCK() - c_begin); MM_TRACE(p, 38, (long long)stages); MM_TRACE(p, 39, c_fence); MM_TRACE(p, 40, c_load); }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
    if (MM_WORLD(p) > 0 && threadIdx.x == 0) publish_count(p.pub, !*abort_flag);
}

// ---------------------------------------------------------------------------------- few rows of A against Q4_K weights

// The few-rows kernel for weights whose scale products stay on the CUDA cores (Q4_K: scales d*sc and mins dmin*m are
// f32).  Same sides as fewrows_kernel: the 128 rows of a tile of B on the lanes of tensor memory, A's rows (BN = 16, 32 or 64)
// as columns; a k-block's sums take BN columns and nothing else, so 64 / BN k-blocks form a batch of 64 columns and
// eight batches are in flight.  Thread (q, lane) owns row n of B: its scale and min of a k-block are two words of shared
// memory, A's scales and scaled code sums are broadcast reads;
//     acc = fma(float(D), sA * (d*sc), acc);  acc = fma(dmin*m, -(sA * sum(qA)), acc)      (the 128-row-tile kernel's order).
// B comes k-block-major (LAY_KBLOCK): three copies a k-block (codes, scales, mins), issued by a lane each; A in its
// few-rows form with f32 planes (one copy a stage).
// HALFQ: Q6_K weights, k-blocks of 16 values (the other half of the instruction's K comes from a patch of zeros on B's
// side; A's may then be anything), no min term.
template <int BN, bool HALFQ>
struct FewQCfg {
    static constexpr int KS = GROUP;
    static constexpr int BATCH = 64 / BN, BCOLS = 64, NB = 512 / BCOLS;
    static constexpr int KC = HALFQ ? 1 : 2;
    static constexpr uint32_t B_KB = TILE * KC * 16, PLANE_KB = TILE * 4, A_KB = BN * KC * 16;
    static constexpr uint32_t O_SB = KS * B_KB, O_MB = O_SB + KS * PLANE_KB, O_A = O_MB + (HALFQ ? 0 : KS * PLANE_KB);
    static constexpr uint32_t A_SLAB = GROUP * A_KB + 2 * GROUP * BN * 4, O_SA = O_A + GROUP * A_KB, O_UA = O_SA + GROUP * BN * 4;
    static constexpr uint32_t STAGE = O_A + A_SLAB;
    static constexpr uint32_t PATCH = HALFQ ? 2048 : 0;
    static constexpr int S_FIT = (int)((MM_SMEM_MAX - MM_HEADER - PATCH) / STAGE);
    static constexpr int S = S_FIT > 6 ? 6 : S_FIT;
    static constexpr uint32_t O_PATCH = MM_HEADER + S * STAGE;
    static constexpr uint32_t SMEM = O_PATCH + PATCH;
    static_assert(BN == 16 || BN == 32 || BN == 64, "at most 64 rows of A");
    static_assert(S >= 2 && 2 * S + 2 * NB + 2 <= 64, "barriers fit the header");
};
template <int BN> __host__ __device__ constexpr int fewq_threads() { return 32 * (4 + 4 * (BN / 16)); }

template <int BN, bool HALFQ>
__global__ void __launch_bounds__(fewq_threads<BN>(), 1) fewq_kernel(const __grid_constant__ MatmulArgs p)
{
    using G = FewQCfg<BN, HALFQ>;
    constexpr int S = G::S, KS = G::KS, BATCH = G::BATCH, NB = G::NB, BPS = KS / BATCH, CG = BN / 16, CW = 16;
    constexpr int THREADS = fewq_threads<BN>();
    extern __shared__ __align__(1024) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = smem_u32(smem);
    const uint32_t full0 = base, empty0 = base + 8 * S, tfull0 = base + 16 * S, tempty0 = tfull0 + 8 * NB;
    const uint32_t holder = tempty0 + 8 * NB;
    volatile int *abort_flag = (volatile int *)(smem + 768);
    volatile uint32_t *holder_ptr = (volatile uint32_t *)(smem + (holder - base));
    constexpr int wmode = MM_WAIT_MODE;
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 2 + 4 * CG);       // both issuers' commits, and the epilogue warps, which read the stage's scales
        }
        for (int t = 0; t < NB; t++) {
            mbar_init(tfull0 + 8 * t, 1);
            mbar_init(tempty0 + 8 * t, 4 * CG);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (G::PATCH) {
        for (int i = threadIdx.x; i < (int)G::PATCH / 16; i += THREADS) *(uint4 *)(smem + G::O_PATCH + i * 16) = make_uint4(0, 0, 0, 0);
        fence_proxy_async();
    }
    if (warp == 1) tmem_alloc(holder, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *holder_ptr;
    uint8_t *ring = smem + MM_HEADER;
    const int ntiles = p.b.rows_pad / TILE, tiles = p.batch * ntiles, groups = p.b.groups;
    const int my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0, stages = my_tiles * groups;
    const int bpt = (p.kb + BATCH - 1) / BATCH;

    if (warp == 0) {
        // ---- producer: lanes 0 .. 23 copy B's codes, scales and mins of the stage's k-blocks, lane 24 A's slab
        asm volatile("griddepcontrol.wait;" ::: "memory");       // the kernel before this one packed A
        bool alive = true;
        for (int sc = 0; sc < stages && alive; sc++) {
            const int s = sc % S, g = sc % groups, tile = blockIdx.x + (sc / groups) * gridDim.x, bi = tile / ntiles, n0 = (tile - bi * ntiles) * TILE;
            const int nkb = min(KS, p.kb - g * KS);
            int ok = 1;
            if (lane == 0 && sc >= S) ok = mm_wait(empty0 + 8 * s, (uint32_t)(sc / S - 1) & 1u, abort_flag, p.status, wmode) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { alive = false; break; }
            const uint32_t dst = smem_u32(ring + (size_t)s * G::STAGE), bar = full0 + 8 * s;
            if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)nkb * (G::B_KB + (HALFQ ? 1 : 2) * G::PLANE_KB) + G::A_SLAB);
            __syncwarp();
            const int kk = lane / 3, what = lane - kk * 3;
            if (lane < 24 && kk < nkb && !(HALFQ && what == 2)) {
                const size_t kb = (size_t)(g * KS + kk);
                const uint8_t *bb = p.b.codes + bi * p.b_stride, *bs = (const uint8_t *)p.b.scales + bi * p.b_stride, *bm = (const uint8_t *)p.b.extra + bi * p.b_stride;
                if (what == 0) bulk_g2s(dst + kk * G::B_KB, bb + (kb * (p.b.rows_pad / 8) + n0 / 8) * (G::KC * 128), G::B_KB, bar);
                else if (what == 1) bulk_g2s(dst + G::O_SB + kk * G::PLANE_KB, bs + (kb * p.b.rows_pad + n0) * 4, G::PLANE_KB, bar);
                else bulk_g2s(dst + G::O_MB + kk * G::PLANE_KB, bm + (kb * p.b.rows_pad + n0) * 4, G::PLANE_KB, bar);
            } else if (lane == 24) bulk_g2s(dst + G::O_A, p.a.codes + bi * p.a_stride + (size_t)g * G::A_SLAB, G::A_SLAB, bar);
        }
        if (*abort_flag && lane == 0) {          // let the copies still in flight land before the block exits
            for (int it = max(0, stages - S); it < stages; it++) {
                long long start = clock64();
                while (!mbar_try_wait(full0 + 8 * (it % S), (uint32_t)(it / S) & 1u) && clock64() - start < WAIT_CYCLES) { }
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ---- MMA issue: the batches of this warp's parity; per k-block the sums (kind::i8, M 128, N BN, K 32), one commit a batch
        if (lane == 0) {
            bool alive = true;
            const int role = warp - 1;
            constexpr uint64_t DESC_HI = (uint64_t)(128u >> 4) << 16 | (uint64_t)((G::KC * 128u) >> 4) << 32 | (uint64_t)1 << 46;
            constexpr uint32_t idesc = idesc_of(0, TILE, BN);
            const uint32_t patch = base + G::O_PATCH;
            for (int sc = 0; sc < stages && alive; sc++) {
                const int s = sc % S, g = sc % groups, nkb = min(KS, p.kb - g * KS);
                const int tc0 = (sc / groups) * bpt + g * BPS;
                if (!mm_poll(full0 + 8 * s, (uint32_t)(sc / S) & 1u, wmode & 3) &&
                    !mm_wait(full0 + 8 * s, (uint32_t)(sc / S) & 1u, abort_flag, p.status, wmode)) { alive = false; break; }
                tc_fence_after();
                const uint32_t st = smem_u32(ring + (size_t)s * G::STAGE);
                const uint64_t bc = DESC_HI | (uint64_t)(st >> 4), ac = DESC_HI | (uint64_t)((st + G::O_A) >> 4);
#pragma unroll
                for (int b = 0; b < BPS; b++) {
                    const int tc = tc0 + b;
                    if (b * BATCH < nkb && (tc & 1) == role) {
                        const int slot = tc & (NB - 1);
                        if (tc >= NB) {
                            const uint32_t par = (uint32_t)(tc / NB - 1) & 1u;
                            if (!mm_poll(tempty0 + 8 * slot, par, wmode & 3) && !mm_wait(tempty0 + 8 * slot, par, abort_flag, p.status, wmode)) { alive = false; break; }
                            tc_fence_after();
                        }
                        const uint32_t d = tmem + (uint32_t)(slot * G::BCOLS);
#pragma unroll
                        for (int j = 0; j < BATCH; j++) {
                            const int kk = b * BATCH + j;
                            if (kk < nkb) {
                                if (HALFQ) {
                                    // the second 16-byte k-chunk of every row of B is the patch of zeros; A's may then be anything
                                    const uint32_t b_at = st + kk * G::B_KB, a_at = st + G::O_A + kk * G::A_KB;
                                    mma_issue<0>(d + j * BN, smem_desc(b_at, patch - b_at, 128), smem_desc(a_at, 128, 128), idesc, 0u);
                                } else mma_issue<0>(d + j * BN, bc + (uint64_t)kk * (G::B_KB >> 4), ac + (uint64_t)kk * (G::A_KB >> 4), idesc, 0u);
                            }
                        }
                        mma_commit(tfull0 + 8 * slot);
                    }
                }
                if (alive) mma_commit(empty0 + 8 * s);
            }
        }
    } else if (warp >= 4) {
        // ---- epilogue: warp (q, cg) reads lanes 32 q .. and columns cg * 16 .. of every k-block's sums
        const int q = warp & 3, cg = (warp - 4) >> 2;
        const uint32_t tlane = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(cg * CW);
        int tc = 0, sc = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
            const int bi = tile / ntiles, n0 = (tile - bi * ntiles) * TILE;
            float acc[CW];
#pragma unroll
            for (int c = 0; c < CW; c++) acc[c] = 0.f;
            for (int i = 0; i < p.kb && alive; i += BATCH, tc++) {
                const int t = tc & (NB - 1), nb = min(BATCH, p.kb - i), s = sc % S, kk0 = i % KS;
                const uint32_t bar = tfull0 + 8 * t, par = (uint32_t)(tc / NB) & 1u;
                if (!mm_poll(bar, par, wmode & 3) && !mm_wait_lanes(bar, par, abort_flag, p.status, wmode)) { alive = false; break; }
                tc_fence_after();
                const uint32_t at = tlane + (uint32_t)(t * G::BCOLS);
                uint32_t v[BATCH][CW];
#pragma unroll
                for (int j = 0; j < BATCH; j++) tmem_ld_cols<CW>(at + j * BN, v[j]);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < BATCH; j++) pin16(v[j]);
                tc_fence_before();
                if (lane == 0) mbar_arrive(tempty0 + 8 * t);
                // the stage's planes (complete long since: the products that filled the batch read the same stage; the poll is
                // this thread's own sight of the copies)
                if (kk0 == 0 && !mm_poll(full0 + 8 * s, (uint32_t)(sc / S) & 1u, wmode & 3) &&
                    !mm_wait_lanes(full0 + 8 * s, (uint32_t)(sc / S) & 1u, abort_flag, p.status, wmode)) { alive = false; break; }
                const uint8_t *stage = ring + (size_t)s * G::STAGE;
#pragma unroll
                for (int j = 0; j < BATCH; j++) {
                    if (j < nb) {
                        const int kk = kk0 + j;
                        const float sb = ((const float *)(stage + G::O_SB))[kk * TILE + q * 32 + lane];
                        const float wb = HALFQ ? 0.f : ((const float *)(stage + G::O_MB))[kk * TILE + q * 32 + lane];
                        const float4 *sa4 = (const float4 *)(stage + G::O_SA) + (kk * BN + cg * CW) / 4;
                        const float4 *ua4 = (const float4 *)(stage + G::O_UA) + (kk * BN + cg * CW) / 4;
#pragma unroll
                        for (int c4 = 0; c4 < CW / 4; c4++) {
                            const float4 sa = sa4[c4], ua = ua4[c4];
                            const float sav[4] = { sa.x, sa.y, sa.z, sa.w }, uav[4] = { ua.x, ua.y, ua.z, ua.w };
#pragma unroll
                            for (int c = 0; c < 4; c++) {
                                float a1 = __fmaf_rn((float)(int32_t)v[j][4 * c4 + c], __fmul_rn(sav[c], sb), acc[4 * c4 + c]);
                                acc[4 * c4 + c] = HALFQ ? a1 : __fmaf_rn(wb, -uav[c], a1);
                            }
                        }
                    }
                }
                if (kk0 + BATCH >= KS || i + BATCH >= p.kb) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty0 + 8 * s);          // this warp has read the stage's planes
                    sc++;
                }
            }
            const int col = n0 + q * 32 + lane;
            float *c_out = p.c + bi * p.c_stride;
            if (alive && col < p.n) {
#pragma unroll
                for (int r = 0; r < CW; r++) if (cg * CW + r < p.m) c_out[(size_t)(cg * CW + r) * p.ldc + col] = acc[r];
                for (int pw = 0; pw < MM_WORLD(p); pw++) {          // the sharded product: into the other GPUs' copies of C
                    float *peer = p.pub.out[pw];
                    if (!peer) continue;
#pragma unroll
                    for (int r = 0; r < CW; r++) if (cg * CW + r < p.m) peer[(size_t)(cg * CW + r) * p.ldc + col] = acc[r];
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
    if (MM_WORLD(p) > 0 && threadIdx.x == 0) publish_count(p.pub, !*abort_flag);
}

// ---------------------------------------------------------------------------------- the tensor pipe's own rate

// One thread of one block issues `iters` x 4 tcgen05.mma kind::i8 (M 128, N 128, K 32, the product's instruction) on
// whatever bytes shared memory holds, into two alternating accumulators, commits once and waits for the commit with a
// bound: clock cycles from the first issue to the completion, what the tensor pipe of one multiprocessor does with no
// epilogue, no copies and nothing else on the chip.  out[0] = cycles, out[1] = 1 when the wait completed.
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int iters, long long *out)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t base = smem_u32(smem), bar = base, holder = base + 64;
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        mbar_fence_init();
    }
    for (int i = threadIdx.x; i < 16384 / 4; i += 128) ((uint32_t *)(smem + 1024))[i] = 0x01010101u * (uint32_t)(i & 3);
    fence_proxy_async();
    if (threadIdx.x < 32) tmem_alloc(holder, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *(volatile uint32_t *)(smem + 64);
    if (threadIdx.x == 0) {
        const uint32_t idesc = idesc_of(0, TILE, 128);
        const uint64_t a = smem_desc(base + 1024, 128, 256), b = smem_desc(base + 1024 + 8192, 128, 256);
        const long long t0 = clock64();
        for (int i = 0; i < iters; i++) {
#pragma unroll
            for (int k = 0; k < 4; k++) mma_issue<0>(tmem + (uint32_t)(k & 1) * 128, a, b, idesc, 0u);
        }
        mma_commit(bar);
        bool done = false;
        while (!(done = mbar_try_wait(bar, 0u)) && clock64() - t0 < WAIT_CYCLES) { }
        out[0] = clock64() - t0;
        out[1] = done ? 1 : 0;
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) tmem_dealloc(tmem, 512);
}

// Cycles one tcgen05.mma kind::i8 of the product's shape takes on one multiprocessor (64.0 at the rate the data sheet's
// dense int8 figure implies); 0 when the measurement did not complete.  Allocates 16 bytes for its result.
int matmul_mma_rate(double *cycles_per_mma, cudaStream_t stream)
{
    const int iters = 512;
    long long *out = nullptr, host[2] = { 0, 0 };
    cudaError_t e = cudaMalloc((void **)&out, 2 * sizeof(long long));
    if (e) return (int)e;
    if ((e = cudaFuncSetAttribute(mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768))) { cudaFree(out); return (int)e; }
    mma_rate_kernel<<<1, 128, 32768, stream>>>(iters, out);
    if (!(e = cudaGetLastError())) e = cudaMemcpyAsync(host, out, sizeof host, cudaMemcpyDeviceToHost, stream);
    if (!e) e = cudaStreamSynchronize(stream);
    cudaFree(out);
    if (e) return (int)e;
    *cycles_per_mma = host[1] ? (double)host[0] / (4.0 * iters) : 0.0;
    return 0;
}

// ---------------------------------------------------------------------------------- host side

static int *g_mm_status = nullptr;
#ifdef QB_MM_TUNING
static long long *g_mm_trace = nullptr;
extern "C" void qb200_mm_set_trace(long long *buffer) { g_mm_trace = buffer; }
#endif
static int g_mm_sms = 0;
static int g_mm_kind = 0;          // the tensor kind the library packs for and multiplies with
static int g_mm_tcs = 1;           // scale products of plain f16 scales on the tensor cores
static int g_mm_few = 64;          // most rows of A the kernel with the operands' sides exchanged takes
static int g_mm_raw_few = 1;       // that kernel re-lays raw weights itself where it can
static int g_mm_raw_tma = 1;       // ... fetching the raw rows by 2-D TMA tile copies
// cuTensorMapEncodeTiled, fetched through the runtime (the library does not link the driver); null when it is not there
typedef CUresult (*EncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiled g_encode_tiled = nullptr;


template <int BN, int RAW>
static cudaError_t set_few_attr()
{
    return cudaFuncSetAttribute(fewrows_kernel<BN, RAW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FewCfg<BN, RAW>::SMEM);
}

template <int KIND, int SUMS, int VAR>
static cudaError_t set_mm_attr_var()
{
    return cudaFuncSetAttribute(matmul_kernel<KIND, SUMS, VAR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)Cfg<KIND, VAR == VAR_MINS, VAR == VAR_HALF, VAR == VAR_TCS>::SMEM);
}
template <int KIND, int SUMS>
static cudaError_t set_mm_attr()
{
    cudaError_t e;
    if ((e = set_mm_attr_var<KIND, SUMS, VAR_PLAIN>()) || (e = set_mm_attr_var<KIND, SUMS, VAR_MINS>())) return e;
    if ((e = set_mm_attr_var<KIND, SUMS, VAR_HALF>())) return e;
    return set_mm_attr_var<KIND, SUMS, VAR_TCS>();
}

cudaError_t matmul_init(int sm_count, int max_smem, int *status)
{
    g_mm_status = status;
    g_mm_sms = sm_count;
    if ((int)MM_SMEM_MAX > max_smem) return cudaErrorInvalidValue;
#ifdef QB_MM_TUNING
    const char *kind = getenv("QB200_MM_KIND"), *tcs = getenv("QB200_MM_TCS");
    g_mm_kind = kind && *kind ? atoi(kind) != 0 : 0;
    g_mm_tcs = tcs && *tcs ? atoi(tcs) != 0 : 1;
    const char *few = getenv("QB200_MM_FEW");
    g_mm_few = few && *few ? atoi(few) : 64;
    const char *rawfew = getenv("QB200_MM_RAW_FEW");
    g_mm_raw_few = rawfew && *rawfew ? atoi(rawfew) != 0 : 1;
    const char *rawtma = getenv("QB200_MM_RAW_TMA");
    g_mm_raw_tma = rawtma && *rawtma ? atoi(rawtma) != 0 : 1;
#endif
    cudaError_t e;
    if ((e = set_few_attr<16, 0>()) || (e = set_few_attr<32, 0>()) || (e = set_few_attr<64, 0>())) return e;
    if ((e = set_few_attr<16, 1>()) || (e = set_few_attr<32, 1>())) return e;
    if ((e = set_few_attr<16, 2>()) || (e = set_few_attr<32, 2>())) return e;
    if ((e = set_few_attr<16, 3>()) || (e = set_few_attr<32, 3>()) || (e = set_few_attr<64, 3>())) return e;
    if ((e = set_few_attr<16, 4>()) || (e = set_few_attr<32, 4>()) || (e = set_few_attr<64, 4>())) return e;
    {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult found;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found) == cudaSuccess && found == cudaDriverEntryPointSuccess)
            g_encode_tiled = (EncodeTiled)fn;
        else (void)cudaGetLastError();
    }
    if ((e = cudaFuncSetAttribute(fewq_kernel<16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FewQCfg<16, false>::SMEM))) return e;
    if ((e = cudaFuncSetAttribute(fewq_kernel<32, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FewQCfg<32, false>::SMEM))) return e;
    if ((e = cudaFuncSetAttribute(fewq_kernel<16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FewQCfg<16, true>::SMEM))) return e;
    if ((e = cudaFuncSetAttribute(fewq_kernel<32, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FewQCfg<32, true>::SMEM))) return e;
    if ((e = cudaFuncSetAttribute(fewq_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FewQCfg<64, false>::SMEM))) return e;
    if ((e = cudaFuncSetAttribute(fewq_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FewQCfg<64, true>::SMEM))) return e;
    if ((e = set_mm_attr<0, 0>()) || (e = set_mm_attr<0, 1>()) || (e = set_mm_attr<0, 2>())) return e;
    if ((e = set_mm_attr<1, 0>()) || (e = set_mm_attr<1, 1>())) return e;
    return cudaSuccess;
}

// k-blocks of the product: 32 values each, 16 against Q6_K rows
static int k_blocks(int fmt_b, int k) { return fmt_b == QB200_Q6_K ? k / 16 : k / 32; }
static int pad_rows(int rows) { return (rows + TILE - 1) / TILE * TILE; }
static size_t align256(size_t v) { return (v + 255) / 256 * 256; }
static size_t codes_bytes(int rows, int k) { return (size_t)pad_rows(rows) * k * (g_mm_kind ? 2 : 1); }
// a plane of per-(row, k-block) values: f32, or the 16-byte rows of the tensor cores' scale product
static size_t plane_bytes(int rows, int kbs, bool tcs = false) { return (size_t)pad_rows(rows) * kbs * (tcs ? 16 : 4); }
// whether the scale products of a product against fmt_b rows run on the tensor cores
static bool use_tcs(int fmt_b) { return g_mm_tcs && (fmt_b == QB200_Q8_0 || fmt_b == QB200_Q4_0); }

// A packed operand in one buffer.  LAY_GROUPED: the slabs alone.  LAY_TILE / LAY_KBLOCK: codes, scales, extra plane, each
// on a 256-byte boundary (the extra plane is only written when B is Q4_K, but always has its place).
static int kc_of(int k, int kbs) { return (k / kbs) * (g_mm_kind ? 2 : 1) / 16; }
static size_t packed_bytes(int layout, int rows, int k, int kbs, bool tcs)
{
    if (layout == LAY_GROUPED) return align256((size_t)(pad_rows(rows) / TILE) * groups_of(kbs) * grouped_slab(kc_of(k, kbs)));
    return align256(codes_bytes(rows, k)) + align256(plane_bytes(rows, kbs, tcs)) + align256(plane_bytes(rows, kbs));
}
// A's slab of the workspace: its LAY_TILE form, or its LAY_FEW form where that is larger (whole groups of k-blocks)
static int few_bn(int m) { return m <= 16 ? 16 : m <= 32 ? 32 : 64; }
static size_t a_packed_bytes(int m, int k, int kbs, bool tcs)
{
    const size_t tile = packed_bytes(LAY_TILE, m, k, kbs, tcs);
    const size_t few = tcs && m <= 64 ? align256((size_t)groups_of(kbs) * few_slab(few_bn(m), kc_of(k, kbs))) :
                       !tcs && m <= 64 ? align256((size_t)groups_of(kbs) * fewq_slab(few_bn(m), kc_of(k, kbs))) : 0;
    return tile > few ? tile : few;
}
// B with plain f16 scales is grouped for the tensor cores' scale product, any other B is k-block-major with f32 planes
static int b_layout(int fmt_b) { return use_tcs(fmt_b) ? LAY_GROUPED : LAY_KBLOCK; }

size_t matmul_prepacked_bytes(int fmt_b, int n, int k) { return packed_bytes(b_layout(fmt_b), n, k, k_blocks(fmt_b, k), false); }

// Scratch of a call: every product's packed A (one when A is the same for all), then every distinct packed B
// (none when the caller brings B prepacked).
size_t matmul_workspace_bytes(int fmt_b, int m, int n, int k, const MatmulBatch &batch, bool b_prepacked)
{
    const int kbs = k_blocks(fmt_b, k);
    const size_t a_sets = batch.stride_a ? batch.count : 1, b_sets = b_prepacked ? 0 : (batch.stride_b ? batch.count : 1);
    return a_sets * a_packed_bytes(m, k, kbs, use_tcs(fmt_b)) + b_sets * packed_bytes(b_layout(fmt_b), n, k, kbs, false);
}

// bytes between two products' raw operands `stride` values apart (whole blocks)
static size_t raw_bytes(int fmt, long long stride) { return (size_t)(stride / block_values(fmt)) * block_bytes(fmt); }

// `bn`: rows kept in LAY_FEW
static PackTarget target_in(void *buffer, int rows, int k, int kbs, int layout, bool tcs, int bn = 0)
{
    uint8_t *w = (uint8_t *)buffer;
    PackTarget t;
    t.codes = w;
    t.scales = (float *)(w + align256(codes_bytes(rows, k)));
    t.extra = (float *)(w + align256(codes_bytes(rows, k)) + align256(plane_bytes(rows, kbs, tcs)));
    t.layout = layout;
    t.tcs = tcs ? 1 : 0;
    t.rows_pad = layout == LAY_FEW ? (bn < 32 ? 32 : bn) : pad_rows(rows);      // the pack kernels take 32 rows a block
    t.kbs = kbs;
    t.kc = kc_of(k, kbs);
    t.kind = g_mm_kind;
    t.bn = bn;
    return t;
}

static cudaError_t pack(int fmt, const void *raw, int rows, int k, const PackTarget &t, bool want_usums, bool split, cudaStream_t stream)
{
    const int kb32 = k / 32, padded = t.rows_pad;
    const uint8_t *r = (const uint8_t *)raw;
    if (fmt == QB200_Q4_K) {
        if ((long long)(padded / 128) * (kb32 / 8) >= 2ll * g_mm_sms) pack_q4_k_kernel<128><<<dim3(padded / 128, kb32 / 8), 256, 0, stream>>>(r, rows, kb32, t);
        else pack_q4_k_kernel<32><<<dim3(padded / 32, kb32 / 8), 256, 0, stream>>>(r, rows, kb32, t);
    }
    else if (fmt == QB200_Q6_K) pack_q6_k_kernel<<<dim3(padded / 32, k / 256), 256, 0, stream>>>(r, rows, k / 16, t);
    else {
        const int us = want_usums ? 1 : 0, kgroups = (kb32 + 7) / 8;
        const bool large = (long long)(padded / 128) * kgroups >= 2ll * g_mm_sms;
        const dim3 grid(large ? padded / 128 : padded / 32, kgroups);
        if (fmt == QB200_Q8_0) {
            if (split) { if (large) pack_rows_kernel<QB200_Q8_0, true, 128><<<grid, 256, 0, stream>>>(r, rows, kb32, t, us); else pack_rows_kernel<QB200_Q8_0, true, 32><<<grid, 256, 0, stream>>>(r, rows, kb32, t, us); }
            else { if (large) pack_rows_kernel<QB200_Q8_0, false, 128><<<grid, 256, 0, stream>>>(r, rows, kb32, t, us); else pack_rows_kernel<QB200_Q8_0, false, 32><<<grid, 256, 0, stream>>>(r, rows, kb32, t, us); }
        } else {
            if (split) { if (large) pack_rows_kernel<QB200_Q4_0, true, 128><<<grid, 256, 0, stream>>>(r, rows, kb32, t, us); else pack_rows_kernel<QB200_Q4_0, true, 32><<<grid, 256, 0, stream>>>(r, rows, kb32, t, us); }
            else { if (large) pack_rows_kernel<QB200_Q4_0, false, 128><<<grid, 256, 0, stream>>>(r, rows, kb32, t, us); else pack_rows_kernel<QB200_Q4_0, false, 32><<<grid, 256, 0, stream>>>(r, rows, kb32, t, us); }
        }
    }
    return cudaGetLastError();
}

// B (n x k, fmt_b) re-laid for the product into `packed` (matmul_prepacked_bytes): the weights' half of a call's packing,
// done once by a caller that keeps the result.
int matmul_prepack_b(int fmt_b, const void *b, int n, int k, void *packed, cudaStream_t stream)
{
    const PackTarget t = target_in(packed, n, k, k_blocks(fmt_b, k), b_layout(fmt_b), false);
    return (int)pack(fmt_b, b, n, k, t, false, false, stream);
}

template <int BN, int RAW>
static cudaError_t launch_few(int grid, const MatmulArgs &args, const CUtensorMap &bmap, cudaStream_t stream)
{
    // launched as a programmatic dependent of A's packing: its prologue and its first loads of B run beside it
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(few_threads<BN, RAW>()); cfg.dynamicSmemBytes = FewCfg<BN, RAW>::SMEM;
    cfg.stream = stream; cfg.attrs = &attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, fewrows_kernel<BN, RAW>, args, bmap);
}
template <int RAW>
static cudaError_t launch_few_rows(int bn, int grid, const MatmulArgs &args, const CUtensorMap &bmap, cudaStream_t stream)
{
    if (bn == 16) return launch_few<16, RAW>(grid, args, bmap, stream);
    if (bn == 32) return launch_few<32, RAW>(grid, args, bmap, stream);
    if constexpr (RAW == 0 || RAW >= 3) return launch_few<64, RAW>(grid, args, bmap, stream);
    else return cudaErrorInvalidValue;         // raw weights by the converters' own loads: at most 32 rows of A (their registers)
}

// A tensor map over B's raw rows as 16-bit elements: tiles of 128 rows x one group of eight blocks; rows past n read as zeros.
static bool raw_rows_map(CUtensorMap &map, const void *b, int fmt_b, int n, int kbs)
{
    if (!g_encode_tiled) return false;
    const cuuint64_t row_bytes = (cuuint64_t)kbs * block_bytes(fmt_b);
    const cuuint64_t dims[2] = { row_bytes / 2, (cuuint64_t)n }, strides[1] = { row_bytes };
    const cuuint32_t box[2] = { (cuuint32_t)(GROUP * block_bytes(fmt_b) / 2), (cuuint32_t)TILE }, estr[2] = { 1, 1 };
    return g_encode_tiled(&map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(b), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
template <int KIND, int SUMS, int VAR>
static void launch_var(int grid, const MatmulArgs &args, cudaStream_t stream)
{
    // a programmatic dependent of A's packing (the launch before it): its prologue runs beside that kernel, its producer
    // waits for it before the first copy
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(mm_threads(VAR == VAR_TCS) + (SUMS == 2 ? 32 : 0)); cfg.stream = stream; cfg.attrs = &attr; cfg.numAttrs = 1;
    cfg.dynamicSmemBytes = Cfg<KIND, VAR == VAR_MINS, VAR == VAR_HALF, VAR == VAR_TCS>::SMEM;
    cudaLaunchKernelEx(&cfg, matmul_kernel<KIND, SUMS, VAR>, args);
}

template <int KIND, int SUMS>
static void launch_product(int var, int grid, const MatmulArgs &args, cudaStream_t stream)
{
    if (var == VAR_MINS) launch_var<KIND, SUMS, VAR_MINS>(grid, args, stream);
    else if (var == VAR_HALF) launch_var<KIND, SUMS, VAR_HALF>(grid, args, stream);
    else if (var == VAR_TCS) launch_var<KIND, SUMS, VAR_TCS>(grid, args, stream);
    else launch_var<KIND, SUMS, VAR_PLAIN>(grid, args, stream);
}

template <int KIND>
static void launch_kind(bool sums, int var, int grid, const MatmulArgs &args, cudaStream_t stream)
{
    if (sums) launch_product<KIND, 1>(var, grid, args, stream);
    else launch_product<KIND, 0>(var, grid, args, stream);
}

// fmt_a: Q8_0 / Q4_0; fmt_b: Q8_0 / Q4_0 / Q4_K / Q6_K (k then in whole super-blocks of 256).  `b_packed`: B as
// matmul_prepack_b left it, or null to pack `b` into the workspace now.  `c_blocks`: optional `Back` of C as fmt_c.
int matmul_launch(int fmt_a, int fmt_b, const void *a, const void *b, const void *b_packed, float *c, int32_t *sums, int fmt_c,
                  void *c_blocks, int m, int n, int k, const MatmulBatch &batch, void *workspace, cudaStream_t stream, int ldc, const void *publish)
{
    if (publish && (sums || c_blocks || batch.count != 1)) return QB200_E_SHAPE;
    const bool mins = fmt_b == QB200_Q4_K, half = fmt_b == QB200_Q6_K;
    const int kbs = k_blocks(fmt_b, k);
    cudaError_t e;
    // every product's A, and every distinct B, is packed into a slab of its own
    const bool tcs = use_tcs(fmt_b);
    // few rows of A: B's rows become the lanes of tensor memory (fewrows_kernel), A is packed for that
    const bool few = tcs && !sums && g_mm_kind == 0 && m <= g_mm_few;
    // ... and against Q4_K weights (scale products on the CUDA cores) with at most 64 rows, lanes only
    const bool fewq = (mins || half) && !sums && !c_blocks && g_mm_kind == 0 && m <= 64 && m <= g_mm_few;
    const int bn = few_bn(m), a_layout = few || fewq ? LAY_FEW : LAY_TILE, lay_b = b_layout(fmt_b);
    const size_t a_slab = a_packed_bytes(m, k, kbs, tcs), b_slab = packed_bytes(lay_b, n, k, kbs, false);
    // ... and on raw weights that come in whole groups of eight blocks, 16-byte aligned, the kernel re-lays B itself
    // (its rows fetched by the TMA unit where a tensor map over them can be made; else by the converters' own loads, at most 32 rows of A)
    const bool raw_able = few && !b_packed && batch.count == 1 && kbs % GROUP == 0 && ((uintptr_t)b & 15) == 0 && g_mm_raw_few;
    CUtensorMap bmap;
    memset(&bmap, 0, sizeof bmap);
    const bool raw_tma = raw_able && g_mm_raw_tma && raw_rows_map(bmap, b, fmt_b, n, kbs);
    const bool raw_few = raw_tma || (raw_able && m <= 32);
    const int b_sets = b_packed || raw_few ? 0 : (batch.stride_b ? batch.count : 1);
    const size_t a_raw = raw_bytes(fmt_a, batch.stride_a), b_raw = raw_bytes(fmt_b, batch.stride_b);
    // B first: A's packing is then the launch right before the product, whose start the few-rows kernel overlaps
    const int a_sets = batch.stride_a ? batch.count : 1;
    uint8_t *b_area = (uint8_t *)workspace + a_sets * a_slab;
    PackTarget tb = target_in(b_packed ? (void *)b_packed : (void *)b_area, n, k, kbs, lay_b, false);
    for (int i = 0; i < b_sets; i++) {
        PackTarget t = target_in(b_area + i * b_slab, n, k, kbs, lay_b, false);
        if ((e = pack(fmt_b, (const uint8_t *)b + i * b_raw, n, k, t, false, false, stream))) return (int)e;
    }
    const PackTarget ta = target_in(workspace, m, k, kbs, a_layout, tcs, bn);
    for (int i = 0; i < batch.count; i++) {
        PackTarget t = target_in((uint8_t *)workspace + i * a_slab, m, k, kbs, a_layout, tcs, bn);
        if ((e = pack(fmt_a, (const uint8_t *)a + i * a_raw, m, k, t, mins, half, stream))) return (int)e;
        if (!batch.stride_a) break;
    }
    MatmulArgs args;
    args.a.codes = ta.codes; args.a.scales = ta.scales; args.a.extra = mins ? ta.extra : nullptr;
    args.b.codes = tb.codes; args.b.scales = tb.scales; args.b.extra = mins ? tb.extra : nullptr; args.b.rows_pad = tb.rows_pad; args.b.groups = groups_of(kbs);
    args.c = c; args.sums = sums; args.status = g_mm_status;
    args.cb = (uint8_t *)c_blocks; args.fmt_c = fmt_c;
    args.m = m; args.n = n; args.kb = kbs;
    args.ldc = ldc > 0 ? ldc : n;
    if (publish) args.pub = *(const GemvPublish *)publish;
    else memset(&args.pub, 0, sizeof args.pub);
    args.probe = 0;
    args.trace = nullptr;
#ifdef QB_MM_TUNING
    { const char *pr = getenv("QB200_MM_PROBE"); args.probe = pr && *pr ? atoi(pr) : 0; }
    args.trace = g_mm_trace;
#endif
    args.unit = 32;          // columns a warp of the epilogue owns: pieces are whole units
    args.units = (n + args.unit - 1) / args.unit;
    args.mtiles = (m + TILE - 1) / TILE;
    args.b_raw = raw_few ? (const uint8_t *)b : nullptr;
    args.batch = batch.count;
    args.a_stride = batch.stride_a ? a_slab : 0;
    args.b_stride = !b_packed && batch.stride_b ? b_slab : 0;
    args.c_stride = (size_t)batch.stride_c;
    if (fewq) {
        const int tiles = batch.count * (tb.rows_pad / TILE), grid = tiles < g_mm_sms ? tiles : g_mm_sms;
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.gridDim = dim3(grid); cfg.stream = stream; cfg.attrs = &attr; cfg.numAttrs = 1;
        cfg.blockDim = dim3(bn == 16 ? fewq_threads<16>() : bn == 32 ? fewq_threads<32>() : fewq_threads<64>());
        if (half) {
            if (bn == 16) { cfg.dynamicSmemBytes = FewQCfg<16, true>::SMEM; e = cudaLaunchKernelEx(&cfg, fewq_kernel<16, true>, args); }
            else if (bn == 32) { cfg.dynamicSmemBytes = FewQCfg<32, true>::SMEM; e = cudaLaunchKernelEx(&cfg, fewq_kernel<32, true>, args); }
            else { cfg.dynamicSmemBytes = FewQCfg<64, true>::SMEM; e = cudaLaunchKernelEx(&cfg, fewq_kernel<64, true>, args); }
        } else {
            if (bn == 16) { cfg.dynamicSmemBytes = FewQCfg<16, false>::SMEM; e = cudaLaunchKernelEx(&cfg, fewq_kernel<16, false>, args); }
            else if (bn == 32) { cfg.dynamicSmemBytes = FewQCfg<32, false>::SMEM; e = cudaLaunchKernelEx(&cfg, fewq_kernel<32, false>, args); }
            else { cfg.dynamicSmemBytes = FewQCfg<64, false>::SMEM; e = cudaLaunchKernelEx(&cfg, fewq_kernel<64, false>, args); }
        }
        return (int)e;
    }
    if (few) {
        const int tiles = batch.count * (tb.rows_pad / TILE), grid = tiles < g_mm_sms ? tiles : g_mm_sms;
        if (raw_tma)
            e = fmt_b == QB200_Q8_0 ? launch_few_rows<3>(bn, grid, args, bmap, stream) : launch_few_rows<4>(bn, grid, args, bmap, stream);
        else if (raw_few) e = fmt_b == QB200_Q8_0 ? launch_few_rows<1>(bn, grid, args, bmap, stream) : launch_few_rows<2>(bn, grid, args, bmap, stream);
        else e = launch_few_rows<0>(bn, grid, args, bmap, stream);
        return (int)e;
    }
    const long long total = (long long)args.batch * args.mtiles * args.units;
    const int grid = (int)(total < g_mm_sms ? total : g_mm_sms);
    const int var = mins ? VAR_MINS : half ? VAR_HALF : tcs ? VAR_TCS : VAR_PLAIN;
    if (publish) launch_product<0, 2>(var, grid, args, stream);       // (the exchange: integer sums on the tensor cores only)
    else if (g_mm_kind) launch_kind<1>(sums != nullptr, var, grid, args, stream);
    else launch_kind<0>(sums != nullptr, var, grid, args, stream);
    return (int)cudaGetLastError();
}

}  // namespace qb
