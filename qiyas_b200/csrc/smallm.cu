// Block-scaled A.B^T for a few rows of A (m <= 16): C (m x n, f32) = A (m x k) . B (n x k)^T, A and B in Q8_0 / Q4_0 rows.
//
// The same product as matmul.cu and the same arithmetic, bit for bit (reference src/MatMulBlocks.cs:339-347: per k-block of
// 32 the exact integer sum D, then acc = fma(float(D), sA*sB, acc), k-blocks in ascending order), without the tensor
// cores: a 128-row tensor tile would be seven eighths padding, while the raw blocks of B, read once, bound the time.
// This is the gemv's shape (B streams from HBM, A stays on the chip) with up to sixteen activations a weight.
//
// A block keeps all of A in shared memory (int8 codes, f32 scales).  A warp takes two rows of B at a time and walks them in
// chunks of 32 k-blocks: lane l takes k-block l of the chunk of both rows (the raw block straight from global memory: a
// warp's lanes read consecutive blocks of a row), forms its integer sums against every row of A with dp4a, and leaves them
// in shared memory; then lane (r, i) - row r of the two, row i of A - runs the chunk's 32 scaled additions in order.
#include "common.cuh"
#include "launch.h"

namespace qb {

constexpr int SM_ROWS = 16;               // rows of A at most
constexpr int SM_WARPS = 8;
constexpr int SM_THREADS = 32 * SM_WARPS;
constexpr int SM_DPITCH = 17;             // ints a k-block in the sums' staging: an odd pitch keeps lanes on different banks
constexpr int SM_RAW_BYTES = 32 * 34 + 32; // a chunk of 32 raw blocks (Q8_0 the larger) and padding for the reads past a block
constexpr int SM_STAGE_INTS = 2 * 32 * SM_DPITCH + 64 + 2 * SM_RAW_BYTES / 4;     // a warp's staging area

struct SmallMArgs {
    const uint8_t *a, *b;
    float *c;
    int m, n, kb;
    int fmt_a;
};

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// The 32 values of the raw block at q (2-byte aligned) as eight words of int8 (Q4_0: q - 8) and its scale.
template <int FMT>
__device__ __forceinline__ void load_raw_block(const uint8_t *q, uint32_t (&w)[8], float &d)
{
    const uint16_t *p = (const uint16_t *)q;
    d = half_bits_to_float(__ldg(p));
    if (FMT == QB200_Q8_0) {
#pragma unroll
        for (int i = 0; i < 8; i++) w[i] = (uint32_t)__ldg(p + 1 + 2 * i) | (uint32_t)__ldg(p + 2 + 2 * i) << 16;
    } else {
        // value i in the low nibble of byte i, value i + 16 in the high nibble, each minus 8 (src/MatMulBlocks.cs:282-299)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t n = (uint32_t)__ldg(p + 1 + 2 * i) | (uint32_t)__ldg(p + 2 + 2 * i) << 16;
            w[i] = __vsub4(n & 0x0F0F0F0Fu, 0x08080808u);
            w[i + 4] = __vsub4((n >> 4) & 0x0F0F0F0Fu, 0x08080808u);
        }
    }
}

// The same from a 2-byte aligned address in shared memory, by aligned 32-bit reads and funnel shifts (branch-free: the lanes
// of a warp alternate between the two alignments).  Reads up to 6 bytes past the block (the staging area is padded).
template <int FMT>
__device__ __forceinline__ void load_staged_block(const uint8_t *q, uint32_t (&w)[8], float &d)
{
    const uint32_t *t = (const uint32_t *)((uintptr_t)q & ~(uintptr_t)3);
    const bool odd = ((uintptr_t)q & 2) != 0;                 // the block starts in the upper half of t[0]
    const uint32_t sh = odd ? 0u : 16u;
    const int o = odd ? 1 : 0;
    const uint32_t first = t[0];
    d = half_bits_to_float(odd ? first >> 16 : first & 0xFFFFu);
    constexpr int NW = FMT == QB200_Q8_0 ? 8 : 4;
    uint32_t c[NW];
#pragma unroll
    for (int i = 0; i < NW; i++) c[i] = __funnelshift_r(t[i + o], t[i + o + 1], sh);
    if (FMT == QB200_Q8_0) {
#pragma unroll
        for (int i = 0; i < 8; i++) w[i] = c[i < NW ? i : 0];
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            w[i] = __vsub4(c[i] & 0x0F0F0F0Fu, 0x08080808u);
            w[i + 4] = __vsub4((c[i] >> 4) & 0x0F0F0F0Fu, 0x08080808u);
        }
    }
}

// Shared memory: A's codes [row][k-block][32 bytes] with the two 16-byte halves of a k-block swapped where bit 2 of the
// k-block is set (eight consecutive lanes, reading one half each of eight consecutive k-blocks, then cover all banks);
// A's scales [k-block][16]; and a staging area of the sums and B's scales a warp.
// FAST: every 32-block chunk of every row of B starts on 16 bytes and k is whole chunks: a warp copies a chunk to its
// staging area with 16-byte loads (three a lane) and the lanes take their blocks from there; otherwise every lane reads
// its block from global memory two bytes at a time.
template <int FMT_B, bool FAST>
__global__ void __launch_bounds__(SM_THREADS, 1) smallm_kernel(const SmallMArgs p)
{
    extern __shared__ __align__(16) uint8_t smem[];
    const int kb = p.kb, m = p.m;
    uint8_t *codes = smem;
    float *sa = (float *)(smem + (size_t)SM_ROWS * kb * 32);
    int *stage = (int *)(sa + (size_t)kb * SM_ROWS);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int *dsum = stage + warp * SM_STAGE_INTS;                       // [2][32][17] sums, then [2][32] scales of B, then two raw chunks
    float *sbs = (float *)(dsum + 2 * 32 * SM_DPITCH);
    uint8_t *raw = (uint8_t *)(sbs + 64);

    // ---- A into shared memory (rows past m: zero codes, zero scales)
    for (int idx = threadIdx.x; idx < SM_ROWS * kb; idx += SM_THREADS) {
        const int i = idx / kb, b = idx - i * kb;
        uint32_t w[8] = { 0, 0, 0, 0, 0, 0, 0, 0 };
        float d = 0.f;
        if (i < m) {
            if (p.fmt_a == QB200_Q8_0) load_raw_block<QB200_Q8_0>(p.a + ((size_t)i * kb + b) * 34, w, d);
            else load_raw_block<QB200_Q4_0>(p.a + ((size_t)i * kb + b) * 18, w, d);
        }
        const int swap = (b >> 2) & 1;
        uint4 *dst = (uint4 *)(codes + ((size_t)i * kb + b) * 32);
        dst[swap] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[swap ^ 1] = make_uint4(w[4], w[5], w[6], w[7]);
        sa[(size_t)b * SM_ROWS + i] = d;
    }
    __syncthreads();

    constexpr int BB = block_bytes(FMT_B);
    constexpr int VECS = 32 * BB / 16, VPL = (VECS + 31) / 32;     // 16-byte pieces of a chunk, and a lane's share of them
    constexpr int AHEAD = 3;                                       // chunks in flight from global memory a warp
    const int pairs = (p.n + 1) / 2, chunks = (kb + 31) / 32;
    const int r_of = lane >> 4, i_of = lane & 15;                  // the chain's lane: row r of the pair, row i of A
    const int first = blockIdx.x * SM_WARPS + warp, stride = gridDim.x * SM_WARPS;
    const int my_pairs = first < pairs ? (pairs - first + stride - 1) / stride : 0;
    const long long total = (long long)my_pairs * chunks;          // this warp's (pair, chunk) steps, in order
    // FAST: the raw chunks of the next AHEAD steps wait in registers (global latency is long and a block has few warps)
    uint4 held[FAST ? AHEAD : 1][2][FAST ? VPL : 1];
    auto fetch = [&](long long step, uint4 (&into)[2][FAST ? VPL : 1]) {
        if (!FAST || step >= total) return;
        const int j0 = 2 * (first + (int)(step / chunks) * stride), k0 = (int)(step % chunks) * 32;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const uint4 *src = (const uint4 *)(p.b + ((size_t)min(j0 + r, p.n - 1) * kb + k0) * BB);
#pragma unroll
            for (int v = 0; v < VPL; v++) {
                const int at = lane + 32 * v;
                into[r][v] = at < VECS ? __ldg(src + at) : make_uint4(0, 0, 0, 0);
            }
        }
    };
    if (FAST) {
#pragma unroll
        for (int d = 0; d < AHEAD; d++) fetch(d, held[d]);
    }
    float acc = 0.f;
    for (long long step = 0; step < total; step++) {
        const int j0 = 2 * (first + (int)(step / chunks) * stride), k0 = (int)(step % chunks) * 32;
        const int b = k0 + lane;
        if (k0 == 0) acc = 0.f;
        if (FAST) {
            // the oldest held chunk into the staging area, its registers refilled with the chunk AHEAD steps on
#pragma unroll
            for (int r = 0; r < 2; r++) {
                uint4 *dst = (uint4 *)(raw + r * SM_RAW_BYTES);
#pragma unroll
                for (int v = 0; v < VPL; v++)
                    if (lane + 32 * v < VECS) dst[lane + 32 * v] = held[0][r][v];
            }
#pragma unroll
            for (int d = 0; d + 1 < AHEAD; d++) {
#pragma unroll
                for (int r = 0; r < 2; r++) {
#pragma unroll
                    for (int v = 0; v < VPL; v++) held[d][r][v] = held[d + 1][r][v];
                }
            }
            fetch(step + AHEAD, held[AHEAD - 1]);
            __syncwarp();
        }
        // ---- the integer sums of this lane's k-block, both rows of the pair against every row of A
        if (b < kb) {
            const int swap = (b >> 2) & 1;
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const int j = j0 + r;
                uint32_t w[8] = { 0, 0, 0, 0, 0, 0, 0, 0 };
                float d = 0.f;
                if (j < p.n) {
                    if (FAST) load_staged_block<FMT_B>(raw + r * SM_RAW_BYTES + lane * BB, w, d);
                    else load_raw_block<FMT_B>(p.b + ((size_t)j * kb + b) * BB, w, d);
                }
                sbs[r * 32 + lane] = d;
                // the words that meet the physically first half of A's k-block, and the others
                const uint32_t f0 = swap ? w[4] : w[0], f1 = swap ? w[5] : w[1], f2 = swap ? w[6] : w[2], f3 = swap ? w[7] : w[3];
                const uint32_t g0 = swap ? w[0] : w[4], g1 = swap ? w[1] : w[5], g2 = swap ? w[2] : w[6], g3 = swap ? w[3] : w[7];
#pragma unroll
                for (int i = 0; i < SM_ROWS; i++) {
                    if (i < m) {
                        const uint4 *src = (const uint4 *)(codes + ((size_t)i * kb + b) * 32);
                        const uint4 x = src[0], y = src[1];
                        int e = dp4a_ss(f0, x.x, 0), o = dp4a_ss(f1, x.y, 0);
                        e = dp4a_ss(f2, x.z, e); o = dp4a_ss(f3, x.w, o);
                        e = dp4a_ss(g0, y.x, e); o = dp4a_ss(g1, y.y, o);
                        e = dp4a_ss(g2, y.z, e); o = dp4a_ss(g3, y.w, o);
                        dsum[(r * 32 + lane) * SM_DPITCH + i] = e + o;
                    }
                }
            }
        }
        __syncwarp();
        // ---- the chunk's scaled additions, in k-block order: acc = fma(float(D), sA*sB, acc)
        if (i_of < m) {
            const int steps = min(32, kb - k0);
            const int *dr = dsum + r_of * 32 * SM_DPITCH + i_of;
            const float *sar = sa + (size_t)k0 * SM_ROWS + i_of, *sbr = sbs + r_of * 32;
            if (steps == 32) {
                // all of the chunk's operands first (independent reads), then the 32 dependent additions
                float dv[32], sc[32];
#pragma unroll
                for (int t = 0; t < 32; t++) {
                    dv[t] = (float)dr[t * SM_DPITCH];
                    sc[t] = __fmul_rn(sar[t * SM_ROWS], sbr[t]);
                }
#pragma unroll
                for (int t = 0; t < 32; t++) acc = __fmaf_rn(dv[t], sc[t], acc);
            } else {
                for (int t = 0; t < steps; t++)
                    acc = __fmaf_rn((float)dr[t * SM_DPITCH], __fmul_rn(sar[t * SM_ROWS], sbr[t]), acc);
            }
        }
        __syncwarp();
        if (k0 + 32 >= kb) {
            const int j = j0 + r_of;
            if (i_of < m && j < p.n) p.c[(size_t)i_of * p.n + j] = acc;
        }
    }
}

static int g_sm_sms = 0, g_sm_max_smem = 0;

cudaError_t smallm_init(int sm_count, int max_smem)
{
    g_sm_sms = sm_count;
    g_sm_max_smem = max_smem;
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(smallm_kernel<QB200_Q8_0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem))) return e;
    if ((e = cudaFuncSetAttribute(smallm_kernel<QB200_Q8_0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem))) return e;
    if ((e = cudaFuncSetAttribute(smallm_kernel<QB200_Q4_0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem))) return e;
    return cudaFuncSetAttribute(smallm_kernel<QB200_Q4_0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
}

static size_t smallm_smem(int kb)
{
    return (size_t)SM_ROWS * kb * 32 + (size_t)kb * SM_ROWS * 4 + (size_t)SM_WARPS * SM_STAGE_INTS * 4;
}

// Whether this path takes the product: a few rows of A, plain block formats, A small enough for shared memory.
bool smallm_takes(int fmt_a, int fmt_b, int m, int k)
{
    if (m < 1 || m > SM_ROWS || k % 32) return false;
    if ((fmt_a != QB200_Q8_0 && fmt_a != QB200_Q4_0) || (fmt_b != QB200_Q8_0 && fmt_b != QB200_Q4_0)) return false;
    return g_sm_sms > 0 && smallm_smem(k / 32) <= (size_t)g_sm_max_smem;
}

int smallm_launch(int fmt_a, int fmt_b, const void *a, const void *b, float *c, int m, int n, int k, cudaStream_t stream)
{
    SmallMArgs args;
    args.a = (const uint8_t *)a; args.b = (const uint8_t *)b; args.c = c;
    args.m = m; args.n = n; args.kb = k / 32; args.fmt_a = fmt_a;
    const int pairs = (n + 1) / 2, tiles = (pairs + SM_WARPS - 1) / SM_WARPS;
    const int grid = tiles < g_sm_sms ? tiles : g_sm_sms;
    const size_t smem = smallm_smem(args.kb);
    const size_t row_bytes = (size_t)args.kb * block_bytes(fmt_b);
    const bool fast = args.kb % 32 == 0 && (((uintptr_t)b | row_bytes) & 15) == 0;
    if (fmt_b == QB200_Q8_0) {
        if (fast) smallm_kernel<QB200_Q8_0, true><<<grid, SM_THREADS, smem, stream>>>(args);
        else smallm_kernel<QB200_Q8_0, false><<<grid, SM_THREADS, smem, stream>>>(args);
    } else {
        if (fast) smallm_kernel<QB200_Q4_0, true><<<grid, SM_THREADS, smem, stream>>>(args);
        else smallm_kernel<QB200_Q4_0, false><<<grid, SM_THREADS, smem, stream>>>(args);
    }
    return (int)cudaGetLastError();
}

}  // namespace qb
