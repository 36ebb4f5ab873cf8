// Block codecs on the device: f32 lanes -> blocks (the reference's Ptx.LanesToBlock, src/Ptx.Blocks.cs:11-331, the
// `Back` step after every block-typed product, src/GpuOps.cs:964-975) and blocks -> f32 lanes (Ptx.Widen,
// src/Ptx.Attention.cs:202-219 with Codec.BlockDecode, src/Ptx.cs:151-277).  The arithmetic is the CPU codec's
// (src/Blocks.cs:31-215) operation for operation, in IEEE round-to-nearest f32 with no contraction, so the bytes and
// values equal the CPU's; Q4_0's rounding is the reference device's fma + floor (src/Ptx.Blocks.cs:80-85).
#include "common.cuh"
#include "encode_blocks.cuh"
#include "launch.h"

namespace qb {

__device__ __forceinline__ uint16_t get16(const uint8_t *p) { return (uint16_t)(p[0] | p[1] << 8); }

// values [first, first + count) of the lane array, zero past n (src/Ptx.Blocks.cs:36-44)
template <int COUNT>
__device__ __forceinline__ void load_lanes(const float *lanes, int64_t first, int64_t n, float *v)
{
#pragma unroll 8
    for (int i = 0; i < COUNT; i++) v[i] = first + i < n ? lanes[first + i] : 0.f;
}

// EncodeQ8_0 / EncodeQ4_0, a thread a block (the block arithmetic is in encode_blocks.cuh)
__global__ void encode_q8_0_kernel(const float *lanes, uint8_t *out, int64_t n, int64_t blocks)
{
    int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    float v[32];
    load_lanes<32>(lanes, b * 32, n, v);
    encode_q8_0_block(v, out + b * 34);
}

__global__ void encode_q4_0_kernel(const float *lanes, uint8_t *out, int64_t n, int64_t blocks)
{
    int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    float v[32];
    load_lanes<32>(lanes, b * 32, n, v);
    encode_q4_0_block(v, out + b * 18);
}

// EncodeQ4_K (src/Blocks.cs:98-148), a thread a super-block
__global__ void encode_q4_k_kernel(const float *lanes, uint8_t *out, int64_t n, int64_t blocks)
{
    int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    const int64_t first = b * 256;
    float scales[8], mins[8], max_scale = 0.f, max_min = 0.f;
    for (int j = 0; j < 8; j++) {
        float lo = 3.40282347e38f, hi = -3.40282347e38f;
        for (int i = 0; i < 32; i++) {
            int64_t at = first + j * 32 + i;
            float x = at < n ? lanes[at] : 0.f;
            lo = fminf(lo, x);
            hi = fmaxf(hi, x);
        }
        lo = fminf(lo, 0.f);
        scales[j] = __fdiv_rn(__fsub_rn(hi, lo), 15.f);
        mins[j] = -lo;
        max_scale = fmaxf(max_scale, scales[j]);
        max_min = fmaxf(max_min, mins[j]);
    }
    uint8_t *o = out + b * 144;
    uint16_t hd = f2h_bits(__fdiv_rn(max_scale, 63.f)), hm = f2h_bits(__fdiv_rn(max_min, 63.f));
    put16(o, hd);
    put16(o + 2, hm);
    const float d = h2f_bits(hd), dmin = h2f_bits(hm);
    int ls[8], lm[8];
    for (int j = 0; j < 8; j++) {
        ls[j] = d == 0.f ? 0 : round_clamp(__fdiv_rn(scales[j], d), 0, 63);
        lm[j] = dmin == 0.f ? 0 : round_clamp(__fdiv_rn(mins[j], dmin), 0, 63);
    }
    uint8_t sc[12];
    for (int j = 0; j < 4; j++) {
        sc[j] = (uint8_t)(ls[j] | ((ls[j + 4] >> 4) << 6));
        sc[j + 4] = (uint8_t)(lm[j] | ((lm[j + 4] >> 4) << 6));
        sc[j + 8] = (uint8_t)((ls[j + 4] & 15) | ((lm[j + 4] & 15) << 4));
    }
    for (int j = 0; j < 12; j++) o[4 + j] = sc[j];
    for (int pair = 0; pair < 4; pair++) {
        const float d0 = __fmul_rn(d, (float)ls[2 * pair]), m0 = __fmul_rn(dmin, (float)lm[2 * pair]);
        const float d1 = __fmul_rn(d, (float)ls[2 * pair + 1]), m1 = __fmul_rn(dmin, (float)lm[2 * pair + 1]);
        for (int i = 0; i < 32; i++) {
            int64_t a0 = first + pair * 64 + i, a1 = a0 + 32;
            float x0 = a0 < n ? lanes[a0] : 0.f, x1 = a1 < n ? lanes[a1] : 0.f;
            int q0 = d0 == 0.f ? 0 : round_clamp(__fdiv_rn(__fadd_rn(x0, m0), d0), 0, 15);
            int q1 = d1 == 0.f ? 0 : round_clamp(__fdiv_rn(__fadd_rn(x1, m1), d1), 0, 15);
            o[16 + pair * 32 + i] = (uint8_t)(q0 | q1 << 4);
        }
    }
}

// EncodeQ6_K (src/Blocks.cs:175-215), a thread a super-block
__global__ void encode_q6_k_kernel(const float *lanes, uint8_t *out, int64_t n, int64_t blocks)
{
    int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    const int64_t first = b * 256;
    float scales[16], max_scale = 0.f;
    for (int j = 0; j < 16; j++) {
        float amax = 0.f;
        for (int i = 0; i < 16; i++) {
            int64_t at = first + j * 16 + i;
            amax = fmaxf(amax, fabsf(at < n ? lanes[at] : 0.f));
        }
        scales[j] = __fdiv_rn(amax, 31.f);
        max_scale = fmaxf(max_scale, scales[j]);
    }
    uint8_t *o = out + b * 210;
    uint16_t hd = f2h_bits(__fdiv_rn(max_scale, 127.f));
    put16(o + 208, hd);
    const float d = h2f_bits(hd);
    float dj[16];
    for (int j = 0; j < 16; j++) {
        int ls = d == 0.f ? 0 : round_clamp(__fdiv_rn(scales[j], d), -127, 127);
        o[192 + j] = (uint8_t)(int8_t)ls;
        dj[j] = __fmul_rn(d, (float)ls);
    }
    for (int half = 0; half < 2; half++) {
        for (int l = 0; l < 32; l++) {
            int q[4];
            for (int g = 0; g < 4; g++) {
                int idx = half * 128 + g * 32 + l;
                int64_t at = first + idx;
                float x = at < n ? lanes[at] : 0.f, s = dj[idx / 16];
                q[g] = (s == 0.f ? 0 : round_clamp(__fdiv_rn(x, s), -32, 31)) + 32;
            }
            o[half * 64 + l] = (uint8_t)((q[0] & 15) | ((q[2] & 15) << 4));
            o[half * 64 + l + 32] = (uint8_t)((q[1] & 15) | ((q[3] & 15) << 4));
            o[128 + half * 32 + l] = (uint8_t)(((q[0] >> 4) & 3) | (((q[1] >> 4) & 3) << 2) | (((q[2] >> 4) & 3) << 4) | (((q[3] >> 4) & 3) << 6));
        }
    }
}

// Blocks.Decode* (src/Blocks.cs:31-35,48-56,79-96,151-173), a thread a value
template <int FMT>
__global__ void decode_kernel(const uint8_t *blocks, float *lanes, int64_t n)
{
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    constexpr int BV = block_values(FMT), BB = block_bytes(FMT);
    const uint8_t *b = blocks + i / BV * BB;
    const int at = (int)(i % BV);
    float v;
    if (FMT == QB200_Q8_0) v = __fmul_rn(h2f_bits(get16(b)), (float)(int8_t)b[2 + at]);
    else if (FMT == QB200_Q4_0) {
        int q = at < 16 ? b[2 + at] & 15 : b[2 + at - 16] >> 4;
        v = __fmul_rn(h2f_bits(get16(b)), (float)(q - 8));
    } else if (FMT == QB200_Q4_K) {
        const int j = at / 32, l = at % 32;
        const uint8_t *sc = b + 4;
        int scale, mn;
        if (j < 4) { scale = sc[j] & 63; mn = sc[j + 4] & 63; }
        else { scale = (sc[j + 4] & 15) | ((sc[j - 4] >> 6) << 4); mn = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
        const uint8_t byte = b[16 + j / 2 * 32 + l];
        const int q = j % 2 ? byte >> 4 : byte & 15;
        v = __fsub_rn(__fmul_rn(__fmul_rn(h2f_bits(get16(b)), (float)scale), (float)q), __fmul_rn(h2f_bits(get16(b + 2)), (float)mn));
    } else {
        const int half = at / 128, g = (at % 128) / 32, l = at % 32;
        const uint8_t lo = b[half * 64 + (g & 1) * 32 + l], hb = b[128 + half * 32 + l];
        const int q = ((g < 2 ? lo & 15 : lo >> 4) | (((hb >> (2 * g)) & 3) << 4)) - 32;
        v = __fmul_rn(__fmul_rn(h2f_bits(get16(b + 208)), (float)(int8_t)b[192 + at / 16]), (float)q);
    }
    lanes[i] = v;
}

int encode_launch(int fmt, const float *lanes, void *blocks, int64_t n, cudaStream_t stream)
{
    if (n == 0) return 0;
    const int64_t nb = (n + block_values(fmt) - 1) / block_values(fmt);
    const int threads = fmt == QB200_Q8_0 || fmt == QB200_Q4_0 ? 128 : 64;
    const unsigned grid = (unsigned)((nb + threads - 1) / threads);
    uint8_t *out = (uint8_t *)blocks;
    switch (fmt) {
    case QB200_Q8_0: encode_q8_0_kernel<<<grid, threads, 0, stream>>>(lanes, out, n, nb); break;
    case QB200_Q4_0: encode_q4_0_kernel<<<grid, threads, 0, stream>>>(lanes, out, n, nb); break;
    case QB200_Q4_K: encode_q4_k_kernel<<<grid, threads, 0, stream>>>(lanes, out, n, nb); break;
    default: encode_q6_k_kernel<<<grid, threads, 0, stream>>>(lanes, out, n, nb); break;
    }
    return (int)cudaGetLastError();
}

int decode_launch(int fmt, const void *blocks, float *lanes, int64_t n, cudaStream_t stream)
{
    if (n == 0) return 0;
    const unsigned grid = (unsigned)((n + 255) / 256);
    const uint8_t *in = (const uint8_t *)blocks;
    switch (fmt) {
    case QB200_Q8_0: decode_kernel<QB200_Q8_0><<<grid, 256, 0, stream>>>(in, lanes, n); break;
    case QB200_Q4_0: decode_kernel<QB200_Q4_0><<<grid, 256, 0, stream>>>(in, lanes, n); break;
    case QB200_Q4_K: decode_kernel<QB200_Q4_K><<<grid, 256, 0, stream>>>(in, lanes, n); break;
    default: decode_kernel<QB200_Q6_K><<<grid, 256, 0, stream>>>(in, lanes, n); break;
    }
    return (int)cudaGetLastError();
}

}  // namespace qb
