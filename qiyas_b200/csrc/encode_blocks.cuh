// One block of 32 f32 lanes -> a Q8_0 / Q4_0 block, as device functions shared by the codec kernels and by the gemv
// that encodes its own output.  The arithmetic is the CPU encoder's (reference src/Blocks.cs:37-45, 58-70) operation
// for operation in IEEE round-to-nearest f32 with no contraction; Q4_0 rounds as the reference's device encoder does,
// fma(v, 1/d, 8.5) then floor (src/Ptx.Blocks.cs:80-85).
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace qb {

__device__ __forceinline__ uint16_t f2h_bits(float v) { return __half_as_ushort(__float2half_rn(v)); }
__device__ __forceinline__ float h2f_bits(uint16_t h) { return __half2float(__ushort_as_half(h)); }
// blocks are 2-byte aligned and every f16 field sits at an even offset: one 16-bit store
__device__ __forceinline__ void put16(uint8_t *p, uint16_t v) { *reinterpret_cast<volatile uint16_t *>(p) = v; }
__device__ __forceinline__ int round_clamp(float x, int lo, int hi) { return max(lo, min(hi, __float2int_rn(x))); }

// EncodeQ8_0 (src/Blocks.cs:37-45; device src/Ptx.Blocks.cs:54-73): 34 bytes at o
__device__ __forceinline__ void encode_q8_0_block(const float (&v)[32], uint8_t *o)
{
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(v[i]));
    const uint16_t h = f2h_bits(__fdiv_rn(amax, 127.f));
    const float d = h2f_bits(h), id = d == 0.f ? 0.f : __fdiv_rn(1.f, d);
    put16(o, h);
#pragma unroll
    for (int i = 0; i < 32; i++) o[2 + i] = (uint8_t)(int8_t)round_clamp(__fmul_rn(v[i], id), -127, 127);
}

// EncodeQ4_0 (src/Blocks.cs:58-70) with the device's rounding (src/Ptx.Blocks.cs:80-85): 18 bytes at o
__device__ __forceinline__ void encode_q4_0_block(const float (&v)[32], uint8_t *o)
{
    float amax = 0.f, mx = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i++) {
        const float a = fabsf(v[i]);
        if (a > amax) { amax = a; mx = v[i]; }
    }
    const uint16_t h = f2h_bits(__fdiv_rn(mx, -8.f));
    const float d = h2f_bits(h), id = d == 0.f ? 0.f : __fdiv_rn(1.f, d);
    put16(o, h);
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const int lo = max(0, min(15, __float2int_rd(__fmaf_rn(v[i], id, 8.5f))));
        const int hi = max(0, min(15, __float2int_rd(__fmaf_rn(v[i + 16], id, 8.5f))));
        o[2 + i] = (uint8_t)(lo | hi << 4);
    }
}

}  // namespace qb
