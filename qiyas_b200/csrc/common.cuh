// Shared device helpers of libqiyas_b200: format traits, f16 scales, mbarrier / bulk-copy (TMA) and
// tcgen05 wrappers in inline PTX for sm_100a, and the bounded waits every kernel uses.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qiyas_b200.h"

namespace qb {

// ---------------------------------------------------------------------------------- formats
__host__ __device__ constexpr int block_values(int fmt) { return fmt == QB200_Q8_0 || fmt == QB200_Q4_0 ? 32 : fmt == QB200_Q4_K || fmt == QB200_Q6_K ? 256 : 0; }
__host__ __device__ constexpr int block_bytes(int fmt) { return fmt == QB200_Q8_0 ? 34 : fmt == QB200_Q4_0 ? 18 : fmt == QB200_Q4_K ? 144 : fmt == QB200_Q6_K ? 210 : 0; }

// Status bits a kernel sets, in the device word its arguments point at, when a bounded wait gives up
// (read by qb200_device_status).
constexpr int STATUS_GEMV_WAIT = 1;
constexpr int STATUS_MATMUL_WAIT = 2;
constexpr int STATUS_SHARD_WAIT = 4;

// A wait gives up after this many clock cycles (about a second at 2 GHz).
constexpr long long WAIT_CYCLES = 2000000000LL;

__device__ __forceinline__ float half_bits_to_float(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---------------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) { asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(20000u)      // the thread may sleep up to this many ns inside the instruction
        : "memory");
    return done != 0;
}

// Waits for the phase with the given parity to complete; gives up after WAIT_CYCLES or as soon as another thread of
// the block has given up (*abort != 0).  Returns false when it gave up: the caller then leaves its loop.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort, int *status, int status_bit)
{
    if (mbar_try_wait(bar, parity)) return true;
    long long start = clock64();
    for (int spins = 0;; spins++) {
        if (mbar_try_wait(bar, parity)) return true;
#ifdef QB_WAIT_SLEEP_NS
        __nanosleep(QB_WAIT_SLEEP_NS);          // a waiting warp should not take issue slots from the working ones
#endif
        if ((spins & 15) != 15) continue;       // the give-up conditions are looked at every 16th poll
        if (*abort) return false;
        if (clock64() - start > WAIT_CYCLES) {
            *abort = 1;
            atomicOr(status, status_bit);
            return false;
        }
    }
}

// The same for a whole warp: lane 0 waits and every lane gets its answer, so the warp stays converged whatever happens
// (warp-wide instructions follow these waits); the shuffle also orders the lanes' later reads after lane 0's acquire.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int *abort, int *status, int status_bit)
{
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort, status, status_bit) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// Every lane polls (one warp instruction a poll, no shuffle afterwards); all lanes see the same barrier, so they leave
// together except in the give-up case, where the abort word makes the stragglers follow within a poll.
__device__ __forceinline__ bool mbar_wait_lanes(uint32_t bar, uint32_t parity, volatile int *abort, int *status, int status_bit)
{
    bool ok = mbar_wait(bar, parity, abort, status, status_bit);
    return __all_sync(0xffffffffu, ok);
}

// ---------------------------------------------------------------------------------- bulk copies (TMA, untiled)
// global -> shared, both addresses 16-byte aligned, bytes a multiple of 16; completion counted on the mbarrier.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// Orders generic-proxy writes to shared memory before later async-proxy (TMA, tcgen05) accesses.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }
// A named barrier of `threads` threads that also tells every one of them whether `mine` held for all.
__device__ __forceinline__ bool named_bar_and(int id, int threads, bool mine)
{
    uint32_t all;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, %2, %3, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(all) : "r"(mine ? 1u : 0u), "r"(id), "r"(threads) : "memory");
    return all != 0;
}

}  // namespace qb
