// N-row sharding of a product across the GPUs of one box: the shard plan, the sharded gemv with its fused output
// exchange (the gemv kernel's publishing variant, gemv.cu), the bounded wait for the peers' flags, and the CUDA IPC
// helpers the one-process-per-GPU model needs.  The reference is single-device (src/Gpu.cs:94-96): nothing here
// replaces reference code; it is the parallel strategy the path's multi-GPU configuration asks for.
#include "common.cuh"
#include "launch.h"

namespace qb {

// blocks of a publishing grid that have finished (one publishing launch a device is in flight at a time)
static __device__ unsigned int g_publish_counter;
static unsigned int *g_publish_counter_ptr = nullptr;
static int *g_shard_status = nullptr;

cudaError_t shard_init(int *status)
{
    g_shard_status = status;
    void *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_publish_counter);
    if (e) return e;
    g_publish_counter_ptr = (unsigned int *)ptr;
    return cudaMemset(ptr, 0, sizeof(unsigned int));
}

// A rank without rows still owes its peers its flag.
__global__ void shard_flag_kernel(GemvPublish pub)
{
    __shared__ unsigned int epoch;
    if (threadIdx.x == 0) epoch = pub.epoch ? pub.epoch : atomicAdd(pub.epoch_counter, 1u) + 1u;
    __syncthreads();
    if (threadIdx.x < pub.world) {
        unsigned int *f = pub.flag[threadIdx.x];
        if (f) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
    }
}

// Thread w waits until word w of this rank's flag array has reached `epoch` (the words only grow), for at most `limit`
// cycles; then it gives up, sets the status bit and returns.  The acquire pairs with the publisher's release: what
// follows this kernel in the stream sees every row the peers stored.
// The kernel is launched as a programmatic dependent of the publishing gemv before it: it is resident and polling while
// that gemv still runs (the peers' flags do not depend on it), lets the kernel after it be scheduled at once, and only at
// its end waits for the gemv's completion, so that whatever follows it in the stream, waiting for this kernel, has
// waited for both the peers' rows and this rank's own.
__global__ void shard_wait_kernel(unsigned int *flags, int world, unsigned int epoch, long long limit, int *status)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ unsigned int counted;
    if (epoch == 0) {           // the wait's number is counted on the device, as the publisher's is
        if (threadIdx.x == 0) counted = atomicAdd(flags + QB200_SHARD_MAX + 1, 1u) + 1u;
        __syncthreads();
        epoch = counted;
    }
    if (threadIdx.x < world) {
        const unsigned int *f = flags + threadIdx.x;
        const long long start = clock64();
        for (;;) {
            unsigned int v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if ((int)(v - epoch) >= 0) break;
            if (clock64() - start > limit) {
                atomicOr(status, STATUS_SHARD_WAIT);
                break;
            }
            __nanosleep(50);
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

int shard_gemv(int fmt_a, int fmt_x, const void *a_shard, const void *x, int rows_total, int cols, const void *peers_v, unsigned int epoch,
               const void *after_v, unsigned int after_epoch, long long limit_cycles, cudaStream_t stream)
{
    const qb200_shard_peers_t *peers = (const qb200_shard_peers_t *)peers_v, *after = (const qb200_shard_peers_t *)after_v;
    int first = 0, count = 0;
    qb200_shard_range(rows_total, peers->world, peers->rank, &first, &count);
    GemvPublish pub;
    memset(&pub, 0, sizeof pub);
    pub.world = peers->world;
    pub.epoch = epoch;
    pub.counter = g_publish_counter_ptr;
    pub.epoch_counter = peers->flags[peers->rank] + QB200_SHARD_MAX;
    for (int w = 0; w < peers->world; w++) {
        pub.out[w] = w == peers->rank ? nullptr : peers->out[w] + first;
        pub.flag[w] = peers->flags[w] + peers->rank;
    }
    if (after) {
        pub.wait_flags = after->flags[after->rank];
        pub.wait_epoch = after_epoch;
        pub.wait_limit = limit_cycles > 0 ? limit_cycles : WAIT_CYCLES;
    }
    if (count == 0) {
        // a rank without rows: its flag, after the wait its peers' kernels make inside (so that its counters keep step)
        if (after) {
            int rc = shard_wait(after_v, after_epoch, limit_cycles, stream);
            if (rc) return rc;
        }
        shard_flag_kernel<<<1, 32, 0, stream>>>(pub);
        return (int)cudaGetLastError();
    }
    return gemv_launch(fmt_a, fmt_x, a_shard, x, peers->out[peers->rank] + first, nullptr, 0, nullptr, count, cols, stream, &pub);
}

// The sharded A.B^T.  C's columns are B's rows, so rank r computes the column block [first, first + count) of the m x
// n_total C and the product kernel's epilogue stores it, row stride n_total, into every rank's copy of C; the flags and
// the wait are the gemv's.
int shard_matmul(int fmt_a, int fmt_b, const void *a, const void *b_shard, const void *b_packed, int m, int n_total, int k, const void *peers_v,
                 unsigned int epoch, void *workspace, cudaStream_t stream)
{
    const qb200_shard_peers_t *peers = (const qb200_shard_peers_t *)peers_v;
    int first = 0, count = 0;
    qb200_shard_range(n_total, peers->world, peers->rank, &first, &count);
    GemvPublish pub;
    memset(&pub, 0, sizeof pub);
    pub.world = peers->world;
    pub.epoch = epoch;
    pub.counter = g_publish_counter_ptr;
    pub.epoch_counter = peers->flags[peers->rank] + QB200_SHARD_MAX;
    for (int w = 0; w < peers->world; w++) {
        pub.out[w] = w == peers->rank ? nullptr : peers->out[w] + first;
        pub.flag[w] = peers->flags[w] + peers->rank;
    }
    if (count == 0) {
        shard_flag_kernel<<<1, 32, 0, stream>>>(pub);
        return (int)cudaGetLastError();
    }
    const MatmulBatch one = {1, 0, 0, 0};
    return matmul_launch(fmt_a, fmt_b, a, b_shard, b_packed, peers->out[peers->rank] + first, nullptr, 0, nullptr, m, count, k, one, workspace, stream,
                         n_total, &pub);
}

int shard_wait(const void *peers_v, unsigned int epoch, long long limit_cycles, cudaStream_t stream)
{
    const qb200_shard_peers_t *peers = (const qb200_shard_peers_t *)peers_v;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, shard_wait_kernel, peers->flags[peers->rank], peers->world, epoch,
                                       limit_cycles > 0 ? limit_cycles : WAIT_CYCLES, g_shard_status);
    // everything launched so far on this stream is complete once this kernel is: the next gemv may wait for it by
    // griddepcontrol.wait alone
    if (!e) gemv_history_everything(stream);
    return (int)e;
}

}  // namespace qb
