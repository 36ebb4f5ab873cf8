// Internal launch interface between the C ABI (api.cu) and the kernel files.  Every function returns 0, a negative
// QB200_E_* code or a positive cudaError_t; arguments have been validated by the caller.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/qiyas_b200.h"

namespace qb {

// The sharded gemv's output exchange (world = 0: none).  A rank's y is a slice of the whole output vector; `out[w]` is
// where that slice starts in rank w's copy of the whole vector, as this GPU addresses it (peer-mapped memory; null for
// this rank itself, whose copy y already is), `flag[w]` the word of rank w's flag array that belongs to this rank.  When
// the last block of the grid has published its rows, `epoch` is stored to every flag.
struct GemvPublish {
    float *out[QB200_SHARD_MAX];
    unsigned int *flag[QB200_SHARD_MAX];
    unsigned int *counter;        // blocks of this grid that have published (device-local, returns to zero)
    unsigned int *epoch_counter;  // this rank's count of published calls (device-local), used when epoch is 0
    int world;
    unsigned int epoch;           // the value stored to the flags; 0: the next value of epoch_counter
    // optional: x is the output of an earlier exchange; the consumers wait (bounded) for its flags before they read x
    const unsigned int *wait_flags;   // this rank's flag array of that exchange (null: no wait)
    unsigned int wait_epoch;          // the epoch to wait for; 0: that exchange's count of published calls
    long long wait_limit;             // clock cycles
};

cudaError_t gemv_init(int sm_count, int max_smem, int *status);
// y_blocks (optional) = y again as fmt_y blocks (Q8_0 / Q4_0), encoded in the same launch
// publish (optional) = a GemvPublish (host memory, copied into the launch): the launch also stores y into the other GPUs' copies of it
int gemv_launch(int fmt_a, int fmt_x, const void *a, const void *x, float *y, int32_t *sums, int fmt_y, void *y_blocks, int rows,
                int cols, cudaStream_t stream, const void *publish = nullptr);
// forgets what earlier launches touched: the next call orders itself after everything in its stream
void gemv_forget_history();
// the stream's newest launch touches memory the history cannot describe and has itself waited for everything before it:
// the next gemv on that stream waits for it (by griddepcontrol.wait)
void gemv_history_everything(cudaStream_t stream);
int gemv_launch_noalloc(int fmt_a, int fmt_x, const void *a, const void *x, float *y, int rows, int cols, cudaStream_t stream);
int gemv_noalloc_status(int *value);

// The sharded gemv (shard.cu): rows [first, first + count) of a rows_total-row product on this rank, published to the peers.
cudaError_t shard_init(int *status);
// after: optional peers of the exchange that produced x (waited for inside the kernel), with its epoch and limit
int shard_gemv(int fmt_a, int fmt_x, const void *a_shard, const void *x, int rows_total, int cols, const void *peers, unsigned int epoch,
               const void *after, unsigned int after_epoch, long long limit_cycles, cudaStream_t stream);
int shard_wait(const void *peers, unsigned int epoch, long long limit_cycles, cudaStream_t stream);
// The sharded A.B^T: rows [first, first + count) of B on this rank give columns [first, first + count) of the m x n_total C,
// stored into every rank's copy (peers->out[w] = rank w's C).  b_packed: null, or the shard as matmul_prepack_b left it.
int shard_matmul(int fmt_a, int fmt_b, const void *a, const void *b_shard, const void *b_packed, int m, int n_total, int k, const void *peers,
                 unsigned int epoch, void *workspace, cudaStream_t stream);

int encode_launch(int fmt, const float *lanes, void *blocks, int64_t n, cudaStream_t stream);
int decode_launch(int fmt, const void *blocks, float *lanes, int64_t n, cudaStream_t stream);

cudaError_t matmul_init(int sm_count, int max_smem, int *status);
// `count` products in one call: operands stride_a / stride_b values apart (0: the same operand for every product;
// else whole blocks), results stride_c values apart.  One product: {1, 0, 0, 0}.
struct MatmulBatch { int count; long long stride_a, stride_b, stride_c; };
// scratch of one call: packed A of every product, then packed B of every distinct one (none when B comes prepacked)
size_t matmul_workspace_bytes(int fmt_b, int m, int n, int k, const MatmulBatch &batch, bool b_prepacked);
// B as matmul_prepack_b lays it (the layout does not depend on m)
size_t matmul_prepacked_bytes(int fmt_b, int n, int k);
int matmul_prepack_b(int fmt_b, const void *b, int n, int k, void *packed, cudaStream_t stream);
// b_packed: null, or B as matmul_prepack_b left it (then `b` is not read); c_blocks: null, or C again as blocks of fmt_c
// ldc: values from a row of C to the next (0: n); publish (optional, one product, lanes only) = a GemvPublish whose out[w]
// is where this call's C starts in rank w's copy of a wider matrix of the same ldc: the launch stores C there as well
int matmul_launch(int fmt_a, int fmt_b, const void *a, const void *b, const void *b_packed, float *c, int32_t *sums, int fmt_c,
                  void *c_blocks, int m, int n, int k, const MatmulBatch &batch, void *workspace, cudaStream_t stream, int ldc = 0,
                  const void *publish = nullptr);

// clock cycles a tcgen05.mma kind::i8 (M 128, N 128, K 32) takes on one multiprocessor, measured now
int matmul_mma_rate(double *cycles_per_mma, cudaStream_t stream);


}  // namespace qb
