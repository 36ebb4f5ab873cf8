// Internal launch interface between the C ABI (api.cu) and the kernel files.  Every function returns 0, a negative
// QB200_E_* code or a positive cudaError_t; arguments have been validated by the caller.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

namespace qb {

cudaError_t gemv_init(int sm_count, int max_smem, int *status);
void gemv_set_device_limits(int sm_count, int max_smem);
size_t gemv_scratch_bytes(int cols);
// y_blocks (optional) = y again as fmt_y blocks (Q8_0 / Q4_0), encoded in the same launch
int gemv_launch(int fmt_a, int fmt_x, const void *a, const void *x, float *y, int32_t *sums, int fmt_y, void *y_blocks, int rows,
                int cols, void *scratch, cudaStream_t stream);
// forgets what earlier launches touched: the next call orders itself after everything in its stream
void gemv_forget_history();
int gemv_launch_noalloc(int fmt_a, int fmt_x, const void *a, const void *x, float *y, int rows, int cols, cudaStream_t stream);
int gemv_noalloc_status(int *value);
void gemv_describe(int fmt_a, int rows, int cols, int *out9);

int encode_launch(int fmt, const float *lanes, void *blocks, int64_t n, cudaStream_t stream);
int decode_launch(int fmt, const void *blocks, float *lanes, int64_t n, cudaStream_t stream);

cudaError_t matmul_init(int sm_count, int max_smem, int *status);
size_t matmul_workspace_bytes(int fmt_a, int fmt_b, int m, int n, int k);
int matmul_launch(int fmt_a, int fmt_b, const void *a, const void *b, float *c, int32_t *sums, int m, int n, int k, void *workspace,
                  cudaStream_t stream);

}  // namespace qb
