// placeholder until the tcgen05 product lands
#include "common.cuh"
#include "launch.h"
namespace qb {
cudaError_t matmul_init(int, int, int *) { return cudaSuccess; }
size_t matmul_workspace_bytes(int, int, int, int, int) { return 256; }
int matmul_launch(int, int, const void *, const void *, float *, int32_t *, int, int, int, void *, cudaStream_t) { return QB200_E_DEVICE; }
}
