// The C ABI of libqiyas_b200.so (declared in include/qiyas_b200.h): argument checks in the reference's terms,
// error text, device binding, and the launches.  No entry point has a CPU path: on a machine without an sm_100 device
// qb200_init fails and every other call returns QB200_E_DEVICE.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"
#include "launch.h"

namespace {

thread_local char t_error[512] = "";
bool g_ready = false;
qb200_caps_t g_caps;

// grow-only device buffers the library keeps: staging for the host-buffer calls, scratch for A.B^T without a workspace
struct Kept {
    void *ptr = nullptr;
    size_t bytes = 0;
};
Kept g_stage_a, g_stage_x, g_stage_y, g_scratch;
int *g_status = nullptr;      // device word the kernels OR their STATUS_* bits into
int g_bound = -1;             // the device the kept buffers and the status word live on

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof t_error, fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char *what)
{
    snprintf(t_error, sizeof t_error, "%s: %s", what, cudaGetErrorString(e));
    return (int)e;
}

int finish(int rc, const char *what)
{
    if (rc > 0) return cuda_fail((cudaError_t)rc, what);
    if (rc == QB200_E_LIMIT) return fail(rc, "%s: the shape is beyond what the kernel's shared memory takes", what);
    if (rc < 0) return fail(rc, "%s: argument error %d", what, rc);
    return 0;
}

// A launch that is not a gemv: the gemv's record of launches in flight (which lets an unrelated gemv start beside its
// predecessors) does not describe what this one touches, so the next gemv on the stream orders itself after everything.
int finish_other(int rc, const char *what, void *stream)
{
    if (rc == 0) qb::gemv_history_everything((cudaStream_t)stream);
    return finish(rc, what);
}

const char *fmt_name(int fmt)
{
    switch (fmt) {
    case QB200_Q8_0: return "q8_0";
    case QB200_Q4_0: return "q4_0";
    case QB200_Q4_K: return "q4_k";
    case QB200_Q6_K: return "q6_k";
    case QB200_F32: return "f32";
    default: return "?";
    }
}

int keep(Kept &k, size_t bytes)
{
    if (k.bytes >= bytes) return 0;
    if (k.ptr) cudaFree(k.ptr);
    k.ptr = nullptr;
    k.bytes = 0;
    size_t want = bytes + bytes / 4 + 4096;
    cudaError_t e = cudaMalloc(&k.ptr, want);
    if (e) return cuda_fail(e, "cudaMalloc");
    k.bytes = want;
    return 0;
}

void release_kept()
{
    Kept *all[] = { &g_stage_a, &g_stage_x, &g_stage_y, &g_scratch };
    for (Kept *k : all) {
        if (k->ptr) cudaFree(k->ptr);
        *k = Kept();
    }
    if (g_status) cudaFree(g_status);
    g_status = nullptr;
}

int check_gemv(int fmt_a, int fmt_x, const void *a, const void *x, const float *y, int rows, int cols)
{
    if (!g_ready) return fail(QB200_E_DEVICE, "qb200_init has not succeeded");
    const int bv = qb::block_values(fmt_a);
    if (!bv) return fail(QB200_E_FORMAT, "%s: the block product takes Q8_0, Q4_0, Q4_K or Q6_K rows", fmt_name(fmt_a));
    const bool k_quant = fmt_a == QB200_Q4_K || fmt_a == QB200_Q6_K;
    if (!(fmt_x == QB200_Q8_0 || fmt_x == QB200_F32 || (fmt_x == QB200_Q4_0 && !k_quant)))
        return fail(QB200_E_FORMAT, "%s x %s: x comes in Q8_0 or f32 (or Q4_0 against Q8_0 / Q4_0 rows)", fmt_name(fmt_a), fmt_name(fmt_x));
    if (rows < 0 || cols <= 0 || cols % bv != 0)
        return fail(QB200_E_SHAPE, "%s: the block product takes columns in whole blocks of %d (rows %d, cols %d)", fmt_name(fmt_a), bv, rows, cols);
    const int widest = fmt_a == QB200_Q6_K ? 32768 : 65536;
    if (cols > widest) return fail(QB200_E_LIMIT, "cols %d: at most %d columns in %s rows", cols, widest, fmt_name(fmt_a));
    if (rows == 0) return 0;
    if (!a || !x || !y) return fail(QB200_E_POINTER, "null operand");
    if (((uintptr_t)a & 1) || ((uintptr_t)x & (fmt_x == QB200_F32 ? 3 : 1)) || ((uintptr_t)y & 3)) return fail(QB200_E_POINTER, "misaligned operand");
    return 0;
}

int check_matmul(int fmt_a, int fmt_b, const void *a, const void *b, const float *c, int m, int n, int k)
{
    if (!g_ready) return fail(QB200_E_DEVICE, "qb200_init has not succeeded");
    if ((fmt_a != QB200_Q8_0 && fmt_a != QB200_Q4_0) || (fmt_b != QB200_Q8_0 && fmt_b != QB200_Q4_0 && fmt_b != QB200_Q4_K && fmt_b != QB200_Q6_K))
        return fail(QB200_E_FORMAT, "%s x %s: the block product takes Q8_0 or Q4_0 (B also Q4_K, Q6_K) with k in whole blocks", fmt_name(fmt_a), fmt_name(fmt_b));
    if (m <= 0 || n <= 0 || k <= 0 || k % qb::block_values(fmt_b) != 0)
        return fail(QB200_E_SHAPE, "the block product takes k in whole blocks of both operands (m %d, n %d, k %d)", m, n, k);
    if (!g_caps.tcgen05) return fail(QB200_E_DEVICE, "the block product needs the s8 tensor instruction (tcgen05, sm_100)");
    if (!a || !b || !c) return fail(QB200_E_POINTER, "null operand");
    if (((uintptr_t)a & 1) || ((uintptr_t)b & 1) || ((uintptr_t)c & 3)) return fail(QB200_E_POINTER, "misaligned operand");
    return 0;
}

}  // namespace

extern "C" {

int qb200_init(int device)
{
    g_ready = false;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e) return cuda_fail(e, "cudaGetDeviceCount");
    if (device < 0 || device >= count) return fail(QB200_E_DEVICE, "device %d of %d", device, count);
    if ((e = cudaSetDevice(device))) return cuda_fail(e, "cudaSetDevice");
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device))) return cuda_fail(e, "cudaGetDeviceProperties");
    memset(&g_caps, 0, sizeof g_caps);
    g_caps.device = device;
    g_caps.sm_major = prop.major;
    g_caps.sm_minor = prop.minor;
    g_caps.sm_count = prop.multiProcessorCount;
    g_caps.tcgen05 = prop.major == 10 ? 1 : 0;
    g_caps.max_shared_bytes = (int)prop.sharedMemPerBlockOptin;
    g_caps.l2_bytes = prop.l2CacheSize;
    g_caps.global_bytes = (int64_t)prop.totalGlobalMem;
    if (prop.major != 10) return fail(QB200_E_DEVICE, "device %d is sm_%d%d: the kernels are built for sm_100a only", device, prop.major, prop.minor);
    // What an earlier binding kept lives on its device: released there before this one takes over (a second qb200_init of
    // the same device keeps it all).
    if (g_bound >= 0 && g_bound != device) {
        cudaSetDevice(g_bound);
        release_kept();
        if ((e = cudaSetDevice(device))) return cuda_fail(e, "cudaSetDevice");
    }
    if (!g_status) {
        if ((e = cudaMalloc((void **)&g_status, 256))) return cuda_fail(e, "cudaMalloc status");
        if ((e = cudaMemset(g_status, 0, 256))) return cuda_fail(e, "cudaMemset status");
    }
    g_bound = device;
    if ((e = qb::gemv_init(g_caps.sm_count, g_caps.max_shared_bytes, g_status))) return cuda_fail(e, "gemv attributes");
    if ((e = qb::matmul_init(g_caps.sm_count, g_caps.max_shared_bytes, g_status))) return cuda_fail(e, "matmul attributes");
    if ((e = qb::shard_init(g_status))) return cuda_fail(e, "shard set-up");
    g_ready = true;
    t_error[0] = 0;
    return 0;
}

int qb200_caps(qb200_caps_t *out)
{
    if (!g_ready) return fail(QB200_E_DEVICE, "qb200_init has not succeeded");
    if (!out) return fail(QB200_E_POINTER, "null caps");
    *out = g_caps;
    return 0;
}

const char *qb200_last_error(void) { return t_error; }

int qb200_block_product_available(void) { return g_ready && g_caps.tcgen05 ? 1 : 0; }

const char *qb200_lane_name(int op, int fmt_a)
{
    (void)fmt_a;
    return op == QB200_OP_MATMUL ? "s8 tcgen05 blocks" : "s8dp blocks";
}

int qb200_device_status(int *status)
{
    if (!g_ready) return fail(QB200_E_DEVICE, "qb200_init has not succeeded");
    cudaError_t e = cudaDeviceSynchronize();
    if (e) return cuda_fail(e, "cudaDeviceSynchronize");
    int value = 0, zero = 0;
    if ((e = cudaMemcpy(&value, g_status, sizeof value, cudaMemcpyDeviceToHost))) return cuda_fail(e, "status read");
    if (value && (e = cudaMemcpy(g_status, &zero, sizeof zero, cudaMemcpyHostToDevice))) return cuda_fail(e, "status clear");
    if (status) *status = value;
    return 0;
}

int qb200_gemv_blocks(int fmt_a, int fmt_x, const void *a, const void *x, float *y, int rows, int cols, void *stream)
{
    int rc = check_gemv(fmt_a, fmt_x, a, x, y, rows, cols);
    if (rc) return rc;
    return finish(qb::gemv_launch(fmt_a, fmt_x, a, x, y, nullptr, 0, nullptr, rows, cols, (cudaStream_t)stream), "gemv_blocks");
}

// The block branch of the public gemv (reference src/GpuOps.cs:277-285) in one launch: f32 lanes and their `Back`.
int qb200_gemv_blocks_back(int fmt_a, int fmt_x, const void *a, const void *x, float *y_lanes, int fmt_y, void *y_blocks, int rows,
                           int cols, void *stream)
{
    int rc = check_gemv(fmt_a, fmt_x, a, x, y_lanes, rows, cols);
    if (rc) return rc;
    if (fmt_y != QB200_Q8_0 && fmt_y != QB200_Q4_0)
        return fail(QB200_E_FORMAT, "%s: the gemv encodes its output as Q8_0 or Q4_0; use qb200_encode for the others", fmt_name(fmt_y));
    if (rows > 0 && (!y_blocks || ((uintptr_t)y_blocks & 1))) return fail(QB200_E_POINTER, "null or misaligned y_blocks");
    return finish(qb::gemv_launch(fmt_a, fmt_x, a, x, y_lanes, nullptr, fmt_y, y_blocks, rows, cols, (cudaStream_t)stream),
                  "gemv_blocks_back");
}

int qb200_gemv_block_sums(int fmt_a, int fmt_x, const void *a, const void *x, float *y, int32_t *sums, int rows, int cols, void *stream)
{
    int rc = check_gemv(fmt_a, fmt_x, a, x, y, rows, cols);
    if (rc) return rc;
    if (rows > 0 && (!sums || ((uintptr_t)sums & 3))) return fail(QB200_E_POINTER, "null or misaligned sums");
    return finish(qb::gemv_launch(fmt_a, fmt_x, a, x, y, sums, 0, nullptr, rows, cols, (cudaStream_t)stream), "gemv_block_sums");
}

int qb200_gemv_blocks_host(int fmt_a, int fmt_x, const void *a, const void *x, float *y, int rows, int cols)
{
    if (!g_ready) return fail(QB200_E_DEVICE, "qb200_init has not succeeded");
    const int bv = qb::block_values(fmt_a);
    if (!bv || rows < 0 || cols <= 0 || cols % bv) return fail(QB200_E_SHAPE, "the block product takes columns in whole blocks");
    if (rows == 0) return 0;
    if (!a || !x || !y) return fail(QB200_E_POINTER, "null operand");
    const size_t a_bytes = (size_t)rows * (cols / bv) * qb::block_bytes(fmt_a);
    const size_t x_bytes = fmt_x == QB200_F32 ? (size_t)cols * 4 : (size_t)(cols / 32) * qb::block_bytes(fmt_x);
    int rc;
    if ((rc = keep(g_stage_a, a_bytes)) || (rc = keep(g_stage_x, x_bytes)) || (rc = keep(g_stage_y, (size_t)rows * 4))) return rc;
    cudaError_t e;
    if ((e = cudaMemcpyAsync(g_stage_a.ptr, a, a_bytes, cudaMemcpyHostToDevice, 0))) return cuda_fail(e, "upload a");
    if ((e = cudaMemcpyAsync(g_stage_x.ptr, x, x_bytes, cudaMemcpyHostToDevice, 0))) return cuda_fail(e, "upload x");
    if ((rc = qb200_gemv_blocks(fmt_a, fmt_x, g_stage_a.ptr, g_stage_x.ptr, (float *)g_stage_y.ptr, rows, cols, nullptr))) return rc;
    if ((e = cudaMemcpyAsync(y, g_stage_y.ptr, (size_t)rows * 4, cudaMemcpyDeviceToHost, 0))) return cuda_fail(e, "download y");
    if ((e = cudaStreamSynchronize(0))) return cuda_fail(e, "synchronize");
    return 0;
}

// The gemv with its scratch in a static device array (see the header): no allocation, no qb200_init needed.
int qb200_gemv_blocks_noalloc(int fmt_a, int fmt_x, const void *a, const void *x, float *y, int rows, int cols, void *stream)
{
    const int bv = qb::block_values(fmt_a);
    if (!bv) return fail(QB200_E_FORMAT, "%s: the block product takes Q8_0, Q4_0, Q4_K or Q6_K rows", fmt_name(fmt_a));
    const bool k_quant = fmt_a == QB200_Q4_K || fmt_a == QB200_Q6_K;
    if (!(fmt_x == QB200_Q8_0 || fmt_x == QB200_F32 || (fmt_x == QB200_Q4_0 && !k_quant)))
        return fail(QB200_E_FORMAT, "%s x %s: x comes in Q8_0 or f32 (or Q4_0 against Q8_0 / Q4_0 rows)", fmt_name(fmt_a), fmt_name(fmt_x));
    if (rows < 0 || cols <= 0 || cols % bv != 0)
        return fail(QB200_E_SHAPE, "%s: the block product takes columns in whole blocks of %d (rows %d, cols %d)", fmt_name(fmt_a), bv, rows, cols);
    if (cols > QB200_NOALLOC_MAX_COLS)
        return fail(QB200_E_LIMIT, "cols %d: the no-allocation gemv holds x for at most %d columns in its static scratch; use qb200_gemv_blocks",
                    cols, QB200_NOALLOC_MAX_COLS);
    if (rows == 0) return 0;
    if (!a || !x || !y) return fail(QB200_E_POINTER, "null operand");
    if (((uintptr_t)a & 1) || ((uintptr_t)x & (fmt_x == QB200_F32 ? 3 : 1)) || ((uintptr_t)y & 3)) return fail(QB200_E_POINTER, "misaligned operand");
    const int rc = qb::gemv_launch_noalloc(fmt_a, fmt_x, a, x, y, rows, cols, (cudaStream_t)stream);
    if (rc == QB200_E_DEVICE) return fail(rc, "gemv_blocks_noalloc: the current device is not sm_100");
    return finish(rc, "gemv_blocks_noalloc");
}

int qb200_gemv_noalloc_status(int *status)
{
    if (!status) return fail(QB200_E_POINTER, "null status");
    return finish(qb::gemv_noalloc_status(status), "gemv_noalloc_status");
}

// The scratch a product call needs, and where it comes from: the caller's workspace, or the buffer the library keeps.
static int take_workspace(void *&workspace, size_t workspace_bytes, size_t need)
{
    if (workspace) {
        if (workspace_bytes < need) return fail(QB200_E_WORKSPACE, "workspace of %zu bytes, %zu needed", workspace_bytes, need);
        if ((uintptr_t)workspace & 255) return fail(QB200_E_WORKSPACE, "workspace not 256-byte aligned");
        return 0;
    }
    int rc = keep(g_scratch, need);
    if (rc) return rc;
    workspace = g_scratch.ptr;
    return 0;
}

static const qb::MatmulBatch ONE = { 1, 0, 0, 0 };

size_t qb200_matmul_workspace_bytes(int fmt_a, int fmt_b, int m, int n, int k)
{
    (void)fmt_a;
    if (m <= 0 || n <= 0 || k <= 0 || !qb::block_values(fmt_b) || k % qb::block_values(fmt_b)) return 0;
    return qb::matmul_workspace_bytes(fmt_b, m, n, k, ONE, false);
}

int qb200_matmul_blocks(int fmt_a, int fmt_b, const void *a, const void *b, float *c, int m, int n, int k, void *workspace,
                        size_t workspace_bytes, void *stream)
{
    int rc = check_matmul(fmt_a, fmt_b, a, b, c, m, n, k);
    if (rc) return rc;
    // a few rows of A: the weights stream once past activations held on the chip, no re-laying, no tensor tile of padding
    if ((rc = take_workspace(workspace, workspace_bytes, qb::matmul_workspace_bytes(fmt_b, m, n, k, ONE, false)))) return rc;
    return finish_other(qb::matmul_launch(fmt_a, fmt_b, a, b, nullptr, c, nullptr, 0, nullptr, m, n, k, ONE, workspace, (cudaStream_t)stream), "matmul_blocks", stream);
}

// GpuOps.MatMulViewBlocks<TN> (reference src/MatMulBlocks.cs:414-424) in one product launch: the f32 lanes and their `Back`.
int qb200_matmul_blocks_back(int fmt_a, int fmt_b, const void *a, const void *b, float *c_lanes, int fmt_c, void *c_blocks, int m, int n,
                             int k, void *workspace, size_t workspace_bytes, void *stream)
{
    int rc = check_matmul(fmt_a, fmt_b, a, b, c_lanes, m, n, k);
    if (rc) return rc;
    if (fmt_c != QB200_Q8_0 && fmt_c != QB200_Q4_0)
        return fail(QB200_E_FORMAT, "%s: the product encodes its output as Q8_0 or Q4_0; use qb200_encode for the others", fmt_name(fmt_c));
    if (!c_blocks || ((uintptr_t)c_blocks & 1)) return fail(QB200_E_POINTER, "null or misaligned c_blocks");
    if ((rc = take_workspace(workspace, workspace_bytes, qb::matmul_workspace_bytes(fmt_b, m, n, k, ONE, false)))) return rc;
    // a block of C (32 consecutive values of the row-major m x n array) lies inside one row only when n is whole blocks,
    // and the encoding threads read the lanes 16 bytes at a time; otherwise `Back` is the launch of its own it is in the reference
    const bool fused = n % 32 == 0 && ((uintptr_t)c_lanes & 15) == 0;
    rc = qb::matmul_launch(fmt_a, fmt_b, a, b, nullptr, c_lanes, nullptr, fmt_c, fused ? c_blocks : nullptr, m, n, k, ONE, workspace, (cudaStream_t)stream);
    if (rc == 0 && !fused) rc = qb::encode_launch(fmt_c, c_lanes, c_blocks, (int64_t)m * n, (cudaStream_t)stream);
    return finish_other(rc, "matmul_blocks_back", stream);
}

size_t qb200_matmul_prepacked_bytes(int fmt_b, int n, int k)
{
    if (n <= 0 || k <= 0 || !qb::block_values(fmt_b) || k % qb::block_values(fmt_b)) return 0;
    return qb::matmul_prepacked_bytes(fmt_b, n, k);
}

int qb200_matmul_prepack(int fmt_b, const void *b, int n, int k, void *packed, size_t packed_bytes, void *stream)
{
    if (!g_ready) return fail(QB200_E_DEVICE, "qb200_init has not succeeded");
    if (!qb::block_values(fmt_b)) return fail(QB200_E_FORMAT, "%s: not a block format", fmt_name(fmt_b));
    if (n <= 0 || k <= 0 || k % qb::block_values(fmt_b)) return fail(QB200_E_SHAPE, "k in whole blocks of B (n %d, k %d)", n, k);
    if (!b || ((uintptr_t)b & 1)) return fail(QB200_E_POINTER, "null or misaligned operand");
    if (!packed || ((uintptr_t)packed & 255)) return fail(QB200_E_WORKSPACE, "the packed operand needs a 256-byte aligned buffer");
    const size_t need = qb::matmul_prepacked_bytes(fmt_b, n, k);
    if (packed_bytes < need) return fail(QB200_E_WORKSPACE, "packed buffer of %zu bytes, %zu needed", packed_bytes, need);
    return finish_other(qb::matmul_prepack_b(fmt_b, b, n, k, packed, (cudaStream_t)stream), "matmul_prepack", stream);
}

size_t qb200_matmul_prepacked_workspace_bytes(int fmt_a, int fmt_b, int m, int k)
{
    (void)fmt_a;
    if (m <= 0 || k <= 0 || !qb::block_values(fmt_b) || k % qb::block_values(fmt_b)) return 0;
    return qb::matmul_workspace_bytes(fmt_b, m, 1, k, ONE, true);
}

int qb200_matmul_blocks_prepacked(int fmt_a, int fmt_b, const void *a, const void *b_packed, float *c, int m, int n, int k,
                                  void *workspace, size_t workspace_bytes, void *stream)
{
    int rc = check_matmul(fmt_a, fmt_b, a, b_packed, c, m, n, k);
    if (rc) return rc;
    if ((uintptr_t)b_packed & 255) return fail(QB200_E_WORKSPACE, "the packed operand is 256-byte aligned");
    if ((rc = take_workspace(workspace, workspace_bytes, qb::matmul_workspace_bytes(fmt_b, m, n, k, ONE, true)))) return rc;
    return finish_other(qb::matmul_launch(fmt_a, fmt_b, a, nullptr, b_packed, c, nullptr, 0, nullptr, m, n, k, ONE, workspace, (cudaStream_t)stream),
                  "matmul_blocks_prepacked", stream);
}

static int check_batch(int fmt_a, int fmt_b, int m, int n, int k, int batch, int64_t stride_a, int64_t stride_b, int64_t stride_c)
{
    if (batch < 1) return fail(QB200_E_SHAPE, "batch %d", batch);
    if (stride_a < 0 || stride_b < 0 || stride_c < 0) return fail(QB200_E_SHAPE, "negative batch stride");
    if (stride_a % qb::block_values(fmt_a) || stride_b % qb::block_values(fmt_b))
        return fail(QB200_E_SHAPE, "a batch's operands start on whole blocks (strides %lld, %lld values)", (long long)stride_a, (long long)stride_b);
    if (batch > 1 && stride_c < (int64_t)m * n) return fail(QB200_E_SHAPE, "the batch's results overlap (stride %lld values, %lld a product)", (long long)stride_c, (long long)m * n);
    (void)k;
    return 0;
}

size_t qb200_matmul_batched_workspace_bytes(int fmt_a, int fmt_b, int m, int n, int k, int batch, int64_t stride_a, int64_t stride_b)
{
    (void)fmt_a;
    if (m <= 0 || n <= 0 || k <= 0 || batch < 1 || !qb::block_values(fmt_b) || k % qb::block_values(fmt_b)) return 0;
    const qb::MatmulBatch bt = { batch, batch > 1 ? stride_a : 0, batch > 1 ? stride_b : 0, 0 };
    return qb::matmul_workspace_bytes(fmt_b, m, n, k, bt, false);
}

// ProductView with Batch > 1 (reference src/Products.cs:15-22) on the block product: every product of the batch in one launch.
int qb200_matmul_blocks_batched(int fmt_a, int fmt_b, const void *a, const void *b, float *c, int m, int n, int k, int batch,
                                int64_t stride_a, int64_t stride_b, int64_t stride_c, void *workspace, size_t workspace_bytes, void *stream)
{
    int rc = check_matmul(fmt_a, fmt_b, a, b, c, m, n, k);
    if (rc) return rc;
    if ((rc = check_batch(fmt_a, fmt_b, m, n, k, batch, stride_a, stride_b, stride_c))) return rc;
    const qb::MatmulBatch bt = { batch, batch > 1 ? stride_a : 0, batch > 1 ? stride_b : 0, batch > 1 ? stride_c : 0 };
    if ((rc = take_workspace(workspace, workspace_bytes, qb::matmul_workspace_bytes(fmt_b, m, n, k, bt, false)))) return rc;
    return finish_other(qb::matmul_launch(fmt_a, fmt_b, a, b, nullptr, c, nullptr, 0, nullptr, m, n, k, bt, workspace, (cudaStream_t)stream),
                  "matmul_blocks_batched", stream);
}

int qb200_matmul_block_sums(int fmt_a, int fmt_b, const void *a, const void *b, float *c, int32_t *sums, int m, int n, int k, void *stream)
{
    int rc = check_matmul(fmt_a, fmt_b, a, b, c, m, n, k);
    if (rc) return rc;
    if (!sums || ((uintptr_t)sums & 3)) return fail(QB200_E_POINTER, "null or misaligned sums");
    const int per = fmt_b == QB200_Q6_K ? 16 : 32;
    if ((int64_t)m * n * (k / per) > (1 << 24)) return fail(QB200_E_LIMIT, "block sums are for small shapes: m*n*(k/%d) at most 2^24", per);
    if ((rc = keep(g_scratch, qb::matmul_workspace_bytes(fmt_b, m, n, k, ONE, false)))) return rc;
    return finish_other(qb::matmul_launch(fmt_a, fmt_b, a, b, nullptr, c, sums, 0, nullptr, m, n, k, ONE, g_scratch.ptr, (cudaStream_t)stream), "matmul_block_sums", stream);
}

int qb200_tensor_rate(double *cycles_per_mma)
{
    if (!g_ready) return fail(QB200_E_DEVICE, "qb200_init has not succeeded");
    if (!g_caps.tcgen05) return fail(QB200_E_DEVICE, "no tcgen05 on this device");
    if (!cycles_per_mma) return fail(QB200_E_POINTER, "null result");
    return finish(qb::matmul_mma_rate(cycles_per_mma, nullptr), "tensor_rate");
}

int qb200_encode(int fmt, const float *lanes, void *blocks, int64_t n, void *stream)
{
    if (!g_ready) return fail(QB200_E_DEVICE, "qb200_init has not succeeded");
    if (!qb::block_values(fmt)) return fail(QB200_E_FORMAT, "%s: not a block format", fmt_name(fmt));
    if (n < 0 || n > 2147483647LL) return fail(QB200_E_SHAPE, "count %lld", (long long)n);
    if (n && (!lanes || !blocks || ((uintptr_t)lanes & 3))) return fail(QB200_E_POINTER, "null or misaligned operand");
    return finish_other(qb::encode_launch(fmt, lanes, blocks, n, (cudaStream_t)stream), "encode", stream);
}

int qb200_decode(int fmt, const void *blocks, float *lanes, int64_t n, void *stream)
{
    if (!g_ready) return fail(QB200_E_DEVICE, "qb200_init has not succeeded");
    if (!qb::block_values(fmt)) return fail(QB200_E_FORMAT, "%s: not a block format", fmt_name(fmt));
    if (n < 0 || n > 2147483647LL) return fail(QB200_E_SHAPE, "count %lld", (long long)n);
    if (n && (!lanes || !blocks || ((uintptr_t)lanes & 3))) return fail(QB200_E_POINTER, "null or misaligned operand");
    return finish_other(qb::decode_launch(fmt, blocks, lanes, n, (cudaStream_t)stream), "decode", stream);
}

int qb200_shard_range(int rows, int world, int rank, int *first, int *count)
{
    if (rows < 0 || world < 1 || rank < 0 || rank >= world) return fail(QB200_E_SHAPE, "rank %d of %d over %d rows", rank, world, rows);
    const int per = (rows + world - 1) / world;
    const int lo = (long long)rank * per < rows ? rank * per : rows, hi = lo + per < rows ? lo + per : rows;
    if (first) *first = lo;
    if (count) *count = hi - lo;
    return 0;
}

static int check_peers(const qb200_shard_peers_t *peers)
{
    if (!g_ready) return fail(QB200_E_DEVICE, "qb200_init has not succeeded");
    if (!peers) return fail(QB200_E_POINTER, "null peers");
    if (peers->world < 1 || peers->world > QB200_SHARD_MAX || peers->rank < 0 || peers->rank >= peers->world)
        return fail(QB200_E_SHAPE, "rank %d of %d (at most %d ranks)", peers->rank, peers->world, QB200_SHARD_MAX);
    for (int w = 0; w < peers->world; w++) {
        if (!peers->out[w] || !peers->flags[w]) return fail(QB200_E_POINTER, "rank %d's output or flags are not mapped", w);
        if (((uintptr_t)peers->out[w] & 15) || ((uintptr_t)peers->flags[w] & 3)) return fail(QB200_E_POINTER, "rank %d's output or flags are misaligned", w);
    }
    return 0;
}

int qb200_shard_gemv(int fmt_a, int fmt_x, const void *a_shard, const void *x, int rows_total, int cols, const qb200_shard_peers_t *peers,
                     unsigned int epoch, void *stream)
{
    int rc = check_peers(peers);
    if (rc) return rc;
    int first = 0, count = 0;
    if ((rc = qb200_shard_range(rows_total, peers->world, peers->rank, &first, &count))) return rc;
    // the slice as an ordinary gemv: formats, whole blocks, limits, alignment (a rank without rows has nothing to check but x)
    if ((rc = check_gemv(fmt_a, fmt_x, count ? a_shard : x, x, peers->out[peers->rank] + first, count, cols))) return rc;
    return finish(qb::shard_gemv(fmt_a, fmt_x, a_shard, x, rows_total, cols, peers, epoch, nullptr, 0, 0, (cudaStream_t)stream), "shard_gemv");
}

int qb200_shard_matmul(int fmt_a, int fmt_b, const void *a, const void *b_shard, const void *b_shard_packed, int m, int n_total, int k,
                       const qb200_shard_peers_t *peers, unsigned int epoch, void *workspace, size_t workspace_bytes, void *stream)
{
    int rc = check_peers(peers);
    if (rc) return rc;
    int first = 0, count = 0;
    if ((rc = qb200_shard_range(n_total, peers->world, peers->rank, &first, &count))) return rc;
    if (count) {
        // the column block as an ordinary product: formats, whole blocks, limits, alignment
        const void *b = b_shard_packed ? b_shard_packed : b_shard;
        if ((rc = check_matmul(fmt_a, fmt_b, a, b, peers->out[peers->rank] + first, m, count, k))) return rc;
        if ((uintptr_t)b_shard_packed & 255) return fail(QB200_E_WORKSPACE, "the packed operand is 256-byte aligned");
        if ((rc = take_workspace(workspace, workspace_bytes, qb::matmul_workspace_bytes(fmt_b, m, count, k, ONE, b_shard_packed != nullptr)))) return rc;
    }
    return finish_other(qb::shard_matmul(fmt_a, fmt_b, a, b_shard, b_shard_packed, m, n_total, k, peers, epoch, workspace, (cudaStream_t)stream), "shard_matmul", stream);
}

int qb200_shard_gemv_after(int fmt_a, int fmt_x, const void *a_shard, const void *x, int rows_total, int cols, const qb200_shard_peers_t *peers,
                           unsigned int epoch, const qb200_shard_peers_t *after, unsigned int after_epoch, long long limit_cycles, void *stream)
{
    int rc = check_peers(peers);
    if (rc || (rc = check_peers(after))) return rc;
    if (after->world != peers->world || after->rank != peers->rank) return fail(QB200_E_SHAPE, "the two exchanges must be between the same ranks");
    int first = 0, count = 0;
    if ((rc = qb200_shard_range(rows_total, peers->world, peers->rank, &first, &count))) return rc;
    if ((rc = check_gemv(fmt_a, fmt_x, count ? a_shard : x, x, peers->out[peers->rank] + first, count, cols))) return rc;
    return finish(qb::shard_gemv(fmt_a, fmt_x, a_shard, x, rows_total, cols, peers, epoch, after, after_epoch, limit_cycles, (cudaStream_t)stream),
                  "shard_gemv_after");
}

int qb200_shard_wait(const qb200_shard_peers_t *peers, unsigned int epoch, long long limit_cycles, void *stream)
{
    int rc = check_peers(peers);
    if (rc) return rc;
    return finish(qb::shard_wait(peers, epoch, limit_cycles, (cudaStream_t)stream), "shard_wait");
}

int qb200_ipc_export(const void *ptr, void *handle64)
{
    if (!ptr || !handle64) return fail(QB200_E_POINTER, "null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is 64 bytes");
    cudaError_t e = cudaIpcGetMemHandle((cudaIpcMemHandle_t *)handle64, (void *)ptr);
    return e ? cuda_fail(e, "cudaIpcGetMemHandle") : 0;
}

int qb200_ipc_import(const void *handle64, void **ptr)
{
    if (!ptr || !handle64) return fail(QB200_E_POINTER, "null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof h);
    cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
    return e ? cuda_fail(e, "cudaIpcOpenMemHandle") : 0;
}

int qb200_ipc_close(void *ptr)
{
    cudaError_t e = cudaIpcCloseMemHandle(ptr);
    return e ? cuda_fail(e, "cudaIpcCloseMemHandle") : 0;
}

int qb200_malloc(void **ptr, size_t bytes)
{
    if (!ptr) return fail(QB200_E_POINTER, "null out pointer");
    cudaError_t e = cudaMalloc(ptr, bytes ? bytes : 1);
    return e ? cuda_fail(e, "cudaMalloc") : 0;
}

int qb200_free(void *ptr)
{
    cudaError_t e = cudaFree(ptr);
    return e ? cuda_fail(e, "cudaFree") : 0;
}

int qb200_malloc_host(void **ptr, size_t bytes)
{
    if (!ptr) return fail(QB200_E_POINTER, "null out pointer");
    cudaError_t e = cudaMallocHost(ptr, bytes ? bytes : 1);
    return e ? cuda_fail(e, "cudaMallocHost") : 0;
}

int qb200_free_host(void *ptr)
{
    cudaError_t e = cudaFreeHost(ptr);
    return e ? cuda_fail(e, "cudaFreeHost") : 0;
}

int qb200_memcpy_h2d(void *dst, const void *src, size_t bytes, void *stream)
{
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream);
    return e ? cuda_fail(e, "cudaMemcpyAsync h2d") : 0;
}

int qb200_memcpy_d2h(void *dst, const void *src, size_t bytes, void *stream)
{
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    return e ? cuda_fail(e, "cudaMemcpyAsync d2h") : 0;
}

int qb200_memset(void *dst, int value, size_t bytes, void *stream)
{
    cudaError_t e = cudaMemsetAsync(dst, value, bytes, (cudaStream_t)stream);
    return e ? cuda_fail(e, "cudaMemsetAsync") : 0;
}

int qb200_synchronize(void)
{
    cudaError_t e = cudaDeviceSynchronize();
    qb::gemv_forget_history();          // nothing launched before can still be running
    return e ? cuda_fail(e, "cudaDeviceSynchronize") : 0;
}

}  // extern "C"
