/*
 * qiyas_b200.h -- C ABI of libqiyas_b200.so: the block-scaled quantized products of Qiyas
 * (gemv and A.B^T over the GGUF block formats Q8_0, Q4_0, Q4_K, Q6_K) as hand-written
 * sm_100a CUDA kernels.
 *
 * The library replaces, for this path only, Qiyas's run-time PTX generation and its driver
 * binding (src/Gpu.cs:46-66,142-182,290-301).  Every entry point cites the reference
 * interface it stands in for.  Conventions shared by all of them:
 *
 *  - Device pointers are plain addresses in the current device's primary context (what
 *    cuMemAlloc_v2 returns to the reference's Gpu.Rent, src/Gpu.cs:227-249).  Operands need
 *    2-byte alignment only (a 34- or 18-byte block is 2-byte aligned, src/BlockProducts.cs:108);
 *    f32 arrays need 4-byte alignment.
 *  - `stream` is a cudaStream_t / CUstream passed as void*; NULL is the legacy default stream,
 *    which is where the reference launches (src/Gpu.cs:300).  Calls are asynchronous and never
 *    synchronize; the caller orders them as it orders the reference's launches: by stream order.
 *  - Stream order, precisely.  The gemv kernels are launched as programmatic dependents of the work
 *    before them in the stream, and a gemv call none of whose buffers is read or written by a gemv
 *    launch of this library that may still be running starts beside those launches instead of after
 *    them (every other call waits for all earlier work, as plain stream order would have it).  Two
 *    assumptions come with that.  (1) Kernels of other origin in the same stream are launched the
 *    plain way, as the reference launches everything (cuLaunchKernel, src/Gpu.cs:290-301): a foreign
 *    kernel that itself releases its dependents early (griddepcontrol.launch_dependents before its
 *    last store) and writes a gemv operand must be separated from the gemv by an event or by a
 *    plainly launched kernel.  (2) The record of launches in flight is kept per host thread: all
 *    calls on one stream come from one host thread (the reference is single-threaded by
 *    construction, src/Gpu.cs:85-89), or the caller synchronizes when the stream changes hands.
 *  - Return value: 0 success; < 0 an argument error (the reference throws NotSupportedException
 *    or ArgumentException there); > 0 a cudaError_t (the reference throws
 *    InvalidOperationException, src/Gpu.cs:74-79).  qb200_last_error() gives the text.
 *  - Nothing is retained from the caller's buffers; outputs are overwritten whole.
 *  - No entry point falls back to a CPU path: without a usable sm_100 device they fail.
 */
#ifndef QIYAS_B200_H
#define QIYAS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Format ids.  Names and layouts: src/Blocks.cs:10-17 and the type structs at :261-331. */
#define QB200_Q8_0 0   /* 32 values / 34 bytes: f16 d, 32 int8                          */
#define QB200_Q4_0 1   /* 32 values / 18 bytes: f16 d, 16 bytes of nibbles, value d(q-8) */
#define QB200_Q4_K 2   /* 256 values / 144 bytes                                          */
#define QB200_Q6_K 3   /* 256 values / 210 bytes                                          */
#define QB200_F32 100  /* plain float32 lanes                                             */

/* Argument errors (negative returns). */
#define QB200_E_FORMAT (-1)     /* format not taken by this entry point                    */
#define QB200_E_SHAPE (-2)      /* columns / k not in whole blocks, or a dimension <= 0     */
#define QB200_E_POINTER (-3)    /* null or misaligned pointer                               */
#define QB200_E_WORKSPACE (-4)  /* workspace missing or too small                           */
#define QB200_E_DEVICE (-5)     /* no sm_100 device / library not initialised               */
#define QB200_E_LIMIT (-6)      /* a size beyond what the kernels take (see each call)      */

/* Operations, for qb200_lane_name. */
#define QB200_OP_GEMV 0
#define QB200_OP_MATMUL 1

typedef struct qb200_caps {
    int device;              /* ordinal the library is bound to                              */
    int sm_major, sm_minor;  /* compute capability                                           */
    int sm_count;            /* multiprocessors                                              */
    int tcgen05;             /* 1 when the int8 tcgen05 product can run (sm_100)             */
    int max_shared_bytes;    /* opt-in shared memory per block                               */
    int64_t l2_bytes;        /* L2 cache size                                                */
    int64_t global_bytes;    /* device memory                                                */
} qb200_caps_t;

/* Binds the library to `device` (the reference always takes ordinal 0, src/Gpu.cs:94-96) and
 * sets the kernels' attributes.  Must be called once before any other call. */
int qb200_init(int device);
int qb200_caps(qb200_caps_t *out);

/* Text of the last error on the calling thread ("" if none). */
const char *qb200_last_error(void);

/* GpuOps.BlockProductAvailable (src/MatMulBlocks.cs:392): 1 when the tensor product can run. */
int qb200_block_product_available(void);

/* The lane-name string the reference's operators return (src/BlockProducts.cs:185,
 * src/MatMulBlocks.cs:402): "s8dp blocks" for gemv, "s8 tcgen05 blocks" for A.B^T. */
const char *qb200_lane_name(int op, int fmt_a);

/* Reads and clears the device-side status word.  0 = every kernel so far ran to the end;
 * non-zero = a bounded wait inside a kernel gave up (bit 0: gemv ring, bit 1: A.B^T pipeline,
 * bit 2: a sharded product's wait for its peers).
 * Synchronizes the device. */
int qb200_device_status(int *status);

/* ---- gemv -------------------------------------------------------------------------------
 * GpuOps.GemvBlocks<TN>(a, x, y, rows, cols) (src/BlockProducts.cs:178-186; kernel it replaces:
 * Ptx.GemvBlocks, :78-172):  y[r] = sum over blocks of (dA*dX) * (sum_32 qA*qX), f32 lanes.
 *   fmt_a: Q8_0, Q4_0 (the reference's two) or Q4_K, Q6_K (no block product in the reference:
 *          its gemv decodes them to f32, src/GpuOps.cs:287-300).
 *   fmt_x: Q8_0 or Q4_0 blocks (the reference passes x in a's format), or QB200_F32: x is then
 *          encoded to Q8_0 inside the kernel exactly as lanes_to_q8_0 encodes it
 *          (src/Ptx.Blocks.cs:52-73), and the product is taken on those blocks.
 *          With fmt_a Q4_K / Q6_K, fmt_x is Q8_0 or F32.
 *   cols must be whole blocks of a's format, and at most 65536 (32768 with fmt_a Q6_K).  rows >= 0. */
int qb200_gemv_blocks(int fmt_a, int fmt_x, const void *a, const void *x, float *y, int rows, int cols, void *stream);

/* The block branch of the public gemv, GpuOps.Gemv<TN> (src/GpuOps.cs:277-285: rent f32 lanes,
 * GemvBlocks, then Back, src/GpuOps.cs:964-975 -> Ptx.LanesToBlock, src/Ptx.Blocks.cs:11-96), in one
 * launch: y_lanes[rows] as qb200_gemv_blocks writes it, and y_blocks = those lanes as
 * ceil(rows/32) blocks of fmt_y (Q8_0 or Q4_0; values past `rows` count as zero), byte for byte
 * what qb200_encode gives on y_lanes.  y_lanes is the f32 scratch the reference rents; it must be
 * given.  Other arguments as qb200_gemv_blocks. */
int qb200_gemv_blocks_back(int fmt_a, int fmt_x, const void *a, const void *x, float *y_lanes, int fmt_y, void *y_blocks, int rows,
                           int cols, void *stream);

/* As qb200_gemv_blocks, and also writes the exact s32 sum of every 32-value block,
 * sums[r * (cols/32) + b] (Q8_0 / Q4_0: sum qA*qX with Q4_0's q-8; Q4_K: sum q*qX per sub-block;
 * Q6_K: scA*sum16 + scB*sum16 with q-32).  For parity checks of the integer part. */
int qb200_gemv_block_sums(int fmt_a, int fmt_x, const void *a, const void *x, float *y, int32_t *sums, int rows, int cols,
                          void *stream);

/* The same product on HOST buffers: copies a and x to the device, runs the kernel, copies y
 * back and waits (what Checks.GemvRun does around the operator, src/Checks.cs:1983-1997:
 * Rent, Upload, op, Synchronize, Download).  Device staging is kept by the library and grows
 * on demand. */
int qb200_gemv_blocks_host(int fmt_a, int fmt_x, const void *a, const void *x, float *y, int rows, int cols);

/* No counterpart in the reference.  The same gemv for callers that must not allocate device memory: a host
 * application that owns all of it through its own pool (the reference's Gpu.Rent / Arena, src/Gpu.cs:227-249, would be
 * one: an allocation behind its back escapes its accounting and makes the driver synchronize the device), or a
 * latency-critical loop in which a cudaMalloc stall is not acceptable.  The other entry points lean on qb200_init, which
 * allocates the library's status word (and, for the host-buffer and workspace-less calls, staging that grows on demand);
 * this one needs no qb200_init and calls no cudaMalloc / cudaFree.  Its scratch - x re-laid for the kernel by a small
 * kernel of its own, where qb200_gemv_blocks re-lays x inside the gemv kernel - is a fixed array compiled into the
 * library (20 736 bytes of every GPU that loads the library, held until the process exits), so it takes at most
 * QB200_NOALLOC_MAX_COLS columns and returns QB200_E_LIMIT beyond that.
 * The first call on each device looks up the array's device address and sets the kernels' attributes on that device:
 * make that first call outside any stream capture.  All calls on a device share the one array and the one status
 * word: two calls whose kernels could overlap on the GPU (different streams, no ordering between them) race, and the
 * caller must order them.  Same arguments, arithmetic and results as qb200_gemv_blocks. */
#define QB200_NOALLOC_MAX_COLS 16384
int qb200_gemv_blocks_noalloc(int fmt_a, int fmt_x, const void *a, const void *x, float *y, int rows, int cols, void *stream);
/* Reads and clears the status word of the no-allocation path on the current device: non-zero when a bounded wait inside
 * one of its kernels gave up in any call since the last reading (as qb200_device_status; synchronizes the device). */
int qb200_gemv_noalloc_status(int *status);

/* ---- A.B^T ------------------------------------------------------------------------------
 * GpuOps.MatMulBlocks<TN>(a, b, cLanes, m, n, k) (src/MatMulBlocks.cs:395-403; kernel it
 * replaces: Ptx.MatMulBlocks, :178-386):  C[i,j] = sum over k-blocks of
 * fma(float(D_kb[i,j]), sA[i,kb]*sB[j,kb], acc), kb ascending, D_kb the exact s32 of 32 products.
 *   fmt_a, fmt_b: Q8_0 or Q4_0 each (the reference takes one format for both).
 *   fmt_b may also be Q4_K (no block product in the reference: its Q4_K products decode both
 *   operands to f32 first, src/GpuOps.Products.cs:28-42).  Every 32-value sub-block is then a
 *   k-block with scale d*sc and min dmin*m as DecodeQ4_K rounds them (src/Blocks.cs:88-93):
 *   acc = fma(float(D), sA*(d*sc), acc); acc = fma(dmin*m, -(sA*float(sum of qA)), acc).
 *   With fmt_b Q6_K every 16-value sub-block is a k-block with scale d*sc (src/Blocks.cs:167-170).
 *   k whole blocks of both operands (32; 256 with Q4_K / Q6_K); m, n >= 1.
 *   Block scales must be finite: with Q8_0 / Q4_0 on both sides the products sA*sB are taken by the
 *   tensor cores together with the zero terms of the neighbouring k-blocks, which an infinite scale
 *   would turn into NaN (the result is then NaN where the reference gives +-inf or NaN).
 *   With at most 64 rows of A the rows of B take the lanes of tensor memory instead of A's (same bits);
 *   with k a multiple of 256 and b on a 16-byte boundary as well, Q8_0 / Q4_0 weights are not re-laid in
 *   memory at all: the product kernel fetches the raw blocks by TMA tile copies and converts them as it
 *   streams them (same bits again; at most 32 rows of A where the driver offers no tensor-map encoder).
 *   workspace: device scratch of qb200_matmul_workspace_bytes(...) bytes, 256-byte aligned,
 *   private to the call until it completes on `stream` (the operands are re-laid there for
 *   the tensor cores).  Pass NULL/0 to use one scratch buffer the library keeps and grows: calls
 *   that use it must all be on one stream and come from one host thread, since a second call
 *   re-lays its operands over the first's. */
size_t qb200_matmul_workspace_bytes(int fmt_a, int fmt_b, int m, int n, int k);
int qb200_matmul_blocks(int fmt_a, int fmt_b, const void *a, const void *b, float *c, int m, int n, int k, void *workspace,
                        size_t workspace_bytes, void *stream);

/* GpuOps.MatMulViewBlocks<TN> (src/MatMulBlocks.cs:414-424: rent f32 lanes, MatMulBlocks, then Back,
 * src/GpuOps.cs:964-975 -> Ptx.LanesToBlock): c_lanes as qb200_matmul_blocks writes it and c_blocks = those
 * m*n lanes as blocks of fmt_c (Q8_0 or Q4_0), byte for byte what qb200_encode gives on c_lanes.  When n is
 * whole blocks of 32 and c_lanes is 16-byte aligned the blocks are encoded by the product kernel itself;
 * otherwise by a second launch, as in the reference.  c_lanes is the scratch the reference rents; it must be given. */
int qb200_matmul_blocks_back(int fmt_a, int fmt_b, const void *a, const void *b, float *c_lanes, int fmt_c, void *c_blocks, int m, int n,
                             int k, void *workspace, size_t workspace_bytes, void *stream);

/* No counterpart in the reference, whose kernel reads raw blocks on every call (src/MatMulBlocks.cs:234-254).
 * The weights' half of the re-laying, done once: qb200_matmul_prepack writes B (n x k, fmt_b) into `packed`
 * (qb200_matmul_prepacked_bytes bytes, 256-byte aligned) in the tensor cores' layout, which does not depend on m;
 * qb200_matmul_blocks_prepacked then multiplies any A against it and gives the same bits as qb200_matmul_blocks
 * on the raw B.  Its workspace holds the re-laid A only (qb200_matmul_prepacked_workspace_bytes; NULL/0 as above).
 * The packed form belongs to this build of the library: do not store it in files. */
size_t qb200_matmul_prepacked_bytes(int fmt_b, int n, int k);
int qb200_matmul_prepack(int fmt_b, const void *b, int n, int k, void *packed, size_t packed_bytes, void *stream);
size_t qb200_matmul_prepacked_workspace_bytes(int fmt_a, int fmt_b, int m, int k);
int qb200_matmul_blocks_prepacked(int fmt_a, int fmt_b, const void *a, const void *b_packed, float *c, int m, int n, int k,
                                  void *workspace, size_t workspace_bytes, void *stream);

/* ProductView with Batch > 1 (src/Products.cs:15-22: `Batch` products at strides StrideA, StrideB, StrideC in
 * values, 0 broadcasting an operand across the batch) on the block product, all products in one launch.  The
 * reference's BlockView (src/MatMulBlocks.cs:410-411) sends batches to its decoded route; here product i reads
 * A at a + i*stride_a values, B at b + i*stride_b values and writes c + i*stride_c f32 lanes.  Strides are
 * whole blocks of their operand; stride_c >= m*n. */
size_t qb200_matmul_batched_workspace_bytes(int fmt_a, int fmt_b, int m, int n, int k, int batch, int64_t stride_a, int64_t stride_b);
int qb200_matmul_blocks_batched(int fmt_a, int fmt_b, const void *a, const void *b, float *c, int m, int n, int k, int batch,
                                int64_t stride_a, int64_t stride_b, int64_t stride_c, void *workspace, size_t workspace_bytes, void *stream);

/* As qb200_matmul_blocks for a tiny shape, also writing every exact block sum
 * sums[(i*n + j)*kbs + kb], kbs = k/32 k-blocks a row (k/16 with fmt_b Q6_K); m*n*kbs must be at most 2^24. */
int qb200_matmul_block_sums(int fmt_a, int fmt_b, const void *a, const void *b, float *c, int32_t *sums, int m, int n, int k,
                            void *stream);

/* No counterpart in the reference.  The tensor pipe's own rate on the bound device, for rooflines: clock cycles one
 * tcgen05.mma kind::i8 of the product's shape (M 128, N 128, K 32: 2^20 int8 operations) takes on one multiprocessor when
 * nothing else runs (a short kernel, a few microseconds, synchronizes the default stream); 0 when the measurement did
 * not complete.  Dense int8 peak = 2^20 / cycles x multiprocessors x SM clock. */
int qb200_tensor_rate(double *cycles_per_mma);

/* ---- codecs -----------------------------------------------------------------------------
 * qb200_encode: Ptx.LanesToBlock, the `Back` step (src/Ptx.Blocks.cs:11-331, src/GpuOps.cs:964-975):
 * n f32 lanes -> whole blocks of fmt, zeros read past n; byte-for-byte the CPU encoder
 * (src/Blocks.cs:37-45,58-70,98-148,175-215) with the device's rounding for Q4_0.
 * qb200_decode: Ptx.Widen (src/Ptx.Attention.cs:202-219, src/Ptx.cs:151-277): value i of a block
 * array as f32, bit-for-bit Blocks.Decode* (src/Blocks.cs:31-35,48-56,79-96,151-173). */
int qb200_encode(int fmt, const float *lanes, void *blocks, int64_t n, void *stream);
int qb200_decode(int fmt, const void *blocks, float *lanes, int64_t n, void *stream);

/* ---- N-row sharding across the GPUs of one box -------------------------------------------
 * No counterpart in the reference, which runs on device ordinal 0 alone (src/Gpu.cs:94-96).  The output rows of a
 * product are independent, so rank r of `world` keeps rows [first, first + count) of the weights (qb200_shard_range:
 * ceil(rows / world) rows a rank, the last ranks fewer or none) and computes that slice of y with the single-GPU
 * kernels; x is replicated.  Where every rank needs the whole y, the slices are exchanged by the gemv kernel itself:
 * its blocks store the rows they computed into every other rank's copy of y through peer-mapped pointers (plain
 * stores over NVLink: no copy engine, no collective launch), and the grid's last block then stores `epoch` into this
 * rank's word of every rank's flag array.  qb200_shard_wait puts a small kernel in the stream that waits, for at most
 * `limit_cycles` clock cycles (<= 0: about a second), until every rank's word of the local flag array has reached
 * `epoch`; work queued after it on that stream sees the whole y.  A wait that runs out sets bit 2 of the status word
 * (qb200_device_status) and returns: nothing hangs when a peer is late or gone.
 *
 * One process drives one GPU (qb200_init(device) in each); the ranks map one another's buffers with the CUDA IPC
 * helpers below (or, in one process, with peer access).  peers->out[w] is rank w's y (rows_total f32, 16-byte aligned),
 * peers->flags[w] its flag array (2 * QB200_SHARD_MAX words, zeroed once before the first call: a word a rank, then the
 * owner's own counters), both as THIS process addresses them.  Successive calls pass increasing epochs (1, 2, ...), or
 * all pass 0: publisher and waiter then count their calls on the device, which is what a captured CUDA graph needs, since
 * its replays repeat the captured arguments (every rank must then make the same sequence of calls).  A rank must not overwrite its x or start the
 * next qb200_shard_gemv into the same buffers before its own qb200_shard_wait for the previous epoch is in its stream:
 * that wait is also what tells it the peers have finished writing into its y.  All of a rank's sharded calls go to one
 * stream.  An NCCL all-gather of the slices gives the same y and remains the choice across boxes. */
#define QB200_SHARD_MAX 8
typedef struct qb200_shard_peers {
    int world, rank;
    float *out[QB200_SHARD_MAX];
    unsigned int *flags[QB200_SHARD_MAX];
} qb200_shard_peers_t;
int qb200_shard_range(int rows, int world, int rank, int *first, int *count);
int qb200_shard_gemv(int fmt_a, int fmt_x, const void *a_shard, const void *x, int rows_total, int cols, const qb200_shard_peers_t *peers,
                     unsigned int epoch, void *stream);
int qb200_shard_wait(const qb200_shard_peers_t *peers, unsigned int epoch, long long limit_cycles, void *stream);
/* The sharded A.B^T.  B's rows are C's columns: rank r keeps rows [first, first + count) of B (qb200_shard_range over
 * n_total) and computes that column block of the m x n_total C; peers->out[w] is rank w's copy of the whole C
 * (row-major, m * n_total floats), and the product kernel's epilogue stores the block, row stride n_total, into every
 * copy (plain peer stores), then raises the flags as qb200_shard_gemv does; qb200_shard_wait completes it in the same way.
 * b_shard: the rank's rows as raw blocks, or NULL when b_shard_packed (qb200_matmul_prepack of those rows) is given.
 * workspace: as qb200_matmul_blocks / _prepacked for an m x count x k product.  Lanes only (no sums, no `Back`). */
int qb200_shard_matmul(int fmt_a, int fmt_b, const void *a, const void *b_shard, const void *b_shard_packed, int m, int n_total, int k,
                       const qb200_shard_peers_t *peers, unsigned int epoch, void *workspace, size_t workspace_bytes, void *stream);
/* A chain of sharded products, each reading the whole output of the one before it (the layers of a model): as
 * qb200_shard_gemv, but x is rank `peers->rank`'s copy of the output of the exchange `after`, and the kernel itself waits
 * (bounded by limit_cycles as qb200_shard_wait is; status bit 2 when it runs out) until every rank's word of after's
 * local flag array has reached after_epoch (0: counted, as above) before it reads x -- while its copies of the weights
 * are already running.  No qb200_shard_wait is needed between the two products; the last product of the chain is followed
 * by one.  `after` and `peers` are two exchanges between the same ranks with buffers of their own (alternate two of them
 * along the chain): a rank that is a product ahead must not store into the y its peers are still reading. */
int qb200_shard_gemv_after(int fmt_a, int fmt_x, const void *a_shard, const void *x, int rows_total, int cols, const qb200_shard_peers_t *peers,
                           unsigned int epoch, const qb200_shard_peers_t *after, unsigned int after_epoch, long long limit_cycles, void *stream);
/* A device allocation of this process (qb200_malloc) as a 64-byte handle another process on the same box can open
 * (cudaIpcGetMemHandle / cudaIpcOpenMemHandle / cudaIpcCloseMemHandle); opening enables peer access to the owner's GPU. */
int qb200_ipc_export(const void *ptr, void *handle64);
int qb200_ipc_import(const void *handle64, void **ptr);
int qb200_ipc_close(void *ptr);

/* ---- plain device memory for hosts without a CUDA binding of their own (tests, bench) ---- */
int qb200_malloc(void **ptr, size_t bytes);
int qb200_free(void *ptr);
int qb200_malloc_host(void **ptr, size_t bytes);   /* pinned host memory */
int qb200_free_host(void *ptr);
int qb200_memcpy_h2d(void *dst, const void *src, size_t bytes, void *stream);
int qb200_memcpy_d2h(void *dst, const void *src, size_t bytes, void *stream);
int qb200_memset(void *dst, int value, size_t bytes, void *stream);
int qb200_synchronize(void);

#ifdef __cplusplus
}
#endif
#endif
