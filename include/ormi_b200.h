/*
 * ormi_b200 — C ABI of the B200 (sm_100a) backend for the realize path of Ormi's lazy
 * tensor graph.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns 0 on success
 * and a non-zero code on failure (the text is available from ormi_b200_last_error()), and
 * never throws.  The C++ seams of ormi-core (IAllocator, cuda::execute_jit, cuda::compile,
 * cuda::matmul, cuda::sum, execute_graph) translate a non-zero return into
 * std::runtime_error, which is the reference's own error convention
 * (ormi-core/csrc/utils/macros.h:8-19).
 *
 * Each declaration cites the reference interface it replaces, by path inside the Ormi
 * project.
 */
#ifndef ORMI_B200_H
#define ORMI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORMI_B200_MAX_DIMS 8

/* Operation codes: same order and values as ormi::ops::OpEnum (ormi-core/csrc/core/ops.h:4-10). */
enum ormi_b200_op {
    ORMI_OP_LEAF = 0, ORMI_OP_CONST = 1,
    ORMI_OP_NEG = 2, ORMI_OP_EXP = 3, ORMI_OP_LOG = 4, ORMI_OP_SIN = 5, ORMI_OP_COS = 6,
    ORMI_OP_ADD = 7, ORMI_OP_SUB = 8, ORMI_OP_MUL = 9, ORMI_OP_DIV = 10, ORMI_OP_POW = 11,
    ORMI_OP_MATMUL = 12,
    ORMI_OP_SUM = 13, ORMI_OP_TRANSPOSE = 14, ORMI_OP_RESHAPE = 15, ORMI_OP_EXPAND = 16,
    ORMI_OP_FRAC_DERIV = 17,
    /* Extension ops: no counterpart in ormi::ops::OpEnum (the reference cannot express a maximum).  Additive; the
     * values stay clear of the reference's range.  MAXIMUM and GE are binary pointwise ops that broadcast like ADD
     * (GE yields 1.0f where a >= b, else 0.0f); MAX is a reduction with SUM's axes / keepdims rules. */
    ORMI_OP_MAXIMUM = 100, ORMI_OP_GE = 101, ORMI_OP_MAX = 102
};

/* Node flags (in). */
#define ORMI_NODE_KEEP   1u  /* somebody outside the graph holds this node: it must own a buffer after realize */
#define ORMI_NODE_TWIN16 8u  /* "bf16" matmul arithmetic: a later matmul will read this root (a weight an update produces): write
                              * its bf16 copy along with it, so that no conversion pass is needed then */
#define ORMI_NODE_BF16   16u /* "bf16" matmul arithmetic, first-class bf16 tensors (the reference has the DType enum and nothing behind it,
                              * ormi-core/csrc/core/dtype.h:4-8, core/memory.cpp:88).  On an un-realized root or KEEP node: materialize
                              * it as bf16 ONLY — `data` comes back as a contiguous bf16 matrix of data_bytes = 2 * elements, with this
                              * flag set.  On a realized node: `data` is such a matrix.  A bf16 tensor can only be an operand of a
                              * matmul that runs on the tensor cores (2-D, last dimension a multiple of 8); anything else is refused. */
/* Node flags (out, set by ormi_b200_realize). */
#define ORMI_NODE_OWNED  2u  /* `data` is a fresh pool buffer now owned by the caller (free with ormi_b200_free) */
#define ORMI_NODE_ALIAS  4u  /* `data` aliases the buffer of the node's view base (ormi-core/csrc/backend/runtime.cpp:20-23) */

/*
 * One node of the lazy graph, flattened: the fields of ormi::Node that the realize path
 * reads (ormi-core/csrc/core/node.h:12-37) — op, parents, view {shape, strides}, the
 * ReduceAttrs of a SUM (ormi-core/csrc/core/attributes.h:8-11) and the realized buffer.
 * Nodes are stored in topological order: a parent's index is lower than its child's.
 */
typedef struct ormi_b200_node {
    int32_t  op;                           /* enum ormi_b200_op */
    int32_t  n_parents;                    /* 0, 1 or 2 */
    int32_t  parents[2];                   /* indices into the node array */
    int32_t  ndim;
    int32_t  shape[ORMI_B200_MAX_DIMS];    /* node->view.shape */
    int32_t  strides[ORMI_B200_MAX_DIMS];  /* node->view.strides, in elements */
    int32_t  n_axes;                       /* SUM: number of reduced axes; 0 = reduce every axis */
    int32_t  axes[ORMI_B200_MAX_DIMS];
    int32_t  keepdims;
    uint32_t flags;
    void*    data;                         /* device pointer of node->data->ptr, NULL when not realized */
    int64_t  data_bytes;                   /* node->data->bytes */
} ormi_b200_node;

typedef struct ormi_b200_ctx ormi_b200_ctx;

/* ------------------------------------------------------------------ context, memory ---- */

/* Binds device `device`, creates the compute stream and the buffer pool.
 * Replaces the CUDAAllocator constructor (ormi-core/csrc/backend/cuda/allocator.cu:20-25) and the
 * per-call cuInit/context retain of execute_jit (ormi-core/csrc/backend/cuda/jit.cu:16-19).
 * Fails (non-zero) when no CUDA device is present; the reference's tests use exactly that failure to
 * detect CUDA (ormi-core/csrc/tests/test_utils.h:17-21). */
int ormi_b200_init(int device, ormi_b200_ctx** out_ctx);
int ormi_b200_shutdown(ormi_b200_ctx* ctx);

/* Text of the last error raised on the calling thread. */
const char* ormi_b200_last_error(void);

/* Exact-size caching pool: a freed block is handed back for the next request of the same byte size
 * (contract pinned by ormi-core/csrc/tests/core/test_allocator.cpp:12-47).
 * Replaces CUDAAllocator::allocate / free (allocator.cu:36-55).
 * The pool is ordered by the context's COMPUTE stream: a freed block may be handed out again at once, which is safe for
 * work queued on that stream only.  A buffer whose last use is on another stream — an all-reduce queued with
 * overlap = 1, an asynchronous copy — must not be freed before the compute stream has waited for that use
 * (ormi_b200_comm_join / ormi_b200_comm_wait / ormi_b200_copy_wait).
 * Every pointer handed out is 256-byte aligned.  Buffers the caller brings from elsewhere may be passed to every entry
 * point; when one does not start on a 16-byte boundary the kernels of that call are generated with scalar accesses. */
int ormi_b200_alloc(ormi_b200_ctx* ctx, size_t bytes, void** out_ptr);
int ormi_b200_free(ormi_b200_ctx* ctx, void* ptr, size_t bytes);
/* Returns every cached block to the driver (the reference never does; additive). */
int ormi_b200_trim(ormi_b200_ctx* ctx);

/* CUDAAllocator::memset / memcpy / fill_n / copy_* (allocator.cu:57-95).  The host copies are complete
 * on return; device-side work is ordered on the context's stream. */
int ormi_b200_memset(ormi_b200_ctx* ctx, void* ptr, int value, size_t bytes);
int ormi_b200_memcpy_d2d(ormi_b200_ctx* ctx, void* dst, const void* src, size_t bytes);
int ormi_b200_memcpy_h2d(ormi_b200_ctx* ctx, void* dst, const void* src, size_t bytes);
int ormi_b200_memcpy_d2h(ormi_b200_ctx* ctx, void* dst, const void* src, size_t bytes);
int ormi_b200_fill_u32(ormi_b200_ctx* ctx, void* dst, uint32_t pattern, size_t count);
int ormi_b200_fill_u8(ormi_b200_ctx* ctx, void* dst, uint8_t pattern, size_t count);
/* Copies that do not stop the caller (no counterpart in the reference, whose copies are synchronous cuMemcpy calls,
 * allocator.cu:89-95): for loops that move the next batch in and the last results out while kernels run.  Each
 * direction has a stream of its own beside the compute stream; host memory should be pinned (pageable memory makes the
 * copy synchronous).  One cudaMemcpyAsync per call.
 *   h2d_async  after_compute != 0: the upload first waits for everything queued on the compute stream so far (the
 *              kernels that still read the old contents of `dst`); 0: it starts as soon as the upload stream is free.
 *   d2h_async  always starts after everything queued on the compute stream so far (the kernels that write `src`).
 *   copy_wait  direction 0: the COMPUTE STREAM waits for every upload queued so far (call it before launching what reads
 *              them; the host does not block); direction 1: the HOST waits for every download queued so far, and a
 *              device-side error is reported as by ormi_b200_sync.
 * A buffer with an upload or download in flight must not be freed before the matching copy_wait. */
int ormi_b200_memcpy_h2d_async(ormi_b200_ctx* ctx, void* dst, const void* src, size_t bytes, int after_compute);
int ormi_b200_memcpy_d2h_async(ormi_b200_ctx* ctx, void* dst, const void* src, size_t bytes);
int ormi_b200_copy_wait(ormi_b200_ctx* ctx, int direction);
/* Finer than copy_wait(ctx, 0), for loops that queue uploads well ahead of the kernels that read them:
 *   upload_mark(slot)  remembers the upload stream's current tail in one of 32 slots (call it right after queueing the
 *                      uploads of one batch);
 *   upload_wait(slot)  makes the compute stream wait for exactly that point (call it right before the kernels of that
 *                      batch), not for uploads queued later.  A slot never marked is already complete. */
int ormi_b200_upload_mark(ormi_b200_ctx* ctx, int slot);
int ormi_b200_upload_wait(ormi_b200_ctx* ctx, int slot);
/* Waits for everything queued on the context's stream. */
int ormi_b200_sync(ormi_b200_ctx* ctx);
/* The context's compute stream as a cudaStream_t, for callers that time with CUDA events. */
void* ormi_b200_stream(ormi_b200_ctx* ctx);

/* ------------------------------------------------------------------ realize path ------- */

/* Realizes `roots` (and every KEEP-flagged ancestor) of a flattened graph.
 * Replaces ormi::execute_graph for DeviceEnum::CUDA (ormi-core/csrc/backend/runtime.cpp:13-39),
 * cuda::execute_jit (ormi-core/csrc/backend/cuda/jit.cu:13-44) and the CUDA graph breakers
 * (kernels/blas/matmul.cu:114-124, kernels/reduce/sum.cu:86-97), with a fusion scheduler in front:
 * pointwise chains, their trailing row / column / global sums and reduce-then-broadcast groups run as
 * single generated sm_100a kernels.  On return every root, every KEEP node and every node the scheduler
 * had to materialize has `data`/`data_bytes` set and ORMI_NODE_OWNED (or ORMI_NODE_ALIAS for a view). */
int ormi_b200_realize(ormi_b200_ctx* ctx, ormi_b200_node* nodes, int n_nodes, const int* roots, int n_roots);

/* The schedule of the same call as text (JSON): buffers, kernel launches with their generated CUDA C
 * source, GEMM steps.  Needs no device; ctx may be NULL.  Writes at most `cap` bytes (NUL-terminated)
 * and stores the full length in *out_len.  Counterpart of cuda::compile's `kernel_code`
 * (ormi-core/csrc/backend/cuda/compiler.cuh:8-16) for a whole graph. */
int ormi_b200_plan_json(const ormi_b200_node* nodes, int n_nodes, const int* roots, int n_roots,
                        char* buf, size_t cap, size_t* out_len);

/* The same, for a schedule that depends on options: `options` is "key=value,key=value" with the keys of
 * ormi_b200_set_option that shape a schedule ("matmul", "fusion", "tune.*") plus "aligned=0" for inputs that do not
 * start on 16-byte boundaries.  NULL or "" gives the defaults. */
int ormi_b200_plan_json_opts(const ormi_b200_node* nodes, int n_nodes, const int* roots, int n_roots, const char* options,
                             char* buf, size_t cap, size_t* out_len);

/* cuda::compile (ormi-core/csrc/backend/cuda/compiler.cu:53-112): CUDA C source of the guarded scalar
 * `fused_kernel` for the un-realized pointwise sub-graph under `root`, with the leaves in argument order.
 * `leaf_index[i]` receives the node index of LEAF_i. */
int ormi_b200_compile_source(const ormi_b200_node* nodes, int n_nodes, int root,
                             char* buf, size_t cap, size_t* out_len,
                             int* leaf_index, int leaf_cap, int* n_leaves);

/* The per-op plug-in point of the reference's CUDA compiler, CUDALoweringRegistry
 * (ormi-core/csrc/backend/cuda/lowering_registry.h:11-38; consulted for every tape entry, compiler.cu:104-108): replaces
 * the C expression the code generator emits for pointwise op `op` — in the fused kernels, the GEMM epilogues and the
 * source ormi_b200_compile_source returns alike.  `expr` is CUDA C over the operand placeholders $0 and $1, e.g.
 * "fmaxf($0, $1)"; NULL or "" restores the built-in expression.  Process-wide, like the reference's registry; schedules
 * cached before the change are not reused.  Not to be called while another thread realizes a graph. */
int ormi_b200_set_lowering(int op, const char* expr);

/* compile_ptx (ormi-core/csrc/backend/cuda/utils.cu:6-27): NVRTC, but straight to an sm_100a cubin.
 * Needs no device.  The image is written to `buf` when it fits; *out_len is its size. */
int ormi_b200_compile_cubin(const char* source, char* buf, size_t cap, size_t* out_len);

/* cuda::sum (ormi-core/csrc/backend/cuda/kernels/reduce/sum.cu:12-84) on raw buffers: deterministic
 * reduction of `in` (shape/strides of in_view) over `axes` (n_axes == 0: all) into the contiguous `out`. */
int ormi_b200_sum(ormi_b200_ctx* ctx, const float* in, int ndim, const int32_t* shape, const int32_t* strides,
                  const int32_t* axes, int n_axes, float* out);

/* cuda::matmul (ormi-core/csrc/backend/cuda/kernels/blas/matmul.cu:19-112) on raw buffers and views:
 * C[b] = op(A[b]) op(B[b]); transposition from the last-dimension stride, leading dimensions broadcast.
 * `out` is the contiguous [batch..., M, N] result. */
int ormi_b200_matmul(ormi_b200_ctx* ctx,
                     const float* A, int ndim_a, const int32_t* shape_a, const int32_t* strides_a,
                     const float* B, int ndim_b, const int32_t* shape_b, const int32_t* strides_b,
                     float* out, int ndim_out, const int32_t* shape_out);

/* The two halves of the bf16 tensor-core matmul, for callers that keep bf16 copies of their operands (weights that
 * change once per step) instead of converting inside every matmul.  No counterpart in the reference, whose matmul is
 * one cublasSgemmBatched call (kernels/blas/matmul.cu:98-105).
 *   cvt:  dst[r][k] = bf16(src[r * row_stride + k * k_stride]) for r < rows, k < K; dst is rows x Kp bf16 with
 *         Kp = K rounded up to a multiple of 64, the padding zero ("K-major" staging layout).
 *   gemm: C[M,N] (fp32, contiguous) = A16[M][Kp] * B16[N][Kp]^T, fp32 accumulation (tcgen05.mma, TMEM, TMA). */
int ormi_b200_cvt_bf16_kmajor(ormi_b200_ctx* ctx, const float* src, int64_t row_stride, int64_t k_stride,
                              int rows, int K, void* dst);
int ormi_b200_gemm_bf16_kmajor(ormi_b200_ctx* ctx, const void* a16, const void* b16, float* C, int M, int N, int Kp);

/* The bf16 tensor-core matmul on operands the caller already holds in bf16, each in its own row-major layout (no
 * counterpart in the reference; inside ormi_b200_realize the same kernel runs behind "matmul" = "bf16", with the bf16
 * copies cached per buffer or written by the kernel that produced the fp32 values).
 *   cvt:  dst[r][c] = bf16(src[r * ld + c]) for r < rows, c < cols; dst is contiguous [rows][cols]; cols % 8 == 0.
 *   gemm: C[M,N] (fp32, contiguous) = A * B with fp32 accumulation (tcgen05.mma on a pair of SMs, TMEM, TMA).
 *         a_transposed = 0: A is stored [M][K];  1: stored [K][M] (what a TRANSPOSE view of a row-major matrix is).
 *         b_transposed = 0: B is stored [K][N];  1: stored [N][K].
 *         The contiguous dimension of each operand must be a multiple of 8, N a multiple of 4, pointers 16-byte
 *         aligned.  Ragged M, N and K are handled by the kernel (zero fill on load, clipped stores). */
int ormi_b200_cvt_bf16(ormi_b200_ctx* ctx, const float* src, int64_t ld, int rows, int cols, void* dst);
int ormi_b200_gemm_bf16(ormi_b200_ctx* ctx, const void* a16, int a_transposed, const void* b16, int b_transposed,
                        float* C, int M, int N, int K);

/* ------------------------------------------------------------------ multi-GPU combine -- */

/* Batch-sharded runs: one process per GPU, each realizes its own row shard; parameter gradients (and column / global
 * sums of sharded inputs) are summed over the ranks with NCCL over NVLink.  The reference has no counterpart (single
 * device).  `id` is NCCL's 128-byte unique id: create it on one rank, hand it to the others by any host channel.
 * allreduce: in-place fp32 sum of `n` buffers (one NCCL group).  overlap = 0 queues it on the compute stream;
 * overlap = 1 queues it on a second stream behind everything queued so far, so later kernels run beside it —
 * ormi_b200_comm_join then makes the compute stream wait for the results.  For a wait that comes later than the
 * point where the bucket was queued (another bucket, or the next step's first kernels, in between):
 * ormi_b200_comm_mark(slot) remembers the second stream's current tail in one of 8 slots and
 * ormi_b200_comm_wait(slot) makes the compute stream wait for exactly that point. */
int ormi_b200_comm_unique_id(char id[128]);
int ormi_b200_comm_init(ormi_b200_ctx* ctx, const char id[128], int rank, int world_size);
int ormi_b200_allreduce_sum_f32(ormi_b200_ctx* ctx, void* const* buffers, const size_t* counts, int n, int overlap);
int ormi_b200_comm_join(ormi_b200_ctx* ctx);
int ormi_b200_comm_mark(ormi_b200_ctx* ctx, int slot);
int ormi_b200_comm_wait(ormi_b200_ctx* ctx, int slot);
int ormi_b200_comm_destroy(ormi_b200_ctx* ctx);

/* Column sums of a contiguous fp32 matrix, out[c] = sum over r of in[r * cols + c], WITHOUT allocating anything.
 * No counterpart in the reference: it exists for callers that cannot call cudaMalloc when they need the
 * reduction — their device memory is already owned, whole, by another allocator, or they sit in a steady-state
 * loop that must not hit an allocation's device-wide synchronisation.  The per-block partials that
 * ormi_b200_sum takes from the context's pool live here in a fixed 2 MiB array inside the library image (every
 * GPU that loads the library holds it until exit).  Limits and rules:
 *   - cols <= 65536, otherwise the call fails with an explanatory error (use ormi_b200_sum instead);
 *   - runs on the CURRENT device, on `stream` (a cudaStream_t, NULL = default stream); needs no context;
 *   - all calls share the one scratch array: calls that overlap on the GPU (other streams, other threads) race;
 *   - the first call on a device also fetches the array's device address; make it before any stream capture.
 * Results are deterministic; they differ from ormi_b200_sum only by fp32 summation order. */
int ormi_b200_colsum_static(const float* in, int64_t rows, int64_t cols, float* out, void* stream);

/* ------------------------------------------------------------------ options, counters -- */

/* Self-test of the device-side bounded waits (no counterpart in the reference): queues a one-warp kernel that waits on a
 * barrier nobody arrives on, with a limit of `limit_ms` (1..1000).  The wait gives up, the kernel returns, and the next
 * ormi_b200_sync / ormi_b200_memcpy_d2h fails once with "a bounded device-side wait ran out (code 9 ...)"; the
 * context stays usable.  This is how the error path of the tensor-core GEMM and of the staged row kernels is exercised
 * without faulting or hanging a GPU. */
int ormi_b200_selftest_wait_timeout(ormi_b200_ctx* ctx, int limit_ms);

/* Options (additive; the reference has none).
 *   "matmul":  arithmetic of ormi_b200_realize / ormi_b200_matmul: "fp32" (SIMT FFMA, default), "bf16" (tcgen05, fp32
 *              accumulate; pointwise work behind a matmul runs in the GEMM's epilogue and matmul operands are kept as
 *              bf16 copies beside their fp32 buffers — those buffers must then only be written through this ABI),
 *              "tf32", "3xtf32".
 *   "fusion":  "on" (default) / "off" (one kernel per node, like the reference scheduler).
 *   "intermediates": "keep" (default): every node a plan materializes comes back realized, as the reference realizes
 *              every node it executes (runtime.cpp:13-39).  "free": only roots and ORMI_NODE_KEEP nodes come back; a
 *              materialized node nobody outside the call holds is scratch, returned to the pool after the last step
 *              that reads it (a later call that reaches it again recomputes it).
 *   "auto_graph": "on" (default) / "off".  ormi_b200_realize replays the launches of a plan with two or more of them as a
 *              CUDA graph when the buffers of the call come out at the same addresses as in an earlier call (a loop in its
 *              steady state); recorded at the second such call, up to 32 address sets per plan.  Plans with tensor-core
 *              matmuls are left out (they look up or make bf16 operand copies as they go).
 *   "pool_canary": "on" / "off" (default).  A debugging aid in place of a memory checker: every block the pool hands out
 *              from then on carries a 256-byte guard zone behind it, read back (synchronously) when the block returns; an
 *              overwritten zone makes that call — ormi_b200_free, or the realize call that returns scratch — fail with
 *              the block's size in the message.  The environment variable ORMI_B200_POOL_CANARY=1 starts every context
 *              with it on.
 *   "tc_pair": "on" (default: one tcgen05.mma per pair of SMs, 256 x 256 tiles) / "off" (one per SM, 128 x 256) /
 *              "auto" (pairs, except for GEMMs queued while an overlapped all-reduce is in flight: a collective holds
 *              single SMs, and a pair needs both SMs of a TPC — measured 5 % slower than "on" on 2 and on 4 GPUs).
 *   "tune.rows_vpt", "tune.rows_minb", "tune.rows_grid", "tune.rows_stage", "tune.rows_nstage", "tune.rows_dynamic",
 *   "tune.flat_unroll", "tune.rows_hoist", "tune.epi_unroll", "tune.epi_wpq", "tune.gemm_bn" (128 / 256 columns per
 *   tensor-core GEMM tile), "tune.epi_node_major" (1: GEMM epilogue text column by column instead of node by node): integer overrides of the code generator's measured defaults, for
 *              experiments ("0" = default; for the on/off ones 1 = off, 2 = on). */
int ormi_b200_set_option(ormi_b200_ctx* ctx, const char* key, const char* value);

/* Step capture (additive; the reference launches every kernel from the host, ormi-core/csrc/backend/cuda/jit.cu:13-44).
 * Between capture_begin and capture_end everything the context queues on its compute stream — ormi_b200_realize,
 * ormi_b200_sum / _matmul / _gemm_bf16, device-to-device copies, fills — is recorded into a CUDA graph instead of run;
 * ormi_b200_graph_launch replays the whole step with one call.  Rules: run the step once before capturing it (kernels
 * compiled, every block it needs cached by the pool: nothing is taken from the driver inside a capture); calls that wait
 * for the device, copy to or from the host, or use the second stream (collectives) fail while a capture is open; the
 * replays read the inputs and write the results at the addresses the capture saw, so every pool block handed out during
 * the capture — results included — belongs to the graph until ormi_b200_graph_destroy: ormi_b200_free of one of them is
 * a no-op while the graph lives, and the results die with the graph.  Not with "pool_canary" on. */
int ormi_b200_capture_begin(ormi_b200_ctx* ctx);
int ormi_b200_capture_end(ormi_b200_ctx* ctx, void** out_graph);
int ormi_b200_graph_launch(ormi_b200_ctx* ctx, void* graph);
int ormi_b200_graph_destroy(ormi_b200_ctx* ctx, void* graph);

/* Counters since init: "kernels_compiled", "kernel_cache_hits", "plan_cache_hits", "launches",
 * "gemm_launches", "bytes_allocated", "pool_hits". */
int ormi_b200_get_counter(ormi_b200_ctx* ctx, const char* name, int64_t* out_value);

#ifdef __cplusplus
}
#endif
#endif /* ORMI_B200_H */
