// extern "C" surface of the backend (include/ormi_b200.h): argument checking, exception -> error code.
#include <algorithm>
#include <cstring>

#include "context.h"
#include "ormi_b200.h"

using namespace ormi_b200;

static thread_local std::string g_last_error;

template <typename F>
static int guarded(F&& f) {
    try { f(); return 0; }
    catch (const std::exception& e) { g_last_error = e.what(); return 1; }
    catch (...) { g_last_error = "unknown error"; return 1; }
}

static void need(bool cond, const char* msg) { if (!cond) throw Error(msg); }

// Every entry point that takes a context makes the context's device current first: a process may hold contexts on
// several devices, and stream operations fail when another device is current.
static void bind(ormi_b200_ctx* ctx, const char* who, bool capturable = false) {
    if (!ctx) throw Error(std::string(who) + ": ctx is NULL");
    ORMI_CUDA(cudaSetDevice(ctx->device));
    // while a step is being captured only calls that queue work on the compute stream (or touch the pool) may run:
    // a host wait, a copy to or from the host or a collective would end the capture with an error of the driver's
    if (ctx->capturing && !capturable) throw Error(std::string(who) + ": not allowed while a step is being captured");
    // An error that an earlier runtime call of this thread left behind and nobody consumed (another library in the
    // process, or a collective library called from here, may do that with a call it expected to fail) must not be
    // blamed on the next kernel this library launches: it is taken off here and counted.  Sticky errors stay and are
    // reported by the call that meets them.  ORMI_B200_CHECK_STALE=1 reports the leftover instead, naming the entry
    // point that found it.
    const cudaError_t stale = cudaGetLastError();
    if (stale != cudaSuccess) {
        static const bool report = std::getenv("ORMI_B200_CHECK_STALE") != nullptr;
        if (report) throw Error(std::string("CUDA Error: ") + cudaGetErrorString(stale) + " (left behind before " + who + ")");
        ctx->counters["stale_errors_cleared"]++;
    }
}

namespace ormi_b200 {
void set_last_error(const std::string& msg) { g_last_error = msg; }
void gemm_dispatch(ormi_b200_ctx* ctx, const GemmArgs& g) {
    if (ctx->matmul_mode == MatmulMode::BF16) gemm_bf16(ctx, g);
    else if (ctx->matmul_mode == MatmulMode::TF32) gemm_tf32(ctx, g, 1);
    else if (ctx->matmul_mode == MatmulMode::TF32X3) gemm_tf32(ctx, g, 3);
    else gemm_ffma(ctx, g);
}
}  // namespace ormi_b200

extern "C" {

const char* ormi_b200_last_error(void) { return g_last_error.c_str(); }

int ormi_b200_init(int device, ormi_b200_ctx** out_ctx) {
    return guarded([&] {
        need(out_ctx != nullptr, "ormi_b200_init: out_ctx is NULL");
        int count = 0;
        cudaError_t e = cudaGetDeviceCount(&count);
        if (e != cudaSuccess) { cudaGetLastError(); throw Error(std::string("CUDA Error: ") + cudaGetErrorString(e)); }
        if (device < 0 || device >= count) throw Error("CUDA Error: no such device " + std::to_string(device));
        ORMI_CUDA(cudaSetDevice(device));
        cudaDeviceProp prop;
        ORMI_CUDA(cudaGetDeviceProperties(&prop, device));
        if (prop.major != 10) throw Error("ormi_b200 is built for sm_100a only; device is sm_" + std::to_string(prop.major) + std::to_string(prop.minor));
        auto ctx = std::make_unique<ormi_b200_ctx>();
        ctx->device = device;
        ctx->num_sms = prop.multiProcessorCount;
        ORMI_CUDA(cudaFree(0));
        ctx->drv.load();
        ORMI_CUDA(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
        // ORMI_B200_POOL_CANARY=1: every context starts with the option "pool_canary" on (a whole test session under guard zones)
        ctx->pool_canary = std::getenv("ORMI_B200_POOL_CANARY") != nullptr;
        *out_ctx = ctx.release();
    });
}

int ormi_b200_shutdown(ormi_b200_ctx* ctx) {
    return guarded([&] {
        if (!ctx) return;
        cudaSetDevice(ctx->device);
        comm_destroy(ctx);
        cudaStreamSynchronize(ctx->stream);
        for (auto& kv : ctx->kernel_cache) if (kv.second.module) ctx->drv.ModuleUnload(kv.second.module);
        for (auto& kv : ctx->shadows) cudaFree(kv.second.ptr);
        for (auto& kv : ctx->free_blocks) for (void* p : kv.second) cudaFree(p);
        if (ctx->gemm_err) cudaFree(ctx->gemm_err);
        if (ctx->up_stream) { cudaStreamSynchronize(ctx->up_stream); cudaStreamSynchronize(ctx->down_stream); cudaStreamDestroy(ctx->up_stream); cudaStreamDestroy(ctx->down_stream); cudaEventDestroy(ctx->copy_event); for (auto& e : ctx->upload_marks) cudaEventDestroy(e); }
        cudaStreamDestroy(ctx->stream);
        delete ctx;
    });
}

int ormi_b200_alloc(ormi_b200_ctx* ctx, size_t bytes, void** out_ptr) {
    return guarded([&] { need(out_ptr != nullptr, "ormi_b200_alloc: NULL argument"); bind(ctx, "ormi_b200_alloc", true); *out_ptr = pool_alloc(ctx, bytes); });
}

int ormi_b200_free(ormi_b200_ctx* ctx, void* ptr, size_t bytes) {
    return guarded([&] { bind(ctx, "ormi_b200_free", true); pool_free(ctx, ptr, bytes); });
}

int ormi_b200_trim(ormi_b200_ctx* ctx) {
    return guarded([&] {
        bind(ctx, "ormi_b200_trim");
        ORMI_CUDA(cudaStreamSynchronize(ctx->stream));
        std::lock_guard<std::mutex> lock(ctx->pool_mutex);
        cudaError_t first = cudaSuccess;
        for (auto& kv : ctx->free_blocks) for (void* p : kv.second) {
            const cudaError_t e = cudaFree(p);
            if (e != cudaSuccess && first == cudaSuccess) first = e;
            ctx->pool_held_bytes -= (long long)kv.first;
        }
        ctx->free_blocks.clear();
        ctx->pooled.clear();
        if (first != cudaSuccess) { cudaGetLastError(); throw Error(std::string("CUDA Error: ") + cudaGetErrorString(first) + " (cudaFree of a pool block)"); }
    });
}

int ormi_b200_memset(ormi_b200_ctx* ctx, void* ptr, int value, size_t bytes) {
    return guarded([&] { bind(ctx, "ormi_b200_memset", true); shadow_drop(ctx, ptr, bytes); ORMI_CUDA(cudaMemsetAsync(ptr, value, bytes, ctx->stream)); });
}

int ormi_b200_memcpy_d2d(ormi_b200_ctx* ctx, void* dst, const void* src, size_t bytes) {
    return guarded([&] { bind(ctx, "ormi_b200_memcpy_d2d", true); shadow_drop(ctx, dst, bytes); ORMI_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream)); });
}

int ormi_b200_memcpy_h2d(ormi_b200_ctx* ctx, void* dst, const void* src, size_t bytes) {
    return guarded([&] {
        bind(ctx, "ormi_b200_memcpy_h2d");
        shadow_drop(ctx, dst, bytes);
        ORMI_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
        ORMI_CUDA(cudaStreamSynchronize(ctx->stream));   // the host buffer may be reused on return
    });
}

int ormi_b200_memcpy_d2h(ormi_b200_ctx* ctx, void* dst, const void* src, size_t bytes) {
    return guarded([&] {
        bind(ctx, "ormi_b200_memcpy_d2h");
        ORMI_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
        comm_guarded_sync(ctx, ctx->stream);
        check_gemm_error(ctx);
    });
}

static void copy_streams(ormi_b200_ctx* ctx) {
    if (ctx->up_stream) return;
    ORMI_CUDA(cudaStreamCreateWithFlags(&ctx->up_stream, cudaStreamNonBlocking));
    ORMI_CUDA(cudaStreamCreateWithFlags(&ctx->down_stream, cudaStreamNonBlocking));
    ORMI_CUDA(cudaEventCreateWithFlags(&ctx->copy_event, cudaEventDisableTiming));
    for (auto& e : ctx->upload_marks) ORMI_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
}

int ormi_b200_memcpy_h2d_async(ormi_b200_ctx* ctx, void* dst, const void* src, size_t bytes, int after_compute) {
    return guarded([&] {
        bind(ctx, "ormi_b200_memcpy_h2d_async");
        need(dst && src, "ormi_b200_memcpy_h2d_async: NULL argument");
        copy_streams(ctx);
        shadow_drop(ctx, dst, bytes);
        if (after_compute) {
            ORMI_CUDA(cudaEventRecord(ctx->copy_event, ctx->stream));
            ORMI_CUDA(cudaStreamWaitEvent(ctx->up_stream, ctx->copy_event, 0));
        }
        ORMI_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->up_stream));
    });
}

int ormi_b200_memcpy_d2h_async(ormi_b200_ctx* ctx, void* dst, const void* src, size_t bytes) {
    return guarded([&] {
        bind(ctx, "ormi_b200_memcpy_d2h_async");
        need(dst && src, "ormi_b200_memcpy_d2h_async: NULL argument");
        copy_streams(ctx);
        ORMI_CUDA(cudaEventRecord(ctx->copy_event, ctx->stream));
        ORMI_CUDA(cudaStreamWaitEvent(ctx->down_stream, ctx->copy_event, 0));
        ORMI_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->down_stream));
    });
}

int ormi_b200_copy_wait(ormi_b200_ctx* ctx, int direction) {
    return guarded([&] {
        bind(ctx, "ormi_b200_copy_wait");
        need(direction == 0 || direction == 1, "ormi_b200_copy_wait: direction must be 0 (uploads) or 1 (downloads)");
        copy_streams(ctx);
        if (direction == 0) {
            ORMI_CUDA(cudaEventRecord(ctx->copy_event, ctx->up_stream));
            ORMI_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->copy_event, 0));
        } else {
            comm_guarded_sync(ctx, ctx->down_stream);
            check_gemm_error(ctx);
        }
    });
}

int ormi_b200_upload_mark(ormi_b200_ctx* ctx, int slot) {
    return guarded([&] {
        bind(ctx, "ormi_b200_upload_mark");
        need(slot >= 0 && slot < 32, "ormi_b200_upload_mark: slot must be 0..31");
        copy_streams(ctx);
        ORMI_CUDA(cudaEventRecord(ctx->upload_marks[slot], ctx->up_stream));
    });
}

int ormi_b200_upload_wait(ormi_b200_ctx* ctx, int slot) {
    return guarded([&] {
        bind(ctx, "ormi_b200_upload_wait");
        need(slot >= 0 && slot < 32, "ormi_b200_upload_wait: slot must be 0..31");
        copy_streams(ctx);
        ORMI_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->upload_marks[slot], 0));
    });
}

__global__ void fill_u32_kernel(uint32_t* dst, uint32_t v, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) dst[i] = v;
}

int ormi_b200_fill_u32(ormi_b200_ctx* ctx, void* dst, uint32_t pattern, size_t count) {
    return guarded([&] {
        bind(ctx, "ormi_b200_fill_u32", true);
        if (count == 0) return;
        shadow_drop(ctx, dst, count * 4);
        int grid = (int)std::min<size_t>((count + 255) / 256, (size_t)ctx->num_sms * 8);
        fill_u32_kernel<<<grid, 256, 0, ctx->stream>>>((uint32_t*)dst, pattern, count);
        ORMI_CUDA(cudaGetLastError());
    });
}

int ormi_b200_fill_u8(ormi_b200_ctx* ctx, void* dst, uint8_t pattern, size_t count) {
    return guarded([&] { bind(ctx, "ormi_b200_fill_u8", true); shadow_drop(ctx, dst, count); ORMI_CUDA(cudaMemsetAsync(dst, pattern, count, ctx->stream)); });
}

int ormi_b200_sync(ormi_b200_ctx* ctx) {
    return guarded([&] { bind(ctx, "ormi_b200_sync"); comm_guarded_sync(ctx, ctx->stream); check_gemm_error(ctx); });
}

void* ormi_b200_stream(ormi_b200_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int ormi_b200_realize(ormi_b200_ctx* ctx, ormi_b200_node* nodes, int n_nodes, const int* roots, int n_roots) {
    return guarded([&] {
        need(nodes && roots && n_nodes > 0 && n_roots > 0, "ormi_b200_realize: bad arguments");
        bind(ctx, "ormi_b200_realize", true);
        realize(ctx, nodes, n_nodes, roots, n_roots);
    });
}

int ormi_b200_plan_json(const ormi_b200_node* nodes, int n_nodes, const int* roots, int n_roots,
                        char* buf, size_t cap, size_t* out_len) {
    return guarded([&] {
        need(nodes && roots && n_nodes > 0 && n_roots > 0, "ormi_b200_plan_json: bad arguments");
        Plan p = build_plan(nodes, n_nodes, roots, n_roots, SchedOptions());
        std::string js = plan_to_json(p);
        if (out_len) *out_len = js.size();
        if (buf && cap) { size_t c = std::min(cap - 1, js.size()); std::memcpy(buf, js.data(), c); buf[c] = 0; }
    });
}

int ormi_b200_plan_json_opts(const ormi_b200_node* nodes, int n_nodes, const int* roots, int n_roots, const char* options,
                             char* buf, size_t cap, size_t* out_len) {
    return guarded([&] {
        need(nodes && roots && n_nodes > 0 && n_roots > 0, "ormi_b200_plan_json_opts: bad arguments");
        const SchedOptions opt = parse_sched_options(options);
        Plan p = build_plan(nodes, n_nodes, roots, n_roots, opt);
        std::string js = plan_to_json(p);
        if (out_len) *out_len = js.size();
        if (buf && cap) { size_t c = std::min(cap - 1, js.size()); std::memcpy(buf, js.data(), c); buf[c] = 0; }
    });
}

int ormi_b200_compile_source(const ormi_b200_node* nodes, int n_nodes, int root, char* buf, size_t cap, size_t* out_len,
                             int* leaf_index, int leaf_cap, int* n_leaves) {
    return guarded([&] {
        need(nodes && n_nodes > 0, "ormi_b200_compile_source: bad arguments");
        SimpleKernel k = compile_simple(nodes, n_nodes, root);
        if (!k.error.empty()) throw Error(k.error);
        if (out_len) *out_len = k.source.size();
        if (buf && cap) { size_t c = std::min(cap - 1, k.source.size()); std::memcpy(buf, k.source.data(), c); buf[c] = 0; }
        if (n_leaves) *n_leaves = (int)k.leaves.size();
        for (int i = 0; leaf_index && i < leaf_cap && i < (int)k.leaves.size(); ++i) leaf_index[i] = k.leaves[i];
    });
}

int ormi_b200_set_lowering(int op, const char* expr) {
    return guarded([&] {
        const bool pointwise = (op >= ORMI_OP_NEG && op <= ORMI_OP_POW) || op == ORMI_OP_MAXIMUM || op == ORMI_OP_GE;
        need(pointwise, "ormi_b200_set_lowering: only pointwise ops have a lowering");
        set_lowering(op, expr ? expr : "");
    });
}

int ormi_b200_compile_cubin(const char* source, char* buf, size_t cap, size_t* out_len) {
    return guarded([&] {
        need(source != nullptr, "ormi_b200_compile_cubin: source is NULL");
        std::vector<char> cubin = compile_cubin(source);
        if (out_len) *out_len = cubin.size();
        if (buf && cap >= cubin.size()) std::memcpy(buf, cubin.data(), cubin.size());
    });
}

static void fill_node(ormi_b200_node& nd, int op, int ndim, const int32_t* shape, const int32_t* strides, void* data) {
    std::memset(&nd, 0, sizeof nd);
    nd.op = op; nd.ndim = ndim;
    int64_t elems = 1;
    for (int d = 0; d < ndim; ++d) { nd.shape[d] = shape[d]; elems *= shape[d]; }
    if (strides) for (int d = 0; d < ndim; ++d) nd.strides[d] = strides[d];
    else { int acc = 1; for (int d = ndim - 1; d >= 0; --d) { nd.strides[d] = acc; acc *= shape[d]; } }
    nd.data = data;
    // extent of the buffer behind the view (for the "one float" rule only the value 4 matters)
    int64_t extent = 1;
    for (int d = 0; d < ndim; ++d) extent += (int64_t)(nd.shape[d] - 1) * (nd.strides[d] < 0 ? -nd.strides[d] : nd.strides[d]);
    nd.data_bytes = data ? extent * 4 : 0;
}

int ormi_b200_sum(ormi_b200_ctx* ctx, const float* in, int ndim, const int32_t* shape, const int32_t* strides,
                  const int32_t* axes, int n_axes, float* out) {
    return guarded([&] {
        need(in && out && ndim >= 0 && ndim <= ORMI_B200_MAX_DIMS, "ormi_b200_sum: bad arguments");
        bind(ctx, "ormi_b200_sum", true);
        ormi_b200_node g[2];
        fill_node(g[0], ORMI_OP_LEAF, ndim, shape, strides, (void*)in);
        int32_t oshape[ORMI_B200_MAX_DIMS]; int ond = 0;
        for (int d = 0; d < ndim; ++d) {
            bool red = n_axes == 0;
            for (int a = 0; a < n_axes; ++a) red |= (axes[a] == d);
            if (!red) oshape[ond++] = shape[d];
        }
        fill_node(g[1], ORMI_OP_SUM, ond, oshape, nullptr, nullptr);
        g[1].n_parents = 1; g[1].parents[0] = 0; g[1].n_axes = n_axes;
        for (int a = 0; a < n_axes; ++a) g[1].axes[a] = axes[a];
        int root = 1;
        std::vector<std::pair<int, void*>> pre{{1, (void*)out}};
        realize(ctx, g, 2, &root, 1, &pre);
    });
}

int ormi_b200_matmul(ormi_b200_ctx* ctx,
                     const float* A, int ndim_a, const int32_t* shape_a, const int32_t* strides_a,
                     const float* B, int ndim_b, const int32_t* shape_b, const int32_t* strides_b,
                     float* out, int ndim_out, const int32_t* shape_out) {
    return guarded([&] {
        need(A && B && out, "ormi_b200_matmul: NULL argument");
        bind(ctx, "ormi_b200_matmul", true);
        need(ndim_a >= 2 && ndim_b >= 2 && ndim_a <= ORMI_B200_MAX_DIMS && ndim_b <= ORMI_B200_MAX_DIMS && ndim_out <= ORMI_B200_MAX_DIMS,
             "MATMUL requires operands to have at least 2 dimensions.");
        ormi_b200_node g[3];
        fill_node(g[0], ORMI_OP_LEAF, ndim_a, shape_a, strides_a, (void*)A);
        fill_node(g[1], ORMI_OP_LEAF, ndim_b, shape_b, strides_b, (void*)B);
        if (g[0].data_bytes == 4) g[0].data_bytes = 8;   // a 1x1 operand is still a matrix, not a broadcast scalar
        if (g[1].data_bytes == 4) g[1].data_bytes = 8;
        fill_node(g[2], ORMI_OP_MATMUL, ndim_out, shape_out, nullptr, nullptr);
        g[2].n_parents = 2; g[2].parents[0] = 0; g[2].parents[1] = 1;
        int root = 2;
        std::vector<std::pair<int, void*>> pre{{2, (void*)out}};
        realize(ctx, g, 3, &root, 1, &pre);
    });
}

int ormi_b200_cvt_bf16_kmajor(ormi_b200_ctx* ctx, const float* src, int64_t row_stride, int64_t k_stride, int rows, int K, void* dst) {
    return guarded([&] {
        need(src && dst && rows > 0 && K > 0, "ormi_b200_cvt_bf16_kmajor: bad arguments");
        bind(ctx, "ormi_b200_cvt_bf16_kmajor", true);
        cvt_bf16_kmajor(ctx, src, row_stride, k_stride, rows, K, dst);
    });
}

int ormi_b200_gemm_bf16_kmajor(ormi_b200_ctx* ctx, const void* a16, const void* b16, float* C, int M, int N, int Kp) {
    return guarded([&] {
        need(a16 && b16 && C, "ormi_b200_gemm_bf16_kmajor: NULL argument");
        bind(ctx, "ormi_b200_gemm_bf16_kmajor", true);
        gemm_bf16_kmajor(ctx, a16, b16, C, M, N, Kp);
    });
}

int ormi_b200_cvt_bf16(ormi_b200_ctx* ctx, const float* src, int64_t ld, int rows, int cols, void* dst) {
    return guarded([&] {
        need(src && dst, "ormi_b200_cvt_bf16: NULL argument");
        bind(ctx, "ormi_b200_cvt_bf16", true);
        cvt_bf16(ctx, src, ld, rows, cols, dst);
    });
}

int ormi_b200_gemm_bf16(ormi_b200_ctx* ctx, const void* a16, int a_transposed, const void* b16, int b_transposed,
                        float* C, int M, int N, int K) {
    return guarded([&] {
        need(a16 && b16 && C, "ormi_b200_gemm_bf16: NULL argument");
        bind(ctx, "ormi_b200_gemm_bf16", true);
        shadow_drop(ctx, C, (size_t)M * N * 4);
        gemm_tc(ctx, a16, a_transposed ? 1 : 0, b16, b_transposed ? 0 : 1, C, M, N, K);
    });
}

int ormi_b200_comm_unique_id(char id[128]) {
    return guarded([&] { need(id != nullptr, "ormi_b200_comm_unique_id: NULL argument"); comm_unique_id(id); });
}

int ormi_b200_comm_init(ormi_b200_ctx* ctx, const char id[128], int rank, int world_size) {
    return guarded([&] { need(id != nullptr, "ormi_b200_comm_init: NULL argument"); bind(ctx, "ormi_b200_comm_init"); comm_init(ctx, id, rank, world_size); });
}

int ormi_b200_allreduce_sum_f32(ormi_b200_ctx* ctx, void* const* buffers, const size_t* counts, int n, int overlap) {
    return guarded([&] {
        need(buffers && counts && n > 0, "ormi_b200_allreduce_sum_f32: bad arguments");
        bind(ctx, "ormi_b200_allreduce_sum_f32");
        comm_allreduce(ctx, buffers, counts, n, overlap);
    });
}

int ormi_b200_comm_join(ormi_b200_ctx* ctx) {
    return guarded([&] { bind(ctx, "ormi_b200_comm_join"); comm_join(ctx); });
}

int ormi_b200_comm_mark(ormi_b200_ctx* ctx, int slot) {
    return guarded([&] { bind(ctx, "ormi_b200_comm_mark"); comm_mark(ctx, slot); });
}

int ormi_b200_comm_wait(ormi_b200_ctx* ctx, int slot) {
    return guarded([&] { bind(ctx, "ormi_b200_comm_wait"); comm_wait(ctx, slot); });
}

int ormi_b200_comm_destroy(ormi_b200_ctx* ctx) {
    return guarded([&] { bind(ctx, "ormi_b200_comm_destroy"); comm_destroy(ctx); });
}

int ormi_b200_selftest_wait_timeout(ormi_b200_ctx* ctx, int limit_ms) {
    return guarded([&] { bind(ctx, "ormi_b200_selftest_wait_timeout"); selftest_wait_timeout(ctx, limit_ms); });
}

int ormi_b200_set_option(ormi_b200_ctx* ctx, const char* key, const char* value) {
    return guarded([&] {
        need(key && value, "ormi_b200_set_option: NULL argument");
        bind(ctx, "ormi_b200_set_option", true);
        std::string k = key, v = value;
        if (k == "matmul") {
            if (v == "fp32") ctx->matmul_mode = MatmulMode::FP32;
            else if (v == "bf16") ctx->matmul_mode = MatmulMode::BF16;
            else if (v == "tf32") ctx->matmul_mode = MatmulMode::TF32;
            else if (v == "3xtf32") ctx->matmul_mode = MatmulMode::TF32X3;
            else throw Error("unknown matmul mode: " + v);
        } else if (k == "comm_timeout_ms") {
            // wall-clock deadline of collectives and of host-side waits behind them; past it the communicator is aborted
            const int ms = std::atoi(v.c_str());
            if (ms < 0) throw Error("comm_timeout_ms must be >= 0 (0 = the default of ten minutes)");
            ctx->comm_timeout_ms = ms;
        } else if (k == "pool_limit_bytes") {
            // refuse allocations that would take the pool past this many bytes, as the driver does when memory is
            // exhausted (0 = no limit): lets a host test walk the out-of-memory path without exhausting a GPU
            ctx->pool_limit_bytes = std::atoll(v.c_str());
        } else if (k == "auto_graph") {
            // realize replays the launches of a plan as a CUDA graph once the same buffer addresses come round again
            if (v == "on") ctx->auto_graph = true; else if (v == "off") ctx->auto_graph = false; else throw Error("auto_graph must be on or off");
        } else if (k == "pool_canary") {
            // debugging aid: a 256-byte guard zone behind every block taken from now on, checked when the block comes back
            if (v == "on") ctx->pool_canary = true; else if (v == "off") ctx->pool_canary = false; else throw Error("pool_canary must be on or off");
        } else if (k == "tc_pair") {
            // bf16 GEMM: "on" (default) = one tcgen05.mma per pair of SMs (256 x 256 tiles), "off" = one per SM (128 x 256),
            // "auto" = pairs, except while an overlapped all-reduce is in flight beside the GEMM
            if (v == "auto") { ctx->tc_cta_group = 2; ctx->tc_pair_auto = true; }
            else if (v == "on") { ctx->tc_cta_group = 2; ctx->tc_pair_auto = false; }
            else if (v == "off") { ctx->tc_cta_group = 1; ctx->tc_pair_auto = false; }
            else throw Error("tc_pair must be auto, on or off");
        } else if (k.rfind("tune.", 0) == 0) {
            // overrides of the code generator's measured defaults (experiments); "0" restores the default
            const int which = tune_knob_index(k.substr(5));
            if (which < 0) throw Error("unknown option: " + k);
            ctx->tune[which] = std::atoi(v.c_str());
        } else if (k == "fusion") {
            if (v == "on") ctx->fusion = true; else if (v == "off") ctx->fusion = false; else throw Error("fusion must be on or off");
        } else if (k == "intermediates") {
            // "keep" (default): every node a plan materializes is handed back, as the reference realizes every node.
            // "free": only roots and ORMI_NODE_KEEP nodes are; the other materialized nodes are scratch of the call.
            if (v == "keep") ctx->free_intermediates = false; else if (v == "free") ctx->free_intermediates = true; else throw Error("intermediates must be keep or free");
        } else throw Error("unknown option: " + k);
    });
}

// ------------------------------------------------------------------------------------------------ step capture
struct CapturedStep {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    std::vector<std::pair<void*, size_t>> blocks;      // every pool block the step touched: owned until the graph is destroyed
};

int ormi_b200_capture_begin(ormi_b200_ctx* ctx) {
    return guarded([&] {
        bind(ctx, "ormi_b200_capture_begin");
        if (ctx->pool_canary) throw Error("ormi_b200_capture_begin: not with pool_canary on (its checks wait for the device)");
        if (ctx->comm_inflight > 0) throw Error("ormi_b200_capture_begin: a collective is in flight on the second stream");
        device_error_word(ctx);                         // exists before the capture: nothing is allocated inside it
        check_gemm_error(ctx);
        ORMI_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        ctx->capture_blocks.clear();
        ctx->capturing = true;
    });
}

int ormi_b200_capture_end(ormi_b200_ctx* ctx, void** out_graph) {
    return guarded([&] {
        if (!ctx || !out_graph) throw Error("ormi_b200_capture_end: NULL argument");
        ORMI_CUDA(cudaSetDevice(ctx->device));
        if (!ctx->capturing) throw Error("ormi_b200_capture_end: no capture is open");
        ctx->capturing = false;
        auto step = std::make_unique<CapturedStep>();
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &step->graph);
        if (e == cudaSuccess) e = cudaGraphInstantiate(&step->exec, step->graph, 0);
        if (e != cudaSuccess) {
            cudaGetLastError();
            if (step->graph) cudaGraphDestroy(step->graph);
            ctx->capture_blocks.clear();
            throw Error(std::string("CUDA Error: ") + cudaGetErrorString(e) + " (ending the capture)");
        }
        // Every block the pool handed out during the capture is read or written by the replays: the graph owns them all
        // from here on.  Those that went back to the pool in the meantime are taken out of it again; freeing one of
        // the others (a result the caller holds) is a no-op while the graph lives.
        std::lock_guard<std::mutex> lock(ctx->pool_mutex);
        for (auto& kv : ctx->capture_blocks) {
            step->blocks.push_back(kv);
            ctx->graph_owned.insert(kv.first);
            if (ctx->pooled.erase(kv.first)) {
                auto& v = ctx->free_blocks[kv.second];
                v.erase(std::remove(v.begin(), v.end(), kv.first), v.end());
            }
        }
        ctx->capture_blocks.clear();
        ctx->counters["captured_steps"]++;
        *out_graph = step.release();
    });
}

int ormi_b200_graph_launch(ormi_b200_ctx* ctx, void* graph) {
    return guarded([&] {
        bind(ctx, "ormi_b200_graph_launch");
        if (!graph) throw Error("ormi_b200_graph_launch: NULL graph");
        ORMI_CUDA(cudaGraphLaunch(((CapturedStep*)graph)->exec, ctx->stream));
        ctx->gemm_err_pending = true;
        ctx->counters["graph_launches"]++;
    });
}

int ormi_b200_graph_destroy(ormi_b200_ctx* ctx, void* graph) {
    return guarded([&] {
        bind(ctx, "ormi_b200_graph_destroy");
        if (!graph) return;
        std::unique_ptr<CapturedStep> step((CapturedStep*)graph);
        cudaGraphExecDestroy(step->exec);
        cudaGraphDestroy(step->graph);
        {
            std::lock_guard<std::mutex> lock(ctx->pool_mutex);
            for (auto& b : step->blocks) ctx->graph_owned.erase(b.first);
        }
        // bf16 twins that live in the graph's blocks go with them; the blocks return to the pool behind the replays
        // already queued on the compute stream
        for (auto it = ctx->shadows.begin(); it != ctx->shadows.end();) {
            bool mine = false;
            for (auto& b : step->blocks) if (b.first == it->second.ptr) mine = true;
            it = mine ? ctx->shadows.erase(it) : std::next(it);
        }
        for (auto& b : step->blocks) pool_free(ctx, b.first, b.second);
    });
}

int ormi_b200_get_counter(ormi_b200_ctx* ctx, const char* name, int64_t* out_value) {
    return guarded([&] {
        need(ctx && name && out_value, "ormi_b200_get_counter: NULL argument");
        auto it = ctx->counters.find(name);
        *out_value = it == ctx->counters.end() ? 0 : it->second;
    });
}

}  // extern "C"
