// Per-device state of the backend: stream, buffer pool, kernel cache, plan cache, counters.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "plan.h"

namespace ormi_b200 {

struct Error : std::runtime_error { using std::runtime_error::runtime_error; };

#define ORMI_CUDA(call)                                                                            \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) throw ::ormi_b200::Error(std::string("CUDA Error: ") + cudaGetErrorString(e_) + " (" #call ")"); \
    } while (0)

// Driver entry points, fetched through the runtime so the library itself has no link-time dependency on
// libcuda (it must load, and its symbols be listed, on a machine without a GPU driver).
struct DriverApi {
    CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
    CUresult (*ModuleUnload)(CUmodule) = nullptr;
    CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
    CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void**, void**) = nullptr;
    CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
    CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
    CUresult (*TensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                     const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
    void load();
    void check(CUresult r, const char* what) const;
};

struct CompiledKernel {
    CUmodule module = nullptr;
    CUfunction func = nullptr;
};

// The launches of a plan for one set of buffer addresses, as an instantiated CUDA graph (runtime.cu, realize).
struct StepGraph {
    std::vector<void*> at;     // what every step saw: steps x buffers
    void* exec = nullptr;      // cudaGraphExec_t
    int launches = 0;
    uint64_t stamp = 0;
};

struct CachedPlan {
    ~CachedPlan();
    std::vector<StepGraph> graphs;                 // most recently used address sets
    std::vector<std::vector<void*>> seen;          // address sets met once: the second meeting records a graph
    uint64_t graph_clock = 0;
    Plan plan;
    std::vector<CompiledKernel*> kernels;   // per step (nullptr for GEMM steps)
    // liveness of the scratch (Temp) buffers: the step that first touches buffer b and the step after which nothing
    // reads it; -1 for buffers that are not scratch
    std::vector<int> first_use, last_use;
    std::vector<int> twin_result;   // per buffer: for a bf16 twin of a node that is handed out, the node's fp32 buffer; else -1
};

enum class MatmulMode { FP32, BF16, TF32, TF32X3 };

// bf16 twin of an fp32 matrix that matmuls read (gemm_tc.cu): contiguous [rows][cols] copy of the fp32 data at the
// key pointer (row pitch ld, src_bytes long).
struct Shadow16 {
    void* ptr = nullptr;
    size_t bytes = 0, src_bytes = 0;
    int rows = 0, cols = 0;
    long long ld = 0;
};

struct TcKernel { CompiledKernel* kernel = nullptr; int block = 0, smem = 0; };

// Generated epilogue of the run-time compiled tensor-core GEMM: text spliced into the kernel template plus the
// device pointers of its extra parameters, in parameter order.
struct TcEpilogue {
    std::string prelude, params, init, cols, pre, body, end;
    int wpq = 1;                       // epilogue warps per TMEM lane quarter (1, 2 or 4)
    int unroll = 8;                    // unrolled row steps per chunk
    std::vector<void*> args;
};

}  // namespace ormi_b200

namespace ormi_b200 { constexpr int kErrorWords = 64, kTileCounterWord = 32; }

struct ormi_b200_ctx {
    int device = 0;
    int num_sms = 148;
    cudaStream_t stream = nullptr;
    // asynchronous host copies (abi.cu): one stream per direction, created on first use
    cudaStream_t up_stream = nullptr, down_stream = nullptr;
    cudaEvent_t copy_event = nullptr;
    cudaEvent_t upload_marks[32] = {};   // ormi_b200_upload_mark / ormi_b200_upload_wait
    ormi_b200::DriverApi drv;

    std::mutex pool_mutex;
    long long pool_limit_bytes = 0, pool_held_bytes = 0;   // option "pool_limit_bytes": simulated memory exhaustion
    std::unordered_map<size_t, std::vector<void*>> free_blocks;
    // step capture (ormi_b200_capture_begin .. _end): blocks the pool hands out meanwhile, and the blocks live graphs own
    bool auto_graph = true;                // option "auto_graph": realize replays a plan's launches as a CUDA graph when the addresses repeat
    bool capturing = false;
    std::unordered_map<void*, size_t> capture_blocks;
    std::unordered_set<void*> graph_owned;
    bool pool_canary = false;              // option "pool_canary": a guard zone behind every block, checked when the block comes back
    std::unordered_map<void*, size_t> canaries;   // block -> bytes asked for, of the blocks that carry a guard zone
    std::unordered_set<void*> pooled;      // every block that sits in free_blocks: a block returned twice is caught, not handed to two owners

    std::unordered_map<std::string, ormi_b200::CompiledKernel> kernel_cache;   // source hash -> module
    std::unordered_map<std::string, std::unique_ptr<ormi_b200::CachedPlan>> plan_cache;   // by graph_key (runtime.cu)
    bool free_intermediates = false;   // option "intermediates": materialized nodes the caller does not hold are scratch
    int tune[ormi_b200::kTuneKnobs] = {};   // code-generator overrides (SchedOptions::tune), 0 = default

    ormi_b200::MatmulMode matmul_mode = ormi_b200::MatmulMode::FP32;
    bool fusion = true;

    // bf16 twins of fp32 matmul operands, by fp32 pointer (dropped when that buffer is freed or written through the ABI)
    std::unordered_map<const void*, ormi_b200::Shadow16> shadows;
    std::unordered_map<std::string, ormi_b200::TcKernel> tc_kernels;   // compiled variants of the tensor-core GEMM
    int tc_cta_group = 2;             // CTAs per tcgen05.mma of the bf16 GEMM: 2 = a pair of SMs per 256 x 256 tile
    bool tc_pair_auto = false;        // "auto": one SM per MMA while a collective of the second stream may run beside the GEMM (measured slower: off by default)
    int comm_inflight = 0;            // overlapped all-reduces queued and not yet waited for (host order = stream order)
    int comm_last_mark = -1;
    // kErrorWords ints: word 0 is the error word, word kTileCounterWord (its own 128-byte line) the GEMM's tile counter
    int* gemm_err = nullptr;          // device word: non-zero when a bounded wait inside the tensor-core GEMM ran out
    bool gemm_err_pending = false;    // a kernel with bounded waits was launched since the word was last read
    bool gemm_attr_set = false;

    std::map<std::string, int64_t> counters;
    void* nccl = nullptr;   // opaque: collective state (comm.cu)
    int comm_timeout_ms = 0;   // wall-clock deadline of collectives and of host waits behind them; 0 = ten minutes
};

namespace ormi_b200 {

void* pool_alloc(ormi_b200_ctx* ctx, size_t bytes);
void pool_free(ormi_b200_ctx* ctx, void* ptr, size_t bytes);

// NVRTC: CUDA C -> sm_100a cubin.  Throws Error with the compiler log on failure.  Needs no device.
std::vector<char> compile_cubin(const std::string& source, std::string* log = nullptr);

CompiledKernel* get_kernel(ormi_b200_ctx* ctx, const KernelStep& k);
void launch_kernel(ormi_b200_ctx* ctx, CompiledKernel* k, int grid, int block, std::vector<void*>& pointer_args, int dyn_smem = 0);
int* device_error_word(ormi_b200_ctx* ctx);

// GEMM launchers (gemm_ffma.cu, gemm_tcgen05.cu)
struct GemmArgs {
    const float* A; const float* B; float* C;
    int M, N, K;
    int trans_a, trans_b, lda, ldb;
    int batch, nbatch;
    int32_t bshape[ORMI_B200_MAX_DIMS];
    int64_t astride[ORMI_B200_MAX_DIMS], bstride[ORMI_B200_MAX_DIMS];
};
void gemm_ffma(ormi_b200_ctx* ctx, const GemmArgs& g);
void gemm_dispatch(ormi_b200_ctx* ctx, const GemmArgs& g);
void gemm_bf16(ormi_b200_ctx* ctx, const GemmArgs& g);
void gemm_tf32(ormi_b200_ctx* ctx, const GemmArgs& g, int parts);   // parts = 1: tf32, 3: 3xTF32 split
void selftest_wait_timeout(ormi_b200_ctx* ctx, int limit_ms);   // queues a wait that must run out (code 9)
void check_gemm_error(ormi_b200_ctx* ctx);   // throws when the tensor-core kernel reported a wait that ran out
void gemm_bf16_kmajor(ormi_b200_ctx* ctx, const void* a16, const void* b16, float* C, int M, int N, int Kp);
void cvt_bf16_kmajor(ormi_b200_ctx* ctx, const float* src, long long s_row, long long s_k, int rows, int K, void* dst);

// run-time compiled tensor-core GEMM on bf16 operands in their natural row-major layout (gemm_tc.cu)
bool gemm_tc_supported(const GemmArgs& g);
void gemm_tc(ormi_b200_ctx* ctx, const void* a16, int a_mn, const void* b16, int b_mn, float* C, int M, int N, int K,
             const TcEpilogue* epi = nullptr);
void gemm_tc_from_fp32(ormi_b200_ctx* ctx, const GemmArgs& g, const void* a16 = nullptr, const void* b16 = nullptr,
                       const TcEpilogue* epi = nullptr);
void cvt_bf16(ormi_b200_ctx* ctx, const float* src, long long ld, int rows, int cols, void* dst);
const void* shadow_of(ormi_b200_ctx* ctx, const float* src, int rows, int cols, long long ld);
const void* shadow_find(ormi_b200_ctx* ctx, const void* src, int rows, int cols, long long ld);
void shadow_register(ormi_b200_ctx* ctx, const void* src, void* p16, int rows, int cols, long long ld);
void shadow_drop(ormi_b200_ctx* ctx, const void* ptr, size_t bytes);

// collectives (comm.cu)
void comm_unique_id(char* out128);
void comm_init(ormi_b200_ctx* ctx, const char* id128, int rank, int world);
void comm_allreduce(ormi_b200_ctx* ctx, void* const* bufs, const size_t* counts, int n, int overlap);
void comm_join(ormi_b200_ctx* ctx);
void comm_mark(ormi_b200_ctx* ctx, int slot);
void comm_wait(ormi_b200_ctx* ctx, int slot);
void comm_destroy(ormi_b200_ctx* ctx);
void comm_guarded_sync(ormi_b200_ctx* ctx, cudaStream_t stream);   // cudaStreamSynchronize under the collective deadline

// `preassigned`: optional (node, pointer) pairs — write that node's value into a caller-owned buffer
// instead of a fresh pool block (used by the raw-buffer sum / matmul entry points).
void realize(ormi_b200_ctx* ctx, ormi_b200_node* nodes, int n_nodes, const int* roots, int n_roots,
             const std::vector<std::pair<int, void*>>* preassigned = nullptr);

}  // namespace ormi_b200
