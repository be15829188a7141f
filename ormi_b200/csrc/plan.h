// Execution plan of one realize call: what the fusion scheduler hands to the executor.
//
// The plan is device independent (it can be built and printed without a GPU): buffers are symbolic,
// kernels are CUDA C source plus launch geometry, GEMMs are described by their views.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "ormi_b200.h"

namespace ormi_b200 {

// Word of the context's error-word buffer where generated row kernels keep their row counter pair (the tensor-core GEMM
// keeps its tile counter in another line of the same buffer).
constexpr int kRowCounterWord = 48;

enum class BufKind { External, NodeOut, Temp, ErrorWord /* the context's device error word */,
                     Twin16 /* contiguous bf16 copy of a node's value, read by tensor-core matmuls */ };

struct PlanBuffer {
    BufKind kind;
    int     node;    // External: node whose `data` is read; NodeOut: node that owns the buffer afterwards; Twin16: the node copied
    int64_t bytes;
    int     rows = 0, cols = 0;   // Twin16: the matrix shape under which matmuls read it
};

struct KernelStep {
    std::string name;        // entry point
    std::string source;      // CUDA C (NVRTC)
    std::string key;         // cache key (hash of the source)
    int grid = 1, block = 1;
    int dyn_smem = 0;        // dynamic shared memory per block (bytes)
    bool err_arg = false;    // the kernel takes the device error word as its last argument
    std::vector<int> args;   // plan buffer ids, in kernel-argument order (every argument is a pointer)
    std::string what;        // human-readable summary (template, domain, outputs)
    int64_t bytes_read = 0, bytes_written = 0;   // algorithmic traffic of the launch
};

// C[b] = op(A[b]) op(B[b]) with the view semantics of ormi::cuda::matmul
// (ormi-core/csrc/backend/cuda/kernels/blas/matmul.cu:29-79).
struct GemmStep {
    int a = -1, b = -1, c = -1;          // plan buffer ids
    int M = 0, N = 0, K = 0;
    int trans_a = 0, trans_b = 0;        // operand stored transposed (last-dimension stride != 1)
    int lda = 0, ldb = 0;
    int batch = 1;
    int nbatch = 0;                      // number of leading (batch) dims of the output
    int32_t bshape[ORMI_B200_MAX_DIMS] = {0};
    int64_t astride[ORMI_B200_MAX_DIMS] = {0};   // per output batch dim; 0 = broadcast
    int64_t bstride[ORMI_B200_MAX_DIMS] = {0};
    int node = -1;
    // "bf16" matmul arithmetic on the run-time compiled tensor-core kernel (gemm_tc.cu)
    bool tc = false;                     // the shapes qualify (decided when the plan is built)
    int a16 = -1, b16 = -1;              // Twin16 plan buffers written earlier in the plan (-1: the context's twin cache, or a conversion)
    bool store_c = true;                 // write the fp32 product to `c`
    bool has_epi = false;                // pointwise work fused behind the accumulator
    std::string epi_prelude, epi_params, epi_init, epi_cols, epi_pre, epi_body, epi_end, epi_what;
    int epi_wpq = 1, epi_unroll = 8;
    std::vector<int> epi_args;           // plan buffer ids, in the epilogue's parameter order
};

struct Step {
    enum Type { Kernel, Gemm } type = Kernel;
    KernelStep k;
    GemmStep g;
};

struct NodeResult {
    int node;
    int buffer;     // plan buffer id holding the node's value
    bool alias;     // view: shares the buffer of its base
    bool bf16 = false;   // the buffer is the node's bf16-only form (ORMI_NODE_BF16)
};

struct Plan {
    std::vector<PlanBuffer> buffers;
    std::vector<Step> steps;
    std::vector<NodeResult> results;   // nodes that receive `data` when the plan has run
    std::string error;                 // non-empty: scheduling failed
};

// Overrides of the code generator's measured defaults, for experiments (ormi_b200_set_option "tune.<name>"); 0 keeps the
// default.  They are part of the plan key.
enum TuneKnob { TUNE_ROWS_VPT = 0, TUNE_ROWS_MINB, TUNE_ROWS_GRID, TUNE_ROWS_STAGE /* 1 off, 2 on */, TUNE_ROWS_NSTAGE,
                TUNE_ROWS_DYNAMIC /* 1 off, 2 on */, TUNE_FLAT_UNROLL, TUNE_ROWS_HOIST /* 1 off, 2 on */,
                TUNE_EPI_UNROLL /* unrolled row steps of a GEMM epilogue chunk: 1, 2, 4, 8 */, TUNE_EPI_WPQ /* epilogue warps per quarter: 1, 2, 4 */,
                TUNE_GEMM_BN /* columns per tensor-core GEMM tile: 128, 256 */,
                TUNE_EPI_NODE_MAJOR /* GEMM epilogue text node by node over the four columns: 1 off, 2 on */ };
constexpr int kTuneKnobs = 12;

struct SchedOptions {
    int  num_sms = 148;
    bool fusion = true;
    bool bf16_matmul = false;   // matmuls run on the tensor-core kernel: fuse epilogues, let producers write bf16 twins
    bool aligned = true;        // every realized input starts on a 16-byte boundary (else: no 128-bit accesses, no bulk copies)
    bool free_intermediates = false;   // materialized nodes the caller does not hold (no root, no KEEP) are scratch of the call
    int  tune[kTuneKnobs] = {};
};

Plan build_plan(const ormi_b200_node* nodes, int n_nodes, const int* roots, int n_roots, const SchedOptions& opt);
// "rows_vpt" -> TUNE_ROWS_VPT, ...; -1 for a name that is no knob.
int tune_knob_index(const std::string& name);
// "matmul=bf16,fusion=on,intermediates=free,aligned=0,tune.rows_vpt=8": the schedule-shaping options as one string (what
// ormi_b200_plan_json_opts takes).  Throws std::runtime_error on an unknown key.
SchedOptions parse_sched_options(const char* text);
std::string plan_to_json(const Plan& plan);

// The reference-shaped single-kernel compiler (ormi::cuda::compile): guarded scalar `fused_kernel`.
struct SimpleKernel {
    std::string source;
    std::vector<int> leaves;   // node indices in LEAF_i order
    int tensor_size = 0;
    std::string error;
};
SimpleKernel compile_simple(const ormi_b200_node* nodes, int n_nodes, int root);

// Process-wide overrides of the expression emitted for a pointwise op (ormi_b200_set_lowering); `$0`, `$1` stand for
// the operands.  lowering_generation() changes with every edit and is part of the plan key.
void set_lowering(int op, const std::string& expr);
bool lowering_for(int op, std::string* expr);
uint64_t lowering_generation();

uint64_t fnv1a(const std::string& s);
std::string device_prelude();

}  // namespace ormi_b200
