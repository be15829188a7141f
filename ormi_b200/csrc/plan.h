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

enum class BufKind { External, NodeOut, Temp, ErrorWord /* the context's device error word */ };

struct PlanBuffer {
    BufKind kind;
    int     node;    // External: node whose `data` is read; NodeOut: node that owns the buffer afterwards
    int64_t bytes;
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
};

struct Plan {
    std::vector<PlanBuffer> buffers;
    std::vector<Step> steps;
    std::vector<NodeResult> results;   // nodes that receive `data` when the plan has run
    std::string error;                 // non-empty: scheduling failed
};

struct SchedOptions {
    int  num_sms = 148;
    bool fusion = true;
};

Plan build_plan(const ormi_b200_node* nodes, int n_nodes, const int* roots, int n_roots, const SchedOptions& opt);
std::string plan_to_json(const Plan& plan);

// The reference-shaped single-kernel compiler (ormi::cuda::compile): guarded scalar `fused_kernel`.
struct SimpleKernel {
    std::string source;
    std::vector<int> leaves;   // node indices in LEAF_i order
    int tensor_size = 0;
    std::string error;
};
SimpleKernel compile_simple(const ormi_b200_node* nodes, int n_nodes, int root);

uint64_t fnv1a(const std::string& s);
std::string device_prelude();

}  // namespace ormi_b200
