// What the scheduler tells the code generator about one fused kernel.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "plan.h"

namespace ormi_b200 {

struct KRef {
    enum T { NODE, LOAD } t;
    int id;   // NODE: graph node index; LOAD: index into KernelSpec::loads
};

// A read of a realized (or materialized) buffer, addressed by the kernel's domain coordinates.
struct KLoad {
    int src_node;               // node whose buffer is read
    std::vector<int64_t> st;    // element stride per domain dim (0 = broadcast)
    bool acc = false;           // GEMM epilogue only: the value is the accumulator of the matmul, not a memory read
};

struct KNode {
    enum { OP_ROWSUM = 1000, OP_ID = 1001 };
    int node;
    int op;                     // ormi_b200_op of a pointwise node, OP_ROWSUM or OP_ID
    bool row;                   // one value per row (row sum or pointwise work on row sums)
    bool scalar = false;        // one value for the whole domain (arithmetic on rank-0 operands)
    bool is_max = false;        // OP_ROWSUM only: the reduction keeps the maximum instead of adding (ORMI_OP_MAX)
    std::vector<KRef> operands;
};

struct KOutput {
    enum Kind { FULL, ROW, COLSUM, GLOBALSUM } kind;
    int node;                   // materialized node (-1: anonymous gather target)
    KRef value;                 // what is stored (FULL/ROW) or accumulated (COLSUM/GLOBALSUM)
    bool is_max = false;        // COLSUM/GLOBALSUM: keep the maximum instead of adding (ORMI_OP_MAX)
    // FULL only: `store` = write the fp32 values; `twin` = also (or only) write a contiguous bf16 copy, the form in
    // which a tensor-core matmul of the same plan reads this node.  Argument order: fp32 pointer (if store), then
    // bf16 pointer (if twin).
    bool store = true;
    bool twin = false;
};

struct KernelSpec {
    std::vector<int> D;         // squeezed domain
    int k = -1;                 // rows = D[:k], columns = D[k:]; -1 = no row/column structure needed
    std::vector<KLoad> loads;
    std::vector<KNode> nodes;   // in topological (index) order
    std::vector<KOutput> outputs;
    int num_sms = 148;
    bool aligned = true;        // every buffer starts on a 16-byte boundary (else scalar accesses only, no bulk copies)
    int tune[kTuneKnobs] = {};   // SchedOptions::tune
};

struct GeneratedKernel {
    KernelStep step;            // args left empty: the scheduler binds buffers
    int64_t cols = 0;           // row template: number of columns (size of one column-sum partial)
    bool unsupported_sums = false;
    std::string error;
};

// Argument order of a generated fused kernel: one pointer per load (in order), then one per output
// (FULL/ROW: the output buffer; COLSUM/GLOBALSUM: a scratch buffer of grid x {cols|1} partials).
GeneratedKernel generate_kernel(const KernelSpec& spec, const std::string& name, const ormi_b200_node* nodes);
// Epilogue of the run-time compiled tensor-core GEMM: the pointwise work of `spec` (domain [M, N], every output FULL)
// on the accumulator, as text for the kernel template.  The load flagged `acc` is the matmul itself; `store_c` /
// `twin_c` say whether the raw product is written as fp32 / as bf16.  A COLSUM output leaves one partial row per
// 32-row block of the product ([ceil(M / 32) rounded up to whole tiles][N] floats, added up by a finalize kernel).
// Kernel-argument order: every other load in order, then per output the fp32 pointer (if store; for a COLSUM the
// partial buffer) and the bf16 pointer (if twin), then the product's bf16 pointer (if twin_c).
struct GeneratedEpilogue {
    std::string prelude, params, init, cols, pre, body, end;   // pre: per row step, before the bounds guard of body
    int wpq = 1;
    int unroll = 8;             // how many of the 8 row steps of a chunk are unrolled (heavy bodies: 1, for the instruction cache)
    std::string error;
};
GeneratedEpilogue generate_gemm_epilogue(const KernelSpec& spec, bool store_c, bool twin_c);

// out[c] = sum over p < parts of partial[p * width + c]   (fixed order: deterministic)
// `count` > 1: one launch adds up `count` partial buffers of the same geometry (arguments: part0, out0, part1, out1, ...;
// is_max then holds one flag per pair, packed as bits).
GeneratedKernel generate_finalize(int parts, int64_t width, const std::string& name, bool is_max = false, int count = 1, unsigned max_bits = 0);
// One thread per output element, serial sum over the reduced coordinates, arbitrary input strides.
GeneratedKernel generate_generic_sum(const std::vector<int>& shape, const std::vector<int>& strides,
                                     const std::vector<bool>& reduced, const std::string& name, bool is_max = false);

}  // namespace ormi_b200
