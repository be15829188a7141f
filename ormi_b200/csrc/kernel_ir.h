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
};

struct KernelSpec {
    std::vector<int> D;         // squeezed domain
    int k = -1;                 // rows = D[:k], columns = D[k:]; -1 = no row/column structure needed
    std::vector<KLoad> loads;
    std::vector<KNode> nodes;   // in topological (index) order
    std::vector<KOutput> outputs;
    int num_sms = 148;
    // rows template tuning: elements per thread (0 = default), keep row-invariant vectors in registers,
    // minimum resident blocks per SM for __launch_bounds__ (0 = none), blocks per SM in the grid (0 = default)
    int tune_vpt = 0;
    int tune_hoist = 1;
    int tune_minblocks = 0;
    int tune_grid = 0;
    int tune_stage = -1;        // stage row operands through shared memory with bulk async copies (-1 = automatic)
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
// out[c] = sum over p < parts of partial[p * width + c]   (fixed order: deterministic)
GeneratedKernel generate_finalize(int parts, int64_t width, const std::string& name, bool is_max = false);
// One thread per output element, serial sum over the reduced coordinates, arbitrary input strides.
GeneratedKernel generate_generic_sum(const std::vector<int>& shape, const std::vector<int>& strides,
                                     const std::vector<bool>& reduced, const std::string& name, bool is_max = false);

}  // namespace ormi_b200
