// Fusion scheduler of the realize path.
//
// Replaces the CUDA branch of ormi::execute_graph (ormi-core/csrc/backend/runtime.cpp:13-39), which
// realizes every parent first and therefore runs one kernel per node, and the graph walk of
// ormi::cuda::compile / build_ir (ormi-core/csrc/backend/cuda/compiler.cu:22-51).
//
// Input:  the flattened lazy graph (ormi_b200_node[], topologically ordered).
// Output: a Plan — a handful of generated kernels, GEMM steps and the buffers that connect them.
//
// Method
//   1. classify every node: realized input, view, pointwise, SUM (row / column / global / generic), MATMUL;
//   2. give every un-realized compute node a *domain* (a squeezed shape D and a split k: rows = D[:k],
//      columns = D[k:]) — a row SUM lives in the domain of its operand, and pointwise work on row sums
//      stays in that domain too (that is what makes softmax / layernorm one kernel);
//   3. decide which nodes must be written to memory (roots, externally held nodes, MATMUL operands and
//      results, column/global sums, anything reached through a view that is not a plain
//      broadcast/permutation-free mapping).  Everything else is recomputed inside the kernel that needs it;
//   4. merge materialized nodes of one domain into multi-output kernels when that creates no cycle;
//   5. emit each kernel (codegen.cpp) and order the steps topologically.
#include <algorithm>
#include <cstring>
#include <functional>
#include <map>
#include <set>
#include <sstream>
#include <stdexcept>

#include "kernel_ir.h"
#include "plan.h"

namespace ormi_b200 {

namespace {

bool is_view_op(int op) { return op == ORMI_OP_TRANSPOSE || op == ORMI_OP_RESHAPE || op == ORMI_OP_EXPAND; }
bool is_pw_op(int op) { return (op >= ORMI_OP_NEG && op <= ORMI_OP_POW) || op == ORMI_OP_MAXIMUM || op == ORMI_OP_GE; }
bool is_reduce_op(int op) { return op == ORMI_OP_SUM || op == ORMI_OP_MAX; }

enum Kind { K_NONE, K_INPUT, K_VIEW, K_PW, K_IDSUM, K_ROWSUM, K_COLSUM, K_GLOBALSUM, K_GENSUM, K_MATMUL };

struct Info {
    Kind kind = K_NONE;
    bool needed = false;
    std::vector<int> shape, strides, sq;
    int64_t numel = 1;
    int base = -1;                 // K_VIEW: first non-view ancestor
    std::vector<int> vmap;         // K_VIEW over an un-realized base: view dim -> base dim, or -1
    bool vmap_ok = false;
    std::vector<int> D;            // domain of an un-realized compute node
    int k = -1;                    // split; -1: any
    bool row_cls = false;          // value per row (row sum, or pointwise work on row sums)
    bool in_M = false;             // materialized
    bool bf16_in = false;          // realized input whose buffer holds bf16 (ORMI_NODE_BF16): a matmul operand only
    int step = -1;                 // step that produces it
};

std::vector<int> squeeze(const std::vector<int>& s) {
    std::vector<int> r;
    for (int v : s) if (v != 1) r.push_back(v);
    return r;
}

std::vector<int> contiguous(const std::vector<int>& shape) {
    std::vector<int> st(shape.size(), 1);
    for (int i = (int)shape.size() - 2; i >= 0; --i) st[i] = st[i + 1] * shape[i + 1];
    return st;
}

// canonical dim map of a value with `shape` inside a domain: the non-1 dims, in order, are driven by
// domain dims 0,1,2,...
std::vector<int> canonical_dm(const std::vector<int>& shape) {
    std::vector<int> dm(shape.size(), -1);
    int next = 0;
    for (size_t j = 0; j < shape.size(); ++j) if (shape[j] != 1) dm[j] = next++;
    return dm;
}

// One operand of a MATMUL as the kernel sees it: source buffer, the matrix (rows x cols of the operand), strides.
struct OperandView {
    int src = -1;
    std::vector<int> sh, st;
    int rows = 0, cols = 0, s_row = 0, s_col = 0;
    bool ok_n = false, ok_t = false;   // rows contiguous / columns contiguous
    // the stored matrix behind the operand: [srows][scols] with pitch ld (the operand itself, or its transpose)
    int srows = 0, scols = 0, ld = 0;
    bool dense = false;                // the stored matrix is the whole source buffer, contiguous
};

struct Scheduler {
    const ormi_b200_node* nodes;
    int n;
    SchedOptions opt;
    std::vector<Info> info;
    std::set<int> force_generic;   // SUM nodes the fused templates could not take
    std::string error;

    struct Dep { int node; bool mergeable; };

    Scheduler(const ormi_b200_node* nd, int count, const SchedOptions& o) : nodes(nd), n(count), opt(o) {}

    bool fail(const std::string& msg) { if (error.empty()) error = msg; return false; }

    // ------------------------------------------------------------------ classification
    bool classify(const int* roots, int n_roots) {
        info.assign(n, Info());
        for (int i = 0; i < n; ++i) {
            const auto& nd = nodes[i];
            if (nd.ndim < 0 || nd.ndim > ORMI_B200_MAX_DIMS) return fail("node with a bad rank");
            Info& I = info[i];
            I.shape.assign(nd.shape, nd.shape + nd.ndim);
            I.strides.assign(nd.strides, nd.strides + nd.ndim);
            I.sq = squeeze(I.shape);
            for (int s : I.shape) { if (s <= 0) return fail("empty or negative dimension"); I.numel *= s; }
            // Generated kernels index with 32-bit ints.  A grid-stride loop steps past the end by up to one grid of
            // vector accesses (at most 148 * 8 blocks * 256 threads * 4 elements = 2^21 * 0.58) before its bound check,
            // and strided views are addressed by their extent, not their element count: both must stay below 2^31.
            constexpr int64_t kIndexLimit = (int64_t(1) << 31) - (int64_t(1) << 22);
            if (I.numel >= kIndexLimit) return fail("tensor with 2^31 or more elements (the limit is 2^31 - 2^22: index arithmetic is 32-bit)");
            int64_t extent = 1;
            for (size_t d = 0; d < I.shape.size(); ++d) extent += (int64_t)(I.shape[d] - 1) * (I.strides[d] < 0 ? -(int64_t)I.strides[d] : (int64_t)I.strides[d]);
            if (extent >= kIndexLimit) return fail("tensor view that spans 2^31 or more elements (index arithmetic is 32-bit)");
            for (int p = 0; p < nd.n_parents; ++p)
                if (nd.parents[p] < 0 || nd.parents[p] >= i) return fail("graph is not in topological order");
        }
        // needed set
        std::vector<int> stack(roots, roots + n_roots);
        while (!stack.empty()) {
            int i = stack.back(); stack.pop_back();
            if (i < 0 || i >= n) return fail("root index out of range");
            if (info[i].needed) continue;
            info[i].needed = true;
            if (nodes[i].data) continue;
            for (int p = 0; p < nodes[i].n_parents; ++p) stack.push_back(nodes[i].parents[p]);
        }
        for (int i = 0; i < n; ++i) {
            Info& I = info[i];
            if (!I.needed) continue;
            const auto& nd = nodes[i];
            if (nd.data) { I.kind = K_INPUT; I.bf16_in = (nd.flags & ORMI_NODE_BF16) != 0; continue; }
            if (nd.op == ORMI_OP_LEAF || nd.op == ORMI_OP_CONST) return fail("leaf without data");
            if (is_view_op(nd.op)) {
                if (nd.n_parents != 1) return fail("view op needs one parent");
                I.kind = K_VIEW;
                int p = nd.parents[0];
                I.base = info[p].kind == K_VIEW ? info[p].base : p;
                if (info[I.base].kind != K_INPUT) compute_vmap(i);
                continue;
            }
            if (nd.op == ORMI_OP_MATMUL) { if (nd.n_parents != 2) return fail("MATMUL needs two parents"); I.kind = K_MATMUL; continue; }
            if (is_reduce_op(nd.op)) { if (nd.n_parents != 1) return fail("SUM needs one parent"); if (!classify_sum(i)) return false; continue; }
            if (is_pw_op(nd.op)) {
                int want = (nd.op <= ORMI_OP_COS) ? 1 : 2;
                if (nd.n_parents != want) return fail("pointwise op with a wrong operand count");
                I.kind = K_PW;
                classify_pw(i);
                continue;
            }
            return fail("op " + std::to_string(nd.op) + " has no CUDA lowering");
        }
        return true;
    }

    // view dims -> dims of the (contiguous, once materialized) base
    void compute_vmap(int v) {
        Info& V = info[v];
        const Info& B = info[V.base];
        std::vector<int> cs = contiguous(B.shape);
        V.vmap.assign(V.shape.size(), -1);
        std::vector<bool> used(B.shape.size(), false);
        bool ok = true;
        for (size_t j = 0; j < V.shape.size() && ok; ++j) {
            if (V.shape[j] == 1 || V.strides[j] == 0) continue;
            bool found = false;
            for (size_t d = 0; d < B.shape.size(); ++d) {
                if (!used[d] && B.shape[d] != 1 && cs[d] == V.strides[j] && B.shape[d] == V.shape[j]) {
                    used[d] = true; V.vmap[j] = (int)d; found = true; break;
                }
            }
            if (!found) ok = false;
        }
        for (size_t d = 0; d < B.shape.size() && ok; ++d) if (B.shape[d] != 1 && !used[d]) ok = false;
        V.vmap_ok = ok;
    }

    bool classify_sum(int i) {
        Info& I = info[i];
        const auto& nd = nodes[i];
        int p = nd.parents[0];
        const Info& P = info[p];
        std::vector<bool> red(P.shape.size(), nd.n_axes == 0);
        for (int a = 0; a < nd.n_axes; ++a) {
            if (nd.axes[a] < 0 || nd.axes[a] >= (int)P.shape.size()) return fail("SUM axis out of range");
            red[nd.axes[a]] = true;
        }
        int64_t kept = 1;
        for (size_t d = 0; d < P.shape.size(); ++d) if (!red[d]) kept *= P.shape[d];
        if (kept != I.numel) return fail("SUM output shape does not match its axes");
        std::vector<bool> sred;
        for (size_t d = 0; d < P.shape.size(); ++d) if (P.shape[d] != 1) sred.push_back(red[d]);
        int nd_sq = (int)sred.size(), nred = 0;
        for (bool b : sred) nred += b;
        I.D = P.sq;
        bool parent_plain = (P.kind != K_VIEW) && !force_generic.count(i) && opt.fusion;
        if (nred == 0) { I.kind = K_IDSUM; I.k = -1; if (P.kind == K_VIEW || !opt.fusion) { I.kind = K_GENSUM; } return inherit_idsum(i); }
        if (!parent_plain) { I.kind = K_GENSUM; return true; }
        if (nred == nd_sq) { I.kind = K_GLOBALSUM; I.k = -1; return true; }
        bool trailing = true, leading = true;
        for (int d = 0; d < nd_sq; ++d) {
            if (sred[d] != (d >= nd_sq - nred)) trailing = false;
            if (sred[d] != (d < nred)) leading = false;
        }
        if (trailing) { I.kind = K_ROWSUM; I.k = nd_sq - nred; I.row_cls = true; return true; }
        if (leading) { I.kind = K_COLSUM; I.k = nred; return true; }
        I.kind = K_GENSUM;
        return true;
    }

    // a SUM over size-1 axes copies its operand: it behaves like a unary pointwise op
    bool inherit_idsum(int i) {
        Info& I = info[i];
        if (I.kind != K_IDSUM) return true;
        const Info& P = info[nodes[i].parents[0]];
        I.D = I.sq;
        if ((P.kind == K_PW || P.kind == K_IDSUM || P.kind == K_ROWSUM) && !P.D.empty()) {
            if (P.row_cls && std::vector<int>(P.D.begin(), P.D.begin() + P.k) == I.sq && P.D != I.sq) { I.D = P.D; I.k = P.k; I.row_cls = true; }
            else if (P.D == I.sq) I.k = P.k;
        }
        return true;
    }

    // un-realized compute operand behind an operand index (through plain views), or -1
    int compute_base(int o) const {
        const Info& O = info[o];
        if (O.kind == K_VIEW) {
            if (info[O.base].kind == K_INPUT || !O.vmap_ok) return -1;
            return O.base;
        }
        if (O.kind == K_INPUT) return -1;
        return o;
    }

    void classify_pw(int i) {
        Info& I = info[i];
        I.D = I.sq;
        I.k = -1;
        I.row_cls = false;
        if (!opt.fusion) return;
        const auto& nd = nodes[i];
        bool full_match = false;
        int row_src = -1;
        for (int p = 0; p < nd.n_parents; ++p) {
            int q = compute_base(nd.parents[p]);
            if (q < 0) continue;
            const Info& Q = info[q];
            if (Q.kind != K_PW && Q.kind != K_ROWSUM && Q.kind != K_IDSUM) continue;
            if (Q.D == I.sq) { full_match = true; if (I.k < 0 && Q.k >= 0) I.k = Q.k; }
            else if (Q.row_cls && Q.k >= 0 && std::vector<int>(Q.D.begin(), Q.D.begin() + Q.k) == I.sq && row_src < 0) row_src = q;
        }
        if (!full_match && row_src >= 0) { I.D = info[row_src].D; I.k = info[row_src].k; I.row_cls = true; }
    }

    // ------------------------------------------------------------------ walking one kernel
    struct Walk {
        std::vector<int> D; int k;
        std::set<int> outputs;                 // M nodes computed by this kernel
        std::vector<int> members;              // in-kernel nodes (sorted later)
        std::set<int> member_set;
        std::vector<KLoad> loads;
        std::map<int, std::vector<KRef>> operands;   // node -> operand refs
        std::vector<Dep> deps;                 // un-realized boundary nodes
        bool k_conflict = false;
    };

    static std::vector<int64_t> strides_over_domain(const std::vector<int>& dm, const std::vector<int>& st, size_t nd) {
        std::vector<int64_t> r(nd, 0);
        for (size_t j = 0; j < dm.size(); ++j) if (dm[j] >= 0) r[dm[j]] += st[j];
        return r;
    }

    int add_load(Walk& w, int src, const std::vector<int64_t>& st) {
        for (size_t i = 0; i < w.loads.size(); ++i) if (w.loads[i].src_node == src && w.loads[i].st == st) return (int)i;
        w.loads.push_back(KLoad{src, st});
        return (int)w.loads.size() - 1;
    }

    bool k_compatible(int a, int b) const { return a < 0 || b < 0 || a == b; }

    // Is compute node q, reached with dim map dm, a value this kernel can hold in registers?
    bool eligible(const Walk& w, int q, const std::vector<int>& dm) const {
        const Info& Q = info[q];
        if (!opt.fusion) return false;
        if (Q.kind != K_PW && Q.kind != K_ROWSUM && Q.kind != K_IDSUM) return false;
        if ((Q.kind == K_PW || Q.kind == K_IDSUM) && Q.numel == 1) return true;   // scalar arithmetic rides along in any kernel
        if (Q.D != w.D || !k_compatible(Q.k, w.k)) return false;
        if (dm != canonical_dm(Q.shape)) return false;
        if (Q.row_cls) {
            if (Q.k < 0 || (int)Q.sq.size() != Q.k) return false;
        } else if (Q.sq != w.D) return false;
        return true;
    }

    // Resolves operand `o` (seen with dim map dm over o's own dims) into a register value or a load.
    KRef resolve(Walk& w, int o, const std::vector<int>& dm, bool discover) {
        const Info& O = info[o];
        size_t nd = w.D.size();
        if (O.kind == K_INPUT) {
            if (O.bf16_in) fail("a bf16 tensor can only be an operand of a tensor-core matmul");
            std::vector<int64_t> st(nd, 0);
            if (!(O.shape.empty() || nodes[o].data_bytes == 4)) st = strides_over_domain(dm, O.strides, nd);
            return KRef{KRef::LOAD, add_load(w, o, st)};
        }
        if (O.kind == K_VIEW) {
            int b = O.base;
            const Info& B = info[b];
            if (B.kind == K_INPUT && B.bf16_in) fail("a bf16 tensor can only be an operand of a tensor-core matmul");
            if (B.kind == K_INPUT) {
                std::vector<int64_t> st(nd, 0);
                if (nodes[b].data_bytes != 4) st = strides_over_domain(dm, O.strides, nd);
                return KRef{KRef::LOAD, add_load(w, b, st)};
            }
            if (O.vmap_ok) {
                std::vector<int> dmb(B.shape.size(), -1);
                for (size_t j = 0; j < O.vmap.size(); ++j) if (O.vmap[j] >= 0) dmb[O.vmap[j]] = dm[j];
                if (eligible(w, b, dmb) && (!info[b].in_M || w.outputs.count(b))) return enter(w, b, discover);
                bool mergeable = eligible(w, b, dmb);
                return boundary(w, b, strides_over_domain(dm, O.strides, nd), mergeable, discover);
            }
            return boundary(w, b, strides_over_domain(dm, O.strides, nd), false, discover);
        }
        // un-realized compute node
        if (eligible(w, o, dm) && (!O.in_M || w.outputs.count(o))) return enter(w, o, discover);
        return boundary(w, o, strides_over_domain(dm, contiguous(O.shape), nd), eligible(w, o, dm), discover);
    }

    KRef boundary(Walk& w, int q, const std::vector<int64_t>& st, bool mergeable, bool discover) {
        if (discover) info[q].in_M = true;
        bool seen = false;
        for (auto& d : w.deps) if (d.node == q) { seen = true; d.mergeable = d.mergeable && mergeable; }
        if (!seen) w.deps.push_back(Dep{q, mergeable});
        return KRef{KRef::LOAD, add_load(w, q, st)};
    }

    KRef enter(Walk& w, int q, bool discover) {
        if (!w.member_set.count(q)) {
            w.member_set.insert(q);
            const Info& Q = info[q];
            if (Q.k >= 0) { if (w.k < 0) w.k = Q.k; else if (w.k != Q.k) w.k_conflict = true; }
            std::vector<KRef> ops;
            const auto& nd = nodes[q];
            if (Q.kind == K_PW) {
                std::vector<int> dmq = canonical_dm(Q.shape);
                for (int p = 0; p < nd.n_parents; ++p) {
                    const Info& P = info[nd.parents[p]];
                    int off = (int)Q.shape.size() - (int)P.shape.size();
                    std::vector<int> dmo(P.shape.size(), -1);
                    for (size_t j = 0; j < P.shape.size(); ++j) dmo[j] = (P.shape[j] == 1) ? -1 : dmq[j + off];
                    ops.push_back(resolve(w, nd.parents[p], dmo, discover));
                }
            } else {  // K_ROWSUM / K_IDSUM: the operand is seen in its own canonical layout
                const Info& P = info[nd.parents[0]];
                ops.push_back(resolve(w, nd.parents[0], canonical_dm(P.shape), discover));
            }
            w.operands[q] = ops;
            w.members.push_back(q);
        }
        return KRef{KRef::NODE, q};
    }

    // domain of the kernel that computes materialized node m
    void kernel_domain(int m, std::vector<int>& D, int& k) const {
        const Info& I = info[m];
        D = I.D; k = I.k;
    }

    // value of a terminal sum's operand (register value or load)
    KRef sum_operand(Walk& w, int m, bool discover) {
        int p = nodes[m].parents[0];
        return resolve(w, p, canonical_dm(info[p].shape), discover);
    }

    void walk_output(Walk& w, int m, bool discover, std::vector<KOutput>* outs) {
        const Info& I = info[m];
        KOutput o;
        o.node = m;
        o.is_max = nodes[m].op == ORMI_OP_MAX;
        if (I.kind == K_PW || I.kind == K_IDSUM || I.kind == K_ROWSUM) {
            o.kind = I.row_cls ? KOutput::ROW : KOutput::FULL;
            o.value = enter(w, m, discover);
        } else if (I.kind == K_COLSUM) {
            o.kind = KOutput::COLSUM;
            if (w.k < 0) w.k = I.k; else if (w.k != I.k) w.k_conflict = true;
            o.value = sum_operand(w, m, discover);
        } else {  // K_GLOBALSUM
            o.kind = KOutput::GLOBALSUM;
            o.value = sum_operand(w, m, discover);
        }
        if (outs) outs->push_back(o);
    }

    bool fusable_output(int m) const {
        Kind kd = info[m].kind;
        return kd == K_PW || kd == K_IDSUM || kd == K_ROWSUM || kd == K_COLSUM || kd == K_GLOBALSUM;
    }

    // source buffer + logical view of a MATMUL / generic-SUM operand; marks bases for materialization
    void operand_view(int o, int& src, std::vector<int>& shape, std::vector<int>& strides, bool discover) {
        const Info& O = info[o];
        shape = O.shape;
        if (O.kind == K_INPUT) { src = o; strides = O.strides; return; }
        if (O.kind == K_VIEW) { src = O.base; strides = O.strides; if (info[src].kind != K_INPUT && discover) info[src].in_M = true; return; }
        src = o; strides = contiguous(O.shape);
        if (discover) info[o].in_M = true;
    }

    OperandView matmul_operand(int o, bool discover) {
        OperandView v;
        operand_view(o, v.src, v.sh, v.st, discover);
        const int nd = (int)v.sh.size();
        if (nd < 2) return v;
        v.rows = v.sh[nd - 2]; v.cols = v.sh[nd - 1];
        v.s_row = v.st[nd - 2]; v.s_col = v.st[nd - 1];
        v.ok_n = (v.s_col == 1 || v.cols == 1) && (v.rows == 1 || v.s_row >= v.cols);
        v.ok_t = (v.s_row == 1 || v.rows == 1) && (v.cols == 1 || v.s_col >= v.rows);
        if (v.ok_n) { v.srows = v.rows; v.scols = v.cols; v.ld = v.s_row; }
        else if (v.ok_t) { v.srows = v.cols; v.scols = v.rows; v.ld = v.s_col; }
        v.dense = (v.ok_n || v.ok_t) && v.rows > 1 && v.cols > 1 && v.ld == v.scols &&
                  (int64_t)v.srows * v.scols == info[v.src].numel;
        return v;
    }

    // Does MATMUL node m qualify for the tensor-core kernel (gemm_tc.cu)?  One product (no batch), large enough to be
    // worth it, both operands row- or column-contiguous with a contiguous dimension of whole 16-byte pieces of bf16.
    bool tc_eligible(int m) {
        if (!opt.bf16_matmul || !opt.aligned || info[m].kind != K_MATMUL) return false;
        const auto& nd = nodes[m];
        OperandView a = matmul_operand(nd.parents[0], false), b = matmul_operand(nd.parents[1], false);
        if (a.sh.size() < 2 || b.sh.size() < 2) return false;
        int64_t batch = 1;
        for (size_t d = 0; d + 2 < info[m].shape.size(); ++d) batch *= info[m].shape[d];
        const int64_t M = a.rows, K = a.cols, N = b.cols;
        if (batch != 1 || b.rows != K || M * N * K < (int64_t(1) << 21) || K < 64 || N % 4 != 0) return false;
        for (const OperandView* v : {&a, &b}) {
            if (!(v->ok_n || v->ok_t) || v->rows <= 1 || v->cols <= 1 || v->scols % 8 != 0 || v->ld % 8 != 0) return false;
            for (size_t d = 0; d + 2 < v->sh.size(); ++d) if (v->sh[d] != 1) return false;
        }
        return true;
    }

    // ------------------------------------------------------------------ the plan
    Plan run(const int* roots, int n_roots);
};

struct StepNode {
    enum T { FUSED, GEMM, GENSUM } type;
    std::vector<int> outputs;     // M nodes
    std::vector<int> D; int k = -1;
    std::set<int> succ;
    bool dead = false;            // FUSED: absorbed into a GEMM step as its epilogue
    std::vector<int> epi_outputs; // GEMM: outputs of the absorbed step
    bool tc = false;              // GEMM: runs on the tensor-core kernel (decided from shapes and options)
};


Plan Scheduler::run(const int* roots, int n_roots) {
    Plan plan;
    if (!classify(roots, n_roots)) { plan.error = error; return plan; }

    // ---- 3. materialization set
    std::vector<bool> handed(n, false);     // roots, KEEP nodes and the bases of such views: the caller receives these
    for (int r = 0; r < n_roots; ++r) {
        int i = roots[r];
        if (info[i].kind == K_INPUT) continue;
        int b = info[i].kind == K_VIEW ? info[i].base : i;
        if (info[b].kind != K_INPUT) { info[b].in_M = true; handed[b] = true; }
    }
    for (int i = 0; i < n; ++i) {
        if (!info[i].needed || info[i].kind == K_INPUT) continue;
        if (nodes[i].flags & ORMI_NODE_KEEP) {
            int b = info[i].kind == K_VIEW ? info[i].base : i;
            if (info[b].kind != K_INPUT) { info[b].in_M = true; handed[b] = true; }
        }
        if (info[i].kind == K_MATMUL || info[i].kind == K_GENSUM || info[i].kind == K_COLSUM || info[i].kind == K_GLOBALSUM) info[i].in_M = true;
        if (!opt.fusion && info[i].kind != K_VIEW) info[i].in_M = true;
    }
    // Discovery runs from the last node to the first: a walk only ever marks nodes with a lower index, so
    // every materialized node is visited after it was marked.  The dependency lists are taken in a second
    // sweep, once the set is final (a node walked through here may have been materialized later on).
    std::vector<std::vector<Dep>> deps(n);
    for (int pass = 0; pass < 2; ++pass)
    for (int m = n - 1; m >= 0; --m) {
        if (!info[m].in_M) continue;
        if (fusable_output(m)) {
            Walk w; kernel_domain(m, w.D, w.k);
            w.outputs.insert(m);
            walk_output(w, m, pass == 0, nullptr);
            deps[m] = w.deps;
        } else if (pass == 0) {
            const auto& nd = nodes[m];
            for (int p = 0; p < nd.n_parents; ++p) {
                int src; std::vector<int> sh, st;
                operand_view(nd.parents[p], src, sh, st, true);
                if (info[src].kind != K_INPUT) deps[m].push_back(Dep{src, false});
            }
        }
    }

    // ---- 4. steps: merge materialized nodes of one domain into multi-output kernels
    std::vector<StepNode> steps;
    auto reaches = [&](int from, int to) {
        std::vector<int> st{from}; std::set<int> seen;
        while (!st.empty()) { int s = st.back(); st.pop_back(); if (s == to) return true; if (!seen.insert(s).second) continue; for (int t : steps[s].succ) st.push_back(t); }
        return false;
    };
    for (int m = 0; m < n; ++m) {
        if (!info[m].in_M) continue;
        int chosen = -1;
        if (fusable_output(m)) {
            std::vector<int> D; int k; kernel_domain(m, D, k);
            for (int s = (int)steps.size() - 1; s >= 0 && chosen < 0; --s) {
                StepNode& S = steps[s];
                if (S.type != StepNode::FUSED || S.D != D || !k_compatible(S.k, k)) continue;
                bool ok = true;
                for (const Dep& d : deps[m]) {
                    int ds = info[d.node].step;
                    if (ds == s) { if (!d.mergeable) { ok = false; break; } }
                    else if (reaches(s, ds)) { ok = false; break; }
                }
                if (ok) chosen = s;
            }
            if (chosen < 0) {
                StepNode S; S.type = StepNode::FUSED; S.D = D; S.k = k;
                steps.push_back(S); chosen = (int)steps.size() - 1;
            }
            if (steps[chosen].k < 0) steps[chosen].k = k;
        } else {
            StepNode S; S.type = info[m].kind == K_MATMUL ? StepNode::GEMM : StepNode::GENSUM;
            steps.push_back(S); chosen = (int)steps.size() - 1;
        }
        steps[chosen].outputs.push_back(m);
        info[m].step = chosen;
        for (const Dep& d : deps[m]) { int ds = info[d.node].step; if (ds != chosen) steps[ds].succ.insert(chosen); }
    }

    // ---- 4b. matmuls on the tensor-core kernel: which qualify, what follows them, who writes their bf16 operands
    std::vector<bool> need_twin(n, false), drop_f32(n, false), bf16_out(n, false);
    std::vector<std::pair<int, int>> twin_shape(n, {0, 0});
    std::vector<std::vector<int>> consumers(n);          // materialized node -> materialized nodes whose step reads it
    for (int x = 0; x < n; ++x) if (info[x].in_M) for (const Dep& d : deps[x]) consumers[d.node].push_back(x);
    for (int x = 0; x < n; ++x)
        if (info[x].needed && (nodes[x].flags & ORMI_NODE_BF16) && !(opt.bf16_matmul && opt.fusion)) {
            plan.error = "bf16 tensors need the \"bf16\" matmul arithmetic (ormi_b200_set_option \"matmul\")";
            return plan;
        }
    if (opt.bf16_matmul && opt.fusion) {
        for (auto& S : steps) if (S.type == StepNode::GEMM) S.tc = tc_eligible(S.outputs[0]);
        // (a) epilogues: a flat kernel over the [M, N] domain of a qualifying matmul that reads the product moves into
        //     the GEMM kernel, unless that would make the GEMM wait for something that itself waits for the GEMM.
        for (size_t gs = 0; gs < steps.size(); ++gs) {
            StepNode& Gs = steps[gs];
            if (Gs.type != StepNode::GEMM || !Gs.tc) continue;
            const int m = Gs.outputs[0];
            if (info[m].sq.size() != 2) continue;
            for (size_t fs = 0; fs < steps.size(); ++fs) {
                StepNode& Fs = steps[fs];
                if (Fs.type != StepNode::FUSED || Fs.dead || Fs.D != info[m].sq || !(Fs.k < 0 || Fs.k == 1)) continue;
                bool reads_m = false, ok = true;
                for (int o : Fs.outputs) {
                    // full pointwise results, and column sums over the rows of the product (a bias gradient)
                    const bool full = (info[o].kind == K_PW || info[o].kind == K_IDSUM) && !info[o].row_cls;
                    const bool colsum = info[o].kind == K_COLSUM && info[o].k == 1 && info[o].D == Fs.D;
                    const bool globalsum = info[o].kind == K_GLOBALSUM && info[o].D == Fs.D;      // e.g. the loss behind the last matmul
                    if (!full && !colsum && !globalsum) ok = false;
                    for (const Dep& d : deps[o]) {
                        if (d.node == m) { reads_m = true; continue; }
                        const int ds = info[d.node].step;
                        if (ds == (int)fs) continue;
                        if (ds == (int)gs || reaches((int)gs, ds)) ok = false;
                    }
                }
                if (!ok || !reads_m) continue;
                // the product must be read element for element (not transposed or broadcast) by every member
                Walk w; w.D = Fs.D; w.k = Fs.k;
                for (int o : Fs.outputs) w.outputs.insert(o);
                for (int o : Fs.outputs) walk_output(w, o, false, nullptr);
                int acc_loads = 0;
                for (const KLoad& l : w.loads) if (l.src_node == m) { ++acc_loads; if (l.st != std::vector<int64_t>{(int64_t)Fs.D[1], 1}) ok = false; }
                for (int q : w.members) if (info[q].kind == K_ROWSUM || info[q].row_cls) ok = false;     // no per-row values in an epilogue
                if (!ok || acc_loads != 1 || w.k_conflict) continue;
                // absorb: the outputs of Fs become outputs of the GEMM step
                Fs.dead = true;
                Gs.epi_outputs = Fs.outputs;
                for (int o : Fs.outputs) info[o].step = (int)gs;
                for (auto& T : steps) if (T.succ.erase((int)fs) && &T != &Gs) T.succ.insert((int)gs);
                for (int t : Fs.succ) if (t != (int)gs) Gs.succ.insert(t);
                Fs.succ.clear();
                break;                                   // one epilogue per matmul
            }
        }
        // (b) bf16 twins: an operand that is produced inside this plan is written as bf16 by its producer
        auto want_twin = [&](int src, int rows, int cols) {
            need_twin[src] = true;
            if (!twin_shape[src].first) twin_shape[src] = {rows, cols};
        };
        for (auto& S : steps) {
            if (S.type != StepNode::GEMM || !S.tc) continue;
            const auto& nd = nodes[S.outputs[0]];
            for (int p = 0; p < 2; ++p) {
                OperandView v = matmul_operand(nd.parents[p], false);
                if (info[v.src].kind == K_INPUT || !v.dense) continue;
                const Kind pk = info[v.src].kind;
                const StepNode& Ps = steps[info[v.src].step];
                bool producer_ok = (pk == K_MATMUL && Ps.tc) ||
                                   ((pk == K_PW || pk == K_IDSUM) && !info[v.src].row_cls && (Ps.type == StepNode::FUSED || Ps.type == StepNode::GEMM));
                if (producer_ok) want_twin(v.src, v.srows, v.scols);
            }
        }
        // a root the caller flagged: its bf16 twin is written along and remembered by the context
        for (int x = 0; x < n; ++x) {
            if (!info[x].in_M || !(nodes[x].flags & ORMI_NODE_TWIN16) || info[x].sq.size() != 2 || info[x].sq[1] % 8 != 0) continue;
            const Kind pk = info[x].kind;
            if ((pk == K_MATMUL && steps[info[x].step].tc) || ((pk == K_PW || pk == K_IDSUM) && !info[x].row_cls)) want_twin(x, info[x].sq[0], info[x].sq[1]);
        }
        // a root the caller wants as bf16 ONLY: the twin is the result, the fp32 form is never written
        for (int x = 0; x < n; ++x) {
            if (!info[x].in_M || !handed[x] || !(nodes[x].flags & ORMI_NODE_BF16)) continue;
            const Kind pk = info[x].kind;
            const bool producer_ok = (pk == K_MATMUL && steps[info[x].step].tc) || ((pk == K_PW || pk == K_IDSUM) && !info[x].row_cls);
            if (!producer_ok || info[x].sq.size() != 2 || info[x].sq[1] % 8 != 0 || info[x].sq != info[x].shape) {
                plan.error = "a node can be materialized as bf16 only when it is a 2-D pointwise result or tensor-core product whose last dimension is a multiple of 8";
                return plan;
            }
            want_twin(x, info[x].sq[0], info[x].sq[1]);
            bf16_out[x] = true;
            drop_f32[x] = true;
        }
        // (c) a pointwise result nobody but tensor-core matmuls reads is not written as fp32 at all
        for (int x = 0; x < n; ++x) {
            if (!need_twin[x] || handed[x] || info[x].kind == K_MATMUL) continue;
            bool only_tc = true, any = false;
            for (int y : consumers[x]) {
                if (info[y].step == info[x].step) continue;     // an output of the same kernel reads the value from registers
                any = true;
                if (!(info[y].kind == K_MATMUL && steps[info[y].step].tc)) only_tc = false;
            }
            only_tc = only_tc && any;
            for (int y : consumers[x]) {       // and each of those reads it as the dense matrix the twin is
                if (!only_tc) break;
                if (info[y].kind != K_MATMUL) continue;
                for (int p = 0; p < 2; ++p) {
                    OperandView v = matmul_operand(nodes[y].parents[p], false);
                    if (v.src == x && !v.dense) only_tc = false;
                }
            }
            drop_f32[x] = only_tc;
        }
    }

    // ---- 5. buffers
    std::map<int, int> buf_of_node;   // node -> plan buffer
    auto buffer_for = [&](int node) {
        auto it = buf_of_node.find(node);
        if (it != buf_of_node.end()) return it->second;
        PlanBuffer b;
        b.kind = info[node].kind == K_INPUT ? BufKind::External : BufKind::NodeOut;
        b.node = node;
        b.bytes = info[node].kind == K_INPUT ? nodes[node].data_bytes : std::max<int64_t>(4, info[node].numel * 4);
        plan.buffers.push_back(b);
        buf_of_node[node] = (int)plan.buffers.size() - 1;
        return (int)plan.buffers.size() - 1;
    };
    auto temp_buffer = [&](int64_t bytes) {
        plan.buffers.push_back(PlanBuffer{BufKind::Temp, -1, std::max<int64_t>(4, bytes)});
        return (int)plan.buffers.size() - 1;
    };
    std::map<int, int> twin_of_node;  // node -> Twin16 plan buffer
    auto twin_for = [&](int node) {
        auto it = twin_of_node.find(node);
        if (it != twin_of_node.end()) return it->second;
        PlanBuffer b{BufKind::Twin16, node, info[node].numel * 2};
        b.rows = twin_shape[node].first; b.cols = twin_shape[node].second;
        plan.buffers.push_back(b);
        twin_of_node[node] = (int)plan.buffers.size() - 1;
        return (int)plan.buffers.size() - 1;
    };

    // topological order of the steps (Kahn, lowest first output first)
    std::vector<int> indeg(steps.size(), 0), order;
    for (auto& S : steps) for (int t : S.succ) indeg[t]++;
    std::set<std::pair<int, int>> ready;
    size_t live_steps = 0;
    for (auto& S : steps) live_steps += !S.dead;
    for (size_t s = 0; s < steps.size(); ++s) if (!indeg[s] && !steps[s].dead) ready.insert({steps[s].outputs[0], (int)s});
    while (!ready.empty()) {
        int s = ready.begin()->second; ready.erase(ready.begin());
        order.push_back(s);
        for (int t : steps[s].succ) if (--indeg[t] == 0) ready.insert({steps[t].outputs[0], t});
    }
    if (order.size() != live_steps) { plan.error = "internal: cyclic kernel graph"; return plan; }
    if (!error.empty()) { plan.error = error; return plan; }

    int kernel_serial = 0;
    for (int s : order) {
        StepNode& S = steps[s];
        if (S.type == StepNode::GEMM) {
            int m = S.outputs[0];
            const auto& nd = nodes[m];
            int srcs[2]; std::vector<int> sh[2], st[2];
            for (int p = 0; p < 2; ++p) operand_view(nd.parents[p], srcs[p], sh[p], st[p], false);
            for (int p = 0; p < 2; ++p) if (sh[p].size() < 2) { plan.error = "MATMUL requires operands to have at least 2 dimensions."; return plan; }
            GemmStep g;
            g.node = m;
            int na = (int)sh[0].size(), nb = (int)sh[1].size();
            g.M = sh[0][na - 2]; g.K = sh[0][na - 1]; g.N = sh[1][nb - 1];
            if (sh[1][nb - 2] != g.K) { plan.error = "MATMUL inner dimensions must match (K_a != K_b)."; return plan; }
            int bufs[2];
            for (int p = 0; p < 2; ++p) {
                int nd_p = (int)sh[p].size();
                int rows = sh[p][nd_p - 2], cols = sh[p][nd_p - 1];
                int s_row = st[p][nd_p - 2], s_col = st[p][nd_p - 1];
                bool ok_n = (s_col == 1 || cols == 1) && (rows == 1 || s_row >= cols);
                bool ok_t = (s_row == 1 || rows == 1) && (cols == 1 || s_col >= rows);
                bufs[p] = buffer_for(srcs[p]);
                if (!ok_n && !ok_t) {
                    // neither row- nor column-contiguous: gather into a contiguous temporary first
                    KernelSpec ks;
                    ks.D = squeeze(sh[p]);
                    ks.k = -1;
                    ks.num_sms = opt.num_sms; ks.aligned = opt.aligned; std::copy(opt.tune, opt.tune + kTuneKnobs, ks.tune);
                    std::vector<int> dm = canonical_dm(sh[p]);
                    KLoad ld{srcs[p], strides_over_domain(dm, st[p], ks.D.size())};
                    ks.loads.push_back(ld);
                    KOutput o; o.node = -1; o.kind = KOutput::FULL; o.value = KRef{KRef::LOAD, 0};
                    ks.outputs.push_back(o);
                    int64_t elems = 1; for (int v : sh[p]) elems *= v;
                    int tmp = temp_buffer(elems * 4);
                    GeneratedKernel gk = generate_kernel(ks, "ormi_gather_" + std::to_string(kernel_serial++), nodes);
                    if (!gk.error.empty()) { plan.error = gk.error; return plan; }
                    Step stp; stp.type = Step::Kernel; stp.k = gk.step;
                    stp.k.args = {bufs[p], tmp};
                    plan.steps.push_back(stp);
                    bufs[p] = tmp;
                    st[p] = contiguous(sh[p]);
                    s_row = st[p][nd_p - 2]; s_col = st[p][nd_p - 1];
                    ok_n = true;
                }
                bool trans = !ok_n;
                int ld = trans ? s_col : s_row;
                if (trans && cols == 1) ld = std::max(ld, rows);
                if (!trans && rows == 1) ld = std::max(ld, cols);
                if (p == 0) { g.trans_a = trans; g.lda = ld; } else { g.trans_b = trans; g.ldb = ld; }
            }
            g.a = bufs[0]; g.b = bufs[1]; g.c = buffer_for(m);
            const Info& Mo = info[m];
            g.nbatch = (int)Mo.shape.size() - 2;
            g.batch = 1;
            for (int d = 0; d < g.nbatch; ++d) {
                g.bshape[d] = Mo.shape[d]; g.batch *= Mo.shape[d];
                for (int p = 0; p < 2; ++p) {
                    int td = d - (g.nbatch - ((int)sh[p].size() - 2));
                    int64_t v = (td >= 0 && sh[p][td] > 1) ? st[p][td] : 0;
                    (p == 0 ? g.astride : g.bstride)[d] = v;
                }
            }
            g.tc = S.tc;
            if (!S.tc) for (int p = 0; p < 2; ++p) if (info[srcs[p]].kind == K_INPUT && info[srcs[p]].bf16_in) {
                plan.error = "a bf16 tensor can only be an operand of a tensor-core matmul (this one does not qualify: see the shape rules)";
                return plan;
            }
            if (S.tc) {
                for (int p = 0; p < 2; ++p) {      // operands some earlier step of this plan writes as bf16, or the caller holds as bf16
                    OperandView v = matmul_operand(nd.parents[p], false);
                    if (info[v.src].kind != K_INPUT && need_twin[v.src] && v.dense) (p == 0 ? g.a16 : g.b16) = twin_for(v.src);
                    if (info[v.src].kind == K_INPUT && info[v.src].bf16_in) {
                        if (!v.dense) { plan.error = "a bf16 matmul operand must be the whole contiguous matrix (or its transpose)"; return plan; }
                        (p == 0 ? g.a16 : g.b16) = bufs[p];
                    }
                }
                const bool twin_c = need_twin[m];
                bool c_read = (handed[m] && !bf16_out[m]) || (S.epi_outputs.empty() && !twin_c);
                for (int y : consumers[m]) if (info[y].step != s) c_read = true;
                g.store_c = c_read;
                if (!c_read) drop_f32[m] = true;
                std::vector<Step> finalizes;
                if (!S.epi_outputs.empty() || twin_c || !c_read) {
                    Walk w; w.D = info[m].sq; w.k = -1;
                    for (int o : S.epi_outputs) if (info[o].kind == K_COLSUM) w.k = 1;
                    for (int o : S.epi_outputs) w.outputs.insert(o);
                    KernelSpec ks;
                    for (int o : S.epi_outputs) walk_output(w, o, false, &ks.outputs);
                    std::sort(w.members.begin(), w.members.end());
                    ks.D = w.D; ks.k = -1; ks.num_sms = opt.num_sms; ks.aligned = opt.aligned; std::copy(opt.tune, opt.tune + kTuneKnobs, ks.tune);
                    ks.loads = w.loads;
                    for (KLoad& l : ks.loads) if (l.src_node == m) l.acc = true;
                    for (int q : w.members) {
                        KNode kn;
                        kn.node = q;
                        kn.op = info[q].kind == K_PW ? nodes[q].op : KNode::OP_ID;
                        kn.row = false;
                        kn.scalar = false;
                        kn.operands = w.operands[q];
                        ks.nodes.push_back(kn);
                    }
                    for (KOutput& o : ks.outputs) if (o.kind == KOutput::FULL) { o.twin = need_twin[o.node]; o.store = !drop_f32[o.node]; }
                    GeneratedEpilogue ge = generate_gemm_epilogue(ks, g.store_c, twin_c);
                    if (!ge.error.empty()) { plan.error = ge.error; return plan; }
                    g.has_epi = true;
                    g.epi_prelude = ge.prelude; g.epi_params = ge.params; g.epi_init = ge.init; g.epi_cols = ge.cols; g.epi_body = ge.body;
                    g.epi_end = ge.end; g.epi_pre = ge.pre;
                    g.epi_wpq = ge.wpq; g.epi_unroll = ge.unroll;
                    for (const KLoad& l : ks.loads) if (!l.acc) g.epi_args.push_back(buffer_for(l.src_node));
                    for (const KOutput& o : ks.outputs) {
                        if (o.kind == KOutput::COLSUM || o.kind == KOutput::GLOBALSUM) {
                            // one partial row per 32-row block of the product (a global sum: one value per block and
                            // 32-column chunk); blocks past the last row (the tile grid is rounded up to 256 rows) are
                            // written too, as zeros, and not read
                            const bool col = o.kind == KOutput::COLSUM;
                            const int64_t blocks = (g.M + 31) / 32, padded = ((g.M + 255) / 256) * 8, chunks = (g.N + 31) / 32;
                            int tmp = temp_buffer(padded * (col ? (int64_t)g.N : chunks) * 4);
                            g.epi_args.push_back(tmp);
                            GeneratedKernel fk = generate_finalize((int)(col ? blocks : blocks * chunks), col ? (int64_t)g.N : 1, "ormi_finalize_" + std::to_string(kernel_serial++), o.is_max);
                            Step fs; fs.type = Step::Kernel; fs.k = fk.step;
                            fs.k.args = {tmp, buffer_for(o.node)};
                            finalizes.push_back(fs);
                            continue;
                        }
                        if (o.store) g.epi_args.push_back(buffer_for(o.node));
                        if (o.twin) g.epi_args.push_back(twin_for(o.node));
                    }
                    if (twin_c) g.epi_args.push_back(twin_for(m));
                    std::ostringstream what;
                    what << "epilogue[nodes=" << ks.nodes.size() << ",loads=" << ks.loads.size() - 1 << ",outs=";
                    for (const KOutput& o : ks.outputs) what << (o.kind == KOutput::COLSUM ? "C" : "") << (o.kind == KOutput::GLOBALSUM ? "G" : "") << (o.kind == KOutput::FULL && o.store ? "F" : "") << (o.twin ? "h" : "");
                    what << ",product=" << (g.store_c ? "F" : "") << (twin_c ? "h" : "") << ",wpq=" << ge.wpq << "]";
                    g.epi_what = what.str();
                }
                Step stp; stp.type = Step::Gemm; stp.g = g;
                plan.steps.push_back(stp);
                for (const Step& f : finalizes) plan.steps.push_back(f);
                continue;
            }
            Step stp; stp.type = Step::Gemm; stp.g = g;
            plan.steps.push_back(stp);
            continue;
        }
        if (S.type == StepNode::GENSUM) {
            int m = S.outputs[0];
            int src; std::vector<int> sh, st;
            operand_view(nodes[m].parents[0], src, sh, st, false);
            if (info[src].kind == K_INPUT && info[src].bf16_in) { plan.error = "a bf16 tensor can only be an operand of a tensor-core matmul"; return plan; }
            std::vector<bool> red(sh.size(), nodes[m].n_axes == 0);
            for (int a = 0; a < nodes[m].n_axes; ++a) red[nodes[m].axes[a]] = true;
            if (info[src].kind == K_INPUT && nodes[src].data_bytes == 4) std::fill(st.begin(), st.end(), 0);
            GeneratedKernel gk = generate_generic_sum(sh, st, red, "ormi_sum_" + std::to_string(kernel_serial++), nodes[m].op == ORMI_OP_MAX);
            Step stp; stp.type = Step::Kernel; stp.k = gk.step;
            stp.k.args = {buffer_for(src), buffer_for(m)};
            plan.steps.push_back(stp);
            continue;
        }
        // fused kernel: final walk over all outputs
        Walk w; w.D = S.D; w.k = S.k;
        for (int m : S.outputs) w.outputs.insert(m);
        KernelSpec ks;
        for (int m : S.outputs) walk_output(w, m, false, &ks.outputs);
        if (w.k_conflict) { plan.error = "internal: kernel with two different row/column splits"; return plan; }
        std::sort(w.members.begin(), w.members.end());
        ks.D = w.D; ks.k = w.k; ks.num_sms = opt.num_sms; ks.aligned = opt.aligned; std::copy(opt.tune, opt.tune + kTuneKnobs, ks.tune);
        ks.loads = w.loads;
        for (int q : w.members) {
            KNode kn;
            kn.node = q;
            kn.op = info[q].kind == K_PW ? nodes[q].op : (info[q].kind == K_ROWSUM ? KNode::OP_ROWSUM : KNode::OP_ID);
            kn.row = info[q].row_cls;
            kn.is_max = info[q].kind == K_ROWSUM && nodes[q].op == ORMI_OP_MAX;
            kn.scalar = (info[q].kind == K_PW || info[q].kind == K_IDSUM) && info[q].numel == 1 && !w.D.empty();
            kn.operands = w.operands[q];
            ks.nodes.push_back(kn);
        }
        for (KOutput& o : ks.outputs) if (o.kind == KOutput::FULL && o.node >= 0) { o.twin = need_twin[o.node]; o.store = !drop_f32[o.node]; }
        GeneratedKernel gk = generate_kernel(ks, "ormi_fused_" + std::to_string(kernel_serial++), nodes);
        if (!gk.error.empty()) {
            if (gk.unsupported_sums) {   // the row/column template cannot take this shape: retry with generic sums
                bool added = false;
                for (int q : w.members) if (info[q].kind == K_ROWSUM) added |= force_generic.insert(q).second;
                for (int m : S.outputs) if (info[m].kind == K_ROWSUM || info[m].kind == K_COLSUM) added |= force_generic.insert(m).second;
                if (added) return run(roots, n_roots);
            }
            plan.error = gk.error; return plan;
        }
        Step stp; stp.type = Step::Kernel; stp.k = gk.step;
        for (const KLoad& l : ks.loads) stp.k.args.push_back(buffer_for(l.src_node));
        std::vector<std::pair<int, int>> finals;   // (scratch buffer, output index)
        for (size_t oi = 0; oi < ks.outputs.size(); ++oi) {
            const KOutput& o = ks.outputs[oi];
            if (o.kind == KOutput::FULL || o.kind == KOutput::ROW) {
                if (o.store) stp.k.args.push_back(buffer_for(o.node));
                if (o.twin) stp.k.args.push_back(twin_for(o.node));
            } else {
                int64_t per = o.kind == KOutput::COLSUM ? gk.cols : 1;
                int tmp = temp_buffer(per * 4 * gk.step.grid);
                stp.k.args.push_back(tmp);
                finals.push_back({tmp, (int)oi});
            }
        }
        if (gk.step.err_arg) {
            int eb = -1;
            for (size_t b = 0; b < plan.buffers.size(); ++b) if (plan.buffers[b].kind == BufKind::ErrorWord) eb = (int)b;
            if (eb < 0) { plan.buffers.push_back(PlanBuffer{BufKind::ErrorWord, -1, 4}); eb = (int)plan.buffers.size() - 1; }
            stp.k.args.push_back(eb);
        }
        plan.steps.push_back(stp);
        // one finalize launch per geometry: the column partials of all outputs together, the global partials together
        for (int colwise = 1; colwise >= 0; --colwise) {
            std::vector<std::pair<int, int>> group;
            for (auto& f : finals) if ((ks.outputs[f.second].kind == KOutput::COLSUM) == (colwise == 1)) group.push_back(f);
            if (group.empty()) continue;
            unsigned max_bits = 0;
            for (size_t i = 0; i < group.size(); ++i) if (ks.outputs[group[i].second].is_max) max_bits |= 1u << i;
            const int64_t per = colwise ? gk.cols : 1;
            GeneratedKernel fk = generate_finalize(gk.step.grid, per, "ormi_finalize_" + std::to_string(kernel_serial++), max_bits != 0, (int)group.size(), max_bits);
            Step fs; fs.type = Step::Kernel; fs.k = fk.step;
            for (auto& f : group) { fs.k.args.push_back(f.first); fs.k.args.push_back(buffer_for(ks.outputs[f.second].node)); }
            plan.steps.push_back(fs);
        }
    }

    // ---- results: every materialized node, plus roots / KEEP nodes that are views (aliases)
    for (int i = 0; i < n; ++i) {
        if (!info[i].needed || info[i].kind == K_INPUT) continue;
        if (info[i].in_M && !drop_f32[i]) {
            // A materialized node nobody outside the call can reach again is scratch under "intermediates=free": its
            // block goes back to the pool right after the last step that reads it.
            if (opt.free_intermediates && !handed[i]) plan.buffers[buffer_for(i)].kind = BufKind::Temp;
            else plan.results.push_back(NodeResult{i, buffer_for(i), false});
        }
        if (info[i].in_M && bf16_out[i]) { NodeResult r{i, twin_for(i), false}; r.bf16 = true; plan.results.push_back(r); }
    }
    auto alias_result = [&](int i) {
        if (info[i].kind != K_VIEW) return;
        for (auto& r : plan.results) if (r.node == i) return;
        plan.results.push_back(NodeResult{i, buffer_for(info[i].base), true});
    };
    for (int r = 0; r < n_roots; ++r) alias_result(roots[r]);
    for (int i = 0; i < n; ++i) if (info[i].needed && (nodes[i].flags & ORMI_NODE_KEEP)) alias_result(i);
    if (!error.empty() && plan.error.empty()) plan.error = error;
    return plan;
}

std::string json_escape(const std::string& s) {
    std::string o;
    for (char c : s) {
        switch (c) {
            case '"': o += "\\\""; break;
            case '\\': o += "\\\\"; break;
            case '\n': o += "\\n"; break;
            case '\t': o += "\\t"; break;
            case '\r': break;
            default: o += c;
        }
    }
    return o;
}

}  // namespace

int tune_knob_index(const std::string& name) {
    static const char* names[kTuneKnobs] = {"rows_vpt", "rows_minb", "rows_grid", "rows_stage", "rows_nstage", "rows_dynamic",
                                            "flat_unroll", "rows_hoist", "epi_unroll", "epi_wpq", "gemm_bn", "epi_node_major"};
    for (int i = 0; i < kTuneKnobs; ++i) if (name == names[i]) return i;
    return -1;
}

SchedOptions parse_sched_options(const char* options) {
    SchedOptions opt;
    const std::string text = options ? options : "";
    size_t pos = 0;
    while (pos < text.size()) {
        size_t end = text.find(',', pos);
        if (end == std::string::npos) end = text.size();
        const std::string item = text.substr(pos, end - pos);
        pos = end + 1;
        if (item.empty()) continue;
        const size_t eq = item.find('=');
        if (eq == std::string::npos) throw std::runtime_error("option without a value: " + item);
        const std::string k = item.substr(0, eq), v = item.substr(eq + 1);
        if (k == "matmul") opt.bf16_matmul = (v == "bf16");
        else if (k == "fusion") opt.fusion = (v != "off");
        else if (k == "intermediates") opt.free_intermediates = (v == "free");
        else if (k == "aligned") opt.aligned = (v != "0");
        else if (k.rfind("tune.", 0) == 0 && tune_knob_index(k.substr(5)) >= 0) opt.tune[tune_knob_index(k.substr(5))] = std::atoi(v.c_str());
        else throw std::runtime_error("unknown option: " + k);
    }
    return opt;
}

Plan build_plan(const ormi_b200_node* nodes, int n_nodes, const int* roots, int n_roots, const SchedOptions& opt) {
    Scheduler s(nodes, n_nodes, opt);
    return s.run(roots, n_roots);
}

std::string plan_to_json(const Plan& plan) {
    std::ostringstream o;
    o << "{\"error\": \"" << json_escape(plan.error) << "\", \"buffers\": [";
    for (size_t i = 0; i < plan.buffers.size(); ++i) {
        const auto& b = plan.buffers[i];
        o << (i ? ", " : "") << "{\"kind\": \"" << (b.kind == BufKind::External ? "external" : b.kind == BufKind::NodeOut ? "node" : b.kind == BufKind::ErrorWord ? "error" : b.kind == BufKind::Twin16 ? "twin16" : "temp")
          << "\", \"node\": " << b.node << ", \"bytes\": " << b.bytes << "}";
    }
    o << "], \"steps\": [";
    for (size_t i = 0; i < plan.steps.size(); ++i) {
        const auto& s = plan.steps[i];
        o << (i ? ", " : "");
        if (s.type == Step::Kernel) {
            o << "{\"type\": \"kernel\", \"name\": \"" << s.k.name << "\", \"grid\": " << s.k.grid << ", \"block\": " << s.k.block << ", \"dyn_smem\": " << s.k.dyn_smem
              << ", \"what\": \"" << json_escape(s.k.what) << "\", \"bytes_read\": " << s.k.bytes_read << ", \"bytes_written\": " << s.k.bytes_written
              << ", \"args\": [";
            for (size_t a = 0; a < s.k.args.size(); ++a) o << (a ? ", " : "") << s.k.args[a];
            o << "], \"source\": \"" << json_escape(s.k.source) << "\"}";
        } else {
            const auto& g = s.g;
            o << "{\"type\": \"gemm\", \"node\": " << g.node << ", \"a\": " << g.a << ", \"b\": " << g.b << ", \"c\": " << g.c
              << ", \"M\": " << g.M << ", \"N\": " << g.N << ", \"K\": " << g.K << ", \"trans_a\": " << g.trans_a << ", \"trans_b\": " << g.trans_b
              << ", \"lda\": " << g.lda << ", \"ldb\": " << g.ldb << ", \"batch\": " << g.batch << ", \"bshape\": [";
            for (int d = 0; d < g.nbatch; ++d) o << (d ? ", " : "") << g.bshape[d];
            o << "], \"astride\": [";
            for (int d = 0; d < g.nbatch; ++d) o << (d ? ", " : "") << g.astride[d];
            o << "], \"bstride\": [";
            for (int d = 0; d < g.nbatch; ++d) o << (d ? ", " : "") << g.bstride[d];
            o << "], \"tc\": " << (g.tc ? "true" : "false") << ", \"a16\": " << g.a16 << ", \"b16\": " << g.b16
              << ", \"store_c\": " << (g.store_c ? "true" : "false") << ", \"epilogue\": \"" << json_escape(g.epi_what) << "\", \"epi_args\": [";
            for (size_t a = 0; a < g.epi_args.size(); ++a) o << (a ? ", " : "") << g.epi_args[a];
            o << "], \"epi_body\": \"" << json_escape(g.epi_body) << "\", \"epi_cols\": \"" << json_escape(g.epi_cols) << "\", \"epi_init\": \""
              << json_escape(g.epi_init) << "\", \"epi_pre\": \"" << json_escape(g.epi_pre) << "\", \"epi_end\": \"" << json_escape(g.epi_end) << "\", \"epi_params\": \"" << json_escape(g.epi_params) << "\", \"epi_prelude\": \"" << json_escape(g.epi_prelude) << "\"}";
        }
    }
    o << "], \"results\": [";
    for (size_t i = 0; i < plan.results.size(); ++i) {
        const auto& r = plan.results[i];
        o << (i ? ", " : "") << "{\"node\": " << r.node << ", \"buffer\": " << r.buffer << ", \"alias\": " << (r.alias ? "true" : "false") << ", \"bf16\": " << (r.bf16 ? "true" : "false") << "}";
    }
    o << "]}";
    return o.str();
}

uint64_t fnv1a(const std::string& s) {
    uint64_t h = 1469598103934665603ull;
    for (unsigned char c : s) { h ^= c; h *= 1099511628211ull; }
    return h;
}

}  // namespace ormi_b200
