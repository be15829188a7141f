/*
 * TEST INFRASTRUCTURE — never linked or loaded by the product.
 *
 * C-ABI driver around the UNMODIFIED reference engine (core + CPU backend + runtime), which the
 * Makefile beside this file compiles from the reference checkout into oracle/_ref/.  It lets the
 * Python tests and the CPU-baseline leg of the benchmark run a graph on the reference's own CPU
 * backend without pybind11:
 *
 *   - oracle_ref_run():    rebuild a flattened forward graph with the reference's Node constructors,
 *                          optionally seed gradients and call ormi::compute_gradients
 *                          (ormi-core/csrc/core/autograd.cpp:24-47), realize the requested values /
 *                          gradients through ormi::execute_graph (ormi-core/csrc/backend/runtime.cpp:13-39)
 *                          on DeviceEnum::CPU and copy them out (view strides applied, like
 *                          Tensor.numpy(), ormi-core/src/ormi_core/tensor.py:165-174).
 *   - oracle_ref_export(): the same, but instead of realizing, flatten the graph that the reference's
 *                          autograd produced, so the host-side mirror of that autograd can be compared
 *                          node for node.
 *
 * The two CUDA symbols the reference runtime refers to are stubbed: this library is CPU-only.
 */
#include <chrono>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "core/node.h"
#include "core/memory.h"
#include "core/allocator.h"
#include "core/autograd.h"
#include "core/shape.h"
#include "backend/runtime.h"
#include "backend/cuda/jit.cuh"

#include "ormi_b200.h"

namespace ormi {
    IAllocator* get_cuda_allocator() { throw std::runtime_error("oracle build: no CUDA backend"); }
    namespace cuda { void execute_jit(std::shared_ptr<Node>) { throw std::runtime_error("oracle build: no CUDA backend"); } }
}

using namespace ormi;
using NodeP = std::shared_ptr<Node>;

#define ORACLE_REQUIRES_GRAD 0x100u

static thread_local std::string g_err;

static std::vector<int> vec(const int32_t* p, int n) { return std::vector<int>(p, p + n); }

static std::vector<NodeP> build_forward(const ormi_b200_node* nodes, int n) {
    std::vector<NodeP> out(n);
    Device dev(DeviceEnum::CPU, 0);
    for (int i = 0; i < n; ++i) {
        const ormi_b200_node& d = nodes[i];
        auto op = static_cast<ops::OpEnum>(d.op);
        if (op == ops::OpEnum::LEAF) {
            auto buf = empty(vec(d.shape, d.ndim), DeviceEnum::CPU);
            std::memcpy(buf->ptr, d.data, buf->bytes);
            out[i] = std::make_shared<Node>(buf, (d.flags & ORACLE_REQUIRES_GRAD) != 0, dev);
            continue;
        }
        std::vector<NodeP> parents;
        for (int p = 0; p < d.n_parents; ++p) parents.push_back(out[d.parents[p]]);
        OpAttributes attrs = NoAttrs{};
        if (op == ops::OpEnum::SUM) attrs = ReduceAttrs{vec(d.axes, d.n_axes), d.keepdims != 0};
        else if (op == ops::OpEnum::TRANSPOSE) attrs = PermuteAttrs{vec(d.axes, d.n_axes)};
        else if (op == ops::OpEnum::RESHAPE) attrs = ReshapeAttrs{vec(d.shape, d.ndim)};
        else if (op == ops::OpEnum::EXPAND) attrs = ExpandAttrs{vec(d.shape, d.ndim)};
        out[i] = std::make_shared<Node>(op, parents, dev, attrs);
    }
    return out;
}

static void apply_seeds_and_backward(std::vector<NodeP>& g, const int32_t* seed_nodes, const int32_t* seed_leaves,
                                     int n_seeds, int backward_root) {
    for (int i = 0; i < n_seeds; ++i) g[seed_nodes[i]]->grad = g[seed_leaves[i]];
    if (backward_root >= 0) compute_gradients(g[backward_root]);
}

static NodeP pick(std::vector<NodeP>& g, int node, int kind) {
    NodeP t = (kind == 1) ? g[node]->grad : g[node];
    if (!t) throw std::runtime_error("requested gradient does not exist");
    return t;
}

extern "C" const char* oracle_ref_last_error(void) { return g_err.c_str(); }

extern "C" const char* oracle_cblas_backend(void);
extern "C" int oracle_cblas_threads(void);
extern "C" const char* oracle_ref_blas(void) { return oracle_cblas_backend(); }
extern "C" int oracle_ref_blas_threads(void) { return oracle_cblas_threads(); }

extern "C" int oracle_ref_run(const ormi_b200_node* nodes, int n,
                              const int32_t* seed_nodes, const int32_t* seed_leaves, int n_seeds,
                              int32_t backward_root,
                              const int32_t* out_nodes, const int32_t* out_kinds, int n_out,
                              float** out_data, const int64_t* out_cap,
                              int32_t* out_ndim, int32_t* out_shape, double* seconds) {
    try {
        auto g = build_forward(nodes, n);
        auto t0 = std::chrono::steady_clock::now();
        apply_seeds_and_backward(g, seed_nodes, seed_leaves, n_seeds, backward_root);
        std::vector<NodeP> targets;
        for (int i = 0; i < n_out; ++i) {
            targets.push_back(pick(g, out_nodes[i], out_kinds[i]));
            targets.back()->realize();
        }
        auto t1 = std::chrono::steady_clock::now();
        if (seconds) *seconds = std::chrono::duration<double>(t1 - t0).count();
        for (int i = 0; i < n_out; ++i) {
            const NodeP& t = targets[i];
            const auto& shape = t->view.shape;
            const auto& strides = t->view.strides;
            int64_t numel = 1;
            for (int s : shape) numel *= s;
            out_ndim[i] = (int32_t)shape.size();
            for (size_t d = 0; d < shape.size(); ++d) out_shape[i * ORMI_B200_MAX_DIMS + d] = shape[d];
            if (numel > out_cap[i]) throw std::runtime_error("output buffer too small");
            const float* src = static_cast<const float*>(t->data->ptr);
            float* dst = out_data[i];
            std::vector<int> idx(shape.size(), 0);
            for (int64_t e = 0; e < numel; ++e) {
                int64_t off = 0;
                for (size_t d = 0; d < shape.size(); ++d) off += (int64_t)idx[d] * strides[d];
                dst[e] = src[off];
                for (int d = (int)shape.size() - 1; d >= 0; --d) { if (++idx[d] < shape[d]) break; idx[d] = 0; }
            }
        }
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return 1; }
}

/* Flattens what the reference built.  origin[i] = index of the node in the caller's forward graph, or -1
 * for a node created by the reference's autograd; for a created LEAF, leaf_value[i] is its (constant) fill. */
extern "C" int oracle_ref_export(const ormi_b200_node* nodes, int n,
                                 const int32_t* seed_nodes, const int32_t* seed_leaves, int n_seeds,
                                 int32_t backward_root,
                                 const int32_t* out_nodes, const int32_t* out_kinds, int n_out,
                                 ormi_b200_node* exp_nodes, int cap, int32_t* n_exp,
                                 int32_t* origin, float* leaf_value, int32_t* out_index) {
    try {
        auto g = build_forward(nodes, n);
        apply_seeds_and_backward(g, seed_nodes, seed_leaves, n_seeds, backward_root);
        std::unordered_map<Node*, int> orig;
        for (int i = 0; i < n; ++i) orig[g[i].get()] = i;
        std::unordered_map<Node*, int> index;
        std::vector<NodeP> order;
        // iterative post-order DFS (parents before children)
        for (int o = 0; o < n_out; ++o) {
            std::vector<std::pair<NodeP, size_t>> stack;
            stack.push_back({pick(g, out_nodes[o], out_kinds[o]), 0});
            while (!stack.empty()) {
                auto& top = stack.back();
                if (index.count(top.first.get())) { stack.pop_back(); continue; }
                if (top.second < top.first->parents.size()) {
                    NodeP p = top.first->parents[top.second++];
                    if (!index.count(p.get())) stack.push_back({p, 0});
                } else {
                    index[top.first.get()] = (int)order.size();
                    order.push_back(top.first);
                    stack.pop_back();
                }
            }
            out_index[o] = index[pick(g, out_nodes[o], out_kinds[o]).get()];
        }
        if ((int)order.size() > cap) throw std::runtime_error("export buffer too small");
        *n_exp = (int32_t)order.size();
        for (size_t i = 0; i < order.size(); ++i) {
            const NodeP& t = order[i];
            ormi_b200_node& d = exp_nodes[i];
            std::memset(&d, 0, sizeof d);
            d.op = static_cast<int32_t>(t->op);
            d.n_parents = (int32_t)t->parents.size();
            for (size_t p = 0; p < t->parents.size() && p < 2; ++p) d.parents[p] = index[t->parents[p].get()];
            d.ndim = (int32_t)t->view.shape.size();
            for (int k = 0; k < d.ndim; ++k) { d.shape[k] = t->view.shape[k]; d.strides[k] = t->view.strides[k]; }
            if (auto* r = std::get_if<ReduceAttrs>(&t->attrs)) {
                d.n_axes = (int32_t)r->axes.size();
                for (int k = 0; k < d.n_axes; ++k) d.axes[k] = r->axes[k];
                d.keepdims = r->keepdims ? 1 : 0;
            } else if (auto* p = std::get_if<PermuteAttrs>(&t->attrs)) {
                d.n_axes = (int32_t)p->axes.size();
                for (int k = 0; k < d.n_axes; ++k) d.axes[k] = p->axes[k];
            }
            if (t->requires_grad) d.flags |= ORACLE_REQUIRES_GRAD;
            auto it = orig.find(t.get());
            origin[i] = it == orig.end() ? -1 : it->second;
            leaf_value[i] = 0.0f;
            if (t->op == ops::OpEnum::LEAF && t->data) {
                d.data_bytes = (int64_t)t->data->bytes;
                if (origin[i] < 0) leaf_value[i] = static_cast<const float*>(t->data->ptr)[0];
            }
        }
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return 1; }
}
