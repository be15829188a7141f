// The six C++ seams through which ormi-core reaches its CUDA backend, re-implemented on top of the C ABI of
// include/ormi_b200.h.  This file is compiled INSIDE ormi-core (it includes ormi-core's own headers and is built
// together with ormi-core's unmodified core/, backend/graph_breakers.cpp and backend/cpu/): it replaces
//   backend/cuda/allocator.cu            -> B200Allocator, get_cuda_allocator            (seam 1)
//   backend/cuda/jit.cu                  -> cuda::execute_jit                            (seam 2)
//   backend/cuda/compiler.cu             -> cuda::compile                                (seam 3)
//   backend/cuda/kernels/blas/matmul.cu  -> cuda::matmul, matmul_handler, registration   (seam 4)
//   backend/cuda/kernels/reduce/sum.cu   -> cuda::sum, sum_handler, registration         (seam 4)
//   backend/cuda/utils.cu                -> cuda::compile_ptx                            (seam 5)
//   backend/cuda/lowerings/pointwise.cpp -> the CUDALoweringRegistry entries             (seam 6)
// Errors keep the reference's convention: std::runtime_error carrying the backend's message.
#include <algorithm>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <unordered_map>
#include <unordered_set>

#include "ormi_b200.h"
#include "b200_backend.h"

#include "core/allocator.h"
#include "core/memory.h"
#include "core/node.h"
#include "core/registry.h"
#include "core/shape.h"
#include "backend/graph_breakers.h"
#include "backend/cuda/compiler.cuh"
#include "backend/cuda/jit.cuh"
#include "backend/cuda/utils.cuh"
#include "backend/cuda/lowering_registry.h"
#include "backend/cuda/kernels/blas/cuda_matmul.cuh"
#include "backend/cuda/kernels/reduce/cuda_sum.cuh"

namespace ormi {

namespace {

[[noreturn]] void raise() { throw std::runtime_error(ormi_b200_last_error()); }
#define B200(call) do { if ((call) != 0) raise(); } while (0)

// One backend context per CUDA device, created on first use.  ormi::Device carries an id (core/device.h:10), but the
// allocator interface has none and every Buffer is built with id 0 (core/memory.cpp:94): so allocations go to the
// ACTIVE device (cuda::set_active_device, default 0 — one process per GPU sets it once to its local rank), every
// pointer remembers the device that owns it, and a graph runs on the context that owns its inputs.  A node whose
// Device.id names another device than its inputs live on is an error, not a silent copy.  Creating a context fails
// without a GPU, which the callers rely on (csrc/tests/test_utils.h:17-21).
std::mutex g_ctx_mutex;
std::unordered_map<int, ormi_b200_ctx*> g_contexts;
int g_active_device = 0;
std::unordered_map<const void*, int> g_owner;      // device pointer -> device id (pool blocks handed out through the allocator)

ormi_b200_ctx* ctx(int device = -1) {
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    if (device < 0) device = g_active_device;
    auto it = g_contexts.find(device);
    if (it != g_contexts.end()) return it->second;
    ormi_b200_ctx* p = nullptr;
    if (ormi_b200_init(device, &p) != 0) raise();
    g_contexts[device] = p;
    return p;
}

int owner_of(const void* ptr) {
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    auto it = g_owner.find(ptr);
    return it == g_owner.end() ? g_active_device : it->second;
}

// The pointwise expressions this backend emits for the ops of the reference's registry, in the registry's own notation
// ("<expr>;" over the operand names).  An entry that differs — somebody registered a lowering of their own — is handed
// to the code generator; one that matches (or was restored) clears the override.
const std::pair<ops::OpEnum, const char*> kDefaultLowerings[] = {
    {ops::OpEnum::ADD, "$0 + $1;"}, {ops::OpEnum::SUB, "$0 - $1;"}, {ops::OpEnum::MUL, "$0 * $1;"}, {ops::OpEnum::DIV, "$0 / $1;"},
    {ops::OpEnum::POW, "ormi_pow($0, $1);"}, {ops::OpEnum::NEG, "-$0;"}, {ops::OpEnum::EXP, "expf($0);"}, {ops::OpEnum::LOG, "logf($0);"},
    {ops::OpEnum::SIN, "sinf($0);"}, {ops::OpEnum::COS, "cosf($0);"}};

void sync_lowerings() {
    static std::unordered_map<int, std::string> sent;
    for (const auto& d : kDefaultLowerings) {
        std::string text;
        try { text = cuda::CUDALoweringRegistry::get(d.first)({"$0", "$1"}); } catch (const std::exception&) { continue; }
        const int op = static_cast<int>(d.first);
        std::string expr = text == d.second ? std::string() : text;
        while (!expr.empty() && (expr.back() == ';' || expr.back() == ' ' || expr.back() == '\n')) expr.pop_back();
        auto it = sent.find(op);
        if ((it == sent.end() && expr.empty()) || (it != sent.end() && it->second == expr)) continue;
        B200(ormi_b200_set_lowering(op, expr.c_str()));
        sent[op] = expr;
    }
}

bool is_view(ops::OpEnum op) { return ViewOpRegistry::get().contains(op); }

std::shared_ptr<Node> base_of(std::shared_ptr<Node> n) {
    while (is_view(n->op) && !n->parents.empty()) n = n->parents[0];
    return n;
}

void fill(ormi_b200_node& d, const Node& n) {
    std::memset(&d, 0, sizeof d);
    d.op = static_cast<int32_t>(n.op);
    if (n.view.shape.size() > ORMI_B200_MAX_DIMS) throw std::runtime_error("tensor rank above 8 is not supported by the B200 backend");
    d.ndim = (int32_t)n.view.shape.size();
    for (int k = 0; k < d.ndim; ++k) { d.shape[k] = n.view.shape[k]; d.strides[k] = n.view.strides[k]; }
    if (auto* r = std::get_if<ReduceAttrs>(&n.attrs)) {
        d.n_axes = (int32_t)r->axes.size();
        for (int k = 0; k < d.n_axes; ++k) d.axes[k] = r->axes[k];
        d.keepdims = r->keepdims ? 1 : 0;
    } else if (auto* p = std::get_if<PermuteAttrs>(&n.attrs)) {
        d.n_axes = (int32_t)p->axes.size();
        for (int k = 0; k < d.n_axes; ++k) d.axes[k] = p->axes[k];
    }
    if (n.data) { d.data = n.data->ptr; d.data_bytes = (int64_t)n.data->bytes; }
}

// The graph under `root`, flattened in post-order; the walk stops at realized nodes.
struct Flat {
    std::vector<ormi_b200_node> nodes;
    std::vector<std::shared_ptr<Node>> order;
};

Flat flatten(const std::shared_ptr<Node>& root, bool mark_held) {
    Flat f;
    std::unordered_map<Node*, int> index;
    std::vector<std::pair<std::shared_ptr<Node>, size_t>> stack{{root, 0}};
    while (!stack.empty()) {
        auto& top = stack.back();
        if (index.count(top.first.get())) { stack.pop_back(); continue; }
        const bool leaf = top.first->is_realized();
        if (!leaf && top.second < top.first->parents.size()) {
            auto p = top.first->parents[top.second++];
            if (!index.count(p.get())) stack.push_back({p, 0});
        } else {
            index[top.first.get()] = (int)f.order.size();
            f.order.push_back(top.first);
            stack.pop_back();
        }
    }
    f.nodes.resize(f.order.size());
    // references that live inside the flattened graph: parent slots of its nodes, grad fields of its nodes, and the
    // one this function holds in `order`
    std::unordered_map<Node*, long> inside;
    for (auto& n : f.order) {
        inside[n.get()] += 1;
        if (!n->is_realized()) for (auto& p : n->parents) inside[p.get()] += 1;
        if (n->grad) inside[n->grad.get()] += 1;
    }
    for (size_t i = 0; i < f.order.size(); ++i) {
        const auto& n = f.order[i];
        ormi_b200_node& d = f.nodes[i];
        fill(d, *n);
        if (!n->is_realized()) {
            d.n_parents = (int32_t)std::min<size_t>(2, n->parents.size());
            for (int p = 0; p < d.n_parents; ++p) d.parents[p] = index[n->parents[p].get()];
            // Somebody outside this graph still holds the node (a C++ variable, a Python object, a node that was not
            // walked): it must come out realized, like every node does in the reference scheduler
            // (csrc/tests/backend/test_runtime.cpp:42 observes exactly that).
            if (mark_held && n.get() != root.get() && n.use_count() > inside[n.get()]) d.flags |= ORMI_NODE_KEEP;
        } else {
            d.op = ORMI_OP_LEAF;      // a realized node is an input, whatever produced it
        }
    }
    return f;
}

void adopt_results(Flat& f) {
    for (size_t i = 0; i < f.nodes.size(); ++i) {
        const ormi_b200_node& d = f.nodes[i];
        if (f.order[i]->is_realized() || !(d.flags & ORMI_NODE_OWNED)) continue;
        f.order[i]->data = std::make_shared<Buffer>(d.data, (size_t)d.data_bytes, f.order[i]->view.shape, Device(DeviceEnum::CUDA));
    }
    for (size_t i = 0; i < f.nodes.size(); ++i) {     // views share the Buffer of their base (backend/runtime.cpp:20-23)
        if (f.order[i]->is_realized() || !(f.nodes[i].flags & ORMI_NODE_ALIAS)) continue;
        f.order[i]->data = base_of(f.order[i])->data;
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------------- seam 1
class B200Allocator : public IAllocator {
public:
    B200Allocator() { ctx(); }
    void* allocate(size_t bytes) override {
        int dev;
        { std::lock_guard<std::mutex> lock(g_ctx_mutex); dev = g_active_device; }
        void* p = nullptr;
        B200(ormi_b200_alloc(ctx(dev), bytes, &p));
        std::lock_guard<std::mutex> lock(g_ctx_mutex);
        g_owner[p] = dev;
        return p;
    }
    void free(void* ptr, size_t bytes) override {
        if (!ptr) return;
        const int dev = owner_of(ptr);
        { std::lock_guard<std::mutex> lock(g_ctx_mutex); g_owner.erase(ptr); }
        ormi_b200_free(ctx(dev), ptr, bytes);
    }
    void memset(void* ptr, int value, size_t bytes) override { B200(ormi_b200_memset(ctx(owner_of(ptr)), ptr, value, bytes)); }
    void memcpy(void* dst, const void* src, size_t size) override { B200(ormi_b200_memcpy_d2d(ctx(owner_of(dst)), dst, src, size)); }
    void fill_n(void* dst, const void* val_ptr, size_t elements, DType dtype) override {
        ormi_b200_ctx* c = ctx(owner_of(dst));
        switch (dtype) {
            case DType::Float32:
            case DType::Int32: B200(ormi_b200_fill_u32(c, dst, *static_cast<const uint32_t*>(val_ptr), elements)); break;
            case DType::Bool: B200(ormi_b200_fill_u8(c, dst, *static_cast<const uint8_t*>(val_ptr), elements)); break;
            default: throw std::runtime_error("DType is not supported.");
        }
    }
    void copy_device_to_host(void* dst, const void* src, size_t bytes) override { B200(ormi_b200_memcpy_d2h(ctx(owner_of(src)), dst, src, bytes)); }
    void copy_host_to_device(void* dst, const void* src, size_t bytes) override { B200(ormi_b200_memcpy_h2d(ctx(owner_of(dst)), dst, src, bytes)); }
    bool is_host_visible() const override { return false; }
};

IAllocator* get_cuda_allocator() {
    static B200Allocator instance;
    return &instance;
}

// Additive, for hosts above ormi-core (the Python module loads this library anyway): the backend's options
// ("matmul" = fp32 | bf16 | tf32 | 3xtf32, "fusion" = on | off) and counters of the process-wide context.  The
// reference has no runtime options.  Both return non-zero / -1 when there is no GPU.
extern "C" int ormi_engine_b200_set_option(const char* key, const char* value) {
    try { return ormi_b200_set_option(ctx(), key, value); } catch (...) { return 1; }
}
// The device later allocations (and so the graphs built on them) go to; one process per GPU calls it once with its
// local rank.  Non-zero when the device does not exist.
extern "C" int ormi_engine_b200_set_device(int device) {
    try { cuda::set_active_device(device); return 0; } catch (...) { return 1; }
}
extern "C" long long ormi_engine_b200_counter(const char* name) {
    try {
        int64_t v = 0;
        return ormi_b200_get_counter(ctx(), name, &v) == 0 ? (long long)v : -1;
    } catch (...) { return -1; }
}

namespace cuda {

// ---------------------------------------------------------------------------------------------- seam 2
// Realizes the whole un-realized graph under `root` in one call: the fusion scheduler decides what becomes a
// kernel.  Post-conditions of the reference (jit.cu:26-28): root->data set, root->view contiguous.
void set_active_device(int device) {
    ctx(device);                                   // throws when there is no such device
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    g_active_device = device;
}

int active_device() {
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    return g_active_device;
}

ormi_b200_ctx* b200_context(int device) { return ctx(device); }

// The context a graph runs on: the one that owns its realized inputs.  Inputs on two devices, or a node that names
// another device (Device.id) than its inputs live on, are refused.
static int device_of_graph(const Flat& f, const Node& root) {
    int dev = -1;
    for (size_t i = 0; i < f.order.size(); ++i) {
        if (!f.order[i]->is_realized() || !f.nodes[i].data) continue;
        const int d = owner_of(f.nodes[i].data);
        if (dev >= 0 && d != dev) throw std::runtime_error("the graph reads tensors that live on cuda:" + std::to_string(dev) + " and cuda:" + std::to_string(d));
        dev = d;
    }
    if (dev < 0) dev = active_device();
    if (root.device.id != 0 && root.device.id != dev)
        throw std::runtime_error("node placed on cuda:" + std::to_string(root.device.id) + " but its inputs live on cuda:" + std::to_string(dev));
    return dev;
}

void execute_jit(std::shared_ptr<Node> root) {
    if (root->is_realized()) return;
    sync_lowerings();
    Flat f = flatten(root, true);
    int r = (int)f.nodes.size() - 1;
    const int dev = device_of_graph(f, *root);
    B200(ormi_b200_realize(ctx(dev), f.nodes.data(), (int)f.nodes.size(), &r, 1));
    {   // what the backend handed out belongs to that device
        std::lock_guard<std::mutex> lock(g_ctx_mutex);
        for (const auto& d : f.nodes) if (d.flags & ORMI_NODE_OWNED) g_owner[d.data] = dev;
    }
    adopt_results(f);
    if (!is_view(root->op)) root->view.strides = calc_contiguous_strides(root->view.shape);
}

// ---------------------------------------------------------------------------------------------- seam 3
CompilationResult compile(std::shared_ptr<Node> root) {
    sync_lowerings();
    Flat f = flatten(root, false);
    std::vector<char> src(1 << 20);
    std::vector<int> leaves(f.nodes.size() + 1);
    size_t len = 0;
    int n_leaves = 0;
    B200(ormi_b200_compile_source(f.nodes.data(), (int)f.nodes.size(), (int)f.nodes.size() - 1, src.data(), src.size(), &len,
                                  leaves.data(), (int)leaves.size(), &n_leaves));
    CompilationResult res;
    res.kernel_code.assign(src.data(), std::min(len, src.size() - 1));
    for (int i = 0; i < n_leaves; ++i) {
        res.leaf_nodes.push_back(f.order[leaves[i]]);
        res.leaf_names.push_back("LEAF_" + std::to_string(i));
    }
    res.out_shape = root->view.shape;
    res.tensor_size = 1;
    for (int d : root->view.shape) res.tensor_size *= d;
    return res;
}

// ---------------------------------------------------------------------------------------------- seam 5
std::vector<char> compile_ptx(const std::string& kernel_code, CUdevice) {
    size_t len = 0;
    B200(ormi_b200_compile_cubin(kernel_code.c_str(), nullptr, 0, &len));
    std::vector<char> image(len);
    B200(ormi_b200_compile_cubin(kernel_code.c_str(), image.data(), image.size(), &len));
    return image;
}

// ---------------------------------------------------------------------------------------------- seam 4
std::shared_ptr<Buffer> matmul(std::shared_ptr<Buffer> A, const TensorView& view_A, std::shared_ptr<Buffer> B,
                               const TensorView& view_B, const TensorView& out_view) {
    auto out = empty(out_view.shape, DeviceEnum::CUDA);
    B200(ormi_b200_matmul(ctx(owner_of(A->ptr)), static_cast<const float*>(A->ptr), (int)view_A.shape.size(), view_A.shape.data(), view_A.strides.data(),
                          static_cast<const float*>(B->ptr), (int)view_B.shape.size(), view_B.shape.data(), view_B.strides.data(),
                          static_cast<float*>(out->ptr), (int)out_view.shape.size(), out_view.shape.data()));
    return out;
}

void matmul_handler(std::shared_ptr<Node> root) {
    root->data = cuda::matmul(root->parents[0]->data, root->parents[0]->view, root->parents[1]->data, root->parents[1]->view, root->view);
}

std::shared_ptr<Buffer> sum(std::shared_ptr<Buffer> in_buf, const TensorView& in_view, const std::vector<int>& axes,
                            const TensorView& out_view, const bool) {
    auto out = empty(out_view.shape, DeviceEnum::CUDA);
    B200(ormi_b200_sum(ctx(owner_of(in_buf->ptr)), static_cast<const float*>(in_buf->ptr), (int)in_view.shape.size(), in_view.shape.data(), in_view.strides.data(),
                       axes.data(), (int)axes.size(), static_cast<float*>(out->ptr)));
    return out;
}

void sum_handler(std::shared_ptr<Node> root) {
    const auto& attrs = std::get<ReduceAttrs>(root->attrs);
    root->data = cuda::sum(root->parents[0]->data, root->parents[0]->view, attrs.axes, root->view, attrs.keepdims);
}

static RegisterGraphBreaker reg_b200_matmul(DeviceEnum::CUDA, ops::OpEnum::MATMUL, matmul_handler);
static RegisterGraphBreaker reg_b200_sum(DeviceEnum::CUDA, ops::OpEnum::SUM, sum_handler);

// ---------------------------------------------------------------------------------------------- seam 6
// The per-op plug-in point stays populated with the C expressions of the ten pointwise ops.
using Names = const std::vector<std::string>&;
static RegisterCudaLowering low_add(ops::OpEnum::ADD, [](Names o) { return o[0] + " + " + o[1] + ";"; });
static RegisterCudaLowering low_sub(ops::OpEnum::SUB, [](Names o) { return o[0] + " - " + o[1] + ";"; });
static RegisterCudaLowering low_mul(ops::OpEnum::MUL, [](Names o) { return o[0] + " * " + o[1] + ";"; });
static RegisterCudaLowering low_div(ops::OpEnum::DIV, [](Names o) { return o[0] + " / " + o[1] + ";"; });
static RegisterCudaLowering low_pow(ops::OpEnum::POW, [](Names o) { return "ormi_pow(" + o[0] + ", " + o[1] + ");"; });
static RegisterCudaLowering low_neg(ops::OpEnum::NEG, [](Names o) { return "-" + o[0] + ";"; });
static RegisterCudaLowering low_exp(ops::OpEnum::EXP, [](Names o) { return "expf(" + o[0] + ");"; });
static RegisterCudaLowering low_log(ops::OpEnum::LOG, [](Names o) { return "logf(" + o[0] + ");"; });
static RegisterCudaLowering low_sin(ops::OpEnum::SIN, [](Names o) { return "sinf(" + o[0] + ");"; });
static RegisterCudaLowering low_cos(ops::OpEnum::COS, [](Names o) { return "cosf(" + o[0] + ");"; });

}  // namespace cuda
}  // namespace ormi
