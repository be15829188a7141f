// ormi::execute_graph with the one change the B200 backend needs (replaces backend/runtime.cpp when ormi-core is
// built with this backend): on DeviceEnum::CUDA the whole un-realized graph is handed to the backend BEFORE any parent
// is realized, because the reference order — parents first (backend/runtime.cpp:16-18) — leaves nothing to fuse.
// The CPU branch keeps the reference order: parents, view aliasing, graph breakers, JIT.
#include <stdexcept>

#include "backend/runtime.h"
#include "backend/graph_breakers.h"
#include "core/registry.h"
#include "backend/cpu/jit.h"
#include "backend/cuda/jit.cuh"

namespace ormi {

void execute_graph(std::shared_ptr<Node> root) {
    if (root->is_realized()) return;
    if (root->device.type == DeviceEnum::CUDA) {
        cuda::execute_jit(root);
        return;
    }
    for (auto& parent : root->parents) execute_graph(parent);
    if (ViewOpRegistry::get().contains(root->op)) {
        root->data = root->parents[0]->data;
        return;
    }
    if (try_execute_graph_break(root)) return;
    if (root->device.type != DeviceEnum::CPU) throw std::runtime_error("FATAL: Unsupported device for JIT compiler.");
    cpu::execute_jit(root);
}

}  // namespace ormi
