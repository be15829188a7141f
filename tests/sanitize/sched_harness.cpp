// C entry point over the fusion scheduler and the code generator alone (no CUDA): what the AddressSanitizer /
// UndefinedBehaviorSanitizer build of tests/test_sanitizers.py links and drives.
#include <cstring>
#include <string>

#include "plan.h"

extern "C" int sched_plan_json(const ormi_b200_node* nodes, int n_nodes, const int* roots, int n_roots, const char* options,
                               char* buf, size_t cap, size_t* out_len) {
    try {
        const ormi_b200::SchedOptions opt = ormi_b200::parse_sched_options(options);
        const ormi_b200::Plan p = ormi_b200::build_plan(nodes, n_nodes, roots, n_roots, opt);
        const std::string js = ormi_b200::plan_to_json(p);
        if (out_len) *out_len = js.size();
        if (buf && cap) { const size_t c = js.size() < cap - 1 ? js.size() : cap - 1; std::memcpy(buf, js.data(), c); buf[c] = 0; }
        return 0;
    } catch (const std::exception& e) {
        if (buf && cap) { std::strncpy(buf, e.what(), cap - 1); buf[cap - 1] = 0; }
        return 1;
    }
}

extern "C" int sched_compile_simple(const ormi_b200_node* nodes, int n_nodes, int root, size_t* out_len) {
    try {
        const ormi_b200::SimpleKernel k = ormi_b200::compile_simple(nodes, n_nodes, root);
        if (out_len) *out_len = k.source.size();
        return k.error.empty() ? 0 : 2;
    } catch (const std::exception&) { return 1; }
}
