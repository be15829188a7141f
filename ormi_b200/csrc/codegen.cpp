// CUDA C code generation for fused kernels (NVRTC input, compiled for sm_100a).
//
// Replaces ormi::cuda::compile (ormi-core/csrc/backend/cuda/compiler.cu:53-112), which emits one scalar,
// one-element-per-thread kernel per node with a div/mod chain per leaf, and the NVRTC `sum_kernel` of
// ormi::cuda::sum (ormi-core/csrc/backend/cuda/kernels/reduce/sum.cu:29-66), which issues one atomicAdd per
// input element.
//
// Two templates:
//   flat  — pointwise domains (optionally with global sums): grid-stride loop, 128-bit loads/stores,
//           broadcast operands addressed with strides baked in as literals, scalars hoisted.
//   rows  — domains split into rows x columns: a group of T threads owns a row, keeps its VPT elements in
//           registers, and evaluates the expression level by level; a row SUM is a register sum + warp
//           shuffles + (T > 32) one shared-memory exchange, in a fixed order (deterministic, no atomics).
//           Column sums and global sums accumulate in registers across the rows of a persistent block and
//           leave one partial per block; a finalize kernel adds the partials in block order.
//
// Arithmetic follows the reference CPU backend op for op: every + - * / is a separately rounded IEEE fp32
// operation (__fadd_rn etc. forbid FMA contraction, which the CPU interpreter cannot do either:
// ormi-core/csrc/backend/cpu/lowerings/pointwise.cpp:5-15), and exp/log/sin/cos are the accurate CUDA
// functions, never the fast intrinsics.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <functional>
#include <map>
#include <mutex>
#include <sstream>

#include "kernel_ir.h"

namespace ormi_b200 {

std::string device_prelude() {
    return R"PRE(
#ifndef ORMI_PRELUDE
#define ORMI_PRELUDE
// x ** y with the exponents the graphs actually use (0.5, 2, 3, 1, -1, -0.5) evaluated the way a correctly
// rounded powf would come out; anything else is powf.  The rare paths are kept out of line: inlined at every use
// they multiply the code size of an unrolled kernel body and push it out of the instruction cache.
#ifndef ORMI_EMULATE
#define ORMI_NOINLINE __noinline__
#else
#define ORMI_NOINLINE
#endif
__device__ ORMI_NOINLINE float ormi_pow_general(float x, float y) { return powf(x, y); }
__device__ ORMI_NOINLINE float ormi_cube_wide(float x) { return (float)((double)x * (double)x * (double)x); }
// x * x * x as a correctly rounded cube: x*x = x2 + e2 and x2*x = hi + e3 exactly (fused multiply-add residuals), so
// hi + (e3 + e2*x) is the cube to about 2^-46 before the last rounding — no trip through fp64 and its conversion pipe.
__device__ __forceinline__ float ormi_cube(float x) {
    const float x2 = __fmul_rn(x, x), e2 = __fmaf_rn(x, x, -x2);
    const float hi = __fmul_rn(x2, x), e3 = __fmaf_rn(x2, x, -hi);
    const float ah = fabsf(hi);
    if (ah > 1e-25f && ah < 1e38f) return __fadd_rn(hi, __fmaf_rn(e2, x, e3));
    return ormi_cube_wide(x);                                // residuals under- or overflow out here
}
// The comparisons are on a value that does not change inside an element loop (the exponent is a constant leaf in every
// graph seen so far): the compiler hoists them out of the loop by itself.  (Passing a precomputed integer "mode" and
// switching on it was tried: the switch is lowered to an indirect branch per element and cost 10-15 % on the row
// kernels.)
__device__ __forceinline__ float ormi_pow(float x, float y) {
    if (y == 0.5f) return sqrtf(x);
    if (y == 2.0f) return __fmul_rn(x, x);
    if (y == 3.0f) return ormi_cube(x);
    if (y == 1.0f) return x;
    if (y == -1.0f) return __fdiv_rn(1.0f, x);
    if (y == -0.5f) return __frsqrt_rn(x);       // the derivative of a square root: sits on the per-row path of layernorm's backward
    return ormi_pow_general(x, y);
}
// The same for four values and one exponent: one chain of comparisons for the four, and the four results of the branch
// taken are independent instruction streams (GEMM epilogues, where every branch splits what the compiler may interleave).
__device__ __forceinline__ void ormi_pow4(const float* x, float y, float* out) {
    if (y == 0.5f) { for (int j = 0; j < 4; ++j) out[j] = sqrtf(x[j]); }
    else if (y == 2.0f) { for (int j = 0; j < 4; ++j) out[j] = __fmul_rn(x[j], x[j]); }
    else if (y == 3.0f) { for (int j = 0; j < 4; ++j) out[j] = ormi_cube(x[j]); }
    else if (y == 1.0f) { for (int j = 0; j < 4; ++j) out[j] = x[j]; }
    else if (y == -1.0f) { for (int j = 0; j < 4; ++j) out[j] = __fdiv_rn(1.0f, x[j]); }
    else if (y == -0.5f) { for (int j = 0; j < 4; ++j) out[j] = __frsqrt_rn(x[j]); }
    else { for (int j = 0; j < 4; ++j) out[j] = ormi_pow_general(x[j], y); }
}
// GEMM epilogue: sum over the four lanes that hold the same columns of a 32-row block (lanes l, l^8, l^16, l^24)
#ifndef ORMI_EMULATE
// ... and over all 32 lanes (a global sum: one value per 32-row block and 32-column chunk)
__device__ __forceinline__ float ormi_epi_all(float v, bool is_max) {
    for (int o = 16; o > 0; o >>= 1) { const float t = __shfl_xor_sync(0xffffffffu, v, o); v = is_max ? (t > v ? t : v) : __fadd_rn(v, t); }
    return v;
}
__device__ __forceinline__ float ormi_epi_rows(float v, bool is_max) {
    float o = __shfl_xor_sync(0xffffffffu, v, 8);  v = is_max ? (o > v ? o : v) : __fadd_rn(v, o);
    o = __shfl_xor_sync(0xffffffffu, v, 16);       v = is_max ? (o > v ? o : v) : __fadd_rn(v, o);
    return v;
}
#else
__device__ __forceinline__ float ormi_epi_rows(float v, bool) { return v; }   /* the emulator walks the lanes one after the other and carries the sums */
__device__ __forceinline__ float ormi_epi_all(float v, bool) { return v; }
#endif
__device__ __forceinline__ float ormi_warp_sum(float v, int width) {
    for (int o = width >> 1; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float ormi_max(float a, float b) { return b > a ? b : a; }
__device__ __forceinline__ float ormi_warp_max(float v, int width) {
    for (int o = width >> 1; o > 0; o >>= 1) v = ormi_max(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
#define ORMI_NEG_INF __int_as_float(0xff800000)
// fp32 -> bf16, round to nearest even (what the tensor-core matmul reads): one value, and four packed into 8 bytes.
#ifndef ORMI_EMULATE
__device__ __forceinline__ unsigned short ormi_bf16(float x) { unsigned short r; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(x)); return r; }
__device__ __forceinline__ unsigned ormi_pack_bf16(float lo, float hi) { unsigned r; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r; }
#else
__device__ __forceinline__ unsigned short ormi_bf16(float x) {
    unsigned u = __float_as_uint(x);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (unsigned short)0x7fff;
    return (unsigned short)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
__device__ __forceinline__ unsigned ormi_pack_bf16(float lo, float hi) { return (unsigned)ormi_bf16(lo) | ((unsigned)ormi_bf16(hi) << 16); }
#endif
__device__ __forceinline__ void ormi_store_bf16x4(unsigned short* p, float a, float b, float c, float d) {
    *reinterpret_cast<uint2*>(p) = make_uint2(ormi_pack_bf16(a, b), ormi_pack_bf16(c, d));
}
#ifndef ORMI_EMULATE
// Rows staged in shared memory by bulk asynchronous copies (the TMA engine), completion counted on an mbarrier.
#define ORMI_DYN_SMEM(name) extern __shared__ __align__(1024) unsigned char name[]
__device__ __forceinline__ unsigned ormi_smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ormi_mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ormi_smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void ormi_mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void ormi_async_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void ormi_mbar_expect(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ormi_smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ormi_bulk_load(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(ormi_smem_addr(dst)), "l"(src), "r"(bytes), "r"(ormi_smem_addr(bar)) : "memory");
}
__device__ __forceinline__ unsigned long long ormi_global_ns() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
// Bounded wait (about one second): false means the copy never arrived; the caller raises the error word and leaves.
__device__ __forceinline__ bool ormi_mbar_wait(unsigned long long* bar, unsigned parity) {
    const unsigned addr = ormi_smem_addr(bar);
    unsigned long long t0 = 0;
    for (unsigned spin = 0;; ++spin) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
        if ((spin & 255u) == 255u) {
            const unsigned long long now = ormi_global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > 1000000000ull) return false;
        }
    }
}
__device__ __forceinline__ void ormi_drain() { const unsigned long long t0 = ormi_global_ns(); while (ormi_global_ns() - t0 < 200000ull) { } }
#endif
#endif
)PRE";
}

namespace {
std::mutex g_lowering_mutex;
std::map<int, std::string> g_lowerings;
std::atomic<uint64_t> g_lowering_generation{0};
}  // namespace

void set_lowering(int op, const std::string& expr) {
    std::lock_guard<std::mutex> lock(g_lowering_mutex);
    if (expr.empty()) g_lowerings.erase(op); else g_lowerings[op] = expr;
    ++g_lowering_generation;
}

bool lowering_for(int op, std::string* expr) {
    std::lock_guard<std::mutex> lock(g_lowering_mutex);
    auto it = g_lowerings.find(op);
    if (it == g_lowerings.end()) return false;
    if (expr) *expr = it->second;
    return true;
}

uint64_t lowering_generation() { return g_lowering_generation.load(); }

namespace {

int64_t prod(const std::vector<int>& v, size_t a, size_t b) { int64_t p = 1; for (size_t i = a; i < b; ++i) p *= v[i]; return p; }

std::string op_expr(int op, const std::string& a, const std::string& b) {
    std::string custom;
    if (op < 1000 && lowering_for(op, &custom)) {      // a registered lowering replaces the built-in expression
        std::string out;
        for (size_t i = 0; i < custom.size(); ++i) {
            if (custom[i] == '$' && i + 1 < custom.size() && (custom[i + 1] == '0' || custom[i + 1] == '1')) { out += "(" + (custom[i + 1] == '0' ? a : b) + ")"; ++i; }
            else out += custom[i];
        }
        return "(" + out + ")";
    }
    switch (op) {
        case ORMI_OP_ADD: return "__fadd_rn(" + a + ", " + b + ")";
        case ORMI_OP_SUB: return "__fsub_rn(" + a + ", " + b + ")";
        case ORMI_OP_MUL: return "__fmul_rn(" + a + ", " + b + ")";
        case ORMI_OP_DIV: return "__fdiv_rn(" + a + ", " + b + ")";
        case ORMI_OP_POW: return "ormi_pow(" + a + ", " + b + ")";
        case ORMI_OP_NEG: return "-" + a;
        case ORMI_OP_EXP: return "expf(" + a + ")";
        case ORMI_OP_LOG: return "logf(" + a + ")";
        case ORMI_OP_SIN: return "sinf(" + a + ")";
        case ORMI_OP_COS: return "cosf(" + a + ")";
        case ORMI_OP_MAXIMUM: return "(" + a + " >= " + b + " ? " + a + " : " + b + ")";
        case ORMI_OP_GE: return "(" + a + " >= " + b + " ? 1.0f : 0.0f)";
        case KNode::OP_ID: return a;
    }
    return "0.0f /* unknown op */";
}

// identity element, combining expression and warp reduction of a reduction (sum, or maximum for ORMI_OP_MAX)
std::string red_ident(bool is_max) { return is_max ? "ORMI_NEG_INF" : "0.0f"; }
std::string red_comb(bool is_max, const std::string& a, const std::string& b) { return (is_max ? "ormi_max(" : "__fadd_rn(") + a + ", " + b + ")"; }
std::string red_warp(bool is_max) { return is_max ? "ormi_warp_max" : "ormi_warp_sum"; }

int ceil_pow2(int64_t v) { int p = 1; while (p < v) p <<= 1; return p; }

struct LoadInfo {
    bool scalar = true;          // every stride 0
    // rows template
    bool row_var = false;        // depends on the row
    bool elem = false;           // depends on the column
    int64_t sc = 0;              // column stride after collapsing D[k:]
    bool row_collapsed = true;   // row offset = r * sr
    int64_t sr = 0;
};

int64_t touched_bytes(const KLoad& l, const std::vector<int>& D) {
    int64_t e = 1;
    for (size_t d = 0; d < D.size(); ++d) if (l.st[d] != 0) e *= D[d];
    return e * 4;
}

// kernel parameters: one pointer per load, then per output the fp32 pointer (unless only a bf16 twin is wanted) and
// the bf16 twin pointer
std::string param_list(const KernelSpec& spec) {
    std::ostringstream s;
    bool first = true;
    auto sep = [&]() { std::string r = first ? "" : ", "; first = false; return r; };
    for (size_t l = 0; l < spec.loads.size(); ++l) s << sep() << "const float* __restrict__ in" << l;
    for (size_t o = 0; o < spec.outputs.size(); ++o) {
        if (spec.outputs[o].store) s << sep() << "float* __restrict__ out" << o;
        if (spec.outputs[o].twin) s << sep() << "unsigned short* __restrict__ out16_" << o;
    }
    return s.str();
}

// ---------------------------------------------------------------------------------------- flat template
GeneratedKernel generate_flat(const KernelSpec& spec, const std::string& name) {
    GeneratedKernel out;
    const size_t nd = spec.D.size();
    // collapse adjacent dims that every load walks contiguously
    std::vector<int64_t> cs;                     // collapsed sizes
    std::vector<std::vector<int64_t>> lst(spec.loads.size());   // per load, per collapsed dim
    for (size_t d = 0; d < nd; ++d) {
        bool merge = !cs.empty();
        if (merge) for (size_t l = 0; l < spec.loads.size(); ++l) if (lst[l].back() != spec.loads[l].st[d] * spec.D[d]) merge = false;
        if (merge) { cs.back() *= spec.D[d]; for (size_t l = 0; l < spec.loads.size(); ++l) lst[l].back() = spec.loads[l].st[d]; }
        else { cs.push_back(spec.D[d]); for (size_t l = 0; l < spec.loads.size(); ++l) lst[l].push_back(spec.loads[l].st[d]); }
    }
    const size_t cd = cs.size();
    int64_t total = 1; for (int v : spec.D) total *= v;
    int V = 4;
    if (cd == 0 || cs.back() % 4 != 0 || !spec.aligned) V = 1;
    for (size_t l = 0; l < spec.loads.size() && V == 4; ++l) {
        int64_t inner = lst[l].back();
        if (inner != 0 && inner != 1) V = 1;
        if (inner == 1) for (size_t d = 0; d + 1 < cd; ++d) if (lst[l][d] % 4 != 0) V = 1;
    }
    const int NT = 256;
    const int64_t nvec = total / V;
    int grid = (int)std::min<int64_t>((nvec + NT - 1) / NT, (int64_t)spec.num_sms * 8);
    if (grid < 1) grid = 1;
    int n_global = 0;
    for (auto& o : spec.outputs) n_global += (o.kind == KOutput::GLOBALSUM);

    std::ostringstream s;
    s << device_prelude();
    s << "extern \"C\" __global__ void __launch_bounds__(" << NT << ") " << name << "(";
    s << param_list(spec);
    s << ") {\n";
    std::vector<bool> scalar(spec.loads.size());
    for (size_t l = 0; l < spec.loads.size(); ++l) {
        scalar[l] = std::all_of(lst[l].begin(), lst[l].end(), [](int64_t v) { return v == 0; });
        if (scalar[l]) s << "    const float S" << l << " = in" << l << "[0];\n";
    }
    for (size_t o = 0; o < spec.outputs.size(); ++o) if (spec.outputs[o].kind == KOutput::GLOBALSUM) s << "    float gacc" << o << " = " << red_ident(spec.outputs[o].is_max) << ";\n";
    {   // long arithmetic chains are bound by instruction issue, not by memory: two iterations in flight hide the
        // load latency behind the other iteration's arithmetic (measured: GELU forward 165 -> 151 us at 8192 x 8192)
        const int unroll = spec.tune[TUNE_FLAT_UNROLL] > 0 ? spec.tune[TUNE_FLAT_UNROLL] : (spec.nodes.size() >= 8 ? 2 : 1);
        if (unroll > 1) s << "    #pragma unroll " << unroll << "\n";
    }
    s << "    for (int i = blockIdx.x * " << NT << " + threadIdx.x; i < " << nvec << "; i += gridDim.x * " << NT << ") {\n";
    s << "        const int e0 = i * " << V << ";\n";
    if (cd > 1) {
        s << "        int rem = e0;\n";
        for (size_t d = cd; d-- > 1;) s << "        const int c" << d << " = rem % " << cs[d] << "; rem /= " << cs[d] << ";\n";
        s << "        const int c0 = rem;\n";
    } else if (cd == 1) {
        s << "        const int c0 = e0;\n";
    }
    auto ref = [&](const KRef& r) {
        if (r.t == KRef::LOAD) return scalar[r.id] ? "S" + std::to_string(r.id) : "L" + std::to_string(r.id) + "[j]";
        return "v" + std::to_string(r.id) + "[j]";
    };
    for (size_t l = 0; l < spec.loads.size(); ++l) {
        if (scalar[l]) continue;
        s << "        float L" << l << "[" << V << "];\n        {\n            const int off = 0";
        for (size_t d = 0; d < cd; ++d) if (lst[l][d] != 0) s << " + c" << d << " * " << lst[l][d];
        s << ";\n";
        int64_t inner = lst[l].back();
        if (V == 4 && inner == 1) {
            s << "            const float4 t = *reinterpret_cast<const float4*>(in" << l << " + off);\n"
              << "            L" << l << "[0] = t.x; L" << l << "[1] = t.y; L" << l << "[2] = t.z; L" << l << "[3] = t.w;\n";
        } else if (V == 4) {
            s << "            const float t = in" << l << "[off];\n            L" << l << "[0] = t; L" << l << "[1] = t; L" << l << "[2] = t; L" << l << "[3] = t;\n";
        } else {
            s << "            L" << l << "[0] = in" << l << "[off];\n";
        }
        s << "        }\n";
    }
    for (const KNode& kn : spec.nodes) s << "        float v" << kn.node << "[" << V << "];\n";
    s << "        #pragma unroll\n        for (int j = 0; j < " << V << "; ++j) {\n";
    for (const KNode& kn : spec.nodes) {
        std::string a = ref(kn.operands[0]);
        std::string b = kn.operands.size() > 1 ? ref(kn.operands[1]) : "";
        s << "            v" << kn.node << "[j] = " << op_expr(kn.op, a, b) << ";\n";
    }
    s << "        }\n";
    for (size_t o = 0; o < spec.outputs.size(); ++o) {
        const KOutput& ko = spec.outputs[o];
        auto val = [&](int j) {
            if (ko.value.t == KRef::LOAD) return scalar[ko.value.id] ? "S" + std::to_string(ko.value.id) : "L" + std::to_string(ko.value.id) + "[" + std::to_string(j) + "]";
            return "v" + std::to_string(ko.value.id) + "[" + std::to_string(j) + "]";
        };
        if (ko.kind == KOutput::GLOBALSUM) {
            for (int j = 0; j < V; ++j) s << "        gacc" << o << " = " << red_comb(ko.is_max, "gacc" + std::to_string(o), val(j)) << ";\n";
        } else if (V == 4) {
            if (ko.store) s << "        *reinterpret_cast<float4*>(out" << o << " + e0) = make_float4(" << val(0) << ", " << val(1) << ", " << val(2) << ", " << val(3) << ");\n";
            if (ko.twin) s << "        ormi_store_bf16x4(out16_" << o << " + e0, " << val(0) << ", " << val(1) << ", " << val(2) << ", " << val(3) << ");\n";
        } else {
            if (ko.store) s << "        out" << o << "[e0] = " << val(0) << ";\n";
            if (ko.twin) s << "        out16_" << o << "[e0] = ormi_bf16(" << val(0) << ");\n";
        }
    }
    s << "    }\n";
    if (n_global) {
        s << "    __shared__ float gsm[" << n_global << "][" << NT / 32 << "];\n";
        int gi = 0;
        for (size_t o = 0; o < spec.outputs.size(); ++o) if (spec.outputs[o].kind == KOutput::GLOBALSUM) {
            s << "    gacc" << o << " = " << red_warp(spec.outputs[o].is_max) << "(gacc" << o << ", 32);\n";
            s << "    if ((threadIdx.x & 31) == 0) gsm[" << gi << "][threadIdx.x >> 5] = gacc" << o << ";\n";
            ++gi;
        }
        s << "    __syncthreads();\n    if (threadIdx.x == 0) {\n";
        gi = 0;
        for (size_t o = 0; o < spec.outputs.size(); ++o) if (spec.outputs[o].kind == KOutput::GLOBALSUM) {
            s << "        { float a = " << red_ident(spec.outputs[o].is_max) << "; for (int w = 0; w < " << NT / 32 << "; ++w) a = " << red_comb(spec.outputs[o].is_max, "a", "gsm[" + std::to_string(gi) + "][w]") << "; out" << o << "[blockIdx.x] = a; }\n";
            ++gi;
        }
        s << "    }\n";
    }
    s << "}\n";

    out.step.name = name;
    out.step.source = s.str();
    out.step.grid = grid;
    out.step.block = NT;
    out.cols = 1;
    std::ostringstream w;
    w << "flat[total=" << total << ",V=" << V << ",dims=" << cd << "] nodes=" << spec.nodes.size() << " loads=" << spec.loads.size() << " outs=" << spec.outputs.size();
    out.step.what = w.str();
    for (auto& l : spec.loads) out.step.bytes_read += touched_bytes(l, spec.D);
    for (auto& o : spec.outputs) out.step.bytes_written += (o.kind == KOutput::GLOBALSUM) ? 4 * (int64_t)grid : total * ((o.store ? 4 : 0) + (o.twin ? 2 : 0));
    return out;
}

// ---------------------------------------------------------------------------------------- rows template
GeneratedKernel generate_rows(const KernelSpec& spec, const std::string& name) {
    GeneratedKernel out;
    const size_t nd = spec.D.size();
    const int k = spec.k;
    auto unsupported = [&](const std::string& why) { out.error = "row template: " + why; out.unsupported_sums = true; return out; };
    if (k < 1 || k >= (int)nd) return unsupported("no row/column split");
    const int64_t R = prod(spec.D, 0, k), C = prod(spec.D, k, nd);

    std::vector<LoadInfo> li(spec.loads.size());
    bool need_row_coords = false;
    for (size_t l = 0; l < spec.loads.size(); ++l) {
        const auto& st = spec.loads[l].st;
        LoadInfo& I = li[l];
        for (size_t d = k; d + 1 < nd; ++d) if (st[d] != st[d + 1] * spec.D[d + 1]) return unsupported("operand columns are not uniformly strided");
        I.sc = st[nd - 1];
        I.elem = false;
        for (size_t d = k; d < nd; ++d) if (st[d] != 0) I.elem = true;
        if (!I.elem) I.sc = 0;
        I.row_var = false;
        for (int d = 0; d < k; ++d) if (st[d] != 0) I.row_var = true;
        I.scalar = !I.elem && !I.row_var;
        I.row_collapsed = true;
        for (int d = 0; d + 1 < k; ++d) if (st[d] != st[d + 1] * spec.D[d + 1]) I.row_collapsed = false;
        I.sr = st[k - 1];
        if (I.row_var && !I.row_collapsed) need_row_coords = true;
    }
    int V = (C % 4 == 0 && spec.aligned) ? 4 : 1;
    for (size_t l = 0; l < spec.loads.size() && V == 4; ++l) {
        if (!li[l].elem) continue;
        if (li[l].sc != 1) V = 1;
        for (int d = 0; d < k; ++d) if (spec.loads[l].st[d] % 4 != 0) V = 1;
    }
    // Measured defaults below; spec.tune (ormi_b200_set_option "tune.*") overrides them for experiments.
    auto knob = [&](int which, int dflt) { return spec.tune[which] > 0 ? spec.tune[which] : dflt; };
    auto toggle = [&](int which, bool dflt) { return spec.tune[which] == 1 ? false : (spec.tune[which] == 2 ? true : dflt); };
    // Depth = number of dependent row-sum levels.  Defaults measured on B200 at [16384, 4096] (GB/s of algorithmic
    // bytes, measured copy bandwidth 6537):
    //   depth 4 (layernorm fwd+bwd): 16 elements/thread, registers capped for 2 blocks/SM, grid 2/SM, next rows
    //            staged in shared memory (2 stages) -> 5190; same without staging -> 4470; uncapped registers -> 2420.
    //   depth 2 (softmax fwd+bwd):   16 elements/thread, 3 blocks/SM, grid 3/SM, direct loads -> 6370; staged -> 5800.
    //   depth <= 1 (config 1, a 46 us kernel): 8 elements/thread, 2 blocks/SM, staged -> 4570; direct -> 4320.
    int depth = 0;
    {
        std::map<int, int> lvl;
        for (const KNode& kn : spec.nodes) {
            int lv = 0;
            for (auto& r : kn.operands) if (r.t == KRef::NODE) lv = std::max(lv, lvl[r.id]);
            if (kn.op == KNode::OP_ROWSUM) lv += 1;
            lvl[kn.node] = lv;
            depth = std::max(depth, lv);
        }
    }
    // Register demand of the row body: per-element values that must survive a block barrier (defined at or before a
    // reduction level and still read after it) stay in registers across it, next to the vectors that are always live
    // (row-invariant operands held for every row, the column accumulators).  Counted in vectors of VPT elements.
    int live_vectors = 0;
    {
        std::map<int, int> lvl, last;                     // node -> level it is computed at / last level that reads it
        std::vector<int> load_last(spec.loads.size(), 0);
        auto use = [&](const KRef& r, int at) {
            if (r.t == KRef::NODE) last[r.id] = std::max(last[r.id], at);
            else load_last[r.id] = std::max(load_last[r.id], at);
        };
        for (const KNode& kn : spec.nodes) {
            int lv = 0;
            for (auto& r : kn.operands) if (r.t == KRef::NODE) lv = std::max(lv, lvl[r.id]);
            for (auto& r : kn.operands) use(r, lv);       // a row sum reads its operand at the level below its own
            if (kn.op == KNode::OP_ROWSUM) lv += 1;
            lvl[kn.node] = lv;
        }
        for (auto& o : spec.outputs) use(o.value, o.value.t == KRef::NODE ? lvl[o.value.id] : 0);
        int always = 0;
        for (auto& o : spec.outputs) if (o.kind == KOutput::COLSUM) ++always;
        for (size_t l = 0; l < spec.loads.size(); ++l) if (li[l].elem && !li[l].row_var) ++always;
        for (int b = 0; b < depth; ++b) {                 // the barrier between level b and level b + 1
            int live = 0;
            for (const KNode& kn : spec.nodes) if (!(kn.row || kn.scalar) && lvl[kn.node] <= b && last[kn.node] > b) ++live;
            for (size_t l = 0; l < spec.loads.size(); ++l) if (li[l].elem && li[l].row_var && load_last[l] > b) ++live;
            live_vectors = std::max(live_vectors, live + always);
        }
    }
    //   depth <= 1 with no column / global partials, re-measured with three rotated input sets (no operand left in
    //            L2): 8 elements/thread, 4 blocks/SM, grid 4/SM, direct loads -> 5275; 2 blocks/SM staged -> 4880.
    bool pure_rows = true;
    for (auto& o : spec.outputs) if (o.kind == KOutput::COLSUM || o.kind == KOutput::GLOBALSUM) pure_rows = false;
    const bool shallow = depth <= 1 && pure_rows;
    const int target = knob(TUNE_ROWS_VPT, (V == 4 && depth >= 2) ? 16 : 8);
    const bool hoist = toggle(TUNE_ROWS_HOIST, true);
    int T = std::min(1024, std::max(32, ceil_pow2((C + target - 1) / target)));
    int64_t VPT = (C + T - 1) / T;
    VPT = (VPT + V - 1) / V * V;
    //   depth 4 with more live values than two blocks per SM leave registers for (both graphs of the benchmark step in
    //            one kernel: 9 vectors of 16 across a barrier = 144 registers; the 128-register cap spilled 116 bytes per
    //            thread): one block per SM, uncapped, with a 3-stage ring -> 5950; 2 blocks/SM -> 5370.  The layernorm
    //            kernel alone (7 vectors = 112 registers) keeps two blocks: 6000 against 5560.
    const bool heavy = depth >= 3 && live_vectors * VPT > 120;
    int minb = knob(TUNE_ROWS_MINB, shallow ? 4 : (depth == 2 ? 3 : (heavy ? 1 : 2)));
    const int grid_mult = knob(TUNE_ROWS_GRID, shallow ? 4 : (depth == 2 ? 3 : (heavy ? 1 : 2)));
    if (VPT > 32) return unsupported("row of " + std::to_string(C) + " elements does not fit in registers");
    const int NT = std::max(T, 256), G = NT / T, NV = (int)VPT / V, NW = T / 32;
    if (NT * minb > 1024) minb = 0;     // never squeeze a block below 64 registers per thread
    const bool col_pred = (VPT * T != C);
    const bool row_pred = (R % G != 0);
    int grid = (int)std::min<int64_t>((R + G - 1) / G, (int64_t)spec.num_sms * (grid_mult > 0 ? grid_mult : (NT <= 256 ? 4 : (NT <= 512 ? 2 : 1))));
    if (grid < 1) grid = 1;
    if (!hoist) for (auto& I : li) if (I.elem && !I.row_var) I.row_var = true;   // re-read row-invariant vectors every row (L1/L2 hits)

    // Staging: the row-variant operands of the NEXT rows are fetched into a shared-memory ring by bulk asynchronous
    // copies while the current row is being reduced, so global-load latency no longer sits between the barrier phases.
    std::vector<size_t> staged;
    int stages = 0;
    {
        const bool want = toggle(TUNE_ROWS_STAGE, depth != 2 && !shallow);
        bool can = want && V == 4 && G == 1 && !col_pred;
        for (size_t l = 0; can && l < spec.loads.size(); ++l) {
            bool varies = false;
            for (int d = 0; d < k; ++d) if (spec.loads[l].st[d] != 0) varies = true;
            if (!li[l].elem || !varies) continue;
            if (li[l].sc != 1 || !li[l].row_collapsed || li[l].sr % 4 != 0) can = false;
            else staged.push_back(l);
        }
        if (can && !staged.empty()) {
            const int64_t per_stage = (int64_t)staged.size() * C * 4;
            const int64_t budget = (int64_t)(minb >= 3 ? 70 : (minb == 2 ? 100 : 200)) * 1024;
            stages = (int)std::min<int64_t>(knob(TUNE_ROWS_NSTAGE, heavy ? 3 : 2), budget / per_stage);
            if (stages < 2) stages = 0;
        }
        if (!stages) staged.clear();
    }
    auto staged_slot = [&](size_t l) { for (size_t i = 0; i < staged.size(); ++i) if (staged[i] == l) return (int)i; return -1; };

    // levels
    std::map<int, int> level;       // node -> level
    std::map<int, const KNode*> by_id;
    auto ref_level = [&](const KRef& r) { return r.t == KRef::LOAD ? 0 : level[r.id]; };
    int max_level = 0, max_sums_per_level = 0;
    std::map<int, int> sums_at;
    for (const KNode& kn : spec.nodes) {
        by_id[kn.node] = &kn;
        int lv = 0;
        for (auto& r : kn.operands) lv = std::max(lv, ref_level(r));
        if (kn.op == KNode::OP_ROWSUM) { lv += 1; max_sums_per_level = std::max(max_sums_per_level, ++sums_at[lv]); }
        level[kn.node] = lv;
        max_level = std::max(max_level, lv);
    }
    auto rowv = [&](const KNode* kn) { return kn->row || kn->scalar; };
    auto is_elem = [&](const KRef& r) { return r.t == KRef::LOAD ? li[r.id].elem : !rowv(by_id[r.id]); };
    auto ref = [&](const KRef& r, const std::string& j) {
        if (r.t == KRef::LOAD) return "L" + std::to_string(r.id) + (li[r.id].elem ? "[" + j + "]" : "");
        return "v" + std::to_string(r.id) + (rowv(by_id[r.id]) ? "" : "[" + j + "]");
    };
    int n_col = 0, n_glob = 0;
    for (auto& o : spec.outputs) { n_col += (o.kind == KOutput::COLSUM); n_glob += (o.kind == KOutput::GLOBALSUM); }

    std::ostringstream s;
    s << device_prelude();
    s << "extern \"C\" __global__ void __launch_bounds__(" << NT << (minb > 0 ? ", " + std::to_string(minb) : "") << ") " << name << "(";
    s << param_list(spec);
    // Rows handed out dynamically (an atomic counter in the context's word buffer, the next index fetched one row ahead):
    // a block that becomes resident late, because a collective of the second stream holds its SM for a while, takes what
    // is left instead of a fixed share the others would have to wait for.  Only for kernels whose outputs do not depend
    // on which block handled which row (no column / global partials — those stay bit-reproducible with fixed shares)
    // and only when the row loop has a block barrier of its own to publish the next index.
    const bool dyn_rows = !stages && n_col == 0 && n_glob == 0 && max_sums_per_level > 0 && NW > 1 && toggle(TUNE_ROWS_DYNAMIC, true);
    if (stages || dyn_rows) s << ", int* __restrict__ err";
    s << ") {\n";
    s << "    // rows=" << R << " cols=" << C << " threads/row=" << T << " rows/block=" << G << " elems/thread=" << VPT << " vec=" << V << "\n";
    s << "    const int tid = threadIdx.x % " << T << ";\n    const int grp = threadIdx.x / " << T << ";\n";
    // Per-warp partials of the row reductions: one array per level and per row parity, so that a level needs ONE block
    // barrier (write, barrier, read).  The next write to the same array is two rows later, and every row has at least
    // one barrier of its own in between, so no second barrier is needed to protect the reads.
    const bool use_red = max_sums_per_level && NW > 1;
    if (use_red) s << "    __shared__ float red[2][" << std::max(1, max_level) << "][" << max_sums_per_level << "][" << G << "][" << NW << "];\n    int rpar = 0;\n";
    auto col_of = [&](const std::string& q, const std::string& e) { return "((" + q + ") * " + std::to_string(T) + " + tid) * " + std::to_string(V) + " + (" + e + ")"; };
    auto emit_array_load = [&](size_t l, const std::string& ro, const std::string& ind, bool rowp) {
        std::string L = "L" + std::to_string(l), P = "in" + std::to_string(l);
        s << ind << "float " << L << "[" << VPT << "];\n";
        s << ind << "#pragma unroll\n" << ind << "for (int q = 0; q < " << NV << "; ++q) {\n";
        s << ind << "    const int col = " << col_of("q", "0") << ";\n";
        std::string pred;
        if (rowp) pred = "rok";
        if (col_pred) pred += std::string(pred.empty() ? "" : " && ") + "col < " + std::to_string(C);
        if (V == 4) {
            s << ind << "    float4 t = make_float4(0.0f, 0.0f, 0.0f, 0.0f);\n";
            s << ind << "    " << (pred.empty() ? "" : "if (" + pred + ") ") << "t = *reinterpret_cast<const float4*>(" << P << " + " << ro << " + col);\n";
            s << ind << "    " << L << "[4 * q] = t.x; " << L << "[4 * q + 1] = t.y; " << L << "[4 * q + 2] = t.z; " << L << "[4 * q + 3] = t.w;\n";
        } else {
            s << ind << "    " << L << "[q] = " << (pred.empty() ? "" : "(" + pred + ") ? ") << P << "[" << ro << " + col * " << li[l].sc << "]" << (pred.empty() ? "" : " : 0.0f") << ";\n";
        }
        s << ind << "}\n";
    };
    // hoisted loads: row-invariant
    for (size_t l = 0; l < spec.loads.size(); ++l) {
        if (li[l].row_var) continue;
        if (li[l].scalar) s << "    const float L" << l << " = in" << l << "[0];\n";
        else emit_array_load(l, "0", "    ", false);
    }
    for (size_t o = 0; o < spec.outputs.size(); ++o) {
        const std::string ident = red_ident(spec.outputs[o].is_max);
        if (spec.outputs[o].kind == KOutput::COLSUM) { s << "    float cacc" << o << "[" << VPT << "];\n    #pragma unroll\n    for (int j = 0; j < " << VPT << "; ++j) cacc" << o << "[j] = " << ident << ";\n"; }
        if (spec.outputs[o].kind == KOutput::GLOBALSUM) s << "    float gacc" << o << " = " << ident << ";\n";
    }
    if (stages) {
        s << "    ORMI_DYN_SMEM(dsm);\n    float* const ring = reinterpret_cast<float*>(dsm);\n";
        s << "    __shared__ unsigned long long fullbar[" << stages << "];\n";
        s << "    const int n_mine = (" << R << " - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;\n";
        s << "    auto issue = [&](int i) {\n        const int rr = blockIdx.x + i * gridDim.x;\n        const int st = i % " << stages << ";\n";
        s << "        ormi_mbar_expect(&fullbar[st], " << staged.size() * C * 4 << "u);\n";
        for (size_t i = 0; i < staged.size(); ++i)
            s << "        ormi_bulk_load(ring + (st * " << staged.size() << " + " << i << ") * " << C << ", in" << staged[i] << " + (long long)rr * " << li[staged[i]].sr
              << ", " << C * 4 << "u, &fullbar[st]);\n";
        s << "    };\n";
        s << "    if (threadIdx.x == 0) {\n        for (int st = 0; st < " << stages << "; ++st) ormi_mbar_init(&fullbar[st], 1);\n        ormi_mbar_fence_init();\n    }\n";
        s << "    __syncthreads();\n";
        s << "    if (threadIdx.x == 0) for (int i = 0; i < " << stages - 1 << " && i < n_mine; ++i) issue(i);\n";
        s << "    for (int it = 0; it < n_mine; ++it) {\n        const int r = blockIdx.x + it * gridDim.x;\n";
        s << "        const int stg = it % " << stages << ";\n";
        s << "        const bool arrived = ormi_mbar_wait(&fullbar[stg], (unsigned)(it / " << stages << ") & 1u);\n";
    } else {
        if (dyn_rows) {
            s << "    __shared__ int nextrb[2];\n    int* const rowctr = err + " << kRowCounterWord << ";\n";
            // (Giving every block its own index as its first row, to save the round trip to the counter before the first
            // load, was measured on the config-0 row sum: 4900-5000 GB/s against 5370-5400 with every row from the counter.)
            s << "    if (threadIdx.x == 0) nextrb[0] = atomicAdd(rowctr, " << G << ");\n    __syncthreads();\n";
            s << "    for (int it = 0;; ++it) {\n        const int rb = nextrb[it & 1];\n        if (rb >= " << R << ") break;\n";
            s << "        if (threadIdx.x == 0) nextrb[(it + 1) & 1] = atomicAdd(rowctr, " << G << ");     // visible after this row's barriers\n";
        } else {
            s << "    for (int rb = blockIdx.x * " << G << "; rb < " << R << "; rb += gridDim.x * " << G << ") {\n";
        }
        s << "        const int r = rb + grp;\n";
    }
    if (row_pred) s << "        const bool rok = r < " << R << ";\n";
    if (need_row_coords) {
        s << "        int rrem = " << (row_pred ? "rok ? r : 0" : "r") << ";\n";
        for (int d = k - 1; d >= 1; --d) s << "        const int rc" << d << " = rrem % " << spec.D[d] << "; rrem /= " << spec.D[d] << ";\n";
        s << "        const int rc0 = rrem;\n";
    }
    for (size_t l = 0; l < spec.loads.size(); ++l) {
        if (!li[l].row_var) continue;
        std::string ro = "ro" + std::to_string(l);
        bool invariant = true;
        for (int d = 0; d < k; ++d) if (spec.loads[l].st[d] != 0) invariant = false;
        if (invariant) s << "        const int " << ro << " = 0;\n";
        else if (li[l].row_collapsed) s << "        const int " << ro << " = r * " << li[l].sr << ";\n";
        else {
            s << "        const int " << ro << " = 0";
            for (int d = 0; d < k; ++d) if (spec.loads[l].st[d] != 0) s << " + rc" << d << " * " << spec.loads[l].st[d];
            s << ";\n";
        }
        if (li[l].elem && staged_slot(l) >= 0) {
            s << "        float L" << l << "[" << VPT << "];\n        #pragma unroll\n        for (int q = 0; q < " << NV << "; ++q) {\n";
            s << "            const float4 t = *reinterpret_cast<const float4*>(ring + (stg * " << staged.size() << " + " << staged_slot(l) << ") * " << C << " + " << col_of("q", "0") << ");\n";
            s << "            L" << l << "[4 * q] = t.x; L" << l << "[4 * q + 1] = t.y; L" << l << "[4 * q + 2] = t.z; L" << l << "[4 * q + 3] = t.w;\n        }\n";
        }
        else if (li[l].elem) emit_array_load(l, ro, "        ", row_pred);
        else s << "        const float L" << l << " = " << (row_pred ? "rok ? " : "") << "in" << l << "[" << ro << "]" << (row_pred ? " : 0.0f" : "") << ";\n";
    }
    // The stage that the next bulk copy refills was read at the top of an earlier row, and every thread has passed a block
    // barrier since then if the row body has one (a reduction level over more than one warp).  The vote on whether this
    // row's copy arrived then rides on the first such barrier instead of costing one of its own; until then the row's
    // values are only summed, nothing is stored.
    bool level_barrier = false;
    if (NW > 1) for (const KNode& kn : spec.nodes) if (kn.op == KNode::OP_ROWSUM) level_barrier = true;
    const std::string arrival_vote =
        "        if (__syncthreads_or(!arrived)) {\n            if (threadIdx.x == 0) atomicExch(err, 101);\n            ormi_drain();\n            break;\n        }\n"
        "        if (threadIdx.x == 0 && it + " + std::to_string(stages - 1) + " < n_mine) { ormi_async_fence(); issue(it + " + std::to_string(stages - 1) + "); }\n";
    bool vote_pending = stages > 0;
    if (stages && !level_barrier) { s << arrival_vote; vote_pending = false; }
    for (const KNode& kn : spec.nodes) if (!rowv(&kn)) s << "        float v" << kn.node << "[" << VPT << "];\n";

    auto ok_expr = [&](const std::string& j) {
        std::string p;
        if (row_pred) p = "rok";
        if (col_pred) p += std::string(p.empty() ? "" : " && ") + "(" + col_of(j + " / " + std::to_string(V), j + " % " + std::to_string(V)) + ") < " + std::to_string(C);
        return p;
    };
    // An output is written as soon as its value exists (at the end of the level that computes it), not after the last
    // level: a block barrier keeps the compiler from moving a store up, so a late store holds its registers through every
    // level in between.  Nothing is stored before the arrival vote of a staged row.
    std::vector<bool> out_done(spec.outputs.size(), false);
    auto emit_output = [&](size_t o) {
        const KOutput& ko = spec.outputs[o];
        bool elem = is_elem(ko.value);
        if (ko.kind == KOutput::FULL) {
            s << "        #pragma unroll\n        for (int q = 0; q < " << NV << "; ++q) {\n            const int col = " << col_of("q", "0") << ";\n";
            std::string pred;
            if (row_pred) pred = "rok";
            if (col_pred) pred += std::string(pred.empty() ? "" : " && ") + "col < " + std::to_string(C);
            auto v = [&](int e) { return elem ? ref(ko.value, std::to_string(V) + " * q + " + std::to_string(e)) : ref(ko.value, "0"); };
            s << "            " << (pred.empty() ? "" : "if (" + pred + ") ") << "{\n";
            if (V == 4) {
                if (ko.store) s << "                *reinterpret_cast<float4*>(out" << o << " + r * " << C << " + col) = make_float4(" << v(0) << ", " << v(1) << ", " << v(2) << ", " << v(3) << ");\n";
                if (ko.twin) s << "                ormi_store_bf16x4(out16_" << o << " + r * " << C << " + col, " << v(0) << ", " << v(1) << ", " << v(2) << ", " << v(3) << ");\n";
            } else {
                if (ko.store) s << "                out" << o << "[r * " << C << " + col] = " << v(0) << ";\n";
                if (ko.twin) s << "                out16_" << o << "[r * " << C << " + col] = ormi_bf16(" << v(0) << ");\n";
            }
            s << "            }\n        }\n";
        } else if (ko.kind == KOutput::ROW) {
            s << "        if (tid == 0" << (row_pred ? " && rok" : "") << ") out" << o << "[r] = " << ref(ko.value, "0") << ";\n";
        } else if (ko.kind == KOutput::COLSUM) {
            s << "        #pragma unroll\n        for (int j = 0; j < " << VPT << "; ++j) cacc" << o << "[j] = "
              << red_comb(ko.is_max, "cacc" + std::to_string(o) + "[j]", row_pred ? "(rok ? " + ref(ko.value, "j") + " : " + red_ident(ko.is_max) + ")" : ref(ko.value, "j")) << ";\n";
        } else {
            s << "        #pragma unroll\n        for (int j = 0; j < " << VPT << "; ++j) {\n";
            std::string ok = ok_expr("j");
            s << "            gacc" << o << " = " << red_comb(ko.is_max, "gacc" + std::to_string(o), ok.empty() ? ref(ko.value, "j") : "((" + ok + ") ? " + ref(ko.value, "j") + " : " + red_ident(ko.is_max) + ")") << ";\n        }\n";
        }
    };
    const bool custom_div = lowering_for(ORMI_OP_DIV, nullptr);     // a registered lowering for DIV is emitted as written
    for (int lv = 0; lv <= max_level; ++lv) {
        // (a) per-row scalars of this level
        for (const KNode& kn : spec.nodes) {
            if (!rowv(&kn) || kn.op == KNode::OP_ROWSUM || level[kn.node] != lv) continue;
            std::string a = ref(kn.operands[0], "0"), b = kn.operands.size() > 1 ? ref(kn.operands[1], "0") : "";
            s << "        const float v" << kn.node << " = " << op_expr(kn.op, a, b) << ";\n";
        }
        // (b) per-element values of this level
        bool any = false;
        for (const KNode& kn : spec.nodes) if (!rowv(&kn) && level[kn.node] == lv) any = true;
        if (any) {
            // A division of a per-element value by a per-row (or scalar) divisor becomes one correctly rounded
            // reciprocal per row and a multiplication per element: at most ~2 ulp (2.4e-7) away from the IEEE
            // quotient, inside the 1e-6 pointwise tolerance, and about ten instructions per element cheaper —
            // the deep row kernels are instruction-issue bound, not only bandwidth bound.
            for (const KNode& kn : spec.nodes) {
                if (rowv(&kn) || level[kn.node] != lv || kn.op != ORMI_OP_DIV || is_elem(kn.operands[1]) || custom_div) continue;
                s << "        const float rcp" << kn.node << " = __frcp_rn(" << ref(kn.operands[1], "0") << ");\n";
            }
            s << "        #pragma unroll\n        for (int j = 0; j < " << VPT << "; ++j) {\n";
            for (const KNode& kn : spec.nodes) {
                if (rowv(&kn) || level[kn.node] != lv) continue;
                std::string a = ref(kn.operands[0], "j"), b = kn.operands.size() > 1 ? ref(kn.operands[1], "j") : "";
                if (kn.op == ORMI_OP_DIV && !is_elem(kn.operands[1]) && !custom_div)
                    s << "            v" << kn.node << "[j] = __fmul_rn(" << a << ", rcp" << kn.node << ");\n";
                else
                    s << "            v" << kn.node << "[j] = " << op_expr(kn.op, a, b) << ";\n";
            }
            s << "        }\n";
        }
        // (c) row sums that become available after this level
        std::vector<const KNode*> sums;
        for (const KNode& kn : spec.nodes) if (kn.op == KNode::OP_ROWSUM && level[kn.node] == lv + 1) sums.push_back(&kn);
        if (!sums.empty()) {
            for (auto* kn : sums) s << "        float v" << kn->node << " = " << red_ident(kn->is_max) << ";\n";
            s << "        #pragma unroll\n        for (int j = 0; j < " << VPT << "; ++j) {\n";
            std::string ok = ok_expr("j");
            if (!ok.empty()) s << "            const bool ok = " << ok << ";\n";
            for (auto* kn : sums) {
                std::string val = ref(kn->operands[0], "j");
                s << "            v" << kn->node << " = " << red_comb(kn->is_max, "v" + std::to_string(kn->node), ok.empty() ? val : "(ok ? " + val + " : " + red_ident(kn->is_max) + ")") << ";\n";
            }
            s << "        }\n";
            for (auto* kn : sums) s << "        v" << kn->node << " = " << red_warp(kn->is_max) << "(v" << kn->node << ", " << std::min(T, 32) << ");\n";
            if (NW > 1) {
                s << "        if ((threadIdx.x & 31) == 0) {";
                for (size_t i = 0; i < sums.size(); ++i) s << " red[rpar][" << lv << "][" << i << "][grp][tid >> 5] = v" << sums[i]->node << ";";
                s << " }\n";
                if (vote_pending) { s << arrival_vote; vote_pending = false; }
                else s << "        __syncthreads();\n";
                for (size_t i = 0; i < sums.size(); ++i)
                    s << "        { float a = " << red_ident(sums[i]->is_max) << "; for (int w = 0; w < " << NW << "; ++w) a = " << red_comb(sums[i]->is_max, "a", "red[rpar][" + std::to_string(lv) + "][" + std::to_string(i) + "][grp][w]") << "; v" << sums[i]->node << " = a; }\n";
            }
        }
        if (!vote_pending)
            for (size_t o = 0; o < spec.outputs.size(); ++o)
                if (!out_done[o] && ref_level(spec.outputs[o].value) <= lv) { emit_output(o); out_done[o] = true; }
    }
    if (vote_pending) { s << arrival_vote; vote_pending = false; }
    for (size_t o = 0; o < spec.outputs.size(); ++o) if (!out_done[o]) { emit_output(o); out_done[o] = true; }
    if (use_red) s << "        rpar ^= 1;\n";
    s << "    }\n";
    if (dyn_rows)   // every block drew exactly one index past the end; the last one to say so leaves the pair at zero
        s << "    if (threadIdx.x == 0 && atomicAdd(rowctr + 1, 1) == (int)gridDim.x - 1) { rowctr[1] = 0; __threadfence(); atomicExch(rowctr, 0); }\n";
    // epilogue: one partial per block
    if (n_col) {
        if (G > 1) s << "    __shared__ float csm[" << G << "][" << T * VPT << "];\n";
        for (size_t o = 0; o < spec.outputs.size(); ++o) {
            if (spec.outputs[o].kind != KOutput::COLSUM) continue;
            if (G > 1) {
                s << "    #pragma unroll\n    for (int j = 0; j < " << VPT << "; ++j) csm[grp][j * " << T << " + tid] = cacc" << o << "[j];\n    __syncthreads();\n";
                s << "    if (grp == 0) {\n        #pragma unroll\n        for (int j = 0; j < " << VPT << "; ++j) { float a = " << red_ident(spec.outputs[o].is_max) << "; for (int g = 0; g < " << G << "; ++g) a = " << red_comb(spec.outputs[o].is_max, "a", "csm[g][j * " + std::to_string(T) + " + tid]") << "; cacc" << o << "[j] = a; }\n    }\n    __syncthreads();\n";
            }
            s << "    if (grp == 0) {\n        #pragma unroll\n        for (int q = 0; q < " << NV << "; ++q) {\n            const int col = " << col_of("q", "0") << ";\n";
            s << "            " << (col_pred ? "if (col < " + std::to_string(C) + ") " : "");
            if (V == 4) s << "*reinterpret_cast<float4*>(out" << o << " + blockIdx.x * " << C << " + col) = make_float4(cacc" << o << "[4 * q], cacc" << o << "[4 * q + 1], cacc" << o << "[4 * q + 2], cacc" << o << "[4 * q + 3]);\n";
            else s << "out" << o << "[blockIdx.x * " << C << " + col] = cacc" << o << "[q];\n";
            s << "        }\n    }\n";
        }
    }
    if (n_glob) {
        s << "    __shared__ float gsm[" << n_glob << "][" << NT / 32 << "];\n";
        int gi = 0;
        for (size_t o = 0; o < spec.outputs.size(); ++o) if (spec.outputs[o].kind == KOutput::GLOBALSUM) {
            s << "    gacc" << o << " = " << red_warp(spec.outputs[o].is_max) << "(gacc" << o << ", 32);\n    if ((threadIdx.x & 31) == 0) gsm[" << gi << "][threadIdx.x >> 5] = gacc" << o << ";\n";
            ++gi;
        }
        s << "    __syncthreads();\n    if (threadIdx.x == 0) {\n";
        gi = 0;
        for (size_t o = 0; o < spec.outputs.size(); ++o) if (spec.outputs[o].kind == KOutput::GLOBALSUM) {
            s << "        { float a = " << red_ident(spec.outputs[o].is_max) << "; for (int w = 0; w < " << NT / 32 << "; ++w) a = " << red_comb(spec.outputs[o].is_max, "a", "gsm[" + std::to_string(gi) + "][w]") << "; out" << o << "[blockIdx.x] = a; }\n";
            ++gi;
        }
        s << "    }\n";
    }
    s << "}\n";

    out.step.name = name;
    out.step.source = s.str();
    out.step.grid = grid;
    out.step.block = NT;
    out.step.dyn_smem = stages ? (int)(stages * (int64_t)staged.size() * C * 4) : 0;
    out.step.err_arg = stages > 0 || dyn_rows;
    out.cols = C;
    std::ostringstream w;
    w << "rows[R=" << R << ",C=" << C << ",T=" << T << ",G=" << G << ",VPT=" << VPT << ",V=" << V << ",levels=" << max_level << ",stages=" << stages << (dyn_rows ? ",dyn" : "") << ",live=" << live_vectors << "] nodes=" << spec.nodes.size()
      << " loads=" << spec.loads.size() << " outs=";
    for (auto& o : spec.outputs) w << (o.kind == KOutput::FULL ? "F" : o.kind == KOutput::ROW ? "R" : o.kind == KOutput::COLSUM ? "C" : "G");
    out.step.what = w.str();
    for (auto& l : spec.loads) out.step.bytes_read += touched_bytes(l, spec.D);
    for (auto& o : spec.outputs) {
        if (o.kind == KOutput::FULL) out.step.bytes_written += R * C * ((o.store ? 4 : 0) + (o.twin ? 2 : 0));
        else if (o.kind == KOutput::ROW) out.step.bytes_written += R * 4;
        else if (o.kind == KOutput::COLSUM) out.step.bytes_written += (int64_t)grid * C * 4;
        else out.step.bytes_written += (int64_t)grid * 4;
    }
    return out;
}

}  // namespace

GeneratedKernel generate_kernel(const KernelSpec& spec, const std::string& name, const ormi_b200_node*) {
    bool rows = false;
    for (auto& kn : spec.nodes) if (kn.row || kn.op == KNode::OP_ROWSUM) rows = true;
    for (auto& o : spec.outputs) if (o.kind == KOutput::ROW || o.kind == KOutput::COLSUM) rows = true;
    GeneratedKernel g = rows ? generate_rows(spec, name) : generate_flat(spec, name);
    if (g.error.empty()) g.step.key = std::to_string(fnv1a(g.step.source));
    return g;
}

// The pointwise work that follows a matmul, as the epilogue of the tensor-core GEMM template (gemm_tc_template.cuh).
// The template hands this code `acc` (float4: four adjacent columns of one row of the product), `grow`, `gcol`, `M`, `N`;
// every global access below is a 16-byte piece of a row, eight lanes covering a full 128-byte line.  The text is
// spliced in through macros, so it holds no comments and no preprocessor lines.
GeneratedEpilogue generate_gemm_epilogue(const KernelSpec& spec, bool store_c, bool twin_c) {
    GeneratedEpilogue g;
    if (spec.D.size() != 2) { g.error = "epilogue: domain is not [M, N]"; return g; }
    const int64_t N = spec.D[1];
    if (N % 4 != 0) { g.error = "epilogue: N is not a multiple of 4"; return g; }
    std::ostringstream params, init, cols, pre, body, end;
    for (size_t l = 0; l < spec.loads.size(); ++l) {
        const KLoad& ld = spec.loads[l];
        if (ld.acc) continue;
        const int64_t sm = ld.st[0], sn = ld.st[1];
        params << ", const float* __restrict__ ein" << l;
        const std::string P = "ein" + std::to_string(l), L = "L" + std::to_string(l);
        if (sm == 0 && sn == 0) {
            init << "const float S" << l << " = " << P << "[0]; ";
        } else if (sm == 0) {
            cols << "float " << L << "[4]; ";
            if (sn == 1) cols << "{ const float4 t = *reinterpret_cast<const float4*>(" << P << " + gc); " << L << "[0] = t.x; " << L << "[1] = t.y; " << L << "[2] = t.z; " << L << "[3] = t.w; } ";
            else cols << "for (int j = 0; j < 4; ++j) " << L << "[j] = " << P << "[(long long)(gc + j) * " << sn << "]; ";
        } else {
            body << "float " << L << "[4]; ";
            if (sn == 1 && sm % 4 == 0) {
                // A full matrix read beside the accumulator: the piece for the NEXT row step (4 rows further down) is
                // requested before this step's arithmetic, so the load's latency hides behind it even when the row
                // loop is not unrolled.  N<l> carries the piece from one step to the next.
                const std::string Nx = "N" + std::to_string(l);
                cols << "float4 " << Nx << " = make_float4(0.0f, 0.0f, 0.0f, 0.0f); if (row0 + rsub < M && gcol < N) " << Nx
                     << " = *reinterpret_cast<const float4*>(" << P << " + (long long)(row0 + rsub) * " << sm << " + gcol); ";
                pre << "const float4 T" << l << " = " << Nx << "; if (p < 7 && grow + 4 < M && gcol < N) " << Nx
                    << " = *reinterpret_cast<const float4*>(" << P << " + (long long)(grow + 4) * " << sm << " + gcol); ";
                body << L << "[0] = T" << l << ".x; " << L << "[1] = T" << l << ".y; " << L << "[2] = T" << l << ".z; " << L << "[3] = T" << l << ".w; ";
            } else if (sn == 0) {
                body << "{ const float t = " << P << "[(long long)grow * " << sm << "]; " << L << "[0] = t; " << L << "[1] = t; " << L << "[2] = t; " << L << "[3] = t; } ";
            } else {
                body << "for (int j = 0; j < 4; ++j) " << L << "[j] = " << P << "[(long long)grow * " << sm << " + (long long)(gcol + j) * " << sn << "]; ";
            }
        }
    }
    // lanes whose columns lie beyond N (the last 32-column chunk may run past it) read column 0 instead and store nothing
    const bool col_loads = !cols.str().empty();
    for (size_t o = 0; o < spec.outputs.size(); ++o)
        if (spec.outputs[o].kind == KOutput::COLSUM) cols << "float cs" << o << "[4] = {" << red_ident(spec.outputs[o].is_max) << ", " << red_ident(spec.outputs[o].is_max) << ", "
                                                          << red_ident(spec.outputs[o].is_max) << ", " << red_ident(spec.outputs[o].is_max) << "}; ";
        else if (spec.outputs[o].kind == KOutput::GLOBALSUM) cols << "float gs" << o << " = " << red_ident(spec.outputs[o].is_max) << "; ";
    std::string cols_text = cols.str();
    if (col_loads) cols_text = "const int gc = gcol < N ? gcol : 0; " + cols_text;
    auto ref = [&](const KRef& r) {
        if (r.t == KRef::LOAD) {
            const KLoad& ld = spec.loads[r.id];
            if (ld.acc) return std::string("A[j]");
            if (ld.st[0] == 0 && ld.st[1] == 0) return "S" + std::to_string(r.id);
            return "L" + std::to_string(r.id) + "[j]";
        }
        return "v" + std::to_string(r.id) + "[j]";
    };
    body << "const float A[4] = {acc.x, acc.y, acc.z, acc.w}; ";
    for (const KNode& kn : spec.nodes) body << "float v" << kn.node << "[4]; ";
    // Node by node over the four columns (not column by column over the nodes): the four chains are side by side in
    // program order, and a POW by a per-kernel exponent decides its special case once for the four.
    const bool node_major = spec.tune[TUNE_EPI_NODE_MAJOR] != 1;
    if (!spec.nodes.empty() && node_major) {
        auto at_j = [](std::string r, int j) { size_t p = r.find("[j]"); if (p != std::string::npos) r.replace(p, 3, "[" + std::to_string(j) + "]"); return r; };
        for (const KNode& kn : spec.nodes) {
            const std::string a = ref(kn.operands[0]);
            const std::string b = kn.operands.size() > 1 ? ref(kn.operands[1]) : "";
            const bool a_elem = a.find("[j]") != std::string::npos, b_elem = b.find("[j]") != std::string::npos;
            if (kn.op == ORMI_OP_POW && a_elem && !b_elem && !lowering_for(ORMI_OP_POW, nullptr)) {
                body << "ormi_pow4(" << a.substr(0, a.find("[j]")) << ", " << b << ", v" << kn.node << "); ";
                continue;
            }
            for (int j = 0; j < 4; ++j) body << "v" << kn.node << "[" << j << "] = " << op_expr(kn.op, at_j(a, j), at_j(b, j)) << "; ";
        }
    } else if (!spec.nodes.empty()) {
        body << "_Pragma(\"unroll\") for (int j = 0; j < 4; ++j) { ";
        for (const KNode& kn : spec.nodes) {
            std::string a = ref(kn.operands[0]);
            std::string b = kn.operands.size() > 1 ? ref(kn.operands[1]) : "";
            body << "v" << kn.node << "[j] = " << op_expr(kn.op, a, b) << "; ";
        }
        body << "} ";
    }
    const std::string at = " + (long long)grow * " + std::to_string(N) + " + gcol";
    if (store_c) body << "*reinterpret_cast<float4*>(C" << at << ") = acc; ";
    for (size_t o = 0; o < spec.outputs.size(); ++o) {
        const KOutput& ko = spec.outputs[o];
        if (ko.kind != KOutput::FULL && ko.kind != KOutput::COLSUM && ko.kind != KOutput::GLOBALSUM) { g.error = "epilogue: row outputs are not supported"; return g; }
        auto val = [&](int j) {
            std::string r = ref(ko.value);
            size_t p = r.find("[j]");
            if (p != std::string::npos) r.replace(p, 3, "[" + std::to_string(j) + "]");
            return r;
        };
        if (ko.kind == KOutput::COLSUM) {
            // per chunk: this lane adds its rows of its four columns, the four lanes that share those columns are
            // combined, and one of them writes the 32-row block's partial; a finalize kernel adds the blocks in order
            params << ", float* __restrict__ eout" << o;
            for (int j = 0; j < 4; ++j) body << "cs" << o << "[" << j << "] = " << red_comb(ko.is_max, "cs" + std::to_string(o) + "[" + std::to_string(j) + "]", val(j)) << "; ";
            end << "{ ";
            for (int j = 0; j < 4; ++j) end << "cs" << o << "[" << j << "] = ormi_epi_rows(cs" << o << "[" << j << "], " << (ko.is_max ? "true" : "false") << "); ";
            end << "if (rsub == 0 && gcol < N) *reinterpret_cast<float4*>(eout" << o << " + (long long)(row0 >> 5) * " << N << " + gcol) = make_float4(cs" << o << "[0], cs" << o
                << "[1], cs" << o << "[2], cs" << o << "[3]); } ";
            continue;
        }
        if (ko.kind == KOutput::GLOBALSUM) {
            // one partial per 32-row block and 32-column chunk: [row block][chunk], added up in that order by a finalize kernel
            params << ", float* __restrict__ eout" << o;
            for (int j = 0; j < 4; ++j) body << "gs" << o << " = " << red_comb(ko.is_max, "gs" + std::to_string(o), val(j)) << "; ";
            end << "{ gs" << o << " = ormi_epi_all(gs" << o << ", " << (ko.is_max ? "true" : "false") << "); if (lane == 0) eout" << o << "[(long long)(row0 >> 5) * "
                << (N + 31) / 32 << " + (col0 >> 5)] = gs" << o << "; } ";
            continue;
        }
        if (ko.store) {
            params << ", float* __restrict__ eout" << o;
            body << "*reinterpret_cast<float4*>(eout" << o << at << ") = make_float4(" << val(0) << ", " << val(1) << ", " << val(2) << ", " << val(3) << "); ";
        }
        if (ko.twin) {
            params << ", unsigned short* __restrict__ eout16_" << o;
            body << "ormi_store_bf16x4(eout16_" << o << at << ", " << val(0) << ", " << val(1) << ", " << val(2) << ", " << val(3) << "); ";
        }
    }
    if (twin_c) {
        params << ", unsigned short* __restrict__ ec16";
        body << "ormi_store_bf16x4(ec16" << at << ", acc.x, acc.y, acc.z, acc.w); ";
    }
    g.prelude = device_prelude();
    g.params = params.str();
    g.init = init.str();
    g.cols = cols_text;
    g.pre = pre.str();
    g.body = body.str();
    g.end = end.str();
    g.unroll = spec.nodes.size() <= 4 ? 8 : (spec.nodes.size() <= 10 ? 2 : 1);
    if (spec.tune[TUNE_EPI_UNROLL] == 1 || spec.tune[TUNE_EPI_UNROLL] == 2 || spec.tune[TUNE_EPI_UNROLL] == 4 || spec.tune[TUNE_EPI_UNROLL] == 8) g.unroll = spec.tune[TUNE_EPI_UNROLL];
    // exact exp / division chains cost tens of instructions per element: give them more epilogue warps
    g.wpq = spec.nodes.size() <= 2 ? 1 : (spec.nodes.size() <= 6 ? 2 : 4);
    if (spec.tune[TUNE_EPI_WPQ] == 1 || spec.tune[TUNE_EPI_WPQ] == 2 || spec.tune[TUNE_EPI_WPQ] == 4) g.wpq = spec.tune[TUNE_EPI_WPQ];
    return g;
}

GeneratedKernel generate_finalize(int parts, int64_t width, const std::string& name, bool is_max, int count, unsigned max_bits) {
    GeneratedKernel g;
    std::ostringstream s;
    if (count == 1) max_bits = is_max ? 1u : 0u;
    s << device_prelude();
    s << "extern \"C\" __global__ void __launch_bounds__(256) " << name << "(";
    for (int i = 0; i < count; ++i) s << (i ? ", " : "") << "const float* __restrict__ part" << i << ", float* __restrict__ out" << i;
    s << ") {\n";
    if (width == 1) {
        // one block per pair
        s << "    __shared__ float sm[8];\n";
        for (int i = 0; i < count; ++i) {
            const bool mx = (max_bits >> i) & 1u;
            s << "    if (blockIdx.x == " << i << ") {\n        float a = " << red_ident(mx) << ";\n"
              << "        for (int p = threadIdx.x; p < " << parts << "; p += 256) a = " << red_comb(mx, "a", "part" + std::to_string(i) + "[p]") << ";\n"
              << "        a = " << red_warp(mx) << "(a, 32);\n        if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = a;\n        __syncthreads();\n"
              << "        if (threadIdx.x == 0) { float t = " << red_ident(mx) << "; for (int w = 0; w < 8; ++w) t = " << red_comb(mx, "t", "sm[w]") << "; out" << i << "[0] = t; }\n    }\n";
        }
        s << "}\n";
        g.step.grid = count;
    } else {
        // 32 columns per block; the 8 warps split the partials (warp w takes p = w, w + 8, ...), so a column's chain of
        // dependent additions is parts / 8 long and every load is a full 128-byte line; the 8 sub-sums are added in order.
        const int bx = (int)((width + 31) / 32);
        s << "    __shared__ float sm[8][32];\n"
          << "    const int pair = blockIdx.x / " << bx << ";\n"
          << "    const int c = (blockIdx.x % " << bx << ") * 32 + (threadIdx.x & 31), w = threadIdx.x >> 5;\n";
        for (int i = 0; i < count; ++i) {
            const bool mx = (max_bits >> i) & 1u;
            s << "    if (pair == " << i << ") {\n        float a = " << red_ident(mx) << ";\n"
              << "        if (c < " << width << ") for (int p = w; p < " << parts << "; p += 8) a = " << red_comb(mx, "a", "part" + std::to_string(i) + "[(long long)p * " + std::to_string(width) + " + c]") << ";\n"
              << "        sm[w][threadIdx.x & 31] = a;\n        __syncthreads();\n"
              << "        if (w == 0 && c < " << width << ") { float t = sm[0][threadIdx.x]; for (int k = 1; k < 8; ++k) t = " << red_comb(mx, "t", "sm[k][threadIdx.x]") << "; out" << i << "[c] = t; }\n    }\n";
        }
        s << "}\n";
        g.step.grid = bx * count;
    }
    g.step.block = 256;
    g.step.name = name;
    g.step.source = s.str();
    g.step.key = std::to_string(fnv1a(g.step.source));
    g.step.what = std::string(max_bits ? "finalize_max" : "finalize") + "[parts=" + std::to_string(parts) + ",width=" + std::to_string(width) + (count > 1 ? ",outputs=" + std::to_string(count) : "") + "]";
    g.step.bytes_read = (int64_t)parts * width * 4 * count;
    g.step.bytes_written = width * 4 * count;
    return g;
}

GeneratedKernel generate_generic_sum(const std::vector<int>& shape, const std::vector<int>& strides,
                                     const std::vector<bool>& reduced, const std::string& name, bool is_max) {
    GeneratedKernel g;
    int64_t n_out = 1, n_red = 1;
    for (size_t d = 0; d < shape.size(); ++d) (reduced[d] ? n_red : n_out) *= shape[d];
    std::ostringstream s;
    s << device_prelude();
    // Few outputs over many inputs (a global or near-global sum of a transposed or expanded tensor): one BLOCK per
    // output — its threads stride over the reduced coordinates, then a fixed-order tree — instead of one thread
    // walking 10^8 elements on its own.  Many outputs: one thread each, as the inputs of neighbouring threads then sit
    // side by side.
    const bool block_per_output = n_out < 4096 && n_red >= 1024;
    s << "extern \"C\" __global__ void __launch_bounds__(256) " << name << "(const float* __restrict__ in, float* __restrict__ out) {\n";
    if (block_per_output) s << "    const int o = blockIdx.x;\n";
    else s << "    const int o = blockIdx.x * 256 + threadIdx.x;\n    if (o >= " << n_out << ") return;\n";
    s << "    int base = 0;\n    {\n        int rem = o;\n";
    for (size_t d = shape.size(); d-- > 0;) if (!reduced[d]) s << "        base += (rem % " << shape[d] << ") * " << strides[d] << "; rem /= " << shape[d] << ";\n";
    s << "    }\n    float a = " << red_ident(is_max) << ";\n";
    s << "    for (int e = " << (block_per_output ? "threadIdx.x" : "0") << "; e < " << n_red << "; e += " << (block_per_output ? 256 : 1) << ") {\n        int rem = e, off = base;\n";
    for (size_t d = shape.size(); d-- > 0;) if (reduced[d]) s << "        off += (rem % " << shape[d] << ") * " << strides[d] << "; rem /= " << shape[d] << ";\n";
    s << "        a = " << red_comb(is_max, "a", "in[off]") << ";\n    }\n";
    if (block_per_output) {
        s << "    __shared__ float sm[8];\n    a = " << red_warp(is_max) << "(a, 32);\n    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = a;\n    __syncthreads();\n"
          << "    if (threadIdx.x == 0) { float t = " << red_ident(is_max) << "; for (int w = 0; w < 8; ++w) t = " << red_comb(is_max, "t", "sm[w]") << "; out[o] = t; }\n}\n";
        g.step.grid = (int)n_out;
    } else {
        s << "    out[o] = a;\n}\n";
        g.step.grid = (int)((n_out + 255) / 256);
    }
    g.step.block = 256;
    g.step.name = name;
    g.step.source = s.str();
    g.step.key = std::to_string(fnv1a(g.step.source));
    g.step.what = std::string("generic_sum[out=") + std::to_string(n_out) + ",red=" + std::to_string(n_red) + (block_per_output ? ",block" : "") + "]";
    g.step.bytes_read = n_out * n_red * 4;
    g.step.bytes_written = n_out * 4;
    return g;
}

// ---------------------------------------------------------------------------------------- reference-shaped compile()
SimpleKernel compile_simple(const ormi_b200_node* nodes, int n_nodes, int root) {
    SimpleKernel k;
    if (root < 0 || root >= n_nodes) { k.error = "root out of range"; return k; }
    std::map<int, std::string> visited;
    struct Stmt { std::string var; int op; std::vector<std::string> operands; };
    std::vector<Stmt> tape;
    int var_counter = 0;
    std::string err;
    std::function<std::string(int)> build = [&](int i) -> std::string {
        auto it = visited.find(i);
        if (it != visited.end()) return it->second;
        const auto& nd = nodes[i];
        if (nd.data) {
            std::string v = "val_LEAF_" + std::to_string(k.leaves.size());
            k.leaves.push_back(i);
            visited[i] = v;
            return v;
        }
        std::vector<std::string> ops;
        for (int p = 0; p < nd.n_parents; ++p) ops.push_back(build(nd.parents[p]));
        if (nd.op == ORMI_OP_MATMUL) { err = "FATAL: MATMUL cannot be fused into a 1D element-wise kernel."; return "0"; }
        if (!(nd.op >= ORMI_OP_NEG && nd.op <= ORMI_OP_POW)) { err = "CUDA JIT Compiler Error: No lowering rule registered for this operation."; return "0"; }
        std::string v = "v" + std::to_string(var_counter++);
        tape.push_back(Stmt{v, nd.op, ops});
        visited[i] = v;
        return v;
    };
    std::string root_var = build(root);
    if (!err.empty()) { k.error = err; return k; }
    const auto& rn = nodes[root];
    k.tensor_size = 1;
    for (int d = 0; d < rn.ndim; ++d) k.tensor_size *= rn.shape[d];
    std::ostringstream s;
    s << device_prelude();
    s << "extern \"C\" __global__\nvoid fused_kernel(float* OUT_Z";
    for (size_t l = 0; l < k.leaves.size(); ++l) s << ", const float* LEAF_" << l;
    s << ") {\n    int idx = blockIdx.x * blockDim.x + threadIdx.x;\n    if (idx >= " << k.tensor_size << ") return;\n\n";
    std::vector<int> ostr(rn.ndim, 1);
    for (int d = rn.ndim - 2; d >= 0; --d) ostr[d] = ostr[d + 1] * rn.shape[d + 1];
    for (size_t l = 0; l < k.leaves.size(); ++l) {
        const auto& lf = nodes[k.leaves[l]];
        bool scalar = lf.ndim == 0 || lf.data_bytes == 4;
        if (scalar) { s << "    float val_LEAF_" << l << " = LEAF_" << l << "[0];\n"; continue; }
        int off = rn.ndim - lf.ndim;
        s << "    int leaf_idx_" << l << " = 0;\n    {\n        int rem = idx;\n";
        for (int d = 0; d < rn.ndim; ++d) {
            int od = d - off;
            int st = (od >= 0 && lf.shape[od] != 1) ? lf.strides[od] : 0;
            if (st != 0) s << "        leaf_idx_" << l << " += (rem / " << ostr[d] << ") * " << st << ";\n";
            s << "        rem %= " << ostr[d] << ";\n";
        }
        s << "    }\n    float val_LEAF_" << l << " = LEAF_" << l << "[leaf_idx_" << l << "];\n";
    }
    s << "\n";
    for (auto& st : tape) {
        std::string e;
        const std::string& a = st.operands[0];
        const std::string b = st.operands.size() > 1 ? st.operands[1] : "";
        std::string custom;
        if (lowering_for(st.op, &custom)) {
            for (size_t i = 0; i < custom.size(); ++i) {
                if (custom[i] == '$' && i + 1 < custom.size() && (custom[i + 1] == '0' || custom[i + 1] == '1')) { e += (custom[i + 1] == '0' ? a : b); ++i; }
                else e += custom[i];
            }
        } else
        switch (st.op) {   // plain C operators, as in ormi-core/csrc/backend/cuda/lowerings/pointwise.cpp:4-13; -fmad=false keeps them un-fused
            case ORMI_OP_ADD: e = a + " + " + b; break;
            case ORMI_OP_SUB: e = a + " - " + b; break;
            case ORMI_OP_MUL: e = a + " * " + b; break;
            case ORMI_OP_DIV: e = a + " / " + b; break;
            case ORMI_OP_POW: e = "ormi_pow(" + a + ", " + b + ")"; break;
            case ORMI_OP_NEG: e = "-" + a; break;
            case ORMI_OP_EXP: e = "expf(" + a + ")"; break;
            case ORMI_OP_LOG: e = "logf(" + a + ")"; break;
            case ORMI_OP_SIN: e = "sinf(" + a + ")"; break;
            case ORMI_OP_COS: e = "cosf(" + a + ")"; break;
        }
        s << "    float " << st.var << " = " << e << ";\n";
    }
    s << "\n    OUT_Z[idx] = " << root_var << ";\n}\n";
    k.source = s.str();
    return k;
}

}  // namespace ormi_b200
