// Context, buffer pool, kernel cache and plan executor of the B200 backend.
//
// Replaces, from the reference CUDA backend:
//   CUDAAllocator            ormi-core/csrc/backend/cuda/allocator.cu:11-105   (pool, copies, fills)
//   compile_ptx              ormi-core/csrc/backend/cuda/utils.cu:6-27         (NVRTC; here straight to an sm_100a cubin)
//   execute_jit              ormi-core/csrc/backend/cuda/jit.cu:13-44          (module load + launch; here cached and on a stream)
// Differences by design: the device is bound once, every launch and copy goes to one non-blocking stream
// (the reference uses the legacy default stream and re-initialises the driver on every call), compiled
// kernels are cached by source hash and whole schedules by graph structure, so a training loop that
// rebuilds the same graph every step pays for scheduling, code generation and NVRTC once.
#include <algorithm>
#include <map>
#include <nvrtc.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <sys/stat.h>
#include <unistd.h>

#include "context.h"

namespace ormi_b200 {

// ------------------------------------------------------------------------------------------------ driver
void DriverApi::load() {
    auto get = [](const char* name, void** fn) {
        cudaDriverEntryPointQueryResult st;
        cudaError_t e = cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &st);
        if (e != cudaSuccess || st != cudaDriverEntryPointSuccess || !*fn)
            throw Error(std::string("CUDA Error: driver entry point not found: ") + name);
    };
    get("cuModuleLoadData", (void**)&ModuleLoadData);
    get("cuModuleUnload", (void**)&ModuleUnload);
    get("cuModuleGetFunction", (void**)&ModuleGetFunction);
    get("cuLaunchKernel", (void**)&LaunchKernel);
    get("cuGetErrorString", (void**)&GetErrorString);
    get("cuFuncSetAttribute", (void**)&FuncSetAttribute);
    get("cuTensorMapEncodeTiled", (void**)&TensorMapEncodeTiled);
}

void DriverApi::check(CUresult r, const char* what) const {
    if (r == CUDA_SUCCESS) return;
    const char* msg = nullptr;
    if (GetErrorString) GetErrorString(r, &msg);
    throw Error(std::string("CUDA Error: ") + (msg ? msg : "unknown") + " (" + what + ")");
}

// ------------------------------------------------------------------------------------------------ pool
// Debug option "pool_canary": every block gets kCanaryBytes more than was asked for, filled with a pattern; when the block
// comes back the pattern is read (a synchronous copy: slow, a debugging aid) and an overwritten zone is reported with the
// block's size — a kernel that wrote past the end of its output.  The pool is keyed by the real size.
constexpr size_t kCanaryBytes = 256;
constexpr int kCanaryByte = 0xA5;

void* pool_alloc(ormi_b200_ctx* ctx, size_t asked) {
    if (asked == 0) asked = 4;
    const bool canary = ctx->pool_canary;
    const size_t bytes = asked + (canary ? kCanaryBytes : 0);
    void* p = nullptr;
    {
        std::lock_guard<std::mutex> lock(ctx->pool_mutex);
        auto it = ctx->free_blocks.find(bytes);
        if (it != ctx->free_blocks.end() && !it->second.empty()) {
            p = it->second.back();
            it->second.pop_back();
            ctx->pooled.erase(p);
            ctx->counters["pool_hits"]++;
        }
    }
    if (!p && ctx->capturing)
        throw Error("capture: the pool holds no free block of " + std::to_string(bytes) + " bytes (run the step once before capturing it: nothing may be taken from the driver while a step is captured)");
    if (!p) {
        auto over_limit = [&]() { return ctx->pool_limit_bytes > 0 && ctx->pool_held_bytes + (long long)bytes > ctx->pool_limit_bytes; };
        cudaError_t e = over_limit() ? cudaErrorMemoryAllocation : cudaMalloc(&p, bytes);
        if (e == cudaErrorMemoryAllocation) {   // give cached blocks back and try once more
            cudaGetLastError();
            {
                std::lock_guard<std::mutex> lock(ctx->pool_mutex);
                cudaStreamSynchronize(ctx->stream);
                for (auto& kv : ctx->free_blocks) for (void* q : kv.second) { cudaFree(q); ctx->pool_held_bytes -= (long long)kv.first; }
                ctx->free_blocks.clear();
                ctx->pooled.clear();
                ctx->counters["pool_trims"]++;
            }
            e = over_limit() ? cudaErrorMemoryAllocation : cudaMalloc(&p, bytes);
        }
        if (e != cudaSuccess) throw Error(std::string("CUDA Error: ") + cudaGetErrorString(e) + " (allocating " + std::to_string(bytes) + " bytes)");
        ctx->counters["bytes_allocated"] += (int64_t)bytes;
        ctx->pool_held_bytes += (long long)bytes;
    }
    if (ctx->capturing) { std::lock_guard<std::mutex> lock(ctx->pool_mutex); ctx->capture_blocks[p] = bytes; }
    if (canary) {
        const cudaError_t e = cudaMemsetAsync((char*)p + asked, kCanaryByte, kCanaryBytes, ctx->stream);
        if (e != cudaSuccess) { pool_free(ctx, p, bytes); throw Error(std::string("CUDA Error: ") + cudaGetErrorString(e) + " (filling a guard zone)"); }
        std::lock_guard<std::mutex> lock(ctx->pool_mutex);
        ctx->canaries[p] = asked;
    }
    return p;
}

void pool_free(ormi_b200_ctx* ctx, void* ptr, size_t bytes) {
    if (!ptr) return;
    if (bytes == 0) bytes = 4;
    {   // a block that a captured step reads or writes on every replay stays with that graph until the graph is destroyed
        std::lock_guard<std::mutex> lock(ctx->pool_mutex);
        if (ctx->graph_owned.count(ptr)) return;
    }
    shadow_drop(ctx, ptr, bytes);      // a bf16 twin of this buffer goes back to the pool with it
    bool guarded_block = false;
    {
        std::lock_guard<std::mutex> lock(ctx->pool_mutex);
        auto it = ctx->canaries.find(ptr);
        if (it != ctx->canaries.end()) { guarded_block = true; bytes = it->second; ctx->canaries.erase(it); }
    }
    std::string damage;
    if (guarded_block) {
        unsigned char zone[kCanaryBytes];
        cudaError_t e = cudaMemcpyAsync(zone, (const char*)ptr + bytes, kCanaryBytes, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) damage = std::string("CUDA Error: ") + cudaGetErrorString(e) + " (reading a guard zone)";
        else for (size_t i = 0; i < kCanaryBytes; ++i)
            if (zone[i] != kCanaryByte) { damage = "guard zone behind a " + std::to_string(bytes) + "-byte block overwritten at byte +" + std::to_string(i); break; }
        bytes += kCanaryBytes;
    }
    {
        std::lock_guard<std::mutex> lock(ctx->pool_mutex);
        if (!ctx->pooled.insert(ptr).second) throw Error("internal: a pool block was returned twice (" + std::to_string(bytes) + " bytes)");
        ctx->free_blocks[bytes].push_back(ptr);
    }
    if (!damage.empty()) { ctx->counters["canary_hits"]++; throw Error(damage); }
}

// ------------------------------------------------------------------------------------------------ NVRTC
std::vector<char> compile_cubin(const std::string& source, std::string* log_out) {
    nvrtcProgram prog;
    if (nvrtcCreateProgram(&prog, source.c_str(), "ormi_fused.cu", 0, nullptr, nullptr) != NVRTC_SUCCESS)
        throw Error("NVRTC Error: cannot create program");
    // ORMI_B200_NVRTC_LOG=1 adds ptxas -v (registers, spills, shared memory) and prints the compiler log
    const bool verbose = std::getenv("ORMI_B200_NVRTC_LOG") != nullptr;
    const char* opts[] = {"--gpu-architecture=sm_100a", "--fmad=false", "--std=c++17", "-default-device", "--ptxas-options=-v"};
    nvrtcResult r = nvrtcCompileProgram(prog, verbose ? 5 : 4, opts);
    size_t log_size = 0;
    nvrtcGetProgramLogSize(prog, &log_size);
    std::string log(log_size, '\0');
    if (log_size > 1) nvrtcGetProgramLog(prog, &log[0]);
    if (log_out) *log_out = log;
    if (verbose && log_size > 1) fprintf(stderr, "%s\n", log.c_str());
    if (r != NVRTC_SUCCESS) {
        nvrtcDestroyProgram(&prog);
        throw Error("NVRTC Compilation failed: \n" + log);
    }
    size_t size = 0;
    if (nvrtcGetCUBINSize(prog, &size) != NVRTC_SUCCESS || size == 0) { nvrtcDestroyProgram(&prog); throw Error("NVRTC Error: no cubin produced"); }
    std::vector<char> cubin(size);
    nvrtcGetCUBIN(prog, cubin.data());
    nvrtcDestroyProgram(&prog);
    return cubin;
}

// On-disk cache of compiled kernels, so that a new process does not pay NVRTC (some 0.3-1 s per generated kernel) for
// sources an earlier process already compiled.  Directory: $ORMI_B200_CACHE_DIR ("off" disables the cache), else
// $XDG_CACHE_HOME/ormi_b200, else $HOME/.cache/ormi_b200.  A file is named after two independent hashes of the source,
// its length and the compiler version; it is written to a temporary name and renamed, so readers never see half a file.
static std::string cubin_cache_dir() {
    const char* d = std::getenv("ORMI_B200_CACHE_DIR");
    if (d) return std::string(d) == "off" ? std::string() : std::string(d);
    if (const char* x = std::getenv("XDG_CACHE_HOME")) return std::string(x) + "/ormi_b200";
    if (const char* h = std::getenv("HOME")) return std::string(h) + "/.cache/ormi_b200";
    return std::string();
}

static std::string cubin_cache_path(const std::string& source) {
    const std::string dir = cubin_cache_dir();
    if (dir.empty()) return dir;
    uint64_t h2 = 0x9e3779b97f4a7c15ull;                       // a second, different mix of the same bytes
    for (unsigned char c : source) { h2 = (h2 ^ c) * 0x100000001b3ull; h2 ^= h2 >> 29; }
    int major = 0, minor = 0;
    nvrtcVersion(&major, &minor);
    char name[160];
    snprintf(name, sizeof name, "/k_%016llx_%016llx_%zu_nvrtc%d.%d_sm100a_v1.cubin", (unsigned long long)fnv1a(source),
             (unsigned long long)h2, source.size(), major, minor);
    return dir + name;
}

static bool read_file(const std::string& path, std::vector<char>& out) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return false;
    fseek(f, 0, SEEK_END);
    long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    bool ok = n > 0;
    if (ok) { out.resize((size_t)n); ok = fread(out.data(), 1, (size_t)n, f) == (size_t)n; }
    fclose(f);
    return ok;
}

static void write_file_atomically(const std::string& path, const std::vector<char>& data) {
    const std::string dir = path.substr(0, path.rfind('/'));
    for (size_t i = 1; i <= dir.size(); ++i)                    // mkdir -p
        if (i == dir.size() || dir[i] == '/') mkdir(dir.substr(0, i).c_str(), 0755);
    const std::string tmp = path + ".tmp" + std::to_string((long long)getpid());
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) return;                                            // the cache is best effort: a read-only home is not an error
    const bool ok = fwrite(data.data(), 1, data.size(), f) == data.size();
    fclose(f);
    if (!ok || rename(tmp.c_str(), path.c_str()) != 0) remove(tmp.c_str());
}

CompiledKernel* get_kernel(ormi_b200_ctx* ctx, const KernelStep& k) {
    auto it = ctx->kernel_cache.find(k.key + ":" + k.name);
    if (it != ctx->kernel_cache.end()) { ctx->counters["kernel_cache_hits"]++; return &it->second; }
    std::vector<char> cubin;
    const std::string disk = std::getenv("ORMI_B200_NVRTC_LOG") ? std::string() : cubin_cache_path(k.source);
    if (!disk.empty() && read_file(disk, cubin)) ctx->counters["cubin_disk_hits"]++;
    else {
        cubin = compile_cubin(k.source);
        ctx->counters["nvrtc_compiles"]++;
        if (!disk.empty()) write_file_atomically(disk, cubin);
    }
    CompiledKernel ck;
    if (ctx->drv.ModuleLoadData(&ck.module, cubin.data()) != CUDA_SUCCESS) {
        // a file from the disk cache that the driver does not take (another driver, a damaged file): compile afresh
        cubin = compile_cubin(k.source);
        ctx->counters["nvrtc_compiles"]++;
        if (!disk.empty()) write_file_atomically(disk, cubin);
        ctx->drv.check(ctx->drv.ModuleLoadData(&ck.module, cubin.data()), "cuModuleLoadData");
    }
    ctx->drv.check(ctx->drv.ModuleGetFunction(&ck.func, ck.module, k.name.c_str()), "cuModuleGetFunction");
    if (k.dyn_smem > 0)     // static shared memory counts against the 48 KB default too: always raise the limit
        ctx->drv.check(ctx->drv.FuncSetAttribute(ck.func, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, k.dyn_smem), "cuFuncSetAttribute");
    ctx->counters["kernels_compiled"]++;
    auto res = ctx->kernel_cache.emplace(k.key + ":" + k.name, ck);
    return &res.first->second;
}

void launch_kernel(ormi_b200_ctx* ctx, CompiledKernel* k, int grid, int block, std::vector<void*>& pointer_args, int dyn_smem) {
    std::vector<void*> argv(pointer_args.size());
    for (size_t i = 0; i < pointer_args.size(); ++i) argv[i] = &pointer_args[i];
    ctx->drv.check(ctx->drv.LaunchKernel(k->func, (unsigned)grid, 1, 1, (unsigned)block, 1, 1, (unsigned)dyn_smem, (CUstream)ctx->stream, argv.data(), nullptr),
                   "cuLaunchKernel");
    ctx->counters["launches"]++;
}

// The device word into which kernels with bounded waits (staged row kernels, the tensor-core GEMM) report a wait
// that ran out.  Read back at host-visible boundaries by check_gemm_error.
int* device_error_word(ormi_b200_ctx* ctx) {
    if (!ctx->gemm_err) {
        ORMI_CUDA(cudaMalloc(&ctx->gemm_err, kErrorWords * sizeof(int)));
        ORMI_CUDA(cudaMemsetAsync(ctx->gemm_err, 0, kErrorWords * sizeof(int), ctx->stream));
    }
    return ctx->gemm_err;
}

// ------------------------------------------------------------------------------------------------ realize
// Everything a schedule depends on, as a string of words: the options, and per node the fields the scheduler reads.
// Two calls share a cached plan when their keys are EQUAL (the map is keyed by the text, not by a hash of it).
static std::string graph_key(const ormi_b200_ctx* ctx, const ormi_b200_node* nodes, int n, const int* roots, int n_roots, bool aligned) {
    std::string key;
    key.reserve((size_t)n * 48 + 64);
    auto mix = [&](uint64_t v) { const uint32_t w = (uint32_t)v; key.append(reinterpret_cast<const char*>(&w), 4); };
    mix((uint64_t)n); mix((ctx->fusion ? 1 : 0) | (ctx->free_intermediates ? 2 : 0)); mix((uint64_t)ctx->matmul_mode); mix(aligned ? 1 : 0); mix((uint64_t)ctx->tc_cta_group);
    for (int v : ctx->tune) mix((uint64_t)(uint32_t)v);
    mix(lowering_generation());
    for (int i = 0; i < n; ++i) {
        const auto& nd = nodes[i];
        mix((uint64_t)nd.op); mix((uint64_t)nd.n_parents);
        for (int p = 0; p < nd.n_parents; ++p) mix((uint64_t)nd.parents[p]);
        mix((uint64_t)nd.ndim);
        for (int d = 0; d < nd.ndim; ++d) { mix((uint64_t)(uint32_t)nd.shape[d]); mix((uint64_t)(uint32_t)nd.strides[d]); }
        mix((uint64_t)nd.n_axes);
        for (int a = 0; a < nd.n_axes; ++a) mix((uint64_t)nd.axes[a]);
        mix((uint64_t)nd.keepdims); mix((uint64_t)(nd.flags & (ORMI_NODE_KEEP | ORMI_NODE_TWIN16 | ORMI_NODE_BF16)));
        mix(nd.data ? (nd.data_bytes == 4 ? 2 : 1) : 0);
    }
    mix(0xffffffffu);
    for (int r = 0; r < n_roots; ++r) mix((uint64_t)roots[r]);
    return key;
}

CachedPlan::~CachedPlan() { for (auto& g : graphs) if (g.exec) cudaGraphExecDestroy((cudaGraphExec_t)g.exec); }

void realize(ormi_b200_ctx* ctx, ormi_b200_node* nodes, int n_nodes, const int* roots, int n_roots,
             const std::vector<std::pair<int, void*>>* preassigned) {
    ORMI_CUDA(cudaSetDevice(ctx->device));
    // 128-bit loads, bulk copies and TMA need 16-byte aligned buffers.  Pool blocks are; a caller's own pointer may
    // not be, and then the whole plan is generated with scalar accesses (the bit is part of the plan key).
    bool aligned = true;
    for (int i = 0; i < n_nodes; ++i) if (nodes[i].data && ((uintptr_t)nodes[i].data & 15)) aligned = false;
    if (preassigned) for (auto& pr : *preassigned) if ((uintptr_t)pr.second & 15) aligned = false;
    const std::string key = graph_key(ctx, nodes, n_nodes, roots, n_roots, aligned);
    CachedPlan* cp = nullptr;
    auto it = ctx->plan_cache.find(key);
    if (it != ctx->plan_cache.end()) { cp = it->second.get(); ctx->counters["plan_cache_hits"]++; }
    else {
        SchedOptions opt;
        opt.num_sms = ctx->num_sms;
        opt.fusion = ctx->fusion;
        opt.free_intermediates = ctx->free_intermediates;
        opt.bf16_matmul = ctx->matmul_mode == MatmulMode::BF16;
        opt.aligned = aligned;
        std::copy(std::begin(ctx->tune), std::end(ctx->tune), opt.tune);
        auto fresh = std::make_unique<CachedPlan>();
        fresh->plan = build_plan(nodes, n_nodes, roots, n_roots, opt);
        if (!fresh->plan.error.empty()) throw Error(fresh->plan.error);
        for (const Step& s : fresh->plan.steps) fresh->kernels.push_back(s.type == Step::Kernel ? get_kernel(ctx, s.k) : nullptr);
        // Scratch buffers live from their first to their last step only: they are taken from the pool right before
        // the one and go back right after the other (the pool is ordered by the stream, so a later step of the same
        // realize call may get the same block), instead of all being held for the whole call.
        const Plan& p = fresh->plan;
        fresh->first_use.assign(p.buffers.size(), -1);
        fresh->last_use.assign(p.buffers.size(), -1);
        for (size_t si = 0; si < p.steps.size(); ++si) {
            const Step& s = p.steps[si];
            std::vector<int> used = s.type == Step::Kernel ? s.k.args : std::vector<int>{s.g.a, s.g.b, s.g.c, s.g.a16, s.g.b16};
            if (s.type == Step::Gemm) used.insert(used.end(), s.g.epi_args.begin(), s.g.epi_args.end());
            for (int b : used) {
                if (b < 0 || p.buffers[b].kind == BufKind::External || p.buffers[b].kind == BufKind::ErrorWord) continue;
                if (fresh->first_use[b] < 0) fresh->first_use[b] = (int)si;
                fresh->last_use[b] = (int)si;
            }
        }
        // what is handed out is taken from the pool as late as scratch is (a block that scratch gave back may serve it),
        // but never goes back
        for (size_t b = 0; b < p.buffers.size(); ++b) if (p.buffers[b].kind == BufKind::NodeOut) fresh->last_use[b] = -1;
        for (const NodeResult& r : p.results) fresh->last_use[r.buffer] = -1;
        // the bf16 twin of a node that is handed out stays with the context (later calls find it by the fp32 pointer)
        fresh->twin_result.assign(p.buffers.size(), -1);
        for (size_t b = 0; b < p.buffers.size(); ++b) {
            if (p.buffers[b].kind != BufKind::Twin16) continue;
            for (const NodeResult& r : p.results)
                // (a node handed out as bf16 ONLY is its twin: that result's buffer is b itself, and registering a buffer as
                // its own twin would make freeing it free it twice)
                if (!r.alias && !r.bf16 && r.node == p.buffers[b].node) { fresh->twin_result[b] = r.buffer; fresh->last_use[b] = -1; }
        }
        cp = fresh.get();
        ctx->plan_cache[key] = std::move(fresh);
    }
    const Plan& plan = cp->plan;
    std::vector<void*> bufs(plan.buffers.size(), nullptr);
    std::vector<bool> handed(plan.buffers.size(), false);
    try {
        for (size_t b = 0; b < plan.buffers.size(); ++b) {
            const PlanBuffer& pb = plan.buffers[b];
            if (pb.kind == BufKind::External) {
                bufs[b] = nodes[pb.node].data;
                if (!bufs[b]) throw Error("internal: realized input without a buffer");
            } else if (pb.kind == BufKind::ErrorWord) {
                bufs[b] = device_error_word(ctx);
                handed[b] = true;      // not a pool block
            } else {
                if (preassigned && pb.kind == BufKind::NodeOut)
                    for (auto& pr : *preassigned) if (pr.first == pb.node) { bufs[b] = pr.second; handed[b] = true; }
                if (!bufs[b] && cp->first_use[b] < 0) bufs[b] = pool_alloc(ctx, (size_t)pb.bytes);   // scratch comes later
            }
        }
        // Pass 1, the pool only: every buffer gets its block in the order the steps need them — scratch is taken right
        // before its first step and goes back right after its last one, so a later step of this call may get the same
        // block (the stream orders the kernels that use it).  `at[s]` is what step s sees.
        // Scratch that a step gives back can serve a later step of this call, but it returns to the pool itself only
        // when every launch of the call has been queued: something that takes a block from the pool while the launches
        // are being queued (a bf16 copy of an operand, say) must not get one that a kernel not yet queued will write.
        const size_t nb = plan.buffers.size();
        std::vector<void*> at(plan.steps.size() * nb, nullptr);
        struct Returned {
            ormi_b200_ctx* ctx;
            std::multimap<size_t, void*> blocks;
            // every block goes back; the first complaint of the pool (an overwritten guard zone) is reported afterwards
            void release(bool report) {
                std::string first;
                for (auto& kv : blocks) { try { pool_free(ctx, kv.second, kv.first); } catch (const std::exception& e) { if (first.empty()) first = e.what(); } }
                blocks.clear();
                if (report && !first.empty()) throw Error(first);
            }
            ~Returned() { release(false); }          // the call is failing for another reason
        } returned{ctx, {}};
        for (size_t s = 0; s < plan.steps.size(); ++s) {
            for (size_t b = 0; b < nb; ++b) {
                if (cp->first_use[b] != (int)s || bufs[b]) continue;
                auto again = returned.blocks.find((size_t)plan.buffers[b].bytes);
                if (again != returned.blocks.end()) { bufs[b] = again->second; returned.blocks.erase(again); }
                else bufs[b] = pool_alloc(ctx, (size_t)plan.buffers[b].bytes);
            }
            std::copy(bufs.begin(), bufs.end(), at.begin() + s * nb);
            for (size_t b = 0; b < nb; ++b)
                if (cp->last_use[b] == (int)s && bufs[b]) { returned.blocks.insert({(size_t)plan.buffers[b].bytes, bufs[b]}); bufs[b] = nullptr; handed[b] = true; }
        }
        // Pass 2, the launches.  A plan of several launches whose buffers come out at the same addresses as in an
        // earlier call (a loop in its steady state: the pool hands the same blocks out in the same order) is replayed
        // as a CUDA graph recorded at the second such call: one submission instead of one per kernel, and no gaps
        // between the kernels.  The graph holds nothing but launches and their arguments: the blocks are owned as ever.
        auto launch_steps = [&]() {
            for (size_t s = 0; s < plan.steps.size(); ++s) {
                const Step& st = plan.steps[s];
                void* const* bp = at.data() + s * nb;
                if (st.type == Step::Kernel) {
                    std::vector<void*> args;
                    for (int a : st.k.args) args.push_back(bp[a]);
                    launch_kernel(ctx, cp->kernels[s], st.k.grid, st.k.block, args, st.k.dyn_smem);
                    if (st.k.err_arg) ctx->gemm_err_pending = true;
                } else {
                    GemmArgs g;
                    g.A = (const float*)bp[st.g.a]; g.B = (const float*)bp[st.g.b]; g.C = (float*)bp[st.g.c];
                    g.M = st.g.M; g.N = st.g.N; g.K = st.g.K;
                    g.trans_a = st.g.trans_a; g.trans_b = st.g.trans_b; g.lda = st.g.lda; g.ldb = st.g.ldb;
                    g.batch = st.g.batch; g.nbatch = st.g.nbatch;
                    std::memcpy(g.bshape, st.g.bshape, sizeof g.bshape);
                    std::memcpy(g.astride, st.g.astride, sizeof g.astride);
                    std::memcpy(g.bstride, st.g.bstride, sizeof g.bstride);
                    if (st.g.tc) {
                        TcEpilogue epi;
                        if (st.g.has_epi) {
                            epi.prelude = st.g.epi_prelude; epi.params = st.g.epi_params; epi.init = st.g.epi_init;
                            epi.cols = st.g.epi_cols; epi.pre = st.g.epi_pre; epi.body = st.g.epi_body; epi.end = st.g.epi_end; epi.wpq = st.g.epi_wpq; epi.unroll = st.g.epi_unroll;
                            for (int a : st.g.epi_args) epi.args.push_back(bp[a]);
                        }
                        gemm_tc_from_fp32(ctx, g, st.g.a16 >= 0 ? bp[st.g.a16] : nullptr, st.g.b16 >= 0 ? bp[st.g.b16] : nullptr,
                                          st.g.has_epi ? &epi : nullptr);
                    } else gemm_dispatch(ctx, g);
                }
            }
        };
        bool replayable = ctx->auto_graph && !ctx->capturing && !ctx->pool_canary && plan.steps.size() >= 2;
        for (const Step& st : plan.steps)
            if (st.type != Step::Kernel && (st.g.tc || ctx->matmul_mode != MatmulMode::FP32)) replayable = false;   // those matmuls look up or make operand copies as they go
        if (!replayable) launch_steps();
        else {
            StepGraph* hit = nullptr;
            for (auto& sg : cp->graphs) if (sg.at == at) hit = &sg;
            if (hit) {
                ORMI_CUDA(cudaGraphLaunch((cudaGraphExec_t)hit->exec, ctx->stream));
                hit->stamp = ++cp->graph_clock;
                ctx->counters["launches"] += hit->launches;
                ctx->counters["graph_replays"]++;
                for (const Step& st : plan.steps) if (st.type == Step::Kernel && st.k.err_arg) ctx->gemm_err_pending = true;
            } else if (std::find(cp->seen.begin(), cp->seen.end(), at) == cp->seen.end()) {
                launch_steps();                                  // first sighting of these addresses: remember them
                if (cp->seen.size() >= 32) cp->seen.erase(cp->seen.begin());
                cp->seen.push_back(at);
            } else {
                // second sighting: record the launches and run them as a graph from now on
                const int64_t before = ctx->counters["launches"];
                cudaGraph_t graph = nullptr;
                ORMI_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
                try { launch_steps(); }
                catch (...) { cudaStreamEndCapture(ctx->stream, &graph); if (graph) cudaGraphDestroy(graph); cudaGetLastError(); throw; }
                ORMI_CUDA(cudaStreamEndCapture(ctx->stream, &graph));
                cudaGraphExec_t exec = nullptr;
                const cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
                cudaGraphDestroy(graph);
                if (e != cudaSuccess) throw Error(std::string("CUDA Error: ") + cudaGetErrorString(e) + " (instantiating a step graph)");
                if (cp->graphs.size() >= 32) {                   // keep the 32 most recently used address sets
                    size_t oldest = 0;
                    for (size_t i = 1; i < cp->graphs.size(); ++i) if (cp->graphs[i].stamp < cp->graphs[oldest].stamp) oldest = i;
                    cudaGraphExecDestroy((cudaGraphExec_t)cp->graphs[oldest].exec);
                    cp->graphs.erase(cp->graphs.begin() + oldest);
                }
                StepGraph sg;
                sg.at = at; sg.exec = exec; sg.launches = (int)(ctx->counters["launches"] - before); sg.stamp = ++cp->graph_clock;
                cp->graphs.push_back(std::move(sg));
                cp->seen.erase(std::find(cp->seen.begin(), cp->seen.end(), at));
                ORMI_CUDA(cudaGraphLaunch(exec, ctx->stream));
                ctx->counters["graphs_recorded"]++;
            }
        }
        returned.release(true);
    } catch (...) {
        for (size_t b = 0; b < plan.buffers.size(); ++b)
            if (plan.buffers[b].kind != BufKind::External && bufs[b] && !handed[b]) pool_free(ctx, bufs[b], (size_t)plan.buffers[b].bytes);
        throw;
    }
    for (const NodeResult& r : plan.results) {
        ormi_b200_node& nd = nodes[r.node];
        nd.data = bufs[r.buffer];
        nd.data_bytes = plan.buffers[r.buffer].bytes;
        if (r.bf16) nd.flags |= ORMI_NODE_BF16; else nd.flags &= ~ORMI_NODE_BF16;
        if (r.alias) nd.flags |= ORMI_NODE_ALIAS;
        else if (handed[r.buffer]) nd.flags |= ORMI_NODE_ALIAS;   // caller-owned target
        else { nd.flags |= ORMI_NODE_OWNED; handed[r.buffer] = true; }
    }
    for (size_t b = 0; b < plan.buffers.size(); ++b) {
        if (plan.buffers[b].kind == BufKind::Twin16 && cp->twin_result[b] >= 0 && bufs[b]) {
            shadow_register(ctx, bufs[cp->twin_result[b]], bufs[b], plan.buffers[b].rows, plan.buffers[b].cols, plan.buffers[b].cols);
            handed[b] = true;
        }
    }
    for (size_t b = 0; b < plan.buffers.size(); ++b)
        if (plan.buffers[b].kind != BufKind::External && !handed[b]) pool_free(ctx, bufs[b], (size_t)plan.buffers[b].bytes);
}

}  // namespace ormi_b200
