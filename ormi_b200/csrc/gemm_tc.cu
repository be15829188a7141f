// Host side of the run-time compiled tensor-core GEMM (gemm_tc_template.cuh): tensor maps, kernel variants, launch;
// and the bf16 twins of fp32 buffers that feed it.
//
// Replaces the operand handling of ormi::cuda::matmul (ormi-core/csrc/backend/cuda/kernels/blas/matmul.cu:47-105:
// transposition inferred from the last-dimension stride, three cudaMalloc + memcpy per call) for the "bf16" matmul
// arithmetic: an operand is read in whatever row-major layout it has — a transposed view is simply an MN-major operand
// of tcgen05.mma — so nothing is transposed, padded or copied; the only extra pass is fp32 -> bf16, and that one is
// cached per buffer (weights and inputs that do not change are converted once) or written by the kernel that
// produced the fp32 values in the first place.
#include <cuda_bf16.h>

#include <algorithm>
#include <cstring>

#include "context.h"

namespace ormi_b200 {

namespace {

const char* kTemplate =
#include "gemm_tc_template.cuh"
    ;

constexpr int kMaxSmem = 232448;     // 227 KB: the opt-in limit of dynamic shared memory per block on sm_100

struct Variant { int cta_group, a_mn, b_mn, wpq, bn, tma_store, stages, smem; };

Variant make_variant(int cta_group, int a_mn, int b_mn, int wpq, int bn, int tma_store) {
    Variant v{cta_group, a_mn, b_mn, wpq, bn, tma_store, 0, 0};
    const int stage_bytes = 128 * 64 * 2 + (bn / cta_group) * 64 * 2;
    const int fixed = 1024 /* alignment slack */ + 4 * wpq * 4096 * (tma_store ? 2 : 1) /* staging */ + 64 /* flags, schedule slots */;
    int s = (kMaxSmem - fixed - 8 * 12) / (stage_bytes + 16);
    v.stages = std::min(s, 8);
    v.smem = fixed + v.stages * stage_bytes + 8 * (2 * v.stages + 12);
    return v;
}

KernelStep make_kernel(const Variant& v, const TcEpilogue* epi) {
    std::string src;
    auto def = [&](const std::string& name, const std::string& value) { src += "#define " + name + " " + value + "\n"; };
    // a macro body must sit on one logical line
    auto one_line = [](std::string s) { for (char& c : s) if (c == '\n') c = ' '; return s; };
    def("G_KERNEL_NAME", "ormi_gemm_tc");
    def("G_CTA_GROUP", std::to_string(v.cta_group));
    def("G_A_MN", std::to_string(v.a_mn));
    def("G_B_MN", std::to_string(v.b_mn));
    def("G_EPI_WPQ", std::to_string(v.wpq));
    def("G_BN", std::to_string(v.bn));
    def("G_TMA_STORE", std::to_string(v.tma_store));
    def("G_STAGES", std::to_string(v.stages));
    def("G_EPI_PARAMS", epi ? one_line(epi->params) : "");
    def("G_EPI_INIT", epi ? one_line(epi->init) : "");
    def("G_EPI_COLS", epi ? one_line(epi->cols) : "");
    def("G_EPI_BODY", epi ? one_line(epi->body) : "*reinterpret_cast<float4*>(C + (size_t)grow * N + gcol) = acc;");
    def("G_EPI_PRE", epi ? one_line(epi->pre) : "");
    def("G_EPI_END", epi ? one_line(epi->end) : "");
    def("G_EPI_UNROLL", std::to_string(epi ? epi->unroll : 8));
    if (epi) src += epi->prelude;
    src += kTemplate;
    KernelStep k;
    k.name = "ormi_gemm_tc";
    k.source = src;
    k.key = std::to_string(fnv1a(src));
    k.block = 64 + 32 * 4 * v.wpq;
    k.dyn_smem = v.smem;
    return k;
}

// Tensor map over a bf16 matrix stored [rows][ld] (ld >= cols, both multiples of 8); box = 64 contiguous elements
// (128 bytes, the swizzle span) x box_rows.
// With fp32 = true: a map over an fp32 matrix, box = 32 contiguous elements (the same 128 bytes) x box_rows.
void make_map(ormi_b200_ctx* ctx, CUtensorMap* map, const void* ptr, int rows, int cols, long long ld, int box_rows, bool fp32 = false) {
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * (fp32 ? 4 : 2)};
    cuuint32_t box[2] = {fp32 ? 32u : 64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    ctx->drv.check(ctx->drv.TensorMapEncodeTiled(map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
                   "cuTensorMapEncodeTiled");
}

// dst[r][c] = bf16(src[r * ld + c]); 8 elements per thread and step when the source rows can be read as float4.
__global__ void __launch_bounds__(256)
cvt_bf16_rows(const float* __restrict__ src, long long ld, int rows, int cols, __nv_bfloat16* __restrict__ dst, int vec) {
    const long long groups = (long long)rows * (cols / 8);
    for (long long g = blockIdx.x * 256ll + threadIdx.x; g < groups; g += (long long)gridDim.x * 256) {
        const long long r = g / (cols / 8);
        const int c = (int)(g - r * (cols / 8)) * 8;
        const float* p = src + r * ld + c;
        float v[8];
        if (vec) {
            const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
            #pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = p[i];
        }
        __nv_bfloat162 o[4];
        #pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(dst + r * cols + c) = *reinterpret_cast<const uint4*>(o);
    }
}

}  // namespace

void cvt_bf16(ormi_b200_ctx* ctx, const float* src, long long ld, int rows, int cols, void* dst) {
    if (rows <= 0 || cols <= 0 || cols % 8 != 0 || ld < cols) throw Error("cvt_bf16: cols must be a positive multiple of 8 and ld >= cols");
    if ((uintptr_t)dst & 15) throw Error("cvt_bf16: destination must be 16-byte aligned");
    const int vec = (((uintptr_t)src & 15) == 0 && ld % 4 == 0) ? 1 : 0;
    const long long groups = (long long)rows * (cols / 8);
    const int grid = (int)std::min<long long>((groups + 255) / 256, (long long)ctx->num_sms * 16);
    cvt_bf16_rows<<<grid, 256, 0, ctx->stream>>>(src, ld, rows, cols, (__nv_bfloat16*)dst, vec);
    ORMI_CUDA(cudaGetLastError());
    ctx->counters["launches"]++;
    ctx->counters["cvt_launches"]++;
}

// ------------------------------------------------------------------------------------------------ bf16 twins
// A twin is a contiguous bf16 copy [rows][cols] of the fp32 matrix a matmul reads at `src` (row pitch ld).  It belongs
// to the context, is found again by the fp32 pointer, and lives until that buffer is freed or written through the ABI.
void shadow_drop(ormi_b200_ctx* ctx, const void* ptr, size_t bytes) {
    if (ctx->shadows.empty() || !ptr) return;
    const char* lo = (const char*)ptr;
    const char* hi = lo + std::max<size_t>(bytes, 1);
    for (auto it = ctx->shadows.begin(); it != ctx->shadows.end();) {
        const char* s = (const char*)it->first;
        const char* e = s + it->second.src_bytes;
        if (s < hi && lo < e) {
            void* p = it->second.ptr; size_t n = it->second.bytes;
            it = ctx->shadows.erase(it);
            pool_free(ctx, p, n);          // stream-ordered: a GEMM already queued still reads it safely
        } else ++it;
    }
}

void shadow_register(ormi_b200_ctx* ctx, const void* src, void* p16, int rows, int cols, long long ld) {
    shadow_drop(ctx, src, 1);
    Shadow16 s;
    s.ptr = p16; s.bytes = (size_t)rows * cols * 2; s.rows = rows; s.cols = cols; s.ld = ld;
    s.src_bytes = ((size_t)(rows - 1) * ld + cols) * 4;
    ctx->shadows[src] = s;
}

const void* shadow_find(ormi_b200_ctx* ctx, const void* src, int rows, int cols, long long ld) {
    auto it = ctx->shadows.find(src);
    if (it == ctx->shadows.end()) return nullptr;
    const Shadow16& s = it->second;
    // the same bytes seen as another 2-D shape (a reshape) are the same twin as long as both are contiguous
    const bool same = s.rows == rows && s.cols == cols && s.ld == ld;
    const bool flat = s.ld == s.cols && ld == cols && (long long)s.rows * s.cols == (long long)rows * cols;
    return (same || flat) ? s.ptr : nullptr;
}

const void* shadow_of(ormi_b200_ctx* ctx, const float* src, int rows, int cols, long long ld) {
    if (const void* p = shadow_find(ctx, src, rows, cols, ld)) { ctx->counters["shadow_hits"]++; return p; }
    void* p16 = pool_alloc(ctx, (size_t)rows * cols * 2);
    try { cvt_bf16(ctx, src, ld, rows, cols, p16); }
    catch (...) { pool_free(ctx, p16, (size_t)rows * cols * 2); throw; }
    shadow_register(ctx, src, p16, rows, cols, ld);
    return p16;
}

// ------------------------------------------------------------------------------------------------ launch
bool gemm_tc_supported(const GemmArgs& g) {
    if (g.batch != 1 || (long long)g.M * g.N * g.K < (1ll << 21) || g.K < 64) return false;
    const int a_cols = g.trans_a ? g.M : g.K, b_cols = g.trans_b ? g.K : g.N;
    return a_cols % 8 == 0 && b_cols % 8 == 0 && g.N % 4 == 0 && ((uintptr_t)g.C & 15) == 0;
}

void gemm_tc(ormi_b200_ctx* ctx, const void* a16, int a_mn, const void* b16, int b_mn, float* C, int M, int N, int K,
             const TcEpilogue* epi) {
    if (M <= 0 || N <= 0 || K <= 0) throw Error("gemm_tc: empty problem");
    if ((a_mn ? M : K) % 8 || (b_mn ? N : K) % 8 || N % 4) throw Error("gemm_tc: the contiguous dimension of each bf16 operand must be a multiple of 8 and N a multiple of 4");
    if (((uintptr_t)a16 | (uintptr_t)b16 | (uintptr_t)C) & 15) throw Error("gemm_tc: operands must be 16-byte aligned");
    // A collective running beside the GEMM holds single SMs; a pair needs both SMs of a TPC, so every SM the collective
    // sits on takes its neighbour out of the GEMM too.  While an overlapped all-reduce is in flight: one SM per MMA.
    int cg = (ctx->tc_pair_auto && ctx->comm_inflight > 0) ? 1 : ctx->tc_cta_group;
    // Tile width: 256 columns.  The MMA takes as long for N = 128 as for N = 256 (measured: 128-column tiles halve the
    // throughput of every large shape), so narrow tiles only pay where 256-column tiles would leave more than half of the
    // SMs without one: the drain of an accumulator is bound by the SM's store path (~25 bytes per clock, whatever the
    // number of epilogue warps), and 128 x 128 tiles on single SMs spread it over twice as many SMs as 256 x 256 tiles on pairs.
    int bn = ctx->tune[TUNE_GEMM_BN] ? ctx->tune[TUNE_GEMM_BN] : 256;
    if (bn != 128 && bn != 256) throw Error("tune.gemm_bn must be 128 or 256");
    if (!ctx->tune[TUNE_GEMM_BN] && ((M + 127) / 128) * ((N + 127) / 128) <= ctx->num_sms / 2 + 2) { cg = 1; bn = 128; }
    const int wpq = epi ? epi->wpq : (ctx->tune[TUNE_EPI_WPQ] ? ctx->tune[TUNE_EPI_WPQ] : 1);
    if (wpq != 1 && wpq != 2 && wpq != 4) throw Error("tune.epi_wpq must be 1, 2 or 4");
    // the kernel of this variant: looked up by its few parameters and the epilogue text, not by the whole source
    const int tma_store = epi ? 0 : 1;      // the product itself, nothing else: whole chunks leave through TMA stores
    std::string vkey = std::to_string(cg) + "|" + std::to_string(a_mn) + "|" + std::to_string(b_mn) + "|" + std::to_string(bn) + "|" + std::to_string(wpq) + "|" + std::to_string(tma_store);
    if (epi) vkey += "|" + std::to_string(epi->unroll) + "|" + epi->params + "|" + epi->init + "|" + epi->cols + "|" + epi->pre + "|" + epi->body + "|" + epi->end;
    auto found = ctx->tc_kernels.find(vkey);
    if (found == ctx->tc_kernels.end()) {
        const Variant v = make_variant(cg, a_mn, b_mn, wpq, bn, tma_store);
        const KernelStep made = make_kernel(v, epi);
        TcKernel tk;
        tk.kernel = get_kernel(ctx, made);
        tk.block = made.block; tk.smem = made.dyn_smem;
        found = ctx->tc_kernels.emplace(vkey, tk).first;
    }
    CompiledKernel* k = found->second.kernel;
    struct { int block, dyn_smem; } ks{found->second.block, found->second.smem};
    CUtensorMap map_a, map_b, map_c;
    if (a_mn) make_map(ctx, &map_a, a16, K, M, M, 64);            // stored [K][M]
    else make_map(ctx, &map_a, a16, M, K, K, 128);                // stored [M][K]
    if (b_mn) make_map(ctx, &map_b, b16, K, N, N, 64);            // stored [K][N]
    else make_map(ctx, &map_b, b16, N, K, K, bn / cg);            // stored [N][K]
    int* err = device_error_word(ctx);
    int* counter = err + kTileCounterWord;
    int tiles_m = (M + 128 * cg - 1) / (128 * cg), tiles_n = (N + bn - 1) / bn, num_kb = (K + 63) / 64;
    const int grid = cg * std::min(tiles_m * tiles_n, ctx->num_sms / cg);
    std::vector<void*> argv = {&map_a, &map_b, &C, &M, &N, &num_kb, &tiles_m, &tiles_n, &err, &counter};
    if (tma_store) { make_map(ctx, &map_c, C, M, N, N, 32, true); argv.push_back(&map_c); }
    std::vector<void*> extra;
    if (epi) { extra = epi->args; for (auto& p : extra) argv.push_back(&p); }
    ctx->drv.check(ctx->drv.LaunchKernel(k->func, (unsigned)grid, 1, 1, (unsigned)ks.block, 1, 1, (unsigned)ks.dyn_smem, (CUstream)ctx->stream,
                                         argv.data(), nullptr), "cuLaunchKernel (tensor-core GEMM)");
    ctx->gemm_err_pending = true;
    ctx->counters["gemm_launches"]++;
    ctx->counters["launches"]++;
}

// The matmul of a plan in "bf16" arithmetic: fp32 operands as the graph has them, bf16 twins looked up or made here.
void gemm_tc_from_fp32(ormi_b200_ctx* ctx, const GemmArgs& g, const void* a16, const void* b16, const TcEpilogue* epi) {
    // A(m,k) = A[m*lda + k], or A[k*lda + m] when stored transposed; B(k,n) = B[k*ldb + n], or B[n*ldb + k]
    const int a_rows = g.trans_a ? g.K : g.M, a_cols = g.trans_a ? g.M : g.K;
    const int b_rows = g.trans_b ? g.N : g.K, b_cols = g.trans_b ? g.K : g.N;
    if (!a16) a16 = shadow_of(ctx, g.A, a_rows, a_cols, g.lda);
    if (!b16) b16 = shadow_of(ctx, g.B, b_rows, b_cols, g.ldb);
    gemm_tc(ctx, a16, g.trans_a ? 1 : 0, b16, g.trans_b ? 0 : 1, g.C, g.M, g.N, g.K, epi);
}

}  // namespace ormi_b200
