// fp32 SIMT GEMM (FFMA pipe) — the default matmul arithmetic, kept in true fp32 so results stay within
// 1e-5 of the reference CPU backend's cblas_sgemm.
//
// Replaces the cublasSgemmBatched call of ormi::cuda::matmul
// (ormi-core/csrc/backend/cuda/kernels/blas/matmul.cu:81-109) together with its three cudaMalloc /
// cudaMemcpy / cudaFree of per-call pointer arrays: batch offsets are computed inside the kernel from
// the broadcast strides, and transposition (operand stored with a last-dimension stride != 1,
// matmul.cu:47-52) is a template parameter of the global->shared copy.
//
// Tiling: 128x128 output tile per 256-thread block, K sliced by 16, each thread an 8x8 register tile
// (two 4-wide strips per axis so shared-memory reads are 128-bit and conflict-free).
// Accumulation over k is in ascending order inside a thread: deterministic, no split-K, no atomics.
// Two kernels with identical arithmetic:
//   sgemm_pipe_kernel  operands whose rows move in 16-byte pieces: cp.async into a 4-stage ring, one barrier per
//                      slice, packed fma.rn.f32x2 on pairs of accumulators;
//   sgemm_kernel       everything else (odd leading dimensions, unaligned views): scalar loads staged through
//                      registers into double-buffered shared memory.
#include "context.h"

namespace ormi_b200 {

namespace {

constexpr int BM = 128, BN = 128, BK = 16, NTHREADS = 256;

struct BatchMap {
    int nbatch;
    int32_t bshape[ORMI_B200_MAX_DIMS];
    long long astride[ORMI_B200_MAX_DIMS];
    long long bstride[ORMI_B200_MAX_DIMS];
};

// A element (m, k) lives at A[m * a_sm + k * a_sk]; B element (k, n) at B[k * b_sk + n * b_sn].
template <bool A_KMAJOR, bool B_NMAJOR, bool VEC>
__global__ void __launch_bounds__(NTHREADS)
sgemm_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
             int M, int N, int K, int lda, int ldb, BatchMap bm) {
    __shared__ __align__(16) float As[2][BK][BM];
    __shared__ __align__(16) float Bs[2][BK][BN];

    {   // batch offsets with broadcast (stride 0)
        int b = blockIdx.z;
        long long oa = 0, ob = 0;
        for (int d = bm.nbatch - 1; d >= 0; --d) {
            int c = b % bm.bshape[d];
            b /= bm.bshape[d];
            oa += c * bm.astride[d];
            ob += c * bm.bstride[d];
        }
        A += oa; B += ob;
        C += (long long)blockIdx.z * M * N;
    }
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;

    float acc[8][8];
    #pragma unroll
    for (int i = 0; i < 8; ++i)
        #pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    // global -> register staging: each thread moves 2 x 4 floats of A and of B per slice
    float ra[2][4], rb[2][4];

    auto load_a = [&](int k0) {
        #pragma unroll
        for (int it = 0; it < 2; ++it) {
            int v = tid + it * NTHREADS;            // 0..511 vectors of 4
            if (A_KMAJOR) {                          // 4 consecutive k of one row m
                int m = v / (BK / 4), kq = (v % (BK / 4)) * 4;
                int gm = m0 + m, gk = k0 + kq;
                if (VEC && gm < M && gk + 3 < K) {
                    float4 t = *reinterpret_cast<const float4*>(A + (long long)gm * lda + gk);
                    ra[it][0] = t.x; ra[it][1] = t.y; ra[it][2] = t.z; ra[it][3] = t.w;
                } else {
                    #pragma unroll
                    for (int e = 0; e < 4; ++e) ra[it][e] = (gm < M && gk + e < K) ? A[(long long)gm * lda + gk + e] : 0.0f;
                }
            } else {                                 // 4 consecutive m of one k
                int k = v / (BM / 4), mq = (v % (BM / 4)) * 4;
                int gk = k0 + k, gm = m0 + mq;
                if (VEC && gk < K && gm + 3 < M) {
                    float4 t = *reinterpret_cast<const float4*>(A + (long long)gk * lda + gm);
                    ra[it][0] = t.x; ra[it][1] = t.y; ra[it][2] = t.z; ra[it][3] = t.w;
                } else {
                    #pragma unroll
                    for (int e = 0; e < 4; ++e) ra[it][e] = (gk < K && gm + e < M) ? A[(long long)gk * lda + gm + e] : 0.0f;
                }
            }
        }
    };
    auto load_b = [&](int k0) {
        #pragma unroll
        for (int it = 0; it < 2; ++it) {
            int v = tid + it * NTHREADS;
            if (B_NMAJOR) {                          // 4 consecutive n of one k
                int k = v / (BN / 4), nq = (v % (BN / 4)) * 4;
                int gk = k0 + k, gn = n0 + nq;
                if (VEC && gk < K && gn + 3 < N) {
                    float4 t = *reinterpret_cast<const float4*>(B + (long long)gk * ldb + gn);
                    rb[it][0] = t.x; rb[it][1] = t.y; rb[it][2] = t.z; rb[it][3] = t.w;
                } else {
                    #pragma unroll
                    for (int e = 0; e < 4; ++e) rb[it][e] = (gk < K && gn + e < N) ? B[(long long)gk * ldb + gn + e] : 0.0f;
                }
            } else {                                 // 4 consecutive k of one column n
                int nn = v / (BK / 4), kq = (v % (BK / 4)) * 4;
                int gn = n0 + nn, gk = k0 + kq;
                if (VEC && gn < N && gk + 3 < K) {
                    float4 t = *reinterpret_cast<const float4*>(B + (long long)gn * ldb + gk);
                    rb[it][0] = t.x; rb[it][1] = t.y; rb[it][2] = t.z; rb[it][3] = t.w;
                } else {
                    #pragma unroll
                    for (int e = 0; e < 4; ++e) rb[it][e] = (gn < N && gk + e < K) ? B[(long long)gn * ldb + gk + e] : 0.0f;
                }
            }
        }
    };
    auto store_smem = [&](int buf) {
        #pragma unroll
        for (int it = 0; it < 2; ++it) {
            int v = tid + it * NTHREADS;
            if (A_KMAJOR) {
                int m = v / (BK / 4), kq = (v % (BK / 4)) * 4;
                #pragma unroll
                for (int e = 0; e < 4; ++e) As[buf][kq + e][m] = ra[it][e];
            } else {
                int k = v / (BM / 4), mq = (v % (BM / 4)) * 4;
                *reinterpret_cast<float4*>(&As[buf][k][mq]) = make_float4(ra[it][0], ra[it][1], ra[it][2], ra[it][3]);
            }
            if (B_NMAJOR) {
                int k = v / (BN / 4), nq = (v % (BN / 4)) * 4;
                *reinterpret_cast<float4*>(&Bs[buf][k][nq]) = make_float4(rb[it][0], rb[it][1], rb[it][2], rb[it][3]);
            } else {
                int nn = v / (BK / 4), kq = (v % (BK / 4)) * 4;
                #pragma unroll
                for (int e = 0; e < 4; ++e) Bs[buf][kq + e][nn] = rb[it][e];
            }
        }
    };

    const int nslices = (K + BK - 1) / BK;
    load_a(0); load_b(0);
    store_smem(0);
    __syncthreads();
    for (int s = 0; s < nslices; ++s) {
        const int cur = s & 1;
        if (s + 1 < nslices) { load_a((s + 1) * BK); load_b((s + 1) * BK); }
        #pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[8], b[8];
            float4 a0 = *reinterpret_cast<const float4*>(&As[cur][k][ty * 4]);
            float4 a1 = *reinterpret_cast<const float4*>(&As[cur][k][64 + ty * 4]);
            float4 b0 = *reinterpret_cast<const float4*>(&Bs[cur][k][tx * 4]);
            float4 b1 = *reinterpret_cast<const float4*>(&Bs[cur][k][64 + tx * 4]);
            a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w; a[4] = a1.x; a[5] = a1.y; a[6] = a1.z; a[7] = a1.w;
            b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w; b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
            #pragma unroll
            for (int i = 0; i < 8; ++i)
                #pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (s + 1 < nslices) {
            store_smem(cur ^ 1);
            __syncthreads();
        }
    }

    #pragma unroll
    for (int i = 0; i < 8; ++i) {
        int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (gm >= M) continue;
        #pragma unroll
        for (int h = 0; h < 2; ++h) {
            int gn = n0 + h * 64 + tx * 4;
            float* dst = C + (long long)gm * N + gn;
            if (VEC && gn + 3 < N) {
                *reinterpret_cast<float4*>(dst) = make_float4(acc[i][h * 4], acc[i][h * 4 + 1], acc[i][h * 4 + 2], acc[i][h * 4 + 3]);
            } else {
                #pragma unroll
                for (int e = 0; e < 4; ++e) if (gn + e < N) dst[e] = acc[i][h * 4 + e];
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Pipelined variant for operands whose rows can be moved in 16-byte pieces (the common case): cp.async straight from
// global into a 4-stage shared-memory ring, no staging registers.  Layouts in shared memory:
//   operand contiguous along m / n (A transposed, B not transposed): Xs[k][128 (+4)], filled by 16-byte cp.async, read
//       with two float4 per k;
//   B contiguous along k (B transposed): the same Xs[k][132]; the 16 bytes of global memory go out as four 4-byte
//       cp.async to four different k rows — the transposition happens in the copy, not in registers.  Within a warp 16
//       lanes take 16 neighbouring rows and the two halves neighbouring k quads: the writes cover all 32 banks;
//   A contiguous along k (A not transposed): As[m][16 (+4)], filled by 16-byte cp.async, read with one scalar load per
//       row of the micro-tile (all lanes of a warp that share a row read the same word: a broadcast, no conflict) —
//       the packed multiply-add leaves the issue slots for them.
// One block barrier per k-slice; k ascending inside a thread; packed fma.rn.f32x2 on pairs of accumulators (two
// independent, individually rounded fp32 fused multiply-adds): bit-identical to sgemm_kernel.
constexpr int PSTAGES = 4, LDP = BM + 4, LDK = BK + 4;
constexpr int P_OPERAND_FLOATS = BM * LDK;                     // 2560 floats; Xs[k][132] needs 2112
constexpr int P_SMEM_BYTES = PSTAGES * 2 * P_OPERAND_FLOATS * 4;

__device__ __forceinline__ void cp_async16(float* smem_dst, const float* gsrc, int src_bytes) {
    unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(float* smem_dst, const float* gsrc, int src_bytes) {
    unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One operand tile (16 k x 128 rows) of slice k0 into Xs[k][row].  X(row, k) = X[row * ld + k] when K_CONTIG, else
// X[k * ld + row]; rows past `rows` and k past K arrive as zeros.
// K_CONTIG && DIRECT keeps the memory layout instead: Xs[row][k], 20 floats per row.
template <bool K_CONTIG, bool DIRECT>
__device__ __forceinline__ void fill_operand(float* xs, const float* __restrict__ X, int ld, int r0, int rows, int k0, int K, int tid) {
    #pragma unroll
    for (int it = 0; it < 2; ++it) {
        const int c = tid + it * NTHREADS;                      // 512 pieces of 16 bytes
        if (K_CONTIG && DIRECT) {
            const int r = c >> 2, kq = (c & 3) * 4;
            const int gr = r0 + r, gk = k0 + kq;
            const int n_ok = gr < rows ? max(0, min(4, K - gk)) : 0;
            cp_async16(xs + r * LDK + kq, n_ok ? X + (long long)gr * ld + gk : X, n_ok * 4);
        } else if (K_CONTIG) {
            const int r = (c & 15) | ((c >> 6) << 4), kq = ((c >> 4) & 3) * 4;
            const int gr = r0 + r, gk = k0 + kq;
            const int n_ok = gr < rows ? max(0, min(4, K - gk)) : 0;
            const float* src = n_ok ? X + (long long)gr * ld + gk : X;
            #pragma unroll
            for (int e = 0; e < 4; ++e) cp_async4(xs + (kq + e) * LDP + r, e < n_ok ? src + e : X, e < n_ok ? 4 : 0);
        } else {
            const int k = c >> 5, rq = (c & 31) * 4;
            const int gk = k0 + k, gr = r0 + rq;
            const int n_ok = gk < K ? max(0, min(4, rows - gr)) : 0;
            cp_async16(xs + k * LDP + rq, n_ok ? X + (long long)gk * ld + gr : X, n_ok * 4);
        }
    }
}

template <bool A_KMAJOR, bool B_NMAJOR>
__global__ void __launch_bounds__(NTHREADS, 2)
sgemm_pipe_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                  int M, int N, int K, int lda, int ldb, BatchMap bm) {
    extern __shared__ __align__(16) float psm[];
    {
        int b = blockIdx.z;
        long long oa = 0, ob = 0;
        for (int d = bm.nbatch - 1; d >= 0; --d) {
            int c = b % bm.bshape[d];
            b /= bm.bshape[d];
            oa += c * bm.astride[d];
            ob += c * bm.bstride[d];
        }
        A += oa; B += ob;
        C += (long long)blockIdx.z * M * N;
    }
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;
    auto a_stage = [&](int st) { return psm + (st * 2) * P_OPERAND_FLOATS; };
    auto b_stage = [&](int st) { return psm + (st * 2 + 1) * P_OPERAND_FLOATS; };
    auto issue = [&](int slice) {
        const int st = slice % PSTAGES, k0 = slice * BK;
        fill_operand<A_KMAJOR, true>(a_stage(st), A, lda, m0, M, k0, K, tid);
        fill_operand<!B_NMAJOR, false>(b_stage(st), B, ldb, n0, N, k0, K, tid);
    };

    // Accumulators in pairs of neighbouring columns: one packed instruction per pair halves the instructions and the
    // register-file reads of the inner product.
    float2 acc[8][4];
    #pragma unroll
    for (int i = 0; i < 8; ++i)
        #pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = make_float2(0.0f, 0.0f);

    const int nslices = (K + BK - 1) / BK;
    #pragma unroll
    for (int p = 0; p < PSTAGES - 1; ++p) {
        if (p < nslices) issue(p);
        cp_async_commit();
    }
    for (int s = 0; s < nslices; ++s) {
        cp_async_wait<PSTAGES - 2>();            // slice s has landed (for this thread's copies)
        __syncthreads();                         // ... and everybody's; everybody is also done with slice s - 1
        if (s + PSTAGES - 1 < nslices) issue(s + PSTAGES - 1);     // into the buffer slice s - 1 used
        cp_async_commit();
        const float* as = a_stage(s % PSTAGES);
        const float* bs = b_stage(s % PSTAGES);
        #pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[8];
            if (A_KMAJOR) {
                #pragma unroll
                for (int i = 0; i < 8; ++i) a[i] = as[(i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4) * LDK + k];
            } else {
                const float4 a0 = *reinterpret_cast<const float4*>(as + k * LDP + ty * 4);
                const float4 a1 = *reinterpret_cast<const float4*>(as + k * LDP + 64 + ty * 4);
                a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w; a[4] = a1.x; a[5] = a1.y; a[6] = a1.z; a[7] = a1.w;
            }
            const float4 b0 = *reinterpret_cast<const float4*>(bs + k * LDP + tx * 4);
            const float4 b1 = *reinterpret_cast<const float4*>(bs + k * LDP + 64 + tx * 4);
            const float2 b2[4] = {make_float2(b0.x, b0.y), make_float2(b0.z, b0.w), make_float2(b1.x, b1.y), make_float2(b1.z, b1.w)};
            #pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 aa = make_float2(a[i], a[i]);
                #pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __ffma2_rn(aa, b2[j], acc[i][j]);
            }
        }
    }
    cp_async_wait<0>();

    #pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (gm >= M) continue;
        float* crow = C + (long long)gm * N;
        #pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int gn = n0 + h * 64 + tx * 4;
            const float v[4] = {acc[i][2 * h].x, acc[i][2 * h].y, acc[i][2 * h + 1].x, acc[i][2 * h + 1].y};
            if (gn + 3 < N) *reinterpret_cast<float4*>(crow + gn) = make_float4(v[0], v[1], v[2], v[3]);
            else {
                #pragma unroll
                for (int e = 0; e < 4; ++e) if (gn + e < N) crow[gn + e] = v[e];
            }
        }
    }
}

template <bool AK, bool BN_>
void launch_pipe(ormi_b200_ctx* ctx, const GemmArgs& g, const BatchMap& bm) {
    static bool attr_set = false;      // per instantiation
    if (!attr_set) {
        ORMI_CUDA(cudaFuncSetAttribute(sgemm_pipe_kernel<AK, BN_>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES));
        attr_set = true;
    }
    dim3 grid((g.N + BN - 1) / BN, (g.M + BM - 1) / BM, g.batch);
    sgemm_pipe_kernel<AK, BN_><<<grid, NTHREADS, P_SMEM_BYTES, ctx->stream>>>(g.A, g.B, g.C, g.M, g.N, g.K, g.lda, g.ldb, bm);
    ORMI_CUDA(cudaGetLastError());
}

template <bool AK, bool BN_, bool VEC>
void launch(ormi_b200_ctx* ctx, const GemmArgs& g, const BatchMap& bm) {
    dim3 grid((g.N + BN - 1) / BN, (g.M + BM - 1) / BM, g.batch);
    sgemm_kernel<AK, BN_, VEC><<<grid, NTHREADS, 0, ctx->stream>>>(g.A, g.B, g.C, g.M, g.N, g.K, g.lda, g.ldb, bm);
    ORMI_CUDA(cudaGetLastError());
}

}  // namespace

void gemm_ffma(ormi_b200_ctx* ctx, const GemmArgs& g) {
    BatchMap bm;
    bm.nbatch = g.nbatch;
    for (int d = 0; d < ORMI_B200_MAX_DIMS; ++d) { bm.bshape[d] = g.bshape[d]; bm.astride[d] = g.astride[d]; bm.bstride[d] = g.bstride[d]; }
    if (g.batch > 65535) throw Error("matmul: more than 65535 batches");
    bool vec = (g.lda % 4 == 0) && (g.ldb % 4 == 0) && (g.N % 4 == 0) &&
               ((uintptr_t)g.A % 16 == 0) && ((uintptr_t)g.B % 16 == 0) && ((uintptr_t)g.C % 16 == 0);
    for (int d = 0; d < g.nbatch; ++d) if (g.astride[d] % 4 || g.bstride[d] % 4) vec = false;
    if ((long long)g.M * g.N % 4) vec = false;
    const bool ak = !g.trans_a, bn = !g.trans_b;
    if (vec) {           // rows movable in 16-byte pieces: the pipelined kernel
        if (ak && bn) launch_pipe<true, true>(ctx, g, bm);
        else if (ak && !bn) launch_pipe<true, false>(ctx, g, bm);
        else if (!ak && bn) launch_pipe<false, true>(ctx, g, bm);
        else launch_pipe<false, false>(ctx, g, bm);
    } else {
        if (ak && bn) launch<true, true, false>(ctx, g, bm);
        else if (ak && !bn) launch<true, false, false>(ctx, g, bm);
        else if (!ak && bn) launch<false, true, false>(ctx, g, bm);
        else launch<false, false, false>(ctx, g, bm);
    }
    ctx->counters["gemm_launches"]++;
    ctx->counters["launches"]++;
}

}  // namespace ormi_b200
