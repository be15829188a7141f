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
// (two 4-wide strips per axis so shared-memory reads are 128-bit and conflict-free), double-buffered
// shared memory with the next slice prefetched into registers while the current one is multiplied.
// Accumulation over k is in ascending order inside a thread: deterministic, no split-K, no atomics.
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
    if (vec) {
        if (ak && bn) launch<true, true, true>(ctx, g, bm);
        else if (ak && !bn) launch<true, false, true>(ctx, g, bm);
        else if (!ak && bn) launch<false, true, true>(ctx, g, bm);
        else launch<false, false, true>(ctx, g, bm);
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
