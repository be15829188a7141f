// Tensor-core GEMM for sm_100a (bf16, tf32 and 3xTF32 operands): tcgen05.mma with TMEM accumulators, operands staged by TMA.
//
// Opt-in matmul arithmetic ("matmul" = "bf16") behind ormi::cuda::matmul
// (ormi-core/csrc/backend/cuda/kernels/blas/matmul.cu:19-112, which calls cublasSgemmBatched): fp32 operands
// are rounded to bf16 once, products are accumulated in fp32 in tensor memory, C is written in fp32.
//
//   C[M,N] = A[M,K] * B[K,N]
//
// Layout in HBM.  Both operands are first brought into "K-major" bf16 staging buffers, A as [M][Kp] and B
// transposed as [N][Kp] (Kp = K rounded up to 64, zero padded), whatever strides / transposition the
// views had: one conversion pass each (cvt_kmajor), which is also where fp32 -> bf16 happens.
//
// Kernel.  Persistent, one 192-thread block per SM, tile 128 x 256 x 64:
//   warp 0     producer: one lane issues the TMA loads of the A (128x64) and B (256x64) boxes of the next
//              k-slice into a 4-stage shared-memory ring (128-byte swizzle), completion counted on an mbarrier;
//   warp 1     allocates 512 TMEM columns (two 128x256 fp32 accumulators); one lane issues 4 tcgen05.mma
//              (M=128, N=256, K=16) per stage and commits them to the stage's "empty" barrier; after the last
//              slice of a tile it commits to the accumulator's "full" barrier;
//   warps 2-5  epilogue: each warp owns 32 TMEM lanes (= 32 rows of the tile), reads the accumulator with
//              tcgen05.ld 32 columns at a time and stores fp32 rows to C; then releases the accumulator.
// The two accumulators let the epilogue of tile i overlap the MMAs of tile i+1.  Tiles are walked in groups
// of 16 row-blocks so that concurrently running blocks share A and B panels in L2.
//
// Tiles are handed out dynamically: the producer lane takes the next tile index from a counter in global memory
// (left at zero by the previous launch) and passes it to the other roles through a 4-slot ring in shared memory.  A block
// that becomes resident late — another stream's kernel, a collective for one, holds some SMs — then finds
// only what is left instead of a fixed share the others would have to wait for.
//
// No cluster launch and no multicast anywhere: every block fetches its own boxes.
//
// Every wait is bounded (about two seconds on the global timer).  A wait that runs out raises a block-wide
// abort flag and an error word in global memory; every role then leaves its loop, the block lets copies in
// flight land, frees its tensor memory and exits; the host turns the error word into a failure.
#include <cuda_bf16.h>

#include "context.h"

namespace ormi_b200 {

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16, SCHED = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2, B_STAGE_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr int NUM_THREADS = 192;
constexpr int GROUP_M = 16;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long global_ns() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the block is aborting (this wait ran out, or another role's did).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code,
                                          unsigned long long limit_ns = WAIT_LIMIT_NS) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i) if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_ns() - t0 > limit_ns) { *abort_flag = 1; atomicCAS(err, 0, code); return false; }
    }
}

// Self-test of the bounded wait: a barrier nobody ever arrives on.  The wait gives up after `limit_ns`, leaves code 9 in
// the error word and the kernel returns; nothing faults and the context stays usable.
__global__ void wait_timeout_selftest_kernel(int* err, unsigned long long limit_ns) {
    __shared__ unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_wait(smem_u32(&bar), 0u, &abort_flag, err, 9, limit_ns);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bf16) and were written with the
// 128-byte swizzle: 8-row groups are 1024 bytes apart (SBO), the leading-dimension offset is unused (1),
// descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor: D fp32 (bits 4-5 = 1), A and B format (bits 7-9, 10-12: 1 = bf16, 2 = tf32), both K-major,
// N = 256 (bits 17-22 = N/8), M = 128 (bits 24-28 = M/16).
__host__ __device__ constexpr uint32_t idesc(uint32_t fmt) { return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24); }

// One MMA covers 32 bytes of K per operand row: 16 bf16 (kind::f16) or 8 tf32 (kind::tf32).
template <bool TF32>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t accumulate) {
    if (TF32)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc(2)), "r"(accumulate) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc(1)), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    #pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& mb, int& nb) {
    const int per_group = GROUP_M * tiles_n;
    const int g = t / per_group;
    const int first_m = g * GROUP_M;
    const int gsz = min(GROUP_M, tiles_m - first_m);
    const int in_g = t - g * per_group;
    mb = first_m + in_g % gsz;
    nb = in_g / gsz;
}

// TF32 = false: operands are bf16, a stage row holds 64 elements.  TF32 = true: operands are fp32 words already rounded
// to tf32, a stage row holds 32 elements.  Both are 128 bytes per row, so ring, swizzle and descriptors are the same.
template <bool TF32>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 float* __restrict__ C, int M, int N, int num_kb, int tiles_m, int tiles_n, int* err, int* tile_counter) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;       // swizzled tiles need 1024-byte alignment
    uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + STAGES * STAGE_BYTES;                   // 8-byte mbarriers
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
    auto sfull_bar = [&](int q) { return bars + 8u * (2 * STAGES + 4 + q); };
    auto sempty_bar = [&](int q) { return bars + 8u * (2 * STAGES + 4 + SCHED + q); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 4 + 2 * SCHED));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* sched_tile = reinterpret_cast<volatile int*>(tmem_slot + 2);      // SCHED slots; -1 = no tiles left

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
        for (int q = 0; q < SCHED; ++q) { mbar_init(sfull_bar(q), 1); mbar_init(sempty_bar(q), 5); }   // readers: MMA lane + 4 epilogue warps
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            int s = 0; uint32_t phase = 0;
            int q = 0; uint32_t qphase = 0;
            for (;;) {
                if (!mbar_wait(sempty_bar(q), qphase ^ 1u, abort_flag, err, 5)) break;
                int t = atomicAdd(tile_counter, 1);
                if (t >= num_tiles) {
                    // Every block draws exactly one index past the end; the block that draws the last one leaves the
                    // counter pair zeroed for the next launch on the stream.
                    t = -1;
                    if (atomicAdd(tile_counter + 1, 1) == (int)gridDim.x - 1) { tile_counter[1] = 0; __threadfence(); atomicExch(tile_counter, 0); }
                }
                sched_tile[q] = t;
                mbar_arrive(sfull_bar(q));                    // release: the slot is visible to whoever sees this phase
                if (++q == SCHED) { q = 0; qphase ^= 1u; }
                if (t < 0) break;
                int mb, nb; tile_coords(t, tiles_m, tiles_n, mb, nb);
                bool ok = true;
                for (int kb = 0; kb < num_kb && ok; ++kb) {
                    ok = mbar_wait(empty_bar(s), phase ^ 1u, abort_flag, err, 1);
                    if (!ok) break;
                    mbar_expect_tx(full_bar(s), STAGE_BYTES);
                    tma_load_2d(base + s * STAGE_BYTES, &map_a, full_bar(s), kb * (TF32 ? BK / 2 : BK), mb * BM);
                    tma_load_2d(base + s * STAGE_BYTES + A_STAGE_BYTES, &map_b, full_bar(s), kb * (TF32 ? BK / 2 : BK), nb * BN);
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int s = 0; uint32_t phase = 0;
            int q = 0; uint32_t qphase = 0;
            for (int it = 0;; ++it) {
                if (!mbar_wait(sfull_bar(q), qphase, abort_flag, err, 6)) break;
                const int t = sched_tile[q];
                mbar_arrive(sempty_bar(q));
                if (++q == SCHED) { q = 0; qphase ^= 1u; }
                if (t < 0) break;
                const int a = it & 1;
                const uint32_t aphase = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(tempty_bar(a), aphase ^ 1u, abort_flag, err, 2)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(a * BN);
                bool ok = true;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(full_bar(s), phase, abort_flag, err, 3);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t da = umma_desc_sw128(base + s * STAGE_BYTES);
                    const uint64_t db = umma_desc_sw128(base + s * STAGE_BYTES + A_STAGE_BYTES);
                    #pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)     // 32 bytes further along K inside the swizzle atom
                        umma<TF32>(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(empty_bar(s));                // frees the stage once these MMAs have read it
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(tfull_bar(a));                    // accumulator complete
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;                         // TMEM lanes 32*quarter .. 32*quarter+31
        int q = 0; uint32_t qphase = 0;
        for (int it = 0;; ++it) {
            bool got = mbar_wait(sfull_bar(q), qphase, abort_flag, err, 7);
            got = __all_sync(0xffffffffu, got);
            if (!got) break;
            const int t = sched_tile[q];
            __syncwarp();                                     // every lane has read the slot
            if (lane == 0) mbar_arrive(sempty_bar(q));
            if (++q == SCHED) { q = 0; qphase ^= 1u; }
            if (t < 0) break;
            int mb, nb; tile_coords(t, tiles_m, tiles_n, mb, nb);
            const int a = it & 1;
            const uint32_t aphase = (uint32_t)(it >> 1) & 1u;
            bool ok = mbar_wait(tfull_bar(a), aphase, abort_flag, err, 4);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row = mb * BM + quarter * 32 + lane;
            float* crow = C + (size_t)row * N + (size_t)nb * BN;
            #pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                float v[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(a * BN + c * 32), v);
                const int col0 = nb * BN + c * 32;
                if (row < M) {
                    if (col0 + 32 <= N && (N & 3) == 0) {
                        #pragma unroll
                        for (int i = 0; i < 8; ++i)
                            *reinterpret_cast<float4*>(crow + c * 32 + 4 * i) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    } else {
                        #pragma unroll
                        for (int i = 0; i < 32; ++i) if (col0 + i < N) crow[c * 32 + i] = v[i];
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(a));
        }
    }

    // ------------------------------------------------------------------ teardown
    __syncwarp();
    if (*abort_flag) {                     // let copies that are still in flight land before the block goes away
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) { }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// dst[row * Kp + k] = bf16(src[row * s_row + k * s_k]) for row < rows, k < K; zero for K <= k < Kp.
// One block converts a 64 x 64 tile; every thread ends up writing eight consecutive k of one row as one 16-byte
// store, eight lanes covering a whole 128-byte line of dst.
//   source contiguous along k:    two float4 loads per thread, no shared memory;
//   source contiguous along rows: float4 loads along the rows, transposed through shared memory;
//   anything else (or unaligned): scalar loads through shared memory.
// One launch serves both operands of a GEMM: the first `a.blocks` blocks work on job a, the rest on job b.
struct CvtJob {
    const float* src; long long s_row, s_k; int rows, K, Kp; void* dst;
    int blocks_x, blocks;        // 64 x 64 tiles along k, and in total
    int mode;                    // 0 k-contiguous vector path, 1 row-contiguous vector path, 2 scalar
    int is_b;                    // tf32 split only: a B operand stores (hi, lo, hi), an A operand (hi, hi, lo)
};

constexpr int CT = 64;           // tile edge

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float to_tf32(float x) { uint32_t r; asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x)); return __uint_as_float(r); }

// Eight consecutive k of row r, starting at k.  PARTS = 0: bf16, one 16-byte store.  PARTS = 1: fp32 words rounded to
// tf32.  PARTS = 3 (the "3xTF32" split): hi = tf32(x), lo = tf32(x - hi) stored at k, Kp + k, 2 Kp + k as (hi, hi, lo)
// for an A operand and (hi, lo, hi) for a B operand, so that one GEMM over 3 Kp columns adds up
// A_hi B_hi + A_hi B_lo + A_lo B_hi — fp32 products to about 2^-22.
template <int PARTS>
__device__ __forceinline__ void store8(const CvtJob& j, int r, int k, const float* v) {
    if (PARTS == 0) {
        uint4 o = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(j.dst) + (size_t)r * j.Kp + k) = o;
    } else {
        if (k >= j.Kp) return;                                   // Kp is a multiple of 32 here, the tile is 64 wide
        float* row = static_cast<float*>(j.dst) + (size_t)r * j.Kp * PARTS + k;
        float hi[8], lo[8];
        #pragma unroll
        for (int i = 0; i < 8; ++i) { hi[i] = to_tf32(v[i]); lo[i] = PARTS == 3 ? to_tf32(v[i] - hi[i]) : 0.0f; }
        auto put = [&](float* p, const float* w) {
            *reinterpret_cast<float4*>(p) = make_float4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<float4*>(p + 4) = make_float4(w[4], w[5], w[6], w[7]);
        };
        put(row, hi);
        if (PARTS == 3) { put(row + j.Kp, j.is_b ? lo : hi); put(row + 2 * j.Kp, j.is_b ? hi : lo); }
    }
}

template <int PARTS>
__global__ void __launch_bounds__(256)
cvt_kmajor(const CvtJob a, const CvtJob b) {
    __shared__ float tile[CT][CT + 1];                           // [k][row]
    int bid = blockIdx.x;
    const bool second = bid >= a.blocks;
    const CvtJob& j = second ? b : a;
    if (second) bid -= a.blocks;
    const int r0 = (bid / j.blocks_x) * CT, k0 = (bid % j.blocks_x) * CT;
    const float* __restrict__ src = j.src;
    const int tid = threadIdx.x;
    const int kseg = tid & 7;                                    // which 8 k of the 64
    const int rsub = tid >> 3;                                   // 0..31; rows rsub and rsub + 32

    if (j.mode == 0) {
        #pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = r0 + rsub + 32 * h, k = k0 + 8 * kseg;
            if (r >= j.rows) continue;
            float v[8];
            if (k + 8 <= j.K) {
                const float4 p = *reinterpret_cast<const float4*>(src + r * j.s_row + k);
                const float4 q = *reinterpret_cast<const float4*>(src + r * j.s_row + k + 4);
                v[0] = p.x; v[1] = p.y; v[2] = p.z; v[3] = p.w; v[4] = q.x; v[5] = q.y; v[6] = q.z; v[7] = q.w;
            } else {
                #pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = (k + i < j.K) ? src[r * j.s_row + k + i] : 0.0f;
            }
            store8<PARTS>(j, r, k, v);
        }
        return;
    }

    if (j.mode == 1) {                                           // 16 lanes x float4 = 64 rows of one k; 16 k per pass
        const int rq = (tid & 15) * 4, kk = tid >> 4;
        #pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
            const int kt = kk + 16 * pass, k = k0 + kt, r = r0 + rq;
            float4 p = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (k < j.K) {
                if (r + 4 <= j.rows) p = *reinterpret_cast<const float4*>(src + r + k * j.s_k);
                else {
                    if (r < j.rows) p.x = src[r + k * j.s_k];
                    if (r + 1 < j.rows) p.y = src[r + 1 + k * j.s_k];
                    if (r + 2 < j.rows) p.z = src[r + 2 + k * j.s_k];
                }
            }
            tile[kt][rq] = p.x; tile[kt][rq + 1] = p.y; tile[kt][rq + 2] = p.z; tile[kt][rq + 3] = p.w;
        }
    } else {
        for (int e = tid; e < CT * CT; e += 256) {
            const int kt = e / CT, rt = e % CT;
            const int k = k0 + kt, r = r0 + rt;
            tile[kt][rt] = (r < j.rows && k < j.K) ? src[r * j.s_row + k * j.s_k] : 0.0f;
        }
    }
    __syncthreads();
    #pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int rt = rsub + 32 * h, r = r0 + rt;
        if (r >= j.rows) continue;
        float v[8];
        #pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = tile[8 * kseg + i][rt];
        store8<PARTS>(j, r, k0 + 8 * kseg, v);
    }
}

CvtJob cvt_job(const float* src, long long s_row, long long s_k, int rows, int K, int Kp, void* dst, int is_b = 0) {
    CvtJob j{src, s_row, s_k, rows, K, Kp, dst, (Kp + CT - 1) / CT, 0, 2, is_b};
    j.blocks = j.blocks_x * ((rows + CT - 1) / CT);
    const bool aligned = ((uintptr_t)src & 15) == 0;
    if (s_k == 1 && aligned && s_row % 4 == 0) j.mode = 0;
    else if (s_row == 1 && aligned && s_k % 4 == 0) j.mode = 1;
    return j;
}

void convert(ormi_b200_ctx* ctx, const CvtJob& a, const CvtJob& b, int parts = 0) {
    if (parts == 0) cvt_kmajor<0><<<a.blocks + b.blocks, 256, 0, ctx->stream>>>(a, b);
    else if (parts == 1) cvt_kmajor<1><<<a.blocks + b.blocks, 256, 0, ctx->stream>>>(a, b);
    else cvt_kmajor<3><<<a.blocks + b.blocks, 256, 0, ctx->stream>>>(a, b);
    ORMI_CUDA(cudaGetLastError());
    ctx->counters["launches"]++;
}

// Staging copies of one GEMM call: blocks of the context's pool, taken before the conversion pass and given back as soon
// as the GEMM is queued (the pool is ordered by the stream, so the next call may get the same blocks) — nothing here
// synchronises the stream or calls cudaFree in the middle of a step.
struct Staging {
    ormi_b200_ctx* ctx; void* p[2] = {nullptr, nullptr}; size_t n[2] = {0, 0};
    explicit Staging(ormi_b200_ctx* c) : ctx(c) {}
    void* get(int which, size_t bytes) { p[which] = pool_alloc(ctx, bytes); n[which] = bytes; return p[which]; }
    ~Staging() { for (int i = 0; i < 2; ++i) if (p[i]) pool_free(ctx, p[i], n[i]); }
};

void make_map(ormi_b200_ctx* ctx, CUtensorMap* map, void* ptr, int rows, int Kp, int box_rows, bool fp32 = false) {
    cuuint64_t dims[2] = {(cuuint64_t)Kp, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)Kp * (fp32 ? 4 : 2)};
    cuuint32_t box[2] = {(cuuint32_t)(fp32 ? BK / 2 : BK), (cuuint32_t)box_rows};     // 128 bytes of K either way
    cuuint32_t estr[2] = {1, 1};
    ctx->drv.check(ctx->drv.TensorMapEncodeTiled(map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims, strides, box, estr,
                                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
                   "cuTensorMapEncodeTiled");
}

}  // namespace

void gemm_bf16(ormi_b200_ctx* ctx, const GemmArgs& g) {
    // Small or batched problems stay on the fp32 path (a batch is a loop of independent GEMMs; the tensor path is
    // worth its two conversion passes only for large single products).
    if (g.batch != 1 || (long long)g.M * g.N * g.K < (1ll << 21) || g.K < 64) { gemm_ffma(ctx, g); return; }
    // operands whose rows are whole 16-byte pieces of bf16 go to the run-time compiled kernel, in their own layout
    if (ctx->tc_cta_group != 0 && gemm_tc_supported(g)) { gemm_tc_from_fp32(ctx, g); return; }
    const int Kp = (g.K + BK - 1) / BK * BK;
    Staging staging(ctx);
    __nv_bfloat16* a16 = (__nv_bfloat16*)staging.get(0, (size_t)g.M * Kp * 2);
    __nv_bfloat16* b16 = (__nv_bfloat16*)staging.get(1, (size_t)g.N * Kp * 2);
    // A(m,k) = A[m*lda + k] (or A[k*lda + m] when stored transposed); B(k,n) = B[k*ldb + n] (or B[n*ldb + k])
    convert(ctx, cvt_job(g.A, g.trans_a ? 1 : g.lda, g.trans_a ? g.lda : 1, g.M, g.K, Kp, a16),
            cvt_job(g.B, g.trans_b ? g.ldb : 1, g.trans_b ? 1 : g.ldb, g.N, g.K, Kp, b16));

    gemm_bf16_kmajor(ctx, a16, b16, g.C, g.M, g.N, Kp);
}

// C[M,N] (fp32) = A16[M][Kp] * B16[N][Kp]^T, both operands bf16, K-major, Kp a multiple of 64 (zero padded).
void gemm_bf16_kmajor(ormi_b200_ctx* ctx, const void* a16, const void* b16, float* C, int M, int N, int Kp) {
    if (M <= 0 || N <= 0 || Kp <= 0 || Kp % BK != 0) throw Error("gemm_bf16: K of the staged operands must be a positive multiple of 64");
    if (((uintptr_t)a16 | (uintptr_t)b16 | (uintptr_t)C) & 15) throw Error("gemm_bf16: operands must be 16-byte aligned");
    CUtensorMap map_a, map_b;
    make_map(ctx, &map_a, const_cast<void*>(a16), M, Kp, BM);
    make_map(ctx, &map_b, const_cast<void*>(b16), N, Kp, BN);
    device_error_word(ctx);
    if (!ctx->gemm_attr_set) {
        ORMI_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        ORMI_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        ctx->gemm_attr_set = true;
    }
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
    const int grid = std::min(tiles_m * tiles_n, ctx->num_sms);
    gemm_tc_kernel<false><<<grid, NUM_THREADS, SMEM_BYTES, ctx->stream>>>(map_a, map_b, C, M, N, Kp / BK, tiles_m, tiles_n, ctx->gemm_err,
                                                                           ctx->gemm_err + kTileCounterWord);
    ORMI_CUDA(cudaGetLastError());
    ctx->gemm_err_pending = true;
    ctx->counters["gemm_launches"]++;
    ctx->counters["launches"]++;
}

// fp32 matmul on the tensor cores: operands rounded to tf32 (parts = 1, about 1e-3 relative) or split in two tf32 terms
// each (parts = 3, "3xTF32": three products per k, fp32-grade results at a third of the tf32 rate).
void gemm_tf32(ormi_b200_ctx* ctx, const GemmArgs& g, int parts) {
    if (g.batch != 1 || (long long)g.M * g.N * g.K < (1ll << 21) || g.K < 32) { gemm_ffma(ctx, g); return; }
    const int KB = BK / 2;                                   // 32 fp32 words per stage row
    const int Kp = (g.K + KB - 1) / KB * KB;
    const size_t ld = (size_t)Kp * parts;
    Staging staging(ctx);
    float* a32 = (float*)staging.get(0, (size_t)g.M * ld * 4);
    float* b32 = (float*)staging.get(1, (size_t)g.N * ld * 4);
    convert(ctx, cvt_job(g.A, g.trans_a ? 1 : g.lda, g.trans_a ? g.lda : 1, g.M, g.K, Kp, a32, 0),
            cvt_job(g.B, g.trans_b ? g.ldb : 1, g.trans_b ? 1 : g.ldb, g.N, g.K, Kp, b32, 1), parts);
    CUtensorMap map_a, map_b;
    make_map(ctx, &map_a, a32, g.M, (int)ld, BM, true);
    make_map(ctx, &map_b, b32, g.N, (int)ld, BN, true);
    device_error_word(ctx);
    if (!ctx->gemm_attr_set) {
        ORMI_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        ORMI_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        ctx->gemm_attr_set = true;
    }
    const int tiles_m = (g.M + BM - 1) / BM, tiles_n = (g.N + BN - 1) / BN;
    const int grid = std::min(tiles_m * tiles_n, ctx->num_sms);
    gemm_tc_kernel<true><<<grid, NUM_THREADS, SMEM_BYTES, ctx->stream>>>(map_a, map_b, g.C, g.M, g.N, (int)(ld / KB), tiles_m, tiles_n, ctx->gemm_err,
                                                                          ctx->gemm_err + kTileCounterWord);
    ORMI_CUDA(cudaGetLastError());
    ctx->gemm_err_pending = true;
    ctx->counters["gemm_launches"]++;
    ctx->counters["launches"]++;
}

// dst[row][k] = bf16(src[row * s_row + k * s_k]), rows x Kp bf16 with Kp = K rounded up to 64 (zero padded).
void cvt_bf16_kmajor(ormi_b200_ctx* ctx, const float* src, long long s_row, long long s_k, int rows, int K, void* dst) {
    CvtJob none{};
    convert(ctx, cvt_job(src, s_row, s_k, rows, K, (K + BK - 1) / BK * BK, (__nv_bfloat16*)dst), none);
}

void selftest_wait_timeout(ormi_b200_ctx* ctx, int limit_ms) {
    if (limit_ms < 1 || limit_ms > 1000) throw Error("selftest_wait_timeout: limit must be 1..1000 ms");
    int* err = device_error_word(ctx);
    wait_timeout_selftest_kernel<<<1, 32, 0, ctx->stream>>>(err, (unsigned long long)limit_ms * 1000000ull);
    ORMI_CUDA(cudaGetLastError());
    ctx->gemm_err_pending = true;
}

// Called at host-visible boundaries (sync, device -> host copies): a bounded wait that ran out inside the tensor-core
// kernel left a code in the error word.
void check_gemm_error(ormi_b200_ctx* ctx) {
    if (!ctx->gemm_err || !ctx->gemm_err_pending) return;
    int code = 0;
    ORMI_CUDA(cudaMemcpyAsync(&code, ctx->gemm_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    ORMI_CUDA(cudaStreamSynchronize(ctx->stream));
    ctx->gemm_err_pending = false;
    if (code != 0) {
        // a block that gave up may not have drawn its last index: put the tile counter pair back to zero as well
        ORMI_CUDA(cudaMemsetAsync(ctx->gemm_err, 0, kErrorWords * sizeof(int), ctx->stream));
        throw Error("a bounded device-side wait ran out (code " + std::to_string(code) +
                    ": tensor-core GEMM 1 producer, 2 accumulator, 3 operands, 4 epilogue, 5-7 tile ring; 9 self-test; 101 staged row kernel)");
    }
}

}  // namespace ormi_b200
