R"GEMMTPL(
// Tensor-core GEMM for sm_100a, compiled at run time (NVRTC) with a generated epilogue.
//
//   D[M,N] = A[M,K] * B[K,N]   bf16 operands, fp32 accumulation in tensor memory
//
// Replaces the cublasSgemmBatched call of ormi::cuda::matmul
// (ormi-core/csrc/backend/cuda/kernels/blas/matmul.cu:98-105) when the matmul arithmetic is "bf16".
//
// Operands are bf16 matrices in their NATURAL row-major layout, read through TMA tensor maps:
//   A stored [M][K] (K contiguous, "K-major")        or [K][M] (M contiguous, "MN-major": a transposed view)
//   B stored [N][K] (K contiguous: a transposed view) or [K][N] (N contiguous, "MN-major": the plain row-major B)
// so no operand is ever transposed or padded in memory: K tails and M/N tails are zero-filled by TMA.
//
// Compile-time parameters (macros written in front of this text by the host):
//   G_CTA_GROUP   1: one CTA computes a 128 x 256 tile.  2: a cluster of two CTAs computes 256 x 256 with
//                 tcgen05.mma.cta_group::2 — each CTA loads its own 128 rows of A and its own 128 columns of B
//                 (plain TMA loads, no multicast), the pair's leader issues the MMAs, each CTA owns 128 x 256 of D.
//   G_A_MN, G_B_MN   operand is MN-major (see above)
//   G_EPI_WPQ     epilogue warps per TMEM lane quarter (1, 2 or 4): heavy generated epilogues need more issue slots
//   G_STAGES      depth of the TMA -> MMA shared-memory ring
//   G_EPI_PARAMS  extra kernel parameters of the generated epilogue (text starting with a comma, or empty)
//   G_EPI_INIT    statements run once by every epilogue thread (scalar operands)
//   G_EPI_COLS    statements run once per 32-column chunk: `gcol` is the first of the 4 columns this lane owns
//   G_EPI_PRE     statements run per row step `p` (rows grow = row0 + 4 p + rsub) before the bounds guard: they take the
//                 prefetched pieces of full-matrix operands and request the next step's
//   G_EPI_BODY    statements run per (row, 4 columns): `acc` (float4), `grow`, `gcol`, `M`, `N` are in scope
//   G_EPI_END     statements run once per chunk after its rows (column sums: combine lanes, write the block's partial;
//                 `row0` is the first row of the warp's 32-row block, `rsub` = lane / 8)
//   G_EPI_UNROLL  how many of a chunk's 8 row steps are unrolled (a heavy body must not outgrow the instruction cache)
//
// Roles (warps): 0 producer (one lane issues TMA), 1 MMA issuer (one lane, leader CTA only) and TMEM owner,
// 2.. epilogue.  Two 256-column accumulators in tensor memory let the epilogue of tile i overlap the MMAs of tile i+1.
// Tiles are handed out dynamically (an atomic counter in global memory that the last finisher leaves at zero), so a
// block that becomes resident late — a collective on another stream holds some SMs — takes what is left.
//
// Epilogue data path: tcgen05.ld (lane = row, 32 columns) -> swizzled shared-memory staging -> read back as
// 4 rows x 128 bytes per warp instruction, so every global load and store of the epilogue is a full line.
//
// Every wait is bounded (about two seconds on the global timer); a wait that runs out raises the pair's abort flags
// and the error word in global memory, every role leaves its loop, copies in flight are given time to land, tensor
// memory is freed and the kernel returns.  No TMA load here uses cluster multicast.
#ifndef G_CTA_GROUP
#define G_CTA_GROUP 1
#endif

struct __align__(64) TensorMap { unsigned long long opaque[16]; };

constexpr int CG = G_CTA_GROUP;
constexpr int BM = 128;                       // rows of A (and of D) per CTA
constexpr int BN = G_BN;                      // columns of D per tile: 256, or 128 for problems of few tiles
constexpr int BNC = BN / CG;                  // columns of B this CTA loads
constexpr int BK = 64;                        // k per stage (128 bytes of bf16)
constexpr int UMMA_K = 16;
constexpr int STAGES = G_STAGES;
constexpr int SCHED = 4;
constexpr int EPI_WPQ = G_EPI_WPQ;
constexpr int EPI_UNROLL = G_EPI_UNROLL;
constexpr int EPI_WARPS = 4 * EPI_WPQ;
constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BNC * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STG_BYTES = 4096 * (G_TMA_STORE ? 2 : 1);   // per epilogue warp: 32 rows x 128 bytes (two such buffers when TMA stores them)
constexpr int GROUP_M = 16 / CG;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long global_ns() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ unsigned cluster_rank() {
#if G_CTA_GROUP == 2
    unsigned r; asm volatile("mov.u32 %0, %cluster_ctarank;" : "=r"(r)); return r;
#else
    return 0u;
#endif
}
// Address of the same shared-memory location in CTA `cta` of the pair (shared::cluster window).
__device__ __forceinline__ unsigned in_cta(unsigned addr, unsigned cta) {
#if G_CTA_GROUP == 2
    unsigned r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta)); return r;
#else
    return addr;
#endif
}
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
// Barrier operations come in two strengths.  The per-stage ring and the accumulator hand-over carry no data written
// by ordinary stores (TMA and tcgen05 deliver it, the barriers only count), so they use the default CTA-scope
// forms, also for an arrival on the other CTA's barrier: a cluster-scope release there is a memory fence on the
// producer's critical path, once per 64 k.  The tile schedule slot IS written by an ordinary (remote) store, once per
// tile, so its arrivals release and its waits acquire at cluster scope.  `bar` is a shared::cluster address (in_cta)
// for arrivals and a plain shared::cta address for waits.
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_release_cluster(unsigned bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait_acquire_cluster(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

struct Shared {
    volatile int abort_flag;
    unsigned abort_peer;        // shared::cluster address of the other CTA's abort flag (own flag when CG == 1)
    int* err;
};

__device__ __forceinline__ void raise_abort(Shared& sh, int code) {
    sh.abort_flag = 1;
#if G_CTA_GROUP == 2
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(sh.abort_peer), "r"(1) : "memory");
#endif
    atomicCAS(sh.err, 0, code);
}

// Bounded wait.  Returns false when the pair is aborting (this wait ran out, or another role's did).
template <bool CLUSTER_ACQUIRE = false>
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, Shared& sh, int code) {
    auto poll = [&]() { return CLUSTER_ACQUIRE ? mbar_try_wait_acquire_cluster(bar, parity) : mbar_try_wait(bar, parity); };
    if (poll()) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i) if (poll()) return true;
        if (sh.abort_flag) return false;
        if (global_ns() - t0 > WAIT_LIMIT_NS) { raise_abort(sh, code); return false; }
    }
}

// 2-D TMA load into this CTA's shared memory; completion bytes are counted on `bar`, which may be the leader's barrier
// (shared::cluster address) when two CTAs feed one MMA.
__device__ __forceinline__ void tma_load_2d(unsigned dst, const TensorMap* map, unsigned bar, int x, int y) {
#if G_CTA_GROUP == 2
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
#else
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
#endif
}

// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1.
//   K-major tile:  rows of 128 bytes (64 k), 8-row groups 1024 bytes apart (SBO); LBO unused.
//   MN-major tile: 64 x 64 boxes [k][mn] of 8 KB; 8-k groups 1024 bytes apart (SBO), the next 64 mn 8192 bytes on (LBO).
__device__ __forceinline__ unsigned long long umma_desc(unsigned smem_addr, bool mn_major) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFF) >> 4);
    d |= (unsigned long long)(mn_major ? (8192 >> 4) : 1) << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
// Advance of the descriptor's start-address field for the next 16 k: 32 bytes inside the swizzle atom for a
// K-major tile, two 8-k groups (2048 bytes) for an MN-major tile.
constexpr unsigned A_KSTEP = G_A_MN ? (2048 >> 4) : (32 >> 4);
constexpr unsigned B_KSTEP = G_B_MN ? (2048 >> 4) : (32 >> 4);

// Instruction descriptor: D fp32 (bits 4-5 = 1), A and B bf16 (bits 7-9, 10-12 = 1), bit 15 / 16 = A / B is MN-major,
// N / 8 in bits 17-22, M / 16 in bits 24-28 (M = 128 per CTA: 256 for a pair).
constexpr unsigned IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)G_A_MN << 15) | ((unsigned)G_B_MN << 16) |
                           ((unsigned)(BN >> 3) << 17) | ((unsigned)((BM * CG) >> 4) << 24);

__device__ __forceinline__ void umma(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned accumulate) {
#if G_CTA_GROUP == 2
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(IDESC), "r"(accumulate) : "memory");
#else
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(IDESC), "r"(accumulate) : "memory");
#endif
}
// Arrives on `bar` (the same offset in both CTAs of a pair) once every MMA issued so far has completed.
__device__ __forceinline__ void umma_commit(unsigned bar) {
#if G_CTA_GROUP == 2
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((unsigned short)3) : "memory");
#else
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
#endif
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Two fp32 values rounded to nearest-even bf16, packed (lo in the low half).
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    unsigned r; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r;
}
__device__ __forceinline__ void store_bf16x4(void* p, float a, float b, float c, float d) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(a, b), pack_bf16(c, d));
}

// Tiles are walked in groups of GROUP_M tile rows so that blocks running at the same time share panels in L2.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& mb, int& nb) {
    const int per_group = GROUP_M * tiles_n;
    const int g = t / per_group;
    const int first_m = g * GROUP_M;
    const int gsz = min(GROUP_M, tiles_m - first_m);
    const int in_g = t - g * per_group;
    mb = first_m + in_g % gsz;
    nb = in_g / gsz;
}

extern "C" __global__ void __launch_bounds__(NUM_THREADS, 1)
#if G_CTA_GROUP == 2
__cluster_dims__(2, 1, 1)
#endif
G_KERNEL_NAME(const __grid_constant__ TensorMap map_a, const __grid_constant__ TensorMap map_b,
              float* __restrict__ C, int M, int N, int num_kb, int tiles_m, int tiles_n, int* err, int* tile_counter
#if G_TMA_STORE
              , const __grid_constant__ TensorMap map_c
#endif
              G_EPI_PARAMS) {
    extern __shared__ unsigned char smem_raw[];
    const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;       // swizzled tiles need 1024-byte alignment
    unsigned char* smem = smem_raw + (base - smem_u32(smem_raw));
    const unsigned stg_base = base + STAGES * STAGE_BYTES;               // epilogue staging, 4 KB per epilogue warp
    const unsigned bars = stg_base + EPI_WARPS * STG_BYTES;              // 8-byte mbarriers
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
    auto sfull_bar = [&](int q) { return bars + 8u * (2 * STAGES + 4 + q); };
    auto sempty_bar = [&](int q) { return bars + 8u * (2 * STAGES + 4 + SCHED + q); };
    unsigned char* misc = smem + STAGES * STAGE_BYTES + EPI_WARPS * STG_BYTES + 8 * (2 * STAGES + 4 + 2 * SCHED);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(misc);
    Shared& sh = *reinterpret_cast<Shared*>(misc + 16);
    volatile int* sched_tile = reinterpret_cast<volatile int*>(misc + 48);      // SCHED slots; -1 = no tiles left

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_rank();                                  // 0 = leader of the pair
    const unsigned peer = rank ^ 1u;
    const int num_tiles = tiles_m * tiles_n;
    // The first tile of every CTA (pair) is its own index: nobody waits for the scheduler before the first load.  Later
    // tiles come from the counter, offset by the number of CTAs (pairs).  With no more tiles than CTAs (pairs) there is
    // no later tile and the scheduler (its atomics, its slot ring and the round trip that tells every role to stop) is
    // left out altogether.
    const int groups = (int)(gridDim.x / CG);
    const int first_tile = (int)(blockIdx.x / CG);
    const bool one_wave = num_tiles <= groups;

    if (threadIdx.x == 0) {
        sh.abort_flag = 0;
        sh.abort_peer = in_cta(smem_u32((const void*)&sh.abort_flag), CG == 2 ? peer : 0u);
        sh.err = err;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), CG); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), EPI_WARPS * CG); }
        // a schedule slot is read by the leader's MMA lane and epilogue warps and, in a pair, by the other CTA's
        // producer lane and epilogue warps
        for (int q = 0; q < SCHED; ++q) { mbar_init(sfull_bar(q), 1); mbar_init(sempty_bar(q), 1 + EPI_WARPS + (CG - 1) * (1 + EPI_WARPS)); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        // each CTA allocates all 512 columns of its own tensor memory (one CTA per SM: the base is column 0 in both)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
#if G_CTA_GROUP == 2
    // both CTAs' barriers must exist before either side signals the other
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
#else
    __syncthreads();
#endif
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer (one lane per CTA)
        if (lane == 0) {
            int s = 0; unsigned phase = 0;
            int q = 0; unsigned qphase = 0;
            bool ok = true;
#if G_CTA_GROUP == 2
            if (rank == 0) {
                unsigned other;
                asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(other) : "r"(in_cta(smem_u32(tmem_slot), 1u)) : "memory");
                if (other != tmem_base) { raise_abort(sh, 8); ok = false; }   // the pair must see one accumulator address
            }
#endif
            for (int it = 0; ok; ++it) {
                int t;
                if (it == 0) t = first_tile;
                else if (one_wave) break;
                else if (rank == 0) {
                    if (!mbar_wait<true>(sempty_bar(q), qphase ^ 1u, sh, 5)) break;
                    t = groups + atomicAdd(tile_counter, 1);
                    if (t >= num_tiles) {
                        // Every leader draws exactly one index past the end; the one that draws the last leaves the
                        // counter pair zeroed for the next launch on the stream.
                        t = -1;
                        if (atomicAdd(tile_counter + 1, 1) == (int)(gridDim.x / CG) - 1) { tile_counter[1] = 0; __threadfence(); atomicExch(tile_counter, 0); }
                    }
                    sched_tile[q] = t;
#if G_CTA_GROUP == 2
                    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(in_cta(smem_u32((const void*)&sched_tile[q]), 1u)), "r"(t) : "memory");
                    mbar_arrive_release_cluster(in_cta(sfull_bar(q), 1u));
#endif
                    mbar_arrive_release_cluster(in_cta(sfull_bar(q), 0u));
                    if (++q == SCHED) { q = 0; qphase ^= 1u; }
                } else {
                    if (!mbar_wait<true>(sfull_bar(q), qphase, sh, 5)) break;
                    t = sched_tile[q];
                    mbar_arrive_release_cluster(in_cta(sempty_bar(q), 0u));
                    if (++q == SCHED) { q = 0; qphase ^= 1u; }
                }
                if (t < 0) break;
                int mb, nb; tile_coords(t, tiles_m, tiles_n, mb, nb);
                const int m0 = mb * (BM * CG) + (int)rank * BM;            // first row of A this CTA loads
                const int n0 = nb * BN + (int)rank * BNC;                 // first column of B this CTA loads
                for (int kb = 0; kb < num_kb && ok; ++kb) {
                    ok = mbar_wait(empty_bar(s), phase ^ 1u, sh, 1);
                    if (!ok) break;
                    const unsigned fb = in_cta(full_bar(s), 0u);          // the leader's barrier counts both CTAs' bytes
                    mbar_expect_tx(fb, STAGE_BYTES);
                    const unsigned sa = base + s * STAGE_BYTES, sb = sa + A_BYTES;
#if G_A_MN
                    tma_load_2d(sa, &map_a, fb, m0, kb * BK);
                    tma_load_2d(sa + 8192, &map_a, fb, m0 + 64, kb * BK);
#else
                    tma_load_2d(sa, &map_a, fb, kb * BK, m0);
#endif
#if G_B_MN
                    #pragma unroll
                    for (int j = 0; j < BNC / 64; ++j) tma_load_2d(sb + j * 8192, &map_b, fb, n0 + 64 * j, kb * BK);
#else
                    tma_load_2d(sb, &map_b, fb, kb * BK, n0);
#endif
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
            }
            // Tail: every stage this lane filled has been read by the MMAs (and their completion signals have landed in
            // this CTA) before the block may leave.
            for (int i = 0; i < STAGES && ok; ++i) {
                ok = mbar_wait(empty_bar(s), phase ^ 1u, sh, 1);
                if (++s == STAGES) { s = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            int s = 0; unsigned phase = 0;
            int q = 0; unsigned qphase = 0;
            for (int it = 0;; ++it) {
                int t = first_tile;
                if (it > 0) {
                    if (one_wave) break;
                    if (!mbar_wait<true>(sfull_bar(q), qphase, sh, 6)) break;
                    t = sched_tile[q];
                    mbar_arrive_release_cluster(in_cta(sempty_bar(q), 0u));
                    if (++q == SCHED) { q = 0; qphase ^= 1u; }
                }
                if (t < 0) break;
                const int a = it & 1;
                const unsigned aphase = (unsigned)(it >> 1) & 1u;
                if (!mbar_wait(tempty_bar(a), aphase ^ 1u, sh, 2)) break;
                tc_fence_after();
                const unsigned tmem_d = tmem_base + (unsigned)(a * BN);
                bool ok = true;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(full_bar(s), phase, sh, 3);
                    if (!ok) break;
                    tc_fence_after();
                    const unsigned long long da = umma_desc(base + s * STAGE_BYTES, G_A_MN);
                    const unsigned long long db = umma_desc(base + s * STAGE_BYTES + A_BYTES, G_B_MN);
                    #pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma(tmem_d, da + (unsigned long long)(k * A_KSTEP), db + (unsigned long long)(k * B_KSTEP), (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(empty_bar(s));                // frees the stage (in both CTAs) once these MMAs have read it
                    if (++s == STAGES) { s = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(tfull_bar(a));                    // accumulator complete (signalled in both CTAs)
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2 ..)
        const int quarter = warp & 3;                         // TMEM lanes 32*quarter .. 32*quarter+31 (fixed by the warp index)
        const int sub = (warp - 2) >> 2;                      // which of the EPI_WPQ warps of this quarter
        const unsigned stg = stg_base + (unsigned)(warp - 2) * STG_BYTES;
        const int cq = lane & 7, rsub = lane >> 3;            // read-back: 8 lanes x 16 bytes per row, 4 rows per instruction
        G_EPI_INIT
#if G_TMA_STORE
        int nstore = 0;
#endif
        int q = 0; unsigned qphase = 0;
        for (int it = 0;; ++it) {
            int t = first_tile;
            if (it > 0) {
                if (one_wave) break;
                bool got = mbar_wait<true>(sfull_bar(q), qphase, sh, 7);
                got = __all_sync(0xffffffffu, got);
                if (!got) break;
                t = sched_tile[q];
                __syncwarp();                                 // every lane has read the slot
                if (lane == 0) mbar_arrive_release_cluster(in_cta(sempty_bar(q), 0u));
                if (++q == SCHED) { q = 0; qphase ^= 1u; }
            }
            if (t < 0) break;
            int mb, nb; tile_coords(t, tiles_m, tiles_n, mb, nb);
            const int a = it & 1;
            const unsigned aphase = (unsigned)(it >> 1) & 1u;
            bool ok = mbar_wait(tfull_bar(a), aphase, sh, 4);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row0 = mb * (BM * CG) + (int)rank * BM + quarter * 32;
#if G_TMA_STORE
            // Plain store of the product: the 32 x 32 chunk goes from the swizzled staging buffer to C as one TMA store
            // (the tensor map clips the M and N tails); two buffers per warp, so the store of a chunk drains while the
            // next one is read from tensor memory.  The SM's ordinary store path is about half as fast.
            #pragma unroll 1
            for (int c = sub; c < BN / 32; c += EPI_WPQ) {
                const int col0 = nb * BN + c * 32;
                if (col0 >= N) break;                         // uniform for the warp
                const unsigned sbuf = stg + (unsigned)(nstore & 1) * 4096u;
                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");   // the store before last has read this buffer
                __syncwarp();
                unsigned r[32];
                tmem_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(a * BN + c * 32), r);
                #pragma unroll
                for (int i = 0; i < 8; ++i)
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sbuf + (unsigned)lane * 128u + (unsigned)((i ^ (lane & 7)) << 4)),
                                 "r"(r[4 * i]), "r"(r[4 * i + 1]), "r"(r[4 * i + 2]), "r"(r[4 * i + 3]) : "memory");
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0 && row0 < M) {
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                                 ::"l"(&map_c), "r"(col0), "r"(row0), "r"(sbuf) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                ++nstore;
            }
#else
            #pragma unroll 1
            for (int c = sub; c < BN / 32; c += EPI_WPQ) {
                const int col0 = nb * BN + c * 32;
                if (col0 >= N) break;                         // uniform for the warp
                unsigned r[32];
                tmem_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(a * BN + c * 32), r);
                #pragma unroll
                for (int i = 0; i < 8; ++i)
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stg + (unsigned)lane * 128u + (unsigned)((i ^ (lane & 7)) << 4)),
                                 "r"(r[4 * i]), "r"(r[4 * i + 1]), "r"(r[4 * i + 2]), "r"(r[4 * i + 3]) : "memory");
                __syncwarp();
                const int gcol = col0 + 4 * cq;
                G_EPI_COLS
                #pragma unroll EPI_UNROLL
                for (int p = 0; p < 8; ++p) {
                    const int rl = 4 * p + rsub;
                    const int grow = row0 + rl;
                    float4 acc;
                    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(acc.x), "=f"(acc.y), "=f"(acc.z), "=f"(acc.w)
                                 : "r"(stg + (unsigned)rl * 128u + (unsigned)((cq ^ (rl & 7)) << 4)) : "memory");
                    G_EPI_PRE
                    if (grow < M && gcol < N) {
                        G_EPI_BODY
                    }
                }
                G_EPI_END
                __syncwarp();                                 // the staging buffer is rewritten by the next chunk
            }
#endif
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(in_cta(tempty_bar(a), 0u));
        }
#if G_TMA_STORE
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");    // every store of this warp has landed
#endif
    }

    // ------------------------------------------------------------------ teardown
    __syncwarp();
    if (sh.abort_flag) {                   // let copies that are still in flight land before the block goes away
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) { }
    }
    tc_fence_before();
#if G_CTA_GROUP == 2
    // neither CTA leaves while the other may still signal one of its barriers or read its operand tiles
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
#else
    __syncthreads();
#endif
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}
)GEMMTPL"
