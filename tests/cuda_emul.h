// TEST INFRASTRUCTURE: runs the generated CUDA C kernels on the CPU so the scheduler and the code
// generator can be checked against the oracle on a machine without a GPU.  One OS thread per CUDA
// thread, blocks executed one after the other.  Only the constructs the code generator emits are
// provided; every warp shuffle is executed by all threads of the block at the same program point
// (the generator guarantees it), so shuffles and __syncthreads share one block-wide barrier.
#pragma once
#include <pthread.h>

#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

struct float4 { float x, y, z, w; };
static inline float4 make_float4(float x, float y, float z, float w) { float4 r = {x, y, z, w}; return r; }
struct emul_dim3 { unsigned x, y, z; };

static thread_local emul_dim3 threadIdx, blockIdx;
static emul_dim3 blockDim, gridDim;
static pthread_barrier_t emul_barrier;
static float emul_slots[1024];

#define __global__
#define __device__
#define __forceinline__ inline
#define __launch_bounds__(...)
#define __shared__ static

static inline float __fadd_rn(float a, float b) { return a + b; }
static inline float __fsub_rn(float a, float b) { return a - b; }
static inline float __fmul_rn(float a, float b) { return a * b; }
static inline float __fmaf_rn(float a, float b, float c) { return fmaf(a, b, c); }
static inline float __int_as_float(unsigned int v) { float f; std::memcpy(&f, &v, 4); return f; }
static inline unsigned __float_as_uint(float f) { unsigned v; std::memcpy(&v, &f, 4); return v; }
struct uint2 { unsigned x, y; };
static inline uint2 make_uint2(unsigned x, unsigned y) { uint2 r = {x, y}; return r; }
static inline float __fdiv_rn(float a, float b) { return a / b; }
static inline float __frcp_rn(float a) { return 1.0f / a; }
static inline float __frsqrt_rn(float a) { return (float)(1.0 / sqrt((double)a)); }
static inline void __syncthreads() { pthread_barrier_wait(&emul_barrier); }
static inline float __shfl_xor_sync(unsigned, float v, int lane_mask) {
    unsigned t = threadIdx.x;
    emul_slots[t] = v;
    pthread_barrier_wait(&emul_barrier);
    float r = emul_slots[(t & ~31u) | ((t ^ (unsigned)lane_mask) & 31u)];
    pthread_barrier_wait(&emul_barrier);
    return r;
}

// ---- the staged (bulk asynchronous copy) row kernels: the copy happens at once, the barrier wait is a block barrier
#include <cstring>
#define ORMI_DYN_SMEM(name) static unsigned char name[512 * 1024]
static int emul_or_flag;
static inline int __syncthreads_or(int pred) {
    if (pred) __atomic_store_n(&emul_or_flag, 1, __ATOMIC_SEQ_CST);
    pthread_barrier_wait(&emul_barrier);
    int r = __atomic_load_n(&emul_or_flag, __ATOMIC_SEQ_CST);
    pthread_barrier_wait(&emul_barrier);
    if (threadIdx.x == 0) __atomic_store_n(&emul_or_flag, 0, __ATOMIC_SEQ_CST);
    pthread_barrier_wait(&emul_barrier);
    return r;
}
static inline int atomicExch(int* p, int v) { return __atomic_exchange_n(p, v, __ATOMIC_SEQ_CST); }
static inline int atomicAdd(int* p, int v) { return __atomic_fetch_add(p, v, __ATOMIC_SEQ_CST); }
static inline void __threadfence() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
static inline void ormi_mbar_init(unsigned long long*, unsigned) {}
static inline void ormi_mbar_fence_init() {}
static inline void ormi_async_fence() {}
static inline void ormi_mbar_expect(unsigned long long*, unsigned) {}
static inline void ormi_bulk_load(void* dst, const void* src, unsigned bytes, unsigned long long*) { std::memcpy(dst, src, bytes); }
static inline bool ormi_mbar_wait(unsigned long long*, unsigned) { pthread_barrier_wait(&emul_barrier); return true; }
static inline void ormi_drain() {}

typedef void (*emul_kernel_t)(void*, void*, void*, void*, void*, void*, void*, void*, void*, void*, void*, void*,
                              void*, void*, void*, void*, void*, void*, void*, void*, void*, void*, void*, void*);

extern "C" int emul_launch(void* fn, int grid, int block, void** args, int nargs) {
    if (nargs > 24 || block > 1024) return 1;
    void* a[24] = {0};
    for (int i = 0; i < nargs; ++i) a[i] = args[i];
    pthread_barrier_init(&emul_barrier, nullptr, (unsigned)block);
    gridDim = {(unsigned)grid, 1, 1};
    blockDim = {(unsigned)block, 1, 1};
    emul_kernel_t k = (emul_kernel_t)fn;
    std::vector<std::thread> threads;
    for (int t = 0; t < block; ++t) {
        threads.emplace_back([=] {
            for (int b = 0; b < grid; ++b) {
                threadIdx = {(unsigned)t, 0, 0};
                blockIdx = {(unsigned)b, 0, 0};
                k(a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], a[8], a[9], a[10], a[11], a[12], a[13], a[14], a[15],
                  a[16], a[17], a[18], a[19], a[20], a[21], a[22], a[23]);
                pthread_barrier_wait(&emul_barrier);
            }
        });
    }
    for (auto& th : threads) th.join();
    pthread_barrier_destroy(&emul_barrier);
    return 0;
}
