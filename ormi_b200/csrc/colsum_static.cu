// Column sum of a contiguous fp32 matrix that never allocates: ormi_b200_colsum_static.
//
// For callers that must not allocate device memory at the moment they need a reduction: a process whose
// device memory has already been handed, whole, to another allocator (so a fresh cudaMalloc could fail or
// fragment it), or a steady-state loop that cannot afford the device-wide synchronisation an allocation or a
// free may imply.  The regular path (ormi_b200_sum / ormi_b200_realize) takes its per-block partials from the
// context's pool, which calls cudaMalloc on a miss; this variant keeps the partials in a fixed array that is
// part of the library image instead.
//
// Same algorithm as the column-sum output of the generated row kernels: every block adds up a slice of the
// rows for its columns in registers, writes one partial row, and a second launch adds the partial rows in
// block order (deterministic, no atomics).
//
// The scratch array
//   * is 2 MiB (524288 floats) of device memory on every GPU that loads the library, held until exit;
//   * is shared by every call: two calls that overlap on the GPU (different streams, or different host
//     threads) race on it.  Calls on one stream are safe.
//   * keeps the contents of the last call.  Nothing in it has to start at zero: stage 2 only reads the partial
//     rows that stage 1 of the same call has just written.
// The first call on a device looks the array's device address up (cudaGetSymbolAddress) with that device
// current; make that first call before any stream capture starts.  The address is remembered per device ordinal for the
// life of the process: after a cudaDeviceReset in the same process it would be stale, so do not reset a device that
// this entry point has been used on.
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>
#include <string>

#include "ormi_b200.h"

namespace {

constexpr int64_t kScratchFloats = 512 * 1024;       // 2 MiB
constexpr int kMaxPartials = 128;                    // partial rows per call (blocks along the row axis)
constexpr int64_t kMaxCols = kScratchFloats / 8;     // 65536: at least 8 partial rows always fit
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_colsum_scratch[kScratchFloats];

// In host code `g_colsum_scratch` is only a handle for the symbol, not an address a kernel can use.  The device
// address is fetched once per device and cached here.
float* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

__global__ void __launch_bounds__(256)
colsum_partials(const float* __restrict__ in, int64_t rows, int64_t cols, int parts, float* __restrict__ scratch) {
    const int64_t c = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (c >= cols) return;
    const int p = blockIdx.y;
    float acc = 0.0f;
    for (int64_t r = p; r < rows; r += parts) acc += in[r * cols + c];
    scratch[(int64_t)p * cols + c] = acc;
}

__global__ void __launch_bounds__(256)
colsum_finalize(const float* __restrict__ scratch, int64_t cols, int parts, float* __restrict__ out) {
    const int64_t c = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (c >= cols) return;
    float acc = 0.0f;
    for (int p = 0; p < parts; ++p) acc += scratch[(int64_t)p * cols + c];
    out[c] = acc;
}

}  // namespace

namespace ormi_b200 { void set_last_error(const std::string& msg); }   // the text ormi_b200_last_error() returns

namespace {
int fail(const std::string& msg) { ormi_b200::set_last_error(msg); return 1; }
}  // namespace

extern "C" int ormi_b200_colsum_static(const float* in, int64_t rows, int64_t cols, float* out, void* stream) {
    if (!in || !out) return fail("ormi_b200_colsum_static: NULL buffer");
    if (rows <= 0 || cols <= 0) return fail("ormi_b200_colsum_static: rows and cols must be positive");
    if (cols > kMaxCols)
        return fail("ormi_b200_colsum_static: " + std::to_string(cols) + " columns exceed the fixed scratch (at most " +
                    std::to_string(kMaxCols) + " columns); use ormi_b200_sum, which takes scratch from the pool");
    if (rows * cols >= (int64_t(1) << 40)) return fail("ormi_b200_colsum_static: matrix too large");
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return fail(std::string("CUDA Error: ") + cudaGetErrorString(e));
    if (device < 0 || device >= kMaxDevices) return fail("ormi_b200_colsum_static: device index out of range");
    float* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (!g_scratch_addr[device]) {          // first call on this device (it is the current one)
            float* p = nullptr;
            e = cudaGetSymbolAddress((void**)&p, g_colsum_scratch);
            if (e != cudaSuccess || !p) return fail(std::string("CUDA Error: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
            g_scratch_addr[device] = p;
        }
        scratch = g_scratch_addr[device];
    }
    int64_t parts = kScratchFloats / cols;
    if (parts > kMaxPartials) parts = kMaxPartials;
    if (parts > rows) parts = rows;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    dim3 grid1((unsigned)((cols + 255) / 256), (unsigned)parts);
    cudaGetLastError();          // an error some earlier call left behind is not this call's
    colsum_partials<<<grid1, 256, 0, s>>>(in, rows, cols, (int)parts, scratch);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(std::string("CUDA Error: colsum_partials: ") + cudaGetErrorString(e));   // the second launch is not queued
    colsum_finalize<<<(unsigned)((cols + 255) / 256), 256, 0, s>>>(scratch, cols, (int)parts, out);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(std::string("CUDA Error: colsum_finalize: ") + cudaGetErrorString(e));
    return 0;
}
