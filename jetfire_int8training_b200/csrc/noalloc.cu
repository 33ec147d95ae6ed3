// Allocation-free variant of the residual-add + row-statistics operator.
//
// Some hosts cannot give this library a workspace: a plug-in ABI that passes an operator nothing but its inputs and
// outputs, a runtime that carves up one fixed device arena at start-up and forbids any later allocator call, or a
// latency-critical loop that must not call cudaMalloc (which synchronises the device).  For those callers this file keeps
// the operator's workspace -- the per-tile row partial sums -- in a fixed array that is part of the library image.
//
// The array lives in device memory of every GPU that loads the library, from load until the process exits.  Its name is
// only a host-side handle: host code must not pass it to a kernel.  The device address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and that address is what the kernels receive.
#include <mutex>

#include "jf_common.cuh"

namespace {

constexpr int64_t kMaxScratchFloats = 1 << 20;   // 4 MiB: 2 * M * ceil(N/128) floats must fit (e.g. M = 16384, N = 4096)
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_meanvar_scratch[kMaxScratchFloats];

std::mutex g_mutex;
float* g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the workspace on the current device; resolved on the first call per device.
int scratch_address(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        jf::g_last_cuda_error = (int)e;
        return JF_ERR_LAUNCH;
    }
    if (dev < 0 || dev >= kMaxDevices) return JF_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_meanvar_scratch);
        if (e != cudaSuccess || !p) {
            jf::g_last_cuda_error = (int)e;
            return JF_ERR_LAUNCH;
        }
        g_scratch_addr[dev] = static_cast<float*>(p);
    }
    *out = g_scratch_addr[dev];
    return JF_OK;
}

}  // namespace

extern "C" int jf_int8_add_meanvar_noalloc(const void* x1, int x1_dtype, const int8_t* q2, const void* s2, int64_t M, int64_t N,
                                           float* y1, int8_t* qy, void* sy, float* mean, float* rstd, void* stream) {
    if (M <= 0 || N <= 0 || (M % 32) || (N % 32)) return JF_ERR_SHAPE;
    const int64_t tiles_n = (N + 127) / 128;
    if (M > kMaxScratchFloats || tiles_n > kMaxScratchFloats || 2 * M * tiles_n > kMaxScratchFloats)
        return JF_ERR_SHAPE;   // beyond the built-in workspace: use jf_int8_add_meanvar with a caller-provided one
    float* scratch = nullptr;
    if (int e = scratch_address(&scratch)) return e;
    // Every (row, tile) partial is written before the finishing kernel reads it, so nothing has to be cleared.
    return jf_int8_add_meanvar(x1, x1_dtype, q2, s2, M, N, y1, qy, sy, mean, rstd, scratch, stream);
}
