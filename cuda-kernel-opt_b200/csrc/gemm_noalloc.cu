// Split-K GEMM for callers that must not allocate device memory.
//
// The split-K form of the GEMM writes one fp32 partial product per K slice into scratch memory
// and then sums the slices. The regular entry points take that scratch from the caller. Some
// callers cannot provide it: code that runs inside a region where cudaMalloc is forbidden or
// would synchronise the device (a latency-critical serving loop, a callback running under
// another library's allocator lock, a plugin whose host hands it fixed buffers only). For them
// the scratch lives here, in a file-scope device array that every GPU loading this library holds
// from load to exit.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/b200_gemm.h"
#include "gemm_sm100.cuh"

namespace {

// 32 MiB of scratch: split_k * M * N fp32 values must fit (for example 2 slices of 2048 x 2048).
constexpr size_t kScratchFloats = size_t(8) << 20;
static __device__ __align__(256) float g_splitk_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
float *g_scratch_ptr[kMaxDevices];  // device address of the array on each device, 0 until set up
std::mutex g_setup_mutex;

// In host code the array's name is only a handle for the runtime, not a device address; the
// address on the current device comes from cudaGetSymbolAddress. Done once per device, with that
// device current.
int scratch_address(float **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return b200::record_cuda_error(static_cast<int>(e));
    if (dev < 0 || dev >= kMaxDevices) return B200_UNSUPPORTED_DEVICE;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ptr[dev]) {
        float *ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_splitk_scratch);
        if (e != cudaSuccess || !ptr) return b200::record_cuda_error(static_cast<int>(e != cudaSuccess ? e : cudaErrorUnknown));
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return B200_OK;
}

}  // namespace

extern "C" int b200_gemm_splitk_noalloc(int dtype, const void *A, const void *Bt, const float *C, float *D, float alpha,
                                        float beta, int64_t M, int64_t N, int64_t K, const b200_gemm_params *p,
                                        void *stream) {
    if (!p || p->split_k < 2) return B200_INVALID_CONFIG;  // without a K split no scratch is needed: use b200_gemm_*
    if (M <= 0 || N <= 0 || M > (int64_t(1) << 30) || N > (int64_t(1) << 30)) return B200_INVALID_SHAPE;
    if (p->split_k > 64) return B200_INVALID_CONFIG;   // the product below cannot wrap: 2^6 * 2^30 * 2^30
    const size_t need = static_cast<size_t>(p->split_k) * static_cast<size_t>(M) * static_cast<size_t>(N);
    if (need > kScratchFloats) return B200_WORKSPACE_TOO_SMALL;  // beyond the built-in 32 MiB: pass your own workspace
    float *scratch = nullptr;
    const int st = scratch_address(&scratch);
    if (st != B200_OK) return st;
    if (dtype == B200_BF16)
        return b200_gemm_bf16(A, Bt, C, D, alpha, beta, M, N, K, p, scratch, kScratchFloats * sizeof(float), stream);
    if (dtype == B200_F16)
        return b200_gemm_f16(A, Bt, C, D, alpha, beta, M, N, K, p, scratch, kScratchFloats * sizeof(float), stream);
    return B200_INVALID_CONFIG;
}
