// Library-wide runtime helpers: last-error text, device queries, L2 flush for benchmarks.
#include <stdio.h>
#include <string.h>
#include "common.cuh"

namespace llmk {
static thread_local char g_last_error[512] = "";
void set_last_error(const char* what, cudaError_t e) {
    snprintf(g_last_error, sizeof(g_last_error), "%s -> %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}
// Per-device status word (int32[4] in device memory) registered by the binding layer: kernels with bounded
// waits whose C entry point has no status argument report their failures there.
static int* g_status_word[64];
int* current_status_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    return g_status_word[dev];
}
}  // namespace llmk

using namespace llmk;

LLMK_API int llmk_set_status_word(void* device_ptr) {
    int dev = 0;
    LLMK_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return LLMK_ERR_SHAPE;
    g_status_word[dev] = static_cast<int*>(device_ptr);
    return LLMK_OK;
}

LLMK_API const char* llmk_last_error() { return g_last_error; }

LLMK_API int llmk_version() { return 100; }

LLMK_API int llmk_num_sms() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    return n;
}

// Compute capability as major*10+minor of the current device (100 on B200), or -1.
LLMK_API int llmk_device_cc() {
    int dev = 0, ma = 0, mi = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&ma, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&mi, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) return -1;
    return ma * 10 + mi;
}

__global__ void fill_u32_kernel(uint32_t* p, size_t n, uint32_t v) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) p[i] = v;
}

// Overwrite `bytes` of `buf` (benchmarks pass a buffer larger than the L2 to evict it between runs).
LLMK_API int llmk_flush_l2(void* buf, long bytes, void* stream) {
    fill_u32_kernel<<<1184, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<uint32_t*>(buf), (size_t)bytes / 4,
                                                                             0u);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
