// Allocation-free LayerNorm backward: see layernorm_bwd_noalloc.h for who needs it and the rules.
//
// The partial-sum buffer that llmk_layernorm_bwd takes from its caller lives here as a static device
// array. In host code the array's name is only a handle for the runtime, not a device address, so the
// launcher asks the runtime for the real address once per device (cudaGetSymbolAddress, with that
// device current) and hands that pointer to the same kernels the allocating entry point runs.
#include <mutex>

#include "common.cuh"
#include "layernorm_bwd_noalloc.h"

namespace llmk {
namespace norm {
// implemented in norm.cu: row kernel + fixed-order reduction of the block partials found in `scratch`
int layernorm_bwd_impl(bf16* dinp, bf16* dweight, bf16* dbias, float* scratch, const bf16* dout, const bf16* inp,
                       const bf16* weight, const float* mean, const float* rstd, int N, int C, int accumulate_dinp,
                       cudaStream_t stream);
}  // namespace norm
}  // namespace llmk

namespace {

static __device__ __align__(256) float g_ln_bwd_scratch[LLMK_LN_BWD_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
float* g_scratch_addr[kMaxDevices] = {nullptr};
int g_sm_count[kMaxDevices] = {0};

// Device address of the array and SM count for the current device, resolved on first use.
int setup_current_device(float** scratch, int* sms) {
    int dev = 0;
    LLMK_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return LLMK_ERR_LIMIT;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        float* p = nullptr;
        LLMK_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_ln_bwd_scratch));
        int n = 0;
        LLMK_CUDA_TRY(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
        g_sm_count[dev] = n;
        g_scratch_addr[dev] = p;
    }
    *scratch = g_scratch_addr[dev];
    *sms = g_sm_count[dev];
    return LLMK_OK;
}

}  // namespace

LLMK_API int llmk_layernorm_bwd_noalloc(void* dinp, void* dweight, void* dbias, const void* dout, const void* inp,
                                        const void* weight, const void* mean, const void* rstd, int N, int C,
                                        int accumulate_dinp, void* stream) {
    using llmk::bf16;
    if (N <= 0 || C <= 0 || C % 8 != 0) return LLMK_ERR_SHAPE;
    float* scratch = nullptr;
    int sms = 0;
    const int rc = setup_current_device(&scratch, &sms);
    if (rc != LLMK_OK) return rc;
    // the backward launches at most 4 blocks per SM, each leaving 2 * C partial sums
    const long long needed = 4LL * sms * 2LL * C;
    if (needed > (long long)LLMK_LN_BWD_NOALLOC_SCRATCH_FLOATS) return LLMK_ERR_LIMIT;
    return llmk::norm::layernorm_bwd_impl(static_cast<bf16*>(dinp), static_cast<bf16*>(dweight), static_cast<bf16*>(dbias),
                                          scratch, static_cast<const bf16*>(dout), static_cast<const bf16*>(inp),
                                          static_cast<const bf16*>(weight), static_cast<const float*>(mean),
                                          static_cast<const float*>(rstd), N, C, accumulate_dinp,
                                          reinterpret_cast<cudaStream_t>(stream));
}
