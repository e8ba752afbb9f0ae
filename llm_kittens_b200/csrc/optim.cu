// Optimizer-side kernels: squared gradient norm, clip coefficient, AdamW with stochastic rounding and
// optional fp32 master weights, master -> bf16 re-materialisation, all driven by a SEGMENT TABLE.
//
// A segment is one contiguous run of elements that this rank updates: with ZeRO >= 1 the rank owns,
// for every tensor and every layer slice, the r-th of P equal parts, so its share of the model is a
// list of (parameter offset, gradient offset, state offset, length, flags) tuples rather than one
// range. The table lives on the device as int64[nseg][5]; blockIdx.y walks segments, blockIdx.x
// strides inside one. Counterparts in the reference: adamw_update / init_from_master
// (llmc/adamw.cuh:113-171), global_norm_squared (llmc/global_norm.cuh:77-101); the reference
// launches one kernel per tensor from a host loop (train_gpt2.cu:1283-1348), here one launch covers
// the whole shard.
#include "common.cuh"

namespace llmk {
namespace optim {

constexpr int TPB = 256;
constexpr int SEG_FIELDS = 5;  // p_off, g_off, s_off, len, flags(bit0 = weight decay)

template <typename G>
__device__ __forceinline__ float load_grad(const G* g, size_t i);
template <>
__device__ __forceinline__ float load_grad<bf16>(const bf16* g, size_t i) { return __bfloat162float(g[i]); }
template <>
__device__ __forceinline__ float load_grad<float>(const float* g, size_t i) { return g[i]; }

// four consecutive gradients (8- or 16-byte aligned loads)
template <typename G>
__device__ __forceinline__ void load_grad4(const G* g, size_t i, float* out);
template <>
__device__ __forceinline__ void load_grad4<bf16>(const bf16* g, size_t i, float* out) {
    const uint2 raw = *reinterpret_cast<const uint2*>(g + i);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
}
template <>
__device__ __forceinline__ void load_grad4<float>(const float* g, size_t i, float* out) {
    const float4 r = *reinterpret_cast<const float4*>(g + i);
    out[0] = r.x; out[1] = r.y; out[2] = r.z; out[3] = r.w;
}

// partials[blockIdx.y * gridDim.x + blockIdx.x] = sum of squares of this block's elements
template <typename G>
__global__ void __launch_bounds__(TPB)
norm2_kernel(float* __restrict__ partials, const G* __restrict__ grads, const long long* __restrict__ segs) {
    __shared__ float sh[32];
    const long long* seg = segs + (size_t)blockIdx.y * SEG_FIELDS;
    const size_t g_off = (size_t)seg[1], len = (size_t)seg[3];
    float acc = 0.f;
    // four elements per thread and iteration (offsets and lengths are multiples of 4 by construction)
    for (size_t i = ((size_t)blockIdx.x * TPB + threadIdx.x) * 4; i < len; i += (size_t)gridDim.x * TPB * 4) {
        float g4[4];
        load_grad4<G>(grads, g_off + i, g4);
        acc += g4[0] * g4[0] + g4[1] * g4[1] + g4[2] * g4[2] + g4[3] * g4[3];
    }
    acc = block_sum(acc, sh);
    if (threadIdx.x == 0) partials[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = acc;
}

// out[0] = sum(partials) in fixed order
__global__ void sum_partials_kernel(float* __restrict__ out, const float* __restrict__ partials, int n) {
    __shared__ float sh[32];
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += partials[i];
    s = block_sum(s, sh);
    if (threadIdx.x == 0) out[0] = s;
}

// scale_out[0] = min(1, clip / sqrt(norm2)) ; norm_out[0] = sqrt(norm2). A non-finite norm gives scale 0
// and raises flag_out[0]; the AdamW kernels skip their update when they read that zero.
__global__ void clip_scale_kernel(float* scale_out, float* norm_out, int* flag_out, const float* norm2, float clip) {
    const float n2 = norm2[0];
    const float n = sqrtf(n2);
    norm_out[0] = n;
    if (!isfinite(n)) {
        scale_out[0] = 0.f;
        if (flag_out) flag_out[0] = 1;
    } else {
        scale_out[0] = (clip > 0.f && n > clip) ? clip / n : 1.0f;
        if (flag_out) flag_out[0] = 0;
    }
}

struct AdamArgs {
    float lr, beta1, beta2, beta1_corr, beta2_corr, eps, wd;
    unsigned int seed;
};

template <typename G>
__global__ void __launch_bounds__(TPB)
adamw_kernel(bf16* __restrict__ params, float* __restrict__ master, const G* __restrict__ grads, float* __restrict__ m,
             float* __restrict__ v, const long long* __restrict__ segs, const float* __restrict__ grad_scale_ptr,
             float grad_scale_host, AdamArgs a) {
    const long long* seg = segs + (size_t)blockIdx.y * SEG_FIELDS;
    const size_t p_off = (size_t)seg[0], g_off = (size_t)seg[1], s_off = (size_t)seg[2], len = (size_t)seg[3];
    const float wd = (seg[4] & 1) ? a.wd : 0.f;
    const float gs = grad_scale_ptr ? grad_scale_ptr[0] * grad_scale_host : grad_scale_host;
    // the clip kernel writes scale 0 only for a non-finite gradient norm (0 * inf would poison m, v and the
    // weights): such a step leaves the optimizer state and the parameters as they are
    if (grad_scale_ptr && grad_scale_ptr[0] == 0.f) return;
    const float inv_b1c = 1.0f / a.beta1_corr, inv_b2c = 1.0f / a.beta2_corr;
    // four elements per thread and iteration: 8-byte bf16 and 16-byte fp32 accesses
    for (size_t i = ((size_t)blockIdx.x * TPB + threadIdx.x) * 4; i < len; i += (size_t)gridDim.x * TPB * 4) {
        float g4[4], old4[4], p4[4];
        load_grad4<G>(grads, g_off + i, g4);
        float4 m4 = *reinterpret_cast<const float4*>(m + s_off + i);
        float4 v4 = *reinterpret_cast<const float4*>(v + s_off + i);
        float mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
        if (master) {
            const float4 o = *reinterpret_cast<const float4*>(master + s_off + i);
            old4[0] = o.x; old4[1] = o.y; old4[2] = o.z; old4[3] = o.w;
        } else {
            load_grad4<bf16>(params, p_off + i, old4);
        }
        __align__(8) __nv_bfloat16 out[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float g = gs * g4[j];
            mm[j] = a.beta1 * mm[j] + (1.0f - a.beta1) * g;
            vv[j] = a.beta2 * vv[j] + (1.0f - a.beta2) * g * g;
            const float mh = mm[j] * inv_b1c, vh = vv[j] * inv_b2c;
            p4[j] = old4[j] - a.lr * (mh / (sqrtf(vh) + a.eps) + wd * old4[j]);
            // the rounding noise is keyed on the element's index in the full parameter arena, so every
            // rank (and every sharding) rounds a given parameter the same way
            out[j] = sr_round(p4[j], squirrel5((unsigned int)(p_off + i + j), a.seed));
        }
        *reinterpret_cast<float4*>(m + s_off + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
        *reinterpret_cast<float4*>(v + s_off + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
        *reinterpret_cast<uint2*>(params + p_off + i) = *reinterpret_cast<const uint2*>(out);
        if (master) *reinterpret_cast<float4*>(master + s_off + i) = make_float4(p4[0], p4[1], p4[2], p4[3]);
    }
}

// master[s] = float(params[p])   (first step with master weights)
__global__ void __launch_bounds__(TPB)
master_from_params_kernel(float* __restrict__ master, const bf16* __restrict__ params, const long long* __restrict__ segs) {
    const long long* seg = segs + (size_t)blockIdx.y * SEG_FIELDS;
    const size_t p_off = (size_t)seg[0], s_off = (size_t)seg[2], len = (size_t)seg[3];
    for (size_t i = (size_t)blockIdx.x * TPB + threadIdx.x; i < len; i += (size_t)gridDim.x * TPB)
        master[s_off + i] = __bfloat162float(params[p_off + i]);
}
// params[p] = SR(master[s]) with the same noise the update used (bit-exact resume from master weights)
__global__ void __launch_bounds__(TPB)
params_from_master_kernel(bf16* __restrict__ params, const float* __restrict__ master, const long long* __restrict__ segs,
                          unsigned int seed) {
    const long long* seg = segs + (size_t)blockIdx.y * SEG_FIELDS;
    const size_t p_off = (size_t)seg[0], s_off = (size_t)seg[2], len = (size_t)seg[3];
    for (size_t i = (size_t)blockIdx.x * TPB + threadIdx.x; i < len; i += (size_t)gridDim.x * TPB)
        params[p_off + i] = sr_round(master[s_off + i], squirrel5((unsigned int)(p_off + i), seed));
}

static inline int grid_x_for(long max_len) {
    long g = (max_len + TPB * 4 - 1) / (TPB * 4);
    if (g > 1024) g = 1024;
    if (g < 1) g = 1;
    return (int)g;
}

}  // namespace optim
}  // namespace llmk

using namespace llmk;
using namespace llmk::optim;

// Grid x-extent used for a table whose longest segment has `max_len` elements.
LLMK_API int llmk_optim_grid_x(long max_len) { return grid_x_for(max_len); }

// norm2_out[0] = sum over the table's segments of grad^2; partials needs nseg * llmk_optim_grid_x(max_len) floats.
LLMK_API int llmk_global_norm2(void* norm2_out, void* partials, const void* grads, int grads_fp32, const void* segs, int nseg,
                               long max_len, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (nseg <= 0) return LLMK_ERR_SHAPE;
    const int gx = grid_x_for(max_len);
    dim3 grid(gx, nseg);
    if (grads_fp32) norm2_kernel<float><<<grid, TPB, 0, stream>>>((float*)partials, (const float*)grads, (const long long*)segs);
    else norm2_kernel<bf16><<<grid, TPB, 0, stream>>>((float*)partials, (const bf16*)grads, (const long long*)segs);
    LLMK_LAUNCH_CHECK();
    sum_partials_kernel<<<1, 1024, 0, stream>>>((float*)norm2_out, (const float*)partials, gx * nseg);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

LLMK_API int llmk_clip_scale(void* scale_out, void* norm_out, void* flag_out, const void* norm2, float clip, void* stream) {
    clip_scale_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((float*)scale_out, (float*)norm_out, (int*)flag_out, (const float*)norm2,
                                                         clip);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

LLMK_API int llmk_adamw(void* params, void* master, const void* grads, int grads_fp32, void* m, void* v, const void* segs,
                        int nseg, long max_len, float lr, float beta1, float beta2, float beta1_corr, float beta2_corr,
                        float eps, float wd, const void* grad_scale_ptr, float grad_scale_host, unsigned int seed,
                        void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (nseg <= 0) return LLMK_ERR_SHAPE;
    AdamArgs a{lr, beta1, beta2, beta1_corr, beta2_corr, eps, wd, seed};
    dim3 grid(grid_x_for(max_len), nseg);
    if (grads_fp32)
        adamw_kernel<float><<<grid, TPB, 0, stream>>>((bf16*)params, (float*)master, (const float*)grads, (float*)m, (float*)v,
                                                      (const long long*)segs, (const float*)grad_scale_ptr, grad_scale_host, a);
    else
        adamw_kernel<bf16><<<grid, TPB, 0, stream>>>((bf16*)params, (float*)master, (const bf16*)grads, (float*)m, (float*)v,
                                                     (const long long*)segs, (const float*)grad_scale_ptr, grad_scale_host, a);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

LLMK_API int llmk_master_from_params(void* master, const void* params, const void* segs, int nseg, long max_len, void* stream) {
    dim3 grid(grid_x_for(max_len), nseg);
    master_from_params_kernel<<<grid, TPB, 0, (cudaStream_t)stream>>>((float*)master, (const bf16*)params, (const long long*)segs);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_params_from_master(void* params, const void* master, const void* segs, int nseg, long max_len,
                                     unsigned int seed, void* stream) {
    dim3 grid(grid_x_for(max_len), nseg);
    params_from_master_kernel<<<grid, TPB, 0, (cudaStream_t)stream>>>((bf16*)params, (const float*)master,
                                                                     (const long long*)segs, seed);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
