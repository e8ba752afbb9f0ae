// Shared device/host helpers for every kernel translation unit of the library.
//
// Conventions
//   * activations / parameters / gradients are bf16 ("floatX"), statistics and optimizer state fp32;
//   * every exported function is `extern "C"`, takes raw device pointers plus a `void* stream`
//     (a cudaStream_t) and returns 0 on success or a negative LLMK_ERR_* code: nothing here throws,
//     aborts or calls exit(), so a Python caller can always report the failure;
//   * kernels that wait on something (an mbarrier, a peer flag) use bounded waits and record a
//     non-zero code in a caller-provided `int status[4]` word instead of trapping.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LLMK_API extern "C" __attribute__((visibility("default")))

// ---- error codes returned by host launchers -------------------------------------------------
#define LLMK_OK 0
#define LLMK_ERR_CUDA -1        // a CUDA runtime call failed (see llmk_last_error)
#define LLMK_ERR_SHAPE -2       // unsupported / misaligned shape
#define LLMK_ERR_TMAP -3        // cuTensorMapEncodeTiled failed
#define LLMK_ERR_WORKSPACE -4   // workspace too small
#define LLMK_ERR_DRIVER -5      // driver entry point not found
#define LLMK_ERR_LIMIT -6       // size beyond a compiled-in maximum

// ---- codes written by kernels into status[0] ------------------------------------------------
#define LLMK_ST_OK 0
#define LLMK_ST_TIMEOUT_TMA_FULL 1    // MMA warp never saw a filled pipeline stage
#define LLMK_ST_TIMEOUT_TMA_EMPTY 2   // producer never saw a stage released
#define LLMK_ST_TIMEOUT_ACC_FULL 3    // epilogue never saw an accumulator
#define LLMK_ST_TIMEOUT_ACC_EMPTY 4   // MMA warp never got an accumulator back
#define LLMK_ST_TIMEOUT_PEER 5        // a peer-flag wait ran out
#define LLMK_ST_BOUNDS 6              // a debug bounds check failed (index recorded in status[2..3])

namespace llmk {

typedef __nv_bfloat16 bf16;

// host: remembers the text of the last CUDA error seen by a launcher of this library
void set_last_error(const char* what, cudaError_t e);
int* current_status_word();   // device pointer registered with llmk_set_status_word for the current device, or nullptr

#define LLMK_CUDA_TRY(expr)                                  \
    do {                                                     \
        cudaError_t _e = (expr);                             \
        if (_e != cudaSuccess) {                             \
            ::llmk::set_last_error(#expr, _e);               \
            return LLMK_ERR_CUDA;                            \
        }                                                    \
    } while (0)

#define LLMK_LAUNCH_CHECK() LLMK_CUDA_TRY(cudaGetLastError())

static inline int ceil_div(long a, long b) { return (int)((a + b - 1) / b); }

// Function attributes (opt-in shared memory, carve-out) and device properties belong to a DEVICE, while a
// launcher's `static` lives once per process: a process that drives several GPUs has to configure each of
// them. `first()` is true once per device (the device current at the call), so the usual
// `static PerDeviceOnce once; if (once.first()) { cudaFuncSetAttribute(...); }` configures every device it meets.
constexpr int LLMK_MAX_DEVICES = 64;
struct PerDeviceOnce {
    bool done[LLMK_MAX_DEVICES] = {};
    bool first() {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= LLMK_MAX_DEVICES) return true;   // unknown: configure again
        if (done[dev]) return false;
        done[dev] = true;
        return true;
    }
};

// multiprocessor count of the current device (cached per device)
static inline int sm_count_current_device() {
    static int sms[LLMK_MAX_DEVICES] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= LLMK_MAX_DEVICES) return 0;
    if (sms[dev] == 0 && cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms[dev] = 0;
    return sms[dev];
}

// ---- 128-bit packed access -------------------------------------------------------------------
struct alignas(16) bf16x8 {
    __nv_bfloat162 v[4];
};

__device__ __forceinline__ bf16x8 ld128(const bf16* p) { return *reinterpret_cast<const bf16x8*>(p); }
__device__ __forceinline__ bf16x8 ld128_stream(const bf16* p) {
    int4 r = __ldcs(reinterpret_cast<const int4*>(p));
    return *reinterpret_cast<bf16x8*>(&r);
}
__device__ __forceinline__ void st128(bf16* p, const bf16x8& v) { *reinterpret_cast<bf16x8*>(p) = v; }
__device__ __forceinline__ void st128_stream(bf16* p, const bf16x8& v) {
    __stcs(reinterpret_cast<int4*>(p), *reinterpret_cast<const int4*>(&v));
}
__device__ __forceinline__ void unpack8(const bf16x8& v, float* f) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float2 t = __bfloat1622float2(v.v[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ bf16x8 pack8(const float* f) {
    bf16x8 r;
#pragma unroll
    for (int i = 0; i < 4; i++) r.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return r;
}

// ---- reductions --------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Block-wide sum; every thread of the block must call it (no divergent exits). `sh` holds >= 32 floats.
__device__ __forceinline__ float block_sum(float v, float* sh) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    float r = (lane < nw) ? sh[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* sh) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    float r = (lane < nw) ? sh[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

// ---- activation math (tanh-GELU as used by GPT-2) -------------------------------------------------
__device__ __forceinline__ float fast_tanh(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
#define LLMK_GELU_K 0.7978845608028654f  // sqrt(2/pi)
#define LLMK_GELU_KC (0.7978845608028654f * 0.044715f)
// tanh.approx.f32 (one MUFU op, ~2^-11 relative error) is used by the fused GEMM epilogues and by the
// stand-alone kernels alike, so a recomputed activation equals the one the forward pass produced. The GEMM
// epilogues evaluate the same formulas two values at a time with packed fp32 instructions; every step below is
// an explicitly rounded multiply / FMA in the same order as there, so both give the same bits.
//   u = x * (K + K*c*x^2);  gelu = 0.5x + 0.5x * tanh(u)
__device__ __forceinline__ float gelu_fwd(float x) {
    const float x2 = __fmul_rn(x, x);
    const float inner = __fmaf_rn(x2, LLMK_GELU_KC, LLMK_GELU_K);
    const float t = fast_tanh(__fmul_rn(x, inner));
    const float hx = __fmul_rn(x, 0.5f);
    return __fmaf_rn(hx, t, hx);
}
//   gelu' = 0.5(1+t) + 0.5x (1-t^2) u'  with u' = K + 3K*c*x^2, factored as (1+t) * (0.5 + 0.5x u' (1-t))
__device__ __forceinline__ float gelu_grad(float x) {
    const float x2 = __fmul_rn(x, x);
    const float inner = __fmaf_rn(x2, LLMK_GELU_KC, LLMK_GELU_K);
    const float t = fast_tanh(__fmul_rn(x, inner));
    const float du = __fmaf_rn(x2, 3.0f * LLMK_GELU_KC, LLMK_GELU_K);
    const float a = __fadd_rn(t, 1.0f);
    const float b = __fmaf_rn(t, -1.0f, 1.0f);
    const float w = __fmul_rn(__fmul_rn(x, 0.5f), du);
    const float z = __fmaf_rn(w, b, 0.5f);
    return __fmul_rn(a, z);
}

// ---- counter-based random bits for stochastic rounding ------------------------------------------
// SquirrelNoise5-style integer hash; (position, seed) -> 32 random bits. Stateless, so the same
// (index, seed) pair gives the same rounding decision on every rank and under any launch geometry.
__device__ __host__ __forceinline__ unsigned int squirrel5(unsigned int pos, unsigned int seed) {
    const unsigned int N1 = 0xd2a80a3fu, N2 = 0xa884f197u, N3 = 0x6c736f4bu, N4 = 0xb79f3abbu, N5 = 0x1b56c4f5u;
    unsigned int m = pos;
    m *= N1; m += seed; m ^= (m >> 9);
    m += N2; m ^= (m >> 11);
    m *= N3; m ^= (m >> 13);
    m += N4; m ^= (m >> 15);
    m *= N5; m ^= (m >> 17);
    return m;
}
// fp32 -> bf16 with stochastic rounding: add 16 random bits below the bf16 mantissa, then truncate.
__device__ __forceinline__ bf16 sr_round(float x, unsigned int rnd) {
    unsigned int bits = __float_as_uint(x);
    if ((bits & 0x7f800000u) == 0x7f800000u) return __float2bfloat16_rn(x);  // inf / nan unchanged
    bits += (rnd & 0xffffu);
    bits &= 0xffff0000u;
    return __float2bfloat16_rn(__uint_as_float(bits));
}

}  // namespace llmk
