// LayerNorm / RMSNorm forward (optionally fused with the residual add that precedes them) and
// backward, bf16 data with fp32 statistics.
//
// Same jobs as layernorm_forward / fused_residual_forward5 / layernorm_backward
// (reference llmc/layernorm.cuh:527-584) and rmsnorm_forward / fused_residual_rmsnorm_forward /
// rmsnorm_backward (llmc/rmsnorm.cuh:151-198). New design:
//   * forward: one warp per row, the row cached as bf16 in shared memory between the statistics
//     passes (fp32 mean, then centred variance) and the normalise pass; 128-bit accesses;
//   * backward: persistent blocks; each warp walks rows grid-stride, writes dinp (+=) and adds
//     its dweight/dbias contributions into a PRIVATE fp32 shared-memory accumulator (lane l owns
//     fixed columns, so no atomics); warps are summed in fixed order into one partial per block in a
//     global scratch buffer, and a second kernel sums the block partials in fixed order into the
//     bf16 gradients (+=). The result is bit-reproducible run to run.
#include "common.cuh"

namespace llmk {
namespace norm {

constexpr int FWD_WARPS = 4;
constexpr int BWD_WARPS = 4;

template <bool RMS, bool FUSED_RESIDUAL>
__global__ void __launch_bounds__(FWD_WARPS * 32)
norm_fwd_kernel(bf16* __restrict__ normed, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                bf16* __restrict__ residual_out, const bf16* __restrict__ inp1, const bf16* __restrict__ inp2,
                const bf16* __restrict__ weight, const bf16* __restrict__ bias, int N, int C, float eps) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    bf16* row_s = reinterpret_cast<bf16*>(smem_raw) + (size_t)warp * C;
    const int nvec = C / 8;
    const float inv_c = 1.0f / (float)C;
    for (int row = blockIdx.x * FWD_WARPS + warp; row < N; row += gridDim.x * FWD_WARPS) {
        const bf16* x1 = inp1 + (size_t)row * C;
        float sum = 0.f;
        for (int v = lane; v < nvec; v += 32) {
            bf16x8 a = ld128_stream(x1 + v * 8);
            if (FUSED_RESIDUAL) {
                float fa[8], fb[8];
                unpack8(a, fa);
                unpack8(ld128_stream(inp2 + (size_t)row * C + v * 8), fb);
#pragma unroll
                for (int j = 0; j < 8; j++) fa[j] += fb[j];
                a = pack8(fa);
                st128(residual_out + (size_t)row * C + v * 8, a);
            }
            st128(row_s + v * 8, a);
            float f[8];
            unpack8(a, f);
#pragma unroll
            for (int j = 0; j < 8; j++) sum += RMS ? f[j] * f[j] : f[j];
        }
        sum = warp_sum(sum);
        float mean = 0.f, rstd;
        if (RMS) {
            rstd = rsqrtf(sum * inv_c + eps);
        } else {
            mean = sum * inv_c;
            float var = 0.f;
            for (int v = lane; v < nvec; v += 32) {
                float f[8];
                unpack8(ld128(row_s + v * 8), f);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    float d = f[j] - mean;
                    var += d * d;
                }
            }
            var = warp_sum(var);
            rstd = rsqrtf(var * inv_c + eps);
        }
        if (lane == 0) {
            if (!RMS && mean_out != nullptr) mean_out[row] = mean;
            if (rstd_out != nullptr) rstd_out[row] = rstd;
        }
        bf16* o = normed + (size_t)row * C;
        for (int v = lane; v < nvec; v += 32) {
            float f[8], w[8], b[8];
            unpack8(ld128(row_s + v * 8), f);
            unpack8(ld128(weight + v * 8), w);
            if (!RMS) unpack8(ld128(bias + v * 8), b);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                float n = (f[j] - mean) * rstd;
                f[j] = RMS ? n * w[j] : n * w[j] + b[j];
            }
            st128(o + v * 8, pack8(f));
        }
        __syncwarp();
    }
}

// Backward. scratch layout: [gridDim.x][2][C] fp32 (second plane unused for RMSNorm).
template <bool RMS>
__global__ void __launch_bounds__(BWD_WARPS * 32)
norm_bwd_kernel(bf16* __restrict__ dinp, float* __restrict__ scratch, const bf16* __restrict__ dout,
                const bf16* __restrict__ inp, const bf16* __restrict__ weight, const float* __restrict__ mean,
                const float* __restrict__ rstd, int N, int C, int accumulate_dinp) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int planes = RMS ? 1 : 2;
    float* acc = reinterpret_cast<float*>(smem_raw) + (size_t)warp * planes * C;  // [planes][C] private to the warp
    const int nvec = C / 8;
    for (int i = lane; i < planes * C; i += 32) acc[i] = 0.f;
    __syncwarp();
    const float inv_c = 1.0f / (float)C;
    for (int row = blockIdx.x * BWD_WARPS + warp; row < N; row += gridDim.x * BWD_WARPS) {
        const bf16* dy = dout + (size_t)row * C;
        const bf16* x = inp + (size_t)row * C;
        const float m = RMS ? 0.f : mean[row];
        const float rs = rstd[row];
        float s1 = 0.f, s2 = 0.f;  // sum(dnorm), sum(dnorm * norm)
        for (int v = lane; v < nvec; v += 32) {
            float fd[8], fx[8], fw[8];
            unpack8(ld128_stream(dy + v * 8), fd);
            unpack8(ld128_stream(x + v * 8), fx);
            unpack8(ld128(weight + v * 8), fw);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                float n = (fx[j] - m) * rs;
                float dn = fd[j] * fw[j];
                s1 += dn;
                s2 += dn * n;
                acc[v * 8 + j] += fd[j] * n;
                if (!RMS) acc[C + v * 8 + j] += fd[j];
            }
        }
        s1 = warp_sum(s1) * inv_c;
        s2 = warp_sum(s2) * inv_c;
        bf16* dx = dinp + (size_t)row * C;
        for (int v = lane; v < nvec; v += 32) {
            float fd[8], fx[8], fw[8], fo[8];
            unpack8(ld128(dy + v * 8), fd);
            unpack8(ld128(x + v * 8), fx);
            unpack8(ld128(weight + v * 8), fw);
            if (accumulate_dinp) unpack8(ld128(dx + v * 8), fo);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                float n = (fx[j] - m) * rs;
                float dn = fd[j] * fw[j];
                float d = RMS ? (dn - n * s2) * rs : (dn - s1 - n * s2) * rs;
                fo[j] = accumulate_dinp ? fo[j] + d : d;
            }
            st128(dx + v * 8, pack8(fo));
        }
    }
    __syncthreads();
    // fixed-order sum over the block's warps -> one partial per block
    const float* all = reinterpret_cast<const float*>(smem_raw);
    float* dst = scratch + (size_t)blockIdx.x * 2 * C;
    for (int i = threadIdx.x; i < planes * C; i += blockDim.x) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < BWD_WARPS; w++) s += all[(size_t)w * planes * C + i];
        dst[i] = s;
    }
}

// dweight[c] += sum_b scratch[b][0][c] ; dbias[c] += sum_b scratch[b][1][c]   (fixed order over b)
__global__ void norm_bwd_finish_kernel(bf16* __restrict__ dweight, bf16* __restrict__ dbias, const float* __restrict__ scratch,
                                       int nblocks, int C) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float sw = 0.f, sb = 0.f;
    for (int b = 0; b < nblocks; b++) {
        sw += scratch[(size_t)b * 2 * C + c];
        if (dbias != nullptr) sb += scratch[(size_t)b * 2 * C + C + c];
    }
    dweight[c] = __float2bfloat16_rn(__bfloat162float(dweight[c]) + sw);
    if (dbias != nullptr) dbias[c] = __float2bfloat16_rn(__bfloat162float(dbias[c]) + sb);
}

static int g_sms = 0;
static int num_sms() {
    if (g_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
        if (g_sms <= 0) g_sms = 148;
    }
    return g_sms;
}

template <bool RMS, bool FUSED>
static int launch_fwd(bf16* normed, float* mean, float* rstd, bf16* residual, const bf16* inp1, const bf16* inp2,
                      const bf16* weight, const bf16* bias, int N, int C, float eps, cudaStream_t stream) {
    if (C % 8 != 0 || C > 16384) return LLMK_ERR_SHAPE;
    const int smem = FWD_WARPS * C * 2;
    static bool configured = false;
    if (!configured) {
        LLMK_CUDA_TRY(cudaFuncSetAttribute(norm_fwd_kernel<RMS, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           FWD_WARPS * 16384 * 2));
        configured = true;
    }
    int grid = ceil_div(N, FWD_WARPS);
    const int cap = num_sms() * 32;
    if (grid > cap) grid = cap;
    norm_fwd_kernel<RMS, FUSED><<<grid, FWD_WARPS * 32, smem, stream>>>(normed, mean, rstd, residual, inp1, inp2, weight, bias,
                                                                       N, C, eps);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

}  // namespace norm
}  // namespace llmk

using namespace llmk;
using namespace llmk::norm;

LLMK_API int llmk_layernorm_fwd(void* normed, void* mean, void* rstd, const void* inp, const void* weight, const void* bias,
                                int N, int C, void* stream) {
    return launch_fwd<false, false>((bf16*)normed, (float*)mean, (float*)rstd, nullptr, (const bf16*)inp, nullptr,
                                    (const bf16*)weight, (const bf16*)bias, N, C, 1e-5f, (cudaStream_t)stream);
}
// residual = inp1 + inp2 ; normed = LN(residual)
LLMK_API int llmk_residual_layernorm_fwd(void* residual, void* normed, void* mean, void* rstd, const void* inp1,
                                         const void* inp2, const void* weight, const void* bias, int N, int C, void* stream) {
    return launch_fwd<false, true>((bf16*)normed, (float*)mean, (float*)rstd, (bf16*)residual, (const bf16*)inp1,
                                   (const bf16*)inp2, (const bf16*)weight, (const bf16*)bias, N, C, 1e-5f,
                                   (cudaStream_t)stream);
}
LLMK_API int llmk_rmsnorm_fwd(void* normed, void* rstd, const void* inp, const void* weight, int N, int C, float eps,
                              void* stream) {
    return launch_fwd<true, false>((bf16*)normed, nullptr, (float*)rstd, nullptr, (const bf16*)inp, nullptr,
                                   (const bf16*)weight, nullptr, N, C, eps, (cudaStream_t)stream);
}
LLMK_API int llmk_residual_rmsnorm_fwd(void* residual, void* normed, void* rstd, const void* inp1, const void* inp2,
                                       const void* weight, int N, int C, float eps, void* stream) {
    return launch_fwd<true, true>((bf16*)normed, nullptr, (float*)rstd, (bf16*)residual, (const bf16*)inp1, (const bf16*)inp2,
                                  (const bf16*)weight, nullptr, N, C, eps, (cudaStream_t)stream);
}

// Number of blocks the backward kernels launch (scratch must hold blocks * 2 * C floats).
LLMK_API int llmk_norm_bwd_blocks(int N, int C) {
    const int smem = BWD_WARPS * 2 * C * 4;  // LayerNorm footprint (RMSNorm needs half)
    int per_sm = (200 * 1024) / (smem > 0 ? smem : 1);
    if (per_sm > 4) per_sm = 4;
    if (per_sm < 1) per_sm = 1;
    int grid = num_sms() * per_sm;
    const int need = ceil_div(N, BWD_WARPS);
    return grid < need ? grid : need;
}
LLMK_API long llmk_norm_bwd_scratch_bytes(int N, int C) { return (long)llmk_norm_bwd_blocks(N, C) * 2 * C * 4; }

namespace llmk {
namespace norm {
// LayerNorm backward: launch of the row kernel plus the fixed-order partial reduction.
int layernorm_bwd_impl(bf16* dinp, bf16* dweight, bf16* dbias, float* scratch, const bf16* dout, const bf16* inp,
                       const bf16* weight, const float* mean, const float* rstd, int N, int C, int accumulate_dinp,
                       cudaStream_t stream) {
    if (C % 8 != 0 || C > 12288) return LLMK_ERR_SHAPE;
    static bool configured = false;
    if (!configured) {
        LLMK_CUDA_TRY(cudaFuncSetAttribute(norm_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           BWD_WARPS * 2 * 6144 * 4));
        configured = true;
    }
    const int smem = BWD_WARPS * 2 * C * 4;
    if (smem > BWD_WARPS * 2 * 6144 * 4) return LLMK_ERR_SHAPE;
    const int grid = llmk_norm_bwd_blocks(N, C);
    norm_bwd_kernel<false><<<grid, BWD_WARPS * 32, smem, stream>>>(dinp, scratch, dout, inp, weight, mean, rstd, N, C,
                                                                  accumulate_dinp);
    LLMK_LAUNCH_CHECK();
    norm_bwd_finish_kernel<<<ceil_div(C, 256), 256, 0, stream>>>(dweight, dbias, scratch, grid, C);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
}  // namespace norm
}  // namespace llmk

// dinp (+)= dLN/dinp ; dweight += ; dbias +=   (scratch: llmk_norm_bwd_scratch_bytes(N, C) bytes)
LLMK_API int llmk_layernorm_bwd(void* dinp, void* dweight, void* dbias, void* scratch, const void* dout, const void* inp,
                                const void* weight, const void* mean, const void* rstd, int N, int C, int accumulate_dinp,
                                void* stream) {
    return layernorm_bwd_impl((bf16*)dinp, (bf16*)dweight, (bf16*)dbias, (float*)scratch, (const bf16*)dout, (const bf16*)inp,
                              (const bf16*)weight, (const float*)mean, (const float*)rstd, N, C, accumulate_dinp,
                              (cudaStream_t)stream);
}

LLMK_API int llmk_rmsnorm_bwd(void* dinp, void* dweight, void* scratch, const void* dout, const void* inp, const void* weight,
                              const void* rstd, int N, int C, int accumulate_dinp, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (C % 8 != 0 || C > 12288) return LLMK_ERR_SHAPE;
    static bool configured = false;
    if (!configured) {
        LLMK_CUDA_TRY(cudaFuncSetAttribute(norm_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           BWD_WARPS * 12288 * 4));
        configured = true;
    }
    const int smem = BWD_WARPS * C * 4;
    const int grid = llmk_norm_bwd_blocks(N, C);
    norm_bwd_kernel<true><<<grid, BWD_WARPS * 32, smem, stream>>>((bf16*)dinp, (float*)scratch, (const bf16*)dout,
                                                                 (const bf16*)inp, (const bf16*)weight, nullptr,
                                                                 (const float*)rstd, N, C, accumulate_dinp);
    LLMK_LAUNCH_CHECK();
    norm_bwd_finish_kernel<<<ceil_div(C, 256), 256, 0, stream>>>((bf16*)dweight, nullptr, (const float*)scratch, grid, C);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
