// Fused classifier: softmax + cross-entropy loss + (optionally) dlogits written in place of logits.
//
// Same job as fused_classifier (reference llmc/fused_classifier.cuh:161-258): one block per token row,
// only the first V of the Vp padded columns take part, the padded columns get a zero gradient.
// New design: three passes per row (max, sum of exponentials, gradient) with 128-bit loads issued
// four at a time; only the first pass reads HBM, the other two find the row in the L2. Registers
// stay low so several rows per SM are in flight. Every warp takes part in every barrier; there are
// no divergent early exits.
#include "common.cuh"

namespace llmk {
namespace classifier {

constexpr int TPB = 512;
constexpr int UNROLL = 4;  // 16-byte loads in flight per thread

// Three passes over the row: (1) maximum, (2) sum of exp(x - max), (3) gradient written in place.
// Pass 1 streams the row from HBM; passes 2 and 3 hit the L2 (a row is ~100 KB and only a few rows per
// SM are in flight). One exp per element and pass; loads are issued UNROLL at a time before use.
template <bool WRITE_DLOGITS>
__global__ void __launch_bounds__(TPB)
fused_classifier_kernel(bf16* __restrict__ logits, float* __restrict__ losses, const int* __restrict__ targets, float dloss,
                        int V, int Vp, int accumulate_loss) {
    __shared__ float sh[32];
    // reverse order: the rows written last by the LM-head GEMM are still in the L2
    const size_t row = (size_t)(gridDim.x - 1 - blockIdx.x);
    bf16* x = logits + row * Vp;
    const int target = targets[row];
    const int nvec = Vp / 8;           // Vp is a multiple of 8
    const int nvec_valid = (V + 7) / 8;  // vectors holding at least one real column

    // ---- pass 1: max
    float mx = -INFINITY;
    for (int v0 = threadIdx.x; v0 < nvec_valid; v0 += TPB * UNROLL) {
        bf16x8 r[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++)
            if (v0 + u * TPB < nvec_valid) r[u] = ld128(x + (size_t)(v0 + u * TPB) * 8);
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int v = v0 + u * TPB;
            if (v < nvec_valid) {
                float f[8];
                unpack8(r[u], f);
#pragma unroll
                for (int j = 0; j < 8; j++)
                    if (v * 8 + j < V) mx = fmaxf(mx, f[j]);
            }
        }
    }
    mx = block_max(mx, sh);
    // ---- pass 2: sum of exponentials (exp2 domain)
    const float L2E = 1.4426950408889634f;
    const float mxs = mx * L2E;
    float sum = 0.f;
    for (int v0 = threadIdx.x; v0 < nvec_valid; v0 += TPB * UNROLL) {
        bf16x8 r[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++)
            if (v0 + u * TPB < nvec_valid) r[u] = ld128(x + (size_t)(v0 + u * TPB) * 8);
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int v = v0 + u * TPB;
            if (v < nvec_valid) {
                float f[8];
                unpack8(r[u], f);
#pragma unroll
                for (int j = 0; j < 8; j++)
                    if (v * 8 + j < V) sum += exp2f(f[j] * L2E - mxs);
            }
        }
    }
    sum = block_sum(sum, sh);
    const float inv_sum = 1.0f / sum;
    // loss for this row (the target logit is read before any in-place write: barrier below)
    if (threadIdx.x == 0) {
        const float lt = __bfloat162float(x[target]);
        const float loss = -(lt - mx - __logf(sum));
        losses[row] = accumulate_loss ? losses[row] + loss : loss;
    }
    __syncthreads();
    if (WRITE_DLOGITS) {
        // ---- pass 3: dlogits = (softmax - onehot) * dloss; padded columns get 0
        for (int v0 = threadIdx.x; v0 < nvec; v0 += TPB * UNROLL) {
            bf16x8 r[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; u++)
                if (v0 + u * TPB < nvec) r[u] = ld128(x + (size_t)(v0 + u * TPB) * 8);
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                const int v = v0 + u * TPB;
                if (v < nvec) {
                    float f[8];
                    unpack8(r[u], f);
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const int c = v * 8 + j;
                        const float pr = exp2f(f[j] * L2E - mxs) * inv_sum;
                        f[j] = (c < V) ? (pr - (c == target ? 1.0f : 0.0f)) * dloss : 0.f;
                    }
                    st128_stream(x + (size_t)v * 8, pack8(f));
                }
            }
        }
    }
}

// out[0] (+)= scale * sum(x[0..n)) with a fixed summation order (single block).
__global__ void sum_scaled_kernel(float* __restrict__ out, const float* __restrict__ x, int n, float scale, int accumulate) {
    __shared__ float sh[32];
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
    s = block_sum(s, sh);
    if (threadIdx.x == 0) out[0] = (accumulate ? out[0] : 0.f) + s * scale;
}

}  // namespace classifier
}  // namespace llmk

using namespace llmk;
using namespace llmk::classifier;

// logits: [rows, Vp] bf16, overwritten by dlogits when write_dlogits != 0; losses: [rows] fp32.
LLMK_API int llmk_fused_classifier(void* logits, void* losses, const void* targets, float dloss, int rows, int V, int Vp,
                                   int write_dlogits, int accumulate_loss, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (Vp % 8 || V > Vp || rows <= 0) return LLMK_ERR_SHAPE;
    bf16* lg = (bf16*)logits;
    float* ls = (float*)losses;
    const int* tg = (const int*)targets;
    if (write_dlogits) fused_classifier_kernel<true><<<rows, TPB, 0, stream>>>(lg, ls, tg, dloss, V, Vp, accumulate_loss);
    else fused_classifier_kernel<false><<<rows, TPB, 0, stream>>>(lg, ls, tg, dloss, V, Vp, accumulate_loss);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

LLMK_API int llmk_sum_scaled(void* out, const void* x, int n, float scale, int accumulate, void* stream) {
    sum_scaled_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>((float*)out, (const float*)x, n, scale, accumulate);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
