// Fused classifier: softmax + cross-entropy loss + (optionally) dlogits written in place of logits.
//
// Same job as fused_classifier (reference llmc/fused_classifier.cuh:161-258): one block per token row,
// only the first V of the Vp padded columns take part, the padded columns get a zero gradient.
// New design: a single online (max, sum) pass with 128-bit loads keeps the row's 8-element vectors
// that this thread owns in registers when the row is short enough (V <= 8 * 8 * blockDim), so the
// gradient pass does not re-read the logits; longer rows re-read them (they are L2-resident).
// Every warp takes part in every barrier; there are no divergent early exits.
#include "common.cuh"

namespace llmk {
namespace classifier {

constexpr int TPB = 512;
constexpr int MAXV_REG = 13;  // vectors of 8 per thread kept in registers: covers V <= 13*8*512 = 53248

struct MaxSum {
    float m, s;
};
__device__ __forceinline__ MaxSum combine(MaxSum a, MaxSum b) {
    MaxSum r;
    r.m = fmaxf(a.m, b.m);
    r.s = a.s * __expf(a.m - r.m) + b.s * __expf(b.m - r.m);
    return r;
}

template <bool WRITE_DLOGITS, bool IN_REGS>
__global__ void __launch_bounds__(TPB)
fused_classifier_kernel(bf16* __restrict__ logits, float* __restrict__ losses, const int* __restrict__ targets, float dloss,
                        int V, int Vp, int accumulate_loss) {
    __shared__ float sh_m[32], sh_s[32];
    // reverse order: the rows written last by the LM-head GEMM are still in the L2
    const size_t row = (size_t)(gridDim.x - 1 - blockIdx.x);
    bf16* x = logits + row * Vp;
    const int target = targets[row];
    const int nvec = Vp / 8;       // Vp is a multiple of 8
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    bf16x8 cache[IN_REGS ? MAXV_REG : 1];
    MaxSum ms = {-INFINITY, 0.f};
    if (IN_REGS) {
#pragma unroll
        for (int k = 0; k < MAXV_REG; k++) {
            const int v = threadIdx.x + k * TPB;
            if (v < nvec) {
                cache[k] = ld128_stream(x + v * 8);
                float f[8];
                unpack8(cache[k], f);
                float lm = -INFINITY;
#pragma unroll
                for (int j = 0; j < 8; j++)
                    if (v * 8 + j < V) lm = fmaxf(lm, f[j]);
                if (lm > -INFINITY) {
                    float ls = 0.f;
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        if (v * 8 + j < V) ls += __expf(f[j] - lm);
                    ms = combine(ms, MaxSum{lm, ls});
                }
            }
        }
    } else {
        for (int v = threadIdx.x; v < nvec; v += TPB) {
            float f[8];
            unpack8(ld128(x + v * 8), f);
            float lm = -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (v * 8 + j < V) lm = fmaxf(lm, f[j]);
            if (lm > -INFINITY) {
                float ls = 0.f;
#pragma unroll
                for (int j = 0; j < 8; j++)
                    if (v * 8 + j < V) ls += __expf(f[j] - lm);
                ms = combine(ms, MaxSum{lm, ls});
            }
        }
    }
    // warp then block reduction of (max, sum)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxSum other;
        other.m = __shfl_xor_sync(0xffffffffu, ms.m, o);
        other.s = __shfl_xor_sync(0xffffffffu, ms.s, o);
        if (other.m > -INFINITY || ms.m > -INFINITY) {
            if (ms.m == -INFINITY) ms = other;
            else if (other.m > -INFINITY) ms = combine(ms, other);
        }
    }
    if (lane == 0) {
        sh_m[warp] = ms.m;
        sh_s[warp] = ms.s;
    }
    __syncthreads();
    MaxSum tot = {-INFINITY, 0.f};
    for (int w = 0; w < TPB / 32; w++) {
        MaxSum o = {sh_m[w], sh_s[w]};
        if (o.m > -INFINITY) tot = (tot.m == -INFINITY) ? o : combine(tot, o);
    }
    const float inv_sum = 1.0f / tot.s;
    // loss for this row (the read of the target logit happens before any in-place write: barrier below)
    if (threadIdx.x == 0) {
        const float lt = __bfloat162float(x[target]);
        const float loss = -(lt - tot.m - __logf(tot.s));
        losses[row] = accumulate_loss ? losses[row] + loss : loss;
    }
    __syncthreads();
    if (WRITE_DLOGITS) {
        if (IN_REGS) {
#pragma unroll
            for (int k = 0; k < MAXV_REG; k++) {
                const int v = threadIdx.x + k * TPB;
                if (v < nvec) {
                    float f[8];
                    unpack8(cache[k], f);
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const int c = v * 8 + j;
                        const float pr = __expf(f[j] - tot.m) * inv_sum;
                        f[j] = (c < V) ? (pr - (c == target ? 1.0f : 0.0f)) * dloss : 0.f;
                    }
                    st128(x + v * 8, pack8(f));
                }
            }
        } else {
            for (int v = threadIdx.x; v < nvec; v += TPB) {
                float f[8];
                unpack8(ld128(x + v * 8), f);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int c = v * 8 + j;
                    const float pr = __expf(f[j] - tot.m) * inv_sum;
                    f[j] = (c < V) ? (pr - (c == target ? 1.0f : 0.0f)) * dloss : 0.f;
                }
                st128(x + v * 8, pack8(f));
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
    const bool in_regs = (Vp / 8) <= MAXV_REG * TPB;
    bf16* lg = (bf16*)logits;
    float* ls = (float*)losses;
    const int* tg = (const int*)targets;
    if (write_dlogits) {
        if (in_regs) fused_classifier_kernel<true, true><<<rows, TPB, 0, stream>>>(lg, ls, tg, dloss, V, Vp, accumulate_loss);
        else fused_classifier_kernel<true, false><<<rows, TPB, 0, stream>>>(lg, ls, tg, dloss, V, Vp, accumulate_loss);
    } else {
        fused_classifier_kernel<false, false><<<rows, TPB, 0, stream>>>(lg, ls, tg, dloss, V, Vp, accumulate_loss);
    }
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

LLMK_API int llmk_sum_scaled(void* out, const void* x, int n, float scale, int accumulate, void* stream) {
    sum_scaled_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>((float*)out, (const float*)x, n, scale, accumulate);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
