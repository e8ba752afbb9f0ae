// Fused classifier: softmax + cross-entropy loss + (optionally) dlogits written in place of logits.
//
// Same job as fused_classifier (reference llmc/fused_classifier.cuh:161-258): one block per token row,
// only the first V of the Vp padded columns take part, the padded columns get a zero gradient.
// New design: three passes per row (max, sum of exponentials, gradient) with 128-bit loads issued
// four at a time; only the first pass reads HBM, the other two find the row in the L2. Registers
// stay low so several rows per SM are in flight. Every warp takes part in every barrier; there are
// no divergent early exits.
#include "ptx_sm100.cuh"

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

// Rows that fit twice into shared memory (Vp * 2 bytes <= ~110 KB, e.g. the GPT-2 vocabulary): a persistent block
// per SM streams its rows through a two-slot shared-memory ring with bulk copies, so each logit is read from HBM
// exactly once and the three passes (max, sum, gradient) run out of shared memory while the next row is already
// arriving. The gradient leaves with streaming 128-bit stores. Same arithmetic as fused_classifier_kernel.
constexpr int STPB = 1024;
constexpr int BULK_CHUNK = 16384;

template <bool WRITE_DLOGITS>
__global__ void __launch_bounds__(STPB, 1)
fused_classifier_smem_kernel(bf16* __restrict__ logits, float* __restrict__ losses, const int* __restrict__ targets, float dloss,
                             int rows, int V, int Vp, int accumulate_loss, int* status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ float sh[32];
    __shared__ uint64_t full[2];
    __shared__ int abort_word;
    volatile int* abort_flag = &abort_word;
    const uint32_t row_bytes = (uint32_t)Vp * 2;
    const uint32_t slot_bytes = (row_bytes + 127u) & ~127u;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&full[0], 1);
        ptx::mbar_init(&full[1], 1);
        abort_word = 0;
        ptx::fence_barrier_init();
    }
    __syncthreads();
    const int mine = blockIdx.x < rows ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    // reverse order: the rows written last by the LM-head GEMM are still in the L2
    auto row_of = [&](int i) { return (size_t)(rows - 1 - (blockIdx.x + i * (int)gridDim.x)); };
    auto issue = [&](int i) {   // thread 0 only
        const int slot = i & 1;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(logits + row_of(i) * Vp);
        uint8_t* dst = smem_raw + slot * slot_bytes;
        ptx::mbar_arrive_expect_tx(&full[slot], row_bytes);
        for (uint32_t off = 0; off < row_bytes; off += BULK_CHUNK) {
            const uint32_t n = row_bytes - off < (uint32_t)BULK_CHUNK ? row_bytes - off : (uint32_t)BULK_CHUNK;
            ptx::bulk_load_1d(dst + off, src + off, n, &full[slot]);
        }
    };
    if (threadIdx.x == 0) {
        if (mine > 0) issue(0);
        if (mine > 1) issue(1);
    }
    const int nvec = Vp / 8, nvec_valid = (V + 7) / 8;
    const float L2E = 1.4426950408889634f;
    for (int i = 0; i < mine; i++) {
        const int slot = i & 1;
        const size_t row = row_of(i);
        if (!ptx::mbar_wait(&full[slot], (i >> 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_TMA_FULL, 9000 + slot)) break;
        const bf16* x = reinterpret_cast<const bf16*>(smem_raw + slot * slot_bytes);
        const int target = targets[row];
        // the target logit is read now: pass 2 overwrites the row, and no thread can get there before every thread
        // has passed the barrier inside the first block reduction
        const float lt = __bfloat162float(x[target]);
        // pass 1: maximum with packed bf16 compares (the last, partly valid vector takes the scalar path)
        const int nfull = V / 8;   // vectors whose 8 columns are all real
        __nv_bfloat162 m2 = __float2bfloat162_rn(-INFINITY);
        for (int v = threadIdx.x; v < nfull; v += STPB) {
            const bf16x8 r = *reinterpret_cast<const bf16x8*>(x + v * 8);
            m2 = __hmax2(__hmax2(m2, r.v[0]), __hmax2(r.v[1], __hmax2(r.v[2], r.v[3])));
        }
        float mx = fmaxf(__low2float(m2), __high2float(m2));
        if (threadIdx.x == 0)
            for (int c = nfull * 8; c < V; c++) mx = fmaxf(mx, __bfloat162float(x[c]));
        mx = block_max(mx, sh);
        const float mxs = mx * L2E;
        // pass 2: exponentials, summed in fp32 and (when the gradient is wanted) stored back over the logits as bf16
        float sum = 0.f;
        bf16* xe = const_cast<bf16*>(x);
        for (int v = threadIdx.x; v < nvec; v += STPB) {
            float f[8];
            if (v < nfull) {
                unpack8(*reinterpret_cast<const bf16x8*>(x + v * 8), f);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    f[j] = exp2f(fmaf(f[j], L2E, -mxs));
                    sum += f[j];
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int c = v * 8 + j;
                    f[j] = c < V ? exp2f(fmaf(__bfloat162float(x[c]), L2E, -mxs)) : 0.f;
                    sum += f[j];
                }
            }
            if (WRITE_DLOGITS) *reinterpret_cast<bf16x8*>(xe + v * 8) = pack8(f);
        }
        sum = block_sum(sum, sh);
        if (threadIdx.x == 0) {
            const float loss = -(lt - mx - __logf(sum));
            losses[row] = accumulate_loss ? losses[row] + loss : loss;
        }
        if (WRITE_DLOGITS) {
            // pass 3: dlogits = (softmax - onehot) * dloss from the stored exponentials; padded columns hold 0 already
            const float k = dloss / sum;
            bf16* out = logits + row * Vp;
            const int tv = target >> 3, tj = target & 7;
            for (int v = threadIdx.x; v < nvec; v += STPB) {
                float f[8];
                unpack8(*reinterpret_cast<const bf16x8*>(x + v * 8), f);
#pragma unroll
                for (int j = 0; j < 8; j++) f[j] *= k;
                if (v == tv) {
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        if (j == tj) f[j] -= dloss;
                }
                st128_stream(out + (size_t)v * 8, pack8(f));
            }
        }
        __syncthreads();   // every thread is done with this slot: refill it
        if (threadIdx.x == 0 && i + 2 < mine) issue(i + 2);
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
    const int slot_bytes = (Vp * 2 + 127) & ~127;
    if (2 * slot_bytes <= 220 * 1024) {
        static PerDeviceOnce once_configured;
        if (once_configured.first()) {
            LLMK_CUDA_TRY(cudaFuncSetAttribute(fused_classifier_smem_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
            LLMK_CUDA_TRY(cudaFuncSetAttribute(fused_classifier_smem_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
        }
        int sms = 0, dev = 0;
        LLMK_CUDA_TRY(cudaGetDevice(&dev));
        LLMK_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        const int grid = rows < sms ? rows : sms;
        if (write_dlogits)
            fused_classifier_smem_kernel<true><<<grid, STPB, 2 * slot_bytes, stream>>>(lg, ls, tg, dloss, rows, V, Vp, accumulate_loss,
                                                                                   current_status_word());
        else
            fused_classifier_smem_kernel<false><<<grid, STPB, 2 * slot_bytes, stream>>>(lg, ls, tg, dloss, rows, V, Vp, accumulate_loss,
                                                                                    current_status_word());
        LLMK_LAUNCH_CHECK();
        return LLMK_OK;
    }
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
