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
#include "ptx_sm100.cuh"

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
    // block = (32 columns, 8 partial-row lanes); lane y sums partials y, y+8, ...; then the 8 lanes are
    // added in fixed order, so the result does not depend on scheduling
    __shared__ float shw[8][33], shb[8][33];
    const int c = blockIdx.x * 32 + threadIdx.x;
    float sw = 0.f, sb = 0.f;
    if (c < C) {
        for (int b = threadIdx.y; b < nblocks; b += 8) {
            sw += scratch[(size_t)b * 2 * C + c];
            if (dbias != nullptr) sb += scratch[(size_t)b * 2 * C + C + c];
        }
    }
    shw[threadIdx.y][threadIdx.x] = sw;
    shb[threadIdx.y][threadIdx.x] = sb;
    __syncthreads();
    if (threadIdx.y == 0 && c < C) {
        float tw = 0.f, tb = 0.f;
#pragma unroll
        for (int y = 0; y < 8; y++) {
            tw += shw[y][threadIdx.x];
            tb += shb[y][threadIdx.x];
        }
        dweight[c] = __float2bfloat16_rn(__bfloat162float(dweight[c]) + tw);
        if (dbias != nullptr) dbias[c] = __float2bfloat16_rn(__bfloat162float(dbias[c]) + tb);
    }
}

// ------------------------------------------------------------------------------------------------
// Fast paths for C = 256 * NVEC: the whole row lives in registers (lane l owns the 16-byte vectors
// l, l+32, ...), so global memory is read exactly once, and the backward keeps its dweight / dbias
// sums in registers across all rows of the warp. 8 warps per block, one row per warp at a time.
constexpr int REG_WARPS = 8;

template <bool RMS, bool FUSED_RESIDUAL, int NVEC>
__global__ void __launch_bounds__(REG_WARPS * 32)
norm_fwd_reg_kernel(bf16* __restrict__ normed, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                    bf16* __restrict__ residual_out, const bf16* __restrict__ inp1, const bf16* __restrict__ inp2,
                    const bf16* __restrict__ weight, const bf16* __restrict__ bias, int N, float eps) {
    constexpr int C = NVEC * 256;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float inv_c = 1.0f / (float)C;
    for (int row = blockIdx.x * REG_WARPS + warp; row < N; row += gridDim.x * REG_WARPS) {
        bf16x8 xv[NVEC];
#pragma unroll
        for (int k = 0; k < NVEC; k++) xv[k] = ld128_stream(inp1 + (size_t)row * C + (lane + 32 * k) * 8);
        if (FUSED_RESIDUAL) {
            bf16x8 yv[NVEC];
#pragma unroll
            for (int k = 0; k < NVEC; k++) yv[k] = ld128_stream(inp2 + (size_t)row * C + (lane + 32 * k) * 8);
#pragma unroll
            for (int k = 0; k < NVEC; k++) {
                float a[8], b[8];
                unpack8(xv[k], a);
                unpack8(yv[k], b);
#pragma unroll
                for (int j = 0; j < 8; j++) a[j] += b[j];
                xv[k] = pack8(a);
                st128(residual_out + (size_t)row * C + (lane + 32 * k) * 8, xv[k]);
            }
        }
        float sum = 0.f;
#pragma unroll
        for (int k = 0; k < NVEC; k++) {
            float f[8];
            unpack8(xv[k], f);
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
#pragma unroll
            for (int k = 0; k < NVEC; k++) {
                float f[8];
                unpack8(xv[k], f);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const float d = f[j] - mean;
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
#pragma unroll
        for (int k = 0; k < NVEC; k++) {
            float f[8], w[8], b[8];
            unpack8(xv[k], f);
            unpack8(ld128(weight + (lane + 32 * k) * 8), w);
            if (!RMS) unpack8(ld128(bias + (lane + 32 * k) * 8), b);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float n = (f[j] - mean) * rstd;
                f[j] = RMS ? n * w[j] : n * w[j] + b[j];
            }
            st128(normed + (size_t)row * C + (lane + 32 * k) * 8, pack8(f));
        }
    }
}

// scratch layout as for norm_bwd_kernel: [gridDim.x][2][C] fp32
template <bool RMS, int NVEC>
__global__ void __launch_bounds__(REG_WARPS * 32)
norm_bwd_reg_kernel(bf16* __restrict__ dinp, float* __restrict__ scratch, const bf16* __restrict__ dout,
                    const bf16* __restrict__ inp, const bf16* __restrict__ weight, const float* __restrict__ mean,
                    const float* __restrict__ rstd, int N, int accumulate_dinp) {
    constexpr int C = NVEC * 256;
    constexpr int PLANES = RMS ? 1 : 2;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    float* sh = reinterpret_cast<float*>(smem_raw);  // [REG_WARPS][PLANES][C], used only for the final reduction
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float inv_c = 1.0f / (float)C;
    float dw[NVEC][8], db[RMS ? 1 : NVEC][8];
#pragma unroll
    for (int k = 0; k < NVEC; k++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
            dw[k][j] = 0.f;
            if (!RMS) db[k][j] = 0.f;
        }
    for (int row = blockIdx.x * REG_WARPS + warp; row < N; row += gridDim.x * REG_WARPS) {
        bf16x8 dv[NVEC], xv[NVEC];
#pragma unroll
        for (int k = 0; k < NVEC; k++) {
            dv[k] = ld128_stream(dout + (size_t)row * C + (lane + 32 * k) * 8);
            xv[k] = ld128_stream(inp + (size_t)row * C + (lane + 32 * k) * 8);
        }
        const float m = RMS ? 0.f : mean[row];
        const float rs = rstd[row];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int k = 0; k < NVEC; k++) {
            float fd[8], fx[8], fw[8];
            unpack8(dv[k], fd);
            unpack8(xv[k], fx);
            unpack8(ld128(weight + (lane + 32 * k) * 8), fw);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float n = (fx[j] - m) * rs;
                const float dn = fd[j] * fw[j];
                s1 += dn;
                s2 += dn * n;
                dw[k][j] += fd[j] * n;
                if (!RMS) db[k][j] += fd[j];
            }
        }
        s1 = warp_sum(s1) * inv_c;
        s2 = warp_sum(s2) * inv_c;
#pragma unroll
        for (int k = 0; k < NVEC; k++) {
            float fd[8], fx[8], fw[8], fo[8];
            unpack8(dv[k], fd);
            unpack8(xv[k], fx);
            unpack8(ld128(weight + (lane + 32 * k) * 8), fw);
            bf16* dx = dinp + (size_t)row * C + (lane + 32 * k) * 8;
            if (accumulate_dinp) unpack8(ld128(dx), fo);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float n = (fx[j] - m) * rs;
                const float dn = fd[j] * fw[j];
                const float d = RMS ? (dn - n * s2) * rs : (dn - s1 - n * s2) * rs;
                fo[j] = accumulate_dinp ? fo[j] + d : d;
            }
            st128(dx, pack8(fo));
        }
    }
    // per-warp sums -> shared memory -> fixed-order sum over warps -> one partial per block
#pragma unroll
    for (int k = 0; k < NVEC; k++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
            sh[(size_t)warp * PLANES * C + (lane + 32 * k) * 8 + j] = dw[k][j];
            if (!RMS) sh[(size_t)warp * PLANES * C + C + (lane + 32 * k) * 8 + j] = db[k][j];
        }
    __syncthreads();
    float* dst = scratch + (size_t)blockIdx.x * 2 * C;
    for (int i = threadIdx.x; i < PLANES * C; i += blockDim.x) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < REG_WARPS; w++) s += sh[(size_t)w * PLANES * C + i];
        dst[i] = s;
    }
}

// Backward with a bulk-copy ring: every warp owns rows and streams them (dout, inp and, when accumulating, the old
// dinp) into its own shared-memory ring with cp.async.bulk, STAGES rows ahead, so that about
// warps x STAGES x 3 x C x 2 bytes are in flight per SM whatever the register budget - the register-only kernel above
// has a single row per warp in flight and reaches well under half of the copy bandwidth. The arithmetic and the
// scratch layout are those of norm_bwd_reg_kernel. Every wait is bounded; a failure goes to `status`.
template <int NVEC>
struct BulkCfg {
    static constexpr int C = NVEC * 256;
    static constexpr int ROW = C * 2;
    // narrow rows: 16 warps (two per scheduler hide the reduction latency) with a 2-deep ring; wide rows: 8 warps
    static constexpr int WARPS = NVEC <= 3 ? 16 : 8;
    static constexpr int STAGES = NVEC <= 3 ? 2 : (NVEC == 4 ? 4 : 3);
    static constexpr int WARP_RING = STAGES * 3 * ROW;
    static constexpr int OFF_BAR = WARPS * WARP_RING;
    static constexpr int SMEM = OFF_BAR + WARPS * STAGES * 8;
};

template <bool RMS, int NVEC>
__global__ void __launch_bounds__(BulkCfg<NVEC>::WARPS * 32, 1)
norm_bwd_bulk_kernel(bf16* __restrict__ dinp, float* __restrict__ scratch, const bf16* __restrict__ dout,
                     const bf16* __restrict__ inp, const bf16* __restrict__ weight, const float* __restrict__ mean,
                     const float* __restrict__ rstd, int N, int accumulate_dinp, int* status) {
    using B = BulkCfg<NVEC>;
    constexpr int C = B::C, ROW = B::ROW, STAGES = B::STAGES, WARPS = B::WARPS;
    constexpr int PLANES = RMS ? 1 : 2;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ int abort_word;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* ring = smem_raw + (size_t)warp * B::WARP_RING;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + B::OFF_BAR) + warp * STAGES;
    volatile int* abort_flag = &abort_word;
    if (threadIdx.x == 0) abort_word = 0;
    if (lane == 0) {
        for (int i = 0; i < STAGES; i++) ptx::mbar_init(&full[i], 1);
    }
    ptx::fence_barrier_init();
    __syncthreads();

    const int first = blockIdx.x * WARPS + warp, stride = gridDim.x * WARPS;
    const int nrows = first < N ? (N - first + stride - 1) / stride : 0;
    const uint32_t tx = (accumulate_dinp ? 3u : 2u) * ROW;
    auto issue = [&](int i) {   // lane 0 only
        const int st = i % STAGES;
        const size_t off = (size_t)(first + (size_t)i * stride) * C;
        uint8_t* dst = ring + st * 3 * ROW;
        ptx::mbar_arrive_expect_tx(&full[st], tx);
        ptx::bulk_load_1d(dst, dout + off, ROW, &full[st]);
        ptx::bulk_load_1d(dst + ROW, inp + off, ROW, &full[st]);
        if (accumulate_dinp) ptx::bulk_load_1d(dst + 2 * ROW, dinp + off, ROW, &full[st]);
    };
    if (lane == 0)
        for (int i = 0; i < STAGES && i < nrows; i++) issue(i);

    const float inv_c = 1.0f / (float)C;
    float dw[NVEC][8], db[RMS ? 1 : NVEC][8];
#pragma unroll
    for (int k = 0; k < NVEC; k++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
            dw[k][j] = 0.f;
            if (!RMS) db[k][j] = 0.f;
        }

    bool ok = true;
    for (int i = 0; i < nrows; i++) {
        const int st = i % STAGES;
        const int row = first + i * stride;
        ok = ptx::mbar_wait(&full[st], (i / STAGES) & 1, abort_flag, status, LLMK_ST_TIMEOUT_TMA_FULL, 8000 + st);
        if (!ok) break;
        const uint8_t* src = ring + st * 3 * ROW;
        bf16x8 dv[NVEC], xv[NVEC], ov[NVEC];
#pragma unroll
        for (int k = 0; k < NVEC; k++) {
            dv[k] = *reinterpret_cast<const bf16x8*>(src + (lane + 32 * k) * 16);
            xv[k] = *reinterpret_cast<const bf16x8*>(src + ROW + (lane + 32 * k) * 16);
            if (accumulate_dinp) ov[k] = *reinterpret_cast<const bf16x8*>(src + 2 * ROW + (lane + 32 * k) * 16);
        }
        __syncwarp();   // the stage has been copied into registers by every lane: refill it
        if (lane == 0 && i + STAGES < nrows) issue(i + STAGES);
        const float m = RMS ? 0.f : mean[row];
        const float rs = rstd[row];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int k = 0; k < NVEC; k++) {
            float fd[8], fx[8], fw[8];
            unpack8(dv[k], fd);
            unpack8(xv[k], fx);
            unpack8(ld128(weight + (lane + 32 * k) * 8), fw);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float n = (fx[j] - m) * rs;
                const float dn = fd[j] * fw[j];
                s1 += dn;
                s2 += dn * n;
                dw[k][j] += fd[j] * n;
                if (!RMS) db[k][j] += fd[j];
            }
        }
        s1 = warp_sum(s1) * inv_c;
        s2 = warp_sum(s2) * inv_c;
#pragma unroll
        for (int k = 0; k < NVEC; k++) {
            float fd[8], fx[8], fo[8], fw[8];
            unpack8(dv[k], fd);
            unpack8(xv[k], fx);
            unpack8(ld128(weight + (lane + 32 * k) * 8), fw);
            if (accumulate_dinp) unpack8(ov[k], fo);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float n = (fx[j] - m) * rs;
                const float dn = fd[j] * fw[j];
                const float d = RMS ? (dn - n * s2) * rs : (dn - s1 - n * s2) * rs;
                fo[j] = accumulate_dinp ? fo[j] + d : d;
            }
            st128(dinp + (size_t)row * C + (lane + 32 * k) * 8, pack8(fo));
        }
    }
    // all rings are idle now (every issued copy has been waited for): reuse them for the cross-warp reduction
    __syncthreads();
    if (*abort_flag) return;
    float* sh = reinterpret_cast<float*>(smem_raw);   // [WARPS][PLANES][C]
#pragma unroll
    for (int k = 0; k < NVEC; k++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
            sh[(size_t)warp * PLANES * C + (lane + 32 * k) * 8 + j] = dw[k][j];
            if (!RMS) sh[(size_t)warp * PLANES * C + C + (lane + 32 * k) * 8 + j] = db[k][j];
        }
    __syncthreads();
    float* dst = scratch + (size_t)blockIdx.x * 2 * C;
    for (int i = threadIdx.x; i < PLANES * C; i += blockDim.x) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; w++) acc += sh[(size_t)w * PLANES * C + i];
        dst[i] = acc;
    }
}

// Wide rows (C = NV * 2048): one 256-thread block per row, every thread owns NV 8-element column groups, so the
// weight-gradient accumulators stay at NV * 8 registers per plane however wide the row is and no cross-warp
// reduction of them is needed (each column has one owner per block). The next row is prefetched into registers
// while the block reduces the current one. scratch layout [gridDim.x][2][C] as for the other kernels.
template <bool RMS, int NV>
__global__ void __launch_bounds__(256, NV <= 2 ? 2 : 1)
norm_bwd_wide_kernel(bf16* __restrict__ dinp, float* __restrict__ scratch, const bf16* __restrict__ dout,
                     const bf16* __restrict__ inp, const bf16* __restrict__ weight, const float* __restrict__ mean,
                     const float* __restrict__ rstd, int N, int accumulate_dinp) {
    constexpr int C = NV * 2048;
    __shared__ float red[2][2][8];   // [parity][s1 | s2][warp]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float inv_c = 1.0f / (float)C;
    float dw[NV][8], db[RMS ? 1 : NV][8], fw[NV][8];
#pragma unroll
    for (int k = 0; k < NV; k++) {
        unpack8(ld128(weight + (threadIdx.x + 256 * k) * 8), fw[k]);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            dw[k][j] = 0.f;
            if (!RMS) db[k][j] = 0.f;
        }
    }
    bf16x8 dv[NV], xv[NV], ov[NV], dvn[NV], xvn[NV], ovn[NV];
    auto load = [&](int row, bf16x8* d, bf16x8* x, bf16x8* o) {
#pragma unroll
        for (int k = 0; k < NV; k++) {
            const size_t off = (size_t)row * C + (threadIdx.x + 256 * k) * 8;
            d[k] = ld128_stream(dout + off);
            x[k] = ld128_stream(inp + off);
            if (accumulate_dinp) o[k] = ld128(dinp + off);
        }
    };
    int row = blockIdx.x;
    if (row < N) load(row, dv, xv, ov);
    int par = 0;
    for (; row < N; row += gridDim.x, par ^= 1) {
        const int next = row + gridDim.x;
        if (next < N) load(next, dvn, xvn, ovn);
        const float m = RMS ? 0.f : mean[row];
        const float rs = rstd[row];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int k = 0; k < NV; k++) {
            float fd[8], fx[8];
            unpack8(dv[k], fd);
            unpack8(xv[k], fx);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float n = (fx[j] - m) * rs;
                const float dn = fd[j] * fw[k][j];
                s1 += dn;
                s2 += dn * n;
                dw[k][j] += fd[j] * n;
                if (!RMS) db[k][j] += fd[j];
            }
        }
        s1 = warp_sum(s1);
        s2 = warp_sum(s2);
        if (lane == 0) {
            red[par][0][warp] = s1;
            red[par][1][warp] = s2;
        }
        __syncthreads();   // the other parity's slots are free again once every warp has passed this point
        s1 = 0.f;
        s2 = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) {
            s1 += red[par][0][w];
            s2 += red[par][1][w];
        }
        s1 *= inv_c;
        s2 *= inv_c;
#pragma unroll
        for (int k = 0; k < NV; k++) {
            float fd[8], fx[8], fo[8];
            unpack8(dv[k], fd);
            unpack8(xv[k], fx);
            if (accumulate_dinp) unpack8(ov[k], fo);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float n = (fx[j] - m) * rs;
                const float dn = fd[j] * fw[k][j];
                const float d = RMS ? (dn - n * s2) * rs : (dn - s1 - n * s2) * rs;
                fo[j] = accumulate_dinp ? fo[j] + d : d;
            }
            st128(dinp + (size_t)row * C + (threadIdx.x + 256 * k) * 8, pack8(fo));
        }
#pragma unroll
        for (int k = 0; k < NV; k++) {
            dv[k] = dvn[k];
            xv[k] = xvn[k];
            ov[k] = ovn[k];
        }
    }
    float* dst = scratch + (size_t)blockIdx.x * 2 * C;
#pragma unroll
    for (int k = 0; k < NV; k++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
            dst[(threadIdx.x + 256 * k) * 8 + j] = dw[k][j];
            if (!RMS) dst[C + (threadIdx.x + 256 * k) * 8 + j] = db[k][j];
        }
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
    if (C % 256 == 0) {
        int grid = ceil_div(N, REG_WARPS);
        const int cap = num_sms() * 16;
        if (grid > cap) grid = cap;
#define LLMK_NORM_FWD_CASE(NV)                                                                                              \
    case NV:                                                                                                                \
        norm_fwd_reg_kernel<RMS, FUSED, NV><<<grid, REG_WARPS * 32, 0, stream>>>(normed, mean, rstd, residual, inp1, inp2,   \
                                                                                 weight, bias, N, eps);                     \
        LLMK_LAUNCH_CHECK();                                                                                                \
        return LLMK_OK;
        switch (C / 256) {
            LLMK_NORM_FWD_CASE(1)
            LLMK_NORM_FWD_CASE(2)
            LLMK_NORM_FWD_CASE(3)
            LLMK_NORM_FWD_CASE(4)
            LLMK_NORM_FWD_CASE(5)
            LLMK_NORM_FWD_CASE(6)
            LLMK_NORM_FWD_CASE(8)
            LLMK_NORM_FWD_CASE(16)
            default: break;
        }
#undef LLMK_NORM_FWD_CASE
    }
    const int smem = FWD_WARPS * C * 2;
    static PerDeviceOnce once_configured;
    if (once_configured.first()) {
        LLMK_CUDA_TRY(cudaFuncSetAttribute(norm_fwd_kernel<RMS, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           FWD_WARPS * 16384 * 2));
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
// Upper bound over both backward implementations (at most 4 blocks per SM).
LLMK_API long llmk_norm_bwd_scratch_bytes(int N, int C) { return (long)num_sms() * 4 * 2 * C * 4; }

namespace llmk {
namespace norm {
// Register-resident backward when C = 256 * NVEC and the accumulators fit; returns false if not applicable.
template <bool RMS, int NVEC>
static int launch_bwd_reg(bf16* dinp, bf16* dweight, bf16* dbias, float* scratch, const bf16* dout, const bf16* inp,
                          const bf16* weight, const float* mean, const float* rstd, int N, int accumulate_dinp,
                          cudaStream_t stream) {
    constexpr int C = NVEC * 256;
    if constexpr (NVEC <= 5) {
        using B = BulkCfg<NVEC>;
        static_assert(B::OFF_BAR >= B::WARPS * 2 * C * 4, "the rings must be able to hold the final reduction buffer");
        static PerDeviceOnce once_bulk_configured;
        if (once_bulk_configured.first()) {
            LLMK_CUDA_TRY(cudaFuncSetAttribute(norm_bwd_bulk_kernel<RMS, NVEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, B::SMEM));
        }
        int grid = num_sms();
        const int need = ceil_div(N, B::WARPS);
        if (grid > need) grid = need;
        norm_bwd_bulk_kernel<RMS, NVEC><<<grid, B::WARPS * 32, B::SMEM, stream>>>(dinp, scratch, dout, inp, weight, mean, rstd, N,
                                                                                 accumulate_dinp, current_status_word());
        LLMK_LAUNCH_CHECK();
        norm_bwd_finish_kernel<<<ceil_div(C, 32), dim3(32, 8), 0, stream>>>(dweight, dbias, scratch, grid, C);
        LLMK_LAUNCH_CHECK();
        return LLMK_OK;
    }
    constexpr int SMEM = REG_WARPS * (RMS ? 1 : 2) * C * 4;
    static PerDeviceOnce once_configured;
    if (once_configured.first()) {
        LLMK_CUDA_TRY(cudaFuncSetAttribute(norm_bwd_reg_kernel<RMS, NVEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    }
    int grid = num_sms() * 2;
    const int need = ceil_div(N, REG_WARPS);
    if (grid > need) grid = need;
    norm_bwd_reg_kernel<RMS, NVEC><<<grid, REG_WARPS * 32, SMEM, stream>>>(dinp, scratch, dout, inp, weight, mean, rstd, N,
                                                                          accumulate_dinp);
    LLMK_LAUNCH_CHECK();
    norm_bwd_finish_kernel<<<ceil_div(C, 32), dim3(32, 8), 0, stream>>>(dweight, dbias, scratch, grid, C);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
template <bool RMS, int NV>
static int launch_bwd_wide(bf16* dinp, bf16* dweight, bf16* dbias, float* scratch, const bf16* dout, const bf16* inp,
                           const bf16* weight, const float* mean, const float* rstd, int N, int accumulate_dinp,
                           cudaStream_t stream) {
    constexpr int C = NV * 2048;
    int grid = num_sms() * (NV <= 2 ? 2 : 1);
    if (grid > N) grid = N;
    norm_bwd_wide_kernel<RMS, NV><<<grid, 256, 0, stream>>>(dinp, scratch, dout, inp, weight, mean, rstd, N, accumulate_dinp);
    LLMK_LAUNCH_CHECK();
    norm_bwd_finish_kernel<<<ceil_div(C, 32), dim3(32, 8), 0, stream>>>(dweight, dbias, scratch, grid, C);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
}  // namespace norm
}  // namespace llmk

namespace llmk {
namespace norm {
// LayerNorm backward: launch of the row kernel plus the fixed-order partial reduction.
int layernorm_bwd_impl(bf16* dinp, bf16* dweight, bf16* dbias, float* scratch, const bf16* dout, const bf16* inp,
                       const bf16* weight, const float* mean, const float* rstd, int N, int C, int accumulate_dinp,
                       cudaStream_t stream) {
    if (C % 8 != 0 || C > 12288) return LLMK_ERR_SHAPE;
    switch (C % 2048 == 0 ? C / 2048 : 0) {
        case 1: return launch_bwd_wide<false, 1>(dinp, dweight, dbias, scratch, dout, inp, weight, mean, rstd, N, accumulate_dinp, stream);
        case 2: return launch_bwd_wide<false, 2>(dinp, dweight, dbias, scratch, dout, inp, weight, mean, rstd, N, accumulate_dinp, stream);
        case 3: return launch_bwd_wide<false, 3>(dinp, dweight, dbias, scratch, dout, inp, weight, mean, rstd, N, accumulate_dinp, stream);
        case 4: return launch_bwd_wide<false, 4>(dinp, dweight, dbias, scratch, dout, inp, weight, mean, rstd, N, accumulate_dinp, stream);
        case 6: return launch_bwd_wide<false, 6>(dinp, dweight, dbias, scratch, dout, inp, weight, mean, rstd, N, accumulate_dinp, stream);
        default: break;
    }
    switch (C % 256 == 0 ? C / 256 : 0) {
        case 1: return launch_bwd_reg<false, 1>(dinp, dweight, dbias, scratch, dout, inp, weight, mean, rstd, N, accumulate_dinp, stream);
        case 2: return launch_bwd_reg<false, 2>(dinp, dweight, dbias, scratch, dout, inp, weight, mean, rstd, N, accumulate_dinp, stream);
        case 3: return launch_bwd_reg<false, 3>(dinp, dweight, dbias, scratch, dout, inp, weight, mean, rstd, N, accumulate_dinp, stream);
        case 4: return launch_bwd_reg<false, 4>(dinp, dweight, dbias, scratch, dout, inp, weight, mean, rstd, N, accumulate_dinp, stream);
        case 5: return launch_bwd_reg<false, 5>(dinp, dweight, dbias, scratch, dout, inp, weight, mean, rstd, N, accumulate_dinp, stream);
        default: break;
    }
    static PerDeviceOnce once_configured;
    if (once_configured.first()) {
        LLMK_CUDA_TRY(cudaFuncSetAttribute(norm_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           BWD_WARPS * 2 * 6144 * 4));
    }
    const int smem = BWD_WARPS * 2 * C * 4;
    if (smem > BWD_WARPS * 2 * 6144 * 4) return LLMK_ERR_SHAPE;
    const int grid = llmk_norm_bwd_blocks(N, C);
    norm_bwd_kernel<false><<<grid, BWD_WARPS * 32, smem, stream>>>(dinp, scratch, dout, inp, weight, mean, rstd, N, C,
                                                                  accumulate_dinp);
    LLMK_LAUNCH_CHECK();
    norm_bwd_finish_kernel<<<ceil_div(C, 32), dim3(32, 8), 0, stream>>>(dweight, dbias, scratch, grid, C);
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
#define LLMK_RMS_BWD_CASE(NV)                                                                                             \
    case NV:                                                                                                              \
        return launch_bwd_reg<true, NV>((bf16*)dinp, (bf16*)dweight, nullptr, (float*)scratch, (const bf16*)dout,         \
                                        (const bf16*)inp, (const bf16*)weight, nullptr, (const float*)rstd, N,            \
                                        accumulate_dinp, stream);
#define LLMK_RMS_WIDE_CASE(NV)                                                                                            \
    case NV:                                                                                                              \
        return launch_bwd_wide<true, NV>((bf16*)dinp, (bf16*)dweight, nullptr, (float*)scratch, (const bf16*)dout,        \
                                         (const bf16*)inp, (const bf16*)weight, nullptr, (const float*)rstd, N,           \
                                         accumulate_dinp, stream);
    switch (C % 2048 == 0 ? C / 2048 : 0) {
        LLMK_RMS_WIDE_CASE(1)
        LLMK_RMS_WIDE_CASE(2)
        LLMK_RMS_WIDE_CASE(3)
        LLMK_RMS_WIDE_CASE(4)
        LLMK_RMS_WIDE_CASE(6)
        default: break;
    }
#undef LLMK_RMS_WIDE_CASE
    switch (C % 256 == 0 ? C / 256 : 0) {
        LLMK_RMS_BWD_CASE(1)
        LLMK_RMS_BWD_CASE(2)
        LLMK_RMS_BWD_CASE(3)
        LLMK_RMS_BWD_CASE(4)
        LLMK_RMS_BWD_CASE(5)
        default: break;
    }
#undef LLMK_RMS_BWD_CASE
    static PerDeviceOnce once_configured;
    if (once_configured.first()) {
        LLMK_CUDA_TRY(cudaFuncSetAttribute(norm_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           BWD_WARPS * 12288 * 4));
    }
    const int smem = BWD_WARPS * C * 4;
    const int grid = llmk_norm_bwd_blocks(N, C);
    norm_bwd_kernel<true><<<grid, BWD_WARPS * 32, smem, stream>>>((bf16*)dinp, (float*)scratch, (const bf16*)dout,
                                                                 (const bf16*)inp, (const bf16*)weight, nullptr,
                                                                 (const float*)rstd, N, C, accumulate_dinp);
    LLMK_LAUNCH_CHECK();
    norm_bwd_finish_kernel<<<ceil_div(C, 32), dim3(32, 8), 0, stream>>>((bf16*)dweight, nullptr, (const float*)scratch, grid, C);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
