// Causal flash-attention FORWARD on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// TMEM), for MHA and GQA, reading the packed QKV activation [B*T, (NH+2*NKVH)*HS] through one TMA
// tensor map and writing O as [B*T, NH*HS] plus the log-sum-exp. Same job as attention_forward /
// attention_gqa_forward of the reference (llmc/attention.cuh:261-338, llmc/attention_gqa.cuh:415-481),
// which has no sm_100 path; the warp-level implementation in attention.cu remains as the fallback for
// sequence lengths that are not a multiple of 128.
//
// One CTA per (128 query rows, head, batch); 6 warps:
//   warp 0     TMA producer: Q once, then K/V tiles of 128 rows through a 2-stage ring
//   warp 1     MMA issuer:   S = Q K^T  (128x128xHS, both operands K-major)  -> TMEM columns [0,128)
//                            O_j = P V  (128xHSx128, P K-major from smem, V MN-major) -> TMEM [128,128+HS)
//   warps 2-5  softmax:      one query row per thread (TMEM lane = row, so no cross-thread reductions):
//                            pass 1 reads S for the row maximum, pass 2 re-reads it, writes
//                            P = exp2(S*c - m) as bf16 into 128-byte-swizzled smem for the second MMA and
//                            keeps the running O in registers (O = O*alpha + O_j after each P V).
// TMEM use is 256 columns and shared memory 112 KB for HS = 64, so two CTAs share an SM and one's
// softmax overlaps the other's MMAs. Every wait is bounded and reports through the status word.
#include "ptx_sm100.cuh"

namespace llmk {
namespace gemm {
int make_tmap_2d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_elems, uint32_t box_inner,
                 uint32_t box_outer);
}
namespace attn_tc {

constexpr int BQ = 128, BKV = 128;
constexpr int THREADS = 192;
constexpr int ATOM_BYTES = 128 * 128;  // one 128-row x 64-column (128-byte) swizzle atom column

template <int HS>
struct Cfg {
    static constexpr int TILE_BYTES = BQ * HS * 2;         // Q, K or V tile
    static constexpr int P_BYTES = BQ * BKV * 2;
    static constexpr int SMEM_MAIN = TILE_BYTES * 5 + P_BYTES;
    static constexpr int SMEM_BYTES = SMEM_MAIN + 128;   // tiles + barriers; the dynamic window itself is 1024-byte aligned
    static constexpr int TMEM_COLS = 256;
    static constexpr int CTAS_PER_SM = HS == 64 ? 2 : 1;
};


__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Row maximum over the 128 S columns of this thread's TMEM lane; `DIAG` masks columns after the row.
// The four 32-column loads are double buffered so a load is in flight while the previous chunk is reduced.
template <bool DIAG>
__device__ __forceinline__ float row_max(uint32_t taddr, int r) {
    uint32_t va[32], vb[32];
    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
    ptx::tmem_ld_32x32b_x32(taddr, va);
#pragma unroll
    for (int c4 = 0; c4 < 4; c4++) {
        ptx::tmem_ld_wait();
        uint32_t* cur = (c4 & 1) ? vb : va;
        if (c4 < 3) ptx::tmem_ld_32x32b_x32(taddr + (c4 + 1) * 32, (c4 & 1) ? va : vb);
        if (!DIAG || c4 * 32 <= r) {  // whole chunk masked otherwise
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                float x0 = __uint_as_float(cur[i]), x1 = __uint_as_float(cur[i + 1]);
                float x2 = __uint_as_float(cur[i + 2]), x3 = __uint_as_float(cur[i + 3]);
                if (DIAG) {
                    const int c = c4 * 32 + i;
                    if (c > r) x0 = -INFINITY;
                    if (c + 1 > r) x1 = -INFINITY;
                    if (c + 2 > r) x2 = -INFINITY;
                    if (c + 3 > r) x3 = -INFINITY;
                }
                m0 = fmaxf(m0, x0); m1 = fmaxf(m1, x1); m2 = fmaxf(m2, x2); m3 = fmaxf(m3, x3);
            }
        }
    }
    return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// P = exp2(S*c - m) as bf16 into the swizzled A-operand tile of this row; returns the row sum.
template <bool DIAG>
__device__ __forceinline__ float row_probs(uint32_t taddr, uint8_t* sP, int r, float scale_log2, float m_new) {
    uint32_t va[32], vb[32];
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    const float neg_m = -m_new;
    ptx::tmem_ld_32x32b_x32(taddr, va);
#pragma unroll
    for (int c4 = 0; c4 < 4; c4++) {
        ptx::tmem_ld_wait();
        uint32_t* cur = (c4 & 1) ? vb : va;
        if (c4 < 3) ptx::tmem_ld_32x32b_x32(taddr + (c4 + 1) * 32, (c4 & 1) ? va : vb);
        uint8_t* atom = sP + (c4 >> 1) * ATOM_BYTES + r * 128;
#pragma unroll
        for (int q = 0; q < 4; q++) {
            float p[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                float e = ex2(fmaf(__uint_as_float(cur[q * 8 + i]), scale_log2, neg_m));
                if (DIAG && c4 * 32 + q * 8 + i > r) e = 0.f;
                p[i] = e;
            }
            s0 += p[0] + p[4]; s1 += p[1] + p[5]; s2 += p[2] + p[6]; s3 += p[3] + p[7];
            const int chunk = (c4 & 1) * 4 + q;
            *reinterpret_cast<bf16x8*>(atom + ((chunk ^ (r & 7)) << 4)) = pack8(p);
        }
    }
    return (s0 + s1) + (s2 + s3);
}

template <int HS>
__global__ void __launch_bounds__(THREADS, Cfg<HS>::CTAS_PER_SM)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQKV, bf16* __restrict__ out, float* __restrict__ lse, int T, int NH,
                   int NKVH, float scale_log2, int* status) {
    using C = Cfg<HS>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    if (ptx::smem_u32(smem) & 1023u) {  // swizzled tiles need a 1024-byte aligned window: refuse instead of corrupting
        if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, LLMK_ST_BOUNDS);
        return;
    }
    uint8_t* sQ = smem;
    uint8_t* sK = smem + C::TILE_BYTES;          // [2]
    uint8_t* sV = smem + 3 * C::TILE_BYTES;      // [2]
    uint8_t* sP = smem + 5 * C::TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::SMEM_MAIN);
    uint64_t* q_full = bars;          // [1]
    uint64_t* kv_full = bars + 1;     // [2]
    uint64_t* kv_empty = bars + 3;    // [2]
    uint64_t* s_full = bars + 5;      // [1]
    uint64_t* p_full = bars + 6;      // [1]
    uint64_t* o_full = bars + 7;      // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb = gridDim.x - 1 - blockIdx.x;  // late (long) query blocks first
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (NH / NKVH);
    const int nkv = qb + 1;
    const int row_base = b * T;
    const int q_col = h * HS, k_col = (NH + hk) * HS, v_col = (NH + NKVH + hk) * HS;

    if (threadIdx.x == 0) {
        ptx::mbar_init(q_full, 1);
        for (int i = 0; i < 2; i++) {
            ptx::mbar_init(&kv_full[i], 1);
            ptx::mbar_init(&kv_empty[i], 1);
        }
        ptx::mbar_init(s_full, 1);
        ptx::mbar_init(p_full, 4);
        ptx::mbar_init(o_full, 1);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&tmQKV);
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, C::TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ptx::mbar_arrive_expect_tx(q_full, C::TILE_BYTES);
#pragma unroll
            for (int c = 0; c < HS / 64; c++) ptx::tma_load_2d(sQ + c * ATOM_BYTES, &tmQKV, q_full, q_col + 64 * c, row_base + qb * BQ);
        }
        __syncwarp();
        for (int j = 0; j < nkv; j++) {
            const int s = j & 1;
            if (!ptx::mbar_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag, status, LLMK_ST_TIMEOUT_TMA_EMPTY, j)) break;
            if (lane == 0) {
                ptx::mbar_arrive_expect_tx(&kv_full[s], 2 * C::TILE_BYTES);
#pragma unroll
                for (int c = 0; c < HS / 64; c++) {
                    ptx::tma_load_2d(sK + s * C::TILE_BYTES + c * ATOM_BYTES, &tmQKV, &kv_full[s], k_col + 64 * c, row_base + j * BKV);
                    ptx::tma_load_2d(sV + s * C::TILE_BYTES + c * ATOM_BYTES, &tmQKV, &kv_full[s], v_col + 64 * c, row_base + j * BKV);
                }
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc_s = ptx::make_idesc_bf16(BQ, BKV, 0, 0);
        constexpr uint32_t idesc_o = ptx::make_idesc_bf16(BQ, HS, 0, 1);
        bool ok = ptx::mbar_wait(q_full, 0, abort_flag, status, LLMK_ST_TIMEOUT_TMA_FULL, -1);
        // S(j+1) is issued BEFORE P V(j): the tensor core works through them in order, so the softmax of
        // tile j+1 can start while P V(j) is still running.
        auto issue_s = [&](int j) -> bool {
            const int s = j & 1;
            if (!ptx::mbar_wait(&kv_full[s], (j >> 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_TMA_FULL, j)) return false;
            ptx::tc_fence_after();
            if (lane == 0) {
                const uint32_t q_addr = ptx::smem_u32(sQ), k_addr = ptx::smem_u32(sK + s * C::TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < HS / 16; kk++) {
                    const uint32_t off = (kk / 4) * ATOM_BYTES + (kk % 4) * 32;
                    ptx::mma_f16_ss(tmem_s, ptx::make_smem_desc(q_addr + off, 16, 1024), ptx::make_smem_desc(k_addr + off, 16, 1024),
                                    idesc_s, kk > 0 ? 1u : 0u);
                }
                ptx::mma_commit(s_full);
            }
            __syncwarp();
            return true;
        };
        if (ok) ok = issue_s(0);
        for (int j = 0; j < nkv && ok; j++) {
            const int s = j & 1;
            // P(j) is in shared memory and S(j) has been consumed
            ok = ptx::mbar_wait(p_full, j & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_EMPTY, j);
            if (!ok) break;
            ptx::tc_fence_after();
            if (j + 1 < nkv) {
                ok = issue_s(j + 1);
                if (!ok) break;
            }
            if (lane == 0) {
                const uint32_t p_addr = ptx::smem_u32(sP), v_addr = ptx::smem_u32(sV + s * C::TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < BKV / 16; kk++) {
                    const uint64_t adesc = ptx::make_smem_desc(p_addr + (kk / 4) * ATOM_BYTES + (kk % 4) * 32, 16, 1024);
                    const uint64_t bdesc = ptx::make_smem_desc(v_addr + kk * 2048, ATOM_BYTES, 1024);
                    ptx::mma_f16_ss(tmem_o, adesc, bdesc, idesc_o, kk > 0 ? 1u : 0u);
                }
                ptx::mma_commit(&kv_empty[s]);
                ptx::mma_commit(o_full);
            }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------ softmax warps (one query row per thread)
        const int lane_group = warp & 3;
        const int r = lane_group * 32 + lane;
        const uint32_t lane_off = (uint32_t)(lane_group * 32) << 16;
        float o_reg[HS];
#pragma unroll
        for (int i = 0; i < HS; i++) o_reg[i] = 0.f;
        float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
        bool ok = true;
        for (int j = 0; j < nkv && ok; j++) {
            ok = ptx::mbar_wait(s_full, j & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, j);
            if (!ok) break;
            ptx::tc_fence_after();
            const bool diag = (j == nkv - 1);
            // pass 1: row maximum
            const float mx = diag ? row_max<true>(tmem_s + lane_off, r) : row_max<false>(tmem_s + lane_off, r);
            const float m_new = fmaxf(m, mx * scale_log2);
            const float alpha = ex2(m - m_new);
            // the previous tile's P V must be complete before P and the O accumulator are reused
            if (j > 0) {
                ok = ptx::mbar_wait(o_full, (j - 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, 1000 + j);
                if (!ok) break;
                ptx::tc_fence_after();
#pragma unroll
                for (int h4 = 0; h4 < HS / 32; h4++) {
                    uint32_t v[32];
                    ptx::tmem_ld_32x32b_x32(tmem_o + lane_off + h4 * 32, v);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) o_reg[h4 * 32 + i] = o_reg[h4 * 32 + i] * alpha_prev + __uint_as_float(v[i]);
                }
            }
            // pass 2: probabilities -> smem (A operand of the second MMA), row sum
            const float rs = diag ? row_probs<true>(tmem_s + lane_off, sP, r, scale_log2, m_new)
                                  : row_probs<false>(tmem_s + lane_off, sP, r, scale_log2, m_new);
            l = l * alpha + rs;
            m = m_new;
            alpha_prev = alpha;
            ptx::tc_fence_before();
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(p_full);
        }
        if (ok) {
            ok = ptx::mbar_wait(o_full, (nkv - 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, 2000);
            if (ok) {
                ptx::tc_fence_after();
                const float inv_l = 1.0f / l;
                bf16* orow = out + ((size_t)(row_base + qb * BQ + r) * NH + h) * HS;
#pragma unroll
                for (int h4 = 0; h4 < HS / 32; h4++) {
                    uint32_t v[32];
                    ptx::tmem_ld_32x32b_x32(tmem_o + lane_off + h4 * 32, v);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        float f[8];
#pragma unroll
                        for (int i = 0; i < 8; i++)
                            f[i] = (o_reg[h4 * 32 + q * 8 + i] * alpha_prev + __uint_as_float(v[q * 8 + i])) * inv_l;
                        st128(orow + h4 * 32 + q * 8, pack8(f));
                    }
                }
                lse[((size_t)b * NH + h) * T + qb * BQ + r] = (m + log2f(l)) * 0.6931471805599453f;
            }
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

template <int HS>
static int launch(const CUtensorMap& tm, bf16* out, float* lse, int B, int T, int NH, int NKVH, int* status, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        LLMK_CUDA_TRY(cudaFuncSetAttribute(attn_fwd_tc_kernel<HS>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<HS>::SMEM_BYTES));
        LLMK_CUDA_TRY(cudaFuncSetAttribute(attn_fwd_tc_kernel<HS>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                           cudaSharedmemCarveoutMaxShared));
        configured = true;
    }
    const float scale_log2 = 1.4426950408889634f / sqrtf((float)HS);
    dim3 grid(T / BQ, NH, B);
    attn_fwd_tc_kernel<HS><<<grid, THREADS, Cfg<HS>::SMEM_BYTES, stream>>>(tm, out, lse, T, NH, NKVH, scale_log2, status);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

}  // namespace attn_tc
}  // namespace llmk

using namespace llmk;

// Same contract as llmk_attention_fwd, but T must be a multiple of 128.
LLMK_API int llmk_attention_fwd_tc(void* out, void* lse, const void* qkv, int B, int T, int NH, int NKVH, int HS, int* status,
                                   void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (T % 128 || NH % NKVH || (HS != 64 && HS != 128)) return LLMK_ERR_SHAPE;
    const long width = (long)(NH + 2 * NKVH) * HS;
    CUtensorMap tm;
    const int rc = gemm::make_tmap_2d(&tm, qkv, (uint64_t)width, (uint64_t)B * T, (uint64_t)width, 64, 128);
    if (rc) return rc;
    if (HS == 64) return attn_tc::launch<64>(tm, (bf16*)out, (float*)lse, B, T, NH, NKVH, status, stream);
    return attn_tc::launch<128>(tm, (bf16*)out, (float*)lse, B, T, NH, NKVH, status, stream);
}
