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
//                            copies its S row into registers and releases the S buffer at once (the next
//                            S = Q K^T runs during this tile's softmax), writes P = exp2(S*c - m) as bf16
//                            into 128-byte-swizzled smem for the second MMA. O accumulates in TMEM over
//                            all tiles; m trails the running maximum and O, l are rescaled (TMEM load,
//                            multiply, store) only when a row maximum jumps by more than 2^8.
// TMEM use is 256 columns and shared memory 112 KB for HS = 64, so two CTAs share an SM and one's
// softmax overlaps the other's MMAs. Every wait is bounded and reports through the status word.
#include <cstdlib>

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
    static constexpr int CTAS_PER_SM = 1;   // 128 S values per thread live in registers: two CTAs per SM would spill
};


__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two fp32 -> packed bf16x2 by keeping the upper halves (one byte-permute on the integer pipe). The
// conversion instruction shares the transcendental unit with ex2, which is the bottleneck of the softmax;
// the callers fold log2(1 + 2^-9) into the exponent so that the truncation is unbiased on average.
__device__ __forceinline__ uint32_t pack_trunc2(float lo, float hi) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(d) : "r"(__float_as_uint(lo)), "r"(__float_as_uint(hi)));
    return d;
}
constexpr float TRUNC_BIAS_LOG2 = 0.0028150156f;   // log2(1 + 2^-9)

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Maximum of one 32-column chunk of this thread's S row; `MASK` drops the columns after `lane`
// (the chunk that holds the diagonal of a diagonal tile).
template <bool MASK>
__device__ __forceinline__ float chunk_max(const uint32_t (&s)[32], int lane, float acc) {
    float a0 = acc, a1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        float x0 = __uint_as_float(s[i]), x1 = __uint_as_float(s[i + 1]);
        float x2 = __uint_as_float(s[i + 2]), x3 = __uint_as_float(s[i + 3]);
        if (MASK) {
            if (i > lane) x0 = -INFINITY;
            if (i + 1 > lane) x1 = -INFINITY;
            if (i + 2 > lane) x2 = -INFINITY;
            if (i + 3 > lane) x3 = -INFINITY;
        }
        a0 = max3(a0, x0, x1);
        a1 = max3(a1, x2, x3);
    }
    return fmaxf(a0, a1);
}

// P = exp2(S*c - m) of one 32-column chunk as bf16 into the swizzled A-operand tile; returns the chunk's sum.
// MODE 0: plain, 1: mask the columns after `lane`, 2: the whole chunk is masked (zeros).
template <int MODE>
__device__ __forceinline__ float chunk_probs(const uint32_t (&s)[32], uint8_t* atom, int chunk_base, int r, int lane,
                                             float scale_log2, float neg_m) {
    // packed fp32 pairs: one FMA-pipe instruction per two columns for the exponent argument and the row sum
    const ptx::f32x2 c2 = ptx::pack2(scale_log2, scale_log2), m2 = ptx::pack2(neg_m, neg_m);
    ptx::f32x2 sum2 = ptx::pack2(0.f, 0.f);
#pragma unroll
    for (int q = 0; q < 4; q++) {
        float p[8];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            float e0 = 0.f, e1 = 0.f;
            if (MODE != 2) {
                float x0, x1;
                ptx::unpack2(ptx::fma2(ptx::pack2(__uint_as_float(s[q * 8 + i]), __uint_as_float(s[q * 8 + i + 1])), c2, m2), x0, x1);
                e0 = ex2(x0);
                e1 = ex2(x1);
                if (MODE == 1 && q * 8 + i > lane) e0 = 0.f;
                if (MODE == 1 && q * 8 + i + 1 > lane) e1 = 0.f;
            }
            p[i] = e0;
            p[i + 1] = e1;
        }
        if (MODE != 2) {
#pragma unroll
            for (int i = 0; i < 8; i += 2) sum2 = ptx::add2(sum2, ptx::pack2(p[i], p[i + 1]));
        }
        uint4 w;
        w.x = pack_trunc2(p[0], p[1]);
        w.y = pack_trunc2(p[2], p[3]);
        w.z = pack_trunc2(p[4], p[5]);
        w.w = pack_trunc2(p[6], p[7]);
        *reinterpret_cast<uint4*>(atom + (((chunk_base + q) ^ (r & 7)) << 4)) = w;
    }
    float s0, s1;
    ptx::unpack2(sum2, s0, s1);
    return s0 + s1;
}

template <int HS>
__global__ void __launch_bounds__(THREADS, Cfg<HS>::CTAS_PER_SM)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmKV, bf16* __restrict__ out,
                   float* __restrict__ lse, int T, int Tkv, int causal, int NH, int NKVH, float scale_log2, int* status) {
    // tmKV / Tkv / causal: the keys and values may come from ANOTHER packed QKV tensor of the same layout (a peer's
    // chunk of the sequence in context-parallel attention; the map may cover that peer's memory, loads only, no
    // multicast). causal = 1: queries and keys cover the same positions (the usual case, tmKV == tmQKV); causal = 0:
    // every key precedes every query, all Tkv / 128 key tiles are used unmasked.
    using C = Cfg<HS>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    {   // a failure already recorded in the status word (by an earlier CTA or kernel) makes the rest return at once
        __shared__ int skip;
        if (threadIdx.x == 0) skip = (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0);
        __syncthreads();
        if (skip) return;
    }
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
    uint64_t* s_free = bars + 8;      // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb = gridDim.x - 1 - blockIdx.x;  // late (long) query blocks first
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (NH / NKVH);
    const int nkv = causal ? qb + 1 : Tkv / BKV;
    const int row_base = b * T, kv_row_base = b * Tkv;
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
        ptx::mbar_init(s_free, 4);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&tmQKV);
        ptx::prefetch_tmap(&tmKV);
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
                    ptx::tma_load_2d(sK + s * C::TILE_BYTES + c * ATOM_BYTES, &tmKV, &kv_full[s], k_col + 64 * c, kv_row_base + j * BKV);
                    ptx::tma_load_2d(sV + s * C::TILE_BYTES + c * ATOM_BYTES, &tmKV, &kv_full[s], v_col + 64 * c, kv_row_base + j * BKV);
                }
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc_s = ptx::make_idesc_bf16(BQ, BKV, 0, 0);
        constexpr uint32_t idesc_o = ptx::make_idesc_bf16(BQ, HS, 0, 1);
        bool ok = ptx::mbar_wait(q_full, 0, abort_flag, status, LLMK_ST_TIMEOUT_TMA_FULL, -1);
        // S(j+1) is issued as soon as the softmax warps have copied S(j) into registers (s_free), i.e. while
        // they are still working on tile j; P V(j) follows when P(j) is in shared memory. O accumulates in TMEM.
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
            if (j + 1 < nkv) {
                ok = ptx::mbar_wait(s_free, j & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_EMPTY, 3000 + j);
                if (!ok) break;
                ptx::tc_fence_after();
                ok = issue_s(j + 1);
                if (!ok) break;
            }
            // P(j) is in shared memory (and O has been rescaled if the row maxima moved)
            ok = ptx::mbar_wait(p_full, j & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_EMPTY, j);
            if (!ok) break;
            ptx::tc_fence_after();
            if (lane == 0) {
                const uint32_t p_addr = ptx::smem_u32(sP), v_addr = ptx::smem_u32(sV + s * C::TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < BKV / 16; kk++) {
                    const uint64_t adesc = ptx::make_smem_desc(p_addr + (kk / 4) * ATOM_BYTES + (kk % 4) * 32, 16, 1024);
                    const uint64_t bdesc = ptx::make_smem_desc(v_addr + kk * 2048, ATOM_BYTES, 1024);
                    ptx::mma_f16_ss(tmem_o, adesc, bdesc, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
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
        // m is the reference maximum of the exponentials (log2 units); it trails the true running maximum by at
        // most RESCALE_GAP, so P stays below 2^RESCALE_GAP and O / l are rescaled only when a row maximum jumps.
        constexpr float RESCALE_GAP = 8.f;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < nkv && ok; j++) {
            ok = ptx::mbar_wait(s_full, j & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, j);
            if (!ok) break;
            ptx::tc_fence_after();
            const bool diag = causal && (j == nkv - 1);
            const int nchunks = diag ? lane_group + 1 : 4;   // warp-uniform: later chunks are fully masked
            uint32_t s[4][32];
#pragma unroll
            for (int c4 = 0; c4 < 4; c4++)
                if (c4 < nchunks) ptx::tmem_ld_32x32b_x32(tmem_s + lane_off + c4 * 32, s[c4]);
            ptx::tmem_ld_wait();
            // S(j) now lives in registers: hand the TMEM buffer back so that S(j+1) can be computed meanwhile
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(s_free);
            float mx = -INFINITY;
#pragma unroll
            for (int c4 = 0; c4 < 4; c4++) {
                if (c4 < nchunks) {
                    if (diag && c4 == lane_group) mx = chunk_max<true>(s[c4], lane, mx);
                    else mx = chunk_max<false>(s[c4], lane, mx);
                }
            }
            const float m_new = fmaxf(m, mx * scale_log2);
            if (j > 0) {
                // P V(j-1) must be complete before P is overwritten and before O may be rescaled
                ok = ptx::mbar_wait(o_full, (j - 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, 1000 + j);
                if (!ok) break;
                ptx::tc_fence_after();
                if (__any_sync(0xffffffffu, m_new > m + RESCALE_GAP)) {
                    const float alpha = ex2(m - m_new);
                    l *= alpha;
                    m = m_new;
#pragma unroll
                    for (int h4 = 0; h4 < HS / 32; h4++) {
                        uint32_t v[32];
                        ptx::tmem_ld_32x32b_x32(tmem_o + lane_off + h4 * 32, v);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        ptx::tmem_st_32x32b_x32(tmem_o + lane_off + h4 * 32, v);
                    }
                    ptx::tmem_st_wait();
                }
            } else {
                m = m_new;
            }
            const float neg_m = TRUNC_BIAS_LOG2 - m;   // P is truncated to bf16: see pack_trunc2
            float rs = 0.f;
#pragma unroll
            for (int c4 = 0; c4 < 4; c4++) {
                uint8_t* atom = sP + (c4 >> 1) * ATOM_BYTES + r * 128;
                const int cb = (c4 & 1) * 4;
                if (c4 >= nchunks) chunk_probs<2>(s[c4], atom, cb, r, lane, scale_log2, neg_m);
                else if (diag && c4 == lane_group) rs += chunk_probs<1>(s[c4], atom, cb, r, lane, scale_log2, neg_m);
                else rs += chunk_probs<0>(s[c4], atom, cb, r, lane, scale_log2, neg_m);
            }
            l += rs;
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
                        for (int i = 0; i < 8; i++) f[i] = __uint_as_float(v[q * 8 + i]) * inv_l;
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
static int launch(const CUtensorMap& tm, const CUtensorMap& tm_kv, bf16* out, float* lse, int B, int T, int Tkv, int causal, int NH,
                  int NKVH, int* status, cudaStream_t stream) {
    static PerDeviceOnce once_configured;
    if (once_configured.first()) {
        LLMK_CUDA_TRY(cudaFuncSetAttribute(attn_fwd_tc_kernel<HS>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<HS>::SMEM_BYTES));
        LLMK_CUDA_TRY(cudaFuncSetAttribute(attn_fwd_tc_kernel<HS>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                           cudaSharedmemCarveoutMaxShared));
    }
    const float scale_log2 = 1.4426950408889634f / sqrtf((float)HS);
    dim3 grid(T / BQ, NH, B);
    attn_fwd_tc_kernel<HS><<<grid, THREADS, Cfg<HS>::SMEM_BYTES, stream>>>(tm, tm_kv, out, lse, T, Tkv, causal, NH, NKVH, scale_log2,
                                                                            status);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}


// =====================================================================================================
// HS = 64: two 128-row query tiles per CTA (one CTA per SM), each with its own softmax warpgroup,
// S / O accumulators and P buffer, sharing the K / V tiles of a 3-stage ring. While one warpgroup runs
// its softmax the tensor core works for the other one, and K / V are read once for 256 query rows.
//   warp 0      TMA producer (Q tiles once, K/V ring)
//   warp 1      MMA issuer: per K/V tile j   S_0(j), S_1(j), then P_0 V(j-1), P_1 V(j-1)
//   warps 4-7   softmax of query rows [0,128) of the block; warps 8-11 of rows [128,256)
// The first warpgroup gives most of its registers back (setmaxnreg) so that the softmax threads can hold
// a whole 128-column S row in registers without spilling.
// TMEM (all 512 columns): S_0 [0,128)  S_1 [128,256)  O_0 [256,320)  O_1 [320,384).
// O leaves through shared memory (the warpgroup's P buffer) and one TMA store per 128x64 tile.
namespace pair {
constexpr int HS = 64;
constexpr int STAGES = 3;
constexpr int THREADS = 384;   // warpgroup 0: producer, MMA issuer, two idle warps; warpgroups 1 and 2: softmax
constexpr int TILE_BYTES = BQ * HS * 2;
constexpr int P_BYTES = BQ * BKV * 2;
constexpr int SMEM_MAIN = 2 * TILE_BYTES + 2 * STAGES * TILE_BYTES + 2 * P_BYTES;
constexpr int SMEM_BYTES = SMEM_MAIN + 256;

__global__ void __launch_bounds__(THREADS, 1)
attn_fwd_pair_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmOut, float* __restrict__ lse,
                     int T, int NH, int NKVH, float scale_log2, int* status) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    {   // a failure already recorded in the status word (by an earlier CTA or kernel) makes the rest return at once
        __shared__ int skip;
        if (threadIdx.x == 0) skip = (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0);
        __syncthreads();
        if (skip) return;
    }
    if (ptx::smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, LLMK_ST_BOUNDS);
        return;
    }
    uint8_t* sQ = smem;                                  // [2]
    uint8_t* sK = smem + 2 * TILE_BYTES;                 // [STAGES]
    uint8_t* sV = sK + STAGES * TILE_BYTES;              // [STAGES]
    uint8_t* sP = sV + STAGES * TILE_BYTES;              // [2]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_MAIN);
    uint64_t* q_full = bars;                 // [1]
    uint64_t* kv_full = bars + 1;            // [STAGES]
    uint64_t* kv_empty = kv_full + STAGES;   // [STAGES]
    uint64_t* s_full = kv_empty + STAGES;    // [2]
    uint64_t* s_free = s_full + 2;           // [2]
    uint64_t* p_full = s_free + 2;           // [2]
    uint64_t* o_full = p_full + 2;           // [2]
    uint64_t* epi = o_full + 2;              // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(epi + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb2 = gridDim.x - 1 - blockIdx.x;  // late (long) query blocks first
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (NH / NKVH);
    const int row_base = b * T;
    const int q_col = h * HS, k_col = (NH + hk) * HS, v_col = (NH + NKVH + hk) * HS;
    // tiles per half: the diagonal tile of half i is tile 2*qb2+i; a half past the end of the sequence is idle
    const int n0 = 2 * qb2 + 1;
    const int n1 = ((2 * qb2 + 1) * BQ < T) ? 2 * qb2 + 2 : 0;
    const int nmax = n1 > n0 ? n1 : n0;

    if (threadIdx.x == 0) {
        ptx::mbar_init(q_full, 1);
        for (int i = 0; i < STAGES; i++) {
            ptx::mbar_init(&kv_full[i], 1);
            ptx::mbar_init(&kv_empty[i], 2);   // one arrival per issuer warp
        }
        for (int i = 0; i < 2; i++) {
            ptx::mbar_init(&s_full[i], 1);
            ptx::mbar_init(&s_free[i], 4);
            ptx::mbar_init(&p_full[i], 4);
            ptx::mbar_init(&o_full[i], 1);
            ptx::mbar_init(&epi[i], 4);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&tmQKV);
        ptx::prefetch_tmap(&tmOut);
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, 512);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ptx::mbar_arrive_expect_tx(q_full, (n1 ? 2 : 1) * TILE_BYTES);
            ptx::tma_load_2d(sQ, &tmQKV, q_full, q_col, row_base + qb2 * 2 * BQ);
            if (n1) ptx::tma_load_2d(sQ + TILE_BYTES, &tmQKV, q_full, q_col, row_base + qb2 * 2 * BQ + BQ);
        }
        __syncwarp();
        for (int j = 0; j < nmax; j++) {
            const int s = j % STAGES;
            if (!ptx::mbar_wait(&kv_empty[s], ((j / STAGES) & 1) ^ 1, abort_flag, status, LLMK_ST_TIMEOUT_TMA_EMPTY, j)) break;
            if (lane == 0) {
                ptx::mbar_arrive_expect_tx(&kv_full[s], 2 * TILE_BYTES);
                ptx::tma_load_2d(sK + s * TILE_BYTES, &tmQKV, &kv_full[s], k_col, row_base + j * BKV);
                ptx::tma_load_2d(sV + s * TILE_BYTES, &tmQKV, &kv_full[s], v_col, row_base + j * BKV);
            }
            __syncwarp();
        }
    } else if (warp == 1 || warp == 2) {
        // ------------------------------------------------------------ MMA issuers: warp 1 for half 0, warp 2 for half 1
        // Per K/V tile j: S_i(j) once K(j) has landed and the warpgroup has copied S_i(j-1) out of TMEM (early in
        // its tile), then P_i V(j-1) once P_i(j-1) is in shared memory. The descriptors are built once: inside
        // the loop an MMA costs one integer add, which matters because these warps share their schedulers with
        // the softmax warps.
        const int i = warp - 1;
        const int ni = i ? n1 : n0;
        if (lane == 0) {
            constexpr uint32_t idesc_s = ptx::make_idesc_bf16(BQ, BKV, 0, 0);
            constexpr uint32_t idesc_o = ptx::make_idesc_bf16(BQ, HS, 0, 1);
            const uint32_t tmem_s = tmem_base + i * 128, tmem_o = tmem_base + 256 + i * HS;
            const uint64_t q_desc = ptx::make_smem_desc(ptx::smem_u32(sQ + i * TILE_BYTES), 16, 1024);
            const uint64_t k_desc = ptx::make_smem_desc(ptx::smem_u32(sK), 16, 1024);
            const uint64_t p_desc = ptx::make_smem_desc(ptx::smem_u32(sP + i * P_BYTES), 16, 1024);
            const uint64_t v_desc = ptx::make_smem_desc(ptx::smem_u32(sV), ATOM_BYTES, 1024);
            bool ok = ptx::mbar_wait_spin(q_full, 0, abort_flag, status, LLMK_ST_TIMEOUT_TMA_FULL, -1);
            if (ni == 0) {
                // idle half (sequence ends inside this block): still release the K/V stages for the other issuer
                for (int j = 0; j < nmax && ok; j++) {
                    ok = ptx::mbar_wait_spin(&kv_full[j % STAGES], (j / STAGES) & 1, abort_flag, status, LLMK_ST_TIMEOUT_TMA_FULL, j);
                    if (ok) ptx::mbar_arrive(&kv_empty[j % STAGES]);
                }
            }
            for (int j = 0; j <= ni && ok && ni > 0; j++) {
                if (j < ni) {
                    const int s = j % STAGES;
                    ok = ptx::mbar_wait_spin(&kv_full[s], (j / STAGES) & 1, abort_flag, status, LLMK_ST_TIMEOUT_TMA_FULL, j);
                    if (ok && j > 0) ok = ptx::mbar_wait_spin(&s_free[i], (j - 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_EMPTY, 3000 + j);
                    if (!ok) break;
                    ptx::tc_fence_after();
                    const uint64_t kd = k_desc + (uint64_t)((s * TILE_BYTES) >> 4);
#pragma unroll
                    for (int kk = 0; kk < HS / 16; kk++)
                        ptx::mma_f16_ss(tmem_s, q_desc + (uint64_t)(kk * 2), kd + (uint64_t)(kk * 2), idesc_s, kk > 0 ? 1u : 0u);
                    ptx::mma_commit(&s_full[i]);
                }
                if (j > 0) {
                    const int jj = j - 1, s = jj % STAGES;
                    ok = ptx::mbar_wait_spin(&p_full[i], jj & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_EMPTY, jj);
                    if (!ok) break;
                    ptx::tc_fence_after();
                    const uint64_t vd = v_desc + (uint64_t)((s * TILE_BYTES) >> 4);
#pragma unroll
                    for (int kk = 0; kk < BKV / 16; kk++)
                        ptx::mma_f16_ss(tmem_o, p_desc + (uint64_t)(((kk / 4) * ATOM_BYTES + (kk % 4) * 32) >> 4),
                                        vd + (uint64_t)((kk * 2048) >> 4), idesc_o, (jj > 0 || kk > 0) ? 1u : 0u);
                    ptx::mma_commit(&o_full[i]);
                    ptx::mma_commit(&kv_empty[s]);
                }
            }
        }
        __syncwarp();
    }
    } else {
        // ------------------------------------------------------------ softmax warpgroups
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
        const int half = (warp - 4) >> 2;
        const int nkv = half ? n1 : n0;
        const int lane_group = warp & 3;
        const int r = lane_group * 32 + lane;
        const uint32_t lane_off = (uint32_t)(lane_group * 32) << 16;
        const uint32_t tmem_s = tmem_base + half * 128, tmem_o = tmem_base + 256 + half * HS;
        uint8_t* sPh = sP + half * P_BYTES;
        constexpr float RESCALE_GAP = 8.f;
        float m = -INFINITY, l = 0.f;
        bool ok = nkv > 0;
        for (int j = 0; j < nkv && ok; j++) {
            ok = ptx::mbar_wait(&s_full[half], j & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, j);
            if (!ok) break;
            ptx::tc_fence_after();
            const bool diag = (j == nkv - 1);
            const int nchunks = diag ? lane_group + 1 : 4;
            uint32_t s[4][32];
#pragma unroll
            for (int c4 = 0; c4 < 4; c4++)
                if (c4 < nchunks) ptx::tmem_ld_32x32b_x32(tmem_s + lane_off + c4 * 32, s[c4]);
            ptx::tmem_ld_wait();
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&s_free[half]);
            float mx = -INFINITY;
#pragma unroll
            for (int c4 = 0; c4 < 4; c4++) {
                if (c4 < nchunks) {
                    if (diag && c4 == lane_group) mx = chunk_max<true>(s[c4], lane, mx);
                    else mx = chunk_max<false>(s[c4], lane, mx);
                }
            }
            const float m_new = fmaxf(m, mx * scale_log2);
            if (j > 0) {
                ok = ptx::mbar_wait(&o_full[half], (j - 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, 1000 + j);
                if (!ok) break;
                ptx::tc_fence_after();
                if (__any_sync(0xffffffffu, m_new > m + RESCALE_GAP)) {
                    const float alpha = ex2(m - m_new);
                    l *= alpha;
                    m = m_new;
#pragma unroll
                    for (int h4 = 0; h4 < HS / 32; h4++) {
                        uint32_t v[32];
                        ptx::tmem_ld_32x32b_x32(tmem_o + lane_off + h4 * 32, v);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        ptx::tmem_st_32x32b_x32(tmem_o + lane_off + h4 * 32, v);
                    }
                    ptx::tmem_st_wait();
                }
            } else {
                m = m_new;
            }
            const float neg_m = TRUNC_BIAS_LOG2 - m;   // P is truncated to bf16: see pack_trunc2
            float rs = 0.f;
#pragma unroll
            for (int c4 = 0; c4 < 4; c4++) {
                uint8_t* atom = sPh + (c4 >> 1) * ATOM_BYTES + r * 128;
                const int cb = (c4 & 1) * 4;
                if (c4 >= nchunks) chunk_probs<2>(s[c4], atom, cb, r, lane, scale_log2, neg_m);
                else if (diag && c4 == lane_group) rs += chunk_probs<1>(s[c4], atom, cb, r, lane, scale_log2, neg_m);
                else rs += chunk_probs<0>(s[c4], atom, cb, r, lane, scale_log2, neg_m);
            }
            l += rs;
            ptx::tc_fence_before();
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&p_full[half]);
        }

        if (ok) ok = ptx::mbar_wait(&o_full[half], (nkv - 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, 2000);
        if (ok) {
            // O -> bf16 -> this warpgroup's P buffer (128 rows x 128 B, swizzled like the tensor map) -> one TMA store
            ptx::tc_fence_after();
            const float inv_l = 1.0f / l;
            const int q_row0 = (2 * qb2 + half) * BQ;
#pragma unroll
            for (int h4 = 0; h4 < HS / 32; h4++) {
                uint32_t v[32];
                ptx::tmem_ld_32x32b_x32(tmem_o + lane_off + h4 * 32, v);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    float f[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) f[i] = __uint_as_float(v[q * 8 + i]) * inv_l;
                    *reinterpret_cast<bf16x8*>(sPh + r * 128 + (((h4 * 4 + q) ^ (r & 7)) << 4)) = pack8(f);
                }
            }
            lse[((size_t)b * NH + h) * T + q_row0 + r] = (m + log2f(l)) * 0.6931471805599453f;
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&epi[half]);
            if (lane_group == 0 && lane == 0) {
                if (ptx::mbar_wait(&epi[half], 0, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, 4000)) {
                    ptx::tma_store_2d(&tmOut, sPh, q_col, row_base + q_row0);
                    ptx::tma_store_commit();
                    ptx::tma_store_wait_read<0>();
                }
            }
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, 512);
    }
}

static int launch(const CUtensorMap& tm, const CUtensorMap& tm_out, float* lse, int B, int T, int NH, int NKVH, int* status,
                  cudaStream_t stream) {
    static PerDeviceOnce once_configured;
    if (once_configured.first()) {
        LLMK_CUDA_TRY(cudaFuncSetAttribute(attn_fwd_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    }
    const float scale_log2 = 1.4426950408889634f / sqrtf((float)HS);
    dim3 grid((T + 2 * BQ - 1) / (2 * BQ), NH, B);
    attn_fwd_pair_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(tm, tm_out, lse, T, NH, NKVH, scale_log2, status);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
}  // namespace pair

}  // namespace attn_tc
}  // namespace llmk

using namespace llmk;

// Same contract as llmk_attention_fwd, but T must be a multiple of 128.
LLMK_API int llmk_attention_fwd_tc(void* out, void* lse, const void* qkv, int B, int T, int NH, int NKVH, int HS, int* status,
                                   void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    static const bool single_tile = getenv("LLMK_ATTN_SINGLE_TILE") != nullptr;   // HS=64: one 128-row tile per CTA instead of two
    if (T % 128 || NH % NKVH || (HS != 64 && HS != 128)) return LLMK_ERR_SHAPE;
    const long width = (long)(NH + 2 * NKVH) * HS;
    CUtensorMap tm;
    const int rc = gemm::make_tmap_2d(&tm, qkv, (uint64_t)width, (uint64_t)B * T, (uint64_t)width, 64, 128);
    if (rc) return rc;
    if (HS == 64 && !single_tile) {
        CUtensorMap tm_out;
        const int rc2 = gemm::make_tmap_2d(&tm_out, out, (uint64_t)NH * HS, (uint64_t)B * T, (uint64_t)NH * HS, 64, 128);
        if (rc2) return rc2;
        return attn_tc::pair::launch(tm, tm_out, (float*)lse, B, T, NH, NKVH, status, stream);
    }
    if (HS == 64) return attn_tc::launch<64>(tm, tm, (bf16*)out, (float*)lse, B, T, T, 1, NH, NKVH, status, stream);
    return attn_tc::launch<128>(tm, tm, (bf16*)out, (float*)lse, B, T, T, 1, NH, NKVH, status, stream);
}

// One step of context-parallel (ring) attention, forward: the queries of `qkv` [B, T, W] (this rank's chunk of the
// sequence, packed q | k | v) against the keys and values of `kv_qkv` [B, Tkv, W], which may be ANOTHER rank's chunk in
// peer memory (the K/V tiles are pulled straight from there by TMA loads, no copy and no multicast). `causal` = 1 for
// the rank's own chunk (same positions, T == Tkv), 0 for a chunk that lies entirely before the queries. Writes the
// normalised output of this step and its log-sum-exp; llmk_attention_ring_merge folds the steps together. Job of the
// reference's local ring step (llmc/tk/ring_attention_sm120.cuh:55-189).
LLMK_API int llmk_attention_fwd_ring_step(void* out, void* lse, const void* qkv, const void* kv_qkv, int B, int T, int Tkv, int NH,
                                          int NKVH, int HS, int causal, int* status, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (T % 128 || Tkv % 128 || NH % NKVH || (HS != 64 && HS != 128) || (causal && T != Tkv)) return LLMK_ERR_SHAPE;
    const long width = (long)(NH + 2 * NKVH) * HS;
    CUtensorMap tm, tm_kv;
    int rc = gemm::make_tmap_2d(&tm, qkv, (uint64_t)width, (uint64_t)B * T, (uint64_t)width, 64, 128);
    if (rc) return rc;
    rc = gemm::make_tmap_2d(&tm_kv, kv_qkv, (uint64_t)width, (uint64_t)B * Tkv, (uint64_t)width, 64, 128);
    if (rc) return rc;
    if (HS == 64) return attn_tc::launch<64>(tm, tm_kv, (bf16*)out, (float*)lse, B, T, Tkv, causal ? 1 : 0, NH, NKVH, status, stream);
    return attn_tc::launch<128>(tm, tm_kv, (bf16*)out, (float*)lse, B, T, Tkv, causal ? 1 : 0, NH, NKVH, status, stream);
}

namespace llmk {
namespace attn_tc {
// acc (fp32, [rows, HS] per head row) and lse_acc fold in one more step: new = logaddexp(lse_acc, lse_step),
// acc = acc * exp(lse_acc - new) + step * exp(lse_step - new). `first` initialises instead. One warp per (token, head).
__global__ void __launch_bounds__(256)
ring_merge_kernel(float* __restrict__ acc, float* __restrict__ lse_acc, const bf16* __restrict__ step, const float* __restrict__ lse_step,
                  int B, int T, int NH, int HS, int first) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * 8 + warp;           // (b * T + t) * NH + h
    if (row >= (size_t)B * T * NH) return;
    const int h = row % NH;
    const size_t bt = row / NH;
    const size_t li = ((bt / T) * NH + h) * T + (bt % T);         // lse is [B, NH, T]
    const float ls = lse_step[li];
    float wa = 0.f, ws = 1.f, ln = ls;
    if (!first) {
        const float la = lse_acc[li];
        ln = fmaxf(la, ls) + log1pf(__expf(-fabsf(la - ls)));
        wa = __expf(la - ln);
        ws = __expf(ls - ln);
    }
    for (int i = lane; i < HS; i += 32) {
        const size_t o = row * HS + i;
        const float sv = __bfloat162float(step[o]);
        acc[o] = first ? sv : acc[o] * wa + sv * ws;
    }
    if (lane == 0) lse_acc[li] = ln;
}
// acc[row][c] (+)= step[row][col0 + c] for c < ncols (fp32 accumulator of a column range of a packed bf16 tensor)
__global__ void __launch_bounds__(256)
ring_accumulate_kernel(float* __restrict__ acc, const bf16* __restrict__ step, long rows, int W, int col0, int ncols, int first) {
    const long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= rows * ncols) return;
    const long row = i / ncols;
    const int c = (int)(i - row * ncols);
    float f[8];
    unpack8(ld128(step + row * W + col0 + c), f);
    float4* a = reinterpret_cast<float4*>(acc + i);
    if (!first) {
        const float4 a0 = a[0], a1 = a[1];
        f[0] += a0.x; f[1] += a0.y; f[2] += a0.z; f[3] += a0.w;
        f[4] += a1.x; f[5] += a1.y; f[6] += a1.z; f[7] += a1.w;
    }
    a[0] = make_float4(f[0], f[1], f[2], f[3]);
    a[1] = make_float4(f[4], f[5], f[6], f[7]);
}

// out[row][col0 + c] = bf16(acc[row][c])
__global__ void __launch_bounds__(256)
ring_store_cols_kernel(bf16* __restrict__ out, const float* __restrict__ acc, long rows, int W, int col0, int ncols) {
    const long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= rows * ncols) return;
    const long row = i / ncols;
    const int c = (int)(i - row * ncols);
    const float4 a0 = *reinterpret_cast<const float4*>(acc + i), a1 = *reinterpret_cast<const float4*>(acc + i + 4);
    const float f[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    st128(out + row * W + col0 + c, pack8(f));
}

struct RingPeers {
    const bf16* p[8];
};
// out[row][col0 + c] = sum over ranks r_first..P-1, in rank order, of peer_r[row][col0 + c] (fp32 sum, bf16 result):
// the owner of a sequence chunk collects the dK / dV contributions that the later ranks left in their buffers.
__global__ void __launch_bounds__(256)
ring_sum_peers_kernel(bf16* __restrict__ out, RingPeers peers, long rows, int W, int col0, int ncols, int r_first, int P) {
    const long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= rows * ncols) return;
    const long row = i / ncols;
    const int c = (int)(i - row * ncols);
    const long off = row * W + col0 + c;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = r_first; r < P; r++) {
        float f[8];
        unpack8(ld128(peers.p[r] + off), f);
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] += f[j];
    }
    st128(out + off, pack8(acc));
}
}  // namespace attn_tc
}  // namespace llmk

LLMK_API int llmk_ring_accumulate(void* acc, const void* step, long rows, int W, int col0, int ncols, int first, void* stream) {
    if (ncols % 8 || col0 % 8 || W % 8) return LLMK_ERR_SHAPE;
    attn_tc::ring_accumulate_kernel<<<ceil_div(rows * ncols / 8, 256), 256, 0, (cudaStream_t)stream>>>((float*)acc, (const bf16*)step, rows,
                                                                                                     W, col0, ncols, first);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_ring_store_cols(void* out, const void* acc, long rows, int W, int col0, int ncols, void* stream) {
    if (ncols % 8 || col0 % 8 || W % 8) return LLMK_ERR_SHAPE;
    attn_tc::ring_store_cols_kernel<<<ceil_div(rows * ncols / 8, 256), 256, 0, (cudaStream_t)stream>>>((bf16*)out, (const float*)acc, rows, W,
                                                                                                     col0, ncols);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
// `peer_ptrs`: host array of P device pointers, each to that rank's contribution buffer FOR THIS RANK'S CHUNK.
LLMK_API int llmk_ring_sum_peers(void* out, const long long* peer_ptrs, long rows, int W, int col0, int ncols, int r_first, int P,
                                 void* stream) {
    if (ncols % 8 || col0 % 8 || W % 8 || P > 8 || r_first < 0 || r_first >= P) return LLMK_ERR_SHAPE;
    attn_tc::RingPeers q;
    for (int i = 0; i < 8; i++) q.p[i] = i < P ? reinterpret_cast<const bf16*>(peer_ptrs[i]) : nullptr;
    attn_tc::ring_sum_peers_kernel<<<ceil_div(rows * ncols / 8, 256), 256, 0, (cudaStream_t)stream>>>((bf16*)out, q, rows, W, col0, ncols,
                                                                                                    r_first, P);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

LLMK_API int llmk_attention_ring_merge(void* acc, void* lse_acc, const void* step, const void* lse_step, int B, int T, int NH, int HS,
                                       int first, void* stream) {
    const long rows = (long)B * T * NH;
    attn_tc::ring_merge_kernel<<<ceil_div(rows, 8), 256, 0, (cudaStream_t)stream>>>((float*)acc, (float*)lse_acc, (const bf16*)step,
                                                                                   (const float*)lse_step, B, T, NH, HS, first);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
