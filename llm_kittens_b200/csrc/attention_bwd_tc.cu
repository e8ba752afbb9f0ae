// Causal flash-attention BACKWARD on tcgen05 / TMEM for MHA and GQA, deterministic (no atomics):
//
//   dkv kernel  one CTA per (128-row K/V tile, KV head, batch); loops over the query sub-tiles at or
//               after it and over the query heads that share the KV head. Works on TRANSPOSED scores so
//               a thread owns one key row:
//                   S^T  = K Q^T          dP^T = V dO^T                 (tcgen05, K-major operands)
//                   P^T  = exp2(S^T c - LSE[q])      dS^T = P^T * (dP^T - D[q])     (softmax warps)
//                   dV  += P^T dO         dK  += dS^T Q                 (tcgen05, accumulate in TMEM)
//   dq kernel   one CTA per (128-row query tile, head, batch); loops over the K/V sub-tiles at or before
//               it:  S = Q K^T, dP = dO V^T, dS = P * (dP - D[row]), dQ += dS K.
//
// The looped-over ("inner") tile has BN rows: 64 for head size 64, which keeps a CTA at 256 TMEM columns
// and under half of the SM's shared memory so that two CTAs are resident and one's exponentials overlap
// the other's MMAs; 128 for head size 128. Both kernels recompute P from the saved log-sum-exp;
// D = rowsum(dO * O) comes from the small pre-pass in attention.cu. Inputs are the packed QKV activation
// and dO through TMA tensor maps; outputs go straight into the packed dQKV tensor. Same job as
// attention_backward / attention_gqa_backward in the reference (llmc/attention.cuh:481-604,
// llmc/attention_gqa.cuh:483-572). Warp roles as in the forward kernel (attention_tc.cu): warp 0 TMA
// producer, warp 1 MMA issuer, warps 2-5 one row per thread. All waits are bounded.
#include <cstdlib>

#include "ptx_sm100.cuh"

namespace llmk {
namespace gemm {
int make_tmap_2d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_elems, uint32_t box_inner,
                 uint32_t box_outer);
}
namespace attn_bwd_tc {

constexpr int BM = 128;  // rows of the tile a CTA owns
constexpr int THREADS = 320;   // producer, MMA issuer, and two softmax warps per TMEM lane group (they split the columns)
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two columns of the backward softmax with packed fp32 pairs: e = exp2(s * c + nl) (zero where masked) and
// ds = e * (dp + nd). `nl` / `nd` hold the NEGATED log-sum-exp (exp2 domain) and D, so that the pair forms of
// FMA / ADD / MUL (which take no operand negation) give the same roundings as the scalar s*c - L and dp - D.
__device__ __forceinline__ void prob_pair(uint32_t s0, uint32_t s1, uint32_t dp0, uint32_t dp1, ptx::f32x2 c2, ptx::f32x2 nl,
                                          ptx::f32x2 nd, bool mask0, bool mask1, float* p, float* ds) {
    float x0, x1;
    ptx::unpack2(ptx::fma2(ptx::pack2(__uint_as_float(s0), __uint_as_float(s1)), c2, nl), x0, x1);
    float e0 = ex2(x0), e1 = ex2(x1);
    if (mask0) e0 = 0.f;
    if (mask1) e1 = 0.f;
    p[0] = e0;
    p[1] = e1;
    const ptx::f32x2 t = ptx::add2(ptx::pack2(__uint_as_float(dp0), __uint_as_float(dp1)), nd);
    ptx::unpack2(ptx::mul2(ptx::pack2(e0, e1), t), ds[0], ds[1]);
}

// [ROWS x cols] K-major A/B operand at `base`, stored as atoms of 64 columns (ROWS * 128 bytes each):
// descriptor of k-step kk (16 columns)
template <int ROWS>
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t base, int kk) {
    return ptx::make_smem_desc(base + (kk / 4) * (ROWS * 128) + (kk % 4) * 32, 16, 1024);
}
// the same kind of tile read as an MN-major B operand (n = its columns, k = its ROWS rows): k-step kk (16 rows)
template <int ROWS>
__device__ __forceinline__ uint64_t mnmajor_desc(uint32_t base, int kk) {
    return ptx::make_smem_desc(base + kk * 2048, ROWS * 128, 1024);
}
// The same descriptors by arithmetic on a base descriptor built once per buffer (the start-address field holds
// bytes / 16): inside the issue loops an operand then costs one 64-bit add instead of a rebuild.
template <int ROWS>
__device__ __forceinline__ uint64_t kmajor_step(uint64_t base_desc, int kk) {
    return base_desc + (uint64_t)(((kk / 4) * (ROWS * 128) + (kk % 4) * 32) >> 4);
}
__device__ __forceinline__ uint64_t mnmajor_step(uint64_t base_desc, int kk) { return base_desc + (uint64_t)((kk * 2048) >> 4); }

// Returns true (for the whole CTA) when the status word already holds a failure: the kernel then returns at once.
__device__ __forceinline__ bool already_failed(const int* status) {
    __shared__ int skip;
    if (threadIdx.x == 0) skip = (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0);
    __syncthreads();
    return skip != 0;
}

// One 128-row x 64-column bf16 tile row (this thread's row r) into a TMA-store staging tile, 16-byte chunk `chunk`.
// Backward of interleaved-pair RoPE on 8 consecutive head columns (4 pairs): the transpose rotation of the forward
// one, so the gradients leave the kernel with respect to the un-rotated q / k that the QKV projection produced.
// `fr` = the 4 (cos, sin) entries of this token's row of the frequency table that belong to the pairs.
__device__ __forceinline__ void rope_inverse8(float* f, const float2* __restrict__ fr) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(fr)), b = __ldg(reinterpret_cast<const float4*>(fr) + 1);
    const float c[4] = {a.x, a.z, b.x, b.z}, sn[4] = {a.y, a.w, b.y, b.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float x0 = f[2 * j], x1 = f[2 * j + 1];
        f[2 * j] = x0 * c[j] + x1 * sn[j];
        f[2 * j + 1] = x1 * c[j] - x0 * sn[j];
    }
}

__device__ __forceinline__ void stage_chunk(uint8_t* tile, int r, int chunk, const float* f) {
    *reinterpret_cast<bf16x8*>(tile + r * 128 + ((chunk ^ (r & 7)) << 4)) = pack8(f);
}

template <int HS, int ROWS>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int col, int row) {
#pragma unroll
    for (int c = 0; c < HS / 64; c++) ptx::tma_load_2d(dst + c * (ROWS * 128), tm, bar, col + 64 * c, row);
}
// write 8 bf16 into 16-byte chunk `chunk` of row r of a [128 x BN] K-major tile (atoms of 64 columns)
__device__ __forceinline__ void store_chunk(uint8_t* tile, int r, int chunk, const float* f) {
    uint8_t* atom = tile + (chunk >> 3) * (BM * 128) + r * 128;
    *reinterpret_cast<bf16x8*>(atom + (((chunk & 7) ^ (r & 7)) << 4)) = pack8(f);
}

template <int HS>
struct Inner {
    // HS = 64: 64-query sub-tiles and two CTAs per SM (one CTA's softmax overlaps the other's MMAs); 128-query sub-tiles
    // with one CTA per SM issue a quarter fewer MMAs but measured 1.06 ms against 0.88 ms at B64 T1024 NH12
    static constexpr int BN = HS == 64 ? 64 : 128;
    static constexpr int CTAS = HS == 64 ? 2 : 1;
};

// ====================================================================================== dK, dV
template <int HS>
struct DkvCfg {
    static constexpr int BN = Inner<HS>::BN;
    static constexpr int RING = HS == 64 ? 2 : 1;
    static constexpr int TILE = BM * HS * 2;   // K or V
    static constexpr int RT = BN * HS * 2;     // Q or dO sub-tile
    static constexpr int OFF_K = 0, OFF_V = TILE, OFF_RING = 2 * TILE;   // ring: [RING][Q, dO]
    static constexpr int OFF_PT = OFF_RING + RING * 2 * RT, OFF_DST = OFF_PT + BM * BN * 2;
    static constexpr int OFF_LD = OFF_DST + BM * BN * 2;                  // float [2][2][128]
    static constexpr int OFF_BAR = OFF_LD + 2 * 2 * 128 * 4;
    static constexpr int SMEM_BYTES = OFF_BAR + 128;
    static constexpr int TMEM = (2 * BN + 2 * HS) <= 256 ? 256 : 512;
};

template <int HS>
__global__ void __launch_bounds__(THREADS, Inner<HS>::CTAS)
attn_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmQKVin,
                       const __grid_constant__ CUtensorMap tmDOin, const __grid_constant__ CUtensorMap tmDQKV,
                       const float* __restrict__ lse, const float* __restrict__ dvec, int T, int NH, int NKVH, float scale,
                       int* status, const float2* __restrict__ rope, int Tkv, int causal) {
    // Tkv / causal: in a context-parallel (ring) step the keys and values (tmQKV, and the output tmDQKV) belong to
    // another chunk of the sequence, Tkv rows per batch entry, possibly in a peer's memory; causal = 0 means every key
    // precedes every query, so all query sub-tiles are visited and nothing is masked. Usual case: Tkv = T, causal = 1.
    using C = DkvCfg<HS>;
    constexpr int RING = C::RING, BN = C::BN;
    extern __shared__ __align__(1024) uint8_t smem[];
    if (already_failed(status)) return;
    if (ptx::smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, LLMK_ST_BOUNDS);
        return;
    }
    uint8_t* sK = smem + C::OFF_K;
    uint8_t* sV = smem + C::OFF_V;
    uint8_t* sRing = smem + C::OFF_RING;
    uint8_t* sPt = smem + C::OFF_PT;
    uint8_t* sdSt = smem + C::OFF_DST;
    float* sLD = reinterpret_cast<float*>(smem + C::OFF_LD);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
    uint64_t* kv_full = bars;         // [1]
    uint64_t* ring_full = bars + 1;   // [2]
    uint64_t* ring_empty = bars + 3;  // [2]
    uint64_t* s_full = bars + 5;
    uint64_t* p_full = bars + 6;
    uint64_t* acc_done = bars + 7;
    uint64_t* ld_full = bars + 8;     // [2] LSE / D vectors of a ring slot are in shared memory
    uint64_t* epi = bars + 10;        // dK / dV staged in shared memory
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int hr = NH / NKVH;
    const int kv0 = kt * BM;
    const int q_first = causal ? kv0 : 0;
    const int nq = (T - q_first) / BN;   // query sub-tiles that see these keys
    const int total = nq * hr;
    const int row_base = b * T, kv_row_base = b * Tkv;
    const int k_col = (NH + hk) * HS, v_col = (NH + NKVH + hk) * HS;
    const float scale_log2 = scale * LOG2E;

    if (threadIdx.x == 0) {
        ptx::mbar_init(kv_full, 1);
        for (int i = 0; i < 2; i++) {
            ptx::mbar_init(&ring_full[i], 1);
            ptx::mbar_init(&ring_empty[i], 1);
            ptx::mbar_init(&ld_full[i], 1);
        }
        ptx::mbar_init(s_full, 1);
        ptx::mbar_init(p_full, 8);
        ptx::mbar_init(acc_done, 1);
        ptx::mbar_init(epi, 8);
        *abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, C::TMEM);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t t_st = tmem_base, t_dpt = tmem_base + BN, t_dv = tmem_base + 2 * BN, t_dk = tmem_base + 2 * BN + HS;

    if (warp == 0) {
        if (lane == 0) {
            ptx::mbar_arrive_expect_tx(kv_full, 2 * C::TILE);
            load_tile<HS, BM>(sK, &tmQKV, kv_full, k_col, kv_row_base + kv0);
            load_tile<HS, BM>(sV, &tmQKV, kv_full, v_col, kv_row_base + kv0);
        }
        __syncwarp();
        for (int it = 0; it < total; it++) {
            const int s = it % RING;
            if (!ptx::mbar_wait(&ring_empty[s], ((it / RING) & 1) ^ 1, abort_flag, status, LLMK_ST_TIMEOUT_TMA_EMPTY, it)) break;
            const int hq = hk * hr + it / nq, q0 = q_first + (it % nq) * BN;
            if (lane == 0) {
                ptx::mbar_arrive_expect_tx(&ring_full[s], 2 * C::RT);
                load_tile<HS, BN>(sRing + s * 2 * C::RT, &tmQKVin, &ring_full[s], hq * HS, row_base + q0);
                load_tile<HS, BN>(sRing + s * 2 * C::RT + C::RT, &tmDOin, &ring_full[s], hq * HS, row_base + q0);
            }
            {   // log-sum-exp (in the exp2 domain) and D of the BN queries of this sub-tile
                float* sL = sLD + s * 256;
                const size_t off = ((size_t)b * NH + hq) * T + q0;
#pragma unroll
                for (int i = 0; i < BN / 32; i++) {
                    sL[lane + 32 * i] = -lse[off + lane + 32 * i] * LOG2E;   // negated: the consumers add
                    sL[128 + lane + 32 * i] = -dvec[off + lane + 32 * i];
                }
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&ld_full[s]);
            __syncwarp();
        }
    } else if (warp == 1) {
        constexpr uint32_t idesc_s = ptx::make_idesc_bf16(BM, BN, 0, 0);
        constexpr uint32_t idesc_acc = ptx::make_idesc_bf16(BM, HS, 0, 1);
        bool ok = ptx::mbar_wait(kv_full, 0, abort_flag, status, LLMK_ST_TIMEOUT_TMA_FULL, -1);
        // descriptors are built once; only lane 0 runs the issue loop (it shares its scheduler with softmax warps,
        // so every instruction saved here shortens the critical path)
        const uint64_t k_desc = kmajor_desc<BM>(ptx::smem_u32(sK), 0), v_desc = kmajor_desc<BM>(ptx::smem_u32(sV), 0);
        const uint64_t pt_desc = kmajor_desc<BM>(ptx::smem_u32(sPt), 0), dst_desc = kmajor_desc<BM>(ptx::smem_u32(sdSt), 0);
        const uint32_t ring_addr = ptx::smem_u32(sRing);
        auto issue_s = [&](int it) -> bool {
            const int s = it % RING;
            if (!ptx::mbar_wait(&ring_full[s], (it / RING) & 1, abort_flag, status, LLMK_ST_TIMEOUT_TMA_FULL, it)) return false;
            ptx::tc_fence_after();
            if (lane == 0) {
                const uint64_t q_desc = kmajor_desc<BN>(ring_addr + s * 2 * C::RT, 0), do_desc = kmajor_desc<BN>(ring_addr + s * 2 * C::RT + C::RT, 0);
#pragma unroll
                for (int kk = 0; kk < HS / 16; kk++)
                    ptx::mma_f16_ss(t_st, kmajor_step<BM>(k_desc, kk), kmajor_step<BN>(q_desc, kk), idesc_s, kk > 0 ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < HS / 16; kk++)
                    ptx::mma_f16_ss(t_dpt, kmajor_step<BM>(v_desc, kk), kmajor_step<BN>(do_desc, kk), idesc_s, kk > 0 ? 1u : 0u);
                ptx::mma_commit(s_full);
            }
            __syncwarp();
            return true;
        };
        auto issue_acc = [&](int it) {
            const int s = it % RING;
            if (lane == 0) {
                const uint64_t q_mn = mnmajor_desc<BN>(ring_addr + s * 2 * C::RT, 0), do_mn = mnmajor_desc<BN>(ring_addr + s * 2 * C::RT + C::RT, 0);
#pragma unroll
                for (int kk = 0; kk < BN / 16; kk++)
                    ptx::mma_f16_ss(t_dv, kmajor_step<BM>(pt_desc, kk), mnmajor_step(do_mn, kk), idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < BN / 16; kk++)
                    ptx::mma_f16_ss(t_dk, kmajor_step<BM>(dst_desc, kk), mnmajor_step(q_mn, kk), idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
                ptx::mma_commit(&ring_empty[s]);
                ptx::mma_commit(acc_done);
            }
            __syncwarp();
        };
        if (ok) ok = issue_s(0);
        for (int it = 0; it < total && ok; it++) {
            ok = ptx::mbar_wait(p_full, it & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_EMPTY, it);
            if (!ok) break;
            ptx::tc_fence_after();
            if (RING == 2) {
                if (it + 1 < total) ok = issue_s(it + 1);   // next scores first, so the softmax can overlap the accumulation
                if (!ok) break;
                issue_acc(it);
            } else {
                issue_acc(it);
                if (it + 1 < total) ok = issue_s(it + 1);
            }
        }
    } else {
        const int lane_group = warp & 3;
        const int sub = (warp - 2) >> 2;                     // 0 / 1: which half of the columns this warp handles
        const int r = lane_group * 32 + lane;               // key row inside the tile
        const uint32_t lane_off = (uint32_t)(lane_group * 32) << 16;
        const ptx::f32x2 c2 = ptx::pack2(scale_log2, scale_log2);
        bool ok = true;
        for (int it = 0; it < total && ok; it++) {
            const int dq0 = (it % nq) * BN;                  // first query of the sub-tile relative to the first key
            const int slot = it % RING;
            const float* sL = sLD + slot * 256;
            const float* sD = sL + 128;
            ok = ptx::mbar_wait(&ld_full[slot], (it / RING) & 1, abort_flag, status, LLMK_ST_TIMEOUT_TMA_FULL, 3000 + it);
            if (!ok) break;
            ok = ptx::mbar_wait(s_full, it & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, it);
            if (!ok) break;
            if (it > 0) {   // the previous accumulation MMAs have finished reading P^T / dS^T
                ok = ptx::mbar_wait(acc_done, (it - 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, 1000 + it);
                if (!ok) break;
            }
            ptx::tc_fence_after();
            const bool diag = causal && dq0 < BM;            // some (key, query) pairs of this sub-tile are masked
            // the two TMEM loads of chunk c4+1 are issued before chunk c4 is processed (two register sets)
            uint32_t vsA[32], vdA[32], vsB[32], vdB[32];
            auto process = [&](int c4, const uint32_t (&vs)[32], const uint32_t (&vd)[32]) {
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    float p[8], ds[8], L[8], D[8];
                    *reinterpret_cast<float4*>(L) = *reinterpret_cast<const float4*>(sL + c4 * 32 + q * 8);
                    *reinterpret_cast<float4*>(L + 4) = *reinterpret_cast<const float4*>(sL + c4 * 32 + q * 8 + 4);
                    *reinterpret_cast<float4*>(D) = *reinterpret_cast<const float4*>(sD + c4 * 32 + q * 8);
                    *reinterpret_cast<float4*>(D + 4) = *reinterpret_cast<const float4*>(sD + c4 * 32 + q * 8 + 4);
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        const int c = c4 * 32 + q * 8 + i;   // query column of the sub-tile
                        prob_pair(vs[q * 8 + i], vs[q * 8 + i + 1], vd[q * 8 + i], vd[q * 8 + i + 1], c2, ptx::pack2(L[i], L[i + 1]),
                                  ptx::pack2(D[i], D[i + 1]), diag && r > c + dq0, diag && r > c + 1 + dq0, p + i, ds + i);
                    }
                    store_chunk(sPt, r, c4 * 4 + q, p);
                    store_chunk(sdSt, r, c4 * 4 + q, ds);
                }
            };
            // this warp's share of the sub-tile's columns: chunks [sub * NCH, (sub + 1) * NCH)
            constexpr int NCH = BN / 64;
            const int c_first = sub * NCH;
            ptx::tmem_ld_32x32b_x32(t_st + lane_off + c_first * 32, vsA);
            ptx::tmem_ld_32x32b_x32(t_dpt + lane_off + c_first * 32, vdA);
#pragma unroll
            for (int i4 = 0; i4 < NCH; i4++) {
                const int c4 = c_first + i4;
                ptx::tmem_ld_wait();
                if (i4 + 1 < NCH) {
                    ptx::tmem_ld_32x32b_x32(t_st + lane_off + (c4 + 1) * 32, (i4 & 1) ? vsA : vsB);
                    ptx::tmem_ld_32x32b_x32(t_dpt + lane_off + (c4 + 1) * 32, (i4 & 1) ? vdA : vdB);
                }
                if (i4 & 1) process(c4, vsB, vdB);
                else process(c4, vsA, vdA);
            }
            ptx::tc_fence_before();
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(p_full);
        }
        if (ok) ok = ptx::mbar_wait(acc_done, (total - 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, 2000);
        if (ok) {
            ptx::tc_fence_after();
            // dK (scaled) and dV -> bf16 -> the P^T / dS^T buffers as [128 x 64] staging tiles per 64 columns -> TMA stores
            uint8_t* stage_dk = sPt;    // HS/64 tiles of 16 KB each fit: BM*BN*2 >= BM*HS*2 for both head sizes
            uint8_t* stage_dv = sdSt;
#pragma unroll
            for (int h4 = sub; h4 < HS / 32; h4 += 2) {
                uint32_t v[32];
                ptx::tmem_ld_32x32b_x32(t_dk + lane_off + h4 * 32, v);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    float f[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) f[i] = __uint_as_float(v[q * 8 + i]) * scale;
                    if (rope != nullptr) rope_inverse8(f, rope + (size_t)(kv0 + r) * (HS / 2) + h4 * 16 + q * 4);
                    stage_chunk(stage_dk + (h4 / 2) * (BM * 128), r, (h4 & 1) * 4 + q, f);
                }
                ptx::tmem_ld_32x32b_x32(t_dv + lane_off + h4 * 32, v);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    float f[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) f[i] = __uint_as_float(v[q * 8 + i]);
                    stage_chunk(stage_dv + (h4 / 2) * (BM * 128), r, (h4 & 1) * 4 + q, f);
                }
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(epi);
            if (warp == 2 && lane == 0) {
                if (ptx::mbar_wait(epi, 0, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, 4000)) {
#pragma unroll
                    for (int c = 0; c < HS / 64; c++) {
                        ptx::tma_store_2d(&tmDQKV, stage_dk + c * (BM * 128), k_col + 64 * c, kv_row_base + kv0);
                        ptx::tma_store_2d(&tmDQKV, stage_dv + c * (BM * 128), v_col + 64 * c, kv_row_base + kv0);
                    }
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
        ptx::tmem_dealloc(tmem_base, C::TMEM);
    }
}

// ====================================================================================== dK, dV for HS = 64, pipelined
// One CTA per SM and per 128-key tile; the scores S^T / dP^T of 64-query sub-tiles are double-buffered in TMEM and
// two groups of eight softmax warps take alternate sub-tiles, so the tensor core computes the scores of sub-tile
// it+1 while group (it & 1) turns those of sub-tile `it` into P^T / dS^T. Q / dO sub-tiles come through a 3-deep ring.
// TMEM (512 columns): S^T[2] 0/64, dP^T[2] 128/192, dV 256, dK 320.
namespace dkv2 {
constexpr int HS = 64, BN = 64, RING = 3;
constexpr int THREADS2 = 32 * (2 + 16);
constexpr int TILE = BM * HS * 2;       // K or V: 16 KB
constexpr int RT = BN * HS * 2;         // Q or dO sub-tile: 8 KB
constexpr int PT = BM * BN * 2;         // P^T or dS^T: 16 KB
constexpr int OFF_K = 0, OFF_V = TILE, OFF_RING = 2 * TILE;
constexpr int OFF_PT = OFF_RING + RING * 2 * RT;          // [2]
constexpr int OFF_DST = OFF_PT + 2 * PT;                  // [2]
constexpr int OFF_LD = OFF_DST + 2 * PT;                  // float [RING][2][64]
constexpr int OFF_BAR = OFF_LD + RING * 2 * 64 * 4;
constexpr int SMEM_BYTES = OFF_BAR + 256;

__global__ void __launch_bounds__(THREADS2, 1)
attn_bwd_dkv2_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmQKVin,
                     const __grid_constant__ CUtensorMap tmDOin, const __grid_constant__ CUtensorMap tmDQKV,
                     const float* __restrict__ lse, const float* __restrict__ dvec, int T, int NH, int NKVH, float scale,
                     int* status, const float2* __restrict__ rope) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if (already_failed(status)) return;
    if (ptx::smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, LLMK_ST_BOUNDS);
        return;
    }
    uint8_t* sK = smem + OFF_K;
    uint8_t* sV = smem + OFF_V;
    uint8_t* sRing = smem + OFF_RING;
    uint8_t* sPt = smem + OFF_PT;
    uint8_t* sdSt = smem + OFF_DST;
    float* sLD = reinterpret_cast<float*>(smem + OFF_LD);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* kv_full = bars;             // [1]
    uint64_t* ring_full = bars + 1;       // [3]
    uint64_t* ring_empty = bars + 4;      // [3]
    uint64_t* ld_full = bars + 7;         // [3]
    uint64_t* s_full = bars + 10;         // [2]
    uint64_t* p_full = bars + 12;         // [2]
    uint64_t* acc_done = bars + 14;       // [2]
    uint64_t* epi = bars + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int hr = NH / NKVH;
    const int kv0 = kt * BM;
    const int nq = (T - kv0) / BN;
    const int total = nq * hr;
    const int row_base = b * T;
    const int k_col = (NH + hk) * HS, v_col = (NH + NKVH + hk) * HS;
    const float scale_log2 = scale * LOG2E;

    if (threadIdx.x == 0) {
        ptx::mbar_init(kv_full, 1);
        for (int i = 0; i < RING; i++) {
            ptx::mbar_init(&ring_full[i], 1);
            ptx::mbar_init(&ring_empty[i], 1);
            ptx::mbar_init(&ld_full[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            ptx::mbar_init(&s_full[i], 1);
            ptx::mbar_init(&p_full[i], 8);
            ptx::mbar_init(&acc_done[i], 1);
        }
        ptx::mbar_init(epi, 16);
        *abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, 512);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t t_dv = tmem_base + 256, t_dk = tmem_base + 320;

    if (warp == 0) {
        // ------------------------------------------------------------ producer: K, V once; Q / dO ring; LSE / D vectors
        if (lane == 0) {
            ptx::mbar_arrive_expect_tx(kv_full, 2 * TILE);
            load_tile<HS, BM>(sK, &tmQKV, kv_full, k_col, row_base + kv0);
            load_tile<HS, BM>(sV, &tmQKV, kv_full, v_col, row_base + kv0);
        }
        __syncwarp();
        for (int it = 0; it < total; it++) {
            const int s = it % RING;
            if (!ptx::mbar_wait(&ring_empty[s], ((it / RING) & 1) ^ 1, abort_flag, status, LLMK_ST_TIMEOUT_TMA_EMPTY, it)) break;
            const int hq = hk * hr + it / nq, q0 = kv0 + (it % nq) * BN;
            if (lane == 0) {
                ptx::mbar_arrive_expect_tx(&ring_full[s], 2 * RT);
                load_tile<HS, BN>(sRing + s * 2 * RT, &tmQKVin, &ring_full[s], hq * HS, row_base + q0);
                load_tile<HS, BN>(sRing + s * 2 * RT + RT, &tmDOin, &ring_full[s], hq * HS, row_base + q0);
            }
            float* sL = sLD + s * 128;
            const size_t off = ((size_t)b * NH + hq) * T + q0;
#pragma unroll
            for (int i = 0; i < BN / 32; i++) {
                sL[lane + 32 * i] = -lse[off + lane + 32 * i] * LOG2E;   // negated: the consumers add
                sL[64 + lane + 32 * i] = -dvec[off + lane + 32 * i];
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&ld_full[s]);
            __syncwarp();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (lane 0)
        if (lane == 0) {
            constexpr uint32_t idesc_s = ptx::make_idesc_bf16(BM, BN, 0, 0);
            constexpr uint32_t idesc_acc = ptx::make_idesc_bf16(BM, HS, 0, 1);
            const uint64_t k_desc = kmajor_desc<BM>(ptx::smem_u32(sK), 0), v_desc = kmajor_desc<BM>(ptx::smem_u32(sV), 0);
            const uint32_t ring_addr = ptx::smem_u32(sRing), pt_addr = ptx::smem_u32(sPt), dst_addr = ptx::smem_u32(sdSt);
            bool ok = ptx::mbar_wait_spin(kv_full, 0, abort_flag, status, LLMK_ST_TIMEOUT_TMA_FULL, -1);
            for (int it = 0; it <= total && ok; it++) {
                if (it < total) {
                    // scores of sub-tile `it` into buffer it & 1 (its previous reader, sub-tile it-2, finished before
                    // P(it-2) was published, which the accumulation step below has already waited for)
                    const int s = it % RING, bsel = it & 1;
                    ok = ptx::mbar_wait_spin(&ring_full[s], (it / RING) & 1, abort_flag, status, LLMK_ST_TIMEOUT_TMA_FULL, it);
                    if (!ok) break;
                    ptx::tc_fence_after();
                    const uint64_t q_desc = kmajor_desc<BN>(ring_addr + s * 2 * RT, 0), do_desc = kmajor_desc<BN>(ring_addr + s * 2 * RT + RT, 0);
#pragma unroll
                    for (int kk = 0; kk < HS / 16; kk++)
                        ptx::mma_f16_ss(tmem_base + bsel * 64, kmajor_step<BM>(k_desc, kk), kmajor_step<BN>(q_desc, kk), idesc_s, kk > 0 ? 1u : 0u);
#pragma unroll
                    for (int kk = 0; kk < HS / 16; kk++)
                        ptx::mma_f16_ss(tmem_base + 128 + bsel * 64, kmajor_step<BM>(v_desc, kk), kmajor_step<BN>(do_desc, kk), idesc_s, kk > 0 ? 1u : 0u);
                    ptx::mma_commit(&s_full[bsel]);
                }
                if (it >= 1) {
                    const int j = it - 1, s = j % RING, bsel = j & 1;
                    ok = ptx::mbar_wait_spin(&p_full[bsel], (j >> 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_EMPTY, j);
                    if (!ok) break;
                    ptx::tc_fence_after();
                    const uint64_t q_mn = mnmajor_desc<BN>(ring_addr + s * 2 * RT, 0), do_mn = mnmajor_desc<BN>(ring_addr + s * 2 * RT + RT, 0);
                    const uint64_t pt_desc = kmajor_desc<BM>(pt_addr + bsel * PT, 0), dst_desc = kmajor_desc<BM>(dst_addr + bsel * PT, 0);
#pragma unroll
                    for (int kk = 0; kk < BN / 16; kk++)
                        ptx::mma_f16_ss(t_dv, kmajor_step<BM>(pt_desc, kk), mnmajor_step(do_mn, kk), idesc_acc, (j > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
                    for (int kk = 0; kk < BN / 16; kk++)
                        ptx::mma_f16_ss(t_dk, kmajor_step<BM>(dst_desc, kk), mnmajor_step(q_mn, kk), idesc_acc, (j > 0 || kk > 0) ? 1u : 0u);
                    ptx::mma_commit(&ring_empty[s]);
                    ptx::mma_commit(&acc_done[bsel]);
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ softmax warps: group g takes sub-tiles it with (it & 1) == g
        const int w = warp - 2;                  // 0..15
        const int g = w >> 3;                    // group
        const int lane_group = warp & 3;
        const int sub = (w >> 2) & 1;            // which 32 of the 64 query columns
        const int r = lane_group * 32 + lane;    // key row inside the tile
        const uint32_t lane_off = (uint32_t)(lane_group * 32) << 16;
        uint8_t* myPt = sPt + g * PT;
        uint8_t* mydSt = sdSt + g * PT;
        const uint32_t t_st = tmem_base + g * 64 + sub * 32, t_dpt = tmem_base + 128 + g * 64 + sub * 32;
        const ptx::f32x2 c2 = ptx::pack2(scale_log2, scale_log2);
        bool ok = true;
        int last = -1;
        for (int it = g; it < total && ok; it += 2) {
            last = it;
            const int dq0 = (it % nq) * BN;
            const int slot = it % RING;
            const float* sL = sLD + slot * 128 + sub * 32;
            const float* sD = sL + 64;
            ok = ptx::mbar_wait(&ld_full[slot], (it / RING) & 1, abort_flag, status, LLMK_ST_TIMEOUT_TMA_FULL, 3000 + it);
            if (!ok) break;
            ok = ptx::mbar_wait(&s_full[g], (it >> 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, it);
            if (!ok) break;
            if (it >= 2) {   // the accumulation MMAs of sub-tile it-2 have finished reading this group's P^T / dS^T
                ok = ptx::mbar_wait(&acc_done[g], ((it >> 1) - 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, 1000 + it);
                if (!ok) break;
            }
            ptx::tc_fence_after();
            const bool diag = dq0 < BM;
            uint32_t vs[32], vd[32];
            ptx::tmem_ld_32x32b_x32(t_st + lane_off, vs);
            ptx::tmem_ld_32x32b_x32(t_dpt + lane_off, vd);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 4; q++) {
                float p[8], ds[8], L[8], D[8];
                *reinterpret_cast<float4*>(L) = *reinterpret_cast<const float4*>(sL + q * 8);
                *reinterpret_cast<float4*>(L + 4) = *reinterpret_cast<const float4*>(sL + q * 8 + 4);
                *reinterpret_cast<float4*>(D) = *reinterpret_cast<const float4*>(sD + q * 8);
                *reinterpret_cast<float4*>(D + 4) = *reinterpret_cast<const float4*>(sD + q * 8 + 4);
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    const int c = sub * 32 + q * 8 + i;   // query column of the sub-tile
                    prob_pair(vs[q * 8 + i], vs[q * 8 + i + 1], vd[q * 8 + i], vd[q * 8 + i + 1], c2, ptx::pack2(L[i], L[i + 1]),
                              ptx::pack2(D[i], D[i + 1]), diag && r > c + dq0, diag && r > c + 1 + dq0, p + i, ds + i);
                }
                store_chunk(myPt, r, sub * 4 + q, p);
                store_chunk(mydSt, r, sub * 4 + q, ds);
            }
            ptx::tc_fence_before();
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&p_full[g]);
        }
        // every accumulation has to be complete: the commit of the last sub-tile covers all earlier MMAs
        if (ok) ok = ptx::mbar_wait(&acc_done[(total - 1) & 1], ((total - 1) >> 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, 2000);
        if (ok && total >= 2 && last >= 0)   // ... and this group's own buffers must be idle before they become staging space
            ok = ptx::mbar_wait(&acc_done[g], (last >> 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, 2001);
        if (ok) {
            ptx::tc_fence_after();
            // the 4 warps of a lane group take one 32-column chunk each: dK chunks 0/1 (scaled), dV chunks 0/1
            const int part = w >> 2;                           // 0..3
            const bool is_dk = part < 2;
            const int h4 = part & 1;
            uint8_t* stage = is_dk ? sPt : sdSt;               // [128 x 64] staging tile in buffer 0 of each
            uint32_t v[32];
            ptx::tmem_ld_32x32b_x32((is_dk ? t_dk : t_dv) + lane_off + h4 * 32, v);
            ptx::tmem_ld_wait();
            const float sc = is_dk ? scale : 1.0f;
#pragma unroll
            for (int q = 0; q < 4; q++) {
                float f[8];
#pragma unroll
                for (int i = 0; i < 8; i++) f[i] = __uint_as_float(v[q * 8 + i]) * sc;
                if (is_dk && rope != nullptr) rope_inverse8(f, rope + (size_t)(kv0 + r) * 32 + h4 * 16 + q * 4);
                stage_chunk(stage, r, h4 * 4 + q, f);
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(epi);
            if (warp == 2 && lane == 0) {
                if (ptx::mbar_wait(epi, 0, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, 4000)) {
                    ptx::tma_store_2d(&tmDQKV, sPt, k_col, row_base + kv0);
                    ptx::tma_store_2d(&tmDQKV, sdSt, v_col, row_base + kv0);
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
}  // namespace dkv2

// ====================================================================================== dQ
template <int HS>
struct DqCfg {
    static constexpr int BN = Inner<HS>::BN;
    static constexpr int TILE = BM * HS * 2;   // Q or dO
    static constexpr int RT = BN * HS * 2;     // K or V sub-tile
    static constexpr int OFF_Q = 0, OFF_DO = TILE, OFF_RING = 2 * TILE;   // ring: [2][K, V]
    static constexpr int OFF_DS = OFF_RING + 4 * RT;
    static constexpr int OFF_BAR = OFF_DS + BM * BN * 2;
    static constexpr int SMEM_BYTES = OFF_BAR + 128;
    static constexpr int TMEM = (2 * BN + HS) <= 256 ? 256 : 512;
};

template <int HS>
__global__ void __launch_bounds__(THREADS, Inner<HS>::CTAS)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO,
                      const __grid_constant__ CUtensorMap tmQKVin, const __grid_constant__ CUtensorMap tmDQKV,
                      const float* __restrict__ lse, const float* __restrict__ dvec, int T, int NH, int NKVH, float scale,
                      int* status, const float2* __restrict__ rope, int Tkv, int causal) {
    // Tkv / causal: as in the dK/dV kernel; here tmQKVin (the key / value sub-tiles) may cover another chunk
    using C = DqCfg<HS>;
    constexpr int BN = C::BN;
    extern __shared__ __align__(1024) uint8_t smem[];
    if (already_failed(status)) return;
    if (ptx::smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, LLMK_ST_BOUNDS);
        return;
    }
    uint8_t* sQ = smem + C::OFF_Q;
    uint8_t* sdO = smem + C::OFF_DO;
    uint8_t* sRing = smem + C::OFF_RING;
    uint8_t* sdS = smem + C::OFF_DS;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
    uint64_t* q_full = bars;
    uint64_t* ring_full = bars + 1;   // [2]
    uint64_t* ring_empty = bars + 3;  // [2]
    uint64_t* s_full = bars + 5;
    uint64_t* p_full = bars + 6;
    uint64_t* acc_done = bars + 7;
    uint64_t* epi = bars + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = gridDim.x - 1 - blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (NH / NKVH);
    const int q0 = qt * BM;
    const int nkv = causal ? (q0 + BM) / BN : Tkv / BN;   // key sub-tiles up to and including the diagonal / all of them
    const int row_base = b * T, kv_row_base = b * Tkv;
    const int q_col = h * HS, k_col = (NH + hk) * HS, v_col = (NH + NKVH + hk) * HS;
    const float scale_log2 = scale * LOG2E;

    if (threadIdx.x == 0) {
        ptx::mbar_init(q_full, 1);
        for (int i = 0; i < 2; i++) {
            ptx::mbar_init(&ring_full[i], 1);
            ptx::mbar_init(&ring_empty[i], 1);
        }
        ptx::mbar_init(s_full, 1);
        ptx::mbar_init(p_full, 8);
        ptx::mbar_init(acc_done, 1);
        ptx::mbar_init(epi, 8);
        *abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, C::TMEM);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t t_s = tmem_base, t_dp = tmem_base + BN, t_dq = tmem_base + 2 * BN;

    if (warp == 0) {
        if (lane == 0) {
            ptx::mbar_arrive_expect_tx(q_full, 2 * C::TILE);
            load_tile<HS, BM>(sQ, &tmQKV, q_full, q_col, row_base + q0);
            load_tile<HS, BM>(sdO, &tmDO, q_full, q_col, row_base + q0);
        }
        __syncwarp();
        for (int j = 0; j < nkv; j++) {
            const int s = j & 1;
            if (!ptx::mbar_wait(&ring_empty[s], ((j >> 1) & 1) ^ 1, abort_flag, status, LLMK_ST_TIMEOUT_TMA_EMPTY, j)) break;
            if (lane == 0) {
                ptx::mbar_arrive_expect_tx(&ring_full[s], 2 * C::RT);
                load_tile<HS, BN>(sRing + s * 2 * C::RT, &tmQKVin, &ring_full[s], k_col, kv_row_base + j * BN);
                load_tile<HS, BN>(sRing + s * 2 * C::RT + C::RT, &tmQKVin, &ring_full[s], v_col, kv_row_base + j * BN);
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        constexpr uint32_t idesc_s = ptx::make_idesc_bf16(BM, BN, 0, 0);
        constexpr uint32_t idesc_acc = ptx::make_idesc_bf16(BM, HS, 0, 1);
        bool ok = ptx::mbar_wait(q_full, 0, abort_flag, status, LLMK_ST_TIMEOUT_TMA_FULL, -1);
        const uint64_t q_desc = kmajor_desc<BM>(ptx::smem_u32(sQ), 0), do_desc = kmajor_desc<BM>(ptx::smem_u32(sdO), 0);
        const uint64_t ds_desc = kmajor_desc<BM>(ptx::smem_u32(sdS), 0);
        const uint32_t ring_addr = ptx::smem_u32(sRing);
        auto issue_s = [&](int j) -> bool {
            const int s = j & 1;
            if (!ptx::mbar_wait(&ring_full[s], (j >> 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_TMA_FULL, j)) return false;
            ptx::tc_fence_after();
            if (lane == 0) {
                const uint64_t k_desc = kmajor_desc<BN>(ring_addr + s * 2 * C::RT, 0), v_desc = kmajor_desc<BN>(ring_addr + s * 2 * C::RT + C::RT, 0);
#pragma unroll
                for (int kk = 0; kk < HS / 16; kk++)
                    ptx::mma_f16_ss(t_s, kmajor_step<BM>(q_desc, kk), kmajor_step<BN>(k_desc, kk), idesc_s, kk > 0 ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < HS / 16; kk++)
                    ptx::mma_f16_ss(t_dp, kmajor_step<BM>(do_desc, kk), kmajor_step<BN>(v_desc, kk), idesc_s, kk > 0 ? 1u : 0u);
                ptx::mma_commit(s_full);
            }
            __syncwarp();
            return true;
        };
        if (ok) ok = issue_s(0);
        for (int j = 0; j < nkv && ok; j++) {
            const int s = j & 1;
            ok = ptx::mbar_wait(p_full, j & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_EMPTY, j);
            if (!ok) break;
            ptx::tc_fence_after();
            if (j + 1 < nkv) {
                ok = issue_s(j + 1);
                if (!ok) break;
            }
            if (lane == 0) {
                const uint64_t k_mn = mnmajor_desc<BN>(ring_addr + s * 2 * C::RT, 0);
#pragma unroll
                for (int kk = 0; kk < BN / 16; kk++)
                    ptx::mma_f16_ss(t_dq, kmajor_step<BM>(ds_desc, kk), mnmajor_step(k_mn, kk), idesc_acc, (j > 0 || kk > 0) ? 1u : 0u);
                ptx::mma_commit(&ring_empty[s]);
                ptx::mma_commit(acc_done);
            }
            __syncwarp();
        }
    } else {
        const int lane_group = warp & 3;
        const int sub = (warp - 2) >> 2;                     // 0 / 1: which half of the columns this warp handles
        const int r = lane_group * 32 + lane;   // query row inside the tile
        const uint32_t lane_off = (uint32_t)(lane_group * 32) << 16;
        const size_t roff = ((size_t)b * NH + h) * T + q0 + r;
        const float Lr = lse[roff] * LOG2E, Dr = dvec[roff];
        const ptx::f32x2 nl2 = ptx::pack2(-Lr, -Lr), nd2 = ptx::pack2(-Dr, -Dr), c2 = ptx::pack2(scale_log2, scale_log2);
        bool ok = true;
        for (int j = 0; j < nkv && ok; j++) {
            ok = ptx::mbar_wait(s_full, j & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, j);
            if (!ok) break;
            if (j > 0) {
                ok = ptx::mbar_wait(acc_done, (j - 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, 1000 + j);
                if (!ok) break;
            }
            ptx::tc_fence_after();
            const int dk0 = j * BN - q0;            // first key of the sub-tile relative to the first query
            const bool diag = causal && dk0 + BN > 0;   // reaches past the first query: some pairs are masked
            uint32_t vsA[32], vdA[32], vsB[32], vdB[32];
            auto process = [&](int c4, const uint32_t (&vs)[32], const uint32_t (&vd)[32]) {
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    float ds[8], p[8];
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        const int c = c4 * 32 + q * 8 + i;   // key column of the sub-tile
                        prob_pair(vs[q * 8 + i], vs[q * 8 + i + 1], vd[q * 8 + i], vd[q * 8 + i + 1], c2, nl2, nd2,
                                  diag && c + dk0 > r, diag && c + 1 + dk0 > r, p + i, ds + i);
                    }
                    store_chunk(sdS, r, c4 * 4 + q, ds);
                }
            };
            // this warp's share of the sub-tile's columns: chunks [sub * NCH, (sub + 1) * NCH)
            constexpr int NCH = BN / 64;
            const int c_first = sub * NCH;
            ptx::tmem_ld_32x32b_x32(t_s + lane_off + c_first * 32, vsA);
            ptx::tmem_ld_32x32b_x32(t_dp + lane_off + c_first * 32, vdA);
#pragma unroll
            for (int i4 = 0; i4 < NCH; i4++) {
                const int c4 = c_first + i4;
                ptx::tmem_ld_wait();
                if (i4 + 1 < NCH) {
                    ptx::tmem_ld_32x32b_x32(t_s + lane_off + (c4 + 1) * 32, (i4 & 1) ? vsA : vsB);
                    ptx::tmem_ld_32x32b_x32(t_dp + lane_off + (c4 + 1) * 32, (i4 & 1) ? vdA : vdB);
                }
                if (i4 & 1) process(c4, vsB, vdB);
                else process(c4, vsA, vdA);
            }
            ptx::tc_fence_before();
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(p_full);
        }
        if (ok) ok = ptx::mbar_wait(acc_done, (nkv - 1) & 1, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, 2000);
        if (ok) {
            ptx::tc_fence_after();
            // dQ (scaled) -> bf16 -> the dS buffer as [128 x 64] staging tiles -> TMA stores
#pragma unroll
            for (int h4 = sub; h4 < HS / 32; h4 += 2) {
                uint32_t v[32];
                ptx::tmem_ld_32x32b_x32(t_dq + lane_off + h4 * 32, v);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    float f[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) f[i] = __uint_as_float(v[q * 8 + i]) * scale;
                    if (rope != nullptr) rope_inverse8(f, rope + (size_t)(q0 + r) * (HS / 2) + h4 * 16 + q * 4);
                    stage_chunk(sdS + (h4 / 2) * (BM * 128), r, (h4 & 1) * 4 + q, f);
                }
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(epi);
            if (warp == 2 && lane == 0) {
                if (ptx::mbar_wait(epi, 0, abort_flag, status, LLMK_ST_TIMEOUT_ACC_FULL, 4000)) {
#pragma unroll
                    for (int c = 0; c < HS / 64; c++) ptx::tma_store_2d(&tmDQKV, sdS + c * (BM * 128), q_col + 64 * c, row_base + q0);
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
        ptx::tmem_dealloc(tmem_base, C::TMEM);
    }
}

template <int HS>
// `kv_qkv` / `dkv_out` / `Tkv` / `causal`: a context-parallel step takes its keys and values from another packed tensor
// (possibly a peer's) and writes dK / dV into a tensor shaped like it; the usual backward passes qkv, dqkv, T, 1.
static int launch(const void* qkv, const void* dout, bf16* dqkv, const float* lse, const float* dvec, int B, int T, int NH, int NKVH,
                  int* status, const float2* rope, cudaStream_t stream, const void* kv_qkv = nullptr, bf16* dkv_out = nullptr,
                  int Tkv = 0, int causal = 1) {
    constexpr int BN = Inner<HS>::BN;
    const bool ring = kv_qkv != nullptr;
    if (!ring) { kv_qkv = qkv; dkv_out = dqkv; Tkv = T; causal = 1; }
    static PerDeviceOnce once_configured;
    if (once_configured.first()) {
        LLMK_CUDA_TRY(cudaFuncSetAttribute(attn_bwd_dkv_tc_kernel<HS>, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvCfg<HS>::SMEM_BYTES));
        LLMK_CUDA_TRY(cudaFuncSetAttribute(attn_bwd_dq_tc_kernel<HS>, cudaFuncAttributeMaxDynamicSharedMemorySize, DqCfg<HS>::SMEM_BYTES));
        LLMK_CUDA_TRY(cudaFuncSetAttribute(attn_bwd_dkv_tc_kernel<HS>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                           cudaSharedmemCarveoutMaxShared));
        LLMK_CUDA_TRY(cudaFuncSetAttribute(attn_bwd_dq_tc_kernel<HS>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                           cudaSharedmemCarveoutMaxShared));
    }
    const uint64_t width = (uint64_t)(NH + 2 * NKVH) * HS, rows = (uint64_t)B * T, cw = (uint64_t)NH * HS;
    const uint64_t kv_rows = (uint64_t)B * Tkv;
    // tq / tq_in: the queries (128-row tiles / sub-tiles); tkv / tkv_in: the keys and values; tdqkv / tdkv: outputs
    CUtensorMap tq, tq_in, tdo, tdo_in, tdqkv, tkv, tkv_in, tdkv;
    int rc;
    if ((rc = gemm::make_tmap_2d(&tq, qkv, width, rows, width, 64, BM))) return rc;
    if ((rc = gemm::make_tmap_2d(&tq_in, qkv, width, rows, width, 64, BN))) return rc;
    if ((rc = gemm::make_tmap_2d(&tdo, dout, cw, rows, cw, 64, BM))) return rc;
    if ((rc = gemm::make_tmap_2d(&tdo_in, dout, cw, rows, cw, 64, BN))) return rc;
    if ((rc = gemm::make_tmap_2d(&tdqkv, dqkv, width, rows, width, 64, BM))) return rc;
    if ((rc = gemm::make_tmap_2d(&tkv, kv_qkv, width, kv_rows, width, 64, BM))) return rc;
    if ((rc = gemm::make_tmap_2d(&tkv_in, kv_qkv, width, kv_rows, width, 64, BN))) return rc;
    if ((rc = gemm::make_tmap_2d(&tdkv, dkv_out, width, kv_rows, width, 64, BM))) return rc;
    const float scale = 1.0f / sqrtf((float)HS);
    // The pipelined kernel has no second CTA on its SM to hide its prologue and epilogue behind, so it only pays off
    // when a CTA loops over many sub-tiles (long sequences, grouped queries): measured 1.08 vs 1.12 ms at T=2048 with
    // 4 query heads per KV head, but 1.00 vs 0.90 ms at T=1024 with one. LLMK_ATTN_BWD_DKV=1|2 forces a version.
    const char* dkv_env = getenv("LLMK_ATTN_BWD_DKV");   // read on every call, so that one process can run both versions
    const bool long_loops = (T / 64) * (NH / NKVH) >= 64;
    const bool use_v2 = dkv_env != nullptr ? dkv_env[0] == '2' : long_loops;
    if (HS == 64 && use_v2 && !ring) {
        static PerDeviceOnce once_configured2;
        if (once_configured2.first()) {
            LLMK_CUDA_TRY(cudaFuncSetAttribute(dkv2::attn_bwd_dkv2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dkv2::SMEM_BYTES));
        }
        // this kernel steps over the queries 64 at a time: its own load maps, whatever sub-tile the others use
        CUtensorMap tq_in64, tdo_in64;
        if ((rc = gemm::make_tmap_2d(&tq_in64, qkv, width, rows, width, 64, 64))) return rc;
        if ((rc = gemm::make_tmap_2d(&tdo_in64, dout, cw, rows, cw, 64, 64))) return rc;
        dkv2::attn_bwd_dkv2_kernel<<<dim3(T / BM, NKVH, B), dkv2::THREADS2, dkv2::SMEM_BYTES, stream>>>(tq, tq_in64, tdo_in64, tdqkv, lse, dvec,
                                                                                                    T, NH, NKVH, scale, status, rope);
    } else {
        attn_bwd_dkv_tc_kernel<HS><<<dim3(Tkv / BM, NKVH, B), THREADS, DkvCfg<HS>::SMEM_BYTES, stream>>>(
            tkv, tq_in, tdo_in, tdkv, lse, dvec, T, NH, NKVH, scale, status, rope, Tkv, causal);
    }
    LLMK_LAUNCH_CHECK();
    attn_bwd_dq_tc_kernel<HS><<<dim3(T / BM, NH, B), THREADS, DqCfg<HS>::SMEM_BYTES, stream>>>(tq, tdo, tkv_in, tdqkv, lse, dvec, T, NH,
                                                                                             NKVH, scale, status, rope, Tkv, causal);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

}  // namespace attn_bwd_tc
}  // namespace llmk

using namespace llmk;

// dqkv (packed, fully overwritten) from dout [B*T, NH*HS]; `dvec` must already hold rowsum(dO*O) as [B,NH,T]
// (llmk_attention_bwd_prep). T must be a multiple of 128.
static int attention_bwd_tc_impl(void* dqkv, const void* dvec, const void* dout, const void* qkv, const void* lse, int B, int T,
                                 int NH, int NKVH, int HS, int* status, const void* rope, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (T % 128 || NH % NKVH || (HS != 64 && HS != 128)) return LLMK_ERR_SHAPE;
    if (reinterpret_cast<uintptr_t>(rope) & 15) return LLMK_ERR_SHAPE;
    if (HS == 64)
        return attn_bwd_tc::launch<64>(qkv, dout, (bf16*)dqkv, (const float*)lse, (const float*)dvec, B, T, NH, NKVH, status,
                                       (const float2*)rope, stream);
    return attn_bwd_tc::launch<128>(qkv, dout, (bf16*)dqkv, (const float*)lse, (const float*)dvec, B, T, NH, NKVH, status,
                                    (const float2*)rope, stream);
}

LLMK_API int llmk_attention_bwd_tc(void* dqkv, const void* dvec, const void* dout, const void* qkv, const void* lse, int B, int T,
                                   int NH, int NKVH, int HS, int* status, void* stream_) {
    return attention_bwd_tc_impl(dqkv, dvec, dout, qkv, lse, B, T, NH, NKVH, HS, status, nullptr, stream_);
}

// One step of context-parallel (ring) attention, backward: the queries of `qkv` [B, T, W] with their output gradient
// `dout`, the FINAL log-sum-exp `lse` and D = rowsum(dO * O) of the merged output, against the keys and values of
// `kv_qkv` [B, Tkv, W] (possibly another rank's chunk in peer memory, pulled by TMA loads). Writes this step's dQ into
// the q columns of `dq_step` [B, T, W] and this rank's contribution to the chunk's dK / dV into the k / v columns of
// `dkv_step` [B, Tkv, W]; the caller sums dQ over the steps and the chunk's owner sums dK / dV over the ranks.
LLMK_API int llmk_attention_bwd_ring_step(void* dq_step, void* dkv_step, const void* dvec, const void* dout, const void* qkv,
                                          const void* kv_qkv, const void* lse, int B, int T, int Tkv, int NH, int NKVH, int HS,
                                          int causal, int* status, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (T % 128 || Tkv % 128 || NH % NKVH || (HS != 64 && HS != 128) || (causal && T != Tkv) || kv_qkv == nullptr) return LLMK_ERR_SHAPE;
    if (HS == 64)
        return attn_bwd_tc::launch<64>(qkv, dout, (bf16*)dq_step, (const float*)lse, (const float*)dvec, B, T, NH, NKVH, status, nullptr,
                                       stream, kv_qkv, (bf16*)dkv_step, Tkv, causal ? 1 : 0);
    return attn_bwd_tc::launch<128>(qkv, dout, (bf16*)dq_step, (const float*)lse, (const float*)dvec, B, T, NH, NKVH, status, nullptr,
                                    stream, kv_qkv, (bf16*)dkv_step, Tkv, causal ? 1 : 0);
}

// The same with the backward of RoPE folded into the dQ and dK output tiles: `qkv` holds ROTATED q and k (as the QKV
// projection with the RoPE epilogue wrote them), `rope` is the [T, HS/2] (cos, sin) table of interleaved pairs, and the
// dq / dk columns of `dqkv` come out as gradients of the un-rotated projections. Same job as the in-tile inverse
// rotation of the reference's GQA backward (llmc/attention_gqa.cuh:184-227).
LLMK_API int llmk_attention_bwd_tc_rope(void* dqkv, const void* dvec, const void* dout, const void* qkv, const void* lse, int B,
                                        int T, int NH, int NKVH, int HS, int* status, const void* rope, void* stream_) {
    if (rope == nullptr) return LLMK_ERR_SHAPE;
    return attention_bwd_tc_impl(dqkv, dvec, dout, qkv, lse, B, T, NH, NKVH, HS, status, rope, stream_);
}
