// Causal flash attention, forward and backward, for MHA and GQA, reading the packed QKV activation
// [B, T, (NH + 2*NKVH) * HS] (q heads, then k heads, then v heads) directly and writing the output
// as [B, T, NH*HS] and the gradient again as a packed tensor: no permute / unpermute / pad kernels.
//
// Jobs covered: attention_forward / attention_backward (reference llmc/attention.cuh:261-338,
// 481-604) and attention_gqa_forward / attention_gqa_backward (llmc/attention_gqa.cuh:415-572).
// Design (this file is the warp-level-MMA implementation; tiles move with cp.async into
// XOR-swizzled shared memory, bf16 m16n8k16 MMAs with fp32 accumulation, exp2-domain online softmax):
//   forward : one CTA per (64 query rows, head, batch), 4 warps x 16 rows, K/V tiles double-buffered;
//   backward: deterministic, no atomics. Kernel "dkv" owns a 64-row K/V tile and loops over the
//             query tiles at or after it (and over the query heads that share the KV head), working
//             on transposed scores so that each warp owns 16 rows of dK and dV; kernel "dq" owns a
//             64-row query tile and loops over the K/V tiles at or before it. Both recompute
//             P = exp2(S*c - LSE) from the saved log-sum-exp; D = rowsum(dO * O) comes from a small
//             pre-pass.
#include "common.cuh"

namespace llmk {
namespace attn {

constexpr int BQ = 64;   // query rows per tile
constexpr int BKV = 64;  // key/value rows per tile
constexpr int THREADS = 128;

// ---------------------------------------------------------------- small PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
// d += a(16x16, row) * b(16x8, col)
__device__ __forceinline__ void mma16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Shared-memory tile [rows][HS] bf16, 16-byte chunks XOR-swizzled with the row so that the eight rows
// touched by one ldmatrix phase land in different banks.
template <int HS>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return (uint32_t)(row * (HS * 2) + ((chunk ^ (row & 7)) << 4));
}

// Copy `rows` x HS bf16 from global (row stride `ld` elements) into a swizzled tile (all threads).
template <int HS>
__device__ __forceinline__ void load_tile_async(uint8_t* tile, const bf16* g, int ld, int rows) {
    constexpr int CPR = HS / 8;  // chunks per row
    for (int idx = threadIdx.x; idx < rows * CPR; idx += THREADS) {
        const int r = idx / CPR, c = idx % CPR;
        cp_async16(tile + tile_off<HS>(r, c), g + (size_t)r * ld + c * 8);
    }
}

// A-operand fragments (16 rows x HS) of this warp's rows from a swizzled tile: frag[kk][0..3]
template <int HS>
__device__ __forceinline__ void load_a_frags(uint32_t (*frag)[4], const uint8_t* tile, int row0) {
    const int lane = threadIdx.x & 31;
    const uint32_t base = smem_u32(tile);
#pragma unroll
    for (int kk = 0; kk < HS / 16; kk++) {
        const int r = row0 + (lane & 7) + 8 * ((lane >> 3) & 1);
        const int c = kk * 2 + (lane >> 4);
        ldsm_x4(frag[kk][0], frag[kk][1], frag[kk][2], frag[kk][3], base + tile_off<HS>(r, c));
    }
}

// acc[nb][4] (16 x 64) += A(16 x HS, fragments) * Bt, where the B tile is stored [n = 64 rows][k = HS].
template <int HS>
__device__ __forceinline__ void mma_a_bT(float (*acc)[4], const uint32_t (*afrag)[4], const uint8_t* btile) {
    const int lane = threadIdx.x & 31;
    const uint32_t base = smem_u32(btile);
#pragma unroll
    for (int nb2 = 0; nb2 < 4; nb2++) {
#pragma unroll
        for (int kk = 0; kk < HS / 16; kk++) {
            uint32_t b0, b1, b2, b3;
            const int r = nb2 * 16 + (lane & 7) + 8 * (lane >> 4);
            const int c = kk * 2 + ((lane >> 3) & 1);
            ldsm_x4(b0, b1, b2, b3, base + tile_off<HS>(r, c));
            mma16816(acc[nb2 * 2], afrag[kk], b0, b1);
            mma16816(acc[nb2 * 2 + 1], afrag[kk], b2, b3);
        }
    }
}

// out[nb][4] (16 x HS) += P(16 x 64, fragments pfrag[kk2][4]) * B, where the B tile is stored [k = 64 rows][n = HS].
template <int HS>
__device__ __forceinline__ void mma_p_b(float (*out)[4], const uint32_t (*pfrag)[4], const uint8_t* btile) {
    const int lane = threadIdx.x & 31;
    const uint32_t base = smem_u32(btile);
#pragma unroll
    for (int kk2 = 0; kk2 < 4; kk2++) {
#pragma unroll
        for (int nb2 = 0; nb2 < HS / 16; nb2++) {
            uint32_t b0, b1, b2, b3;
            const int r = kk2 * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
            const int c = nb2 * 2 + (lane >> 4);
            ldsm_x4_t(b0, b1, b2, b3, base + tile_off<HS>(r, c));
            mma16816(out[nb2 * 2], pfrag[kk2], b0, b1);
            mma16816(out[nb2 * 2 + 1], pfrag[kk2], b2, b3);
        }
    }
}

// 16x64 fp32 accumulators -> bf16 A-operand fragments for a following MMA (k = the 64 columns)
__device__ __forceinline__ void acc_to_frags(uint32_t (*frag)[4], const float (*acc)[4]) {
#pragma unroll
    for (int kk2 = 0; kk2 < 4; kk2++) {
        frag[kk2][0] = pack_bf16(acc[2 * kk2][0], acc[2 * kk2][1]);
        frag[kk2][1] = pack_bf16(acc[2 * kk2][2], acc[2 * kk2][3]);
        frag[kk2][2] = pack_bf16(acc[2 * kk2 + 1][0], acc[2 * kk2 + 1][1]);
        frag[kk2][3] = pack_bf16(acc[2 * kk2 + 1][2], acc[2 * kk2 + 1][3]);
    }
}

// Write this warp's 16 x HS fp32 accumulators (scaled per row) as bf16 into a swizzled staging tile.
template <int HS>
__device__ __forceinline__ void store_acc_to_tile(uint8_t* tile, const float (*acc)[4], int row0, float s0, float s1) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int nb = 0; nb < HS / 8; nb++) {
        const uint32_t lo = pack_bf16(acc[nb][0] * s0, acc[nb][1] * s0);
        const uint32_t hi = pack_bf16(acc[nb][2] * s1, acc[nb][3] * s1);
        *reinterpret_cast<uint32_t*>(tile + tile_off<HS>(row0 + g, nb) + t * 4) = lo;
        *reinterpret_cast<uint32_t*>(tile + tile_off<HS>(row0 + g + 8, nb) + t * 4) = hi;
    }
}
// Copy a swizzled [64][HS] tile to global rows (row stride `ld` elements), 16 bytes per thread per step.
template <int HS>
__device__ __forceinline__ void store_tile(bf16* g, int ld, const uint8_t* tile, int rows) {
    constexpr int CPR = HS / 8;
    for (int idx = threadIdx.x; idx < rows * CPR; idx += THREADS) {
        const int r = idx / CPR, c = idx % CPR;
        *reinterpret_cast<int4*>(g + (size_t)r * ld + c * 8) = *reinterpret_cast<const int4*>(tile + tile_off<HS>(r, c));
    }
}

// ================================================================== forward
template <int HS>
__global__ void __launch_bounds__(THREADS)
attn_fwd_kernel(bf16* __restrict__ out, float* __restrict__ lse, const bf16* __restrict__ qkv, int T, int NH, int NKVH,
                float scale_log2) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int TILE = 64 * HS * 2;
    uint8_t* sQ = smem;
    uint8_t* sK = smem + TILE;      // [2]
    uint8_t* sV = smem + 3 * TILE;  // [2]
    const int qt = gridDim.x - 1 - blockIdx.x;  // heavy (late) tiles first
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (NH / NKVH);
    const int width = (NH + 2 * NKVH) * HS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const bf16* qbase = qkv + ((size_t)b * T + qt * BQ) * width + (size_t)h * HS;
    const bf16* kbase = qkv + (size_t)b * T * width + (size_t)(NH + hk) * HS;
    const bf16* vbase = kbase + (size_t)NKVH * HS;
    const int nkv = qt + 1;

    load_tile_async<HS>(sQ, qbase, width, BQ);
    load_tile_async<HS>(sK, kbase, width, BKV);
    load_tile_async<HS>(sV, vbase, width, BKV);
    cp_async_commit();

    uint32_t qf[HS / 16][4];
    float o[HS / 8][4];
#pragma unroll
    for (int i = 0; i < HS / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int j = 0; j < nkv; j++) {
        const int buf = j & 1;
        if (j + 1 < nkv) {
            load_tile_async<HS>(sK + (buf ^ 1) * TILE, kbase + (size_t)(j + 1) * BKV * width, width, BKV);
            load_tile_async<HS>(sV + (buf ^ 1) * TILE, vbase + (size_t)(j + 1) * BKV * width, width, BKV);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (j == 0) load_a_frags<HS>(qf, sQ, warp * 16);

        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        mma_a_bT<HS>(s, qf, sK + buf * TILE);

        if (j == nkv - 1) {  // diagonal tile: mask keys after the query
            const int r0 = warp * 16 + g;
#pragma unroll
            for (int nb = 0; nb < 8; nb++) {
                const int c = nb * 8 + 2 * t;
                if (c > r0) s[nb][0] = -INFINITY;
                if (c + 1 > r0) s[nb][1] = -INFINITY;
                if (c > r0 + 8) s[nb][2] = -INFINITY;
                if (c + 1 > r0 + 8) s[nb][3] = -INFINITY;
            }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < 8; nb++) {
            mx0 = fmaxf(mx0, fmaxf(s[nb][0], s[nb][1]));
            mx1 = fmaxf(mx1, fmaxf(s[nb][2], s[nb][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0 * scale_log2), mn1 = fmaxf(m1, mx1 * scale_log2);
        const float a0 = exp2f(m0 - mn0), a1 = exp2f(m1 - mn1);
        m0 = mn0;
        m1 = mn1;
        float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
        for (int nb = 0; nb < 8; nb++) {
            s[nb][0] = exp2f(s[nb][0] * scale_log2 - mn0);
            s[nb][1] = exp2f(s[nb][1] * scale_log2 - mn0);
            s[nb][2] = exp2f(s[nb][2] * scale_log2 - mn1);
            s[nb][3] = exp2f(s[nb][3] * scale_log2 - mn1);
            rs0 += s[nb][0] + s[nb][1];
            rs1 += s[nb][2] + s[nb][3];
        }
        l0 = l0 * a0 + rs0;
        l1 = l1 * a1 + rs1;
#pragma unroll
        for (int nb = 0; nb < HS / 8; nb++) {
            o[nb][0] *= a0; o[nb][1] *= a0; o[nb][2] *= a1; o[nb][3] *= a1;
        }
        uint32_t pf[4][4];
        acc_to_frags(pf, s);
        mma_p_b<HS>(o, pf, sV + buf * TILE);
        __syncthreads();  // everyone is done with this buffer before it is refilled
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    store_acc_to_tile<HS>(sQ, o, warp * 16, 1.0f / l0, 1.0f / l1);
    if (t == 0) {
        float* lrow = lse + ((size_t)b * NH + h) * T + qt * BQ + warp * 16;
        lrow[g] = (m0 + log2f(l0)) * 0.6931471805599453f;
        lrow[g + 8] = (m1 + log2f(l1)) * 0.6931471805599453f;
    }
    __syncthreads();
    store_tile<HS>(out + ((size_t)b * T + qt * BQ) * (NH * HS) + (size_t)h * HS, NH * HS, sQ, BQ);
}

// ================================================================== backward pre-pass: D = rowsum(dO * O)
// HS/8 lanes per (batch, head, token) row, 16-byte loads; consecutive rows are consecutive tokens of one head,
// so the fp32 results are written coalesced and every 128-byte line of O / dO is read by one lane group.
template <int HS>
__global__ void __launch_bounds__(256) attn_bwd_prep_kernel(float* __restrict__ dvec, const bf16* __restrict__ out,
                                                            const bf16* __restrict__ dout, long rows, int NH, int T) {
    constexpr int G = HS / 8;
    const long row = ((long)blockIdx.x * blockDim.x + threadIdx.x) / G;   // = (b * NH + h) * T + t
    const int sub = threadIdx.x % G;
    float acc = 0.f;
    if (row < rows) {
        const long bh = row / T;
        const int t = (int)(row % T);
        const long b = bh / NH;
        const int h = (int)(bh % NH);
        const size_t off = (((size_t)b * T + t) * NH + h) * HS + sub * 8;
        float o[8], d[8];
        unpack8(ld128_stream(out + off), o);
        unpack8(ld128_stream(dout + off), d);
#pragma unroll
        for (int i = 0; i < 8; i++) acc = fmaf(o[i], d[i], acc);
    }
#pragma unroll
    for (int m = G / 2; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
    if (row < rows && sub == 0) dvec[row] = acc;
}

static int launch_bwd_prep(float* dvec, const bf16* out, const bf16* dout, int B, int T, int NH, int HS, cudaStream_t stream) {
    const long rows = (long)B * NH * T;
    if (HS == 64) attn_bwd_prep_kernel<64><<<ceil_div(rows * 8, 256), 256, 0, stream>>>(dvec, out, dout, rows, NH, T);
    else if (HS == 128) attn_bwd_prep_kernel<128><<<ceil_div(rows * 16, 256), 256, 0, stream>>>(dvec, out, dout, rows, NH, T);
    else return LLMK_ERR_SHAPE;
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

// ================================================================== backward: dK, dV (KV-tile owned)
template <int HS>
__global__ void __launch_bounds__(THREADS)
attn_bwd_dkv_kernel(bf16* __restrict__ dqkv, const bf16* __restrict__ qkv, const bf16* __restrict__ dout,
                    const float* __restrict__ lse, const float* __restrict__ dvec, int T, int NH, int NKVH, float scale,
                    float scale_log2) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int TILE = 64 * HS * 2;
    uint8_t* sK = smem;               // K tile, later dK staging
    uint8_t* sV = smem + TILE;        // V tile, later dV staging
    uint8_t* sQ = smem + 2 * TILE;    // [2]
    uint8_t* sDO = smem + 4 * TILE;   // [2]
    float* sL = reinterpret_cast<float*>(smem + 6 * TILE);  // [2][64] lse * log2e
    float* sD = sL + 128;                                   // [2][64]
    const int kt = blockIdx.x;
    const int hk = blockIdx.y, b = blockIdx.z;
    const int hr = NH / NKVH;
    const int width = (NH + 2 * NKVH) * HS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const bf16* kbase = qkv + ((size_t)b * T + kt * BKV) * width + (size_t)(NH + hk) * HS;
    const bf16* vbase = kbase + (size_t)NKVH * HS;
    const int nq = T / BQ - kt;        // query tiles kt .. T/BQ-1
    const int total = nq * hr;         // iterations: (head in group, query tile)

    load_tile_async<HS>(sK, kbase, width, BKV);
    load_tile_async<HS>(sV, vbase, width, BKV);

    auto issue = [&](int it, int buf) {
        const int hq = hk * hr + it / nq;
        const int qt = kt + it % nq;
        load_tile_async<HS>(sQ + buf * TILE, qkv + ((size_t)b * T + qt * BQ) * width + (size_t)hq * HS, width, BQ);
        load_tile_async<HS>(sDO + buf * TILE, dout + ((size_t)b * T + qt * BQ) * (NH * HS) + (size_t)hq * HS, NH * HS, BQ);
        if (threadIdx.x < 64) {
            const size_t off = ((size_t)b * NH + hq) * T + qt * BQ + threadIdx.x;
            sL[buf * 64 + threadIdx.x] = lse[off] * 1.4426950408889634f;
            sD[buf * 64 + threadIdx.x] = dvec[off];
        }
    };
    issue(0, 0);
    cp_async_commit();

    uint32_t kf[HS / 16][4], vf[HS / 16][4];
    float dk[HS / 8][4], dv[HS / 8][4];
#pragma unroll
    for (int i = 0; i < HS / 8; i++) {
        dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
        dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f;
    }

    for (int it = 0; it < total; it++) {
        const int buf = it & 1;
        if (it + 1 < total) {
            issue(it + 1, buf ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (it == 0) {
            load_a_frags<HS>(kf, sK, warp * 16);
            load_a_frags<HS>(vf, sV, warp * 16);
        }
        const int qt = kt + it % nq;
        // S^T (16 kv rows x 64 q cols) = K Q^T
        float st[8][4];
#pragma unroll
        for (int i = 0; i < 8; i++) st[i][0] = st[i][1] = st[i][2] = st[i][3] = 0.f;
        mma_a_bT<HS>(st, kf, sQ + buf * TILE);
        // dP^T = V dO^T
        float dpt[8][4];
#pragma unroll
        for (int i = 0; i < 8; i++) dpt[i][0] = dpt[i][1] = dpt[i][2] = dpt[i][3] = 0.f;
        mma_a_bT<HS>(dpt, vf, sDO + buf * TILE);
        const bool diag = (qt == kt);
        const int r0 = warp * 16 + g;  // kv row inside the tile
#pragma unroll
        for (int nb = 0; nb < 8; nb++) {
            const int c = nb * 8 + 2 * t;  // q column inside the tile
            const float L0 = sL[buf * 64 + c], L1 = sL[buf * 64 + c + 1];
            const float D0 = sD[buf * 64 + c], D1 = sD[buf * 64 + c + 1];
            float p00 = exp2f(st[nb][0] * scale_log2 - L0), p01 = exp2f(st[nb][1] * scale_log2 - L1);
            float p10 = exp2f(st[nb][2] * scale_log2 - L0), p11 = exp2f(st[nb][3] * scale_log2 - L1);
            if (diag) {  // key row must not come after the query column
                if (r0 > c) p00 = 0.f;
                if (r0 > c + 1) p01 = 0.f;
                if (r0 + 8 > c) p10 = 0.f;
                if (r0 + 8 > c + 1) p11 = 0.f;
            }
            st[nb][0] = p00; st[nb][1] = p01; st[nb][2] = p10; st[nb][3] = p11;
            dpt[nb][0] = p00 * (dpt[nb][0] - D0);
            dpt[nb][1] = p01 * (dpt[nb][1] - D1);
            dpt[nb][2] = p10 * (dpt[nb][2] - D0);
            dpt[nb][3] = p11 * (dpt[nb][3] - D1);
        }
        uint32_t pf[4][4];
        acc_to_frags(pf, st);
        mma_p_b<HS>(dv, pf, sDO + buf * TILE);  // dV += P^T dO
        acc_to_frags(pf, dpt);
        mma_p_b<HS>(dk, pf, sQ + buf * TILE);   // dK += dS^T Q
        __syncthreads();
    }
    // write dK (scaled) and dV through the K/V tiles
    store_acc_to_tile<HS>(sK, dk, warp * 16, scale, scale);
    store_acc_to_tile<HS>(sV, dv, warp * 16, 1.0f, 1.0f);
    __syncthreads();
    bf16* dkbase = dqkv + ((size_t)b * T + kt * BKV) * width + (size_t)(NH + hk) * HS;
    store_tile<HS>(dkbase, width, sK, BKV);
    store_tile<HS>(dkbase + (size_t)NKVH * HS, width, sV, BKV);
}

// ================================================================== backward: dQ (query-tile owned)
template <int HS>
__global__ void __launch_bounds__(THREADS)
attn_bwd_dq_kernel(bf16* __restrict__ dqkv, const bf16* __restrict__ qkv, const bf16* __restrict__ dout,
                   const float* __restrict__ lse, const float* __restrict__ dvec, int T, int NH, int NKVH, float scale,
                   float scale_log2) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int TILE = 64 * HS * 2;
    uint8_t* sQ = smem;             // Q tile, later dQ staging
    uint8_t* sDO = smem + TILE;
    uint8_t* sK = smem + 2 * TILE;  // [2]
    uint8_t* sV = smem + 4 * TILE;  // [2]
    const int qt = gridDim.x - 1 - blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (NH / NKVH);
    const int width = (NH + 2 * NKVH) * HS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const bf16* qbase = qkv + ((size_t)b * T + qt * BQ) * width + (size_t)h * HS;
    const bf16* kbase = qkv + (size_t)b * T * width + (size_t)(NH + hk) * HS;
    const bf16* vbase = kbase + (size_t)NKVH * HS;
    const int nkv = qt + 1;

    load_tile_async<HS>(sQ, qbase, width, BQ);
    load_tile_async<HS>(sDO, dout + ((size_t)b * T + qt * BQ) * (NH * HS) + (size_t)h * HS, NH * HS, BQ);
    load_tile_async<HS>(sK, kbase, width, BKV);
    load_tile_async<HS>(sV, vbase, width, BKV);
    cp_async_commit();

    const size_t roff = ((size_t)b * NH + h) * T + qt * BQ + warp * 16;
    const float L0 = lse[roff + g] * 1.4426950408889634f, L1 = lse[roff + g + 8] * 1.4426950408889634f;
    const float D0 = dvec[roff + g], D1 = dvec[roff + g + 8];

    uint32_t qf[HS / 16][4], dof[HS / 16][4];
    float dq[HS / 8][4];
#pragma unroll
    for (int i = 0; i < HS / 8; i++) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;

    for (int j = 0; j < nkv; j++) {
        const int buf = j & 1;
        if (j + 1 < nkv) {
            load_tile_async<HS>(sK + (buf ^ 1) * TILE, kbase + (size_t)(j + 1) * BKV * width, width, BKV);
            load_tile_async<HS>(sV + (buf ^ 1) * TILE, vbase + (size_t)(j + 1) * BKV * width, width, BKV);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (j == 0) {
            load_a_frags<HS>(qf, sQ, warp * 16);
            load_a_frags<HS>(dof, sDO, warp * 16);
        }
        float s[8][4], dp[8][4];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
            dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
        }
        mma_a_bT<HS>(s, qf, sK + buf * TILE);    // S = Q K^T
        mma_a_bT<HS>(dp, dof, sV + buf * TILE);  // dP = dO V^T
        const bool diag = (j == nkv - 1);
        const int r0 = warp * 16 + g;
#pragma unroll
        for (int nb = 0; nb < 8; nb++) {
            const int c = nb * 8 + 2 * t;
            float p00 = exp2f(s[nb][0] * scale_log2 - L0), p01 = exp2f(s[nb][1] * scale_log2 - L0);
            float p10 = exp2f(s[nb][2] * scale_log2 - L1), p11 = exp2f(s[nb][3] * scale_log2 - L1);
            if (diag) {
                if (c > r0) p00 = 0.f;
                if (c + 1 > r0) p01 = 0.f;
                if (c > r0 + 8) p10 = 0.f;
                if (c + 1 > r0 + 8) p11 = 0.f;
            }
            dp[nb][0] = p00 * (dp[nb][0] - D0);
            dp[nb][1] = p01 * (dp[nb][1] - D0);
            dp[nb][2] = p10 * (dp[nb][2] - D1);
            dp[nb][3] = p11 * (dp[nb][3] - D1);
        }
        uint32_t pf[4][4];
        acc_to_frags(pf, dp);
        mma_p_b<HS>(dq, pf, sK + buf * TILE);  // dQ += dS K
        __syncthreads();
    }
    store_acc_to_tile<HS>(sQ, dq, warp * 16, scale, scale);
    __syncthreads();
    store_tile<HS>(dqkv + ((size_t)b * T + qt * BQ) * width + (size_t)h * HS, width, sQ, BQ);
}

template <int HS>
static int configure() {
    static PerDeviceOnce once_done;
    if (once_done.first()) {
        LLMK_CUDA_TRY(cudaFuncSetAttribute(attn_fwd_kernel<HS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 5 * 64 * HS * 2));
        LLMK_CUDA_TRY(cudaFuncSetAttribute(attn_bwd_dkv_kernel<HS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           6 * 64 * HS * 2 + 1024));
        LLMK_CUDA_TRY(cudaFuncSetAttribute(attn_bwd_dq_kernel<HS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 6 * 64 * HS * 2));
    }
    return LLMK_OK;
}

}  // namespace attn
}  // namespace llmk

using namespace llmk;
using namespace llmk::attn;

// out [B,T,NH*HS], lse [B,NH,T] (natural log) from packed qkv [B,T,(NH+2*NKVH)*HS]; causal; T % 64 == 0.
LLMK_API int llmk_attention_fwd(void* out, void* lse, const void* qkv, int B, int T, int NH, int NKVH, int HS, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (T % 64 || NH % NKVH || (HS != 64 && HS != 128)) return LLMK_ERR_SHAPE;
    const float scale_log2 = 1.4426950408889634f / sqrtf((float)HS);
    dim3 grid(T / BQ, NH, B);
    int rc;
    if (HS == 64) {
        if ((rc = configure<64>())) return rc;
        attn_fwd_kernel<64><<<grid, THREADS, 5 * 64 * 64 * 2, stream>>>((bf16*)out, (float*)lse, (const bf16*)qkv, T, NH, NKVH,
                                                                      scale_log2);
    } else {
        if ((rc = configure<128>())) return rc;
        attn_fwd_kernel<128><<<grid, THREADS, 5 * 64 * 128 * 2, stream>>>((bf16*)out, (float*)lse, (const bf16*)qkv, T, NH, NKVH,
                                                                        scale_log2);
    }
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

// dqkv (packed, fully overwritten) from dout [B,T,NH*HS]; `dvec` is a [B,NH,T] fp32 scratch for rowsum(dO*O).
LLMK_API int llmk_attention_bwd(void* dqkv, void* dvec, const void* dout, const void* qkv, const void* out, const void* lse,
                                int B, int T, int NH, int NKVH, int HS, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (T % 64 || NH % NKVH || (HS != 64 && HS != 128)) return LLMK_ERR_SHAPE;
    const float scale = 1.0f / sqrtf((float)HS);
    const float scale_log2 = 1.4426950408889634f * scale;
    if (int prc = launch_bwd_prep((float*)dvec, (const bf16*)out, (const bf16*)dout, B, T, NH, HS, stream)) return prc;
    dim3 gkv(T / BKV, NKVH, B), gq(T / BQ, NH, B);
    int rc;
    if (HS == 64) {
        if ((rc = configure<64>())) return rc;
        attn_bwd_dkv_kernel<64><<<gkv, THREADS, 6 * 64 * 64 * 2 + 1024, stream>>>(
            (bf16*)dqkv, (const bf16*)qkv, (const bf16*)dout, (const float*)lse, (const float*)dvec, T, NH, NKVH, scale, scale_log2);
        LLMK_LAUNCH_CHECK();
        attn_bwd_dq_kernel<64><<<gq, THREADS, 6 * 64 * 64 * 2, stream>>>((bf16*)dqkv, (const bf16*)qkv, (const bf16*)dout,
                                                                       (const float*)lse, (const float*)dvec, T, NH, NKVH,
                                                                       scale, scale_log2);
    } else {
        if ((rc = configure<128>())) return rc;
        attn_bwd_dkv_kernel<128><<<gkv, THREADS, 6 * 64 * 128 * 2 + 1024, stream>>>(
            (bf16*)dqkv, (const bf16*)qkv, (const bf16*)dout, (const float*)lse, (const float*)dvec, T, NH, NKVH, scale, scale_log2);
        LLMK_LAUNCH_CHECK();
        attn_bwd_dq_kernel<128><<<gq, THREADS, 6 * 64 * 128 * 2, stream>>>((bf16*)dqkv, (const bf16*)qkv, (const bf16*)dout,
                                                                         (const float*)lse, (const float*)dvec, T, NH, NKVH,
                                                                         scale, scale_log2);
    }
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

// D = rowsum(dO * O) as [B, NH, T] fp32: the pre-pass shared by both backward implementations.
LLMK_API int llmk_attention_bwd_prep(void* dvec, const void* dout, const void* out, int B, int T, int NH, int HS, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    return launch_bwd_prep((float*)dvec, (const bf16*)out, (const bf16*)dout, B, T, NH, HS, stream);
}
