// bf16 GEMM family on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM),
// operands staged by TMA into 128-byte-swizzled shared memory, persistent warp-specialised CTAs.
//
//   mode NT : C[M,N] = A[M,K] * B[N,K]^T      forward linear layers (weight stored (out,in))
//   mode NN : C[M,N] = A[M,K] * B[K,N]        input gradients       (B is the same weight, read MN-major)
//   mode TN : C[M,N] = A[K,M]^T * B[K,N]      weight gradients      (both operands read MN-major, K = tokens)
//
// Epilogue flags (compile-time): +bias[N]; tanh-GELU with the pre-activation stored to a second
// output; multiply by GELU'(aux); add a bf16 [M,N] addend (residual add / gradient accumulation);
// or raw fp32 partials for split-K; RoPE on the q / k heads of a packed QKV projection; SwiGLU over an up | gate tile
// pair; rows scattered to peer GPUs (mixture of experts); the bias gradient summed from the A tiles in shared memory
// (mode TN); the attention backward's D = rowsum(dO * O) beside dO (mode NN). Operands that another kernel is still
// filling are polled for, tile by tile (Params::b_ready / a_ready). Same job as matmul_forward / matmul_forward_gelu /
// matmul_backward in the reference (llmc/matmul.cuh:678-785, 1138-1201, 1238-1338), which has no
// sm_100 path; this is a new design:
//
//   warp 0      : TMA producer  (ring of 128x64 A and 256x64 B tiles, mbarrier tx-count)
//   warp 1      : MMA issuer    (one elected lane; tcgen05.mma; commit -> stage release)
//   warps 2..   : epilogue      (tcgen05.ld 32 lanes x 32 columns -> math -> swizzled smem -> TMA store);
//                 8 warps, 16 for the dGELU epilogue
//   4 more warps: column sums of the A stages (EPI_DBIAS only)
//   TMEM        : 2 x 256 fp32 columns, so the epilogue of tile i overlaps the main loop of tile i+1.
//
// Default: clusters of two CTAs (tcgen05.mma.cta_group::2, one 256x256 tile per pair, 256x256x16 MMAs issued by
// the leader, each CTA loading its own 128 rows of A and its half of B; 5 or 6 stages of 32 KiB per CTA). The
// single-CTA kernel (128x256 tile, 3 or 4 stages) remains as the fallback. No load uses cluster multicast: each CTA
// loads its own tiles, reuse comes from the L2 through the grouped tile order; only tcgen05.commit is multicast
// to the pair. Grouped (batched) problems of equal shape run in one launch (llmk_gemm_grouped).
// Every wait is bounded (ptx::mbar_wait) and reports through `status`.
#include <cstdlib>

#include "ptx_sm100.cuh"

namespace llmk {
namespace gemm {

constexpr int BM = 128, BN = 256, BK = 64;
// 4 pipeline stages when the epilogue needs one staging buffer per warp, 3 when it needs two (a second
// output or a TMA-loaded auxiliary input tile).
// PAIR: two CTAs of a cluster share one 256 x 256 tile (tcgen05 cta_group::2): each loads its own 128 rows of A and
// half of B's 256 columns, which cuts the operand traffic from the L2 by a third and leaves room for 6 stages.
template <int EPI, bool PAIR> struct Cfg;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
template <bool PAIR> struct Geo {
    static constexpr int BN_CTA = PAIR ? BN / 2 : BN;          // B columns this CTA keeps in shared memory
    static constexpr int B_STAGE_BYTES = BN_CTA * BK * 2;      // 16 / 32 KiB
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
};
constexpr int CHUNK_BYTES = 64 * BK * 2;          // one 64(MN) x 64(K) MN-major box = 8 KiB
constexpr int STAGING_BYTES = 32 * 128;           // 32 rows x 64 bf16 per epilogue warp buffer
constexpr int NUM_EPI_WARPS = 8;  // two per TMEM lane group; each takes alternate 64-column chunks
constexpr int MAX_EPI_WARPS = 16;
constexpr int MAX_STAGES = 6;
constexpr int GROUP_M = 8;
constexpr int TMEM_COLS = 512;

enum { MODE_NT = 0, MODE_NN = 1, MODE_TN = 2 };
enum { EPI_BIAS = 1, EPI_GELU = 2, EPI_DGELU = 4, EPI_ADD = 8, EPI_PARTIAL = 16, EPI_ROPE = 32, EPI_SCATTER = 64, EPI_SWIGLU = 128,
       EPI_DBIAS = 256, EPI_DROW = 512 };
constexpr int DB_WARPS = 4;   // EPI_DBIAS: column-sum warps per CTA, one per 32 columns of the A stage

template <int EPI, bool PAIR>
struct Cfg {
    static constexpr bool DUAL = (EPI & (EPI_GELU | EPI_DGELU | EPI_ADD | EPI_DROW)) != 0;
    // SwiGLU epilogue (pair kernel only): three outputs per piece (up, gate, activation), so three staging buffers
    // per epilogue warp and a 4-stage operand ring
    static constexpr bool SWI = (EPI & EPI_SWIGLU) != 0;
    static constexpr int STAGES = PAIR ? (SWI ? 4 : (DUAL ? 5 : 6)) : (DUAL ? 3 : 4);
    // Wide epilogue (pair kernel, dGELU): 16 epilogue warps, four per TMEM lane group, one 64-column chunk each per
    // tile; the result overwrites the aux tile in its staging buffer. With K = 768 this epilogue sets the pace of the
    // kernel and it is bound by latency, not by issue slots or a pipe, so twice the warps per scheduler helps
    // (0.33 -> 0.28-0.30 ms at 65536 x 3072 x 768). The GELU epilogue with its two outputs did not gain from it:
    // 0.317 ms with one staging buffer per warp (the second store waits for the first), 0.343 ms with two buffers and
    // a 3-stage ring, against 0.29 ms with 8 warps. The plain and bias epilogues lost as well (qkv 0.16 -> 0.18 ms,
    // lm-head 3.85 -> 4.02 ms with 16 warps and 5 stages).
    static constexpr bool WIDE = PAIR && EPI == EPI_DGELU;
    static constexpr int EPI_WARPS = WIDE ? 16 : NUM_EPI_WARPS;
    // Bias gradient inside the weight-gradient GEMM (mode TN, A = dout [tokens, OC]): four more warps per CTA read every
    // A stage of the tiles in the first tile column out of shared memory, beside the tensor core, and sum it over the
    // tokens; the bias gradient costs no pass over dout of its own. (Two warps, one per 64-column box, could not keep
    // up with the tensor core: the tiles they summed ran at half speed.)
    static constexpr bool DB = (EPI & EPI_DBIAS) != 0;
    static constexpr int NTHREADS = 32 * (2 + EPI_WARPS + (DB ? DB_WARPS : 0));
    static constexpr int NBUF = SWI ? 3 : ((DUAL && !WIDE) ? 2 : 1);   // staging buffers per epilogue warp
    static constexpr int SMEM_MAIN = STAGES * Geo<PAIR>::STAGE_BYTES + EPI_WARPS * NBUF * STAGING_BYTES;
    static constexpr int SMEM_BYTES = SMEM_MAIN + 1024 /*alignment slack*/ + 512 /*barriers*/;
};

// Packed-pair forms of gelu_fwd / gelu_grad (common.cuh): the same explicitly rounded operations in the same order,
// two values per instruction, so the fused epilogues and the stand-alone kernels give identical bits.
__device__ __forceinline__ ptx::f32x2 tanh2(ptx::f32x2 u) {
    float u0, u1;
    ptx::unpack2(u, u0, u1);
    return ptx::pack2(fast_tanh(u0), fast_tanh(u1));
}
__device__ __forceinline__ ptx::f32x2 gelu_fwd2(ptx::f32x2 x) {
    const ptx::f32x2 kc = ptx::pack2(LLMK_GELU_KC, LLMK_GELU_KC), k = ptx::pack2(LLMK_GELU_K, LLMK_GELU_K);
    const ptx::f32x2 inner = ptx::fma2(ptx::mul2(x, x), kc, k);
    const ptx::f32x2 t = tanh2(ptx::mul2(x, inner));
    const ptx::f32x2 hx = ptx::mul2(x, ptx::pack2(0.5f, 0.5f));
    return ptx::fma2(hx, t, hx);
}
__device__ __forceinline__ ptx::f32x2 gelu_grad2(ptx::f32x2 x) {
    const ptx::f32x2 kc = ptx::pack2(LLMK_GELU_KC, LLMK_GELU_KC), k = ptx::pack2(LLMK_GELU_K, LLMK_GELU_K);
    const ptx::f32x2 kc3 = ptx::pack2(3.0f * LLMK_GELU_KC, 3.0f * LLMK_GELU_KC);
    const ptx::f32x2 one = ptx::pack2(1.0f, 1.0f), half = ptx::pack2(0.5f, 0.5f), minus = ptx::pack2(-1.0f, -1.0f);
    const ptx::f32x2 x2 = ptx::mul2(x, x);
    const ptx::f32x2 t = tanh2(ptx::mul2(x, ptx::fma2(x2, kc, k)));
    const ptx::f32x2 du = ptx::fma2(x2, kc3, k);
    const ptx::f32x2 a = ptx::add2(t, one);
    const ptx::f32x2 b = ptx::fma2(t, minus, one);
    const ptx::f32x2 w = ptx::mul2(ptx::mul2(x, half), du);
    return ptx::mul2(a, ptx::fma2(w, b, half));
}

struct Params {
    int M, N, K;
    int tiles_m, tiles_n, splits, kb_total, kb_per_split;   // tiles_m counts 256-row tiles when `pair`
    int pair;
    // Grouped (batched) problems: `group_m` rows of C per group (0 = one problem). Group g of a tile is m0 / group_m.
    // NT: B is [G*N, K] and bias [G*N]; NN: B is [G*K, N]; TN: A is [G*K, M_g], B is [G*K, N], C is [G*M_g, N].
    int group_m;
    // Rotation of the M-tile order (in tiles): every rank of an expert-parallel layer walks its row blocks starting from
    // a different source rank, so that at any moment the ranks' epilogues store to (and their producers wait for)
    // different peers instead of all hitting the same GPU's NVLink port.
    int m_rotate;
    const bf16* bias;  // [N]
    // EPI_DBIAS (mode TN): dbias[m] (+)= sum over the K rows of A[k][m]. One split: written as bf16 by the kernel
    // (added to the old value with EPI_ADD). Split K: every work unit writes its fp32 sums to
    // db_partial[split * tiles_n + tile column][M] and the split-K reduction kernel finishes them.
    bf16* dbias;
    float* db_partial;
    // EPI_DROW (attention projection's input gradient, head size 64): C = dO and, per row and 64-column chunk (= head),
    // drow[(b * NH + h) * T + t] = sum over the chunk of round_bf16(C) * aux, with aux = O (row = b * T + t): the D
    // term of the attention backward, taken while dO is still in registers instead of in a pass of its own
    float* drow;
    int drow_T, drow_NH;
    const bf16* aux;   // [M,N] pre-GELU input (DGELU) or addend (ADD; may alias C)
    float* partial;    // [splits, M, N] fp32 (PARTIAL)
    int* status;
    // Operand readiness (both optional). A kernel that fills an operand while this GEMM already runs (a parameter
    // all-gather into a staging buffer, a token dispatch into an expert's rows) publishes its progress in device
    // memory; the producer warp acquire-polls, with a time limit, what covers a tile before its first TMA load of it.
    //   b_ready: one int per `b_chunk` consecutive ELEMENTS of B (row-major, as stored); ready when >= b_tick.
    //   a_ready: one int per `a_rows` consecutive ROWS of A; ready when >= a_need (an arrival counter).
    const int* b_ready;
    const int* a_ready;
    long long b_chunk;
    int b_tick, a_rows, a_need;
    int b_nflags;          // flags that cover B (0 = unknown); once a CTA has seen them all it stops looking
    long long ready_limit_ns;
    // EPI_ROPE: rotate the q and k heads of a packed QKV projection in the epilogue. Row r of C is token r % rope_T;
    // columns [0, rope_cols) are heads of rope_hs columns whose interleaved pairs (2i, 2i+1) turn by the angle in
    // rope[token][i] = (cos, sin); the columns after them (v) pass through.
    const float2* rope;
    int rope_T, rope_cols, rope_hs;
    // EPI_SCATTER: the rows of C are the outputs of a mixture-of-experts layer's local experts, stacked as
    // [e_local][source rank][slot]; instead of a local C, row m goes straight into the `back` buffer of the rank that
    // sent the token: sc_dst[src] + ((my_rank * Eloc + e_local) * cap + slot) * N (peer stores of whole 128-byte
    // lines). Every stored (32-row x 64-column) piece is counted per block of `cap` rows in sc_count (local memory,
    // left at zero); the piece that completes a block release-stores sc_epoch into entry sc_off + e of that source
    // rank's arrival table (sc_arrive[src]), which is what the combine kernel there waits for.
    const int* b_ready2;   // EPI_SWIGLU: readiness flags of the gate matrix (b_ready: the up matrix), same geometry
    void* sc_dst[8];
    int* sc_arrive[8];
    int* sc_count;
    int sc_cap, sc_P, sc_Eloc, sc_rank, sc_off, sc_epoch;
};

__device__ __forceinline__ int ld_acquire_sys_s32(const int* ptr) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
    return v;
}

// One thread: wait until flags[f0..f1] >= need (f < 64 is remembered in `done`, so every flag is polled once per
// CTA). On expiry: abort flag, LLMK_ST_TIMEOUT_PEER in the status word, false. The flags may be written by another
// kernel of this GPU or by a peer GPU, hence the system-scope acquire; the fence afterwards orders the TMA (async
// proxy) reads of the data behind the flag after the acquire.
__device__ __forceinline__ bool ready_wait(const int* flags, long long f0, long long f1, int need, uint64_t& done,
                                           long long limit_ns, volatile int* abort_flag, int* status, int tag) {
    for (long long f = f0; f <= f1; f++) {
        if (f < 64 && ((done >> f) & 1ull)) continue;
        if (ld_acquire_sys_s32(flags + f) < need) {
            const uint64_t t0 = ptx::globaltimer_ns();
            uint32_t spins = 0;
            while (ld_acquire_sys_s32(flags + f) < need) {
                if ((++spins & 15u) == 0) {
                    if (*abort_flag) return false;
                    if ((long long)(ptx::globaltimer_ns() - t0) > limit_ns) {
                        *abort_flag = 1;
                        if (status != nullptr && atomicCAS(status, 0, LLMK_ST_TIMEOUT_PEER) == 0) {
                            status[1] = tag;
                            status[2] = (int)blockIdx.x;
                            status[3] = (int)f;
                        }
                        return false;
                    }
                }
                __nanosleep(100);
            }
        }
        if (f < 64) done |= 1ull << f;
    }
    asm volatile("fence.proxy.async.global;" ::: "memory");
    return true;
}

struct Work {
    int m0, n0, kb_begin, kb_end, split, g;
};

struct ExtraMaps {
    CUtensorMap b2, y;
};

__device__ __forceinline__ Work decode_unit(const Params& p, int u) {
    Work w;
    const int tile = u / p.splits;
    w.split = u - tile * p.splits;
    const int group_size = GROUP_M * p.tiles_n;
    const int group = tile / group_size;
    const int first_m = group * GROUP_M;
    const int gm = min(p.tiles_m - first_m, GROUP_M);
    const int r = tile - group * group_size;
    int tm = first_m + r % gm;
    if (p.m_rotate > 0) {
        tm += p.m_rotate;
        if (tm >= p.tiles_m) tm -= p.tiles_m;
    }
    w.m0 = tm * (p.pair ? 2 * BM : BM);
    w.n0 = (r / gm) * BN;
    w.kb_begin = w.split * p.kb_per_split;
    w.kb_end = min(p.kb_total, w.kb_begin + p.kb_per_split);
    w.g = p.group_m > 0 ? w.m0 / p.group_m : 0;
    return w;
}

template <int MODE, int EPI, bool PAIR>
__global__ void __launch_bounds__((Cfg<EPI, PAIR>::NTHREADS), 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmX,
            const __grid_constant__ ExtraMaps xm, const Params p) {
    // tmX: second output (GELU pre-activation) or auxiliary [M,N] input (DGELU / ADD); same geometry as tmC
    // xm (EPI_SWIGLU): b2 = the gate weights (tmB = the up weights), y = the third output (gate; tmX = up, tmC = activation)
    constexpr int STAGES = Cfg<EPI, PAIR>::STAGES;
    constexpr int SMEM_MAIN = Cfg<EPI, PAIR>::SMEM_MAIN;
    constexpr bool DUAL = Cfg<EPI, PAIR>::DUAL;
    constexpr bool WIDE = Cfg<EPI, PAIR>::WIDE;
    constexpr int EPI_WARPS = Cfg<EPI, PAIR>::EPI_WARPS;
    constexpr int STAGE_BYTES = Geo<PAIR>::STAGE_BYTES, BN_CTA = Geo<PAIR>::BN_CTA;
    constexpr bool A_MN = (MODE == MODE_TN);
    constexpr bool B_MN = (MODE != MODE_NT);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* staging = smem + STAGES * STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_MAIN);
    uint64_t* full_bar = bars;                         // [MAX_STAGES]
    uint64_t* empty_bar = bars + MAX_STAGES;           // [MAX_STAGES]
    uint64_t* acc_full = bars + 2 * MAX_STAGES;        // [2]
    uint64_t* acc_empty = bars + 2 * MAX_STAGES + 2;   // [2]
    uint64_t* aux_bar = bars + 2 * MAX_STAGES + 4;     // [MAX_EPI_WARPS]
    uint32_t* relay = reinterpret_cast<uint32_t*>(aux_bar + MAX_EPI_WARPS);   // [MAX_STAGES + 2] EPI_DBIAS, pair: see below
    uint32_t* tmem_slot = relay + MAX_STAGES + 2;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_units = p.tiles_m * p.tiles_n * p.splits;
    const int rank = PAIR ? (int)ptx::cluster_ctarank() : 0;                 // 0 = leader of the pair
    const int unit0 = PAIR ? blockIdx.x / 2 : blockIdx.x;                      // first work unit of this CTA (pair)
    const int unit_step = PAIR ? gridDim.x / 2 : gridDim.x;

    // A failure already recorded in the status word (by an earlier kernel or CTA) makes this kernel skip its work,
    // so that one timed-out wait is not followed by thousands more. A pair takes its leader's view.
    __shared__ int skip_word;
    if (threadIdx.x == 0) {
        skip_word = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
        for (int i = 0; i < STAGES; i++) {
            ptx::mbar_init(&full_bar[i], 1);
            // a stage is free again when the MMAs that read it have finished and, with EPI_DBIAS, when this CTA's
            // column-sum warps have read it too
            ptx::mbar_init(&empty_bar[i], Cfg<EPI, PAIR>::DB ? 1 + DB_WARPS : 1);
            relay[i] = 0;
        }
        for (int i = 0; i < 2; i++) {
            ptx::mbar_init(&acc_full[i], 1);
            ptx::mbar_init(&acc_empty[i], PAIR ? 2 * EPI_WARPS : EPI_WARPS);   // pair: both CTAs' epilogue warps
        }
        for (int i = 0; i < EPI_WARPS; i++) ptx::mbar_init(&aux_bar[i], 1);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&tmA);
        ptx::prefetch_tmap(&tmB);
        ptx::prefetch_tmap(&tmC);
        if (DUAL) ptx::prefetch_tmap(&tmX);
    }
    if (warp == 1) {
        if (PAIR) {
            ptx::tmem_alloc_pair(tmem_slot, TMEM_COLS);
            ptx::tmem_relinquish_pair();
        } else {
            ptx::tmem_alloc(tmem_slot, TMEM_COLS);
            ptx::tmem_relinquish();
        }
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (PAIR) ptx::cluster_sync_all();   // the peer's barriers are initialised before anything can signal them
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const bool skip = (PAIR ? ptx::ld_shared_cluster_u32(&skip_word, 0) : (uint32_t)skip_word) != 0;

    if (skip) {
        // nothing to do: fall through to the teardown
    } else if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        auto load = [&](void* dst, const CUtensorMap* tm, uint64_t* bar, int x, int y) {
            if (PAIR) ptx::tma_load_2d_pair(dst, tm, bar, x, y);   // the bytes are credited to the leader's barrier
            else ptx::tma_load_2d(dst, tm, bar, x, y);
        };
        uint64_t b_done = 0, a_done = 0;
        for (int u = unit0; u < total_units && ok; u += unit_step) {
            const Work w = decode_unit(p, u);
            const int m_own = w.m0 + rank * BM, n_own = w.n0 + rank * BN_CTA;
            if (p.a_ready != nullptr && MODE != MODE_TN) {
                // rows [m_own, m_own + BM) of A must have arrived
                bool fl = true;
                if (lane == 0)
                    fl = ready_wait(p.a_ready, m_own / p.a_rows, (min(m_own + BM, p.M) - 1) / p.a_rows, p.a_need, a_done,
                                    p.ready_limit_ns, abort_flag, p.status, 7000);
                if (!__shfl_sync(0xffffffffu, fl, 0)) { ok = false; break; }
            }
            // SwiGLU: the pair's 256 accumulator columns are 128 hidden units of `up` (loaded by the leader from tmB)
            // followed by the same 128 units of `gate` (loaded by the peer from xm.b2); rows [b_row, b_row + 128) of each
            constexpr bool SWI = (EPI & EPI_SWIGLU) != 0;
            const int b_row = SWI ? w.n0 / 2 : n_own;
            const int b_rows_total = SWI ? p.N / 2 : p.N;
            const int* b_flags = (SWI && rank == 1) ? p.b_ready2 : p.b_ready;
            // every flag of B seen by this CTA (at most 64 are remembered): nothing left to poll, and no index arithmetic
            // (the mask lives in lane 0, which does the polling: its answer is broadcast so that the warp branches as one)
            const bool b_all_lane = p.b_nflags > 0 && p.b_nflags <= 64 &&
                                    b_done == (p.b_nflags == 64 ? ~0ull : ((1ull << p.b_nflags) - 1ull));
            const bool b_all = __shfl_sync(0xffffffffu, (int)b_all_lane, 0) != 0;
            if (b_flags != nullptr && !b_all && MODE == MODE_NT && b_row < b_rows_total) {
                // NT: this CTA's rows [b_row, b_row + BN_CTA) of B, all of K
                bool fl = true;
                if (lane == 0) {
                    const long long e0 = (long long)(b_row + w.g * b_rows_total) * p.K;
                    const long long e1 = (long long)(min(b_row + BN_CTA, b_rows_total) + w.g * b_rows_total) * p.K - 1;
                    fl = ready_wait(b_flags, e0 / p.b_chunk, e1 / p.b_chunk, p.b_tick, b_done, p.ready_limit_ns, abort_flag,
                                    p.status, 7100);
                }
                if (!__shfl_sync(0xffffffffu, fl, 0)) { ok = false; break; }
            }
            const bool b_all_nn = b_all;   // decided once per unit
            const bool small_b = (long long)p.K * p.N * (p.group_m > 0 ? (p.M / p.group_m) : 1) < (1ll << 32) && p.b_chunk < (1ll << 32);
            for (int kb = w.kb_begin; kb < w.kb_end; kb++) {
                if (p.b_ready != nullptr && MODE == MODE_NN && !b_all_nn) {
                    // NN: rows [k0, k0 + 64) of B (the K dimension), whole rows. The index arithmetic runs in 32 bits
                    // when B has fewer than 2^32 elements (64-bit divisions in this loop cost more than the loads)
                    bool fl = true;
                    if (lane == 0) {
                        const long long r0 = (long long)kb * BK + (long long)w.g * p.K;
                        const long long r1 = min((long long)(kb + 1) * BK, (long long)p.K) + (long long)w.g * p.K;
                        long long f0, f1;
                        if (small_b) {
                            f0 = (unsigned)((unsigned)r0 * (unsigned)p.N) / (unsigned)p.b_chunk;
                            f1 = (unsigned)((unsigned)r1 * (unsigned)p.N - 1u) / (unsigned)p.b_chunk;
                        } else {
                            f0 = r0 * p.N / p.b_chunk;
                            f1 = (r1 * p.N - 1) / p.b_chunk;
                        }
                        fl = ready_wait(p.b_ready, f0, f1, p.b_tick, b_done, p.ready_limit_ns, abort_flag, p.status, 7200);
                    }
                    if (!__shfl_sync(0xffffffffu, fl, 0)) { ok = false; break; }
                }
                ok = ptx::mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, LLMK_ST_TIMEOUT_TMA_EMPTY, u);
                if (!ok) break;
                if (lane == 0) {
                    uint8_t* sA = smem + s * STAGE_BYTES;
                    uint8_t* sB = sA + A_STAGE_BYTES;
                    // pair: only the leader arms its barrier, for the bytes of both CTAs
                    if (rank == 0) ptx::mbar_arrive_expect_tx(&full_bar[s], (PAIR ? 2 : 1) * STAGE_BYTES);
                    const int k0 = kb * BK;
                    if (A_MN) {   // TN: group g reads token rows [g*K, (g+1)*K) and its own M_g columns of A
#pragma unroll
                        for (int j = 0; j < BM / 64; j++)
                            load(sA + j * CHUNK_BYTES, &tmA, &full_bar[s], m_own - w.g * p.group_m + 64 * j, k0 + w.g * p.K);
                    } else {
                        load(sA, &tmA, &full_bar[s], k0, m_own);
                    }
                    if (B_MN) {   // NN / TN: the rows of B are the K dimension, stacked per group
#pragma unroll
                        for (int j = 0; j < BN_CTA / 64; j++) load(sB + j * CHUNK_BYTES, &tmB, &full_bar[s], n_own + 64 * j, k0 + w.g * p.K);
                    } else {      // NT: the rows of B are the N dimension, stacked per group
                        load(sB, (SWI && rank == 1) ? &xm.b2 : &tmB, &full_bar[s], k0, b_row + w.g * b_rows_total);
                    }
                }
                __syncwarp();
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
        }
        if (ok) {
            // drain: wait until the MMA warp has released every stage, i.e. all loads landed and were used
            for (int i = 0; i < STAGES; i++) {
                if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, LLMK_ST_TIMEOUT_TMA_EMPTY, -1)) break;
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
        }
    } else if (warp == 1 && rank == 0) {
        // ------------------------------------------------------------ MMA issuer (pair: the leader CTA only)
        constexpr uint32_t idesc = ptx::make_idesc_bf16(PAIR ? 2 * BM : BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
        const uint32_t a_addr0 = ptx::smem_u32(smem), b_addr0 = a_addr0 + A_STAGE_BYTES;
        const uint64_t a_desc0 = A_MN ? ptx::make_smem_desc(a_addr0, CHUNK_BYTES, 1024) : ptx::make_smem_desc(a_addr0, 16, 1024);
        const uint64_t b_desc0 = B_MN ? ptx::make_smem_desc(b_addr0, CHUNK_BYTES, 1024) : ptx::make_smem_desc(b_addr0, 16, 1024);
        int s = 0;
        uint32_t ph = 0;
        int it = 0;
        bool ok = true;
        for (int u = unit0; u < total_units && ok; u += unit_step, it++) {
            const Work w = decode_unit(p, u);
            const int a = it & 1;
            const uint32_t acc_ph = (it >> 1) & 1;
            ok = ptx::mbar_wait(&acc_empty[a], acc_ph ^ 1, abort_flag, p.status, LLMK_ST_TIMEOUT_ACC_EMPTY, u);
            if (!ok) break;
            ptx::tc_fence_after();
            const uint32_t d_tmem = tmem_base + a * BN;
            for (int kb = w.kb_begin; kb < w.kb_end; kb++) {
                ok = ptx::mbar_wait(&full_bar[s], ph, abort_flag, p.status, LLMK_ST_TIMEOUT_TMA_FULL, u);
                if (!ok) break;
                ptx::tc_fence_after();
                if (lane == 0) {
                    // descriptors by arithmetic on the stage-0 ones (start-address field = bytes / 16): the issuer shares
                    // its scheduler with two epilogue warps, so its instruction count per k-block is kept minimal
                    const uint64_t ad = a_desc0 + (uint64_t)(s * (STAGE_BYTES >> 4));
                    const uint64_t bd = b_desc0 + (uint64_t)(s * (STAGE_BYTES >> 4));
#pragma unroll
                    for (int kk = 0; kk < BK / 16; kk++) {
                        const uint64_t adk = ad + (uint64_t)((A_MN ? kk * 2048 : kk * 32) >> 4);
                        const uint64_t bdk = bd + (uint64_t)((B_MN ? kk * 2048 : kk * 32) >> 4);
                        const uint32_t acc = (kb > w.kb_begin || kk > 0) ? 1u : 0u;
                        if (PAIR) ptx::mma_f16_ss_pair(d_tmem, adk, bdk, idesc, acc);
                        else ptx::mma_f16_ss(d_tmem, adk, bdk, idesc, acc);
                    }
                    if (PAIR) ptx::mma_commit_pair(&empty_bar[s]);   // frees the stage in both CTAs
                    else ptx::mma_commit(&empty_bar[s]);
                }
                __syncwarp();
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
            if (!ok) break;
            if (lane == 0) {
                if (PAIR) ptx::mma_commit_pair(&acc_full[a]);
                else ptx::mma_commit(&acc_full[a]);
            }
            __syncwarp();
        }
    } else if (warp >= 2 + EPI_WARPS) {
        // ------------------------------------------------------------ column sums of A (EPI_DBIAS, mode TN)
        // An A stage is BM / 64 boxes of 64 (k) rows x 64 (m) columns, 128 bytes per row, 16-byte pieces swizzled by
        // the row number. A warp takes 32 columns (four pieces) of one box: lane (c, r) adds piece c of rows r, r + 8, ...
        // where a quarter warp reads its four pieces of rows q and q + 4, whose swizzles put them into different halves
        // of the 128-byte bank window (no bank conflicts). The reads share the shared-memory bandwidth with the tensor
        // core's operand reads (which keep it about 80 % busy), so a tile whose every stage is summed runs about 12 %
        // longer. With split K the work is therefore dealt out: the unit of tile column j sums the k-blocks kb with
        // kb % tiles_n == j, every unit writes a partial row, and all units slow down a little instead of a few a lot.
        // Without a split the units of the first tile column sum everything and write the result themselves; the
        // other units' warps just keep step with the ring.
        // The stage's bytes are credited to the LEADER's barrier, which the peer CTA cannot wait on: a lane of the
        // leader's first warp passes each completion on by storing the stage's use count into relay[stage] of the peer,
        // which the peer's warps poll. (A remote mbarrier arrive with release semantics instead of the plain store held
        // the leader's warp for about a microsecond per stage: 0.21 -> 0.45 ms at 3072 x 768 x 65536.) The copy into the
        // peer's shared memory is complete before its bytes are credited to the leader's barrier, so it is in place
        // when the count arrives.
        if constexpr (Cfg<EPI, PAIR>::DB) {
            const int dw = warp - (2 + EPI_WARPS);          // 0..3
            const int box = dw >> 1;
            const int c = (dw & 1) * 4 + (lane & 3);        // 16-byte piece of the box's 128-byte rows
            const int kr = ((lane >> 3) & 3) + 4 * ((lane >> 2) & 1);   // first row: q or q + 4 for quarter warp q
            int s = 0;
            uint32_t ph = 0, pass = 1;                      // pass = use count of the stages in this turn of the ring
            bool ok = true;
            for (int u = unit0; u < total_units && ok; u += unit_step) {
                const Work w = decode_unit(p, u);
                constexpr bool DEAL = (EPI & EPI_PARTIAL) != 0;
                const int tn = w.n0 / BN;
                const bool unit_mine = DEAL || tn == 0;
                int r = DEAL ? w.kb_begin % p.tiles_n : 0;
                ptx::f32x2 acc[4];
#pragma unroll
                for (int j = 0; j < 4; j++) acc[j] = ptx::pack2(0.f, 0.f);
                for (int kb = w.kb_begin; kb < w.kb_end; kb++) {
                    if (PAIR && rank == 1) {
                        // bounded poll of the leader's count for this stage
                        uint32_t spins = 0;
                        uint64_t t0 = 0;
                        while (ptx::ld_shared_acquire_cluster_u32(&relay[s]) != pass) {
                            if ((++spins & 0xfffu) == 0) {
                                if (t0 == 0) t0 = ptx::globaltimer_ns();
                                if (*abort_flag) { ok = false; break; }
                                if (ptx::globaltimer_ns() - t0 > LLMK_WAIT_LIMIT_NS) {
                                    *abort_flag = 1;
                                    if (p.status != nullptr && atomicCAS(p.status, 0, LLMK_ST_TIMEOUT_TMA_FULL) == 0) {
                                        p.status[1] = -3;
                                        p.status[2] = (int)blockIdx.x;
                                        p.status[3] = (int)threadIdx.x;
                                    }
                                    ok = false;
                                    break;
                                }
                            }
                        }
                        ok = __all_sync(0xffffffffu, ok);
                        ptx::fence_proxy_async_smem();   // the tile was written through the async proxy
                    } else {
                        ok = ptx::mbar_wait(&full_bar[s], ph, abort_flag, p.status, LLMK_ST_TIMEOUT_TMA_FULL, -3);
                    }
                    if (!ok) break;
                    if (PAIR && rank == 0 && dw == 0 && lane == 0) ptx::st_shared_cluster_u32(&relay[s], 1, pass);
                    const bool mine = DEAL ? r == tn : unit_mine;
                    if (DEAL && ++r == p.tiles_n) r = 0;
                    if (mine) {
                        const uint8_t* sBox = smem + s * STAGE_BYTES + box * CHUNK_BYTES;
#pragma unroll
                        for (int i = 0; i < BK / 8; i++) {
                            const int k = kr + 8 * i;
                            const uint4 v = *reinterpret_cast<const uint4*>(sBox + k * 128 + ((c ^ (k & 7)) << 4));
                            const uint32_t wd[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                            for (int j = 0; j < 4; j++)   // a bf16 pair -> two fp32 values (low half first)
                                acc[j] = ptx::add2(acc[j], ptx::pack2(__uint_as_float(wd[j] << 16), __uint_as_float(wd[j] & 0xffff0000u)));
                        }
                    }
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&empty_bar[s]);
                    if (++s == STAGES) { s = 0; ph ^= 1; pass++; }
                }
                if (!ok) break;
                if (unit_mine) {
                    // the eight lanes with the same c hold the same 8 columns: fixed-order tree, result in lanes 0..3
                    float f[8];
#pragma unroll
                    for (int j = 0; j < 4; j++) ptx::unpack2(acc[j], f[2 * j], f[2 * j + 1]);
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        f[j] += __shfl_xor_sync(0xffffffffu, f[j], 4);
                        f[j] += __shfl_xor_sync(0xffffffffu, f[j], 8);
                        f[j] += __shfl_xor_sync(0xffffffffu, f[j], 16);
                    }
                    const int col = w.m0 + rank * BM + box * 64 + c * 8;
                    if (lane < 4 && col < p.M) {
                        if (EPI & EPI_PARTIAL) {
                            float4* dst = reinterpret_cast<float4*>(p.db_partial + (size_t)(w.split * p.tiles_n + tn) * p.M + col);
                            dst[0] = make_float4(f[0], f[1], f[2], f[3]);
                            dst[1] = make_float4(f[4], f[5], f[6], f[7]);
                        } else {
                            if (EPI & EPI_ADD) {
                                float old[8];
                                unpack8(ld128(p.dbias + col), old);
#pragma unroll
                                for (int j = 0; j < 8; j++) f[j] += old[j];
                            }
                            st128(p.dbias + col, pack8(f));
                        }
                    }
                }
            }
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogue warps
        const int e = warp - 2;              // 0..EPI_WARPS-1
        const int lane_group = warp & 3;     // TMEM lanes [32*lane_group, +32) are visible to this warp
        constexpr int CH_STEP = EPI_WARPS / 4;   // warps per lane group = stride over the 64-column chunks
        const int chunk_sel = e >> 2;        // this warp takes chunks chunk_sel, chunk_sel + CH_STEP, ...
        constexpr int NBUF = Cfg<EPI, PAIR>::NBUF;
        uint8_t* buf = staging + e * NBUF * STAGING_BYTES;            // output tile
        uint8_t* buf2 = NBUF == 2 ? buf + STAGING_BYTES : buf;        // second output / aux input (DUAL); wide dGELU: the same buffer
        constexpr bool AUX_IN = (EPI & (EPI_DGELU | EPI_ADD | EPI_DROW)) != 0;
        uint32_t aux_ph = 0;
        int it = 0;
        bool ok = true;
        for (int u = unit0; u < total_units && ok; u += unit_step, it++) {
            const Work w = decode_unit(p, u);
            const int a = it & 1;
            const uint32_t acc_ph = (it >> 1) & 1;
            const int row0 = w.m0 + rank * BM + lane_group * 32;
            if (AUX_IN && w.n0 + chunk_sel * 64 < p.N) {
                // fetch the first aux tile while the main loop of this tile is still running
                if (lane == 0) {
                    if (WIDE) ptx::tma_store_wait_read<0>();   // wide dGELU: the buffer was the source of the previous tile's store
                    ptx::mbar_arrive_expect_tx(&aux_bar[e], STAGING_BYTES);
                    ptx::tma_load_2d(buf2, &tmX, &aux_bar[e], w.n0 + chunk_sel * 64, row0);
                }
                __syncwarp();
            }
            ok = ptx::mbar_wait(&acc_full[a], acc_ph, abort_flag, p.status, LLMK_ST_TIMEOUT_ACC_FULL, u);
            if (!ok) break;
            ptx::tc_fence_after();
            const int row = row0 + lane;
            const bool row_ok = row < p.M;
            const uint32_t t_row = tmem_base + a * BN + ((uint32_t)(lane_group * 32) << 16);
#pragma unroll 1
            for (int chunk = chunk_sel; chunk < BN / 64; chunk += CH_STEP) {
                const int n_base = w.n0 + chunk * 64;
                if (n_base >= p.N) break;
                if constexpr ((EPI & EPI_SWIGLU) != 0) {
                    // one piece per warp and tile: accumulator chunk `chunk_sel` holds 64 hidden units of `up`, chunk
                    // `chunk_sel + 2` the same units of `gate`. Both are rounded to bf16 and stored (the backward needs
                    // them), and the activation gate * sigmoid(gate) * up is computed from the ROUNDED values, so that
                    // recomputing it later from the stored tensors gives the same bits as the stand-alone kernel.
                    if (chunk != chunk_sel) break;
                    const int hcol = w.n0 / 2 + chunk_sel * 64;      // hidden-unit column of this piece in the [M, H] outputs
                    if (hcol >= p.N / 2) break;
                    uint8_t* bufU = buf + STAGING_BYTES;
                    uint8_t* bufG = buf + 2 * STAGING_BYTES;
                    if (lane == 0) ptx::tma_store_wait_read<0>();      // the previous tile's stores have read the buffers
                    __syncwarp();
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        uint32_t vu[32], vg[32];
                        ptx::tmem_ld_32x32b_x32(t_row + chunk_sel * 64 + half * 32, vu);
                        ptx::tmem_ld_32x32b_x32(t_row + (chunk_sel + 2) * 64 + half * 32, vg);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            float u[8], g[8];
#pragma unroll
                            for (int j = 0; j < 8; j++) {
                                u[j] = __uint_as_float(vu[q * 8 + j]);
                                g[j] = __uint_as_float(vg[q * 8 + j]);
                            }
                            const bf16x8 ub = pack8(u), gb = pack8(g);
                            unpack8(ub, u);
                            unpack8(gb, g);
#pragma unroll
                            for (int j = 0; j < 8; j++) g[j] = g[j] * (1.0f / (1.0f + __expf(-g[j]))) * u[j];
                            const int cc = half * 4 + q;
                            const uint32_t off = lane * 128 + ((cc ^ (lane & 7)) << 4);
                            *reinterpret_cast<bf16x8*>(bufU + off) = ub;
                            *reinterpret_cast<bf16x8*>(bufG + off) = gb;
                            *reinterpret_cast<bf16x8*>(buf + off) = pack8(g);
                        }
                    }
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        ptx::tma_store_2d(&tmC, buf, hcol, row0);
                        ptx::tma_store_2d(&tmX, bufU, hcol, row0);
                        ptx::tma_store_2d(&xm.y, bufG, hcol, row0);
                        ptx::tma_store_commit();
                    }
                    break;
                }
                if constexpr (WIDE) {
                    // dGELU, one chunk per warp and tile, 32 columns at a time: result = acc * GELU'(aux), written over the aux tile
                    ok = ptx::mbar_wait(&aux_bar[e], aux_ph, abort_flag, p.status, LLMK_ST_TIMEOUT_ACC_FULL, -2);
                    aux_ph ^= 1;
                    if (!ok) break;
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        uint32_t v[32];
                        ptx::tmem_ld_32x32b_x32(t_row + chunk * 64 + half * 32, v);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const int cc = half * 4 + q;
                            const uint32_t off = lane * 128 + ((cc ^ (lane & 7)) << 4);
                            float g[8], x[8];
                            unpack8(*reinterpret_cast<const bf16x8*>(buf + off), g);
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                const ptx::f32x2 acc2 = ptx::pack2(__uint_as_float(v[q * 8 + 2 * j]), __uint_as_float(v[q * 8 + 2 * j + 1]));
                                ptx::unpack2(ptx::mul2(acc2, gelu_grad2(ptx::pack2(g[2 * j], g[2 * j + 1]))), x[2 * j], x[2 * j + 1]);
                            }
                            *reinterpret_cast<bf16x8*>(buf + off) = pack8(x);
                        }
                    }
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        ptx::tma_store_2d(&tmC, buf, n_base, row0);
                        ptx::tma_store_commit();
                    }
                    continue;
                }
                if (EPI & EPI_PARTIAL) {
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        uint32_t v[32];
                        ptx::tmem_ld_32x32b_x32(t_row + chunk * 64 + half * 32, v);
                        ptx::tmem_ld_wait();
                        const int col0 = n_base + half * 32;
                        if (row_ok) {
                            float* dst = p.partial + ((size_t)w.split * p.M + row) * p.N + col0;
#pragma unroll
                            for (int q = 0; q < 8; q++) {
                                if (col0 + q * 4 < p.N) {
                                    float4 f = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                                           __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
                                    *reinterpret_cast<float4*>(dst + q * 4) = f;
                                }
                            }
                        }
                    }
                    continue;
                }
                bf16x8 res[8];
                bf16x8 res2[(EPI & EPI_GELU) ? 8 : 1];
                float drow_acc = 0.f;
                // both TMEM loads of the chunk and its bias are in flight before anything waits: a warp has only one other
                // epilogue warp on its scheduler to hide latency behind, so the loads overlap each other instead
                uint32_t vv[2][32];
                ptx::tmem_ld_32x32b_x32(t_row + chunk * 64, vv[0]);
                ptx::tmem_ld_32x32b_x32(t_row + chunk * 64 + 32, vv[1]);
                bf16x8 bias_v[(EPI & EPI_BIAS) ? 8 : 1];
                if (EPI & EPI_BIAS) {
#pragma unroll
                    for (int cc = 0; cc < 8; cc++)
                        if (n_base + cc * 8 < p.N) bias_v[(EPI & EPI_BIAS) ? cc : 0] = *reinterpret_cast<const bf16x8*>(p.bias + (size_t)w.g * p.N + n_base + cc * 8);
                }
                if (AUX_IN) {
                    ok = ptx::mbar_wait(&aux_bar[e], aux_ph, abort_flag, p.status, LLMK_ST_TIMEOUT_ACC_FULL, -2);
                    aux_ph ^= 1;
                }
                ptx::tmem_ld_wait();
                if (!ok) break;
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    const uint32_t (&v)[32] = vv[half];
                    const int col0 = n_base + half * 32;
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        // two values per FMA-pipe instruction: with K = 768 the epilogue of the GELU / dGELU GEMMs has as
                        // many cycles of per-element math as the main loop has of MMA, so its instruction count matters
                        ptx::f32x2 xp[4];
                        float x[8];
#pragma unroll
                        for (int j = 0; j < 4; j++) xp[j] = ptx::pack2(__uint_as_float(v[q * 8 + 2 * j]), __uint_as_float(v[q * 8 + 2 * j + 1]));
                        const int col = col0 + q * 8;
                        const int cc = half * 4 + q;
                        const uint32_t off = lane * 128 + ((cc ^ (lane & 7)) << 4);
                        if ((EPI & EPI_BIAS) && col < p.N) {
                            float b[8];
                            unpack8(bias_v[(EPI & EPI_BIAS) ? cc : 0], b);
#pragma unroll
                            for (int j = 0; j < 4; j++) xp[j] = ptx::add2(xp[j], ptx::pack2(b[2 * j], b[2 * j + 1]));
                        }
                        if ((EPI & EPI_ROPE) && n_base < p.rope_cols) {
                            // 8 columns = 4 pairs of one head; the accumulators are rotated in fp32 and rounded once
                            const int tok = (row_ok ? row : 0) % p.rope_T;
                            const float4* fr = reinterpret_cast<const float4*>(p.rope + (size_t)tok * (p.rope_hs >> 1) +
                                                                               (((n_base % p.rope_hs) + half * 32 + q * 8) >> 1));
                            const float4 f0 = __ldg(fr), f1 = __ldg(fr + 1);
                            const ptx::f32x2 cs[4] = {ptx::pack2(f0.x, f0.x), ptx::pack2(f0.z, f0.z), ptx::pack2(f1.x, f1.x), ptx::pack2(f1.z, f1.z)};
                            const float sn[4] = {f0.y, f0.w, f1.y, f1.w};
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                float x0, x1;
                                ptx::unpack2(xp[j], x0, x1);
                                // (x0, x1) -> (x0 c - x1 s, x1 c + x0 s)
                                xp[j] = ptx::fma2(xp[j], cs[j], ptx::pack2(-x1 * sn[j], x0 * sn[j]));
                            }
                        }
                        if (AUX_IN && !(EPI & EPI_DROW)) {
                            float g[8];
                            unpack8(*reinterpret_cast<const bf16x8*>(buf2 + off), g);
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                const ptx::f32x2 gp = ptx::pack2(g[2 * j], g[2 * j + 1]);
                                xp[j] = (EPI & EPI_DGELU) ? ptx::mul2(xp[j], gelu_grad2(gp)) : ptx::add2(xp[j], gp);
                            }
                        }
#pragma unroll
                        for (int j = 0; j < 4; j++) ptx::unpack2(xp[j], x[2 * j], x[2 * j + 1]);
                        if (EPI & EPI_GELU) {
                            // the activation is computed from the ROUNDED pre-activation, so that recomputing
                            // it later from the stored bf16 tensor gives the same bits
                            const bf16x8 pre = pack8(x);
                            res2[(EPI & EPI_GELU) ? cc : 0] = pre;
                            unpack8(pre, x);
#pragma unroll
                            for (int j = 0; j < 4; j++) ptx::unpack2(gelu_fwd2(ptx::pack2(x[2 * j], x[2 * j + 1])), x[2 * j], x[2 * j + 1]);
                        }
                        res[cc] = pack8(x);
                        if (EPI & EPI_DROW) {
                            // the products use the ROUNDED output, as a pass over the stored tensor would
                            float r[8], o[8];
                            unpack8(res[cc], r);
                            unpack8(*reinterpret_cast<const bf16x8*>(buf2 + off), o);
#pragma unroll
                            for (int j = 0; j < 8; j++) drow_acc = fmaf(o[j], r[j], drow_acc);
                        }
                    }
                }
                if ((EPI & EPI_DROW) && row_ok) {
                    const int bi = row / p.drow_T;
                    p.drow[((size_t)bi * p.drow_NH + (n_base >> 6)) * p.drow_T + (row - bi * p.drow_T)] = drow_acc;
                }
                if (lane == 0) ptx::tma_store_wait_read<0>();  // earlier stores have finished reading the buffers
                __syncwarp();
                if (AUX_IN && chunk + 2 < BN / 64 && n_base + 128 < p.N) {
                    // every lane has consumed the aux tile (res[] is complete): fetch the next one
                    if (lane == 0) {
                        ptx::mbar_arrive_expect_tx(&aux_bar[e], STAGING_BYTES);
                        ptx::tma_load_2d(buf2, &tmX, &aux_bar[e], n_base + 128, row0);
                    }
                }
#pragma unroll
                for (int cc = 0; cc < 8; cc++) {
                    const uint32_t off = lane * 128 + ((cc ^ (lane & 7)) << 4);
                    *reinterpret_cast<bf16x8*>(buf + off) = res[cc];
                    if (EPI & EPI_GELU) *reinterpret_cast<bf16x8*>(buf2 + off) = res2[(EPI & EPI_GELU) ? cc : 0];
                }
                if constexpr ((EPI & EPI_SCATTER) != 0) {
                    // the staged 32 x 64 piece leaves through the generic proxy: 8 lanes write one row's 128 bytes, so
                    // a warp store covers four whole lines of the destination rank's memory
                    __syncwarp();
                    const int blocks_first = row0 / p.sc_cap;
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        const int rr = k * 4 + (lane >> 3), seg = lane & 7;
                        const int m = row0 + rr;
                        if (m < p.M && n_base + seg * 8 < p.N) {
                            const int blk = m / p.sc_cap, slot = m - blk * p.sc_cap;
                            const int src = blk % p.sc_P, el = blk / p.sc_P;
                            bf16* dst = static_cast<bf16*>(p.sc_dst[src]) +
                                        ((size_t)(p.sc_rank * p.sc_Eloc + el) * p.sc_cap + slot) * p.N + n_base + seg * 8;
                            *reinterpret_cast<bf16x8*>(dst) = *reinterpret_cast<const bf16x8*>(buf + rr * 128 + ((seg ^ (rr & 7)) << 4));
                        }
                    }
                    __syncwarp();
                    if (lane == 0) {
                        __threadfence_system();
                        // rows [row0, row0 + 32) lie in at most two blocks (cap >= 32 is checked on the host)
                        const int row_end = min(row0 + 32, p.M);
                        const int per_block = p.sc_cap * ((p.N + 63) / 64);   // pieces are counted in rows
                        for (int blk = blocks_first; blk * p.sc_cap < row_end; blk++) {
                            const int lo = max(row0, blk * p.sc_cap), hi = min(row_end, (blk + 1) * p.sc_cap);
                            if (hi <= lo) continue;
                            if (atomicAdd(p.sc_count + blk, hi - lo) + (hi - lo) == per_block) {
                                p.sc_count[blk] = 0;
                                __threadfence_system();
                                const int src = blk % p.sc_P, el = blk / p.sc_P;
                                asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p.sc_arrive[src] + p.sc_off + p.sc_rank * p.sc_Eloc + el),
                                             "r"(p.sc_epoch)
                                             : "memory");
                            }
                        }
                    }
                    __syncwarp();
                } else {
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        ptx::tma_store_2d(&tmC, buf, n_base, row0);
                        if (EPI & EPI_GELU) ptx::tma_store_2d(&tmX, buf2, n_base, row0);
                        ptx::tma_store_commit();
                    }
                }
            }
            if (!ok) break;
            // accumulator fully read by this warp: hand it back to the MMA warp
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) ptx::mbar_arrive_cluster(&acc_empty[a], 0);   // the leader's barrier counts both CTAs' warps
                else ptx::mbar_arrive(&acc_empty[a]);
            }
        }
        if (lane == 0) ptx::tma_store_wait_all<0>();
        __syncwarp();
    }

    // ---------------------------------------------------------------- teardown (all paths meet here)
    ptx::tc_fence_before();
    __syncthreads();
    if (PAIR) ptx::cluster_sync_all();   // the leader's MMAs read the peer's shared memory and signal its barriers
    if (warp == 1) {
        ptx::tc_fence_after();
        if (PAIR) ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
        else ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// fp32 split-K partials -> bf16 output (optionally += existing contents).
// With `dbias`: the first M / 8 threads also finish the bias gradient from db_partial [db_rows, M] (EPI_DBIAS).
__global__ void splitk_reduce_kernel(bf16* __restrict__ out, const float* __restrict__ partial, size_t n, int splits,
                                     int accumulate, bf16* __restrict__ dbias, const float* __restrict__ db_partial, int M,
                                     int db_rows) {
    size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= n) return;
    if (dbias != nullptr && i < (size_t)M) {
        float d[8];
        if (accumulate) {
            unpack8(ld128(dbias + i), d);
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) d[j] = 0.f;
        }
        for (int s = 0; s < db_rows; s++) {
            const float4* src = reinterpret_cast<const float4*>(db_partial + (size_t)s * M + i);
            const float4 a = src[0], b = src[1];
            d[0] += a.x; d[1] += a.y; d[2] += a.z; d[3] += a.w;
            d[4] += b.x; d[5] += b.y; d[6] += b.z; d[7] += b.w;
        }
        st128(dbias + i, pack8(d));
    }
    float acc[8];
    if (accumulate) {
        unpack8(ld128(out + i), acc);
    } else {
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] = 0.f;
    }
    for (int s = 0; s < splits; s++) {
        const float4* src = reinterpret_cast<const float4*>(partial + (size_t)s * n + i);
        float4 a = __ldcs(src), b = __ldcs(src + 1);
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    st128(out + i, pack8(acc));
}

// ------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// 2-D bf16 row-major tensor [outer, inner] with 128-byte swizzle; box = [box_outer, box_inner].
int make_tmap_2d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_elems,
                 uint32_t box_inner, uint32_t box_outer) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return LLMK_ERR_DRIVER;
    cuuint64_t gdim[2] = {inner, outer};
    cuuint64_t gstride[1] = {row_stride_elems * 2};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? LLMK_OK : LLMK_ERR_TMAP;
}

static int query_pair_clusters();

template <int MODE, int EPI>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const CUtensorMap& tmX, const ExtraMaps& xm,
                  const Params& p, int max_ctas, cudaStream_t stream) {
    const int g_num_sms = sm_count_current_device();
    if (g_num_sms <= 0) return LLMK_ERR_CUDA;
    const int g_pair_clusters = p.pair ? query_pair_clusters() : 0;
    const int units = p.tiles_m * p.tiles_n * p.splits;
    if (p.pair) {
        constexpr int SMEM_BYTES = Cfg<EPI, true>::SMEM_BYTES;
        static PerDeviceOnce once_configured;
        if (once_configured.first()) {
            LLMK_CUDA_TRY(cudaFuncSetAttribute(gemm_kernel<MODE, EPI, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        }
        int clusters = units < g_pair_clusters ? units : g_pair_clusters;
        if (max_ctas > 0 && clusters > max_ctas / 2) clusters = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * clusters);
        cfg.blockDim = dim3(Cfg<EPI, true>::NTHREADS);
        cfg.dynamicSmemBytes = SMEM_BYTES;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        LLMK_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_kernel<MODE, EPI, true>, tmA, tmB, tmC, tmX, xm, p));
        return LLMK_OK;
    }
    if (EPI & (EPI_SWIGLU | EPI_DBIAS)) return LLMK_ERR_SHAPE;   // these epilogues exist for the pair kernel only
    constexpr int SMEM_BYTES = Cfg<EPI, false>::SMEM_BYTES;
    static PerDeviceOnce once_configured;
    if (once_configured.first()) {
        LLMK_CUDA_TRY(cudaFuncSetAttribute(gemm_kernel<MODE, EPI, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    }
    int grid = units < g_num_sms ? units : g_num_sms;
    if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
    gemm_kernel<MODE, EPI, false><<<grid, Cfg<EPI, false>::NTHREADS, SMEM_BYTES, stream>>>(tmA, tmB, tmC, tmX, xm, p);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

// Number of resident CTA pairs for the pair kernel on the current device (queried once per device; 0 disables
// the pair path).
static int query_pair_clusters() {
    static int cached[LLMK_MAX_DEVICES];
    static bool known[LLMK_MAX_DEVICES] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= LLMK_MAX_DEVICES) return 0;
    if (known[dev]) return cached[dev];
    known[dev] = true;
    int& g_pair_clusters = cached[dev];
    g_pair_clusters = 0;
    const char* env = getenv("LLMK_GEMM_PAIR");
    if (env != nullptr && env[0] == '0') return 0;
    constexpr int SMEM_BYTES = Cfg<0, true>::SMEM_BYTES;
    if (cudaFuncSetAttribute(gemm_kernel<MODE_NT, 0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2);
    cfg.blockDim = dim3(Cfg<0, true>::NTHREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_kernel<MODE_NT, 0, true>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    g_pair_clusters = n;
    return n;
}

}  // namespace gemm
}  // namespace llmk

using namespace llmk;
using namespace llmk::gemm;

// How many CTA pairs the pair (cta_group::2) kernel keeps resident; 0 when that path is off (LLMK_GEMM_PAIR=0).
LLMK_API int llmk_gemm_pair_clusters() { return query_pair_clusters(); }

// Bytes of fp32 workspace that llmk_gemm needs for (mode, M, N, K) with the split count it will pick.
LLMK_API long llmk_gemm_workspace_bytes(int mode, int M, int N, int K, int num_sms);

static int pick_splits(int mode, int M, int N, int K, int num_sms, int tile_rows = BM) {
    if (mode != MODE_TN) return 1;
    const int tiles = ceil_div(M, tile_rows) * ceil_div(N, BN);
    const int kb = ceil_div(K, BK);
    if (tiles >= 2 * num_sms) return 1;
    // pick the split count whose work units fill whole waves best; ties go to fewer splits
    int best = 1;
    double best_cost = 1e30;
    for (int s = 1; s <= 16 && s <= kb; s++) {
        const int units = tiles * s;
        const int waves = ceil_div(units, num_sms);
        const double cost = (double)waves * ceil_div(kb, s) + 0.35 * s;  // k-blocks on the critical path + reduce cost
        if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
    }
    return best;
}

long llmk_gemm_workspace_bytes(int mode, int M, int N, int K, int num_sms) {
    // the larger of what the single-CTA and the pair kernel would pick (the choice is made at launch time)
    int s = pick_splits(mode, M, N, K, num_sms > 0 ? num_sms : 148);
    const int s2 = pick_splits(mode, M, N, K, (num_sms > 0 ? num_sms : 148) / 2, 2 * BM);
    if (s2 > s) s = s2;
    return s > 1 ? (long)s * M * N * 4 + (long)s * ceil_div(N, BN) * M * 4 /* bias-gradient partials */ : 0;
}

// C = op(A) op(B) with the epilogue selected by `epi` (bit-or of: 1 bias, 2 GELU with pre-activation
// to C2, 4 multiply by GELU'(aux), 8 add aux). For mode TN, `epi` 8 means C += result and the
// launcher may split K through `workspace`. All matrices are dense row-major bf16; K, N (and M for
// TN) must be multiples of 8 so that every row starts on a 16-byte boundary.
struct Ready {
    const int* b_ready = nullptr;
    const int* a_ready = nullptr;
    long long b_chunk = 1;
    int b_tick = 0, a_rows = 1, a_need = 0, b_nflags = 0;
    long long limit_ns = 0;
    const float2* rope = nullptr;
    int rope_T = 1, rope_cols = 0, rope_hs = 64;
    int rotate_rows = 0;                    // start the walk over the rows of C this many rows in (rounded down to tiles)
    const void* b2 = nullptr;               // EPI_SWIGLU: the gate weights, the third output, the gate's readiness flags
    void* c3 = nullptr;
    const int* b_ready2 = nullptr;
    const long long* sc_dst = nullptr;      // EPI_SCATTER: host arrays of P pointers
    const long long* sc_arrive = nullptr;
    int* sc_count = nullptr;
    int sc_cap = 0, sc_P = 0, sc_Eloc = 0, sc_rank = 0, sc_off = 0, sc_epoch = 0;
    void* dbias = nullptr;                  // EPI_DBIAS: [M] bf16
    float* drow = nullptr;                  // EPI_DROW: [M / T, N / 64, T] fp32
    int drow_T = 1, drow_NH = 1;
};

static int gemm_impl(int mode, int epi, const void* A, const void* B, void* C, void* C2, const void* bias, const void* aux,
                     int M_group, int N, int K, int groups, void* workspace, long workspace_bytes, int* status, int max_ctas,
                     void* stream_, const Ready& ready = Ready()) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (M_group <= 0 || N <= 0 || K <= 0 || groups <= 0) return LLMK_ERR_SHAPE;
    if ((long)M_group * groups > 0x7fffffffL) return LLMK_ERR_SHAPE;
    const int M = M_group * groups;   // rows of C over all groups
    if (epi & EPI_PARTIAL) return LLMK_ERR_SHAPE;   // internal: chosen here when the K dimension is split
    if ((N % 8) || (K % 8 && mode != MODE_TN) || (mode == MODE_TN && (M % 8))) return LLMK_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
        return LLMK_ERR_SHAPE;
    const int g_num_sms = sm_count_current_device();
    if (g_num_sms <= 0) return LLMK_ERR_CUDA;
    Params p;
    p.M = M; p.N = N; p.K = K;
    const int pair_clusters = query_pair_clusters();
    p.pair = pair_clusters > 0 ? 1 : 0;
    p.group_m = 0;
    if (groups > 1) {
        // a tile must not straddle two groups, and a k-block must not run into the next group's rows
        if (M_group % (p.pair ? 2 * BM : BM)) return LLMK_ERR_SHAPE;
        if (mode != MODE_NT && (K % BK)) return LLMK_ERR_SHAPE;
        p.group_m = M_group;
    }
    p.tiles_m = ceil_div(M, p.pair ? 2 * BM : BM);
    p.tiles_n = ceil_div(N, BN);
    p.kb_total = ceil_div(K, BK);
    p.splits = 1;
    p.bias = static_cast<const bf16*>(bias);
    p.aux = static_cast<const bf16*>(aux);
    p.partial = nullptr;
    p.status = status;
    p.b_ready = ready.b_ready; p.a_ready = ready.a_ready;
    p.b_chunk = ready.b_chunk > 0 ? ready.b_chunk : 1;
    p.b_nflags = ready.b_nflags;
    p.m_rotate = 0;
    p.b_tick = ready.b_tick; p.a_rows = ready.a_rows > 0 ? ready.a_rows : 1; p.a_need = ready.a_need;
    p.ready_limit_ns = ready.limit_ns > 0 ? ready.limit_ns : (long long)LLMK_WAIT_LIMIT_NS;
    if ((p.b_ready != nullptr || p.a_ready != nullptr) && mode == MODE_TN) return LLMK_ERR_SHAPE;
    p.rope = ready.rope; p.rope_T = ready.rope_T; p.rope_cols = ready.rope_cols; p.rope_hs = ready.rope_hs;
    p.b_ready2 = ready.b_ready2;
    p.dbias = static_cast<bf16*>(ready.dbias);
    p.db_partial = nullptr;
    if (epi & EPI_DBIAS) {
        if (mode != MODE_TN || !p.pair || ready.dbias == nullptr || (epi & ~(EPI_DBIAS | EPI_ADD)) ||
            (reinterpret_cast<uintptr_t>(ready.dbias) & 15))
            return LLMK_ERR_SHAPE;
    }
    p.drow = ready.drow; p.drow_T = ready.drow_T; p.drow_NH = ready.drow_NH;
    if (epi & EPI_DROW) {
        if (epi != EPI_DROW || mode != MODE_NN || groups != 1 || ready.drow == nullptr || aux == nullptr || ready.drow_T <= 0 ||
            M % ready.drow_T || N != ready.drow_NH * 64)
            return LLMK_ERR_SHAPE;
    }
    if (epi & EPI_SWIGLU) {
        // N is the width of the accumulator tile space: 2 H columns (up | gate per 128 hidden units); outputs are [M, H]
        if (mode != MODE_NT || groups != 1 || !p.pair || ready.b2 == nullptr || ready.c3 == nullptr || C2 == nullptr || (N % 256) ||
            ((reinterpret_cast<uintptr_t>(ready.b2) | reinterpret_cast<uintptr_t>(ready.c3) | reinterpret_cast<uintptr_t>(C2)) & 15))
            return LLMK_ERR_SHAPE;
    }
    for (int i = 0; i < 8; i++) { p.sc_dst[i] = nullptr; p.sc_arrive[i] = nullptr; }
    p.sc_count = ready.sc_count;
    p.sc_cap = ready.sc_cap; p.sc_P = ready.sc_P; p.sc_Eloc = ready.sc_Eloc; p.sc_rank = ready.sc_rank;
    p.sc_off = ready.sc_off; p.sc_epoch = ready.sc_epoch;
    if (epi & EPI_SCATTER) {
        if (ready.sc_dst == nullptr || ready.sc_arrive == nullptr || ready.sc_count == nullptr || mode == MODE_TN || ready.sc_P <= 0 ||
            ready.sc_P > 8 || ready.sc_cap < 32 || ready.sc_Eloc <= 0 || M != ready.sc_Eloc * ready.sc_P * ready.sc_cap || (N % 8))
            return LLMK_ERR_SHAPE;
        for (int i = 0; i < ready.sc_P; i++) {
            p.sc_dst[i] = reinterpret_cast<void*>(ready.sc_dst[i]);
            p.sc_arrive[i] = reinterpret_cast<int*>(ready.sc_arrive[i]);
        }
    }
    if (epi & EPI_ROPE) {
        if (p.rope == nullptr || mode != MODE_NT || p.rope_T <= 0 || (p.rope_hs != 64 && p.rope_hs != 128) ||
            p.rope_cols % p.rope_hs || p.rope_cols > N || (reinterpret_cast<uintptr_t>(p.rope) & 15))
            return LLMK_ERR_SHAPE;
    }
    bool split_accumulate = false;
    const int with_dbias = epi & EPI_DBIAS;
    if (mode == MODE_TN && ((epi & ~EPI_DBIAS) == 0 || (epi & ~EPI_DBIAS) == EPI_ADD)) {
        const int workers = p.pair ? pair_clusters : g_num_sms;
        const int cap = max_ctas > 0 ? (p.pair ? (max_ctas / 2 > 0 ? max_ctas / 2 : 1) : max_ctas) : workers;
        int s = pick_splits(mode, M, N, K, cap < workers ? cap : workers, p.pair ? 2 * BM : BM);
        if (s > 1) {
            if (workspace == nullptr || workspace_bytes < (long)s * M * N * 4 + (with_dbias ? (long)s * p.tiles_n * M * 4 : 0)) return LLMK_ERR_WORKSPACE;
            p.splits = s;
            p.partial = static_cast<float*>(workspace);
            p.db_partial = p.partial + (size_t)s * M * N;   // behind the partials of C (s = the largest split count in use)
            split_accumulate = (epi & EPI_ADD) != 0;
            epi = EPI_PARTIAL | with_dbias;
        }
    }
    if (ready.rotate_rows > 0) p.m_rotate = (ready.rotate_rows / (p.pair ? 2 * BM : BM)) % p.tiles_m;
    p.kb_per_split = ceil_div(p.kb_total, p.splits);
    if ((long)p.kb_per_split * (p.splits - 1) >= p.kb_total) {  // avoid empty trailing splits
        p.splits = ceil_div(p.kb_total, p.kb_per_split);
    }

    CUtensorMap tmA, tmB, tmC, tmX;
    int rc;
    // grouped problems stack their operands along the outer (row) dimension of each matrix
    const uint64_t G = (uint64_t)groups;
    if (mode == MODE_TN) rc = make_tmap_2d(&tmA, A, M_group, G * K, M_group, 64, BK);   // A[G*K,M_g], box 64(m) x 64(k)
    else rc = make_tmap_2d(&tmA, A, K, M, K, BK, BM);                    // A[M,K], box 64(k) x 128(m)
    if (rc) return rc;
    const bool swi = (epi & EPI_SWIGLU) != 0;
    const uint64_t b_rows = swi ? (uint64_t)N / 2 : G * N, c_cols = swi ? (uint64_t)N / 2 : (uint64_t)N;
    if (mode == MODE_NT) rc = make_tmap_2d(&tmB, B, K, b_rows, K, BK, p.pair ? BN / 2 : BN);   // B[G*N,K], box 64(k) x 256(n); pair: 128(n) per CTA
    else rc = make_tmap_2d(&tmB, B, N, G * K, N, 64, BK);                // B[G*K,N], box 64(n) x 64(k)
    if (rc) return rc;
    rc = make_tmap_2d(&tmC, C, c_cols, M, c_cols, 64, 32);
    if (rc) return rc;
    tmX = tmC;
    ExtraMaps xm;
    xm.b2 = tmB;
    xm.y = tmC;
    if (swi) {
        if ((rc = make_tmap_2d(&xm.b2, ready.b2, K, b_rows, K, BK, BN / 2))) return rc;
        if ((rc = make_tmap_2d(&tmX, C2, c_cols, M, c_cols, 64, 32))) return rc;
        if ((rc = make_tmap_2d(&xm.y, ready.c3, c_cols, M, c_cols, 64, 32))) return rc;
    }
    if (epi & (EPI_GELU | EPI_DGELU | EPI_ADD | EPI_DROW)) {
        const void* x = (epi & EPI_GELU) ? C2 : aux;
        if (x == nullptr || (reinterpret_cast<uintptr_t>(x) & 15)) return LLMK_ERR_SHAPE;
        rc = make_tmap_2d(&tmX, x, N, M, N, 64, 32);
        if (rc) return rc;
    }

#define LLMK_GEMM_CASE(MODE_, EPI_) \
    if (mode == MODE_ && epi == (EPI_)) rc = launch<MODE_, EPI_>(tmA, tmB, tmC, tmX, xm, p, max_ctas, stream); else
    rc = LLMK_ERR_SHAPE;
    LLMK_GEMM_CASE(MODE_NT, 0)
    LLMK_GEMM_CASE(MODE_NT, EPI_BIAS)
    LLMK_GEMM_CASE(MODE_NT, EPI_BIAS | EPI_GELU)
    LLMK_GEMM_CASE(MODE_NT, EPI_ADD)
    LLMK_GEMM_CASE(MODE_NT, EPI_BIAS | EPI_ADD)
    LLMK_GEMM_CASE(MODE_NT, EPI_ROPE)
    LLMK_GEMM_CASE(MODE_NT, EPI_SWIGLU)
    LLMK_GEMM_CASE(MODE_NT, EPI_BIAS | EPI_SCATTER)
    LLMK_GEMM_CASE(MODE_NN, EPI_SCATTER)
    LLMK_GEMM_CASE(MODE_NN, 0)
    LLMK_GEMM_CASE(MODE_NN, EPI_DGELU)
    LLMK_GEMM_CASE(MODE_NN, EPI_ADD)
    LLMK_GEMM_CASE(MODE_NN, EPI_DROW)
    LLMK_GEMM_CASE(MODE_TN, 0)
    LLMK_GEMM_CASE(MODE_TN, EPI_ADD)
    LLMK_GEMM_CASE(MODE_TN, EPI_PARTIAL)
    LLMK_GEMM_CASE(MODE_TN, EPI_DBIAS)
    LLMK_GEMM_CASE(MODE_TN, EPI_ADD | EPI_DBIAS)
    LLMK_GEMM_CASE(MODE_TN, EPI_PARTIAL | EPI_DBIAS)
    { rc = LLMK_ERR_SHAPE; }
#undef LLMK_GEMM_CASE
    if (rc) return rc;
    if (epi & EPI_PARTIAL) {
        const size_t n = (size_t)M * N;
        splitk_reduce_kernel<<<ceil_div((long)(n / 8), 256), 256, 0, stream>>>(static_cast<bf16*>(C), p.partial, n, p.splits,
                                                                            split_accumulate ? 1 : 0, with_dbias ? p.dbias : nullptr,
                                                                            p.db_partial, M, p.splits * p.tiles_n);
        LLMK_LAUNCH_CHECK();
    }
    return LLMK_OK;
}

LLMK_API int llmk_gemm(int mode, int epi, const void* A, const void* B, void* C, void* C2, const void* bias,
                       const void* aux, int M, int N, int K, void* workspace, long workspace_bytes, int* status,
                       int max_ctas, void* stream_) {
    return gemm_impl(mode, epi, A, B, C, C2, bias, aux, M, N, K, 1, workspace, workspace_bytes, status, max_ctas, stream_);
}

// Weight gradient and bias gradient of a linear layer in one launch: C[M, N] (+)= A^T B and dbias[M] (+)= the column
// sums of A, where A = dout [K tokens, M output channels] and B = the layer's input [K, N]; `accumulate` adds to the
// old contents of both. The sums are taken from the A tiles in shared memory while the tensor core works on them
// (see Cfg::DB), in a fixed order. CTA-pair kernel only: LLMK_ERR_SHAPE otherwise (the caller then runs llmk_gemm and
// the stand-alone column-sum kernel). Same job as matmul_backward's dbias kernel plus its dweight GEMM
// (llmc/matmul.cuh:465-539, 1238-1338) without the extra pass over dout.
LLMK_API int llmk_gemm_tn_dbias(const void* A, const void* B, void* C, void* dbias, int accumulate, int M, int N, int K, void* workspace,
                                long workspace_bytes, int* status, int max_ctas, void* stream_) {
    Ready r;
    r.dbias = dbias;
    return gemm_impl(MODE_TN, EPI_DBIAS | (accumulate ? EPI_ADD : 0), A, B, C, nullptr, nullptr, accumulate ? C : nullptr, M, N, K, 1,
                     workspace, workspace_bytes, status, max_ctas, stream_, r);
}

// llmk_gemm_tn_dbias for `groups` stacked problems (the experts of a mixture-of-experts layer): A [G*K, M], B [G*K, N],
// C [G*M, N], dbias [G*M]; M a multiple of 256 and K of 64 as for llmk_gemm_grouped, else LLMK_ERR_SHAPE.
LLMK_API int llmk_gemm_grouped_tn_dbias(const void* A, const void* B, void* C, void* dbias, int accumulate, int M, int N, int K,
                                        int groups, void* workspace, long workspace_bytes, int* status, int max_ctas, void* stream_) {
    Ready r;
    r.dbias = dbias;
    return gemm_impl(MODE_TN, EPI_DBIAS | (accumulate ? EPI_ADD : 0), A, B, C, nullptr, nullptr, accumulate ? C : nullptr, M, N, K,
                     groups, workspace, workspace_bytes, status, max_ctas, stream_, r);
}

// Input gradient of the attention output projection with the D term of the attention backward in its epilogue:
// C [M, N] = A B (A = d(residual) [M, K], B = the projection weight [K, N]) is dO, and dvec[b][h][t] = sum over head h's
// 64 columns of dO * O for row b * T + t (O [M, N] = the attention output). Head size 64 only (one epilogue chunk is one
// head). Same job as the D pre-pass of the reference's attention backward (bwd_attend_prep_ker, llmc/tk/attention_h100.cuh:342-395)
// without reading dO back.
LLMK_API int llmk_gemm_nn_drow(const void* A, const void* B, void* C, const void* O, void* dvec, int M, int N, int K, int T, int NH,
                               int* status, int max_ctas, void* stream_) {
    Ready r;
    r.drow = static_cast<float*>(dvec);
    r.drow_T = T;
    r.drow_NH = NH;
    return gemm_impl(MODE_NN, EPI_DROW, A, B, C, nullptr, nullptr, O, M, N, K, 1, nullptr, 0, status, max_ctas, stream_, r);
}

// llmk_gemm whose B operand (a weight matrix, NT or NN) is still being filled by another kernel: `b_ready` holds one
// int per `b_chunk` consecutive elements of B, written (release) with `b_tick` once those elements are in place. The
// producer warp of every CTA acquire-polls the flags that cover a B tile before its first load of it, for at most
// `limit_ns` nanoseconds (then LLMK_ST_TIMEOUT_PEER in the status word and the kernel returns). This is the consumer
// half of the tile-granular parameter all-gather (job of llmc/zero.cuh:543-578 followed by matmul_forward).
LLMK_API int llmk_gemm_b_ready(int mode, int epi, const void* A, const void* B, void* C, void* C2, const void* bias,
                               const void* aux, int M, int N, int K, void* workspace, long workspace_bytes, int* status,
                               int max_ctas, const void* b_ready, long b_chunk, int b_tick, long limit_ns, void* stream_) {
    Ready r;
    r.b_ready = static_cast<const int*>(b_ready);
    r.b_chunk = b_chunk;
    r.b_tick = b_tick;
    r.limit_ns = limit_ns;
    if (b_ready != nullptr && b_chunk <= 0) return LLMK_ERR_SHAPE;
    if (b_ready != nullptr) r.b_nflags = (int)(((long long)N * K + b_chunk - 1) / b_chunk);   // B holds N * K elements in NT and NN
    return gemm_impl(mode, epi, A, B, C, C2, bias, aux, M, N, K, 1, workspace, workspace_bytes, status, max_ctas, stream_, r);
}

// llmk_gemm_grouped whose A rows are still arriving (the token dispatch of an expert-parallel mixture of experts):
// `a_ready` holds one int per `a_rows` consecutive rows of A (NT / NN), ready when >= `a_need`; the producer warp
// polls, for at most limit_ns, only the entries that cover the M tile it is about to load. The counterpart of the
// per-block release stores of llmk_moe_dispatch_signal (jobs of llmc/moe.cuh:121-237 + llmc/gemm_ext.cuh:132-158 +
// llmc/distributed_ext.cuh:28-41 without a barrier between them).
LLMK_API int llmk_gemm_grouped_a_ready(int mode, int epi, const void* A, const void* B, void* C, void* C2, const void* bias,
                                       const void* aux, int M, int N, int K, int groups, void* workspace, long workspace_bytes,
                                       int* status, int max_ctas, const void* a_ready, int a_rows, int a_need, long limit_ns,
                                       int rotate_rows, void* stream_) {
    Ready r;
    r.rotate_rows = rotate_rows;
    r.a_ready = static_cast<const int*>(a_ready);
    r.a_rows = a_rows;
    r.a_need = a_need;
    r.limit_ns = limit_ns;
    if (a_ready != nullptr && a_rows <= 0) return LLMK_ERR_SHAPE;
    return gemm_impl(mode, epi, A, B, C, C2, bias, aux, M, N, K, groups, workspace, workspace_bytes, status, max_ctas, stream_, r);
}

// The second GEMM of a mixture-of-experts layer with the all-to-all back fused into its epilogue: mode NT with bias
// (forward: expert outputs) or NN without (backward: input gradients), `groups` local experts of `P * cap` rows each.
// Nothing is written locally: the epilogue stores every row into the `back` buffer of the rank that sent the token
// (dst_ptrs[src]) and publishes each (source rank, local expert) block in that rank's arrival table when its last
// piece has been stored (see Params::sc_*). `count`: groups * P zeroed ints of local scratch. A local C of the same
// shape must still be passed for the tensor map (it is not written). Jobs of the reference's unpermute +
// all-to-all (llmc/moe.cuh:180-237, llmc/distributed_ext.cuh:28-41) inside grouped_gemm (llmc/gemm_ext.cuh:132-158).
LLMK_API int llmk_gemm_grouped_scatter(int mode, int with_bias, const void* A, const void* B, void* C_shape_only, const void* bias,
                                       int M, int N, int K, int groups, int* status, int max_ctas, const long long* dst_ptrs,
                                       const long long* arrive_ptrs, int arrive_off, void* count, int cap, int P, int my_rank,
                                       int epoch, void* stream_) {
    Ready r;
    r.rotate_rows = ((my_rank + 1) % P) * cap;   // rank r starts with the rows of rank r + 1: no two ranks store to the same peer
    r.sc_dst = dst_ptrs;
    r.sc_arrive = arrive_ptrs;
    r.sc_count = static_cast<int*>(count);
    r.sc_cap = cap; r.sc_P = P; r.sc_Eloc = groups; r.sc_rank = my_rank; r.sc_off = arrive_off; r.sc_epoch = epoch;
    if (M != P * cap) return LLMK_ERR_SHAPE;
    const int epi = EPI_SCATTER | (with_bias ? EPI_BIAS : 0);
    if ((mode == MODE_NT) != (with_bias != 0)) return LLMK_ERR_SHAPE;
    return gemm_impl(mode, epi, A, B, C_shape_only, nullptr, bias, nullptr, M, N, K, groups, nullptr, 0, status, max_ctas, stream_, r);
}

// Llama MLP, first half, in one launch: up = A Wup^T, gate = A Wgate^T and act = gate * sigmoid(gate) * up, with the
// SwiGLU in the epilogue (a CTA pair's accumulator holds 128 hidden units of `up` beside the same units of `gate`: the
// leader loads the up rows, its peer the gate rows). All three [M, H] tensors are written (the backward needs up and
// gate). H must be a multiple of 128 and the CTA-pair kernel available, else LLMK_ERR_SHAPE (the caller then runs
// two GEMMs and the stand-alone SwiGLU kernel). Optional readiness flags for both weights as in llmk_gemm_b_ready.
// Same job as matmul + swiglu_forward of the reference (llmc/swiglu.cuh:27-61) without the extra pass over up / gate.
LLMK_API int llmk_gemm_swiglu(const void* A, const void* Wup, const void* Wgate, void* act, void* up, void* gate, int M, int H, int K,
                              int* status, int max_ctas, const void* up_ready, const void* gate_ready, long b_chunk, int b_tick,
                              long limit_ns, void* stream_) {
    if (H % 128) return LLMK_ERR_SHAPE;
    Ready r;
    r.b_ready = static_cast<const int*>(up_ready);
    r.b_ready2 = static_cast<const int*>(gate_ready);
    r.b_chunk = b_chunk > 0 ? b_chunk : 1;
    r.b_tick = b_tick;
    r.limit_ns = limit_ns;
    if (up_ready != nullptr) r.b_nflags = (int)(((long long)H * K + r.b_chunk - 1) / r.b_chunk);   // per matrix (up and gate alike)
    r.b2 = Wgate;
    r.c3 = gate;
    return gemm_impl(MODE_NT, EPI_SWIGLU, A, Wup, act, up, nullptr, nullptr, M, 2 * H, K, 1, nullptr, 0, status, max_ctas, stream_, r);
}

// QKV projection with RoPE in the epilogue: C = A B^T where C is a packed [tokens, (NH + 2 NKVH) * HS] tensor; the
// q and k heads (the first `rope_cols` columns) are rotated by the (cos, sin) table `rope` [T, HS/2] (interleaved
// pairs) before they are rounded to bf16, v passes through. Row r is token r % T. Optional `b_ready` as in
// llmk_gemm_b_ready. Same job as the in-tile rotation of the reference's GQA attention (llmc/tk/attention_gqa_h100.cuh:66-83),
// moved to where the values are still in fp32 registers.
LLMK_API int llmk_gemm_qkv_rope(const void* A, const void* B, void* C, int M, int N, int K, const void* rope, int T, int rope_cols,
                                int HS, int* status, int max_ctas, const void* b_ready, long b_chunk, int b_tick, long limit_ns,
                                void* stream_) {
    Ready r;
    r.b_ready = static_cast<const int*>(b_ready);
    r.b_chunk = b_chunk > 0 ? b_chunk : 1;
    r.b_tick = b_tick;
    r.limit_ns = limit_ns;
    if (b_ready != nullptr) r.b_nflags = (int)(((long long)N * K + r.b_chunk - 1) / r.b_chunk);
    r.rope = static_cast<const float2*>(rope);
    r.rope_T = T; r.rope_cols = rope_cols; r.rope_hs = HS;
    return gemm_impl(MODE_NT, EPI_ROPE, A, B, C, nullptr, nullptr, nullptr, M, N, K, 1, nullptr, 0, status, max_ctas, stream_, r);
}

// `groups` independent problems of the same shape in ONE persistent launch (the experts of a mixture-of-experts
// layer; same job as grouped_gemm of the reference, llmc/gemm_ext.cuh:132-158, for equal row counts). M, N, K are the
// dimensions of one group; operands are stacked along their rows: NT: A [G*M,K], B [G*N,K], bias [G*N], C [G*M,N];
// NN: A [G*M,K], B [G*K,N]; TN: A [G*K,M], B [G*K,N], C [G*M,N] (K = tokens of one group). M must be a multiple of the
// tile height (256 with CTA pairs, else 128) and, for NN / TN, K a multiple of 64; otherwise LLMK_ERR_SHAPE is
// returned and the caller launches the groups one by one. Workspace for TN: llmk_gemm_workspace_bytes(mode, G*M, N, K).
LLMK_API int llmk_gemm_grouped(int mode, int epi, const void* A, const void* B, void* C, void* C2, const void* bias,
                               const void* aux, int M, int N, int K, int groups, void* workspace, long workspace_bytes,
                               int* status, int max_ctas, void* stream_) {
    return gemm_impl(mode, epi, A, B, C, C2, bias, aux, M, N, K, groups, workspace, workspace_bytes, status, max_ctas, stream_);
}
