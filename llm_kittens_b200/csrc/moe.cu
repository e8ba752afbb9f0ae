// Mixture-of-experts routing, dispatch and combine kernels (the expert MLPs themselves are the
// tcgen05 GEMMs of gemm_tcgen05.cu running on each expert's row block).
//
// Semantics come from the reference's un-wired primitives: softmax -> top-K -> renormalise
// (topk_route, llmc/moe.cuh:40-100), capacity-factor dropping (llmc/moe.cuh:312-335), permute /
// unpermute into per-expert row blocks (llmc/moe.cuh:121-237), the equal-split all-to-all
// (llmc/distributed_ext.cuh:27-48) and the load-balance loss E * sum_e density_e^2
// (llmc/losses.cuh:522-559). Differences by design:
//   * slot assignment is a deterministic prefix sum in (token, k) order instead of first-atomic-wins;
//   * dispatch and combine ARE the all-to-all: a row is stored straight into the receive buffer of
//     the rank that owns the expert (or read from / written to the local one when that rank is this
//     rank) through a table of peer pointers, so there is no packed send buffer and no collective
//     call; padded capacity slots are zero-filled by the sender so they add nothing to any gradient;
//   * every token row of the combine is produced by exactly one warp (no atomic adds);
//   * there is no layer-wide barrier between the stages. The kernel that finishes a block of rows publishes it with a
//     release store into the consumer rank's arrival table, and the consumer waits inside the kernel that needs the
//     rows: the grouped expert GEMM's producer warp polls only the entries that cover the M tile it is about to load
//     (rows of one source rank), the combine kernel polls the owners' "returned" entries before its first load.
//     An entry holds the number of the exchange (a counter that only grows), so nothing is ever reset.
//
// Buffer layouts (C channels, cap = capacity per (source rank, expert), Eloc experts per rank):
//   owner side   recv[e_local][src][cap][C]   rows routed to local expert e_local by rank src
//   source side  back[e][cap][C]              expert outputs (or input gradients) returned to this rank
#include "common.cuh"

namespace llmk {
namespace moe {

constexpr int MAXP = 8;
constexpr int MAXE = 16;
constexpr int MAXK = 4;

struct Peers {
    void* p[MAXP];
};

__device__ __forceinline__ void st_release_sys(int* ptr, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* ptr) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// The CTA that finishes a kernel's work last (an arrival counter in local memory, left at zero again) returns true
// in thread 0, after a system-scope fence that covers the stores of every CTA (each fenced before it arrived).
__device__ __forceinline__ bool last_cta_done(int* counter, int total) {
    __syncthreads();
    if (threadIdx.x != 0) return false;
    __threadfence_system();
    if (atomicAdd(counter, 1) != total - 1) return false;
    *counter = 0;
    __threadfence_system();
    return true;
}

// Threads 0..n-1 of the block poll flags[0..n) until each is >= need, for at most limit_ns; false (to every thread)
// when the time ran out: LLMK_ST_TIMEOUT_PEER goes to the status word and the caller skips its work.
__device__ __forceinline__ bool wait_entries_block(const int* flags, int n, int need, long long limit_ns, int* status, int tag) {
    __shared__ int sh_ok;
    // a failure already recorded (by an earlier kernel or block) ends this wait at once
    if (threadIdx.x == 0) sh_ok = (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) ? 0 : 1;
    __syncthreads();
    if (sh_ok != 0 && (int)threadIdx.x < n) {
        const unsigned long long t0 = now_ns();
        unsigned int spins = 0;
        while (ld_acquire_sys(flags + threadIdx.x) < need) {
            if ((++spins & 31u) == 0 && (long long)(now_ns() - t0) > limit_ns) {
                sh_ok = 0;
                if (status != nullptr && atomicCAS(status, 0, LLMK_ST_TIMEOUT_PEER) == 0) {
                    status[1] = tag;
                    status[2] = (int)blockIdx.x;
                    status[3] = (int)threadIdx.x;
                }
                break;
            }
            __nanosleep(64);
        }
    }
    __syncthreads();
    return sh_ok != 0;
}

// ------------------------------------------------------------------ router
// One warp per token: logits = x . Wr^T (fp32), softmax over E, top-K (ties -> lower expert index),
// weights renormalised to sum 1.
__global__ void __launch_bounds__(256)
router_fwd_kernel(float* __restrict__ probs, int* __restrict__ top_idx, float* __restrict__ top_w, const bf16* __restrict__ x,
                  const bf16* __restrict__ wr, int N, int C, int E, int K) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    bf16* wr_s = reinterpret_cast<bf16*>(smem_raw);  // [E][C]
    for (int i = threadIdx.x * 8; i < E * C; i += blockDim.x * 8) st128(wr_s + i, ld128(wr + i));
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= N) return;
    float acc[MAXE];
#pragma unroll
    for (int e = 0; e < MAXE; e++) acc[e] = 0.f;
    for (int v = lane; v < C / 8; v += 32) {
        float xf[8];
        unpack8(ld128_stream(x + (size_t)row * C + v * 8), xf);
#pragma unroll
        for (int e = 0; e < MAXE; e++) {
            if (e < E) {
                float wf[8];
                unpack8(ld128(wr_s + (size_t)e * C + v * 8), wf);
#pragma unroll
                for (int j = 0; j < 8; j++) acc[e] += xf[j] * wf[j];
            }
        }
    }
#pragma unroll
    for (int e = 0; e < MAXE; e++)
        if (e < E) acc[e] = warp_sum(acc[e]);
    if (lane == 0) {
        float mx = -INFINITY;
        for (int e = 0; e < E; e++) mx = fmaxf(mx, acc[e]);
        float sum = 0.f, p[MAXE];
        for (int e = 0; e < E; e++) {
            p[e] = __expf(acc[e] - mx);
            sum += p[e];
        }
        for (int e = 0; e < E; e++) {
            p[e] /= sum;
            probs[(size_t)row * E + e] = p[e];
        }
        unsigned taken = 0;
        float wsum = 0.f, w[MAXK];
        int idx[MAXK];
        for (int k = 0; k < K; k++) {
            int best = -1;
            float bv = -1.f;
            for (int e = 0; e < E; e++)
                if (!(taken & (1u << e)) && p[e] > bv) {
                    bv = p[e];
                    best = e;
                }
            taken |= 1u << best;
            idx[k] = best;
            w[k] = bv;
            wsum += bv;
        }
        for (int k = 0; k < K; k++) {
            top_idx[(size_t)row * K + k] = idx[k];
            top_w[(size_t)row * K + k] = w[k] / wsum;
        }
    }
}

// ------------------------------------------------------------------ slot assignment
// One block per expert: slot[i] = number of earlier assignments (i = token*K + k order) to this expert,
// or -1 beyond `cap`. counts[e] = min(total, cap). Deterministic.
__global__ void __launch_bounds__(1024)
assign_slots_kernel(int* __restrict__ slot, int* __restrict__ counts, const int* __restrict__ top_idx, int NK, int cap) {
    __shared__ int warp_tot[32];
    __shared__ int running;
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) running = 0;
    __syncthreads();
    for (int base = 0; base < NK; base += 1024) {
        const int i = base + threadIdx.x;
        const int flag = (i < NK && top_idx[i] == e) ? 1 : 0;
        int incl = flag;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        int before = running;
        for (int w = 0; w < warp; w++) before += warp_tot[w];
        if (flag) {
            const int s = before + incl - 1;
            slot[i] = s < cap ? s : -1;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int tot = 0;
            for (int w = 0; w < 32; w++) tot += warp_tot[w];
            running += tot;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[e] = running < cap ? running : cap;
}

// ------------------------------------------------------------------ dispatch (all-to-all out)
// One warp per (token, k): row x[token] * scale -> recv buffer of the owner of expert e at slot s.
// `scale_by_weight`: 0 copies the row (forward), 1 multiplies by the routing weight (backward: dY = w * dout).
__global__ void __launch_bounds__(256)
dispatch_kernel(Peers recv, const bf16* __restrict__ x, const int* __restrict__ top_idx, const int* __restrict__ slot,
                const float* __restrict__ top_w, int N, int K, int C, int cap, int Eloc, int my_rank, int P, int scale_by_weight) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t a = (size_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (a >= (size_t)N * K) return;
    const int s = slot[a];
    if (s < 0) return;
    const int e = top_idx[a];
    const size_t t = a / K;
    const int owner = e / Eloc, el = e % Eloc;
    bf16* dst = static_cast<bf16*>(recv.p[owner]) + ((((size_t)el * P + my_rank) * cap) + s) * C;
    const bf16* src = x + t * C;
    const float w = scale_by_weight ? top_w[a] : 1.0f;
    for (int v = lane; v < C / 8; v += 32) {
        bf16x8 r = ld128(src + v * 8);
        if (scale_by_weight) {
            float f[8];
            unpack8(r, f);
#pragma unroll
            for (int j = 0; j < 8; j++) f[j] *= w;
            r = pack8(f);
        }
        st128(dst + v * 8, r);
    }
}
// Zero the unused slots [counts[e], cap) of this rank's block in every expert's receive buffer.
// `arrive` (optional): the owners' arrival tables. This kernel runs after dispatch_kernel on the same stream, so when
// its last CTA is done every row of this rank has been stored: that CTA release-stores `epoch` into entry
// [e_local * P + my_rank] of the owner of every expert, which is entry (first row of the block) / cap of the
// owner's receive buffer, the index the expert GEMM derives from the rows of a tile.
__global__ void __launch_bounds__(256)
zero_pad_kernel(Peers recv, const int* __restrict__ counts, int E, int C, int cap, int Eloc, int my_rank, int P, Peers arrive,
                int arrive_off, int* done_counter, int epoch) {
    const int e = blockIdx.y;
    const int owner = e / Eloc, el = e % Eloc;
    const int first = counts[e];
    bf16* base = static_cast<bf16*>(recv.p[owner]) + (((size_t)el * P + my_rank) * cap) * C;
    const size_t begin = (size_t)first * C, end = (size_t)cap * C;
    bf16x8 z;
#pragma unroll
    for (int i = 0; i < 4; i++) z.v[i] = __floats2bfloat162_rn(0.f, 0.f);
    for (size_t i = begin + ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < end; i += (size_t)gridDim.x * blockDim.x * 8)
        st128(base + i, z);
    if (done_counter != nullptr && last_cta_done(done_counter, gridDim.x * gridDim.y)) {
        for (int ee = 0; ee < E; ee++)
            st_release_sys(static_cast<int*>(arrive.p[ee / Eloc]) + arrive_off + (ee % Eloc) * P + my_rank, epoch);
    }
}

// ------------------------------------------------------------------ dispatch as a PULL
// Source side: the inverse of the slot assignment, inv_tok[e * cap + s] = token whose assignment got slot s of expert
// e (-1: the slot is unused) and inv_w = its routing weight; both live in peer-readable memory, as does a copy of the
// token rows. Owner side (dispatch_pull_kernel): one warp per row of recv[e_local][src][slot] reads the token index
// from rank src's map and copies that token's row out of rank src's memory with 128-bit peer loads (zeros for unused
// slots, times the routing weight in the backward pass); loads cross NVLink faster than the stores of the push
// variant, nothing is packed or padded on the way, and every (source, expert) block is published in the LOCAL arrival
// table by the block that completes it, which is what the expert GEMM's producer warp polls per M tile.
__global__ void __launch_bounds__(256)
inverse_map_kernel(int* __restrict__ inv_tok, float* __restrict__ inv_w, const int* __restrict__ top_idx, const int* __restrict__ slot,
                   const float* __restrict__ top_w, int NK, int K, int cap) {
    const int a = blockIdx.x * blockDim.x + threadIdx.x;
    if (a >= NK) return;
    const int s = slot[a];
    if (s < 0) return;
    const int e = top_idx[a];
    inv_tok[(size_t)e * cap + s] = a / K;
    inv_w[(size_t)e * cap + s] = top_w[a];
}

struct PullSrc {
    const bf16* x[MAXP];       // the ranks' token rows [N, C]
    const int* inv_tok[MAXP];  // the ranks' inverse maps [E * cap]
    const float* inv_w[MAXP];
};

// grid = (ceil(cap / 8), P, Eloc), 8 warps per block: warp w of block x copies row x * 8 + w of block (el, src).
// `ready` = this rank's arrival entries: [E + src] is written by rank src when its rows and map are in place (waited
// for here, bounded), [el * P + src] is written here when the block is complete.
__global__ void __launch_bounds__(256)
dispatch_pull_kernel(bf16* __restrict__ recv, PullSrc src_tab, int C, int cap, int E, int Eloc, int my_rank, int P, int scale_by_weight,
                     int* __restrict__ ready, int* __restrict__ done_counters, int epoch, long long limit_ns, int* status) {
    const int src = blockIdx.y, el = blockIdx.z;
    __shared__ int sh_ok;
    if (threadIdx.x == 0) {
        sh_ok = (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) ? 0 : 1;
        if (sh_ok) {
            const unsigned long long t0 = now_ns();
            unsigned int spins = 0;
            while (ld_acquire_sys(ready + E + src) < epoch) {
                if ((++spins & 31u) == 0 && (long long)(now_ns() - t0) > limit_ns) {
                    sh_ok = 0;
                    if (status != nullptr && atomicCAS(status, 0, LLMK_ST_TIMEOUT_PEER) == 0) {
                        status[1] = 320;
                        status[2] = src;
                        status[3] = el;
                    }
                    break;
                }
                __nanosleep(64);
            }
        }
    }
    __syncthreads();
    if (!sh_ok) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s = blockIdx.x * 8 + warp;
    if (s < cap) {
        const int e = my_rank * Eloc + el;
        const int t = src_tab.inv_tok[src][(size_t)e * cap + s];
        bf16* dst = recv + (((size_t)el * P + src) * cap + s) * C;
        if (t < 0) {
            bf16x8 z;
#pragma unroll
            for (int i = 0; i < 4; i++) z.v[i] = __floats2bfloat162_rn(0.f, 0.f);
            for (int v = lane; v < C / 8; v += 32) st128(dst + v * 8, z);
        } else {
            const bf16* from = src_tab.x[src] + (size_t)t * C;
            const float w = scale_by_weight ? src_tab.inv_w[src][(size_t)e * cap + s] : 1.0f;
            for (int v = lane; v < C / 8; v += 32) {
                bf16x8 r = ld128_stream(from + v * 8);
                if (scale_by_weight) {
                    float f[8];
                    unpack8(r, f);
#pragma unroll
                    for (int j = 0; j < 8; j++) f[j] *= w;
                    r = pack8(f);
                }
                st128(dst + v * 8, r);
            }
        }
    }
    if (last_cta_done(done_counters + el * P + src, gridDim.x)) st_release_sys(ready + el * P + src, epoch);
}

// ------------------------------------------------------------------ return (all-to-all back)
// Owner side: copy the block of rows that rank `src` sent to local expert `el` back into that rank's
// `back[e][cap][C]` buffer. grid = (chunks, P, Eloc).
// `arrive` (optional): the source ranks' arrival tables; the CTA that finishes the block of (src, el) last
// release-stores `epoch` into entry [arrive_off + e] of rank src (e = this rank's global expert index).
__global__ void __launch_bounds__(256)
return_kernel(Peers back, const bf16* __restrict__ y, int C, int cap, int Eloc, int my_rank, int P, Peers arrive, int arrive_off,
              int* done_counters, int epoch) {
    const int src = blockIdx.y, el = blockIdx.z;
    const int e = my_rank * Eloc + el;
    const bf16* from = y + (((size_t)el * P + src) * cap) * C;
    bf16* to = static_cast<bf16*>(back.p[src]) + ((size_t)e * cap) * C;
    const size_t n = (size_t)cap * C;
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += (size_t)gridDim.x * blockDim.x * 8)
        st128(to + i, ld128(from + i));
    if (done_counters != nullptr && last_cta_done(done_counters + el * P + src, gridDim.x))
        st_release_sys(static_cast<int*>(arrive.p[src]) + arrive_off + e, epoch);
}

// ------------------------------------------------------------------ combine
// out[t] = base[t] + sum_k w[t,k] * back[e(t,k)][slot(t,k)]   (dropped assignments contribute 0).
// With `weights == nullptr` the rows are summed unweighted (input-gradient gather in backward).
// `returned` (optional): this rank's arrival entries of the E experts; every block waits (bounded) until each holds
// `epoch`, i.e. until every owner has stored the rows of this rank into `back`.
__global__ void __launch_bounds__(256)
combine_kernel(bf16* __restrict__ out, const bf16* __restrict__ base, const bf16* __restrict__ back, const int* __restrict__ top_idx,
               const int* __restrict__ slot, const float* __restrict__ weights, int N, int K, int C, int cap,
               const int* __restrict__ returned, int E, int epoch, long long limit_ns, int* status) {
    if (returned != nullptr && !wait_entries_block(returned, E, epoch, limit_ns, status, 300)) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t t = (size_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= (size_t)N) return;
    for (int v = lane; v < C / 8; v += 32) {
        float acc[8];
        if (base != nullptr) {
            unpack8(ld128(base + t * C + v * 8), acc);
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) acc[j] = 0.f;
        }
        for (int k = 0; k < K; k++) {
            const int s = slot[t * K + k];
            if (s < 0) continue;
            const int e = top_idx[t * K + k];
            const float w = weights ? weights[t * K + k] : 1.0f;
            float f[8];
            unpack8(ld128(back + (((size_t)e * cap) + s) * C + v * 8), f);
#pragma unroll
            for (int j = 0; j < 8; j++) acc[j] += w * f[j];
        }
        st128(out + t * C + v * 8, pack8(acc));
    }
}

// The way back as a PULL, fused with the combine: out[t] = base[t] + sum_k w[t,k] * y(e(t,k), slot(t,k)), where the
// row y lives in the memory of the rank that owns expert e: y_ptrs[owner] + ((e_local * P + my_rank) * cap + slot) * C
// (the owner's local expert-output buffer, laid out [e_local][source rank][slot]). Rows are fetched with 128-bit peer
// loads by the warp that combines the token; only rows that are really used cross NVLink (no capacity padding), and
// the owners' expert GEMMs keep their plain local epilogue. `returned` / `epoch`: as in combine_kernel, every block
// first waits until all E owners have published their outputs. `save` (optional, [E * cap, C] local): the fetched
// rows are also kept locally at [e][slot], where the backward pass finds them for the routing-weight gradient.
__global__ void __launch_bounds__(256)
combine_pull_kernel(bf16* __restrict__ out, const bf16* __restrict__ base, Peers y_ptrs, bf16* __restrict__ save,
                    const int* __restrict__ top_idx, const int* __restrict__ slot, const float* __restrict__ weights, int N, int K,
                    int C, int cap, int Eloc, int my_rank, int P, const int* __restrict__ returned, int E, int epoch,
                    long long limit_ns, int* status) {
    if (returned != nullptr && !wait_entries_block(returned, E, epoch, limit_ns, status, 310)) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t t = (size_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= (size_t)N) return;
    const bf16* rows[MAXK];
    bf16* keep[MAXK];
    float wk[MAXK];
    int nk = 0;
    for (int k = 0; k < K; k++) {
        const int s = slot[t * K + k];
        if (s < 0) continue;
        const int e = top_idx[t * K + k];
        const int owner = e / Eloc, el = e % Eloc;
        rows[nk] = static_cast<const bf16*>(y_ptrs.p[owner]) + (((size_t)el * P + my_rank) * cap + s) * C;
        keep[nk] = save != nullptr ? save + ((size_t)e * cap + s) * C : nullptr;
        wk[nk] = weights ? weights[t * K + k] : 1.0f;
        nk++;
    }
    for (int v = lane; v < C / 8; v += 32) {
        float acc[8];
        if (base != nullptr) {
            unpack8(ld128(base + t * C + v * 8), acc);
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) acc[j] = 0.f;
        }
        bf16x8 r[MAXK];
#pragma unroll
        for (int k = 0; k < MAXK; k++)
            if (k < nk) r[k] = ld128_stream(rows[k] + v * 8);      // all of a token's rows in flight before the first is used
#pragma unroll
        for (int k = 0; k < MAXK; k++) {
            if (k < nk) {
                float f[8];
                unpack8(r[k], f);
#pragma unroll
                for (int j = 0; j < 8; j++) acc[j] += wk[k] * f[j];
                if (keep[k] != nullptr) st128(keep[k] + v * 8, r[k]);
            }
        }
        st128(out + t * C + v * 8, pack8(acc));
    }
}

// Owner side of the pull: once everything queued before this launch has finished (the second expert GEMM wrote its
// outputs locally), tell every source rank that the outputs of this rank's experts can be fetched: entry
// [arrive_off + my_rank * Eloc + el] of every rank's arrival table gets `epoch` (release at system scope).
__global__ void publish_kernel(Peers arrive, int arrive_off, int Eloc, int my_rank, int P, int epoch) {
    const int r = threadIdx.x / Eloc, el = threadIdx.x % Eloc;
    if (r < P) {
        __threadfence_system();
        st_release_sys(static_cast<int*>(arrive.p[r]) + arrive_off + my_rank * Eloc + el, epoch);
    }
}

// dw[t,k] = dot(dout[t], back[e][slot])  (gradient of the combine with respect to the routing weight)
__global__ void __launch_bounds__(256)
combine_dweight_kernel(float* __restrict__ dw, const bf16* __restrict__ dout, const bf16* __restrict__ back,
                       const int* __restrict__ top_idx, const int* __restrict__ slot, int N, int K, int C, int cap) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t a = (size_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (a >= (size_t)N * K) return;
    const int s = slot[a];
    float acc = 0.f;
    if (s >= 0) {
        const int e = top_idx[a];
        const size_t t = a / K;
        for (int v = lane; v < C / 8; v += 32) {
            float d[8], f[8];
            unpack8(ld128(dout + t * C + v * 8), d);
            unpack8(ld128(back + (((size_t)e * cap) + s) * C + v * 8), f);
#pragma unroll
            for (int j = 0; j < 8; j++) acc += d[j] * f[j];
        }
    }
    acc = warp_sum(acc);
    if (lane == 0) dw[a] = acc;
}

// ------------------------------------------------------------------ load-balance statistics + router backward
// density[e] = mean_t probs[t,e]  (one block, fixed order)
__global__ void __launch_bounds__(1024)
density_kernel(float* __restrict__ density, float* __restrict__ aux_loss, const float* __restrict__ probs, int N, int E,
               float coef, int accumulate) {
    __shared__ float sh[32];
    __shared__ float dens[MAXE];
    for (int e = 0; e < E; e++) {
        float s = 0.f;
        for (int t = threadIdx.x; t < N; t += blockDim.x) s += probs[(size_t)t * E + e];
        s = block_sum(s, sh);
        if (threadIdx.x == 0) dens[e] = s / (float)N;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        float l = 0.f;
        for (int e = 0; e < E; e++) {
            density[e] = dens[e];
            l += dens[e] * dens[e];
        }
        l *= (float)E * coef;
        aux_loss[0] = accumulate ? aux_loss[0] + l : l;
    }
}
// dlogits[t,e] (bf16, [N, Epad]) from dw[t,k] (gradient w.r.t. renormalised top-k weights) and the
// load-balance term d(aux)/dp[t,e] = coef * E * 2 * density[e] / N * loss_scale.
__global__ void router_bwd_kernel(bf16* __restrict__ dlogits, const float* __restrict__ probs, const int* __restrict__ top_idx,
                                  const float* __restrict__ top_w, const float* __restrict__ dw, const int* __restrict__ slot,
                                  const float* __restrict__ density, int N, int E, int Epad, int K, float aux_scale) {
    const size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (size_t)N) return;
    float p[MAXE], dp[MAXE];
    for (int e = 0; e < E; e++) {
        p[e] = probs[t * E + e];
        dp[e] = aux_scale * density[e];
    }
    float S = 0.f, dot = 0.f;
    for (int k = 0; k < K; k++) {
        S += p[top_idx[t * K + k]];
        const float g = slot[t * K + k] >= 0 ? dw[t * K + k] : 0.f;
        dot += g * top_w[t * K + k];
    }
    for (int k = 0; k < K; k++) {
        const float g = slot[t * K + k] >= 0 ? dw[t * K + k] : 0.f;
        dp[top_idx[t * K + k]] += (g - dot) / S;
    }
    float pd = 0.f;
    for (int e = 0; e < E; e++) pd += dp[e] * p[e];
    for (int e = 0; e < Epad; e++)
        dlogits[t * Epad + e] = __float2bfloat16_rn(e < E ? p[e] * (dp[e] - pd) : 0.f);
}

static inline Peers make_peers(const long long* ptrs, int P) {
    Peers q;
    for (int i = 0; i < MAXP; i++) q.p[i] = i < P ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
    return q;
}

}  // namespace moe
}  // namespace llmk

using namespace llmk;
using namespace llmk::moe;

LLMK_API int llmk_moe_router_fwd(void* probs, void* top_idx, void* top_w, const void* x, const void* wr, int N, int C, int E, int K,
                                 void* stream) {
    if (E > MAXE || K > MAXK || K > E || C % 8 || (long)E * C * 2 > 200 * 1024) return LLMK_ERR_SHAPE;
    const int smem = E * C * 2;
    static PerDeviceOnce once_configured;
    if (once_configured.first()) {
        LLMK_CUDA_TRY(cudaFuncSetAttribute(router_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    }
    router_fwd_kernel<<<ceil_div(N, 8), 256, smem, (cudaStream_t)stream>>>((float*)probs, (int*)top_idx, (float*)top_w,
                                                                          (const bf16*)x, (const bf16*)wr, N, C, E, K);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_moe_assign_slots(void* slot, void* counts, const void* top_idx, int N, int K, int E, int cap, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    LLMK_CUDA_TRY(cudaMemsetAsync(slot, 0xff, (size_t)N * K * 4, st));
    assign_slots_kernel<<<E, 1024, 0, st>>>((int*)slot, (int*)counts, (const int*)top_idx, N * K, cap);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
// recv_ptrs: host array of P pointers to the owners' receive buffers.
LLMK_API int llmk_moe_dispatch(const long long* recv_ptrs, const void* x, const void* top_idx, const void* slot, const void* top_w,
                               const void* counts, int N, int K, int C, int E, int cap, int my_rank, int P, int scale_by_weight,
                               void* stream) {
    if (P > MAXP || E % P || C % 8) return LLMK_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    const Peers recv = make_peers(recv_ptrs, P);
    const int Eloc = E / P;
    dispatch_kernel<<<ceil_div((long)N * K, 8), 256, 0, st>>>(recv, (const bf16*)x, (const int*)top_idx, (const int*)slot,
                                                             (const float*)top_w, N, K, C, cap, Eloc, my_rank, P, scale_by_weight);
    LLMK_LAUNCH_CHECK();
    zero_pad_kernel<<<dim3(32, E), 256, 0, st>>>(recv, (const int*)counts, E, C, cap, Eloc, my_rank, P, recv, 0, nullptr, 0);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
// Dispatch that publishes its completion: `arrive_ptrs` = the P ranks' arrival tables (int), `arrive_off` the first
// entry of this exchange in them, `done_counter` one zeroed int of local scratch, `epoch` the number of the exchange.
LLMK_API int llmk_moe_dispatch_signal(const long long* recv_ptrs, const void* x, const void* top_idx, const void* slot,
                                      const void* top_w, const void* counts, int N, int K, int C, int E, int cap, int my_rank, int P,
                                      int scale_by_weight, const long long* arrive_ptrs, int arrive_off, void* done_counter,
                                      int epoch, void* stream) {
    if (P > MAXP || E % P || C % 8 || arrive_ptrs == nullptr || done_counter == nullptr) return LLMK_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    const Peers recv = make_peers(recv_ptrs, P);
    const int Eloc = E / P;
    dispatch_kernel<<<ceil_div((long)N * K, 8), 256, 0, st>>>(recv, (const bf16*)x, (const int*)top_idx, (const int*)slot,
                                                             (const float*)top_w, N, K, C, cap, Eloc, my_rank, P, scale_by_weight);
    LLMK_LAUNCH_CHECK();
    zero_pad_kernel<<<dim3(32, E), 256, 0, st>>>(recv, (const int*)counts, E, C, cap, Eloc, my_rank, P, make_peers(arrive_ptrs, P),
                                                 arrive_off, (int*)done_counter, epoch);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
// Source side of the pull-style dispatch (forward only: the backward pass reuses the maps): inverse slot maps of this
// rank's assignments. inv_tok / inv_w: [E * cap] in peer-readable memory.
LLMK_API int llmk_moe_inverse_map(void* inv_tok, void* inv_w, const void* top_idx, const void* slot, const void* top_w, int N, int K,
                                  int E, int cap, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    LLMK_CUDA_TRY(cudaMemsetAsync(inv_tok, 0xff, (size_t)E * cap * 4, st));
    inverse_map_kernel<<<ceil_div((long)N * K, 256), 256, 0, st>>>((int*)inv_tok, (float*)inv_w, (const int*)top_idx, (const int*)slot,
                                                                   (const float*)top_w, N * K, K, cap);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
// This rank's rows and maps are in place: entry [arrive_off + E + my_rank] of every rank's arrival table gets `epoch`.
__global__ void source_ready_kernel(Peers arrive, int idx, int P, int epoch) {
    if ((int)threadIdx.x < P) {
        __threadfence_system();
        st_release_sys(static_cast<int*>(arrive.p[threadIdx.x]) + idx, epoch);
    }
}
LLMK_API int llmk_moe_source_ready(const long long* arrive_ptrs, int arrive_off, int E, int my_rank, int P, int epoch, void* stream) {
    if (P > MAXP) return LLMK_ERR_SHAPE;
    source_ready_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(make_peers(arrive_ptrs, P), arrive_off + E + my_rank, P, epoch);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
// Owner side: fill recv[e_local][src][slot][C] from the sources' memory. x_ptrs / tok_ptrs / w_ptrs: host arrays of the P
// ranks' token rows, inverse token maps and inverse weight maps; `ready`: this rank's arrival entries of the exchange
// (2 * E ints: [0, E) block flags written here, [E, E + P) source flags waited for); done_counters: Eloc * P zeroed ints.
LLMK_API int llmk_moe_dispatch_pull(void* recv, const long long* x_ptrs, const long long* tok_ptrs, const long long* w_ptrs, int C, int E,
                                    int cap, int my_rank, int P, int scale_by_weight, void* ready, void* done_counters, int epoch,
                                    long limit_ns, int* status, void* stream) {
    if (P > MAXP || E % P || C % 8) return LLMK_ERR_SHAPE;
    PullSrc t;
    for (int i = 0; i < MAXP; i++) {
        t.x[i] = i < P ? reinterpret_cast<const bf16*>(x_ptrs[i]) : nullptr;
        t.inv_tok[i] = i < P ? reinterpret_cast<const int*>(tok_ptrs[i]) : nullptr;
        t.inv_w[i] = i < P ? reinterpret_cast<const float*>(w_ptrs[i]) : nullptr;
    }
    dispatch_pull_kernel<<<dim3(ceil_div(cap, 8), P, E / P), 256, 0, (cudaStream_t)stream>>>(
        (bf16*)recv, t, C, cap, E, E / P, my_rank, P, scale_by_weight, (int*)ready, (int*)done_counters, epoch, (long long)limit_ns, status);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_moe_return(const long long* back_ptrs, const void* y, int C, int E, int cap, int my_rank, int P, void* stream) {
    if (P > MAXP || E % P) return LLMK_ERR_SHAPE;
    const Peers back = make_peers(back_ptrs, P);
    return_kernel<<<dim3(32, P, E / P), 256, 0, (cudaStream_t)stream>>>(back, (const bf16*)y, C, cap, E / P, my_rank, P, back, 0,
                                                                      nullptr, 0);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
// Return that publishes each (source rank, local expert) block as it completes; `done_counters`: Eloc * P zeroed ints.
LLMK_API int llmk_moe_return_signal(const long long* back_ptrs, const void* y, int C, int E, int cap, int my_rank, int P,
                                    const long long* arrive_ptrs, int arrive_off, void* done_counters, int epoch, void* stream) {
    if (P > MAXP || E % P || arrive_ptrs == nullptr || done_counters == nullptr) return LLMK_ERR_SHAPE;
    return_kernel<<<dim3(32, P, E / P), 256, 0, (cudaStream_t)stream>>>(make_peers(back_ptrs, P), (const bf16*)y, C, cap, E / P,
                                                                      my_rank, P, make_peers(arrive_ptrs, P), arrive_off,
                                                                      (int*)done_counters, epoch);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_moe_combine(void* out, const void* base, const void* back, const void* top_idx, const void* slot,
                              const void* weights, int N, int K, int C, int cap, void* stream) {
    combine_kernel<<<ceil_div(N, 8), 256, 0, (cudaStream_t)stream>>>((bf16*)out, (const bf16*)base, (const bf16*)back,
                                                                    (const int*)top_idx, (const int*)slot, (const float*)weights,
                                                                    N, K, C, cap, nullptr, 0, 0, 0, nullptr);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
// Combine that first waits (inside the kernel, for at most limit_ns) until `returned[0..E)` all hold `epoch`.
LLMK_API int llmk_moe_combine_wait(void* out, const void* base, const void* back, const void* top_idx, const void* slot,
                                   const void* weights, int N, int K, int C, int cap, const void* returned, int E, int epoch,
                                   long limit_ns, int* status, void* stream) {
    if (returned == nullptr || E <= 0 || E > MAXE) return LLMK_ERR_SHAPE;
    combine_kernel<<<ceil_div(N, 8), 256, 0, (cudaStream_t)stream>>>((bf16*)out, (const bf16*)base, (const bf16*)back,
                                                                    (const int*)top_idx, (const int*)slot, (const float*)weights,
                                                                    N, K, C, cap, (const int*)returned, E, epoch,
                                                                    (long long)limit_ns, status);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_moe_combine_pull(void* out, const void* base, const long long* y_ptrs, void* save, const void* top_idx,
                                   const void* slot, const void* weights, int N, int K, int C, int E, int cap, int my_rank, int P,
                                   const void* returned, int epoch, long limit_ns, int* status, void* stream) {
    if (P > MAXP || E % P || E > MAXE || K > MAXK || C % 8) return LLMK_ERR_SHAPE;
    combine_pull_kernel<<<ceil_div(N, 8), 256, 0, (cudaStream_t)stream>>>((bf16*)out, (const bf16*)base, make_peers(y_ptrs, P), (bf16*)save,
                                                                         (const int*)top_idx, (const int*)slot, (const float*)weights,
                                                                         N, K, C, cap, E / P, my_rank, P, (const int*)returned, E, epoch,
                                                                         (long long)limit_ns, status);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_moe_publish(const long long* arrive_ptrs, int arrive_off, int E, int my_rank, int P, int epoch, void* stream) {
    if (P > MAXP || E % P || E > MAXE) return LLMK_ERR_SHAPE;
    publish_kernel<<<1, 128, 0, (cudaStream_t)stream>>>(make_peers(arrive_ptrs, P), arrive_off, E / P, my_rank, P, epoch);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_moe_combine_dweight(void* dw, const void* dout, const void* back, const void* top_idx, const void* slot, int N,
                                      int K, int C, int cap, void* stream) {
    combine_dweight_kernel<<<ceil_div((long)N * K, 8), 256, 0, (cudaStream_t)stream>>>((float*)dw, (const bf16*)dout,
                                                                                      (const bf16*)back, (const int*)top_idx,
                                                                                      (const int*)slot, N, K, C, cap);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_moe_density(void* density, void* aux_loss, const void* probs, int N, int E, float coef, int accumulate,
                              void* stream) {
    if (E > MAXE) return LLMK_ERR_SHAPE;
    density_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>((float*)density, (float*)aux_loss, (const float*)probs, N, E, coef,
                                                        accumulate);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_moe_router_bwd(void* dlogits, const void* probs, const void* top_idx, const void* top_w, const void* dw,
                                 const void* slot, const void* density, int N, int E, int Epad, int K, float aux_scale,
                                 void* stream) {
    if (E > MAXE || K > MAXK) return LLMK_ERR_SHAPE;
    router_bwd_kernel<<<ceil_div(N, 256), 256, 0, (cudaStream_t)stream>>>((bf16*)dlogits, (const float*)probs, (const int*)top_idx,
                                                                        (const float*)top_w, (const float*)dw, (const int*)slot,
                                                                        (const float*)density, N, E, Epad, K, aux_scale);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
