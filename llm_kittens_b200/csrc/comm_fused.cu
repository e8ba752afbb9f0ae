// Data-parallel communication fused into the optimizer path, over NVLink peer memory.
//
// The reference reduces gradients with ncclReduceScatter / ncclAllReduce per tensor on a side stream,
// computes the gradient norm and AdamW in separate kernels and then all-gathers the updated shards
// with ncclAllGather (llmc/zero.cuh:623-668, train_gpt2.cu:1193-1248, 1283-1375). Here the same work
// is three kinds of kernels of our own that read and write the peers' buffers directly (every rank
// maps every other rank's gradient / parameter / control buffer; the pointers arrive as a table):
//
//   rs_bucket_kernel      per layer bucket, as soon as the bucket's gradients are final on all ranks:
//                         waits (bounded) for the peers' "bucket ready" flags, then for this rank's
//                         shard of every tensor slice reads the P copies with 128-bit peer loads, sums
//                         them in rank order in fp32, scales by 1/P, stores the averaged shard as fp32
//                         and leaves a per-block partial of its squared norm
//                         = reduce-scatter + scale + norm partial in one pass, overlapped with backward.
//   norm_exchange_kernel  sums the partials in fixed order, writes the local sum (and this rank's mean
//                         loss) into every peer's control buffer, waits for the peers' values, adds them in
//                         rank order (so every rank gets the same bits) and produces the clip coefficient
//                         and the global mean loss on the device = the scalar all-reduces of a step,
//                         without a library call.
//   adamw_push_kernel     AdamW (+ stochastic rounding, fp32 master) on the rank's fp32 averaged shard,
//                         each updated bf16 value stored straight into the parameter buffer of EVERY
//                         rank (P2P stores) = optimizer + all-gather in one pass.
//   signal / wait kernels release-store and acquire-poll epoch flags in the peers' control buffers.
//
// Only plain peer loads/stores and system-scope release/acquire are used: no multicast objects, no
// TMA from remote memory. Every wait is bounded by a caller-given time limit; on expiry the kernel
// records LLMK_ST_TIMEOUT_PEER in the status word and returns without touching peer data.
#include "common.cuh"

namespace llmk {
namespace comm {

constexpr int MAXP = 8;            // ranks in one NVLink domain served by the fused path
constexpr int TPB = 256;
constexpr int NORM_VAL_OFFSET = 2048;  // float slots for the exchanged norm sums inside the control buffer
constexpr int CTRL_INTS = 4096;

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
__device__ __forceinline__ uint4 ld_volatile_v4(const void* ptr) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr) : "memory");
    return v;
}
__device__ __forceinline__ float ld_volatile_f32(const float* ptr) {
    float v;
    asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(v) : "l"(ptr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Threads 0..P-1 of the block each poll one flag until it reaches `epoch` or the limit runs out.
// Returns (to every thread of the block) whether all flags arrived. Contains __syncthreads.
__device__ __forceinline__ bool wait_flags_block(const int* my_ctrl, int slot, int epoch, int P, long long limit_ns,
                                                 int* status, int tag) {
    __shared__ int sh_ok;
    // a failure already recorded by an earlier wait ends this one at once: one lost peer costs one time limit, not one
    // per kernel that would have waited for it
    if (threadIdx.x == 0) sh_ok = (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) ? 0 : 1;
    __syncthreads();
    if (sh_ok != 0 && (int)threadIdx.x < P) {
        const int* f = my_ctrl + slot * MAXP + threadIdx.x;
        const unsigned long long t0 = now_ns();
        unsigned int spins = 0;
        while (ld_acquire_sys(f) < epoch) {
            if ((++spins & 63u) == 0 && (long long)(now_ns() - t0) > limit_ns) {
                sh_ok = 0;
                if (status != nullptr && atomicCAS(status, 0, LLMK_ST_TIMEOUT_PEER) == 0) {
                    status[1] = tag;
                    status[2] = slot;
                    status[3] = (int)threadIdx.x;  // the peer that never signalled
                }
                break;
            }
            __nanosleep(64);
        }
    }
    __syncthreads();
    return sh_ok != 0;
}

// ctrl[dst][slot][my_rank] = epoch for every dst (release at system scope: everything this rank wrote
// before this kernel is visible to a peer that acquires the flag)
// `epoch_ptr` (optional): the epoch is read from device memory instead, so that a captured CUDA graph of a step can be
// replayed with a counter that the host bumps between replays.
__global__ void signal_kernel(Peers ctrl, int slot, int my_rank, int P, int epoch, const int* __restrict__ epoch_ptr) {
    if (epoch_ptr != nullptr) epoch = *epoch_ptr;
    if ((int)threadIdx.x < P) {
        __threadfence_system();
        st_release_sys(static_cast<int*>(ctrl.p[threadIdx.x]) + slot * MAXP + my_rank, epoch);
    }
}

__global__ void wait_kernel(const int* my_ctrl, int slot, int epoch, int P, long long limit_ns, int* status) {
    wait_flags_block(my_ctrl, slot, epoch, P, limit_ns, status, 100 + slot);
}

// Segment table: int64[nseg][3] = (offset of this rank's slice in the flat gradient buffer,
// offset in the fp32 shard buffer, length); lengths are multiples of 8.
__global__ void __launch_bounds__(TPB)
rs_bucket_kernel(Peers grads, const int* my_ctrl, int slot, int epoch, const long long* __restrict__ segs,
                 float* __restrict__ gshard, float* __restrict__ norm_partials, int P, float inv_p, int accumulate,
                 long long limit_ns, int* status, const int* __restrict__ epoch_ptr) {
    __shared__ float sh[32];
    if (epoch_ptr != nullptr) epoch = *epoch_ptr;
    const bool ok = wait_flags_block(my_ctrl, slot, epoch, P, limit_ns, status, slot);
    const long long* seg = segs + (size_t)blockIdx.y * 3;
    const size_t g_off = (size_t)seg[0], s_off = (size_t)seg[1], len = (size_t)seg[2];
    float nrm = 0.f;
    if (ok) {
        // two 8-element groups per thread and iteration: 2 * P independent 128-bit peer loads are in flight before the
        // first one is used (with P = 2 a single group leaves the links idle most of the time)
        const size_t stride = (size_t)gridDim.x * TPB * 8;
        for (size_t i0 = ((size_t)blockIdx.x * TPB + threadIdx.x) * 8; i0 < len; i0 += 2 * stride) {
            const size_t i1 = i0 + stride;
            const bool two = i1 < len;
            uint4 raw[2][MAXP];
#pragma unroll
            for (int r = 0; r < MAXP; r++)
                if (r < P) {
                    raw[0][r] = ld_volatile_v4(static_cast<const bf16*>(grads.p[r]) + g_off + i0);
                    if (two) raw[1][r] = ld_volatile_v4(static_cast<const bf16*>(grads.p[r]) + g_off + i1);
                }
#pragma unroll
            for (int h = 0; h < 2; h++) {
                if (h == 1 && !two) break;
                const size_t i = h ? i1 : i0;
                float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
                for (int r = 0; r < MAXP; r++) {
                    if (r < P) {
                        float f[8];
                        unpack8(*reinterpret_cast<const bf16x8*>(&raw[h][r]), f);
#pragma unroll
                        for (int j = 0; j < 8; j++) acc[j] += f[j];
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    acc[j] *= inv_p;
                    nrm += acc[j] * acc[j];
                }
                float4* dst = reinterpret_cast<float4*>(gshard + s_off + i);
                if (accumulate) {   // later micro-steps of a sharded-gradient step add to the running shard
                    const float4 o0 = dst[0], o1 = dst[1];
                    acc[0] += o0.x; acc[1] += o0.y; acc[2] += o0.z; acc[3] += o0.w;
                    acc[4] += o1.x; acc[5] += o1.y; acc[6] += o1.z; acc[7] += o1.w;
                }
                dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
                dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
            }
        }
    }
    nrm = block_sum(nrm, sh);
    if (threadIdx.x == 0) norm_partials[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = nrm;
}

// One block. Sums `n` partials, exchanges the sum with the peers, clip coefficient on the device.
__global__ void __launch_bounds__(1024)
norm_exchange_kernel(Peers ctrl, const float* __restrict__ partials, int n, int norm_slot, int my_rank, int P, int epoch,
                     float clip, float* scale_out, float* norm_out, int* flag_out, float* loss_inout, float norm_scale,
                     long long limit_ns, int* status) {
    __shared__ float sh[32];
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += partials[i];
    s = block_sum(s, sh);
    if ((int)threadIdx.x < P) {
        float* dst_val = reinterpret_cast<float*>(static_cast<int*>(ctrl.p[threadIdx.x]) + NORM_VAL_OFFSET) + my_rank;
        *reinterpret_cast<volatile float*>(dst_val) = s;
        if (loss_inout != nullptr) *reinterpret_cast<volatile float*>(dst_val + MAXP) = loss_inout[0];
        __threadfence_system();
        st_release_sys(static_cast<int*>(ctrl.p[threadIdx.x]) + norm_slot * MAXP + my_rank, epoch);
    }
    const int* my_ctrl = static_cast<const int*>(ctrl.p[my_rank]);
    const bool ok = wait_flags_block(my_ctrl, norm_slot, epoch, P, limit_ns, status, 200);
    if (threadIdx.x == 0) {
        float total = 0.f;
        if (ok) {
            const float* vals = reinterpret_cast<const float*>(my_ctrl + NORM_VAL_OFFSET);
            for (int r = 0; r < P; r++) total += ld_volatile_f32(vals + r);
            if (loss_inout != nullptr) {   // mean over ranks of the ranks' mean losses, summed in rank order
                float loss = 0.f;
                for (int r = 0; r < P; r++) loss += ld_volatile_f32(vals + MAXP + r);
                loss_inout[0] = loss / (float)P;
            }
        } else {
            total = NAN;
        }
        // norm_scale = 1/P when every rank holds the complete (replicated) sum and the exchange adds it P times
        const float nv = sqrtf(total * norm_scale);
        norm_out[0] = nv;
        if (!isfinite(nv)) {
            scale_out[0] = 0.f;
            if (flag_out) flag_out[0] = 1;
        } else {
            scale_out[0] = (clip > 0.f && nv > clip) ? clip / nv : 1.0f;
            if (flag_out) flag_out[0] = 0;
        }
    }
}

// All-gather of one bucket for sharded parameters: segment table int64[nseg][3] = (offset of the shard in
// every rank's shard buffer, offset of the full slice in the local staging buffer, shard length);
// blockIdx.z = source rank. Plain 128-bit peer loads, local stores.
__global__ void __launch_bounds__(TPB)
ag_bucket_kernel(Peers shards, bf16* __restrict__ staging, const long long* __restrict__ segs) {
    const long long* seg = segs + (size_t)blockIdx.y * 3;
    const size_t s_off = (size_t)seg[0], d_off = (size_t)seg[1], len = (size_t)seg[2];
    const int r = blockIdx.z;
    const bf16* src = static_cast<const bf16*>(shards.p[r]) + s_off;
    bf16* dst = staging + d_off + (size_t)r * len;
    for (size_t i = ((size_t)blockIdx.x * TPB + threadIdx.x) * 8; i < len; i += (size_t)gridDim.x * TPB * 8) {
        const uint4 v = ld_volatile_v4(src + i);
        *reinterpret_cast<uint4*>(dst + i) = v;
    }
}

// The same gather with its progress published: segment table int64[nseg][5] = (shard offset, staging offset of the
// full slice, shard length, first flag of the tensor, chunks per shard). A chunk (length / chunks consecutive elements
// of one rank's shard) is copied by `bpc` blocks (blockIdx.x = chunk * bpc + part); the block that finishes a chunk
// last (an arrival counter per flag, left at zero again) release-stores `tick` into flags[first + rank * chunks +
// chunk], which is flag (element offset inside the tensor) / (chunk length). A GEMM that consumes the tensor polls
// exactly the flags that cover a tile (llmk_gemm_b_ready), so it can start on the first chunks while the others are
// still crossing NVLink. Four 128-bit peer loads are in flight per thread.
__global__ void __launch_bounds__(TPB)
ag_bucket_flags_kernel(Peers shards, bf16* __restrict__ staging, const long long* __restrict__ segs, int* __restrict__ flags,
                       int* __restrict__ arrivals, int bpc, int tick) {
    const long long* seg = segs + (size_t)blockIdx.y * 5;
    const size_t s_off = (size_t)seg[0], d_off = (size_t)seg[1], len = (size_t)seg[2];
    const int first = (int)seg[3], cps = (int)seg[4];
    const int r = blockIdx.z, x = blockIdx.x / bpc, part = blockIdx.x - x * bpc;
    if (x >= cps) return;
    const size_t chunk = len / cps;
    // this block's part of the chunk: whole 128-bit words, the last part takes the remainder
    const size_t words = chunk / 8, per = (words + bpc - 1) / bpc;
    const size_t w0 = min(words, (size_t)part * per), w1 = min(words, w0 + per);
    const bf16* src = static_cast<const bf16*>(shards.p[r]) + s_off + (size_t)x * chunk + w0 * 8;
    bf16* dst = staging + d_off + (size_t)r * len + (size_t)x * chunk + w0 * 8;
    const size_t n = (w1 - w0) * 8;
    constexpr size_t STEP = (size_t)TPB * 8;
    size_t i = (size_t)threadIdx.x * 8;
    for (; i + 3 * STEP < n; i += 4 * STEP) {
        const uint4 v0 = ld_volatile_v4(src + i), v1 = ld_volatile_v4(src + i + STEP);
        const uint4 v2 = ld_volatile_v4(src + i + 2 * STEP), v3 = ld_volatile_v4(src + i + 3 * STEP);
        *reinterpret_cast<uint4*>(dst + i) = v0;
        *reinterpret_cast<uint4*>(dst + i + STEP) = v1;
        *reinterpret_cast<uint4*>(dst + i + 2 * STEP) = v2;
        *reinterpret_cast<uint4*>(dst + i + 3 * STEP) = v3;
    }
    for (; i < n; i += STEP) *reinterpret_cast<uint4*>(dst + i) = ld_volatile_v4(src + i);
    __syncthreads();
    if (threadIdx.x == 0) {
        const int f = first + r * cps + x;
        __threadfence();
        if (atomicAdd(arrivals + f, 1) == bpc - 1) {
            arrivals[f] = 0;
            __threadfence();
            asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flags + f), "r"(tick) : "memory");
        }
    }
}

struct AdamArgs {
    float lr, beta1, beta2, inv_b1c, inv_b2c, eps, wd;
    unsigned int seed;
};

// Segment table int64[nseg][4] = (parameter offset in the flat buffer, state offset, length, flags).
// The averaged fp32 gradient of element i of a segment is gshard[state offset + i].
__global__ void __launch_bounds__(TPB)
adamw_push_kernel(Peers params, float* __restrict__ master, const float* __restrict__ gshard, float* __restrict__ m,
                  float* __restrict__ v, const long long* __restrict__ segs, const float* __restrict__ grad_scale_ptr, int P,
                  int my_rank, AdamArgs a) {
    const long long* seg = segs + (size_t)blockIdx.y * 4;
    const size_t p_off = (size_t)seg[0], s_off = (size_t)seg[1], len = (size_t)seg[2];
    const float wd = (seg[3] & 1) ? a.wd : 0.f;
    const float gs = grad_scale_ptr ? grad_scale_ptr[0] : 1.0f;
    // the clip kernel writes scale 0 only for a non-finite gradient norm (0 * inf would poison m, v and the
    // weights): the step is skipped here, and every rank's parameter buffer keeps last step's values
    if (grad_scale_ptr && gs == 0.f) return;
    const bf16* my_params = static_cast<const bf16*>(params.p[my_rank]);
    for (size_t i = ((size_t)blockIdx.x * TPB + threadIdx.x) * 8; i < len; i += (size_t)gridDim.x * TPB * 8) {
        float g[8], mm[8], vv[8], old[8], pn[8];
        const float4* gp = reinterpret_cast<const float4*>(gshard + s_off + i);
        const float4* mp = reinterpret_cast<const float4*>(m + s_off + i);
        const float4* vp = reinterpret_cast<const float4*>(v + s_off + i);
        float4 t0 = gp[0], t1 = gp[1];
        g[0] = t0.x; g[1] = t0.y; g[2] = t0.z; g[3] = t0.w; g[4] = t1.x; g[5] = t1.y; g[6] = t1.z; g[7] = t1.w;
        t0 = mp[0]; t1 = mp[1];
        mm[0] = t0.x; mm[1] = t0.y; mm[2] = t0.z; mm[3] = t0.w; mm[4] = t1.x; mm[5] = t1.y; mm[6] = t1.z; mm[7] = t1.w;
        t0 = vp[0]; t1 = vp[1];
        vv[0] = t0.x; vv[1] = t0.y; vv[2] = t0.z; vv[3] = t0.w; vv[4] = t1.x; vv[5] = t1.y; vv[6] = t1.z; vv[7] = t1.w;
        if (master) {
            const float4* op = reinterpret_cast<const float4*>(master + s_off + i);
            t0 = op[0]; t1 = op[1];
            old[0] = t0.x; old[1] = t0.y; old[2] = t0.z; old[3] = t0.w; old[4] = t1.x; old[5] = t1.y; old[6] = t1.z; old[7] = t1.w;
        } else {
            unpack8(ld128(my_params + p_off + i), old);
        }
        bf16x8 outv;
        bf16* out = reinterpret_cast<bf16*>(&outv);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float gj = gs * g[j];
            mm[j] = a.beta1 * mm[j] + (1.0f - a.beta1) * gj;
            vv[j] = a.beta2 * vv[j] + (1.0f - a.beta2) * gj * gj;
            const float mh = mm[j] * a.inv_b1c, vh = vv[j] * a.inv_b2c;
            pn[j] = old[j] - a.lr * (mh / (sqrtf(vh) + a.eps) + wd * old[j]);
            out[j] = sr_round(pn[j], squirrel5((unsigned int)(p_off + i + j), a.seed));
        }
        float4* mo = reinterpret_cast<float4*>(m + s_off + i);
        float4* vo = reinterpret_cast<float4*>(v + s_off + i);
        mo[0] = make_float4(mm[0], mm[1], mm[2], mm[3]); mo[1] = make_float4(mm[4], mm[5], mm[6], mm[7]);
        vo[0] = make_float4(vv[0], vv[1], vv[2], vv[3]); vo[1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
        if (master) {
            float4* po = reinterpret_cast<float4*>(master + s_off + i);
            po[0] = make_float4(pn[0], pn[1], pn[2], pn[3]); po[1] = make_float4(pn[4], pn[5], pn[6], pn[7]);
        }
        // the all-gather: the updated shard goes to every rank's full parameter buffer
#pragma unroll
        for (int r = 0; r < MAXP; r++)
            if (r < P) st128(static_cast<bf16*>(params.p[r]) + p_off + i, outv);
    }
}

static inline Peers make_peers(const long long* ptrs, int P) {
    Peers q;
    for (int i = 0; i < MAXP; i++) q.p[i] = i < P ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
    return q;
}

}  // namespace comm
}  // namespace llmk

using namespace llmk;
using namespace llmk::comm;

LLMK_API int llmk_comm_max_ranks() { return MAXP; }
LLMK_API int llmk_comm_ctrl_ints() { return CTRL_INTS; }

// `ptrs`: host array of P device pointers (one per rank, this rank's own included).
LLMK_API int llmk_comm_signal(const long long* ctrl_ptrs, int slot, int my_rank, int P, int epoch, void* stream) {
    if (P > MAXP || slot < 0 || (slot + 1) * MAXP > NORM_VAL_OFFSET) return LLMK_ERR_SHAPE;
    signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(make_peers(ctrl_ptrs, P), slot, my_rank, P, epoch, nullptr);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

// The same with the epoch taken from device memory when the kernel runs (for launches recorded in a CUDA graph).
LLMK_API int llmk_comm_signal_dev(const long long* ctrl_ptrs, int slot, int my_rank, int P, const void* epoch_ptr, void* stream) {
    if (P > MAXP || slot < 0 || (slot + 1) * MAXP > NORM_VAL_OFFSET || epoch_ptr == nullptr) return LLMK_ERR_SHAPE;
    signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(make_peers(ctrl_ptrs, P), slot, my_rank, P, 0, (const int*)epoch_ptr);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

LLMK_API int llmk_comm_wait(const void* my_ctrl, int slot, int epoch, int P, long limit_ns, int* status, void* stream) {
    if (P > MAXP || slot < 0 || (slot + 1) * MAXP > NORM_VAL_OFFSET) return LLMK_ERR_SHAPE;
    wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((const int*)my_ctrl, slot, epoch, P, (long long)limit_ns, status);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

// Reduce-scatter + 1/P scale + norm partials for one bucket. norm_partials must hold nseg * grid_x floats.
LLMK_API int llmk_comm_rs_bucket(const long long* grad_ptrs, const void* my_ctrl, int slot, int epoch, const void* segs, int nseg,
                                 void* gshard, void* norm_partials, int grid_x, int P, int accumulate, long limit_ns, int* status,
                                 void* stream) {
    if (P > MAXP || nseg <= 0 || grid_x <= 0) return LLMK_ERR_SHAPE;
    dim3 grid(grid_x, nseg);
    rs_bucket_kernel<<<grid, TPB, 0, (cudaStream_t)stream>>>(make_peers(grad_ptrs, P), (const int*)my_ctrl, slot, epoch,
                                                            (const long long*)segs, (float*)gshard, (float*)norm_partials, P,
                                                            1.0f / (float)P, accumulate, (long long)limit_ns, status, nullptr);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

// The same with the epoch taken from device memory when the kernel runs (for launches recorded in a CUDA graph).
LLMK_API int llmk_comm_rs_bucket_dev(const long long* grad_ptrs, const void* my_ctrl, int slot, const void* epoch_ptr,
                                     const void* segs, int nseg, void* gshard, void* norm_partials, int grid_x, int P,
                                     int accumulate, long limit_ns, int* status, void* stream) {
    if (P > MAXP || nseg <= 0 || grid_x <= 0 || epoch_ptr == nullptr) return LLMK_ERR_SHAPE;
    dim3 grid(grid_x, nseg);
    rs_bucket_kernel<<<grid, TPB, 0, (cudaStream_t)stream>>>(make_peers(grad_ptrs, P), (const int*)my_ctrl, slot, 0,
                                                            (const long long*)segs, (float*)gshard, (float*)norm_partials, P,
                                                            1.0f / (float)P, accumulate, (long long)limit_ns, status,
                                                            (const int*)epoch_ptr);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

// Gather one bucket of sharded parameters from all ranks into the local staging buffer.
LLMK_API int llmk_comm_ag_bucket(const long long* shard_ptrs, void* staging, const void* segs, int nseg, int grid_x, int P,
                                 void* stream) {
    if (P > MAXP || nseg <= 0 || grid_x <= 0) return LLMK_ERR_SHAPE;
    ag_bucket_kernel<<<dim3(grid_x, nseg, P), TPB, 0, (cudaStream_t)stream>>>(make_peers(shard_ptrs, P), (bf16*)staging,
                                                                            (const long long*)segs);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

// Gather with per-chunk flags (see ag_bucket_flags_kernel). `max_cps` = the largest "chunks per shard" in the table;
// every shard length must be a multiple of 8 * its chunk count. `flags` and `arrivals` hold one int per chunk of every
// tensor and rank (arrivals start at zero and are left at zero); `bpc` blocks share one chunk.
LLMK_API int llmk_comm_ag_bucket_flags(const long long* shard_ptrs, void* staging, const void* segs, int nseg, int max_cps, int P,
                                       void* flags, void* arrivals, int bpc, int tick, void* stream) {
    if (P > MAXP || nseg <= 0 || max_cps <= 0 || bpc <= 0 || flags == nullptr || arrivals == nullptr) return LLMK_ERR_SHAPE;
    ag_bucket_flags_kernel<<<dim3(max_cps * bpc, nseg, P), TPB, 0, (cudaStream_t)stream>>>(
        make_peers(shard_ptrs, P), (bf16*)staging, (const long long*)segs, (int*)flags, (int*)arrivals, bpc, tick);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

LLMK_API int llmk_comm_norm_exchange(const long long* ctrl_ptrs, const void* partials, int n, int norm_slot, int my_rank, int P,
                                     int epoch, float clip, void* scale_out, void* norm_out, void* flag_out, void* loss_inout,
                                     float norm_scale, long limit_ns, int* status, void* stream) {
    // loss_inout (optional): in = this rank's mean loss of the step, out = the mean over the P ranks
    if (P > MAXP) return LLMK_ERR_SHAPE;
    norm_exchange_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(make_peers(ctrl_ptrs, P), (const float*)partials, n, norm_slot,
                                                              my_rank, P, epoch, clip, (float*)scale_out, (float*)norm_out,
                                                              (int*)flag_out, (float*)loss_inout, norm_scale, (long long)limit_ns,
                                                              status);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}

LLMK_API int llmk_comm_adamw_push(const long long* param_ptrs, void* master, const void* gshard, void* m, void* v, const void* segs,
                                  int nseg, long max_len, float lr, float beta1, float beta2, float beta1_corr, float beta2_corr,
                                  float eps, float wd, const void* grad_scale_ptr, unsigned int seed, int P, int my_rank,
                                  void* stream) {
    if (P > MAXP || nseg <= 0) return LLMK_ERR_SHAPE;
    AdamArgs a{lr, beta1, beta2, 1.0f / beta1_corr, 1.0f / beta2_corr, eps, wd, seed};
    long gx = (max_len + TPB * 8 - 1) / (TPB * 8);
    if (gx > 512) gx = 512;
    if (gx < 1) gx = 1;
    dim3 grid((unsigned)gx, nseg);
    adamw_push_kernel<<<grid, TPB, 0, (cudaStream_t)stream>>>(make_peers(param_ptrs, P), (float*)master, (const float*)gshard,
                                                             (float*)m, (float*)v, (const long long*)segs,
                                                             (const float*)grad_scale_ptr, P, my_rank, a);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
