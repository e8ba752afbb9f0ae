// Bandwidth-bound element-wise kernels: GELU, SwiGLU, RoPE, residual adds, bias-gradient column
// reduction, encoder (token + position embedding) forward / backward, casts.
//
// Counterparts in the reference: llmc/gelu.cuh:57-81, llmc/swiglu.cuh:66-86, llmc/rope.cuh:47-81,
// llmc/encoder.cuh:157-234, matmul_backward_bias (llmc/matmul.cuh:1203-1236) and the Llama-local
// add/gather kernels (train_llama3.cu:189-251). All use 128-bit accesses; everything that sums over
// tokens does so in a fixed order (no atomics), so gradients are bit-reproducible.
#include "common.cuh"

namespace llmk {
namespace ew {

constexpr int TPB = 256;

__global__ void gelu_fwd_kernel(bf16* __restrict__ out, const bf16* __restrict__ inp, size_t n) {
    size_t i = ((size_t)blockIdx.x * TPB + threadIdx.x) * 8;
    if (i >= n) return;
    float f[8];
    unpack8(ld128_stream(inp + i), f);
#pragma unroll
    for (int j = 0; j < 8; j++) f[j] = gelu_fwd(f[j]);
    st128(out + i, pack8(f));
}
// dinout *= gelu'(inp)
__global__ void gelu_bwd_kernel(bf16* __restrict__ dinout, const bf16* __restrict__ inp, size_t n) {
    size_t i = ((size_t)blockIdx.x * TPB + threadIdx.x) * 8;
    if (i >= n) return;
    float f[8], d[8];
    unpack8(ld128_stream(inp + i), f);
    unpack8(ld128(dinout + i), d);
#pragma unroll
    for (int j = 0; j < 8; j++) d[j] *= gelu_grad(f[j]);
    st128(dinout + i, pack8(d));
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }

// out = silu(gate) * up
__global__ void swiglu_fwd_kernel(bf16* __restrict__ out, const bf16* __restrict__ gate, const bf16* __restrict__ up, size_t n) {
    size_t i = ((size_t)blockIdx.x * TPB + threadIdx.x) * 8;
    if (i >= n) return;
    float g[8], u[8];
    unpack8(ld128_stream(gate + i), g);
    unpack8(ld128_stream(up + i), u);
#pragma unroll
    for (int j = 0; j < 8; j++) g[j] = g[j] * sigmoidf_(g[j]) * u[j];
    st128(out + i, pack8(g));
}
// dgate = dout * up * silu'(gate) ; dup = dout * silu(gate)
__global__ void swiglu_bwd_kernel(bf16* __restrict__ dgate, bf16* __restrict__ dup, const bf16* __restrict__ dout,
                                  const bf16* __restrict__ gate, const bf16* __restrict__ up, size_t n) {
    size_t i = ((size_t)blockIdx.x * TPB + threadIdx.x) * 8;
    if (i >= n) return;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(ld128_stream(gate + i), g);
    unpack8(ld128_stream(up + i), u);
    unpack8(ld128_stream(dout + i), d);
#pragma unroll
    for (int j = 0; j < 8; j++) {
        float s = sigmoidf_(g[j]);
        float silu = g[j] * s;
        dg[j] = d[j] * u[j] * (s + silu * (1.0f - s));
        du[j] = d[j] * silu;
    }
    st128(dgate + i, pack8(dg));
    st128(dup + i, pack8(du));
}

// SwiGLU over a fused [rows, 2H] tensor whose first H columns are `up` and last H are `gate`.
__global__ void swiglu_fused_fwd_kernel(bf16* __restrict__ out, const bf16* __restrict__ upgate, int rows, int H) {
    size_t idx = ((size_t)blockIdx.x * TPB + threadIdx.x) * 8;
    if (idx >= (size_t)rows * H) return;
    const size_t r = idx / H, c = idx % H;
    float g[8], u[8];
    unpack8(ld128_stream(upgate + r * 2 * H + c), u);
    unpack8(ld128_stream(upgate + r * 2 * H + H + c), g);
#pragma unroll
    for (int j = 0; j < 8; j++) g[j] = g[j] * sigmoidf_(g[j]) * u[j];
    st128(out + idx, pack8(g));
}
__global__ void swiglu_fused_bwd_kernel(bf16* __restrict__ dupgate, const bf16* __restrict__ dout,
                                        const bf16* __restrict__ upgate, int rows, int H) {
    size_t idx = ((size_t)blockIdx.x * TPB + threadIdx.x) * 8;
    if (idx >= (size_t)rows * H) return;
    const size_t r = idx / H, c = idx % H;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(ld128_stream(upgate + r * 2 * H + c), u);
    unpack8(ld128_stream(upgate + r * 2 * H + H + c), g);
    unpack8(ld128_stream(dout + idx), d);
#pragma unroll
    for (int j = 0; j < 8; j++) {
        float s = sigmoidf_(g[j]);
        float silu = g[j] * s;
        dg[j] = d[j] * u[j] * (s + silu * (1.0f - s));
        du[j] = d[j] * silu;
    }
    st128(dupgate + r * 2 * H + c, pack8(du));
    st128(dupgate + r * 2 * H + H + c, pack8(dg));
}

// out = a + b
__global__ void add_kernel(bf16* __restrict__ out, const bf16* __restrict__ a, const bf16* __restrict__ b, size_t n) {
    size_t i = ((size_t)blockIdx.x * TPB + threadIdx.x) * 8;
    if (i >= n) return;
    float x[8], y[8];
    unpack8(ld128(a + i), x);
    unpack8(ld128(b + i), y);
#pragma unroll
    for (int j = 0; j < 8; j++) x[j] += y[j];
    st128(out + i, pack8(x));
}

// RoPE on the q and k heads of a packed [B, T, (NH + 2*NKVH) * HS] tensor, in place.
// Pairs are (i, i + HS/2) ("half-split", as the reference's CUDA kernels: llmc/rope.cuh:36-43) or
// (2i, 2i+1) ("interleaved", as train_llama3.py:105-115) depending on `interleaved`.
// freqs: [T, HS/2] float2 (cos, sin). `inverse` applies the transpose rotation (backward).
__global__ void rope_qk_kernel(bf16* __restrict__ qkv, const float2* __restrict__ freqs, int B, int T, int NH, int NKVH, int HS,
                               int interleaved, int inverse) {
    const int half = HS / 2;
    const int heads = NH + NKVH;  // q heads then k heads are rotated; v untouched
    const size_t total = (size_t)B * T * heads * half;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int i = idx % half;
    const int h = (idx / half) % heads;
    const int t = (idx / ((size_t)half * heads)) % T;
    const size_t bt = idx / ((size_t)half * heads);
    const int width = (NH + 2 * NKVH) * HS;
    bf16* base = qkv + bt * width + (size_t)h * HS;
    const int i0 = interleaved ? 2 * i : i;
    const int i1 = interleaved ? 2 * i + 1 : i + half;
    float2 cs = freqs[(size_t)t * half + i];
    if (inverse) cs.y = -cs.y;
    const float x0 = __bfloat162float(base[i0]), x1 = __bfloat162float(base[i1]);
    base[i0] = __float2bfloat16_rn(x0 * cs.x - x1 * cs.y);
    base[i1] = __float2bfloat16_rn(x0 * cs.y + x1 * cs.x);
}

// The same rotation with 16-byte accesses: a thread owns 8 pairs (half-split: 8 elements of each half of a head,
// two loads and two stores; interleaved: 16 consecutive elements). Needs HS to be a multiple of 16.
template <bool INTERLEAVED>
__global__ void rope_qk_vec_kernel(bf16* __restrict__ qkv, const float2* __restrict__ freqs, int B, int T, int NH, int NKVH, int HS,
                                   int inverse) {
    const int half = HS / 2;
    const int groups = half / 8;            // groups of 8 pairs per head
    const int heads = NH + NKVH;
    const size_t total = (size_t)B * T * heads * groups;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int gi = idx % groups;
    const int h = (idx / groups) % heads;
    const size_t bt = idx / ((size_t)groups * heads);
    const int t = bt % T;
    const int width = (NH + 2 * NKVH) * HS;
    bf16* base = qkv + bt * width + (size_t)h * HS;
    bf16* p0 = INTERLEAVED ? base + 16 * gi : base + 8 * gi;
    bf16* p1 = INTERLEAVED ? p0 + 8 : p0 + half;
    float a[8], b[8];
    unpack8(ld128(p0), a);
    unpack8(ld128(p1), b);
    const float4* f4 = reinterpret_cast<const float4*>(freqs + (size_t)t * half + 8 * gi);   // 8 (cos, sin) pairs = 64 bytes
    float cs[16];
#pragma unroll
    for (int j = 0; j < 4; j++) *reinterpret_cast<float4*>(cs + 4 * j) = __ldg(f4 + j);
#pragma unroll
    for (int j = 0; j < 8; j++) {
        // pair j of this group: interleaved -> elements (2j, 2j+1) of the 16; half-split -> (a[j], b[j])
        float& x0r = INTERLEAVED ? (j < 4 ? a[2 * j] : b[2 * j - 8]) : a[j];
        float& x1r = INTERLEAVED ? (j < 4 ? a[2 * j + 1] : b[2 * j - 7]) : b[j];
        const float c = cs[2 * j], sn = inverse ? -cs[2 * j + 1] : cs[2 * j + 1];
        const float x0 = x0r, x1 = x1r;
        x0r = x0 * c - x1 * sn;
        x1r = x0 * sn + x1 * c;
    }
    st128(p0, pack8(a));
    st128(p1, pack8(b));
}

// ------------------------------------------------------------------ bias gradient (column sums)
// stage 1: partial[chunk][c] = sum over the chunk's rows of dout[row][c]; stage 2 sums chunks in order.
constexpr int DB_ROWS = 256;  // rows per chunk
__global__ void dbias_partial_kernel(float* __restrict__ partial, const bf16* __restrict__ dout, int rows, int OC) {
    // block = 32 (column vectors of 8) x 8 (row lanes); grid = (OC/256, chunks, groups): group g sums its own `rows`
    // rows of the stacked dout into its own partials
    __shared__ float sh[8][32][8];
    dout += (size_t)blockIdx.z * rows * OC;
    partial += (size_t)blockIdx.z * gridDim.y * OC;
    const int cv = blockIdx.x * 32 + threadIdx.x;  // column vector index
    const int c = cv * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const int r0 = blockIdx.y * DB_ROWS;
    const int r1 = min(rows, r0 + DB_ROWS);
    if (c < OC) {
        // eight independent 16-byte loads in flight per thread (the chunk has 32 rows per row lane)
        for (int r = r0 + threadIdx.y; r < r1; r += 64) {
            bf16x8 v[8];
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (r + 8 * u < r1) v[u] = ld128_stream(dout + (size_t)(r + 8 * u) * OC + c);
#pragma unroll
            for (int u = 0; u < 8; u++) {
                if (r + 8 * u < r1) {
                    float f[8];
                    unpack8(v[u], f);
#pragma unroll
                    for (int j = 0; j < 8; j++) acc[j] += f[j];
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 8; j++) sh[threadIdx.y][threadIdx.x][j] = acc[j];
    __syncthreads();
    if (threadIdx.y == 0 && c < OC) {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float s = 0.f;
#pragma unroll
            for (int y = 0; y < 8; y++) s += sh[y][threadIdx.x][j];
            partial[(size_t)blockIdx.y * OC + c + j] = s;
        }
    }
}
// block = 32 columns x 32 chunk lanes; lane y sums chunks y, y+32, ... and the lanes are added in a fixed order
__global__ void dbias_finish_kernel(bf16* __restrict__ dbias, const float* __restrict__ partial, int chunks, int OC,
                                    int accumulate) {
    __shared__ float sh[32][33];
    dbias += (size_t)blockIdx.y * OC;                 // grid.y = group
    partial += (size_t)blockIdx.y * chunks * OC;
    const int c = blockIdx.x * 32 + threadIdx.x;
    float s = 0.f;
    if (c < OC)
        for (int k = threadIdx.y; k < chunks; k += 32) s += partial[(size_t)k * OC + c];
    sh[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && c < OC) {
        float t = accumulate ? __bfloat162float(dbias[c]) : 0.f;
#pragma unroll
        for (int y = 0; y < 32; y++) t += sh[y][threadIdx.x];
        dbias[c] = __float2bfloat16_rn(t);
    }
}

// ------------------------------------------------------------------ encoder
// out[b,t,:] = wte[tok[b,t],:] (+ wpe[t,:])
__global__ void encoder_fwd_kernel(bf16* __restrict__ out, const int* __restrict__ tokens, const bf16* __restrict__ wte,
                                   const bf16* __restrict__ wpe, int B, int T, int C) {
    const int cvecs = C / 8;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)B * T * cvecs) return;
    const int cv = idx % cvecs;
    const size_t bt = idx / cvecs;
    const int t = bt % T;
    const int tok = tokens[bt];
    float a[8];
    unpack8(ld128(wte + (size_t)tok * C + cv * 8), a);
    if (wpe != nullptr) {
        float p[8];
        unpack8(ld128(wpe + (size_t)t * C + cv * 8), p);
#pragma unroll
        for (int j = 0; j < 8; j++) a[j] += p[j];
    }
    st128(out + idx * 8, pack8(a));
}
// dwpe[t,:] += sum_b dout[b,t,:]
__global__ void wpe_bwd_kernel(bf16* __restrict__ dwpe, const bf16* __restrict__ dout, int B, int T, int C) {
    const int cvecs = C / 8;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)T * cvecs) return;
    const int cv = idx % cvecs;
    const int t = idx / cvecs;
    float acc[8];
    unpack8(ld128(dwpe + (size_t)t * C + cv * 8), acc);
    for (int b = 0; b < B; b++) {
        float f[8];
        unpack8(ld128_stream(dout + ((size_t)b * T + t) * C + cv * 8), f);
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] += f[j];
    }
    st128(dwpe + (size_t)t * C + cv * 8, pack8(acc));
}
// dwte[tok,:] += sum over the positions holding `tok`. `sorted_tok`/`sorted_pos` list the B*T positions
// ordered by token id (stable, so positions ascend inside a run); block i handles the run that starts
// at sorted index i and exits when i is not a run start. Fixed summation order => deterministic.
__global__ void wte_bwd_kernel(bf16* __restrict__ dwte, const bf16* __restrict__ dout, const int* __restrict__ sorted_tok,
                               const int* __restrict__ sorted_pos, int BT, int C) {
    const int i = blockIdx.x;
    const int tok = sorted_tok[i];
    if (i > 0 && sorted_tok[i - 1] == tok) return;
    const int cvecs = C / 8;
    for (int cv = threadIdx.x; cv < cvecs; cv += blockDim.x) {
        float acc[8];
        unpack8(ld128(dwte + (size_t)tok * C + cv * 8), acc);
        for (int k = i; k < BT && sorted_tok[k] == tok; k++) {
            float f[8];
            unpack8(ld128(dout + (size_t)sorted_pos[k] * C + cv * 8), f);
#pragma unroll
            for (int j = 0; j < 8; j++) acc[j] += f[j];
        }
        st128(dwte + (size_t)tok * C + cv * 8, pack8(acc));
    }
}

__global__ void cast_f32_to_bf16_kernel(bf16* __restrict__ out, const float* __restrict__ in, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2bfloat16_rn(in[i]);
}
__global__ void cast_bf16_to_f32_kernel(float* __restrict__ out, const bf16* __restrict__ in, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __bfloat162float(in[i]);
}

}  // namespace ew
}  // namespace llmk

using namespace llmk;
using namespace llmk::ew;

#define VEC_GRID(n) ceil_div((long)((n) / 8), TPB)

LLMK_API int llmk_gelu_fwd(void* out, const void* inp, long n, void* stream) {
    if (n % 8) return LLMK_ERR_SHAPE;
    gelu_fwd_kernel<<<VEC_GRID(n), TPB, 0, (cudaStream_t)stream>>>((bf16*)out, (const bf16*)inp, (size_t)n);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_gelu_bwd_inplace(void* dinout, const void* inp, long n, void* stream) {
    if (n % 8) return LLMK_ERR_SHAPE;
    gelu_bwd_kernel<<<VEC_GRID(n), TPB, 0, (cudaStream_t)stream>>>((bf16*)dinout, (const bf16*)inp, (size_t)n);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_swiglu_fwd(void* out, const void* gate, const void* up, long n, void* stream) {
    if (n % 8) return LLMK_ERR_SHAPE;
    swiglu_fwd_kernel<<<VEC_GRID(n), TPB, 0, (cudaStream_t)stream>>>((bf16*)out, (const bf16*)gate, (const bf16*)up, (size_t)n);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_swiglu_bwd(void* dgate, void* dup, const void* dout, const void* gate, const void* up, long n, void* stream) {
    if (n % 8) return LLMK_ERR_SHAPE;
    swiglu_bwd_kernel<<<VEC_GRID(n), TPB, 0, (cudaStream_t)stream>>>((bf16*)dgate, (bf16*)dup, (const bf16*)dout,
                                                                     (const bf16*)gate, (const bf16*)up, (size_t)n);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_swiglu_fused_fwd(void* out, const void* upgate, int rows, int H, void* stream) {
    if (H % 8) return LLMK_ERR_SHAPE;
    swiglu_fused_fwd_kernel<<<VEC_GRID((long)rows * H), TPB, 0, (cudaStream_t)stream>>>((bf16*)out, (const bf16*)upgate, rows, H);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_swiglu_fused_bwd(void* dupgate, const void* dout, const void* upgate, int rows, int H, void* stream) {
    if (H % 8) return LLMK_ERR_SHAPE;
    swiglu_fused_bwd_kernel<<<VEC_GRID((long)rows * H), TPB, 0, (cudaStream_t)stream>>>((bf16*)dupgate, (const bf16*)dout,
                                                                                        (const bf16*)upgate, rows, H);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_add(void* out, const void* a, const void* b, long n, void* stream) {
    if (n % 8) return LLMK_ERR_SHAPE;
    add_kernel<<<VEC_GRID(n), TPB, 0, (cudaStream_t)stream>>>((bf16*)out, (const bf16*)a, (const bf16*)b, (size_t)n);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_rope_qk(void* qkv, const void* freqs, int B, int T, int NH, int NKVH, int HS, int interleaved, int inverse,
                          void* stream) {
    if (HS % 2) return LLMK_ERR_SHAPE;
    if (HS % 16 == 0 && (reinterpret_cast<uintptr_t>(qkv) & 15) == 0 && (reinterpret_cast<uintptr_t>(freqs) & 15) == 0) {
        const size_t groups = (size_t)B * T * (NH + NKVH) * (HS / 16);
        if (interleaved)
            rope_qk_vec_kernel<true><<<ceil_div((long)groups, TPB), TPB, 0, (cudaStream_t)stream>>>((bf16*)qkv, (const float2*)freqs, B, T,
                                                                                                  NH, NKVH, HS, inverse);
        else
            rope_qk_vec_kernel<false><<<ceil_div((long)groups, TPB), TPB, 0, (cudaStream_t)stream>>>((bf16*)qkv, (const float2*)freqs, B, T,
                                                                                                   NH, NKVH, HS, inverse);
        LLMK_LAUNCH_CHECK();
        return LLMK_OK;
    }
    const size_t total = (size_t)B * T * (NH + NKVH) * (HS / 2);
    rope_qk_kernel<<<ceil_div((long)total, TPB), TPB, 0, (cudaStream_t)stream>>>((bf16*)qkv, (const float2*)freqs, B, T, NH,
                                                                                NKVH, HS, interleaved, inverse);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API long llmk_dbias_scratch_bytes(int rows, int OC) { return (long)ceil_div(rows, DB_ROWS) * OC * 4; }
// dbias (+)= column sums of dout[rows, OC]
LLMK_API int llmk_dbias(void* dbias, void* scratch, const void* dout, int rows, int OC, int accumulate, void* stream) {
    if (OC % 8) return LLMK_ERR_SHAPE;
    const int chunks = ceil_div(rows, DB_ROWS);
    dim3 grid(ceil_div(OC, 256), chunks), block(32, 8);
    dbias_partial_kernel<<<grid, block, 0, (cudaStream_t)stream>>>((float*)scratch, (const bf16*)dout, rows, OC);
    LLMK_LAUNCH_CHECK();
    dbias_finish_kernel<<<ceil_div(OC, 32), dim3(32, 32), 0, (cudaStream_t)stream>>>((bf16*)dbias, (const float*)scratch, chunks,
                                                                                  OC, accumulate);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
// The same for `groups` row blocks stacked in dout [groups * rows, OC] (the local experts of a mixture-of-experts
// layer): dbias [groups, OC] (+)= per-block column sums, two launches in all. scratch: groups * llmk_dbias_scratch_bytes.
LLMK_API int llmk_dbias_grouped(void* dbias, void* scratch, const void* dout, int rows, int OC, int groups, int accumulate,
                                void* stream) {
    if (OC % 8 || groups <= 0 || groups > 65535) return LLMK_ERR_SHAPE;
    const int chunks = ceil_div(rows, DB_ROWS);
    dim3 grid(ceil_div(OC, 256), chunks, groups), block(32, 8);
    dbias_partial_kernel<<<grid, block, 0, (cudaStream_t)stream>>>((float*)scratch, (const bf16*)dout, rows, OC);
    LLMK_LAUNCH_CHECK();
    dbias_finish_kernel<<<dim3(ceil_div(OC, 32), groups), dim3(32, 32), 0, (cudaStream_t)stream>>>((bf16*)dbias, (const float*)scratch,
                                                                                                 chunks, OC, accumulate);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_encoder_fwd(void* out, const void* tokens, const void* wte, const void* wpe, int B, int T, int C, void* stream) {
    if (C % 8) return LLMK_ERR_SHAPE;
    const size_t total = (size_t)B * T * (C / 8);
    encoder_fwd_kernel<<<ceil_div((long)total, TPB), TPB, 0, (cudaStream_t)stream>>>((bf16*)out, (const int*)tokens,
                                                                                    (const bf16*)wte, (const bf16*)wpe, B, T, C);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
// ------------------------------------------------------------------ bucketing positions by token id
// Stable least-significant-digit radix sort of (token id, position) pairs, 9 bits per pass, on the device and without
// a library: the embedding gradient sums the rows of each token id in ascending position order, which is what makes
// it deterministic (job of the host-side bucket construction in the reference, llmc/encoder.cuh:169-234).
// Per pass: (1) one 512-bin histogram per tile of 2048 pairs, (2) an exclusive scan over (digit, tile), (3) a
// stable scatter: one warp walks its tile in order, a pair's rank inside its digit = pairs of that digit in earlier
// tiles (scan) + earlier in this tile (running count in shared memory) + in lower lanes (match_any).
namespace bucket {
constexpr int BITS = 9, BINS = 1 << BITS, TILE = 2048;

__global__ void __launch_bounds__(256)
hist_kernel(int* __restrict__ hist, const int* __restrict__ keys, int n, int shift, int ntiles) {
    __shared__ int h[BINS];
    for (int i = threadIdx.x; i < BINS; i += blockDim.x) h[i] = 0;
    __syncthreads();
    const int base = blockIdx.x * TILE;
    for (int i = threadIdx.x; i < TILE && base + i < n; i += blockDim.x) atomicAdd(&h[(keys[base + i] >> shift) & (BINS - 1)], 1);
    __syncthreads();
    for (int i = threadIdx.x; i < BINS; i += blockDim.x) hist[i * ntiles + blockIdx.x] = h[i];
}

// exclusive prefix sum of `m` ints in place, one block of 1024 threads (each thread owns a contiguous stretch)
__global__ void __launch_bounds__(1024)
scan_kernel(int* __restrict__ data, int m) {
    __shared__ int part[1024];
    const int per = (m + 1023) / 1024;
    const int lo = min(m, (int)threadIdx.x * per), hi = min(m, lo + per);
    int s = 0;
    for (int i = lo; i < hi; i++) s += data[i];
    part[threadIdx.x] = s;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
        const int v = threadIdx.x >= o ? part[threadIdx.x - o] : 0;
        __syncthreads();
        part[threadIdx.x] += v;
        __syncthreads();
    }
    int run = part[threadIdx.x] - s;
    for (int i = lo; i < hi; i++) {
        const int v = data[i];
        data[i] = run;
        run += v;
    }
}

// vals_in == nullptr: the value of pair i is i (first pass)
__global__ void __launch_bounds__(32)
scatter_kernel(int* __restrict__ keys_out, int* __restrict__ vals_out, const int* __restrict__ keys_in,
               const int* __restrict__ vals_in, const int* __restrict__ offsets, int n, int shift, int ntiles) {
    __shared__ int running[BINS];
    const int lane = threadIdx.x;
    for (int i = lane; i < BINS; i += 32) running[i] = offsets[i * ntiles + blockIdx.x];
    __syncwarp();
    const int base = blockIdx.x * TILE;
    for (int it = 0; it < TILE / 32; it++) {
        const int i = base + it * 32 + lane;
        const bool live = i < n;
        const unsigned active = __ballot_sync(0xffffffffu, live);
        if (live) {
            const int key = keys_in[i];
            const int d = (key >> shift) & (BINS - 1);
            const unsigned same = __match_any_sync(active, d);
            const int rank = __popc(same & ((1u << lane) - 1u));
            const int dst = running[d] + rank;
            keys_out[dst] = key;
            vals_out[dst] = vals_in != nullptr ? vals_in[i] : i;
            __syncwarp(active);
            if (rank == 0) running[d] += __popc(same);   // the lowest lane of each digit group
        }
        __syncwarp();
    }
}
}  // namespace bucket

// sorted_tok / sorted_pos (n ints each) = positions 0..n-1 ordered by (tokens[pos], pos). `scratch`: at least
// llmk_bucket_sort_scratch_ints(n) ints. `max_token` bounds the keys (number of 9-bit passes).
LLMK_API long llmk_bucket_sort_scratch_ints(int n) { return 2L * n + (long)bucket::BINS * ceil_div(n, bucket::TILE); }
LLMK_API int llmk_bucket_sort(void* sorted_tok, void* sorted_pos, const void* tokens, int n, int max_token, void* scratch,
                              void* stream) {
    if (n <= 0 || max_token <= 0) return LLMK_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    const int ntiles = ceil_div(n, bucket::TILE);
    if ((long)bucket::BINS * ntiles > (1L << 24)) return LLMK_ERR_SHAPE;
    int passes = 1;
    while (passes * bucket::BITS < 31 && (max_token >> (passes * bucket::BITS)) > 0) passes++;
    int* tmp_k = (int*)scratch;
    int* tmp_v = tmp_k + n;
    int* hist = tmp_v + n;
    const int* kin = (const int*)tokens;
    const int* vin = nullptr;
    for (int p = 0; p < passes; p++) {
        // ping-pong so that the last pass lands in the output arrays
        const bool to_out = ((passes - 1 - p) % 2) == 0;
        int* kout = to_out ? (int*)sorted_tok : tmp_k;
        int* vout = to_out ? (int*)sorted_pos : tmp_v;
        bucket::hist_kernel<<<ntiles, 256, 0, st>>>(hist, kin, n, p * bucket::BITS, ntiles);
        LLMK_LAUNCH_CHECK();
        bucket::scan_kernel<<<1, 1024, 0, st>>>(hist, bucket::BINS * ntiles);
        LLMK_LAUNCH_CHECK();
        bucket::scatter_kernel<<<ntiles, 32, 0, st>>>(kout, vout, kin, vin, hist, n, p * bucket::BITS, ntiles);
        LLMK_LAUNCH_CHECK();
        kin = kout;
        vin = vout;
    }
    return LLMK_OK;
}

// dwte += scatter of dout rows by token, dwpe += sum over batch (dwpe may be null for models without wpe).
LLMK_API int llmk_encoder_bwd(void* dwte, void* dwpe, const void* dout, const void* sorted_tok, const void* sorted_pos, int B,
                              int T, int C, void* stream) {
    if (C % 8) return LLMK_ERR_SHAPE;
    if (dwpe != nullptr) {
        wpe_bwd_kernel<<<ceil_div((long)T * (C / 8), TPB), TPB, 0, (cudaStream_t)stream>>>((bf16*)dwpe, (const bf16*)dout, B, T, C);
        LLMK_LAUNCH_CHECK();
    }
    int threads = C / 8;
    if (threads > 256) threads = 256;
    threads = ((threads + 31) / 32) * 32;
    wte_bwd_kernel<<<B * T, threads, 0, (cudaStream_t)stream>>>((bf16*)dwte, (const bf16*)dout, (const int*)sorted_tok,
                                                              (const int*)sorted_pos, B * T, C);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_cast_f32_to_bf16(void* out, const void* in, long n, void* stream) {
    cast_f32_to_bf16_kernel<<<ceil_div(n, TPB), TPB, 0, (cudaStream_t)stream>>>((bf16*)out, (const float*)in, (size_t)n);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
LLMK_API int llmk_cast_bf16_to_f32(void* out, const void* in, long n, void* stream) {
    cast_bf16_to_f32_kernel<<<ceil_div(n, TPB), TPB, 0, (cudaStream_t)stream>>>((float*)out, (const bf16*)in, (size_t)n);
    LLMK_LAUNCH_CHECK();
    return LLMK_OK;
}
