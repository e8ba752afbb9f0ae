// LayerNorm backward for callers that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference implementation; it exists only in this
// library.
//
// Who needs it: code that runs where cudaMalloc / cudaFree (or any allocating library call, PyTorch's
// caching allocator included) must not happen - for example a host that drives the kernels from
// inside a region in which memory operations are forbidden or would serialise the device, a plug-in
// loaded into a process that owns all device memory itself, or a real-time loop that may not take the
// allocator's locks. Such a caller still owns and passes every input and output tensor; what it
// cannot provide is the temporary buffer the backward pass needs for its per-block partial sums of
// dweight / dbias. Here that buffer is a fixed array inside the library.
//
// Limits and rules
//   * The temporary buffer is a file-scope device array of LLMK_LN_BWD_NOALLOC_SCRATCH_FLOATS floats
//     (16 MiB). Every GPU that loads the library keeps it until the process exits.
//   * A call needs (4 * number of SMs) * 2 * C floats; shapes that need more are rejected with
//     LLMK_ERR_LIMIT (-6) before anything is launched. On a 148-SM GPU this admits C <= 3536.
//   * The first call on each device looks up the device address of the array (no allocation, but a
//     runtime query): make that first call outside any CUDA stream capture.
//   * All calls share the one array and it keeps whatever the previous call left in it. Nothing in it
//     has to start at zero: each call writes every partial it later reads. For the same reason two
//     calls that overlap on the GPU (different streams, or different host threads without ordering)
//     race on it - order them on one stream or with events.
//   * No cudaMalloc, cudaFree or allocating library routine is called on any path of this function.
#pragma once

#define LLMK_LN_BWD_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

// dinp (+)= dLN/dinp (accumulate_dinp != 0 adds to the existing contents), dweight += , dbias += .
// All tensors bf16 except mean / rstd (fp32, one per row); N rows of C channels; `stream` is a
// cudaStream_t. Same arithmetic and results as llmk_layernorm_bwd. Returns 0, or a negative
// LLMK_ERR_* code (LLMK_ERR_LIMIT when the shape exceeds the built-in buffer).
int llmk_layernorm_bwd_noalloc(void* dinp, void* dweight, void* dbias, const void* dout, const void* inp, const void* weight,
                               const void* mean, const void* rstd, int N, int C, int accumulate_dinp, void* stream);

#ifdef __cplusplus
}
#endif
