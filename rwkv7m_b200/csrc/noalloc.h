// LayerNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference code base.
//
// Who needs it: code that runs where cudaMalloc is off limits -- inside a CUDA-graph capture or
// a latency-critical serving loop where an allocation would synchronise the device, plugins
// hosted by a runtime that owns all device memory, or C callers that link this library without
// PyTorch's caching allocator.  The regular LayerNorm backward needs scratch space for the
// per-row-block partial sums of the weight and bias gradients; here that scratch is a
// file-scope __device__ array inside the library, so the caller passes only inputs and outputs.
//
// Contract
//  * dy, x, dx: bf16 [M, C] row-major; w, mean, rstd, dw, db: fp32 ([C], [M], [M], [C], [C]).
//  * dy, x and dx must start on a 16-byte boundary (the kernels use 16-byte vector accesses), the fp32 arrays on a
//    4-byte boundary.  A null or misaligned pointer is rejected with RWKV7M_NOALLOC_ERR_ARG and nothing is launched.
//  * C must be even and at most RWKV7M_NOALLOC_MAX_C; M >= 1.  Larger sizes are rejected with
//    RWKV7M_NOALLOC_ERR_SIZE and nothing is launched.
//  * The scratch array (RWKV7M_NOALLOC_SCRATCH_BYTES, 4 MiB) is held by every GPU that loads the
//    library until the process exits.
//  * The first call on a device looks up the device address of the scratch array
//    (cudaGetSymbolAddress) with that device current.  Make that first call outside any stream
//    capture.
//  * All calls share the one scratch array: two calls whose kernels overlap on the GPU (different
//    streams, no dependency) race on it.  Calls on one stream are safe; the scratch is fully
//    rewritten by each call before it is read.
//  * No cudaMalloc / cudaFree / allocating library routine is called.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define RWKV7M_NOALLOC_MAX_C 8192
#define RWKV7M_NOALLOC_MAX_PARTS 64
#define RWKV7M_NOALLOC_SCRATCH_BYTES (2 * RWKV7M_NOALLOC_MAX_PARTS * RWKV7M_NOALLOC_MAX_C * 4)

#define RWKV7M_NOALLOC_OK 0
#define RWKV7M_NOALLOC_ERR_SIZE 1    /* M or C outside the supported range */
#define RWKV7M_NOALLOC_ERR_CUDA 2    /* a CUDA runtime call failed (symbol lookup or launch) */
#define RWKV7M_NOALLOC_ERR_ARG 3     /* null or misaligned pointer */

/* stream is a cudaStream_t passed as void* (NULL = default stream). */
int rwkv7m_layernorm_bwd_noalloc(const void* dy, const void* x, const float* w, const float* mean,
                                 const float* rstd, void* dx, float* dw, float* db, int M, int C, void* stream);

/* Human-readable text for the codes above. */
const char* rwkv7m_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
