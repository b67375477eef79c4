/* ffk_noalloc.h -- the one entry point of the kernel library that needs no device allocation from anybody.
 *
 * This entry point has no counterpart in the reference framework; it exists for embedders of this library.
 *
 * Who it is for.  Every other ffk_* function that needs working memory takes a caller-provided scratch
 * pointer, which in practice means the caller (or torch on its behalf) called cudaMalloc at some point.
 * Some callers cannot do that:
 *   - a plug-in running inside a host application that owns the whole device heap through its own pool and
 *     forbids foreign cudaMalloc/cudaFree (they fragment the pool, and cudaFree synchronises the device
 *     under the host's feet);
 *   - a latency-critical serving loop in which any implicit device synchronisation -- which cudaMalloc and
 *     cudaFree are -- is a stall, and whose memory budget was fixed at start-up;
 *   - a C or Fortran program that links libffk.so alone, has no tensor framework to lend it a workspace, and
 *     wants to call one function with its own input and output buffers and nothing else.
 * For them the LayerNorm backward below carries its scratch inside the library image: a file-scope
 * __device__ array of FFK_NOALLOC_SCRATCH_BYTES.  Every GPU that loads libffk.so holds that much memory from
 * load until the process exits, whether or not the function is ever called.
 *
 * Rules of use.
 *   - Sizes: 1 <= cols <= FFK_NOALLOC_MAX_COLS, rows >= 1.  Anything else returns FFK_NOALLOC_ERR_SIZE and
 *     prints one line to stderr; nothing is launched.
 *   - The first call on each device looks up the device address of the scratch array
 *     (cudaGetSymbolAddress, with that device current) and caches it.  Make that first call before any
 *     stream capture begins, from the thread that has the device current.
 *   - All calls share the one array and it keeps whatever the previous call left in it.  The kernel zeroes
 *     the slots it accumulates into before it uses them, so stale contents never leak into a result -- but two
 *     calls that overlap on the GPU (different streams, or different host threads) race on it.  Serialise
 *     them: one stream, or an event between them.
 *   - Nothing here calls cudaMalloc, cudaFree or any library routine that allocates.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FFK_NOALLOC_SCRATCH_BYTES (8u << 20) /* 8 MiB per GPU, resident for the life of the process */
#define FFK_NOALLOC_MAX_COLS 16384

#define FFK_NOALLOC_OK 0
#define FFK_NOALLOC_ERR_SIZE (-2)   /* rows/cols outside the supported range */
#define FFK_NOALLOC_ERR_DTYPE (-3)  /* dt is neither 0 (fp32) nor 1 (bf16) */
#define FFK_NOALLOC_ERR_SETUP (-4)  /* the scratch symbol could not be resolved on the current device */
/* any positive value is a cudaError_t from the launch */

/* LayerNorm backward over the last dimension of a [rows, cols] tensor.
 *   dx     [rows, cols] = d(loss)/d(x)           (written, never accumulated)
 *   dgamma [cols]       = sum_rows dy * xhat     (may be NULL together with dbeta)
 *   dbeta  [cols]       = sum_rows dy
 * dy, x, gamma, dx, dgamma, dbeta share the element type dt (0 = float, 1 = __nv_bfloat16); gamma may be NULL
 * (no scale).  mean and rstd are the per-row statistics the forward pass produced (float).  All pointers are
 * device pointers on the current device; the launch goes to `stream`.
 * Same mathematics as ffk_layernorm_bwd, which instead takes the scratch from its caller. */
int ffk_layernorm_bwd_noalloc(const void *dy, const void *x, const void *gamma, const float *mean, const float *rstd, void *dx,
                              void *dgamma, void *dbeta, int rows, int cols, int dt, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
