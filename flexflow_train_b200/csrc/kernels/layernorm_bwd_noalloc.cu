// layernorm_bwd_noalloc.cu -- LayerNorm backward whose working memory lives inside the library.
//
// See ffk_noalloc.h for who needs this and the rules of use.  In short: callers that may not (or cannot)
// allocate device memory -- plug-ins inside an application that owns the device heap, serving loops that
// cannot afford the implicit synchronisation of cudaMalloc/cudaFree, bare C programs without a tensor
// framework -- pass only inputs and outputs; the per-block partial sums of dgamma / dbeta go to the
// file-scope array below.  This file shares no code path with ffk_layernorm_bwd.
#include <cstdio>
#include <mutex>

#include "common.cuh"
#include "ffk_noalloc.h"

namespace {

constexpr int NOALLOC_MAX_BLOCKS = 64;
constexpr size_t NOALLOC_FLOATS = FFK_NOALLOC_SCRATCH_BYTES / sizeof(float);
static_assert(2ull * NOALLOC_MAX_BLOCKS * FFK_NOALLOC_MAX_COLS <= NOALLOC_FLOATS, "scratch too small for the stated maximum");

// The scratch.  In host code this name is only a handle for cudaGetSymbolAddress, never an address a kernel
// could use; the kernels below receive the looked-up device pointer as an argument.
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_FLOATS];

constexpr int MAX_DEVICES = 64;
float *g_scratch_ptr[MAX_DEVICES] = {};
std::mutex g_setup_mutex;

// device address of the scratch on the current device, resolved on first use per device
float *scratch_for_current_device(int *err) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) { *err = FFK_NOALLOC_ERR_SETUP; return nullptr; }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_ptr[dev]) {
    float *ptr = nullptr;
    e = cudaGetSymbolAddress((void **)&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      fprintf(stderr, "ffk_layernorm_bwd_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev, cudaGetErrorString(e));
      *err = FFK_NOALLOC_ERR_SETUP;
      return nullptr;
    }
    g_scratch_ptr[dev] = ptr;
  }
  return g_scratch_ptr[dev];
}

template <typename T> __device__ __forceinline__ float ldv(const T *p);
template <> __device__ __forceinline__ float ldv<float>(const float *p) { return *p; }
template <> __device__ __forceinline__ float ldv<bf16>(const bf16 *p) { return bf2f(*p); }
template <typename T> __device__ __forceinline__ void stv(T *p, float v);
template <> __device__ __forceinline__ void stv<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void stv<bf16>(bf16 *p, float v) { *p = f2bf(v); }

// Block b handles rows b, b + gridDim.x, ...; thread t owns columns t, t + blockDim.x, ... of the block's two
// partial rows in `partial` ([2][gridDim.x][cols]).  Those slots hold whatever the previous call left there,
// so the owning thread clears them first; no other thread ever touches them.
template <typename T>
__global__ void ln_bwd_noalloc_kernel(const T *__restrict__ dy, const T *__restrict__ x, const T *__restrict__ gamma,
                                      const float *__restrict__ mean, const float *__restrict__ rstd, T *__restrict__ dx,
                                      float *__restrict__ partial, int rows, int cols) {
  __shared__ float red[32];
  float *pg = partial + (long long)blockIdx.x * cols;
  float *pb = partial + ((long long)gridDim.x + blockIdx.x) * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) { pg[c] = 0.f; pb[c] = 0.f; }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T *pdy = dy + (long long)row * cols;
    const T *px = x + (long long)row * cols;
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      float g = ldv(pdy + c) * (gamma ? ldv(gamma + c) : 1.f);
      float xh = (ldv(px + c) - mu) * rs;
      s1 += g;
      s2 += g * xh;
    }
    const float m1 = block_sum(s1, red) / cols;
    const float m2 = block_sum(s2, red) / cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      float g0 = ldv(pdy + c);
      float xh = (ldv(px + c) - mu) * rs;
      float g = g0 * (gamma ? ldv(gamma + c) : 1.f);
      stv(dx + (long long)row * cols + c, rs * (g - m1 - xh * m2));
      pg[c] += g0 * xh;
      pb[c] += g0;
    }
  }
}
template <typename T>
__global__ void ln_bwd_noalloc_finish_kernel(const float *__restrict__ partial, int nparts, int cols, T *dgamma, T *dbeta) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float g = 0.f, b = 0.f;
  for (int p = 0; p < nparts; ++p) {
    g += partial[(long long)p * cols + c];
    b += partial[((long long)nparts + p) * cols + c];
  }
  if (dgamma) stv(dgamma + c, g);
  if (dbeta) stv(dbeta + c, b);
}

template <typename T>
int launch(const void *dy, const void *x, const void *gamma, const float *mean, const float *rstd, void *dx, void *dgamma, void *dbeta,
           float *scratch, int rows, int cols, cudaStream_t stream) {
  int grid = rows < NOALLOC_MAX_BLOCKS ? rows : NOALLOC_MAX_BLOCKS;
  ln_bwd_noalloc_kernel<T><<<grid, 256, 0, stream>>>((const T *)dy, (const T *)x, (const T *)gamma, mean, rstd, (T *)dx, scratch, rows, cols);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (dgamma || dbeta) {
    ln_bwd_noalloc_finish_kernel<T><<<(cols + 255) / 256, 256, 0, stream>>>(scratch, grid, cols, (T *)dgamma, (T *)dbeta);
    e = cudaGetLastError();
  }
  return (int)e;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int ffk_layernorm_bwd_noalloc(const void *dy, const void *x, const void *gamma,
                                                                                 const float *mean, const float *rstd, void *dx,
                                                                                 void *dgamma, void *dbeta, int rows, int cols, int dt,
                                                                                 cudaStream_t stream) {
  if (rows < 1 || cols < 1 || cols > FFK_NOALLOC_MAX_COLS) {
    fprintf(stderr,
            "ffk_layernorm_bwd_noalloc: rows=%d cols=%d is outside the supported range (rows >= 1, 1 <= cols <= %d); the built-in "
            "scratch is %u bytes -- use ffk_layernorm_bwd with your own scratch for larger rows\n",
            rows, cols, FFK_NOALLOC_MAX_COLS, (unsigned)FFK_NOALLOC_SCRATCH_BYTES);
    return FFK_NOALLOC_ERR_SIZE;
  }
  if (dt != 0 && dt != 1) {
    fprintf(stderr, "ffk_layernorm_bwd_noalloc: dt=%d is not 0 (fp32) or 1 (bf16)\n", dt);
    return FFK_NOALLOC_ERR_DTYPE;
  }
  int err = 0;
  float *scratch = scratch_for_current_device(&err);
  if (!scratch) return err;
  if (dt == 0) return launch<float>(dy, x, gamma, mean, rstd, dx, dgamma, dbeta, scratch, rows, cols, stream);
  return launch<bf16>(dy, x, gamma, mean, rstd, dx, dgamma, dbeta, scratch, rows, cols, stream);
}
