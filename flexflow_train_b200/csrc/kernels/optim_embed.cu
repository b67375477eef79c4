// optim_embed.cu -- optimizer updates over flat parameter arenas and the
// embedding gather / scatter-add kernels.
//
// Optimizer math follows lib/kernels/src/cuda/optimizer_kernels.cu:23-44 (SGD
// with weight decay, momentum, Nesterov) and :111-133 (Adam with the
// bias-corrected step size alpha_t supplied by the host, cf.
// lib/pcg/src/pcg/optimizer_attrs.cc:7-25).  One launch updates a whole arena:
// fp32 master weights and optimizer state, gradients in bf16 or fp32, and an
// optional bf16 shadow copy written in the same pass for the next forward.
// Embedding kernels correspond to lib/kernels/src/cuda/embedding_kernels.cu:48-310.
#include "common.cuh"

namespace {

template <typename G> __device__ __forceinline__ float ldg(const G *p, long long i);
template <> __device__ __forceinline__ float ldg<float>(const float *p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldg<bf16>(const bf16 *p, long long i) { return bf2f(p[i]); }

template <typename G>
__global__ void adam_kernel(float *__restrict__ w, float *__restrict__ m, float *__restrict__ v,
                            const G *__restrict__ g, bf16 *__restrict__ shadow, long long n, float alpha_t,
                            float beta1, float beta2, float eps, float wd, float gscale,
                            const float *__restrict__ alpha_ptr) {
  // alpha_ptr (optional): bias-corrected step size kept in device memory so that a captured CUDA graph
  // sees the value of the current step.
  if (alpha_ptr) alpha_t = *alpha_ptr;
  long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      float4 w4 = *reinterpret_cast<float4 *>(w + i), m4 = *reinterpret_cast<float4 *>(m + i),
             v4 = *reinterpret_cast<float4 *>(v + i);
      float gg[4] = {ldg(g, i) * gscale, ldg(g, i + 1) * gscale, ldg(g, i + 2) * gscale, ldg(g, i + 3) * gscale};
      float ww[4] = {w4.x, w4.y, w4.z, w4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float gt = gg[j] + wd * ww[j];
        mm[j] = beta1 * mm[j] + (1.f - beta1) * gt;
        vv[j] = beta2 * vv[j] + (1.f - beta2) * gt * gt;
        ww[j] -= alpha_t * mm[j] / (sqrtf(vv[j]) + eps);
      }
      *reinterpret_cast<float4 *>(w + i) = make_float4(ww[0], ww[1], ww[2], ww[3]);
      *reinterpret_cast<float4 *>(m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4 *>(v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      if (shadow) {
        uint2 s = make_uint2(pack_bf162(ww[0], ww[1]), pack_bf162(ww[2], ww[3]));
        *reinterpret_cast<uint2 *>(shadow + i) = s;
      }
    } else {
      for (long long k = i; k < n; ++k) {
        float gt = ldg(g, k) * gscale + wd * w[k];
        float mk = beta1 * m[k] + (1.f - beta1) * gt;
        float vk = beta2 * v[k] + (1.f - beta2) * gt * gt;
        float wk = w[k] - alpha_t * mk / (sqrtf(vk) + eps);
        w[k] = wk; m[k] = mk; v[k] = vk;
        if (shadow) shadow[k] = f2bf(wk);
      }
    }
  }
}

template <typename G>
__global__ void sgd_kernel(float *__restrict__ w, float *__restrict__ mom, const G *__restrict__ g,
                           bf16 *__restrict__ shadow, long long n, float lr, float momentum, int nesterov, float wd,
                           float gscale) {
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float wk = w[i];
    float gt = ldg(g, i) * gscale + wd * wk;
    if (momentum > 0.f) {
      float vk = mom[i] * momentum + gt;
      mom[i] = vk;
      gt = nesterov ? gt + momentum * vk : vk;
    }
    wk -= lr * gt;
    w[i] = wk;
    if (shadow) shadow[i] = f2bf(wk);
  }
}

// out[t, :] = sum_{j<bag} W[idx[t, j], :] (optionally averaged).  One warp per
// (token, 32-column chunk group); rows are read with 16-byte loads when possible.
template <typename W, typename I, typename O>
__global__ void embedding_fwd_kernel(const I *__restrict__ idx, const W *__restrict__ table, O *__restrict__ out,
                                     long long tokens, int bag, int dim, long long entries, int avg) {
  long long total = tokens * dim;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long t = i / dim;
    int c = (int)(i - t * dim);
    float acc = 0.f;
    for (int j = 0; j < bag; ++j) {
      long long e = (long long)idx[t * bag + j];
      if (e >= 0 && e < entries) acc += (float)table[e * dim + c];
    }
    if (avg) acc /= bag;
    out[i] = (O)acc;
  }
}
__device__ __forceinline__ void atomic_add_any(float *p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add_any(bf16 *p, float v) { atomicAdd(p, f2bf(v)); }

template <typename W, typename I, typename O>
__global__ void embedding_bwd_kernel(const I *__restrict__ idx, const O *__restrict__ dout, W *__restrict__ dtable,
                                     long long tokens, int bag, int dim, long long entries, int avg) {
  long long total = tokens * dim;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long t = i / dim;
    int c = (int)(i - t * dim);
    float g = (float)dout[i];
    if (avg) g /= bag;
    for (int j = 0; j < bag; ++j) {
      long long e = (long long)idx[t * bag + j];
      if (e >= 0 && e < entries) atomic_add_any(dtable + e * dim + c, g);
    }
  }
}

// Sparse SGD for embedding tables: W[idx] -= lr * dout, applied straight from
// the output gradient (no dense table gradient is materialised).
template <typename I, typename O>
__global__ void embedding_sgd_kernel(const I *__restrict__ idx, const O *__restrict__ dout, float *__restrict__ table,
                                     long long tokens, int bag, int dim, long long entries, float lr) {
  long long total = tokens * dim;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long t = i / dim;
    int c = (int)(i - t * dim);
    float g = (float)dout[i] * lr;
    for (int j = 0; j < bag; ++j) {
      long long e = (long long)idx[t * bag + j];
      if (e >= 0 && e < entries) atomicAdd(table + e * dim + c, -g);
    }
  }
}

}  // namespace

// grad_dt: 0 = fp32, 1 = bf16.  shadow may be null.
FFK_API int ffk_adam_update(float *w, float *m, float *v, const void *g, void *shadow, long long n, float alpha_t,
                            float beta1, float beta2, float eps, float wd, float gscale, const float *alpha_ptr,
                            int grad_dt, cudaStream_t st) {
  if (n <= 0) return 0;
  int grid = ffk_blocks(n / 4 + 1, 256, 148 * 8);
  if (grad_dt == 1)
    adam_kernel<bf16><<<grid, 256, 0, st>>>(w, m, v, (const bf16 *)g, (bf16 *)shadow, n, alpha_t, beta1, beta2, eps, wd, gscale, alpha_ptr);
  else
    adam_kernel<float><<<grid, 256, 0, st>>>(w, m, v, (const float *)g, (bf16 *)shadow, n, alpha_t, beta1, beta2, eps, wd, gscale, alpha_ptr);
  return (int)cudaGetLastError();
}
FFK_API int ffk_sgd_update(float *w, float *mom, const void *g, void *shadow, long long n, float lr, float momentum,
                           int nesterov, float wd, float gscale, int grad_dt, cudaStream_t st) {
  if (n <= 0) return 0;
  int grid = ffk_blocks(n, 256, 148 * 8);
  if (grad_dt == 1)
    sgd_kernel<bf16><<<grid, 256, 0, st>>>(w, mom, (const bf16 *)g, (bf16 *)shadow, n, lr, momentum, nesterov, wd, gscale);
  else
    sgd_kernel<float><<<grid, 256, 0, st>>>(w, mom, (const float *)g, (bf16 *)shadow, n, lr, momentum, nesterov, wd, gscale);
  return (int)cudaGetLastError();
}

template <typename W, typename I, typename O>
static int emb_launch(int which, const void *idx, const void *table_or_dtable, const void *out_or_dout, long long tokens,
                      int bag, int dim, long long entries, int avg, cudaStream_t st) {
  int grid = ffk_blocks(tokens * dim, 256);
  if (which == 0)
    embedding_fwd_kernel<W, I, O><<<grid, 256, 0, st>>>((const I *)idx, (const W *)table_or_dtable, (O *)out_or_dout,
                                                         tokens, bag, dim, entries, avg);
  else
    embedding_bwd_kernel<W, I, O><<<grid, 256, 0, st>>>((const I *)idx, (const O *)out_or_dout, (W *)table_or_dtable,
                                                         tokens, bag, dim, entries, avg);
  return (int)cudaGetLastError();
}
static int emb_dispatch(int which, const void *idx, const void *table, const void *out, long long tokens, int bag,
                        int dim, long long entries, int avg, int table_dt, int idx_dt, int out_dt, cudaStream_t st) {
  if (tokens <= 0) return 0;
#define EMB_CASE(TD, ID, OD, W, I, O) \
  if (table_dt == TD && idx_dt == ID && out_dt == OD) return emb_launch<W, I, O>(which, idx, table, out, tokens, bag, dim, entries, avg, st);
  EMB_CASE(0, 3, 1, float, long long, bf16)
  EMB_CASE(0, 2, 1, float, int, bf16)
  EMB_CASE(0, 3, 0, float, long long, float)
  EMB_CASE(0, 2, 0, float, int, float)
  EMB_CASE(1, 3, 1, bf16, long long, bf16)
  EMB_CASE(1, 2, 1, bf16, int, bf16)
#undef EMB_CASE
  return -2;
}

// table_dt/out_dt: 0 = fp32, 1 = bf16; idx_dt: 2 = int32, 3 = int64; aggr: 0 = sum, 1 = avg
FFK_API int ffk_embedding_fwd(const void *idx, const void *table, void *out, long long tokens, int bag, int dim,
                              long long entries, int aggr, int table_dt, int idx_dt, int out_dt, cudaStream_t st) {
  return emb_dispatch(0, idx, table, out, tokens, bag, dim, entries, aggr, table_dt, idx_dt, out_dt, st);
}
// dtable += scatter(dout); the caller zeroes dtable at the start of a step.
FFK_API int ffk_embedding_bwd(const void *idx, const void *dout, void *dtable, long long tokens, int bag, int dim,
                              long long entries, int aggr, int table_dt, int idx_dt, int out_dt, cudaStream_t st) {
  return emb_dispatch(1, idx, dtable, dout, tokens, bag, dim, entries, aggr, table_dt, idx_dt, out_dt, st);
}
// fp32 table, plain SGD applied sparsely: table[idx] -= lr * dout
FFK_API int ffk_embedding_sgd(const void *idx, const void *dout, float *table, long long tokens, int bag, int dim,
                              long long entries, float lr, int idx_dt, int out_dt, cudaStream_t st) {
  if (tokens <= 0) return 0;
  int grid = ffk_blocks(tokens * dim, 256);
  if (idx_dt == 3 && out_dt == 1) embedding_sgd_kernel<long long, bf16><<<grid, 256, 0, st>>>((const long long *)idx, (const bf16 *)dout, table, tokens, bag, dim, entries, lr);
  else if (idx_dt == 2 && out_dt == 1) embedding_sgd_kernel<int, bf16><<<grid, 256, 0, st>>>((const int *)idx, (const bf16 *)dout, table, tokens, bag, dim, entries, lr);
  else if (idx_dt == 3 && out_dt == 0) embedding_sgd_kernel<long long, float><<<grid, 256, 0, st>>>((const long long *)idx, (const float *)dout, table, tokens, bag, dim, entries, lr);
  else if (idx_dt == 2 && out_dt == 0) embedding_sgd_kernel<int, float><<<grid, 256, 0, st>>>((const int *)idx, (const float *)dout, table, tokens, bag, dim, entries, lr);
  else return -2;
  return (int)cudaGetLastError();
}
