// norm_softmax.cu -- row-wise kernels: LayerNorm fwd/bwd (with the dX pass the
// reference defines but never launches, lib/kernels/src/cuda/ops/layer_norm_kernels.cu:163),
// softmax fwd/bwd (replaces cudnnSoftmaxForward, softmax_kernels.cu:57), fused
// softmax + sparse categorical cross-entropy, and the loss-gradient kernels of
// lib/kernels/src/cuda/loss_function_kernels.cu:21-51.
//
// All kernels take bf16 or fp32 activations (dt: 0 = fp32, 1 = bf16) and keep
// statistics in fp32.
#include "common.cuh"
#include "rowwise_vec.cuh"

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T *p);
template <> __device__ __forceinline__ float ldf<float>(const float *p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16 *p) { return bf2f(*p); }
template <typename T> __device__ __forceinline__ void stf(T *p, float v);
template <> __device__ __forceinline__ void stf<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16 *p, float v) { *p = f2bf(v); }

// ------------------------------------------------------------------ LayerNorm
// y = LN(a + b) * gamma + beta ; b optional (fused residual add); when b is
// given and xsum is non-null the sum a + b is written too (backward needs it).
template <typename T>
__global__ void layernorm_fwd_kernel(const T *__restrict__ a, const T *__restrict__ b, const T *__restrict__ gamma,
                                     const T *__restrict__ beta, T *__restrict__ xsum, T *__restrict__ y,
                                     float *__restrict__ mean, float *__restrict__ rstd, int rows, int cols,
                                     float eps) {
  __shared__ float red[32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T *pa = a + (long long)row * cols;
    const T *pb = b ? b + (long long)row * cols : nullptr;
    float s = 0.f, ss = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      float v = ldf(pa + c) + (pb ? ldf(pb + c) : 0.f);
      if (pb && xsum) {
        stf(xsum + (long long)row * cols + c, v);
        v = ldf(xsum + (long long)row * cols + c);  // statistics of the rounded value backward will see
      }
      s += v;
      ss += v * v;
    }
    s = block_sum(s, red);
    ss = block_sum(ss, red);
    float mu = s / cols;
    float var = fmaxf(ss / cols - mu * mu, 0.f);
    float rs = rsqrtf(var + eps);
    if (threadIdx.x == 0) {
      if (mean) mean[row] = mu;
      if (rstd) rstd[row] = rs;
    }
    const T *px = (pb && xsum) ? xsum + (long long)row * cols : pa;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      float v = (pb && !xsum) ? ldf(pa + c) + ldf(pb + c) : ldf(px + c);
      float o = (v - mu) * rs;
      if (gamma) o = o * ldf(gamma + c) + (beta ? ldf(beta + c) : 0.f);
      stf(y + (long long)row * cols + c, o);
    }
  }
}

// One pass over (dy, x): writes dx and per-block partial column sums of
// dgamma / dbeta into scratch `partial` laid out [2][gridDim.x][cols].
// Thread t owns columns t, t+blockDim, ... (at most KMAX of them).
template <typename T, int KMAX>
__global__ void layernorm_bwd_kernel(const T *__restrict__ dy, const T *__restrict__ x, const T *__restrict__ gamma,
                                     const float *__restrict__ mean, const float *__restrict__ rstd,
                                     T *__restrict__ dx, T *__restrict__ dx2, float *__restrict__ partial, int rows,
                                     int cols, int accumulate_dx, int accumulate_dx2) {
  __shared__ float red[32];
  float dg[KMAX], db[KMAX];
#pragma unroll
  for (int k = 0; k < KMAX; ++k) { dg[k] = 0.f; db[k] = 0.f; }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T *pdy = dy + (long long)row * cols;
    const T *px = x + (long long)row * cols;
    float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    float vg[KMAX], vx[KMAX];
#pragma unroll
    for (int k = 0; k < KMAX; ++k) {
      int c = threadIdx.x + k * blockDim.x;
      if (c < cols) {
        float g = ldf(pdy + c);
        float xh = (ldf(px + c) - mu) * rs;
        dg[k] += g * xh;
        db[k] += g;
        float gg = gamma ? g * ldf(gamma + c) : g;
        vg[k] = gg;
        vx[k] = xh;
        s1 += gg;
        s2 += gg * xh;
      }
    }
    s1 = block_sum(s1, red);
    s2 = block_sum(s2, red);
    float m1 = s1 / cols, m2 = s2 / cols;
#pragma unroll
    for (int k = 0; k < KMAX; ++k) {
      int c = threadIdx.x + k * blockDim.x;
      if (c < cols) {
        float o = rs * (vg[k] - m1 - vx[k] * m2);
        T *pdx = dx + (long long)row * cols + c;
        stf(pdx, accumulate_dx ? ldf(pdx) + o : o);
        if (dx2) {  // second consumer of the same gradient (the other operand of a fused residual add)
          T *pdx2 = dx2 + (long long)row * cols + c;
          stf(pdx2, accumulate_dx2 ? ldf(pdx2) + o : o);
        }
      }
    }
  }
  if (partial) {
#pragma unroll
    for (int k = 0; k < KMAX; ++k) {
      int c = threadIdx.x + k * blockDim.x;
      if (c < cols) {
        partial[(long long)blockIdx.x * cols + c] = dg[k];
        partial[((long long)gridDim.x + blockIdx.x) * cols + c] = db[k];
      }
    }
  }
}
// ------------------------------------------------------------------ Softmax
// y = softmax(scale * x) over the last dim.  causal_q > 0: row r is query
// position (r % causal_q) and keys past it are masked out.
template <typename T>
__global__ void softmax_fwd_kernel(const T *__restrict__ x, T *__restrict__ y, int rows, int cols, float scale,
                                   int causal_q) {
  __shared__ float red[32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T *px = x + (long long)row * cols;
    int limit = causal_q > 0 ? min(cols, (row % causal_q) + 1) : cols;
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < limit; c += blockDim.x) mx = fmaxf(mx, ldf(px + c) * scale);
    mx = block_max(mx, red);
    float s = 0.f;
    for (int c = threadIdx.x; c < limit; c += blockDim.x) s += __expf(ldf(px + c) * scale - mx);
    s = block_sum(s, red);
    float inv = 1.f / s;
    T *py = y + (long long)row * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x)
      stf(py + c, c < limit ? __expf(ldf(px + c) * scale - mx) * inv : 0.f);
  }
}
// dx = scale * y * (dy - sum(dy * y))
template <typename T>
__global__ void softmax_bwd_kernel(const T *__restrict__ dy, const T *__restrict__ y, T *__restrict__ dx, int rows,
                                   int cols, float scale) {
  __shared__ float red[32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T *pdy = dy + (long long)row * cols;
    const T *py = y + (long long)row * cols;
    float s = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) s += ldf(pdy + c) * ldf(py + c);
    s = block_sum(s, red);
    T *pdx = dx + (long long)row * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) stf(pdx + c, scale * ldf(py + c) * (ldf(pdy + c) - s));
  }
}

// Fused softmax + sparse categorical cross-entropy: per-row loss, optional
// probabilities, and dlogits = (p - onehot(label)) * grad_scale.  Rows whose
// label is negative contribute no loss and no gradient.
template <typename T, typename L>
__global__ void softmax_ce_kernel(const T *__restrict__ logits, const L *__restrict__ labels, T *__restrict__ probs,
                                  T *__restrict__ dlogits, float *__restrict__ loss, int rows, int cols,
                                  float grad_scale) {
  __shared__ float red[32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T *px = logits + (long long)row * cols;
    long long label = (long long)labels[row];
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) mx = fmaxf(mx, ldf(px + c));
    mx = block_max(mx, red);
    float s = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) s += __expf(ldf(px + c) - mx);
    s = block_sum(s, red);
    float inv = 1.f / s;
    bool valid = label >= 0 && label < cols;
    if (threadIdx.x == 0 && loss) loss[row] = valid ? (__logf(s) + mx - ldf(px + label)) : 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      float p = __expf(ldf(px + c) - mx) * inv;
      if (probs) stf(probs + (long long)row * cols + c, p);
      if (dlogits) stf(dlogits + (long long)row * cols + c, valid ? (p - (c == label ? 1.f : 0.f)) * grad_scale : 0.f);
    }
  }
}

// bf16 rows with cols % 8 == 0: 16-byte accesses; one pass finds the row maximum and the sum of exponentials
// together (online softmax), a second pass over the (cache-resident) row writes the gradient.
template <typename L>
__global__ void softmax_ce_vec_kernel(const bf16 *__restrict__ logits, const L *__restrict__ labels, bf16 *__restrict__ probs,
                                      bf16 *__restrict__ dlogits, float *__restrict__ loss, int rows, int cols, float grad_scale) {
  __shared__ float2 red[32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  const int nvec = cols >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const bf16 *px = logits + (long long)row * cols;
    const long long label = (long long)labels[row];
    float m = -INFINITY, s = 0.f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      float v[8];
      vec::ld8(px + i * 8, v);
      float vm = v[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) vm = fmaxf(vm, v[j]);
      const float nm = fmaxf(m, vm);
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += __expf(v[j] - nm);
      s = s * __expf(m - nm) + acc;
      m = nm;
    }
    // combine (m, s) pairs: warp, then block
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
      const float nm = fmaxf(m, om);
      s = (nm == -INFINITY) ? 0.f : s * __expf(m - nm) + os * __expf(om - nm);
      m = nm;
    }
    __syncthreads();  // the previous row's readers are done with `red`
    if (lane == 0) red[wid] = make_float2(m, s);
    __syncthreads();
    float M = -INFINITY, S = 0.f;
    for (int k = 0; k < nw; ++k) M = fmaxf(M, red[k].x);
    for (int k = 0; k < nw; ++k) S += (red[k].x == -INFINITY) ? 0.f : red[k].y * __expf(red[k].x - M);
    const float inv = 1.f / S;
    const bool valid = label >= 0 && label < cols;
    if (threadIdx.x == 0 && loss) loss[row] = valid ? (__logf(S) + M - bf2f(px[valid ? label : 0])) : 0.f;
    if (probs || dlogits) {
      for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        float v[8], g[8];
        vec::ld8(px + i * 8, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __expf(v[j] - M) * inv;
        if (probs) vec::st8(probs + (long long)row * cols + i * 8, v);
        if (dlogits) {
#pragma unroll
          for (int j = 0; j < 8; ++j) g[j] = valid ? (v[j] - ((long long)(i * 8 + j) == label ? 1.f : 0.f)) * grad_scale : 0.f;
          vec::st8(dlogits + (long long)row * cols + i * 8, g);
        }
      }
    }
  }
}

// ------------------------------------------------------------------ loss gradients
enum { LOSS_SPARSE_CCE = 0, LOSS_CCE = 1, LOSS_MSE_AVG = 2, LOSS_IDENTITY = 3, LOSS_MSE_SUM = 4 };
// dlogit for losses whose input is already a probability / prediction tensor.
template <typename T, typename L>
__global__ void loss_bwd_kernel(int kind, const T *__restrict__ pred, const void *__restrict__ target,
                                T *__restrict__ dpred, long long rows, int cols, float scale) {
  long long n = rows * cols;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float p = ldf(pred + i), g;
    if (kind == LOSS_SPARSE_CCE) {
      long long lab = (long long)((const L *)target)[i / cols];
      g = p - ((i % cols) == lab ? 1.f : 0.f);
    } else if (kind == LOSS_CCE) {
      g = p - ldf((const T *)target + i);
    } else if (kind == LOSS_MSE_AVG || kind == LOSS_MSE_SUM) {
      g = 2.f * (p - ldf((const T *)target + i));
    } else {
      g = 1.f;
    }
    stf(dpred + i, g * scale);
  }
}
// per-row loss values for reporting
template <typename T, typename L>
__global__ void loss_fwd_kernel(int kind, const T *__restrict__ pred, const void *__restrict__ target,
                                float *__restrict__ loss, int rows, int cols) {
  __shared__ float red[32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T *pp = pred + (long long)row * cols;
    float acc = 0.f;
    if (kind == LOSS_SPARSE_CCE) {
      long long lab = (long long)((const L *)target)[row];
      if (threadIdx.x == 0 && lab >= 0 && lab < cols) acc = -__logf(fmaxf(ldf(pp + lab), 1e-30f));
    } else {
      const T *pt = (const T *)target + (long long)row * cols;
      for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        float p = ldf(pp + c);
        if (kind == LOSS_CCE) acc += -ldf(pt + c) * __logf(fmaxf(p, 1e-30f));
        else if (kind == LOSS_IDENTITY) acc += p;
        else { float d = p - ldf(pt + c); acc += d * d; }
      }
    }
    acc = block_sum(acc, red);
    if (threadIdx.x == 0) loss[row] = acc;
  }
}

}  // namespace

#define DISPATCH_FLOAT(dt, ...)                                   \
  if ((dt) == 0) { typedef float T; __VA_ARGS__; }                \
  else if ((dt) == 1) { typedef bf16 T; __VA_ARGS__; }            \
  else return -2;

static int rows_grid(int rows) { return rows < 148 * 8 ? rows : 148 * 8; }
static bool aligned16(const void *p) { return (((uintptr_t)p) & 15) == 0; }
// vectors per thread for the vectorised LayerNorm kernels: the smallest of 1/2/4 that gives a block of
// whole warps with at most 512 threads; 0 = not expressible
static int ln_vpt(int cols) {
  if (cols % 8) return 0;
  int nv = cols / 8;
  for (int v = 1; v <= 4; v *= 2)
    if (nv % v == 0 && (nv / v) % 32 == 0 && nv / v <= 512) return v;
  return 0;
}
static bool ln_vec_ok(int cols, const void *a, const void *b, const void *c, const void *d, const void *e, const void *f) {
  return ln_vpt(cols) > 0 && aligned16(a) && aligned16(b) && aligned16(c) && aligned16(d) && aligned16(e) && aligned16(f);
}

FFK_API int ffk_layernorm_fwd(const void *a, const void *b, const void *gamma, const void *beta, void *xsum, void *y,
                              float *mean, float *rstd, int rows, int cols, float eps, int dt, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (dt == 1 && ln_vec_ok(cols, a, b, gamma, beta, xsum, y)) {
    int vpt = ln_vpt(cols), threads = cols / 8 / vpt;
    const bf16 *A = (const bf16 *)a, *B = (const bf16 *)b, *G = (const bf16 *)gamma, *Bt = (const bf16 *)beta;
    // rows of up to 2048 elements in steps of 256: one warp per row, no block-wide barriers in the row loop
    if (cols % 256 == 0 && cols <= 2048 && rows >= 8) {
      const int wv = cols / 256;
      long long want = ((long long)rows + 7) / 8;
      const int grid = (int)(want < 148 * 2 ? want : 148 * 2);
#define LN_WARP(V) vec::layernorm_fwd_warp_kernel<V><<<grid, 256, 0, st>>>(A, B, G, Bt, (bf16 *)xsum, (bf16 *)y, mean, rstd, rows, eps)
      switch (wv) {
        case 1: LN_WARP(1); break;
        case 2: LN_WARP(2); break;
        case 3: LN_WARP(3); break;
        case 4: LN_WARP(4); break;
        case 5: LN_WARP(5); break;
        case 6: LN_WARP(6); break;
        case 7: LN_WARP(7); break;
        default: LN_WARP(8); break;
      }
#undef LN_WARP
      return (int)cudaGetLastError();
    }
    if (vpt == 1) vec::layernorm_fwd_vec_kernel<1><<<rows_grid(rows), threads, 0, st>>>(A, B, G, Bt, (bf16 *)xsum, (bf16 *)y, mean, rstd, rows, cols, eps);
    else if (vpt == 2) vec::layernorm_fwd_vec_kernel<2><<<rows_grid(rows), threads, 0, st>>>(A, B, G, Bt, (bf16 *)xsum, (bf16 *)y, mean, rstd, rows, cols, eps);
    else vec::layernorm_fwd_vec_kernel<4><<<rows_grid(rows), threads, 0, st>>>(A, B, G, Bt, (bf16 *)xsum, (bf16 *)y, mean, rstd, rows, cols, eps);
    return (int)cudaGetLastError();
  }
  int threads = cols >= 2048 ? 512 : 256;
  DISPATCH_FLOAT(dt, (layernorm_fwd_kernel<T><<<rows_grid(rows), threads, 0, st>>>(
                         (const T *)a, (const T *)b, (const T *)gamma, (const T *)beta, (T *)xsum, (T *)y, mean, rstd,
                         rows, cols, eps)));
  return (int)cudaGetLastError();
}

// Persistent blocks of the backward kernel: as many per SM as its registers allow for the block size in use (narrow
// rows mean small blocks, of which two per SM left most of the SM idle); each block writes one partial row of
// dgamma / dbeta, which the fold kernel sums.
static int ln_bwd_grid(int rows, int cols, bool vec) {
  int per_sm = 2;
  if (vec && ln_vpt(cols) > 0) {
    const int threads = cols / 8 / ln_vpt(cols);
    per_sm = 768 / threads;
    if (per_sm < 2) per_sm = 2;
    if (per_sm > 8) per_sm = 8;
  }
  const int g = 148 * per_sm;
  return rows < g ? rows : g;
}
// floats of scratch needed by ffk_layernorm_bwd (the larger of the two kernel forms' needs)
FFK_API long long ffk_layernorm_bwd_scratch(int rows, int cols) {
  const int a = ln_bwd_grid(rows, cols, true), b = ln_bwd_grid(rows, cols, false);
  return 2ll * (a > b ? a : b) * cols;
}

// dx (+)= LN backward; dgamma/dbeta (+)= column sums.  `partial` is scratch of
// ffk_layernorm_bwd_scratch(rows, cols) floats.  cols <= 16384.
FFK_API int ffk_layernorm_bwd(const void *dy, const void *x, const void *gamma, const float *mean, const float *rstd,
                              void *dx, void *dx2, void *dgamma, void *dbeta, float *partial, int rows, int cols, int dt,
                              int accumulate_dx, int accumulate_dx2, int accumulate_params, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (cols > 16384) return -2;
  const bool vec = dt == 1 && ln_vec_ok(cols, dy, x, gamma, dx, dx2, nullptr);
  int grid = ln_bwd_grid(rows, cols, vec);
  float *part = (dgamma || dbeta) ? partial : nullptr;
  if (vec) {
    int vpt = ln_vpt(cols), threads = cols / 8 / vpt;
    const bf16 *DY = (const bf16 *)dy, *X = (const bf16 *)x, *G = (const bf16 *)gamma;
    if (vpt == 1) vec::layernorm_bwd_vec_kernel<1><<<grid, threads, 0, st>>>(DY, X, G, mean, rstd, (bf16 *)dx, (bf16 *)dx2, part, rows, cols, accumulate_dx, accumulate_dx2);
    else if (vpt == 2) vec::layernorm_bwd_vec_kernel<2><<<grid, threads, 0, st>>>(DY, X, G, mean, rstd, (bf16 *)dx, (bf16 *)dx2, part, rows, cols, accumulate_dx, accumulate_dx2);
    else vec::layernorm_bwd_vec_kernel<4><<<grid, threads, 0, st>>>(DY, X, G, mean, rstd, (bf16 *)dx, (bf16 *)dx2, part, rows, cols, accumulate_dx, accumulate_dx2);
    if (part)
      vec::fold_partials_kernel<bf16><<<(cols + 31) / 32, dim3(32, 32), 0, st>>>(part, grid, cols, (bf16 *)dgamma, (bf16 *)dbeta, accumulate_params);
    return (int)cudaGetLastError();
  }
  DISPATCH_FLOAT(dt, {
    if (cols <= 512 * 4)
      layernorm_bwd_kernel<T, 4><<<grid, 512, 0, st>>>((const T *)dy, (const T *)x, (const T *)gamma, mean, rstd,
                                                        (T *)dx, (T *)dx2, part, rows, cols, accumulate_dx, accumulate_dx2);
    else if (cols <= 512 * 16)
      layernorm_bwd_kernel<T, 16><<<grid, 512, 0, st>>>((const T *)dy, (const T *)x, (const T *)gamma, mean, rstd,
                                                         (T *)dx, (T *)dx2, part, rows, cols, accumulate_dx, accumulate_dx2);
    else
      layernorm_bwd_kernel<T, 32><<<grid, 512, 0, st>>>((const T *)dy, (const T *)x, (const T *)gamma, mean, rstd,
                                                         (T *)dx, (T *)dx2, part, rows, cols, accumulate_dx, accumulate_dx2);
    if (part)
      vec::fold_partials_kernel<T><<<(cols + 31) / 32, dim3(32, 32), 0, st>>>(part, grid, cols, (T *)dgamma, (T *)dbeta, accumulate_params);
  });
  return (int)cudaGetLastError();
}

template <int VPT>
static void launch_softmax_fwd_warp(const void *x, void *y, void *yd, int rows, float scale, int causal_q, float p, unsigned long long salt,
                                    const unsigned long long *seed_ptr, cudaStream_t st) {
  int blocks = (rows + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  vec::softmax_fwd_warp_kernel<VPT><<<blocks, 256, 0, st>>>((const bf16 *)x, (bf16 *)y, (bf16 *)yd, rows, scale, causal_q, p, salt, seed_ptr);
}
template <int VPT>
static void launch_softmax_bwd_warp(const void *dy, const void *y, void *dx, int rows, float scale, float p, unsigned long long salt,
                                    const unsigned long long *seed_ptr, cudaStream_t st) {
  int blocks = (rows + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  vec::softmax_bwd_warp_kernel<VPT><<<blocks, 256, 0, st>>>((const bf16 *)dy, (const bf16 *)y, (bf16 *)dx, rows, scale, p, salt, seed_ptr);
}
static bool softmax_vec_ok(int cols, int dt, const void *a, const void *b, const void *c) {
  return dt == 1 && cols % 256 == 0 && cols <= 4096 && (cols / 256 == 1 || cols / 256 == 2 || cols / 256 == 4 || cols / 256 == 8 || cols / 256 == 16) &&
         aligned16(a) && aligned16(b) && aligned16(c);
}
// y = softmax(scale * x); yd (optional, bf16 rows of 256*k columns only) = dropout(y, p) with the mask
// hash(salt, *seed_ptr, element index).  Returns -3 when yd is requested for a shape the fused path cannot take.
FFK_API int ffk_softmax_dropout_fwd(const void *x, void *y, void *yd, int rows, int cols, float scale, int causal_q, float p,
                                    unsigned long long salt, const unsigned long long *seed_ptr, int dt, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (!softmax_vec_ok(cols, dt, x, y, yd)) return -3;
  switch (cols / 256) {
    case 1: launch_softmax_fwd_warp<1>(x, y, yd, rows, scale, causal_q, p, salt, seed_ptr, st); break;
    case 2: launch_softmax_fwd_warp<2>(x, y, yd, rows, scale, causal_q, p, salt, seed_ptr, st); break;
    case 4: launch_softmax_fwd_warp<4>(x, y, yd, rows, scale, causal_q, p, salt, seed_ptr, st); break;
    case 8: launch_softmax_fwd_warp<8>(x, y, yd, rows, scale, causal_q, p, salt, seed_ptr, st); break;
    default: launch_softmax_fwd_warp<16>(x, y, yd, rows, scale, causal_q, p, salt, seed_ptr, st); break;
  }
  return (int)cudaGetLastError();
}
// dx = scale * y * (g - sum(g*y)) with g = dropout_backward(dy) (p = 0: g = dy).  Same shape limits as above.
FFK_API int ffk_softmax_dropout_bwd(const void *dy, const void *y, void *dx, int rows, int cols, float scale, float p,
                                    unsigned long long salt, const unsigned long long *seed_ptr, int dt, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (!softmax_vec_ok(cols, dt, dy, y, dx)) return -3;
  switch (cols / 256) {
    case 1: launch_softmax_bwd_warp<1>(dy, y, dx, rows, scale, p, salt, seed_ptr, st); break;
    case 2: launch_softmax_bwd_warp<2>(dy, y, dx, rows, scale, p, salt, seed_ptr, st); break;
    case 4: launch_softmax_bwd_warp<4>(dy, y, dx, rows, scale, p, salt, seed_ptr, st); break;
    case 8: launch_softmax_bwd_warp<8>(dy, y, dx, rows, scale, p, salt, seed_ptr, st); break;
    default: launch_softmax_bwd_warp<16>(dy, y, dx, rows, scale, p, salt, seed_ptr, st); break;
  }
  return (int)cudaGetLastError();
}

FFK_API int ffk_softmax_fwd(const void *x, void *y, int rows, int cols, float scale, int causal_q, int dt,
                            cudaStream_t st) {
  if (rows <= 0) return 0;
  if (softmax_vec_ok(cols, dt, x, y, nullptr))
    return ffk_softmax_dropout_fwd(x, y, nullptr, rows, cols, scale, causal_q, 0.f, 0, nullptr, dt, st);
  int threads = cols >= 1024 ? 256 : 128;
  DISPATCH_FLOAT(dt, (softmax_fwd_kernel<T><<<rows < 148 * 16 ? rows : 148 * 16, threads, 0, st>>>(
                         (const T *)x, (T *)y, rows, cols, scale, causal_q)));
  return (int)cudaGetLastError();
}
FFK_API int ffk_softmax_bwd(const void *dy, const void *y, void *dx, int rows, int cols, float scale, int dt,
                            cudaStream_t st) {
  if (rows <= 0) return 0;
  if (softmax_vec_ok(cols, dt, dy, y, dx))
    return ffk_softmax_dropout_bwd(dy, y, dx, rows, cols, scale, 0.f, 0, nullptr, dt, st);
  int threads = cols >= 1024 ? 256 : 128;
  DISPATCH_FLOAT(dt, (softmax_bwd_kernel<T><<<rows < 148 * 16 ? rows : 148 * 16, threads, 0, st>>>(
                         (const T *)dy, (const T *)y, (T *)dx, rows, cols, scale)));
  return (int)cudaGetLastError();
}
// label_dt: 2 = int32, 3 = int64
FFK_API int ffk_softmax_ce(const void *logits, const void *labels, void *probs, void *dlogits, float *loss, int rows,
                           int cols, float grad_scale, int dt, int label_dt, cudaStream_t st) {
  if (rows <= 0) return 0;
  int threads = cols >= 4096 ? 1024 : 256;
  int grid = rows < 148 * 4 ? rows : 148 * 4;
  if (dt == 1 && cols % 8 == 0 && (((uintptr_t)logits | (uintptr_t)probs | (uintptr_t)dlogits) & 15) == 0) {
    int vthreads = cols >= 8192 ? 512 : 256;
    int vgrid = rows < 148 * 8 ? rows : 148 * 8;
    if (label_dt == 3)
      softmax_ce_vec_kernel<long long><<<vgrid, vthreads, 0, st>>>((const bf16 *)logits, (const long long *)labels, (bf16 *)probs,
                                                                   (bf16 *)dlogits, loss, rows, cols, grad_scale);
    else
      softmax_ce_vec_kernel<int><<<vgrid, vthreads, 0, st>>>((const bf16 *)logits, (const int *)labels, (bf16 *)probs, (bf16 *)dlogits, loss,
                                                             rows, cols, grad_scale);
    return (int)cudaGetLastError();
  }
  DISPATCH_FLOAT(dt, {
    if (label_dt == 3)
      softmax_ce_kernel<T, long long><<<grid, threads, 0, st>>>((const T *)logits, (const long long *)labels,
                                                                 (T *)probs, (T *)dlogits, loss, rows, cols, grad_scale);
    else
      softmax_ce_kernel<T, int><<<grid, threads, 0, st>>>((const T *)logits, (const int *)labels, (T *)probs,
                                                           (T *)dlogits, loss, rows, cols, grad_scale);
  });
  return (int)cudaGetLastError();
}
FFK_API int ffk_loss_bwd(int kind, const void *pred, const void *target, void *dpred, long long rows, int cols,
                         float scale, int dt, int label_dt, cudaStream_t st) {
  if (rows <= 0) return 0;
  DISPATCH_FLOAT(dt, {
    if (label_dt == 3)
      loss_bwd_kernel<T, long long><<<ffk_blocks(rows * cols, 256), 256, 0, st>>>(kind, (const T *)pred, target,
                                                                                   (T *)dpred, rows, cols, scale);
    else
      loss_bwd_kernel<T, int><<<ffk_blocks(rows * cols, 256), 256, 0, st>>>(kind, (const T *)pred, target, (T *)dpred,
                                                                             rows, cols, scale);
  });
  return (int)cudaGetLastError();
}
FFK_API int ffk_loss_fwd(int kind, const void *pred, const void *target, float *loss, int rows, int cols, int dt,
                         int label_dt, cudaStream_t st) {
  if (rows <= 0) return 0;
  DISPATCH_FLOAT(dt, {
    if (label_dt == 3)
      loss_fwd_kernel<T, long long><<<rows < 2368 ? rows : 2368, 128, 0, st>>>(kind, (const T *)pred, target, loss,
                                                                                rows, cols);
    else
      loss_fwd_kernel<T, int><<<rows < 2368 ? rows : 2368, 128, 0, st>>>(kind, (const T *)pred, target, loss, rows,
                                                                          cols);
  });
  return (int)cudaGetLastError();
}
