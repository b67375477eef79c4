// tensor_ops.cu -- data-movement operators: permute / transpose, strided block copy (concat, split),
// axis reductions, gather, top-k, reverse, broadcast.
//
// Counterparts in the reference: transpose_kernels.cu:34 (index-math permute), concat_kernels.cu:50-82 and
// split_kernels.cu:33-51 (copy_with_stride / add_with_stride), reduce_kernels.cu:59-97 (cudnnReduceTensor),
// gather_kernels.cu:25-52, topk_kernels.cu:337-404, reverse_kernels.cu:22.  All element sizes are handled by
// moving raw 2-, 4- or 8-byte words; arithmetic kernels take fp32 or bf16.
#include "common.cuh"

namespace {

constexpr int MAXD = 6;
struct Dims {
  int n;
  long long size[MAXD];
  long long stride[MAXD];  // stride of the *source* for each *destination* dim
};

template <typename W>
__global__ void permute_kernel(const W *__restrict__ src, W *__restrict__ dst, Dims d, long long total, int accumulate_f32,
                               int accumulate_bf16) {
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long rem = i, off = 0;
#pragma unroll
    for (int k = MAXD - 1; k >= 0; --k) {
      if (k < d.n) {
        long long c = rem % d.size[k];
        rem /= d.size[k];
        off += c * d.stride[k];
      }
    }
    if (accumulate_f32) ((float *)dst)[i] += ((const float *)src)[off];
    else if (accumulate_bf16) ((bf16 *)dst)[i] = f2bf(bf2f(((bf16 *)dst)[i]) + bf2f(((const bf16 *)src)[off]));
    else dst[i] = src[off];
  }
}

// dst[b][c][r] = src[b][r][c], 32x32 tiles through shared memory
template <typename W>
__global__ void transpose2d_kernel(const W *__restrict__ src, W *__restrict__ dst, int rows, int cols) {
  __shared__ W tile[32][33];
  long long base = (long long)blockIdx.z * rows * cols;
  int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = src[base + (long long)r * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) dst[base + (long long)c * rows + r] = tile[threadIdx.x][j];
  }
}

// Copy (or add) a [outer, block] region between tensors whose rows are `src_ld` / `dst_ld` elements apart:
// concat writes each input into its slot of the output row, split reads it back.
template <typename T>
__global__ void block_copy_kernel(const T *__restrict__ src, long long src_ld, T *__restrict__ dst, long long dst_ld,
                                  long long outer, long long block, int accumulate) {
  long long total = outer * block;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long o = i / block, b = i - o * block;
    T v = src[o * src_ld + b];
    T *p = dst + o * dst_ld + b;
    if (accumulate) *p = (T)((float)*p + (float)v);
    else *p = v;
  }
}

// 16-byte form of the same copy: block, both pitches and both bases are multiples of 16 bytes and there are fewer
// than 2^31 pieces, so the row / column split is a multiply-high instead of a 64-bit division per 2-byte element
// (channel concatenation of channels-last activations is this case).
struct CopyDiv {
  unsigned d, mul, sh;
};
__global__ void block_copy_vec_kernel(const uint4 *__restrict__ src, long long src_ld, uint4 *__restrict__ dst, long long dst_ld,
                                      unsigned total, CopyDiv f, int accumulate_bf16) {
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const unsigned o = f.d == 1 ? i : (__umulhi(i, f.mul) >> f.sh), b = i - o * f.d;
    uint4 v = src[(long long)o * src_ld + b];
    uint4 *p = dst + (long long)o * dst_ld + b;
    if (accumulate_bf16) {
      const uint4 w = *p;
      const unsigned *vs = reinterpret_cast<const unsigned *>(&v), *ws = reinterpret_cast<const unsigned *>(&w);
      unsigned r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 x = unpack_bf162(vs[j]), y = unpack_bf162(ws[j]);
        r[j] = pack_bf162(x.x + y.x, x.y + y.y);
      }
      v = make_uint4(r[0], r[1], r[2], r[3]);
    }
    *p = v;
  }
}

enum { RED_SUM = 0, RED_MEAN = 1, RED_MAX = 2, RED_MIN = 3, RED_PROD = 4 };
// x viewed as [outer, red, inner] -> y [outer, inner]
template <typename T>
__global__ void reduce_kernel(const T *__restrict__ x, T *__restrict__ y, long long outer, long long red, long long inner, int op) {
  long long total = outer * inner;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long o = i / inner, in = i - o * inner;
    const T *p = x + o * red * inner + in;
    float acc = (op == RED_MAX) ? -INFINITY : (op == RED_MIN) ? INFINITY : (op == RED_PROD) ? 1.f : 0.f;
    for (long long r = 0; r < red; ++r) {
      float v = (float)p[r * inner];
      acc = (op == RED_MAX) ? fmaxf(acc, v) : (op == RED_MIN) ? fminf(acc, v) : (op == RED_PROD) ? acc * v : acc + v;
    }
    if (op == RED_MEAN) acc /= (float)red;
    y[i] = (T)acc;
  }
}
// backward of sum / mean: dx[o, r, in] (+)= dy[o, in] * scale
template <typename T>
__global__ void reduce_bwd_kernel(const T *__restrict__ dy, T *__restrict__ dx, long long outer, long long red, long long inner,
                                  float scale, int accumulate) {
  long long total = outer * red * inner;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long in = i % inner, o = i / (red * inner);
    float g = (float)dy[o * inner + in] * scale;
    dx[i] = (T)(accumulate ? (float)dx[i] + g : g);
  }
}

// backward of max / min / prod over the middle dim: x, dx [o, r, in]; y, dy [o, in].
//   max, min: the gradient goes to every element equal to the result (each tie gets the whole gradient, as in
//             the derivative of amax/amin taken one-sided); prod: dx = dy * y / x (x == 0: product of the others
//             recomputed).
template <typename T>
__global__ void reduce_select_bwd_kernel(const T *__restrict__ x, const T *__restrict__ y, const T *__restrict__ dy, T *__restrict__ dx,
                                         long long outer, long long red, long long inner, int op, int accumulate) {
  long long total = outer * red * inner;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long in = i % inner, o = i / (red * inner);
    float xv = (float)x[i], yv = (float)y[o * inner + in], g = (float)dy[o * inner + in];
    float r;
    if (op == 4) {
      if (xv != 0.f) r = g * yv / xv;
      else {
        float others = 1.f;
        long long me = (i / inner) % red;
        for (long long j = 0; j < red; ++j)
          if (j != me) others *= (float)x[(o * red + j) * inner + in];
        r = g * others;
      }
    } else {
      r = (xv == yv) ? g : 0.f;
    }
    dx[i] = (T)(accumulate ? (float)dx[i] + r : r);
  }
}

// torch.gather along `dim`: x [outer, xd, inner], index/out [outer, id, inner]
template <typename T, typename I>
__global__ void gather_kernel(const T *__restrict__ x, const I *__restrict__ idx, T *__restrict__ y, long long outer, long long xd,
                              long long id, long long inner) {
  long long total = outer * id * inner;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long in = i % inner, o = i / (id * inner);
    long long j = (long long)idx[i];
    if (j >= 0 && j < xd) y[i] = x[(o * xd + j) * inner + in];
  }
}
template <typename I>
__global__ void gather_bwd_kernel(const float *__restrict__ dy_f, const bf16 *__restrict__ dy_b, const I *__restrict__ idx,
                                  float *dx_f, bf16 *dx_b, long long outer, long long xd, long long id, long long inner) {
  long long total = outer * id * inner;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long in = i % inner, o = i / (id * inner);
    long long j = (long long)idx[i];
    if (j < 0 || j >= xd) continue;
    long long t = (o * xd + j) * inner + in;
    if (dx_f) atomicAdd(dx_f + t, dy_f[i]);
    else atomicAdd(dx_b + t, dy_b[i]);
  }
}

// Top-k per row by repeated selection: one warp per row, k passes.  Rows of attention-sized tensors
// (<= a few thousand columns) and small k are the use case; the cost is O(k * cols / 32) per row.
template <typename T>
__global__ void topk_kernel(const T *__restrict__ x, T *__restrict__ vals, int *__restrict__ idxs, int rows, int cols, int k) {
  int warps_per_block = blockDim.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const T *p = x + (long long)row * cols;
    float last_v = INFINITY;
    int last_i = -1;
    for (int j = 0; j < k; ++j) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int c = lane; c < cols; c += 32) {
        float v = (float)p[c];
        // strictly after (last_v, last_i) in (value desc, index asc) order
        bool eligible = (v < last_v) || (v == last_v && c > last_i);
        if (eligible && (v > best || (v == best && c < bi))) { best = v; bi = c; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
      }
      if (lane == 0) {
        vals[(long long)row * k + j] = (T)best;
        idxs[(long long)row * k + j] = bi;
      }
      last_v = best;
      last_i = bi;
    }
  }
}
template <typename T>
__global__ void topk_bwd_kernel(const T *__restrict__ dvals, const int *__restrict__ idxs, T *__restrict__ dx, int rows, int cols, int k,
                                int accumulate) {
  long long total = (long long)rows * k;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long row = i / k;
    T *p = dx + row * cols + idxs[i];
    *p = (T)((accumulate ? (float)*p : 0.f) + (float)dvals[i]);
  }
}

// x [outer, n, inner] -> y[o, j, :] = x[o, n-1-j, :]
template <typename W>
__global__ void reverse_kernel(const W *__restrict__ x, W *__restrict__ y, long long outer, long long n, long long inner) {
  long long total = outer * n * inner;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long in = i % inner, j = (i / inner) % n, o = i / (n * inner);
    y[i] = x[(o * n + (n - 1 - j)) * inner + in];
  }
}

template <typename F>
int by_elem_size(int es, F &&f) {
  if (es == 2) return f((unsigned short *)nullptr);
  if (es == 4) return f((unsigned int *)nullptr);
  if (es == 8) return f((unsigned long long *)nullptr);
  if (es == 1) return f((unsigned char *)nullptr);
  return -2;
}

}  // namespace

// dst (contiguous, shape `sizes`) = permute of src: src_strides[k] is the element stride in src of dst dim k.
// accumulate: 0 = write, 1 = += in fp32, 2 = += in bf16 (backward of a transpose).
FFK_API int ffk_permute(const void *src, void *dst, int ndim, const long long *sizes, const long long *src_strides, int es,
                        int accumulate, cudaStream_t st) {
  if (ndim > MAXD || ndim < 1) return -2;
  Dims d;
  d.n = ndim;
  long long total = 1;
  for (int i = 0; i < ndim; ++i) { d.size[i] = sizes[i]; d.stride[i] = src_strides[i]; total *= sizes[i]; }
  if (total <= 0) return 0;
  int grid = ffk_blocks(total, 256);
  int r = by_elem_size(es, [&](auto *tag) {
    typedef typename std::remove_pointer<decltype(tag)>::type W;
    permute_kernel<W><<<grid, 256, 0, st>>>((const W *)src, (W *)dst, d, total, accumulate == 1, accumulate == 2);
    return 0;
  });
  return r ? r : (int)cudaGetLastError();
}
FFK_API int ffk_transpose2d(const void *src, void *dst, int batch, int rows, int cols, int es, cudaStream_t st) {
  if (batch <= 0 || rows <= 0 || cols <= 0) return 0;
  dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch), block(32, 8);
  int r = by_elem_size(es, [&](auto *tag) {
    typedef typename std::remove_pointer<decltype(tag)>::type W;
    transpose2d_kernel<W><<<grid, block, 0, st>>>((const W *)src, (W *)dst, rows, cols);
    return 0;
  });
  return r ? r : (int)cudaGetLastError();
}
// dt: 0 = fp32, 1 = bf16 (needed only when accumulate != 0; plain copies use the element size)
FFK_API int ffk_block_copy(const void *src, long long src_ld, void *dst, long long dst_ld, long long outer, long long block, int es,
                           int dt, int accumulate, cudaStream_t st) {
  if (outer * block <= 0) return 0;
  {
    const long long bytes = block * es, sp = src_ld * es, dp = dst_ld * es, pieces = outer * (bytes / 16);
    const bool vec = bytes % 16 == 0 && sp % 16 == 0 && dp % 16 == 0 && ((uintptr_t)src % 16) == 0 && ((uintptr_t)dst % 16) == 0 &&
                     pieces < (1ll << 31) && (!accumulate || dt == 1);
    if (vec) {
      CopyDiv f;
      const unsigned d = (unsigned)(bytes / 16);
      f.d = d; f.mul = 0; f.sh = 0;
      if (d > 1) {
        unsigned l = 0;
        while ((1ull << l) < d) ++l;
        f.mul = (unsigned)(((1ull << (31 + l)) + d - 1) / d);
        f.sh = l - 1;
      }
      block_copy_vec_kernel<<<ffk_blocks(pieces, 256), 256, 0, st>>>((const uint4 *)src, sp / 16, (uint4 *)dst, dp / 16, (unsigned)pieces, f,
                                                                     accumulate);
      return (int)cudaGetLastError();
    }
  }
  int grid = ffk_blocks(outer * block, 256);
  if (accumulate) {
    if (dt == 0) block_copy_kernel<float><<<grid, 256, 0, st>>>((const float *)src, src_ld, (float *)dst, dst_ld, outer, block, 1);
    else if (dt == 1) block_copy_kernel<bf16><<<grid, 256, 0, st>>>((const bf16 *)src, src_ld, (bf16 *)dst, dst_ld, outer, block, 1);
    else return -2;
    return (int)cudaGetLastError();
  }
  if (es == 2) block_copy_kernel<unsigned short><<<grid, 256, 0, st>>>((const unsigned short *)src, src_ld, (unsigned short *)dst, dst_ld, outer, block, 0);
  else if (es == 4) block_copy_kernel<float><<<grid, 256, 0, st>>>((const float *)src, src_ld, (float *)dst, dst_ld, outer, block, 0);
  else if (es == 8) block_copy_kernel<double><<<grid, 256, 0, st>>>((const double *)src, src_ld, (double *)dst, dst_ld, outer, block, 0);
  else if (es == 1) block_copy_kernel<unsigned char><<<grid, 256, 0, st>>>((const unsigned char *)src, src_ld, (unsigned char *)dst, dst_ld, outer, block, 0);
  else return -2;
  return (int)cudaGetLastError();
}
FFK_API int ffk_reduce(const void *x, void *y, long long outer, long long red, long long inner, int op, int dt, cudaStream_t st) {
  if (outer * inner <= 0) return 0;
  int grid = ffk_blocks(outer * inner, 256);
  if (dt == 0) reduce_kernel<float><<<grid, 256, 0, st>>>((const float *)x, (float *)y, outer, red, inner, op);
  else if (dt == 1) reduce_kernel<bf16><<<grid, 256, 0, st>>>((const bf16 *)x, (bf16 *)y, outer, red, inner, op);
  else return -2;
  return (int)cudaGetLastError();
}
FFK_API int ffk_reduce_bwd(const void *dy, void *dx, long long outer, long long red, long long inner, float scale, int dt,
                           int accumulate, cudaStream_t st) {
  if (outer * red * inner <= 0) return 0;
  int grid = ffk_blocks(outer * red * inner, 256);
  if (dt == 0) reduce_bwd_kernel<float><<<grid, 256, 0, st>>>((const float *)dy, (float *)dx, outer, red, inner, scale, accumulate);
  else if (dt == 1) reduce_bwd_kernel<bf16><<<grid, 256, 0, st>>>((const bf16 *)dy, (bf16 *)dx, outer, red, inner, scale, accumulate);
  else return -2;
  return (int)cudaGetLastError();
}
// op: 2 = max, 3 = min, 4 = prod (the codes of ffk_reduce)
FFK_API int ffk_reduce_select_bwd(const void *x, const void *y, const void *dy, void *dx, long long outer, long long red, long long inner,
                                  int op, int dt, int accumulate, cudaStream_t st) {
  if (outer * red * inner <= 0) return 0;
  if (op < 2 || op > 4) return -2;
  int grid = ffk_blocks(outer * red * inner, 256);
  if (dt == 0) reduce_select_bwd_kernel<float><<<grid, 256, 0, st>>>((const float *)x, (const float *)y, (const float *)dy, (float *)dx, outer, red, inner, op, accumulate);
  else if (dt == 1) reduce_select_bwd_kernel<bf16><<<grid, 256, 0, st>>>((const bf16 *)x, (const bf16 *)y, (const bf16 *)dy, (bf16 *)dx, outer, red, inner, op, accumulate);
  else return -2;
  return (int)cudaGetLastError();
}
FFK_API int ffk_gather(const void *x, const void *idx, void *y, long long outer, long long xd, long long id, long long inner, int es,
                       int idx_dt, cudaStream_t st) {
  if (outer * id * inner <= 0) return 0;
  int grid = ffk_blocks(outer * id * inner, 256);
  if (es == 4 && idx_dt == 3) gather_kernel<float, long long><<<grid, 256, 0, st>>>((const float *)x, (const long long *)idx, (float *)y, outer, xd, id, inner);
  else if (es == 4) gather_kernel<float, int><<<grid, 256, 0, st>>>((const float *)x, (const int *)idx, (float *)y, outer, xd, id, inner);
  else if (es == 2 && idx_dt == 3) gather_kernel<unsigned short, long long><<<grid, 256, 0, st>>>((const unsigned short *)x, (const long long *)idx, (unsigned short *)y, outer, xd, id, inner);
  else if (es == 2) gather_kernel<unsigned short, int><<<grid, 256, 0, st>>>((const unsigned short *)x, (const int *)idx, (unsigned short *)y, outer, xd, id, inner);
  else return -2;
  return (int)cudaGetLastError();
}
// dx += scatter(dy); the caller zeroes dx first when it must not accumulate
FFK_API int ffk_gather_bwd(const void *dy, const void *idx, void *dx, long long outer, long long xd, long long id, long long inner, int dt,
                           int idx_dt, cudaStream_t st) {
  if (outer * id * inner <= 0) return 0;
  int grid = ffk_blocks(outer * id * inner, 256);
  const float *dyf = dt == 0 ? (const float *)dy : nullptr;
  const bf16 *dyb = dt == 1 ? (const bf16 *)dy : nullptr;
  float *dxf = dt == 0 ? (float *)dx : nullptr;
  bf16 *dxb = dt == 1 ? (bf16 *)dx : nullptr;
  if (dt != 0 && dt != 1) return -2;
  if (idx_dt == 3) gather_bwd_kernel<long long><<<grid, 256, 0, st>>>(dyf, dyb, (const long long *)idx, dxf, dxb, outer, xd, id, inner);
  else gather_bwd_kernel<int><<<grid, 256, 0, st>>>(dyf, dyb, (const int *)idx, dxf, dxb, outer, xd, id, inner);
  return (int)cudaGetLastError();
}
FFK_API int ffk_topk(const void *x, void *vals, int *idxs, int rows, int cols, int k, int dt, cudaStream_t st) {
  if (rows <= 0) return 0;
  int grid = (rows + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  if (dt == 0) topk_kernel<float><<<grid, 256, 0, st>>>((const float *)x, (float *)vals, idxs, rows, cols, k);
  else if (dt == 1) topk_kernel<bf16><<<grid, 256, 0, st>>>((const bf16 *)x, (bf16 *)vals, idxs, rows, cols, k);
  else return -2;
  return (int)cudaGetLastError();
}
// dx must be zeroed by the caller unless accumulate
FFK_API int ffk_topk_bwd(const void *dvals, const int *idxs, void *dx, int rows, int cols, int k, int dt, int accumulate, cudaStream_t st) {
  if (rows <= 0) return 0;
  int grid = ffk_blocks((long long)rows * k, 256);
  if (dt == 0) topk_bwd_kernel<float><<<grid, 256, 0, st>>>((const float *)dvals, idxs, (float *)dx, rows, cols, k, accumulate);
  else if (dt == 1) topk_bwd_kernel<bf16><<<grid, 256, 0, st>>>((const bf16 *)dvals, idxs, (bf16 *)dx, rows, cols, k, accumulate);
  else return -2;
  return (int)cudaGetLastError();
}
FFK_API int ffk_reverse(const void *x, void *y, long long outer, long long n, long long inner, int es, cudaStream_t st) {
  if (outer * n * inner <= 0) return 0;
  int grid = ffk_blocks(outer * n * inner, 256);
  int r = by_elem_size(es, [&](auto *tag) {
    typedef typename std::remove_pointer<decltype(tag)>::type W;
    reverse_kernel<W><<<grid, 256, 0, st>>>((const W *)x, (W *)y, outer, n, inner);
    return 0;
  });
  return r ? r : (int)cudaGetLastError();
}
