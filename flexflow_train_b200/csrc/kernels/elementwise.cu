// elementwise.cu -- bandwidth-bound pointwise kernels (128-bit vector accesses).
//
// Covers the reference's element_unary / element_binary / dropout / cast /
// helper kernels (lib/kernels/src/cuda/ops/element_unary_kernels.cu:104-310,
// element_binary_kernels.cu:27-412, dropout_kernels.cu:73-89, cast_kernels.cu:25-32,
// cuda_helper.cu:145-195) without any cuDNN call.
#include "common.cuh"
#include "rowwise_vec.cuh"

namespace {

// dtype codes used across the C API
enum { DT_F32 = 0, DT_BF16 = 1, DT_I32 = 2, DT_I64 = 3, DT_F16 = 4, DT_BOOL = 5, DT_F64 = 6 };

enum UnaryOp {
  U_IDENTITY = 0, U_RELU, U_SIGMOID, U_TANH, U_ELU, U_GELU, U_EXP, U_RSQRT, U_SIN, U_COS,
  U_SCALAR_MUL, U_SCALAR_ADD, U_SCALAR_SUB, U_SCALAR_TRUEDIV, U_POW, U_LOG, U_SQRT, U_NEG
};
enum BinaryOp { B_ADD = 0, B_SUB, B_MUL, B_DIV, B_MAX, B_MIN };

__device__ __forceinline__ float unary_apply(int op, float x, float s) {
  switch (op) {
    case U_RELU: return x > 0.f ? x : 0.f;
    case U_SIGMOID: return 1.f / (1.f + __expf(-x));
    case U_TANH: return tanhf(x);
    case U_ELU: return x > 0.f ? x : (__expf(x) - 1.f);
    case U_GELU: return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
    case U_EXP: return __expf(x);
    case U_RSQRT: return rsqrtf(x);
    case U_SIN: return sinf(x);
    case U_COS: return cosf(x);
    case U_SCALAR_MUL: return x * s;
    case U_SCALAR_ADD: return x + s;
    case U_SCALAR_SUB: return x - s;
    case U_SCALAR_TRUEDIV: return x / s;
    case U_POW: return powf(x, s);
    case U_LOG: return __logf(x);
    case U_SQRT: return sqrtf(x);
    case U_NEG: return -x;
    default: return x;
  }
}
// d(out)/d(in) given input x and output y
__device__ __forceinline__ float unary_grad(int op, float x, float y, float s) {
  switch (op) {
    case U_RELU: return x > 0.f ? 1.f : 0.f;
    case U_SIGMOID: return y * (1.f - y);
    case U_TANH: return 1.f - y * y;
    case U_ELU: return x > 0.f ? 1.f : y + 1.f;
    case U_GELU: {
      float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
      return cdf + x * 0.3989422804014327f * __expf(-0.5f * x * x);
    }
    case U_EXP: return y;
    case U_RSQRT: return -0.5f * y / x;
    case U_SIN: return cosf(x);
    case U_COS: return -sinf(x);
    case U_SCALAR_MUL: return s;
    case U_SCALAR_ADD: return 1.f;
    case U_SCALAR_SUB: return 1.f;
    case U_SCALAR_TRUEDIV: return 1.f / s;
    case U_POW: return s * powf(x, s - 1.f);
    case U_LOG: return 1.f / x;
    case U_SQRT: return 0.5f / y;
    case U_NEG: return -1.f;
    default: return 1.f;
  }
}

// 16-byte vector of T viewed as floats
template <typename T> struct V16;
template <> struct V16<float> {
  static constexpr int N = 4;
  __device__ static void load(const float *p, float *v) {
    float4 t = *reinterpret_cast<const float4 *>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  __device__ static void store(float *p, const float *v) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
  __device__ static float ld1(const float *p) { return *p; }
  __device__ static void st1(float *p, float v) { *p = v; }
};
template <> struct V16<bf16> {
  static constexpr int N = 8;
  __device__ static void load(const bf16 *p, float *v) {
    uint4 u = *reinterpret_cast<const uint4 *>(p);
    float2 a = unpack_bf162(u.x), b = unpack_bf162(u.y), c = unpack_bf162(u.z), d = unpack_bf162(u.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
  __device__ static void store(bf16 *p, const float *v) {
    *reinterpret_cast<uint4 *>(p) = make_uint4(pack_bf162(v[0], v[1]), pack_bf162(v[2], v[3]),
                                               pack_bf162(v[4], v[5]), pack_bf162(v[6], v[7]));
  }
  __device__ static float ld1(const bf16 *p) { return bf2f(*p); }
  __device__ static void st1(bf16 *p, float v) { *p = f2bf(v); }
};

template <typename T>
__global__ void unary_fwd_kernel(int op, const T *__restrict__ x, T *__restrict__ y, long long n, float s) {
  constexpr int N = V16<T>::N;
  long long nv = n / N;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    float v[N];
    V16<T>::load(x + i * N, v);
#pragma unroll
    for (int j = 0; j < N; ++j) v[j] = unary_apply(op, v[j], s);
    V16<T>::store(y + i * N, v);
  }
  for (long long i = nv * N + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    V16<T>::st1(y + i, unary_apply(op, V16<T>::ld1(x + i), s));
}

template <typename T>
__global__ void unary_bwd_kernel(int op, const T *__restrict__ x, const T *__restrict__ y, const T *__restrict__ dy,
                                 T *__restrict__ dx, long long n, float s, int accumulate) {
  constexpr int N = V16<T>::N;
  long long nv = n / N;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    float vx[N], vy[N], vd[N], vo[N];
    V16<T>::load(x + i * N, vx);
    V16<T>::load(y + i * N, vy);
    V16<T>::load(dy + i * N, vd);
    if (accumulate) V16<T>::load(dx + i * N, vo);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      float g = vd[j] * unary_grad(op, vx[j], vy[j], s);
      vo[j] = accumulate ? vo[j] + g : g;
    }
    V16<T>::store(dx + i * N, vo);
  }
  for (long long i = nv * N + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float g = V16<T>::ld1(dy + i) * unary_grad(op, V16<T>::ld1(x + i), V16<T>::ld1(y + i), s);
    V16<T>::st1(dx + i, accumulate ? V16<T>::ld1(dx + i) + g : g);
  }
}

__device__ __forceinline__ float binary_apply(int op, float a, float b) {
  switch (op) {
    case B_ADD: return a + b;
    case B_SUB: return a - b;
    case B_MUL: return a * b;
    case B_DIV: return a / b;
    case B_MAX: return fmaxf(a, b);
    default: return fminf(a, b);
  }
}

// y[i] = a[i] (op) b[i % bn] ; bn == n for same-shape operands, bn == trailing
// extent for a row-vector broadcast, bn == 1 for a scalar operand.
template <typename T>
__global__ void binary_fwd_kernel(int op, const T *__restrict__ a, const T *__restrict__ b, T *__restrict__ y,
                                  long long n, long long bn) {
  constexpr int N = V16<T>::N;
  long long stride = (long long)gridDim.x * blockDim.x;
  if (bn == n) {
    long long nv = n / N;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
      float va[N], vb[N];
      V16<T>::load(a + i * N, va);
      V16<T>::load(b + i * N, vb);
#pragma unroll
      for (int j = 0; j < N; ++j) va[j] = binary_apply(op, va[j], vb[j]);
      V16<T>::store(y + i * N, va);
    }
    for (long long i = nv * N + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
      V16<T>::st1(y + i, binary_apply(op, V16<T>::ld1(a + i), V16<T>::ld1(b + i)));
  } else {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
      V16<T>::st1(y + i, binary_apply(op, V16<T>::ld1(a + i), V16<T>::ld1(b + (i % bn))));
  }
}

// Same-shape backward.  da/db may be null; accumulate adds into them.
template <typename T>
__global__ void binary_bwd_kernel(int op, const T *__restrict__ a, const T *__restrict__ b, const T *__restrict__ dy,
                                  T *da, T *db, long long n, int accumulate) {
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float g = V16<T>::ld1(dy + i);
    float av = (op >= B_MUL) ? V16<T>::ld1(a + i) : 0.f, bv = (op >= B_MUL) ? V16<T>::ld1(b + i) : 0.f;
    float ga, gb;
    switch (op) {
      case B_ADD: ga = g; gb = g; break;
      case B_SUB: ga = g; gb = -g; break;
      case B_MUL: ga = g * bv; gb = g * av; break;
      case B_DIV: ga = g / bv; gb = -g * av / (bv * bv); break;
      case B_MAX: ga = av >= bv ? g : 0.f; gb = av >= bv ? 0.f : g; break;
      default: ga = av <= bv ? g : 0.f; gb = av <= bv ? 0.f : g; break;
    }
    if (da) V16<T>::st1(da + i, accumulate ? V16<T>::ld1(da + i) + ga : ga);
    if (db) V16<T>::st1(db + i, accumulate ? V16<T>::ld1(db + i) + gb : gb);
  }
}

// y = dropout(x) [+ r]; the keep mask is a pure function of (seed, index).
template <typename T>
__global__ void dropout_kernel(const T *__restrict__ x, const T *__restrict__ r, T *__restrict__ y, long long n,
                               float p, float scale, unsigned long long seed, const unsigned long long *seed_ptr) {
  // seed_ptr (optional) points at a per-step seed in device memory, so a captured CUDA graph draws a new
  // mask on every replay; `seed` then acts as the per-operator salt.
  if (seed_ptr) seed = seed * 0x9E3779B97F4A7C15ull + *seed_ptr;
  constexpr int N = V16<T>::N;
  long long nv = n / N;
  long long stride = (long long)gridDim.x * blockDim.x;
  const uint32_t thr = ffk_drop_threshold(p);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    float v[N], rv[N];
    V16<T>::load(x + i * N, v);
    if (r) V16<T>::load(r + i * N, rv);
#pragma unroll
    for (int g4 = 0; g4 < N / 4; ++g4) {
      uint32_t keep = ffk_keep4(seed, (unsigned long long)(i * (N / 4) + g4), thr);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[g4 * 4 + j] = ((keep >> j) & 1u ? v[g4 * 4 + j] * scale : 0.f) + (r ? rv[g4 * 4 + j] : 0.f);
    }
    V16<T>::store(y + i * N, v);
  }
  for (long long i = nv * N + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float keep = ffk_keep(seed, (unsigned long long)i, thr) ? scale : 0.f;
    V16<T>::st1(y + i, V16<T>::ld1(x + i) * keep + (r ? V16<T>::ld1(r + i) : 0.f));
  }
}

template <typename T>
__global__ void axpby_kernel(const T *__restrict__ x, T *__restrict__ y, long long n, float a, float b) {
  constexpr int N = V16<T>::N;
  long long nv = n / N;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    float vx[N], vy[N];
    V16<T>::load(x + i * N, vx);
    if (b != 0.f) V16<T>::load(y + i * N, vy);
#pragma unroll
    for (int j = 0; j < N; ++j) vy[j] = a * vx[j] + (b != 0.f ? b * vy[j] : 0.f);
    V16<T>::store(y + i * N, vy);
  }
  for (long long i = nv * N + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    V16<T>::st1(y + i, a * V16<T>::ld1(x + i) + (b != 0.f ? b * V16<T>::ld1(y + i) : 0.f));
}

template <typename T>
__global__ void fill_kernel(T *y, long long n, float v) {
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) V16<T>::st1(y + i, v);
}


__device__ __forceinline__ double load_any(const void *p, long long i, int dt) {
  switch (dt) {
    case DT_F32: return ((const float *)p)[i];
    case DT_BF16: return bf2f(((const bf16 *)p)[i]);
    case DT_I32: return ((const int *)p)[i];
    case DT_I64: return (double)((const long long *)p)[i];
    case DT_F16: return __half2float(((const __half *)p)[i]);
    case DT_BOOL: return ((const unsigned char *)p)[i] ? 1.0 : 0.0;
    default: return ((const double *)p)[i];
  }
}
__device__ __forceinline__ void store_any(void *p, long long i, int dt, double v) {
  switch (dt) {
    case DT_F32: ((float *)p)[i] = (float)v; break;
    case DT_BF16: ((bf16 *)p)[i] = f2bf((float)v); break;
    case DT_I32: ((int *)p)[i] = (int)v; break;
    case DT_I64: ((long long *)p)[i] = (long long)v; break;
    case DT_F16: ((__half *)p)[i] = __float2half((float)v); break;
    case DT_BOOL: ((unsigned char *)p)[i] = v != 0.0; break;
    default: ((double *)p)[i] = v; break;
  }
}
// dst = cast(src)  (accumulate: dst += cast(src), the backward of a cast)
__global__ void cast_kernel(const void *src, int sdt, void *dst, int ddt, long long n, int accumulate) {
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    double v = load_any(src, i, sdt);
    if (accumulate) v += load_any(dst, i, ddt);
    store_any(dst, i, ddt, v);
  }
}
// fast paths for the two casts on the training hot path
__global__ void cast_f32_bf16_kernel(const float *__restrict__ s, bf16 *__restrict__ d, long long n) {
  long long nv = n / 8, stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    float4 a = *reinterpret_cast<const float4 *>(s + i * 8), b = *reinterpret_cast<const float4 *>(s + i * 8 + 4);
    *reinterpret_cast<uint4 *>(d + i * 8) =
        make_uint4(pack_bf162(a.x, a.y), pack_bf162(a.z, a.w), pack_bf162(b.x, b.y), pack_bf162(b.z, b.w));
  }
  for (long long i = nv * 8 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) d[i] = f2bf(s[i]);
}

// dz = dy * act'(saved) ; per-column partial sums of dz go to `partial`
// ([gridDim.y, cols] floats) for the bias gradient.  One block handles a
// 32-column strip over a slab of rows.
template <typename T>
__global__ void bias_act_bwd_kernel(const T *__restrict__ dy, const T *__restrict__ saved, T *__restrict__ dz,
                                    float *__restrict__ partial, int rows, int cols, int act) {
  __shared__ float red[8][33];
  int col = blockIdx.x * 32 + threadIdx.x;  // blockDim = (32, 8)
  float acc = 0.f;
  if (col < cols) {
    for (int r = blockIdx.y * blockDim.y + threadIdx.y; r < rows; r += gridDim.y * blockDim.y) {
      long long i = (long long)r * cols + col;
      float g = V16<T>::ld1(dy + i);
      if (act != ACT_NONE) g *= act_bwd(V16<T>::ld1(saved + i), act);
      if (dz) V16<T>::st1(dz + i, g);
      acc += g;
    }
  }
  red[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && col < cols && partial) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) s += red[j][threadIdx.x];
    partial[(long long)blockIdx.y * cols + col] = s;
  }
}
template <typename T>
__global__ void colsum_finish_kernel(const float *__restrict__ partial, int nparts, int cols, T *out, int accumulate) {
  int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= cols) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partial[(long long)p * cols + col];
  V16<T>::st1(out + col, accumulate ? V16<T>::ld1(out + col) + s : s);
}

}  // namespace

#define DISPATCH_FLOAT(dt, ...)                                   \
  if ((dt) == DT_F32) { typedef float T; __VA_ARGS__; }           \
  else if ((dt) == DT_BF16) { typedef bf16 T; __VA_ARGS__; }      \
  else return -2;

FFK_API int ffk_unary_fwd(int op, const void *x, void *y, long long n, float s, int dt, cudaStream_t st) {
  if (n <= 0) return 0;
  DISPATCH_FLOAT(dt, (unary_fwd_kernel<T><<<ffk_blocks(n / V16<T>::N + 1, 256), 256, 0, st>>>(op, (const T *)x, (T *)y, n, s)));
  return (int)cudaGetLastError();
}
FFK_API int ffk_unary_bwd(int op, const void *x, const void *y, const void *dy, void *dx, long long n, float s, int dt,
                          int accumulate, cudaStream_t st) {
  if (n <= 0) return 0;
  DISPATCH_FLOAT(dt, (unary_bwd_kernel<T><<<ffk_blocks(n / V16<T>::N + 1, 256), 256, 0, st>>>(
                         op, (const T *)x, (const T *)y, (const T *)dy, (T *)dx, n, s, accumulate)));
  return (int)cudaGetLastError();
}
FFK_API int ffk_binary_fwd(int op, const void *a, const void *b, void *y, long long n, long long bn, int dt,
                           cudaStream_t st) {
  if (n <= 0) return 0;
  DISPATCH_FLOAT(dt, (binary_fwd_kernel<T><<<ffk_blocks(n / V16<T>::N + 1, 256), 256, 0, st>>>(
                         op, (const T *)a, (const T *)b, (T *)y, n, bn)));
  return (int)cudaGetLastError();
}
FFK_API int ffk_binary_bwd(int op, const void *a, const void *b, const void *dy, void *da, void *db, long long n,
                           int dt, int accumulate, cudaStream_t st) {
  if (n <= 0) return 0;
  DISPATCH_FLOAT(dt, (binary_bwd_kernel<T><<<ffk_blocks(n, 256), 256, 0, st>>>(op, (const T *)a, (const T *)b,
                                                                                (const T *)dy, (T *)da, (T *)db, n,
                                                                                accumulate)));
  return (int)cudaGetLastError();
}
// y = dropout(x, p; seed) + r   (r optional).  Backward is the same call on dy with r = null.
FFK_API int ffk_dropout(const void *x, const void *r, void *y, long long n, float p, unsigned long long seed,
                        const unsigned long long *seed_ptr, int dt, cudaStream_t st) {
  if (n <= 0) return 0;
  float scale = p < 1.f ? 1.f / (1.f - p) : 0.f;
  DISPATCH_FLOAT(dt, (dropout_kernel<T><<<ffk_blocks(n / V16<T>::N + 1, 256), 256, 0, st>>>(
                         (const T *)x, (const T *)r, (T *)y, n, p, scale, seed, seed_ptr)));
  return (int)cudaGetLastError();
}
// y = a*x + b*y
FFK_API int ffk_axpby(const void *x, void *y, long long n, float a, float b, int dt, cudaStream_t st) {
  if (n <= 0) return 0;
  DISPATCH_FLOAT(dt, (axpby_kernel<T><<<ffk_blocks(n / V16<T>::N + 1, 256), 256, 0, st>>>((const T *)x, (T *)y, n, a, b)));
  return (int)cudaGetLastError();
}
FFK_API int ffk_fill(void *y, long long n, float v, int dt, cudaStream_t st) {
  if (n <= 0) return 0;
  DISPATCH_FLOAT(dt, (fill_kernel<T><<<ffk_blocks(n, 256), 256, 0, st>>>((T *)y, n, v)));
  return (int)cudaGetLastError();
}
FFK_API int ffk_cast(const void *src, int sdt, void *dst, int ddt, long long n, int accumulate, cudaStream_t st) {
  if (n <= 0) return 0;
  if (sdt == DT_F32 && ddt == DT_BF16 && !accumulate && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0)
    cast_f32_bf16_kernel<<<ffk_blocks(n / 8 + 1, 256), 256, 0, st>>>((const float *)src, (bf16 *)dst, n);
  else
    cast_kernel<<<ffk_blocks(n, 256), 256, 0, st>>>(src, sdt, dst, ddt, n, accumulate);
  return (int)cudaGetLastError();
}
// Number of float slots `partial` must hold for ffk_bias_act_bwd.
// Row chunks of the column reduction: at least 64 rows each, and enough chunks that a narrow matrix (768 columns =
// three column blocks) still fills the GPU.
static int bias_act_row_chunks(int rows, int cols) {
  const int col_blocks = (cols + 255) / 256;
  int cap = (148 * 4 + col_blocks - 1) / col_blocks;
  if (cap < 64) cap = 64;
  int gy = rows / 64;
  if (gy < 1) gy = 1;
  if (gy > cap) gy = cap;
  return gy;
}
FFK_API long long ffk_bias_act_bwd_scratch(int rows, int cols) { return (long long)bias_act_row_chunks(rows, cols) * cols; }
// dz = dy * act'(saved); dbias (+)= column sums of dz.  dz may alias dy or be null
// (bias gradient only); dbias may be null.  `partial` is caller-provided scratch.
static int bias_act_bwd_impl(const void *dy, const void *saved, void *dz, void *dbias, float *partial, int rows, int cols, int act, int dt,
                             int accumulate, float drop_p, unsigned long long drop_salt, const void *drop_seed_ptr, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return 0;
  const int gy = bias_act_row_chunks(rows, cols);
  if (dt == DT_BF16 && cols % 8 == 0 && (((uintptr_t)dy | (uintptr_t)saved | (uintptr_t)dz) & 15) == 0) {
    dim3 vgrid((cols + 255) / 256, gy), vblock(32, 8);
    vec::bias_act_bwd_vec_kernel<<<vgrid, vblock, 0, st>>>((const bf16 *)dy, (const bf16 *)saved, (bf16 *)dz, dbias ? partial : nullptr, rows,
                                                          cols, act, drop_p, drop_salt, (const unsigned long long *)drop_seed_ptr);
    if (dbias) vec::fold_partials_kernel<bf16><<<(cols + 31) / 32, dim3(32, 32), 0, st>>>(partial, gy, cols, (bf16 *)dbias, (bf16 *)nullptr, accumulate);
    return (int)cudaGetLastError();
  }
  if (drop_p > 0.f) return -2;  // the fused-dropout form exists for the 16-byte vector path only
  dim3 grid((cols + 31) / 32, gy), block(32, 8);
  DISPATCH_FLOAT(dt, {
    bias_act_bwd_kernel<T><<<grid, block, 0, st>>>((const T *)dy, (const T *)saved, (T *)dz, dbias ? partial : nullptr,
                                                    rows, cols, act);
    if (dbias) colsum_finish_kernel<T><<<(cols + 255) / 256, 256, 0, st>>>(partial, gy, cols, (T *)dbias, accumulate);
  });
  return (int)cudaGetLastError();
}
FFK_API int ffk_bias_act_bwd(const void *dy, const void *saved, void *dz, void *dbias, float *partial, int rows,
                             int cols, int act, int dt, int accumulate, cudaStream_t st) {
  return bias_act_bwd_impl(dy, saved, dz, dbias, partial, rows, cols, act, dt, accumulate, 0.f, 0ull, nullptr, st);
}
// Same, with the gradient first taken back through a dropout applied after the activation (bf16, cols % 8 == 0).
FFK_API int ffk_bias_act_dropout_bwd(const void *dy, const void *saved, void *dz, void *dbias, float *partial, int rows, int cols, int act,
                                     int dt, int accumulate, float drop_p, unsigned long long drop_salt, const void *drop_seed_ptr,
                                     cudaStream_t st) {
  return bias_act_bwd_impl(dy, saved, dz, dbias, partial, rows, cols, act, dt, accumulate, drop_p, drop_salt, drop_seed_ptr, st);
}
