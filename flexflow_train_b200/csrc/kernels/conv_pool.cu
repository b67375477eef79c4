// Convolution support kernels, pooling and batch normalisation for channels-last activations.
//
// Convolutions run as implicit-layout GEMMs on the tcgen05 GEMM of this library: activations are kept
// channels-last ([N, H, W, C]) so that a 1x1 convolution *is* the GEMM [N*H*W, C] x [OC, C]^T with no data
// movement, and a KxK convolution needs one im2col pass into a K-major bf16 matrix [N*OH*OW, KH*KW*C]
// (k = (kh*KW + kw)*C + c, padded with zero columns to a multiple of 8 so every row starts on 16 bytes for TMA).
// Bias and activation are applied by the GEMM epilogue.  Backward is two more GEMMs (dW = dY^T col,
// dcol = dY W) followed by the gather-form col2im below (no atomics).
//
// The reference does these with cuDNN (lib/kernels/src/cuda/ops/conv_2d_kernels.cu, pool_2d_kernels.cu,
// batch_norm_kernels.cu); here they are plain kernels written for HBM bandwidth: every pass is coalesced over
// the channel dimension.
#include "common.cuh"

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T *p);
template <> __device__ __forceinline__ float ldf<float>(const float *p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16 *p) { return bf2f(*p); }
template <typename T> __device__ __forceinline__ void stf(T *p, float v);
template <> __device__ __forceinline__ void stf<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16 *p, float v) { *p = f2bf(v); }

// Division by a runtime constant as multiply-high + shift (numerators below 2^31).  The window kernels decompose a
// flat index into (n, h, w, kernel tap, channel group) for every 16 bytes they move; with hardware 64-bit divisions
// that index arithmetic, not memory, bounded them.
struct FastDiv {
  unsigned d, mul, sh;
};
__device__ __forceinline__ unsigned fdiv(unsigned n, const FastDiv &f) { return f.d == 1 ? n : (__umulhi(n, f.mul) >> f.sh); }
__device__ __forceinline__ void fdivmod(unsigned n, const FastDiv &f, unsigned &q, unsigned &r) {
  q = fdiv(n, f);
  r = n - q * f.d;
}

struct ConvGeom {
  int N, C, H, W, KH, KW, SH, SW, PH, PW, OH, OW, Kp;
  long long sn, sc, sh, sw;  // element strides of the activation tensor
  FastDiv f_c8, f_kk, f_kw, f_ow, f_oh, f_w, f_h, f_sh, f_sw, f_kp, f_c;
};
// flat index -> (c8, a, b, n) where the index runs over [n][b_extent... ] as n, B, A, c8 from slow to fast
__device__ __forceinline__ void split3(long long t, const FastDiv &f_c8, const FastDiv &f_a, const FastDiv &f_b, bool small, int c8n, int A,
                                       int B, int &c8, int &a, int &b, int &n) {
  if (small) {
    unsigned r, r2, uc, ua, ub;
    fdivmod((unsigned)t, f_c8, r, uc);
    fdivmod(r, f_a, r2, ua);
    unsigned un;
    fdivmod(r2, f_b, un, ub);
    c8 = (int)uc; a = (int)ua; b = (int)ub; n = (int)un;
  } else {
    c8 = (int)(t % c8n);
    long long r = t / c8n;
    a = (int)(r % A);
    long long r2 = r / A;
    b = (int)(r2 % B);
    n = (int)(r2 / B);
  }
}

// ------------------------------------------------------------------------------------------- im2col
// vector path: bf16 channels-last, C % 8 == 0; one thread moves 8 channels (16 bytes)
__global__ void im2col_vec_kernel(const bf16 *__restrict__ x, bf16 *__restrict__ col, ConvGeom g, long long total) {
  const int c8n = g.C >> 3, kk_n = g.KH * g.KW;
  const bool small = total < (1ll << 31);
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    int c8, kk, ow, oh, n, kh, kw;
    long long row;
    if (small) {
      unsigned r, uc, uk, urow, r2, uow, uoh, un, ukh;
      fdivmod((unsigned)t, g.f_c8, r, uc);
      fdivmod(r, g.f_kk, urow, uk);
      fdivmod(urow, g.f_ow, r2, uow);
      fdivmod(r2, g.f_oh, un, uoh);
      ukh = fdiv(uk, g.f_kw);
      c8 = (int)uc; kk = (int)uk; row = urow; ow = (int)uow; oh = (int)uoh; n = (int)un; kh = (int)ukh; kw = kk - kh * g.KW;
    } else {
      c8 = (int)(t % c8n);
      long long r = t / c8n;
      kk = (int)(r % kk_n);
      row = r / kk_n;
      ow = (int)(row % g.OW);
      long long r2 = row / g.OW;
      oh = (int)(r2 % g.OH);
      n = (int)(r2 / g.OH);
      kh = kk / g.KW;
      kw = kk - kh * g.KW;
    }
    int ih = oh * g.SH - g.PH + kh, iw = ow * g.SW - g.PW + kw;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W)
      v = *reinterpret_cast<const uint4 *>(x + n * g.sn + ih * g.sh + iw * g.sw + c8 * 8);
    *reinterpret_cast<uint4 *>(col + row * g.Kp + (long long)kk * g.C + c8 * 8) = v;
  }
}
// generic path: any strides / dtype; one thread per (row, k) including the zero padding columns
template <typename T>
__global__ void im2col_kernel(const T *__restrict__ x, bf16 *__restrict__ col, ConvGeom g, long long total) {
  const int K = g.KH * g.KW * g.C;
  const bool small = total < (1ll << 31);
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    int k;
    long long row;
    if (small) {
      unsigned urow, uk;
      fdivmod((unsigned)t, g.f_kp, urow, uk);
      k = (int)uk; row = urow;
    } else {
      k = (int)(t % g.Kp);
      row = t / g.Kp;
    }
    float v = 0.f;
    if (k < K) {
      int kk, c, kh, kw, ow, oh, n;
      if (small) {
        unsigned ukk, uc, ukh, r2, uow, un, uoh;
        fdivmod((unsigned)k, g.f_c, ukk, uc);
        ukh = fdiv(ukk, g.f_kw);
        fdivmod((unsigned)row, g.f_ow, r2, uow);
        fdivmod(r2, g.f_oh, un, uoh);
        kk = (int)ukk; c = (int)uc; kh = (int)ukh; kw = kk - kh * g.KW; ow = (int)uow; oh = (int)uoh; n = (int)un;
      } else {
        kk = k / g.C; c = k - kk * g.C;
        kh = kk / g.KW; kw = kk - kh * g.KW;
        ow = (int)(row % g.OW);
        long long r2 = row / g.OW;
        oh = (int)(r2 % g.OH);
        n = (int)(r2 / g.OH);
      }
      int ih = oh * g.SH - g.PH + kh, iw = ow * g.SW - g.PW + kw;
      if (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) v = ldf(x + n * g.sn + c * g.sc + ih * g.sh + iw * g.sw);
    }
    col[t] = f2bf(v);
  }
}

// ------------------------------------------------------------------------------------------- col2im (gather form)
// dx[n, ih, iw, c] (+)= sum over (kh, kw) with (ih + PH - kh) % SH == 0 ... of dcol[(n, oh, ow), (kh, kw, c)]
template <typename T>
__global__ void col2im_kernel(const bf16 *__restrict__ dcol, T *__restrict__ dx, ConvGeom g, long long total, int accumulate) {
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    int c = (int)(t % g.C);
    long long r = t / g.C;
    int iw = (int)(r % g.W);
    long long r2 = r / g.W;
    int ih = (int)(r2 % g.H);
    int n = (int)(r2 / g.H);
    float acc = 0.f;
    for (int kh = 0; kh < g.KH; ++kh) {
      int a = ih + g.PH - kh;
      if (a < 0) break;
      int oh = a / g.SH;
      if (oh * g.SH != a || oh >= g.OH) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        int b = iw + g.PW - kw;
        if (b < 0) break;
        int ow = b / g.SW;
        if (ow * g.SW != b || ow >= g.OW) continue;
        long long row = ((long long)n * g.OH + oh) * g.OW + ow;
        acc += bf2f(dcol[row * g.Kp + (long long)(kh * g.KW + kw) * g.C + c]);
      }
    }
    T *p = dx + n * g.sn + c * g.sc + ih * g.sh + iw * g.sw;
    if (accumulate) acc += ldf(p);
    stf(p, acc);
  }
}
// vector form: bf16 channels-last output, C % 8 == 0
__global__ void col2im_vec_kernel(const bf16 *__restrict__ dcol, bf16 *__restrict__ dx, ConvGeom g, long long total, int accumulate) {
  const int c8n = g.C >> 3;
  const bool small = total < (1ll << 31);
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    int c8, iw, ih, n;
    split3(t, g.f_c8, g.f_w, g.f_h, small, c8n, g.W, g.H, c8, iw, ih, n);
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int kh = 0; kh < g.KH; ++kh) {
      int a = ih + g.PH - kh;
      if (a < 0) break;
      int oh = (int)fdiv((unsigned)a, g.f_sh);
      if (oh * g.SH != a || oh >= g.OH) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        int b = iw + g.PW - kw;
        if (b < 0) break;
        int ow = (int)fdiv((unsigned)b, g.f_sw);
        if (ow * g.SW != b || ow >= g.OW) continue;
        long long row = ((long long)n * g.OH + oh) * g.OW + ow;
        uint4 v = *reinterpret_cast<const uint4 *>(dcol + row * g.Kp + (long long)(kh * g.KW + kw) * g.C + c8 * 8);
        float2 f0 = unpack_bf162(v.x), f1 = unpack_bf162(v.y), f2 = unpack_bf162(v.z), f3 = unpack_bf162(v.w);
        acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
        acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
      }
    }
    bf16 *p = dx + n * g.sn + ih * g.sh + iw * g.sw + c8 * 8;
    if (accumulate) {
      uint4 v = *reinterpret_cast<const uint4 *>(p);
      float2 f0 = unpack_bf162(v.x), f1 = unpack_bf162(v.y), f2 = unpack_bf162(v.z), f3 = unpack_bf162(v.w);
      acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
      acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
    }
    uint4 o;
    o.x = pack_bf162(acc[0], acc[1]); o.y = pack_bf162(acc[2], acc[3]);
    o.z = pack_bf162(acc[4], acc[5]); o.w = pack_bf162(acc[6], acc[7]);
    *reinterpret_cast<uint4 *>(p) = o;
  }
}

// ------------------------------------------------------------------------------------------- filter repacking
// w [OC, C, KH, KW] -> wp [OC, Kp] with k = (kh*KW + kw)*C + c (zero padding columns)
template <typename T>
__global__ void filter_pack_kernel(const T *__restrict__ w, bf16 *__restrict__ wp, int OC, int C, int KH, int KW, int Kp) {
  long long total = (long long)OC * Kp;
  int K = C * KH * KW;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    int k = (int)(t % Kp);
    int oc = (int)(t / Kp);
    float v = 0.f;
    if (k < K) {
      int kk = k / C, c = k - kk * C;
      v = ldf(w + ((long long)oc * C + c) * KH * KW + kk);
    }
    wp[t] = f2bf(v);
  }
}
// dwp [OC, Kp] (fp32) -> dw [OC, C, KH, KW] (+)=
template <typename T>
__global__ void filter_unpack_kernel(const float *__restrict__ dwp, T *__restrict__ dw, int OC, int C, int KH, int KW, int Kp,
                                     int accumulate) {
  long long total = (long long)OC * C * KH * KW;
  int KK = KH * KW;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    int kk = (int)(t % KK);
    long long r = t / KK;
    int c = (int)(r % C);
    int oc = (int)(r / C);
    float v = dwp[(long long)oc * Kp + (long long)kk * C + c];
    if (accumulate) v += ldf(dw + t);
    stf(dw + t, v);
  }
}

// ------------------------------------------------------------------------------------------- pooling
// output channels-last [N, OH, OW, C]; input with arbitrary strides.  mode 0 = max (argmax window offset saved),
// 1 = average over the valid (unpadded) window elements.
template <typename T>
__global__ void pool_fwd_kernel(const T *__restrict__ x, T *__restrict__ y, unsigned char *__restrict__ arg, ConvGeom g, int mode,
                                long long total) {
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    int c = (int)(t % g.C);
    long long r = t / g.C;
    int ow = (int)(r % g.OW);
    long long r2 = r / g.OW;
    int oh = (int)(r2 % g.OH);
    int n = (int)(r2 / g.OH);
    const T *base = x + n * g.sn + c * g.sc;
    float best = -INFINITY, sum = 0.f;
    int besti = 0, cnt = 0;
    for (int kh = 0; kh < g.KH; ++kh) {
      int ih = oh * g.SH - g.PH + kh;
      if (ih < 0 || ih >= g.H) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        int iw = ow * g.SW - g.PW + kw;
        if (iw < 0 || iw >= g.W) continue;
        float v = ldf(base + ih * g.sh + iw * g.sw);
        if (v > best) { best = v; besti = kh * g.KW + kw; }
        sum += v;
        ++cnt;
      }
    }
    if (mode == 0) {
      stf(y + t, best);
      if (arg) arg[t] = (unsigned char)besti;
    } else {
      stf(y + t, cnt ? sum / cnt : 0.f);
    }
  }
}
// gather-form backward: one thread per input element
template <typename T>
__global__ void pool_bwd_kernel(const T *__restrict__ dy, const unsigned char *__restrict__ arg, T *__restrict__ dx, ConvGeom g, int mode,
                                long long total, int accumulate) {
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    int c = (int)(t % g.C);
    long long r = t / g.C;
    int iw = (int)(r % g.W);
    long long r2 = r / g.W;
    int ih = (int)(r2 % g.H);
    int n = (int)(r2 / g.H);
    float acc = 0.f;
    for (int kh = 0; kh < g.KH; ++kh) {
      int a = ih + g.PH - kh;
      if (a < 0) break;
      int oh = a / g.SH;
      if (oh * g.SH != a || oh >= g.OH) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        int b = iw + g.PW - kw;
        if (b < 0) break;
        int ow = b / g.SW;
        if (ow * g.SW != b || ow >= g.OW) continue;
        long long o = (((long long)n * g.OH + oh) * g.OW + ow) * g.C + c;
        if (mode == 0) {
          if (arg[o] == (unsigned char)(kh * g.KW + kw)) acc += ldf(dy + o);
        } else {
          int h0 = max(oh * g.SH - g.PH, 0), h1 = min(oh * g.SH - g.PH + g.KH, g.H);
          int w0 = max(ow * g.SW - g.PW, 0), w1 = min(ow * g.SW - g.PW + g.KW, g.W);
          acc += ldf(dy + o) / (float)((h1 - h0) * (w1 - w0));
        }
      }
    }
    T *p = dx + n * g.sn + c * g.sc + ih * g.sh + iw * g.sw;
    if (accumulate) acc += ldf(p);
    stf(p, acc);
  }
}

// ------------------------------------------------------------------------------------------- batch normalisation
// x is [R, C] (channels-last rows).  Column statistics are reduced in two steps: BN_ROWS-row chunks produce
// partial sums [chunks, 2, C] (fp32), a second kernel folds them.
constexpr int BN_TX = 32, BN_TY = 8;

template <typename T>
__global__ void bn_partial_kernel(const T *__restrict__ a, const T *__restrict__ b, const T *__restrict__ relu_y, float *__restrict__ part,
                                  const float *__restrict__ mean, const float *__restrict__ rstd, long long R, int C, int rows_per_chunk,
                                  int mode) {
  // mode 0: sums of a and a*a (forward statistics)
  // mode 1: sums of dy and dy * xhat with a = dy, b = x (backward); dy is masked where relu_y <= 0
  __shared__ float s0[BN_TY][BN_TX + 1], s1[BN_TY][BN_TX + 1];
  int c = blockIdx.x * BN_TX + threadIdx.x;
  long long r0 = (long long)blockIdx.y * rows_per_chunk;
  long long r1 = r0 + rows_per_chunk < R ? r0 + rows_per_chunk : R;
  float u = 0.f, v = 0.f;
  if (c < C) {
    float m = mode ? mean[c] : 0.f, rs = mode ? rstd[c] : 0.f;
    for (long long r = r0 + threadIdx.y; r < r1; r += BN_TY) {
      float av = ldf(a + r * C + c);
      if (mode == 0) {
        u += av;
        v += av * av;
      } else {
        if (relu_y && ldf(relu_y + r * C + c) <= 0.f) av = 0.f;
        float xh = (ldf(b + r * C + c) - m) * rs;
        u += av;
        v += av * xh;
      }
    }
  }
  s0[threadIdx.y][threadIdx.x] = u;
  s1[threadIdx.y][threadIdx.x] = v;
  __syncthreads();
  if (threadIdx.y == 0 && c < C) {
#pragma unroll
    for (int i = 1; i < BN_TY; ++i) { u += s0[i][threadIdx.x]; v += s1[i][threadIdx.x]; }
    part[((long long)blockIdx.y * 2 + 0) * C + c] = u;
    part[((long long)blockIdx.y * 2 + 1) * C + c] = v;
  }
}
// Fold the per-chunk partial sums: block = 32 columns x BN_FOLD chunk lanes, fixed summation order.
constexpr int BN_FOLD = 32;
__device__ __forceinline__ void bn_fold(const float *__restrict__ part, int chunks, int C, int c, float &s, float &q) {
  __shared__ float fs[BN_FOLD][33], fq[BN_FOLD][33];
  float a = 0.f, b = 0.f;
  if (c < C)
    for (int k = threadIdx.y; k < chunks; k += BN_FOLD) {
      a += part[((long long)k * 2) * C + c];
      b += part[((long long)k * 2 + 1) * C + c];
    }
  fs[threadIdx.y][threadIdx.x] = a;
  fq[threadIdx.y][threadIdx.x] = b;
  __syncthreads();
  s = q = 0.f;
  if (threadIdx.y == 0)
    for (int i = 0; i < BN_FOLD; ++i) { s += fs[i][threadIdx.x]; q += fq[i][threadIdx.x]; }
}
__global__ void bn_finalize_stats_kernel(const float *__restrict__ part, int chunks, int C, long long R, float eps, float *__restrict__ mean,
                                         float *__restrict__ rstd) {
  int c = blockIdx.x * 32 + threadIdx.x;
  float s, q;
  bn_fold(part, chunks, C, c, s, q);
  if (threadIdx.y != 0 || c >= C) return;
  double m = (double)s / (double)R;
  double var = (double)q / (double)R - m * m;
  if (var < 0.0) var = 0.0;
  mean[c] = (float)m;
  rstd[c] = (float)(1.0 / sqrt(var + (double)eps));
}
// sums[0][c] = sum dy, sums[1][c] = sum dy*xhat; also writes dgamma/dbeta (+)= when given
template <typename T>
__global__ void bn_finalize_grads_kernel(const float *__restrict__ part, int chunks, int C, float *__restrict__ sums, T *__restrict__ dgamma,
                                         T *__restrict__ dbeta, int acc_gamma, int acc_beta) {
  int c = blockIdx.x * 32 + threadIdx.x;
  float s, q;
  bn_fold(part, chunks, C, c, s, q);
  if (threadIdx.y != 0 || c >= C) return;
  sums[c] = s;
  sums[C + c] = q;
  if (dbeta) stf(dbeta + c, s + (acc_beta ? ldf(dbeta + c) : 0.f));
  if (dgamma) stf(dgamma + c, q + (acc_gamma ? ldf(dgamma + c) : 0.f));
}
template <typename T>
__global__ void bn_apply_kernel(const T *__restrict__ x, T *__restrict__ y, const T *__restrict__ gamma, const T *__restrict__ beta,
                                const float *__restrict__ mean, const float *__restrict__ rstd, long long total, int C, int relu) {
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    int c = (int)(t % C);
    float v = (ldf(x + t) - mean[c]) * rstd[c];
    if (gamma) v *= ldf(gamma + c);
    if (beta) v += ldf(beta + c);
    if (relu && v < 0.f) v = 0.f;
    stf(y + t, v);
  }
}
// two elements per thread for bf16 with even C
__global__ void bn_apply_bf16x2_kernel(const bf16 *__restrict__ x, bf16 *__restrict__ y, const bf16 *__restrict__ gamma,
                                       const bf16 *__restrict__ beta, const float *__restrict__ mean, const float *__restrict__ rstd,
                                       long long pairs, int C, int relu) {
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < pairs; t += (long long)gridDim.x * blockDim.x) {
    int c = (int)((t * 2) % C);
    float2 v = unpack_bf162(reinterpret_cast<const uint32_t *>(x)[t]);
    v.x = (v.x - mean[c]) * rstd[c];
    v.y = (v.y - mean[c + 1]) * rstd[c + 1];
    if (gamma) { v.x *= bf2f(gamma[c]); v.y *= bf2f(gamma[c + 1]); }
    if (beta) { v.x += bf2f(beta[c]); v.y += bf2f(beta[c + 1]); }
    if (relu) { v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); }
    reinterpret_cast<uint32_t *>(y)[t] = pack_bf162(v.x, v.y);
  }
}
// dx = gamma * rstd * (dy' - sum_dy / R - xhat * sum_dy_xhat / R)
template <typename T>
__global__ void bn_bwd_apply_kernel(const T *__restrict__ dy, const T *__restrict__ x, const T *__restrict__ relu_y, const T *__restrict__ gamma,
                                    const float *__restrict__ mean, const float *__restrict__ rstd, const float *__restrict__ sums,
                                    T *__restrict__ dx, long long total, int C, float inv_r, int accumulate) {
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    int c = (int)(t % C);
    float g = ldf(dy + t);
    if (relu_y && ldf(relu_y + t) <= 0.f) g = 0.f;
    float xh = (ldf(x + t) - mean[c]) * rstd[c];
    float v = (g - sums[c] * inv_r - xh * sums[C + c] * inv_r) * rstd[c];
    if (gamma) v *= ldf(gamma + c);
    if (accumulate) v += ldf(dx + t);
    stf(dx + t, v);
  }
}


// ---- vector forms for bf16 channels-last data with C % 8 == 0: one thread handles 8 channels (16 bytes)
__device__ __forceinline__ void unpack8(const uint4 &v, float *f) {
  float2 a = unpack_bf162(v.x), b = unpack_bf162(v.y), c = unpack_bf162(v.z), d = unpack_bf162(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float *f) {
  uint4 o;
  o.x = pack_bf162(f[0], f[1]); o.y = pack_bf162(f[2], f[3]); o.z = pack_bf162(f[4], f[5]); o.w = pack_bf162(f[6], f[7]);
  return o;
}

__global__ void pool_fwd_vec_kernel(const bf16 *__restrict__ x, bf16 *__restrict__ y, unsigned char *__restrict__ arg, ConvGeom g, int mode,
                                    long long total) {
  const int c8n = g.C >> 3;
  const bool small = total < (1ll << 31);
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    int c8, ow, oh, n;
    split3(t, g.f_c8, g.f_ow, g.f_oh, small, c8n, g.OW, g.OH, c8, ow, oh, n);
    const bf16 *base = x + n * g.sn + c8 * 8;
    float best[8], sum[8];
    int besti[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { best[i] = -INFINITY; sum[i] = 0.f; besti[i] = 0; }
    int cnt = 0;
    const int h0 = max(oh * g.SH - g.PH, 0), h1 = min(oh * g.SH - g.PH + g.KH, g.H);
    const int w0 = max(ow * g.SW - g.PW, 0), w1 = min(ow * g.SW - g.PW + g.KW, g.W);
    for (int ih = h0; ih < h1; ++ih) {
      for (int iw = w0; iw < w1; ++iw) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4 *>(base + ih * g.sh + iw * g.sw), f);
        const int off = (ih - (oh * g.SH - g.PH)) * g.KW + (iw - (ow * g.SW - g.PW));
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (f[i] > best[i]) { best[i] = f[i]; besti[i] = off; }
          sum[i] += f[i];
        }
        ++cnt;
      }
    }
    if (mode == 0) {
      *reinterpret_cast<uint4 *>(y + t * 8) = pack8(best);
      if (arg) {
        uint2 a;
        a.x = besti[0] | (besti[1] << 8) | (besti[2] << 16) | (besti[3] << 24);
        a.y = besti[4] | (besti[5] << 8) | (besti[6] << 16) | (besti[7] << 24);
        *reinterpret_cast<uint2 *>(arg + t * 8) = a;
      }
    } else {
      const float inv = cnt ? 1.f / cnt : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) sum[i] *= inv;
      *reinterpret_cast<uint4 *>(y + t * 8) = pack8(sum);
    }
  }
}

__global__ void pool_bwd_vec_kernel(const bf16 *__restrict__ dy, const unsigned char *__restrict__ arg, bf16 *__restrict__ dx, ConvGeom g,
                                    int mode, long long total, int accumulate) {
  const int c8n = g.C >> 3;
  const bool small = total < (1ll << 31);
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    int c8, iw, ih, n;
    split3(t, g.f_c8, g.f_w, g.f_h, small, c8n, g.W, g.H, c8, iw, ih, n);
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int kh = 0; kh < g.KH; ++kh) {
      int a = ih + g.PH - kh;
      if (a < 0) break;
      int oh = (int)fdiv((unsigned)a, g.f_sh);
      if (oh * g.SH != a || oh >= g.OH) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        int b = iw + g.PW - kw;
        if (b < 0) break;
        int ow = (int)fdiv((unsigned)b, g.f_sw);
        if (ow * g.SW != b || ow >= g.OW) continue;
        long long o = ((((long long)n * g.OH + oh) * g.OW + ow) * c8n + c8) * 8;
        float f[8];
        unpack8(*reinterpret_cast<const uint4 *>(dy + o), f);
        if (mode == 0) {
          uint2 am = *reinterpret_cast<const uint2 *>(arg + o);
          const unsigned int me = (unsigned int)(kh * g.KW + kw);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (((am.x >> (8 * i)) & 0xFFu) == me) acc[i] += f[i];
            if (((am.y >> (8 * i)) & 0xFFu) == me) acc[4 + i] += f[4 + i];
          }
        } else {
          int h0 = max(oh * g.SH - g.PH, 0), h1 = min(oh * g.SH - g.PH + g.KH, g.H);
          int w0 = max(ow * g.SW - g.PW, 0), w1 = min(ow * g.SW - g.PW + g.KW, g.W);
          const float inv = 1.f / (float)((h1 - h0) * (w1 - w0));
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += f[i] * inv;
        }
      }
    }
    bf16 *p = dx + n * g.sn + ih * g.sh + iw * g.sw + c8 * 8;
    if (accumulate) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4 *>(p), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    *reinterpret_cast<uint4 *>(p) = pack8(acc);
  }
}

// Batch-norm column statistics, vector form.  Thread (g, lane) of a block owns channel group g (8 channels) and
// walks rows lane, lane + lanes, ... of the block's row chunk; consecutive threads read consecutive 16-byte
// pieces of memory (the last group of a row is followed by the first group of the next row).  Per-lane sums go
// through shared memory in a fixed order, so the result does not depend on scheduling.
constexpr int BNV_THREADS = 256;
__global__ void bn_partial_vec_kernel(const bf16 *__restrict__ a, const bf16 *__restrict__ b, const bf16 *__restrict__ relu_y,
                                      float *__restrict__ part, const float *__restrict__ mean, const float *__restrict__ rstd, long long R,
                                      int C, int rows_per_chunk, int mode) {
  extern __shared__ float sred[];  // [lanes][2][C]
  const int groups = C >> 3;
  const int lanes = BNV_THREADS / groups;
  const int gidx = threadIdx.x % groups, lane = threadIdx.x / groups;
  long long r0 = (long long)blockIdx.x * rows_per_chunk;
  long long r1 = r0 + rows_per_chunk < R ? r0 + rows_per_chunk : R;
  float u[8], v[8], m[8], rs[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { u[i] = 0.f; v[i] = 0.f; m[i] = 0.f; rs[i] = 0.f; }
  if (lane < lanes) {
    if (mode) {
#pragma unroll
      for (int i = 0; i < 8; ++i) { m[i] = mean[gidx * 8 + i]; rs[i] = rstd[gidx * 8 + i]; }
    }
    long long r = r0 + lane;
    if (mode == 0) {
      // four rows per trip: four independent 16-byte loads in flight per thread
      for (; r + 3LL * lanes < r1; r += 4LL * lanes) {
        uint4 q0 = *reinterpret_cast<const uint4 *>(a + r * C + gidx * 8);
        uint4 q1 = *reinterpret_cast<const uint4 *>(a + (r + lanes) * C + gidx * 8);
        uint4 q2 = *reinterpret_cast<const uint4 *>(a + (r + 2LL * lanes) * C + gidx * 8);
        uint4 q3 = *reinterpret_cast<const uint4 *>(a + (r + 3LL * lanes) * C + gidx * 8);
        float f0[8], f1[8], f2[8], f3[8];
        unpack8(q0, f0); unpack8(q1, f1); unpack8(q2, f2); unpack8(q3, f3);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          u[i] += (f0[i] + f1[i]) + (f2[i] + f3[i]);
          v[i] += (f0[i] * f0[i] + f1[i] * f1[i]) + (f2[i] * f2[i] + f3[i] * f3[i]);
        }
      }
    }
    for (; r < r1; r += lanes) {
      const long long off = r * C + gidx * 8;
      float av[8];
      unpack8(*reinterpret_cast<const uint4 *>(a + off), av);
      if (mode == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { u[i] += av[i]; v[i] += av[i] * av[i]; }
      } else {
        float xv[8];
        unpack8(*reinterpret_cast<const uint4 *>(b + off), xv);
        if (relu_y) {
          float yv[8];
          unpack8(*reinterpret_cast<const uint4 *>(relu_y + off), yv);
#pragma unroll
          for (int i = 0; i < 8; ++i) if (yv[i] <= 0.f) av[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) { u[i] += av[i]; v[i] += av[i] * (xv[i] - m[i]) * rs[i]; }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      sred[(lane * 2 + 0) * C + gidx * 8 + i] = u[i];
      sred[(lane * 2 + 1) * C + gidx * 8 + i] = v[i];
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < 2 * C; c += BNV_THREADS) {
    float s = 0.f;
    for (int l = 0; l < lanes; ++l) s += sred[l * 2 * C + c];
    part[(long long)blockIdx.x * 2 * C + c] = s;
  }
}
__global__ void bn_apply_vec_kernel(const bf16 *__restrict__ x, bf16 *__restrict__ y, const bf16 *__restrict__ gamma,
                                    const bf16 *__restrict__ beta, const float *__restrict__ mean, const float *__restrict__ rstd,
                                    long long total8, int C, int relu) {
  // the grid-stride step is a multiple of the number of channel groups, so a thread stays on one group and
  // keeps that group's scale and shift in registers: y = x * scale + shift
  const int groups = C >> 3;
  const long long usable = ((long long)gridDim.x * blockDim.x / groups) * groups;
  const long long t0 = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t0 >= usable) return;
  const int c = (int)(t0 % groups) * 8;
  float sc[8], sh[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    sc[i] = rstd[c + i] * (gamma ? bf2f(gamma[c + i]) : 1.f);
    sh[i] = (beta ? bf2f(beta[c + i]) : 0.f) - mean[c + i] * sc[i];
  }
  const float floor_ = relu ? 0.f : -INFINITY;
  for (long long t = t0; t < total8; t += usable) {
    float f[8];
    unpack8(reinterpret_cast<const uint4 *>(x)[t], f);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = fmaxf(fmaf(f[i], sc[i], sh[i]), floor_);
    reinterpret_cast<uint4 *>(y)[t] = pack8(f);
  }
}
__global__ void bn_bwd_apply_vec_kernel(const bf16 *__restrict__ dy, const bf16 *__restrict__ x, const bf16 *__restrict__ relu_y,
                                        const bf16 *__restrict__ gamma, const float *__restrict__ mean, const float *__restrict__ rstd,
                                        const float *__restrict__ sums, bf16 *__restrict__ dx, long long total8, int C, float inv_r,
                                        int accumulate) {
  // dx = a * dy' + b * x + c per channel (constants kept in registers, see bn_apply_vec_kernel):
  //   xh = (x - mean) * rstd;  dx = gamma * rstd * (dy' - s1/R - xh * s2/R)
  const int groups = C >> 3;
  const long long usable = ((long long)gridDim.x * blockDim.x / groups) * groups;
  const long long t0 = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t0 >= usable) return;
  const int c = (int)(t0 % groups) * 8;
  float ka[8], kb[8], kc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float rs = rstd[c + i], g = gamma ? bf2f(gamma[c + i]) : 1.f;
    const float s1 = sums[c + i] * inv_r, s2 = sums[C + c + i] * inv_r;
    ka[i] = g * rs;
    kb[i] = -g * rs * rs * s2;
    kc[i] = g * rs * (mean[c + i] * rs * s2 - s1);
  }
  for (long long t = t0; t < total8; t += usable) {
    float g[8], xv[8], o[8];
    unpack8(reinterpret_cast<const uint4 *>(dy)[t], g);
    unpack8(reinterpret_cast<const uint4 *>(x)[t], xv);
    if (relu_y) {
      float yv[8];
      unpack8(reinterpret_cast<const uint4 *>(relu_y)[t], yv);
#pragma unroll
      for (int i = 0; i < 8; ++i) if (yv[i] <= 0.f) g[i] = 0.f;
    }
    if (accumulate) unpack8(reinterpret_cast<const uint4 *>(dx)[t], o);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float v = fmaf(ka[i], g[i], fmaf(kb[i], xv[i], kc[i]));
      o[i] = accumulate ? o[i] + v : v;
    }
    reinterpret_cast<uint4 *>(dx)[t] = pack8(o);
  }
}

inline FastDiv make_fd(int d_) {
  FastDiv f;
  unsigned d = d_ < 1 ? 1u : (unsigned)d_;
  f.d = d;
  if (d == 1) { f.mul = 0; f.sh = 0; return f; }
  unsigned l = 0;
  while ((1ull << l) < d) ++l;  // ceil(log2(d))
  const unsigned p = 31 + l;
  f.mul = (unsigned)(((1ull << p) + d - 1) / d);
  f.sh = p - 32;
  return f;
}
inline ConvGeom make_geom(const int *p, const long long *strides) {
  ConvGeom g;
  g.N = p[0]; g.C = p[1]; g.H = p[2]; g.W = p[3]; g.KH = p[4]; g.KW = p[5]; g.SH = p[6]; g.SW = p[7]; g.PH = p[8]; g.PW = p[9];
  g.OH = p[10]; g.OW = p[11]; g.Kp = p[12];
  g.sn = strides[0]; g.sc = strides[1]; g.sh = strides[2]; g.sw = strides[3];
  g.f_c8 = make_fd(g.C >> 3); g.f_kk = make_fd(g.KH * g.KW); g.f_kw = make_fd(g.KW); g.f_ow = make_fd(g.OW); g.f_oh = make_fd(g.OH);
  g.f_w = make_fd(g.W); g.f_h = make_fd(g.H); g.f_sh = make_fd(g.SH); g.f_sw = make_fd(g.SW);
  g.f_kp = make_fd(g.Kp); g.f_c = make_fd(g.C);
  return g;
}
inline bool vec_ok(const ConvGeom &g, const void *p) {
  return g.sc == 1 && (g.C % 8) == 0 && (g.sw % 8) == 0 && (g.sh % 8) == 0 && (g.sn % 8) == 0 && ((uintptr_t)p % 16) == 0;
}

}  // namespace

// geom: {N, C, H, W, KH, KW, SH, SW, PH, PW, OH, OW, Kp}; strides: element strides (n, c, h, w) of x.  dt: 0 fp32, 1 bf16.
FFK_API int ffk_im2col(const void *x, void *col, const int *geom, const long long *strides, int dt, cudaStream_t st) {
  ConvGeom g = make_geom(geom, strides);
  long long rows = (long long)g.N * g.OH * g.OW;
  if (rows <= 0) return 0;
  int K = g.KH * g.KW * g.C;
  if (g.Kp < K || (g.Kp % 8) != 0) return -2;
  if (dt == 1 && vec_ok(g, x) && g.Kp == K) {
    long long total = rows * g.KH * g.KW * (g.C / 8);
    im2col_vec_kernel<<<ffk_blocks(total, 256), 256, 0, st>>>((const bf16 *)x, (bf16 *)col, g, total);
  } else {
    long long total = rows * g.Kp;
    if (dt == 1) im2col_kernel<bf16><<<ffk_blocks(total, 256), 256, 0, st>>>((const bf16 *)x, (bf16 *)col, g, total);
    else if (dt == 0) im2col_kernel<float><<<ffk_blocks(total, 256), 256, 0, st>>>((const float *)x, (bf16 *)col, g, total);
    else return -2;
  }
  return (int)cudaGetLastError();
}

FFK_API int ffk_col2im(const void *dcol, void *dx, const int *geom, const long long *strides, int dt, int accumulate, cudaStream_t st) {
  ConvGeom g = make_geom(geom, strides);
  long long total = (long long)g.N * g.H * g.W * g.C;
  if (total <= 0) return 0;
  if (dt == 1 && vec_ok(g, dx)) {
    long long tv = total / 8;
    col2im_vec_kernel<<<ffk_blocks(tv, 256), 256, 0, st>>>((const bf16 *)dcol, (bf16 *)dx, g, tv, accumulate);
  } else if (dt == 1) {
    col2im_kernel<bf16><<<ffk_blocks(total, 256), 256, 0, st>>>((const bf16 *)dcol, (bf16 *)dx, g, total, accumulate);
  } else if (dt == 0) {
    col2im_kernel<float><<<ffk_blocks(total, 256), 256, 0, st>>>((const bf16 *)dcol, (float *)dx, g, total, accumulate);
  } else {
    return -2;
  }
  return (int)cudaGetLastError();
}

FFK_API int ffk_filter_pack(const void *w, void *wp, int OC, int C, int KH, int KW, int Kp, int dt, cudaStream_t st) {
  long long total = (long long)OC * Kp;
  if (total <= 0) return 0;
  if (dt == 1) filter_pack_kernel<bf16><<<ffk_blocks(total, 256), 256, 0, st>>>((const bf16 *)w, (bf16 *)wp, OC, C, KH, KW, Kp);
  else if (dt == 0) filter_pack_kernel<float><<<ffk_blocks(total, 256), 256, 0, st>>>((const float *)w, (bf16 *)wp, OC, C, KH, KW, Kp);
  else return -2;
  return (int)cudaGetLastError();
}

FFK_API int ffk_filter_unpack(const float *dwp, void *dw, int OC, int C, int KH, int KW, int Kp, int dt, int accumulate, cudaStream_t st) {
  long long total = (long long)OC * C * KH * KW;
  if (total <= 0) return 0;
  if (dt == 1) filter_unpack_kernel<bf16><<<ffk_blocks(total, 256), 256, 0, st>>>(dwp, (bf16 *)dw, OC, C, KH, KW, Kp, accumulate);
  else if (dt == 0) filter_unpack_kernel<float><<<ffk_blocks(total, 256), 256, 0, st>>>(dwp, (float *)dw, OC, C, KH, KW, Kp, accumulate);
  else return -2;
  return (int)cudaGetLastError();
}

// mode: 0 max, 1 average.  arg: [N*OH*OW*C] bytes (max only; may be null for inference)
FFK_API int ffk_pool2d_fwd(const void *x, void *y, void *arg, const int *geom, const long long *strides, int mode, int dt, cudaStream_t st) {
  ConvGeom g = make_geom(geom, strides);
  long long total = (long long)g.N * g.OH * g.OW * g.C;
  if (total <= 0) return 0;
  if (g.KH * g.KW > 255) return -2;
  if (dt == 1 && vec_ok(g, x) && ((uintptr_t)y % 16) == 0 && ((uintptr_t)arg % 8) == 0) {
    long long tv = total / 8;
    pool_fwd_vec_kernel<<<ffk_blocks(tv, 256), 256, 0, st>>>((const bf16 *)x, (bf16 *)y, (unsigned char *)arg, g, mode, tv);
    return (int)cudaGetLastError();
  }
  if (dt == 1) pool_fwd_kernel<bf16><<<ffk_blocks(total, 256), 256, 0, st>>>((const bf16 *)x, (bf16 *)y, (unsigned char *)arg, g, mode, total);
  else if (dt == 0) pool_fwd_kernel<float><<<ffk_blocks(total, 256), 256, 0, st>>>((const float *)x, (float *)y, (unsigned char *)arg, g, mode, total);
  else return -2;
  return (int)cudaGetLastError();
}

FFK_API int ffk_pool2d_bwd(const void *dy, const void *arg, void *dx, const int *geom, const long long *strides, int mode, int dt,
                           int accumulate, cudaStream_t st) {
  ConvGeom g = make_geom(geom, strides);
  long long total = (long long)g.N * g.H * g.W * g.C;
  if (total <= 0) return 0;
  if (mode == 0 && !arg) return -2;
  if (dt == 1 && vec_ok(g, dx) && ((uintptr_t)dy % 16) == 0 && ((uintptr_t)arg % 8) == 0) {
    long long tv = total / 8;
    pool_bwd_vec_kernel<<<ffk_blocks(tv, 256), 256, 0, st>>>((const bf16 *)dy, (const unsigned char *)arg, (bf16 *)dx, g, mode, tv,
                                                             accumulate);
    return (int)cudaGetLastError();
  }
  if (dt == 1) pool_bwd_kernel<bf16><<<ffk_blocks(total, 256), 256, 0, st>>>((const bf16 *)dy, (const unsigned char *)arg, (bf16 *)dx, g, mode, total, accumulate);
  else if (dt == 0) pool_bwd_kernel<float><<<ffk_blocks(total, 256), 256, 0, st>>>((const float *)dy, (const unsigned char *)arg, (float *)dx, g, mode, total, accumulate);
  else return -2;
  return (int)cudaGetLastError();
}

static int bn_chunks(long long R, int C, int *rows_per_chunk) {
  int coltiles = (C + BN_TX - 1) / BN_TX;
  long long want = (148 * 8 + coltiles - 1) / coltiles;
  long long maxc = (R + 63) / 64;
  long long chunks = want < maxc ? want : maxc;
  if (chunks < 1) chunks = 1;
  long long rpc = (R + chunks - 1) / chunks;
  chunks = (R + rpc - 1) / rpc;
  *rows_per_chunk = (int)rpc;
  return (int)chunks;
}
static bool bn_vec_ok(int C, const void *a, const void *b, const void *c) {
  return (C % 8) == 0 && C / 8 <= BNV_THREADS && ((uintptr_t)a % 16) == 0 && ((uintptr_t)b % 16) == 0 && ((uintptr_t)c % 16) == 0;
}
static int bn_chunks_vec(long long R, int C, int *rows_per_chunk) {
  const int lanes = BNV_THREADS / (C / 8);
  long long maxc = (R + 4LL * lanes - 1) / (4LL * lanes);  // at least ~4 rows per thread
  long long chunks = maxc < 148 * 4 ? maxc : 148 * 4;
  if (chunks < 1) chunks = 1;
  long long rpc = (R + chunks - 1) / chunks;
  chunks = (R + rpc - 1) / rpc;
  *rows_per_chunk = (int)rpc;
  return (int)chunks;
}
// number of fp32 scratch elements the batch-norm entry points need
FFK_API long long ffk_batchnorm_scratch(long long R, int C) {
  int rpc;
  long long chunks = bn_chunks(R, C, &rpc);
  if ((C % 8) == 0 && C / 8 <= BNV_THREADS) {
    long long cv = bn_chunks_vec(R, C, &rpc);
    if (cv > chunks) chunks = cv;
  }
  return chunks * 2 * C + 2 * (long long)C;
}

// y = act((x - mean) * rstd * gamma + beta) with batch statistics; mean/rstd [C] fp32 are saved for backward
FFK_API int ffk_batchnorm_fwd(const void *x, void *y, const void *gamma, const void *beta, float *mean, float *rstd, float *scratch,
                              long long R, int C, float eps, int relu, int dt, cudaStream_t st) {
  if (R <= 0 || C <= 0) return 0;
  int rpc;
  int chunks = bn_chunks(R, C, &rpc);
  dim3 grid((C + BN_TX - 1) / BN_TX, chunks), block(BN_TX, BN_TY);
  long long total = R * C;
  if (dt == 1 && bn_vec_ok(C, x, y, x)) {
    int rv;
    int cv = bn_chunks_vec(R, C, &rv);
    const int lanes = BNV_THREADS / (C / 8);
    bn_partial_vec_kernel<<<cv, BNV_THREADS, (size_t)lanes * 2 * C * sizeof(float), st>>>((const bf16 *)x, nullptr, nullptr, scratch, nullptr,
                                                                                          nullptr, R, C, rv, 0);
    bn_finalize_stats_kernel<<<(C + 31) / 32, dim3(32, BN_FOLD), 0, st>>>(scratch, cv, C, R, eps, mean, rstd);
    bn_apply_vec_kernel<<<ffk_blocks(total / 8, 256), 256, 0, st>>>((const bf16 *)x, (bf16 *)y, (const bf16 *)gamma, (const bf16 *)beta, mean,
                                                                    rstd, total / 8, C, relu);
    return (int)cudaGetLastError();
  }
  if (dt == 1) {
    bn_partial_kernel<bf16><<<grid, block, 0, st>>>((const bf16 *)x, nullptr, nullptr, scratch, nullptr, nullptr, R, C, rpc, 0);
    bn_finalize_stats_kernel<<<(C + 31) / 32, dim3(32, BN_FOLD), 0, st>>>(scratch, chunks, C, R, eps, mean, rstd);
    if ((C % 2) == 0 && ((uintptr_t)x % 4) == 0 && ((uintptr_t)y % 4) == 0)
      bn_apply_bf16x2_kernel<<<ffk_blocks(total / 2, 256), 256, 0, st>>>((const bf16 *)x, (bf16 *)y, (const bf16 *)gamma, (const bf16 *)beta,
                                                                         mean, rstd, total / 2, C, relu);
    else
      bn_apply_kernel<bf16><<<ffk_blocks(total, 256), 256, 0, st>>>((const bf16 *)x, (bf16 *)y, (const bf16 *)gamma, (const bf16 *)beta, mean,
                                                                    rstd, total, C, relu);
  } else if (dt == 0) {
    bn_partial_kernel<float><<<grid, block, 0, st>>>((const float *)x, nullptr, nullptr, scratch, nullptr, nullptr, R, C, rpc, 0);
    bn_finalize_stats_kernel<<<(C + 31) / 32, dim3(32, BN_FOLD), 0, st>>>(scratch, chunks, C, R, eps, mean, rstd);
    bn_apply_kernel<float><<<ffk_blocks(total, 256), 256, 0, st>>>((const float *)x, (float *)y, (const float *)gamma, (const float *)beta,
                                                                   mean, rstd, total, C, relu);
  } else {
    return -2;
  }
  return (int)cudaGetLastError();
}

// relu_y: the forward output when a ReLU was fused (masks dy), else null.  dgamma/dbeta may be null.
FFK_API int ffk_batchnorm_bwd(const void *dy, const void *x, const void *relu_y, const void *gamma, const float *mean, const float *rstd,
                              void *dx, void *dgamma, void *dbeta, float *scratch, long long R, int C, int dt, int accumulate_dx,
                              int accumulate_gamma, int accumulate_beta, cudaStream_t st) {
  if (R <= 0 || C <= 0) return 0;
  int rpc;
  int chunks = bn_chunks(R, C, &rpc);
  dim3 grid((C + BN_TX - 1) / BN_TX, chunks), block(BN_TX, BN_TY);
  float *sums = scratch + (long long)chunks * 2 * C;
  long long total = R * C;
  float inv_r = 1.0f / (float)R;
  if (dt == 1 && bn_vec_ok(C, dy, x, relu_y) && (!dx || ((uintptr_t)dx % 16) == 0)) {
    int rv;
    int cv = bn_chunks_vec(R, C, &rv);
    const int lanes = BNV_THREADS / (C / 8);
    float *sums_v = scratch + (long long)cv * 2 * C;
    bn_partial_vec_kernel<<<cv, BNV_THREADS, (size_t)lanes * 2 * C * sizeof(float), st>>>((const bf16 *)dy, (const bf16 *)x, (const bf16 *)relu_y,
                                                                                          scratch, mean, rstd, R, C, rv, 1);
    bn_finalize_grads_kernel<bf16><<<(C + 31) / 32, dim3(32, BN_FOLD), 0, st>>>(scratch, cv, C, sums_v, (bf16 *)dgamma, (bf16 *)dbeta, accumulate_gamma,
                                                                     accumulate_beta);
    if (dx)
      bn_bwd_apply_vec_kernel<<<ffk_blocks(total / 8, 256), 256, 0, st>>>((const bf16 *)dy, (const bf16 *)x, (const bf16 *)relu_y,
                                                                          (const bf16 *)gamma, mean, rstd, sums_v, (bf16 *)dx, total / 8, C,
                                                                          inv_r, accumulate_dx);
    return (int)cudaGetLastError();
  }
  if (dt == 1) {
    bn_partial_kernel<bf16><<<grid, block, 0, st>>>((const bf16 *)dy, (const bf16 *)x, (const bf16 *)relu_y, scratch, mean, rstd, R, C, rpc, 1);
    bn_finalize_grads_kernel<bf16><<<(C + 31) / 32, dim3(32, BN_FOLD), 0, st>>>(scratch, chunks, C, sums, (bf16 *)dgamma, (bf16 *)dbeta, accumulate_gamma,
                                                                     accumulate_beta);
    if (dx)
      bn_bwd_apply_kernel<bf16><<<ffk_blocks(total, 256), 256, 0, st>>>((const bf16 *)dy, (const bf16 *)x, (const bf16 *)relu_y,
                                                                        (const bf16 *)gamma, mean, rstd, sums, (bf16 *)dx, total, C, inv_r,
                                                                        accumulate_dx);
  } else if (dt == 0) {
    bn_partial_kernel<float><<<grid, block, 0, st>>>((const float *)dy, (const float *)x, (const float *)relu_y, scratch, mean, rstd, R, C, rpc, 1);
    bn_finalize_grads_kernel<float><<<(C + 31) / 32, dim3(32, BN_FOLD), 0, st>>>(scratch, chunks, C, sums, (float *)dgamma, (float *)dbeta,
                                                                      accumulate_gamma, accumulate_beta);
    if (dx)
      bn_bwd_apply_kernel<float><<<ffk_blocks(total, 256), 256, 0, st>>>((const float *)dy, (const float *)x, (const float *)relu_y,
                                                                         (const float *)gamma, mean, rstd, sums, (float *)dx, total, C, inv_r,
                                                                         accumulate_dx);
  } else {
    return -2;
  }
  return (int)cudaGetLastError();
}
