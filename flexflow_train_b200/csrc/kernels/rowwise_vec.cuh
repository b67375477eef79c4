// rowwise_vec.cuh -- 128-bit vectorised fast paths of the row-wise kernels for bf16 rows whose length
// is a multiple of 8: softmax fwd/bwd (optionally fused with dropout of the probabilities), LayerNorm
// fwd/bwd (fused residual add) and the bias/activation backward with its column reduction.
//
// Each thread owns whole 8-element vectors of a row and keeps them in registers, so a row is read once
// and written once; HBM traffic is the algorithmic minimum.  The scalar kernels in norm_softmax.cu and
// elementwise.cu remain the general path (fp32, odd lengths).
#pragma once
#include "common.cuh"

namespace vec {

__device__ __forceinline__ void ld8(const bf16 *p, float *v) {
  uint4 u = *reinterpret_cast<const uint4 *>(p);
  float2 a = unpack_bf162(u.x), b = unpack_bf162(u.y), c = unpack_bf162(u.z), d = unpack_bf162(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
__device__ __forceinline__ void unpack8(const uint4 &u, float *v) {
  float2 a = unpack_bf162(u.x), b = unpack_bf162(u.y), c = unpack_bf162(u.z), d = unpack_bf162(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
__device__ __forceinline__ void st8(bf16 *p, const float *v) {
  *reinterpret_cast<uint4 *>(p) = make_uint4(pack_bf162(v[0], v[1]), pack_bf162(v[2], v[3]), pack_bf162(v[4], v[5]), pack_bf162(v[6], v[7]));
}

// ---------------------------------------------------------------- softmax: one warp per row
// cols = 256 * VPT.  y = softmax(scale * x); yd (optional) = dropout(y) with keep mask hash(seed, element index).
template <int VPT>
__global__ void softmax_fwd_warp_kernel(const bf16 *__restrict__ x, bf16 *__restrict__ y, bf16 *__restrict__ yd, int rows, float scale,
                                        int causal_q, float p_drop, unsigned long long salt, const unsigned long long *seed_ptr) {
  constexpr int COLS = 256 * VPT;
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  unsigned long long seed = salt;
  if (seed_ptr) seed = salt * 0x9E3779B97F4A7C15ull + *seed_ptr;
  const float keep_scale = p_drop < 1.f ? 1.f / (1.f - p_drop) : 0.f;
  const uint32_t thr = ffk_drop_threshold(p_drop);
  for (long long row = (long long)blockIdx.x * wpb + wib; row < rows; row += (long long)gridDim.x * wpb) {
    const bf16 *px = x + row * COLS;
    float v[VPT][8];
    const int limit = causal_q > 0 ? (int)(row % causal_q) + 1 : COLS;
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int c0 = (i * 32 + lane) * 8;
      ld8(px + c0, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[i][j] = (c0 + j < limit) ? v[i][j] * scale : -INFINITY;
        mx = fmaxf(mx, v[i][j]);
      }
    }
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[i][j] = __expf(v[i][j] - mx);
        s += v[i][j];
      }
    s = warp_sum(s);
    const float inv = 1.f / s;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int c0 = (i * 32 + lane) * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] *= inv;
      st8(y + row * COLS + c0, v[i]);
      if (yd) {
        float d[8];
        const unsigned long long g4 = (unsigned long long)(row * COLS + c0) >> 2;
        const uint32_t keep = ffk_keep4(seed, g4, thr) | (ffk_keep4(seed, g4 + 1, thr) << 4);
#pragma unroll
        for (int j = 0; j < 8; ++j) d[j] = (keep >> j) & 1u ? v[i][j] * keep_scale : 0.f;
        st8(yd + row * COLS + c0, d);
      }
    }
  }
}
// dx = scale * y * (g - sum(g * y)), g = dy (optionally first passed back through the dropout mask)
template <int VPT>
__global__ void softmax_bwd_warp_kernel(const bf16 *__restrict__ dy, const bf16 *__restrict__ y, bf16 *__restrict__ dx, int rows,
                                        float scale, float p_drop, unsigned long long salt, const unsigned long long *seed_ptr) {
  constexpr int COLS = 256 * VPT;
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  unsigned long long seed = salt;
  if (seed_ptr) seed = salt * 0x9E3779B97F4A7C15ull + *seed_ptr;
  const float keep_scale = p_drop < 1.f ? 1.f / (1.f - p_drop) : 0.f;
  const uint32_t thr = ffk_drop_threshold(p_drop);
  for (long long row = (long long)blockIdx.x * wpb + wib; row < rows; row += (long long)gridDim.x * wpb) {
    float g[VPT][8], p[VPT][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int c0 = (i * 32 + lane) * 8;
      ld8(dy + row * COLS + c0, g[i]);
      ld8(y + row * COLS + c0, p[i]);
      uint32_t keep = 0xFFu;
      if (p_drop > 0.f) {
        const unsigned long long g4 = (unsigned long long)(row * COLS + c0) >> 2;
        keep = ffk_keep4(seed, g4, thr) | (ffk_keep4(seed, g4 + 1, thr) << 4);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (p_drop > 0.f) g[i][j] = (keep >> j) & 1u ? g[i][j] * keep_scale : 0.f;
        s += g[i][j] * p[i][j];
      }
    }
    s = warp_sum(s);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int c0 = (i * 32 + lane) * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) g[i][j] = scale * p[i][j] * (g[i][j] - s);
      st8(dx + row * COLS + c0, g[i]);
    }
  }
}

// ---------------------------------------------------------------- LayerNorm: one block per row
// cols = 8 * blockDim.x * VPT.  y = LN(a + b) * gamma + beta, xsum = a + b (when b is given).
template <int VPT>
__global__ void layernorm_fwd_vec_kernel(const bf16 *__restrict__ a, const bf16 *__restrict__ b, const bf16 *__restrict__ gamma,
                                         const bf16 *__restrict__ beta, bf16 *__restrict__ xsum, bf16 *__restrict__ y,
                                         float *__restrict__ mean, float *__restrict__ rstd, int rows, int cols, float eps) {
  // two block reductions per row (mean, then centred variance), each through its own double-buffered slot so
  // that one barrier per reduction suffices
  __shared__ float red_a[2][32], red_b[2][32];
  int parity = 0;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  float gm[VPT][8], bt[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    int c0 = (i * blockDim.x + threadIdx.x) * 8;
    if (gamma) ld8(gamma + c0, gm[i]);
    if (beta) ld8(beta + c0, bt[i]);
  }
  // the next row's 16-byte pieces are fetched into registers before this row's two reductions, so that every
  // thread keeps loads in flight across the barriers
  uint4 na[VPT], nb[VPT];
  if ((int)blockIdx.x < rows) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      long long off = (long long)blockIdx.x * cols + (i * blockDim.x + threadIdx.x) * 8;
      na[i] = *reinterpret_cast<const uint4 *>(a + off);
      if (b) nb[i] = *reinterpret_cast<const uint4 *>(b + off);
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float v[VPT][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      long long off = (long long)row * cols + (i * blockDim.x + threadIdx.x) * 8;
      unpack8(na[i], v[i]);
      if (b) {
        float w[8];
        unpack8(nb[i], w);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += w[j];
        if (xsum) {
          st8(xsum + off, v[i]);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = bf2f(f2bf(v[i][j]));  // statistics of the value backward will read
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[i][j];
    }
    const int next = row + gridDim.x;
    if (next < rows) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        long long off = (long long)next * cols + (i * blockDim.x + threadIdx.x) * 8;
        na[i] = *reinterpret_cast<const uint4 *>(a + off);
        if (b) nb[i] = *reinterpret_cast<const uint4 *>(b + off);
      }
    }
    s = warp_sum(s);
    if (lane == 0) red_a[parity][wid] = s;
    __syncthreads();
    float tot = 0.f;
    for (int k = 0; k < nw; ++k) tot += red_a[parity][k];
    const float mu = tot / cols;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) { float d = v[i][j] - mu; ss += d * d; }
    ss = warp_sum(ss);
    if (lane == 0) red_b[parity][wid] = ss;
    __syncthreads();
    float tot2 = 0.f;
    for (int k = 0; k < nw; ++k) tot2 += red_b[parity][k];
    parity ^= 1;
    const float rs = rsqrtf(tot2 / cols + eps);
    if (threadIdx.x == 0) {
      if (mean) mean[row] = mu;
      if (rstd) rstd[row] = rs;
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      long long off = (long long)row * cols + (i * blockDim.x + threadIdx.x) * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float o = (v[i][j] - mu) * rs;
        v[i][j] = gamma ? o * gm[i][j] + (beta ? bt[i][j] : 0.f) : o;
      }
      st8(y + off, v[i]);
    }
  }
}
// LayerNorm forward, one warp per row: cols = 256 * VPT (up to 2048).  A lane holds VPT 16-byte pieces of the row
// (piece i of lane l = elements [(i * 32 + l) * 8, +8): coalesced), all loaded before anything is computed, so a
// warp has VPT (2 VPT with a fused add) loads in flight and the two row reductions are warp shuffles: no
// block-wide barrier after the one that stages gamma / beta in shared memory.
template <int VPT>
__global__ void __launch_bounds__(256, 2) layernorm_fwd_warp_kernel(const bf16 *__restrict__ a, const bf16 *__restrict__ b,
                                                                    const bf16 *__restrict__ gamma, const bf16 *__restrict__ beta,
                                                                    bf16 *__restrict__ xsum, bf16 *__restrict__ y, float *__restrict__ mean,
                                                                    float *__restrict__ rstd, int rows, float eps) {
  constexpr int COLS = 256 * VPT, NV = 32 * VPT;
  __shared__ uint4 g_s[NV], b_s[NV];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  for (int i = threadIdx.x; i < NV; i += blockDim.x) {
    if (gamma) g_s[i] = reinterpret_cast<const uint4 *>(gamma)[i];
    if (beta) b_s[i] = reinterpret_cast<const uint4 *>(beta)[i];
  }
  __syncthreads();
  for (int row = blockIdx.x * wpb + wid; row < rows; row += gridDim.x * wpb) {
    const long long base = (long long)row * COLS;
    const uint4 *ar = reinterpret_cast<const uint4 *>(a + base);
    uint4 ua[VPT], ub[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) ua[i] = ar[i * 32 + lane];
    if (b) {
      const uint4 *br = reinterpret_cast<const uint4 *>(b + base);
#pragma unroll
      for (int i = 0; i < VPT; ++i) ub[i] = br[i * 32 + lane];
    }
    float v[VPT][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      unpack8(ua[i], v[i]);
      if (b) {
        float w[8];
        unpack8(ub[i], w);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += w[j];
        if (xsum) {
          st8(xsum + base + (i * 32 + lane) * 8, v[i]);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = bf2f(f2bf(v[i][j]));  // statistics of the value backward will read
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[i][j];
    }
    const float mu = warp_sum(s) * (1.0f / COLS);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) { float d = v[i][j] - mu; ss += d * d; }
    const float rs = rsqrtf(warp_sum(ss) * (1.0f / COLS) + eps);
    if (lane == 0) {
      if (mean) mean[row] = mu;
      if (rstd) rstd[row] = rs;
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      float g8[8], b8[8];
      if (gamma) unpack8(g_s[i * 32 + lane], g8);
      if (beta) unpack8(b_s[i * 32 + lane], b8);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float o = (v[i][j] - mu) * rs;
        v[i][j] = gamma ? o * g8[j] + (beta ? b8[j] : 0.f) : o;
      }
      st8(y + base + (i * 32 + lane) * 8, v[i]);
    }
  }
}
// dx (and optionally dx2) (+)= LN backward; per-block partial sums of dgamma/dbeta -> partial[2][grid][cols]
template <int VPT>
__global__ void layernorm_bwd_vec_kernel(const bf16 *__restrict__ dy, const bf16 *__restrict__ x, const bf16 *__restrict__ gamma,
                                         const float *__restrict__ mean, const float *__restrict__ rstd, bf16 *__restrict__ dx,
                                         bf16 *__restrict__ dx2, float *__restrict__ partial, int rows, int cols, int acc1, int acc2) {
  // the two row sums are reduced together through a double-buffered slot: one barrier per row
  __shared__ float2 red2[2][32];
  int parity = 0;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  float gm[VPT][8], dg[VPT][8], db[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    int c0 = (i * blockDim.x + threadIdx.x) * 8;
    if (gamma) ld8(gamma + c0, gm[i]);
#pragma unroll
    for (int j = 0; j < 8; ++j) { dg[i][j] = 0.f; db[i][j] = 0.f; if (!gamma) gm[i][j] = 1.f; }
  }
  // the next row's pieces of dy and x travel while this row is reduced and written (see the forward kernel)
  uint4 ng[VPT], nx[VPT];
  if ((int)blockIdx.x < rows) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      long long off = (long long)blockIdx.x * cols + (i * blockDim.x + threadIdx.x) * 8;
      ng[i] = *reinterpret_cast<const uint4 *>(dy + off);
      nx[i] = *reinterpret_cast<const uint4 *>(x + off);
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mu = mean[row], rs = rstd[row];
    float g[VPT][8], xh[VPT][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      unpack8(ng[i], g[i]);
      unpack8(nx[i], xh[i]);
    }
    const int next = row + gridDim.x;
    if (next < rows) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        long long off = (long long)next * cols + (i * blockDim.x + threadIdx.x) * 8;
        ng[i] = *reinterpret_cast<const uint4 *>(dy + off);
        nx[i] = *reinterpret_cast<const uint4 *>(x + off);
      }
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xh[i][j] = (xh[i][j] - mu) * rs;
        dg[i][j] += g[i][j] * xh[i][j];
        db[i][j] += g[i][j];
        g[i][j] *= gm[i][j];
        s1 += g[i][j];
        s2 += g[i][j] * xh[i][j];
      }
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    if (lane == 0) red2[parity][wid] = make_float2(s1, s2);
    __syncthreads();
    float t1 = 0.f, t2 = 0.f;
    for (int k = 0; k < nw; ++k) { float2 q = red2[parity][k]; t1 += q.x; t2 += q.y; }
    parity ^= 1;
    const float m1 = t1 / cols, m2 = t2 / cols;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      long long off = (long long)row * cols + (i * blockDim.x + threadIdx.x) * 8;
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rs * (g[i][j] - m1 - xh[i][j] * m2);
      if (dx2) {
        float t[8];
        if (acc2) {
          ld8(dx2 + off, t);
#pragma unroll
          for (int j = 0; j < 8; ++j) t[j] += o[j];
          st8(dx2 + off, t);
        } else st8(dx2 + off, o);
      }
      if (acc1) {
        float t[8];
        ld8(dx + off, t);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += t[j];
      }
      st8(dx + off, o);
    }
  }
  if (partial) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int c0 = (i * blockDim.x + threadIdx.x) * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        partial[(long long)blockIdx.x * cols + c0 + j] = dg[i][j];
        partial[((long long)gridDim.x + blockIdx.x) * cols + c0 + j] = db[i][j];
      }
    }
  }
}

// ---------------------------------------------------------------- bias / activation backward
// block (32, 8): thread (tx, ty) owns columns [blockIdx.x*256 + tx*8, +8) of rows ty, ty+8*gridDim.y, ...
// dz = dy * act'(saved); partial[blockIdx.y][col] = column sums over this block's rows.
// With drop_p > 0 the incoming gradient first goes back through the dropout that the forward GEMM epilogue
// applied after the activation (mask regenerated from (seed, flat index)).
static __global__ void bias_act_bwd_vec_kernel(const bf16 *__restrict__ dy, const bf16 *__restrict__ saved, bf16 *__restrict__ dz,
                                        float *__restrict__ partial, int rows, int cols, int act, float drop_p,
                                        unsigned long long drop_salt, const unsigned long long *drop_seed_ptr) {
  const unsigned long long dseed = drop_seed_ptr ? drop_salt * 0x9E3779B97F4A7C15ull + *drop_seed_ptr : drop_salt;
  const uint32_t dthr = ffk_drop_threshold(drop_p);
  const float dscale = drop_p > 0.f ? 1.f / (1.f - drop_p) : 1.f;
  __shared__ float red[8][32][9];
  const int c0 = blockIdx.x * 256 + threadIdx.x * 8;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (c0 < cols) {
    for (int r = blockIdx.y * 8 + threadIdx.y; r < rows; r += gridDim.y * 8) {
      long long off = (long long)r * cols + c0;
      float g[8];
      ld8(dy + off, g);
      if (drop_p > 0.f) {
        const uint32_t k0 = ffk_keep4(dseed, (unsigned long long)(off >> 2), dthr), k1 = ffk_keep4(dseed, (unsigned long long)(off >> 2) + 1, dthr);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          g[j] = ((k0 >> j) & 1u) ? g[j] * dscale : 0.f;
          g[4 + j] = ((k1 >> j) & 1u) ? g[4 + j] * dscale : 0.f;
        }
      }
      if (act != ACT_NONE) {
        float sv[8];
        ld8(saved + off, sv);
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] *= act_bwd(sv[j], act);
      }
      if (dz) st8(dz + off, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += g[j];
    }
  }
  if (!partial) return;
#pragma unroll
  for (int j = 0; j < 8; ++j) red[threadIdx.y][threadIdx.x][j] = acc[j];
  __syncthreads();
  if (threadIdx.y == 0 && c0 < cols) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) s += red[k][threadIdx.x][j];
      partial[(long long)blockIdx.y * cols + c0 + j] = s;
    }
  }
}

// out[c] (+)= sum over p < nparts of partial[p][c], for two stacked partial arrays at once (the second at
// partial + nparts * cols, out2 may be null).  Block (32 columns x 32 part lanes): a lane strides over the parts with
// independent loads, the lanes' sums meet in shared memory in a fixed order (deterministic).  The one-thread-per-column
// form took 60 us for 1184 parts of 768 columns: three blocks, each thread a chain of 1184 dependent additions.
template <typename T>
__global__ void fold_partials_kernel(const float *__restrict__ partial, int nparts, int cols, T *out, T *out2, int accumulate) {
  __shared__ float s1[32][33], s2[32][33];
  const int tx = threadIdx.x, ty = threadIdx.y, c = blockIdx.x * 32 + tx;
  float a = 0.f, b = 0.f;
  if (c < cols) {
    const float *p1 = partial + c, *p2 = partial + (long long)nparts * cols + c;
#pragma unroll 4
    for (int p = ty; p < nparts; p += 32) {
      a += p1[(long long)p * cols];
      if (out2) b += p2[(long long)p * cols];
    }
  }
  s1[ty][tx] = a;
  s2[ty][tx] = b;
  __syncthreads();
  if (ty == 0 && c < cols) {
    float ta = 0.f, tb = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) { ta += s1[k][tx]; tb += s2[k][tx]; }
    if (out) out[c] = (T)(accumulate ? (float)out[c] + ta : ta);
    if (out2) out2[c] = (T)(accumulate ? (float)out2[c] + tb : tb);
  }
}

}  // namespace vec
