// Training metrics accumulated on the device.
//
// One launch adds a batch's contribution to every requested metric into a small device-resident accumulator, so a
// training loop can track accuracy and losses without a host synchronisation per step (the host reads the
// accumulator when it wants the numbers).  Counterpart of update_metrics_sparse_label_kernel /
// update_metrics_label_kernel (lib/kernels/src/cuda/metrics_functions.cu:48-98), which add into a CUDAPerfMetrics
// struct with global atomics, one thread per sample; here one warp reads a sample's row coalesced and a block adds
// its partial sums with one atomic per metric.  The definitions are the reference's: squared and absolute errors are
// summed over a sample's classes (not averaged), sparse labels are compared as one-hot targets, and probabilities
// are clamped at 1e-8 before the logarithm.
#include "common.cuh"

namespace {

// accumulator slots (doubles)
enum { M_ALL = 0, M_CORRECT, M_CCE, M_SCCE, M_MSE, M_RMSE, M_MAE, M_SLOTS };
constexpr float LOG_MIN_VALUE = 1e-8f;
// request bits
enum { F_ACCURACY = 1, F_CCE = 2, F_SCCE = 4, F_MSE = 8, F_RMSE = 16, F_MAE = 32 };

template <typename T> __device__ __forceinline__ float ldm(const T *p, long long i);
template <> __device__ __forceinline__ float ldm<float>(const float *p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldm<bf16>(const bf16 *p, long long i) { return bf2f(p[i]); }

// pred [n, c]; sparse: label_i [n] class ids (int32 or int64 by `label64`); dense: label_d [n, c] targets (type T).
template <typename T>
__global__ void metrics_kernel(const T *__restrict__ pred, const void *__restrict__ label_i, const T *__restrict__ label_d, int label64,
                               long long n, int c, int flags, double *__restrict__ acc) {
  __shared__ float part[M_SLOTS][8];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  float sums[M_SLOTS];
#pragma unroll
  for (int i = 0; i < M_SLOTS; ++i) sums[i] = 0.f;
  for (long long row = (long long)blockIdx.x * wpb + wid; row < n; row += (long long)gridDim.x * wpb) {
    const T *p = pred + row * c;
    // argmax of the prediction (first maximum wins, as torch.argmax)
    float best = -INFINITY;
    int besti = 0x7fffffff;
    float cce = 0.f, se = 0.f, ae = 0.f, tbest = -INFINITY;
    int tbesti = 0x7fffffff;
    long long sparse_t = -1;
    if (!label_d) sparse_t = label64 ? ((const long long *)label_i)[row] : (long long)((const int *)label_i)[row];
    for (int j = lane; j < c; j += 32) {
      const float v = ldm<T>(p, j);
      if (v > best) { best = v; besti = j; }
      float t;
      if (label_d) {
        t = ldm<T>(label_d, row * c + j);
        if (t > tbest) { tbest = t; tbesti = j; }
        cce -= t * logf(fmaxf(v, LOG_MIN_VALUE));
      } else {
        t = (long long)j == sparse_t ? 1.f : 0.f;
      }
      const float d = v - t;
      se += d * d;
      ae += fabsf(d);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
      if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
      const float tb = __shfl_xor_sync(0xffffffffu, tbest, o);
      const int ti = __shfl_xor_sync(0xffffffffu, tbesti, o);
      if (tb > tbest || (tb == tbest && ti < tbesti)) { tbest = tb; tbesti = ti; }
      cce += __shfl_xor_sync(0xffffffffu, cce, o);
      se += __shfl_xor_sync(0xffffffffu, se, o);
      ae += __shfl_xor_sync(0xffffffffu, ae, o);
    }
    if (lane == 0) {
      sums[M_ALL] += 1.f;
      if (label_d) {
        if (flags & F_ACCURACY) sums[M_CORRECT] += besti == tbesti ? 1.f : 0.f;
        if (flags & F_CCE) sums[M_CCE] += cce;
      } else {
        const long long t = sparse_t;
        if (flags & F_ACCURACY) sums[M_CORRECT] += (long long)besti == t ? 1.f : 0.f;
        if ((flags & F_SCCE) && t >= 0 && t < c) sums[M_SCCE] -= logf(fmaxf(ldm<T>(p, t), LOG_MIN_VALUE));
      }
      if (flags & F_MSE) sums[M_MSE] += se;
      if (flags & F_RMSE) sums[M_RMSE] += sqrtf(se);
      if (flags & F_MAE) sums[M_MAE] += ae;
    }
  }
  if (lane == 0 && wid < 8) {
#pragma unroll
    for (int i = 0; i < M_SLOTS; ++i) part[i][wid] = sums[i];
  }
  __syncthreads();
  if (threadIdx.x < M_SLOTS) {
    float s = 0.f;
    for (int w = 0; w < wpb && w < 8; ++w) s += part[threadIdx.x][w];
    if (s != 0.f) atomicAdd(acc + threadIdx.x, (double)s);
  }
}

}  // namespace

// acc: 8 doubles on the device {samples, correct, cce, sparse cce, mse, rmse, mae, unused}, added to (zero it to reset).
// pred_dt: 0 fp32, 1 bf16.  Exactly one of label_sparse (label_dt: 2 int32, 3 int64) and label_dense (same dtype as
// pred) is given.  flags: 1 accuracy, 2 cce, 4 sparse cce, 8 mse, 16 rmse, 32 mae.
FFK_API int ffk_metrics_update(const void *pred, const void *label_sparse, const void *label_dense, long long n, int c, int pred_dt,
                               int label_dt, int flags, double *acc, cudaStream_t st) {
  if (n <= 0 || c <= 0) return 0;
  if ((label_sparse == nullptr) == (label_dense == nullptr)) return -2;
  if (label_sparse && label_dt != 2 && label_dt != 3) return -2;
  long long want = (n + 7) / 8;
  const int grid = (int)(want < 148 * 8 ? want : 148 * 8);
  if (pred_dt == 0)
    metrics_kernel<float><<<grid, 256, 0, st>>>((const float *)pred, label_sparse, (const float *)label_dense, label_dt == 3, n, c, flags, acc);
  else if (pred_dt == 1)
    metrics_kernel<bf16><<<grid, 256, 0, st>>>((const bf16 *)pred, label_sparse, (const bf16 *)label_dense, label_dt == 3, n, c, flags, acc);
  else
    return -2;
  return (int)cudaGetLastError();
}
