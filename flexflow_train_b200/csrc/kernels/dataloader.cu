// dataloader.cu -- batch assembly on the device: the rows of a batch are gathered by sample index straight out of the
// data set, which lives in page-locked host memory that the GPU reads over PCIe / C2C through its unified address (no
// staging copy on the host, no host-side gather for shuffled epochs).  Counterpart of the reference's data loader kernels
// (bindings/python/old/flexflow_dataloader.cu: load_input from zero-copy memory into the batch tensor).
#include "common.cuh"

namespace {

// dst[i, :] = src[idx[i], :] for rows of `vec_per_row` 16-byte vectors; idx == nullptr: rows first .. first + n - 1
__global__ void load_rows_vec_kernel(const uint4 *__restrict__ src, const long long *__restrict__ idx, uint4 *__restrict__ dst, long long n,
                                     long long vec_per_row, long long first, long long num_samples) {
  const long long total = n * vec_per_row;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long i = t / vec_per_row, v = t - i * vec_per_row;
    long long row = idx ? idx[i] : first + i;
    if (row < 0 || row >= num_samples) row = ((row % num_samples) + num_samples) % num_samples;   // wrap instead of faulting
    dst[t] = src[row * vec_per_row + v];
  }
}
__global__ void load_rows_byte_kernel(const unsigned char *__restrict__ src, const long long *__restrict__ idx, unsigned char *__restrict__ dst,
                                      long long n, long long row_bytes, long long first, long long num_samples) {
  const long long total = n * row_bytes;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long i = t / row_bytes, v = t - i * row_bytes;
    long long row = idx ? idx[i] : first + i;
    if (row < 0 || row >= num_samples) row = ((row % num_samples) + num_samples) % num_samples;
    dst[t] = src[row * row_bytes + v];
  }
}

}  // namespace

// src: data set [num_samples, row_bytes] in page-locked, device-accessible host memory (or device memory);
// idx: device array of n sample indices (int64) or null for the contiguous range starting at `first`; dst: device batch.
FFK_API int ffk_load_rows(const void *src, const void *idx, void *dst, long long n, long long row_bytes, long long first, long long num_samples,
                          cudaStream_t st) {
  if (n <= 0 || row_bytes <= 0) return 0;
  if (num_samples <= 0) return -2;
  const bool vec = row_bytes % 16 == 0 && (((uintptr_t)src) & 15) == 0 && (((uintptr_t)dst) & 15) == 0;
  if (vec) {
    const long long total = n * (row_bytes / 16);
    load_rows_vec_kernel<<<ffk_blocks(total, 256), 256, 0, st>>>((const uint4 *)src, (const long long *)idx, (uint4 *)dst, n, row_bytes / 16, first,
                                                                 num_samples);
  } else {
    const long long total = n * row_bytes;
    load_rows_byte_kernel<<<ffk_blocks(total, 256), 256, 0, st>>>((const unsigned char *)src, (const long long *)idx, (unsigned char *)dst, n,
                                                                  row_bytes, first, num_samples);
  }
  return (int)cudaGetLastError();
}
