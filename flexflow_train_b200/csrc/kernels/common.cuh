// Shared device/host helpers for the sm_100a kernel library.
//
// Everything in this library is launched through plain C entry points
// (extern "C", prefix ffk_) that take raw device pointers and a cudaStream_t,
// so the Python side can call them through ctypes with tensor.data_ptr() and
// CUDA graphs can capture them.  No entry point allocates device memory.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define FFK_API extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

// ---------------------------------------------------------------------------
// Error reporting.  Kernels never trap: a bounded wait that runs out records a
// code here and the kernel returns normally; the host reads it on demand.
// ---------------------------------------------------------------------------
enum FfkErr : int {
  FFK_OK = 0,
  FFK_ERR_TIMEOUT_PRODUCER = 1,
  FFK_ERR_TIMEOUT_MMA = 2,
  FFK_ERR_TIMEOUT_EPILOGUE = 3,
  FFK_ERR_TIMEOUT_PEER = 4,
  FFK_ERR_BAD_ARG = 5,
};

__device__ __forceinline__ uint64_t ffk_globaltimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ float bf2f(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ bf16 f2bf(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ uint32_t pack_bf162(float a, float b) {
  bf162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ float2 unpack_bf162(uint32_t u) {
  bf162 v = *reinterpret_cast<bf162 *>(&u);
  return __bfloat1622float2(v);
}

// Activation codes shared by the GEMM epilogue and the elementwise kernels.
enum FfkAct : int { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2, ACT_SIGMOID = 3, ACT_TANH = 4 };

__device__ __forceinline__ float act_fwd(float x, int act) {
  switch (act) {
    case ACT_RELU: return x > 0.f ? x : 0.f;
    case ACT_GELU: return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
    case ACT_SIGMOID: return 1.f / (1.f + __expf(-x));
    case ACT_TANH: return tanhf(x);
    default: return x;
  }
}
// derivative given the pre-activation x (GELU) or, where it suffices, the output y
__device__ __forceinline__ float act_bwd(float x_or_y, int act) {
  switch (act) {
    case ACT_RELU: return x_or_y > 0.f ? 1.f : 0.f;                // from y or x
    case ACT_GELU: {                                                 // from x
      float x = x_or_y;
      float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
      float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
      return cdf + x * pdf;
    }
    case ACT_SIGMOID: return x_or_y * (1.f - x_or_y);               // from y
    case ACT_TANH: return 1.f - x_or_y * x_or_y;                    // from y
    default: return 1.f;
  }
}

// Counter-based RNG (one 32-bit draw per element): a 2-round multiply-xorshift
// hash of (seed, element index).  Forward and backward of dropout regenerate
// the same mask from (seed, index), so no mask tensor is stored.
__device__ __forceinline__ uint32_t ffk_hash_rng(uint64_t seed, uint64_t idx) {
  uint64_t z = idx * 0x9E3779B97F4A7C15ull + seed;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return (uint32_t)(z >> 32);
}
__device__ __forceinline__ float ffk_uniform01(uint64_t seed, uint64_t idx) {
  return (ffk_hash_rng(seed, idx) >> 8) * (1.0f / 16777216.0f);
}
// Dropout masks: one 32-bit word per aligned group of four elements from two multiply-fold steps of (seed, group index),
// then one odd multiplier per element of the group; element j of group g is kept iff word(g) * FFK_RC[j] (mod 2^32) is at
// least p * 2^32 (p rounded down to a multiple of 2^-16).  About sixteen instructions per four elements: the 64-bit
// multiply-xorshift generator this replaces cost about forty and made the dropout kernel instruction-bound (2.4 TB/s).
__device__ __forceinline__ uint32_t ffk_group_word(uint64_t seed, uint64_t group) {
  const uint32_t a = (uint32_t)group * 0xB5297A4Du + ((uint32_t)seed + (uint32_t)(group >> 32) * 0x9E3779B9u);
  const uint64_t m = (uint64_t)a * 0xCC9E2D51u;
  return (uint32_t)m ^ (uint32_t)(m >> 32) ^ (uint32_t)(seed >> 32);
}
#define FFK_RC0 0x9E3779B1u
#define FFK_RC1 0x85EBCA6Bu
#define FFK_RC2 0xC2B2AE35u
#define FFK_RC3 0x27D4EB2Fu
__device__ __forceinline__ uint32_t ffk_drop_threshold(float p) { return (uint32_t)(p * 65536.0f); }   // in units of 2^-16
__device__ __forceinline__ bool ffk_keep(uint64_t seed, uint64_t idx, uint32_t thr) {
  const uint32_t w = ffk_group_word(seed, idx >> 2);
  const uint32_t j = (uint32_t)idx & 3u;
  const uint32_t c = j == 0 ? FFK_RC0 : j == 1 ? FFK_RC1 : j == 2 ? FFK_RC2 : FFK_RC3;
  return w * c >= (thr << 16);
}
// keep flags of the aligned group of four elements starting at idx4*4, one per bit of the result
__device__ __forceinline__ uint32_t ffk_keep4(uint64_t seed, uint64_t idx4, uint32_t thr) {
  const uint32_t w = ffk_group_word(seed, idx4), t = thr << 16;
  return (w * FFK_RC0 >= t ? 1u : 0u) | (w * FFK_RC1 >= t ? 2u : 0u) | (w * FFK_RC2 >= t ? 4u : 0u) | (w * FFK_RC3 >= t ? 8u : 0u);
}

static inline int ffk_blocks(long long n, int per_block, int max_blocks = 148 * 16) {
  long long b = (n + per_block - 1) / per_block;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return (int)b;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum for blocks of up to 1024 threads; `red` is >= 32 floats of smem.
__device__ __forceinline__ float block_sum(float v, float *red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  int nw = (blockDim.x + 31) >> 5;
  float r = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (w == 0) r = warp_sum(r);
  if (threadIdx.x == 0) red[0] = r;
  __syncthreads();
  return red[0];
}
__device__ __forceinline__ float block_max(float v, float *red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  int nw = (blockDim.x + 31) >> 5;
  float r = (threadIdx.x < nw) ? red[threadIdx.x] : -INFINITY;
  if (w == 0) r = warp_max(r);
  if (threadIdx.x == 0) red[0] = r;
  __syncthreads();
  return red[0];
}
