// comm_kernels.cu -- collectives written as kernels over NVLink peer memory.
//
// The reference expresses all parallelism with four parallel operators (Repartition, Combine, Replicate,
// Reduction; lib/op-attrs/include/op-attrs/ops/{repartition,combine,replicate,reduction}_attrs.dtg.toml) but has
// no device implementation of their data movement, and its only collective is one NCCL all-reduce per weight
// before the optimizer (lib/kernels/src/cuda/optimizer_kernels.cu:87-88, 180-186).  Here every rank maps its
// peers' symmetric buffers (CUDA IPC) and the kernels below move and reduce data with plain loads and stores
// over NVLink 5 / NVSwitch:
//   * grad_allreduce_scale  -- backward of Replicate on weights: two-shot all-reduce fused with the gradient
//                              scale, in place on the gradient arena;
//   * push_rows             -- forward of Combine (all-gather) as a push into every peer's staging buffer with
//                              per-source ready flags that the consuming GEMM waits on;
//   * reduce_partials       -- the reduction half of Reduction after a GEMM whose epilogue scattered its
//                              partial tiles to the owning ranks;
//   * alltoall_embedding    -- Repartition around model-parallel embedding tables: gather rows for every
//                              rank's samples from the local tables straight into the owners' buffers;
//   * signal / wait         -- flag exchange used as a device-side barrier.
// No multimem / NVLS is used: plain peer accesses keep a failed rank from faulting its peers' GPUs.
//
// Flags.  Each rank owns an array of 64-bit flags in symmetric memory; flag[s] on rank d is written only by
// rank s (st.release.sys after __threadfence_system) and carries a monotonically increasing epoch, so nothing
// is ever reset and a CUDA graph can replay the kernels (the epoch lives in device memory and is bumped by
// the kernel itself).  Every wait is bounded (~2 s): on expiry the kernel records FFK_ERR_TIMEOUT_PEER in the
// status word and returns.
#include <cstring>

#include "common.cuh"

namespace {

constexpr int MAX_RANKS = 8;
constexpr uint64_t PEER_WAIT_NS = 2000000000ull;

struct PeerPtrs {
  void *p[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(unsigned long long *p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// bounded wait until *flag >= target; false on timeout
__device__ __forceinline__ bool wait_flag(const unsigned long long *flag, unsigned long long target, int *status) {
  if (ld_acquire_sys(flag) >= target) return true;
  uint64_t t0 = ffk_globaltimer();
  while (true) {
    if (ld_acquire_sys(flag) >= target) return true;
    if (ffk_globaltimer() - t0 > PEER_WAIT_NS) {
      if (status) atomicCAS(status, 0, (int)FFK_ERR_TIMEOUT_PEER);
      return false;
    }
    __nanosleep(200);
  }
}

// ---------------------------------------------------------------- barrier
// One block.  Thread p signals peer p and waits for peer p's signal.  `epoch_ctr` (device memory, local)
// holds the last epoch used on this flag row; all ranks call in lock step so the counters agree.
__global__ void signal_wait_kernel(PeerPtrs flags, int flag_base, int rank, int world, unsigned long long *epoch_ctr, int *status) {
  __shared__ unsigned long long epoch;
  if (threadIdx.x == 0) epoch = *epoch_ctr + 1;
  __syncthreads();
  const int p = threadIdx.x;
  if (p < world) {
    __threadfence_system();
    st_release_sys((unsigned long long *)flags.p[p] + flag_base + rank, epoch);
    wait_flag((const unsigned long long *)flags.p[rank] + flag_base + p, epoch, status);
  }
  __syncthreads();
  if (threadIdx.x == 0) *epoch_ctr = epoch;
}

// ---------------------------------------------------------------- grad all-reduce + scale (F3)
// buf.p[r] = rank r's gradient arena (same layout everywhere), n elements.  Rank `rank` owns the slice
// [rank*chunk, (rank+1)*chunk): it sums that slice over all ranks, scales it and writes the result into
// every rank's arena.  A start barrier (gradients complete everywhere) and an end barrier (results complete
// everywhere) are folded into the kernel: block 0 exchanges the flags, the other blocks wait on a local word.
template <typename T>
__device__ __forceinline__ void ld8f(const T *p, float *v);
template <>
__device__ __forceinline__ void ld8f<bf16>(const bf16 *p, float *v) {
  uint4 u = *reinterpret_cast<const uint4 *>(p);
  float2 a = unpack_bf162(u.x), b = unpack_bf162(u.y), c = unpack_bf162(u.z), d = unpack_bf162(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
template <>
__device__ __forceinline__ void ld8f<float>(const float *p, float *v) {
  float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <typename T>
__device__ __forceinline__ void st8f(T *p, const float *v);
template <>
__device__ __forceinline__ void st8f<bf16>(bf16 *p, const float *v) {
  *reinterpret_cast<uint4 *>(p) = make_uint4(pack_bf162(v[0], v[1]), pack_bf162(v[2], v[3]), pack_bf162(v[4], v[5]), pack_bf162(v[6], v[7]));
}
template <>
__device__ __forceinline__ void st8f<float>(float *p, const float *v) {
  *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4 *>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

struct AllReduceSync {
  unsigned long long *epoch_ctr;  // local: last epoch used (two epochs per call)
  unsigned int *started;          // local: set by block 0 once all peers signalled "gradients ready"
  unsigned int *blocks_done;      // local: blocks that finished their slice
};

// Optimizer fused into the all-reduce (sharded update): the rank that reduced a slice of the gradient also owns
// that slice of the fp32 master weights and moments, applies the update there and sends the new bf16 weights
// (not the gradient) to every rank.  The update is thereby done once per element instead of once per rank.
struct UpdateArgs {
  float *w, *m, *v;        // local fp32 master weights and optimizer state (whole arena; only owned slices are touched)
  PeerPtrs shadow;         // bf16 weight arenas of all ranks
  const float *alpha_ptr;  // Adam: bias-corrected step size of this step (device memory)
  int kind;                // 0 Adam, 1 SGD
  float lr, beta1, beta2, eps, wd, momentum;
  int nesterov;
};

__device__ __forceinline__ void fused_update8(const UpdateArgs &u, float alpha_t, long long e, const float *g, int rank, int world) {
  float w[8], o[8];
  *reinterpret_cast<float4 *>(w) = *reinterpret_cast<const float4 *>(u.w + e);
  *reinterpret_cast<float4 *>(w + 4) = *reinterpret_cast<const float4 *>(u.w + e + 4);
  if (u.kind == 0) {
    float m[8], v[8];
    *reinterpret_cast<float4 *>(m) = *reinterpret_cast<const float4 *>(u.m + e);
    *reinterpret_cast<float4 *>(m + 4) = *reinterpret_cast<const float4 *>(u.m + e + 4);
    *reinterpret_cast<float4 *>(v) = *reinterpret_cast<const float4 *>(u.v + e);
    *reinterpret_cast<float4 *>(v + 4) = *reinterpret_cast<const float4 *>(u.v + e + 4);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float gt = g[j] + u.wd * w[j];
      m[j] = u.beta1 * m[j] + (1.f - u.beta1) * gt;
      v[j] = u.beta2 * v[j] + (1.f - u.beta2) * gt * gt;
      w[j] -= alpha_t * m[j] / (sqrtf(v[j]) + u.eps);
    }
    *reinterpret_cast<float4 *>(u.m + e) = *reinterpret_cast<float4 *>(m);
    *reinterpret_cast<float4 *>(u.m + e + 4) = *reinterpret_cast<float4 *>(m + 4);
    *reinterpret_cast<float4 *>(u.v + e) = *reinterpret_cast<float4 *>(v);
    *reinterpret_cast<float4 *>(u.v + e + 4) = *reinterpret_cast<float4 *>(v + 4);
  } else {
    float mo[8];
    if (u.momentum > 0.f) {
      *reinterpret_cast<float4 *>(mo) = *reinterpret_cast<const float4 *>(u.m + e);
      *reinterpret_cast<float4 *>(mo + 4) = *reinterpret_cast<const float4 *>(u.m + e + 4);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float gt = g[j] + u.wd * w[j];
      if (u.momentum > 0.f) {
        mo[j] = mo[j] * u.momentum + gt;
        gt = u.nesterov ? gt + u.momentum * mo[j] : mo[j];
      }
      w[j] -= u.lr * gt;
    }
    if (u.momentum > 0.f) {
      *reinterpret_cast<float4 *>(u.m + e) = *reinterpret_cast<float4 *>(mo);
      *reinterpret_cast<float4 *>(u.m + e + 4) = *reinterpret_cast<float4 *>(mo + 4);
    }
  }
  *reinterpret_cast<float4 *>(u.w + e) = *reinterpret_cast<float4 *>(w);
  *reinterpret_cast<float4 *>(u.w + e + 4) = *reinterpret_cast<float4 *>(w + 4);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = w[j];
#pragma unroll
  for (int k = 0; k < MAX_RANKS; ++k)
    if (k < world) st8f((bf16 *)u.shadow.p[(rank + k) % world] + e, o);
}

template <typename T, bool UPDATE>
__global__ void allreduce_scale_kernel(PeerPtrs buf, PeerPtrs flags, int flag_base, long long offset, long long n, float scale, int rank,
                                       int world, AllReduceSync sync, int *status, UpdateArgs upd) {
  __shared__ unsigned long long epoch;
  __shared__ int go;
  if (threadIdx.x == 0) epoch = *sync.epoch_ctr + 1;
  __syncthreads();
  // ---- start barrier
  if (blockIdx.x == 0) {
    if ((int)threadIdx.x < world) {
      __threadfence_system();
      st_release_sys((unsigned long long *)flags.p[threadIdx.x] + flag_base + rank, epoch);
      wait_flag((const unsigned long long *)flags.p[rank] + flag_base + threadIdx.x, epoch, status);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      atomicExch(sync.started, (unsigned int)epoch);
    }
  }
  if (threadIdx.x == 0) {
    uint64_t t0 = ffk_globaltimer();
    go = 1;
    while (atomicAdd(sync.started, 0u) != (unsigned int)epoch) {
      if (ffk_globaltimer() - t0 > PEER_WAIT_NS || *status != 0) { go = 0; break; }
      __nanosleep(100);
    }
  }
  __syncthreads();
  if (go) {
    // ---- reduce my slice, write it everywhere
    const float alpha_t = (UPDATE && upd.alpha_ptr) ? *upd.alpha_ptr : upd.lr;
    const long long nvec = n / 8;
    const long long per = (nvec + world - 1) / world;
    const long long v0 = per * rank, v1 = min(nvec, per * (rank + 1));
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = v0 + (long long)blockIdx.x * blockDim.x + threadIdx.x;
    // main loop: four vectors per trip so that 4 x (world - 1) remote 16-byte loads are in flight per thread --
    // a peer load takes a few microseconds over NVLink and the link is only filled by many outstanding requests
    for (; i + 3 * stride < v1; i += 4 * stride) {
      float acc[4][8], t[8];
#pragma unroll
      for (int u = 0; u < 4; ++u) ld8f((const T *)buf.p[rank] + offset + (i + u * stride) * 8, acc[u]);
#pragma unroll
      for (int k = 1; k < MAX_RANKS; ++k) {
        if (k < world) {
          const T *src = (const T *)buf.p[(rank + k) % world] + offset;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            ld8f(src + (i + u * stride) * 8, t);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[u][j] += t[j];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[u][j] *= scale;
        if (UPDATE) {
          fused_update8(upd, alpha_t, offset + (i + u * stride) * 8, acc[u], rank, world);
        } else {
#pragma unroll
          for (int k = 0; k < MAX_RANKS; ++k)
            if (k < world) st8f((T *)buf.p[(rank + k) % world] + offset + (i + u * stride) * 8, acc[u]);
        }
      }
    }
    for (; i < v1; i += stride) {
      float acc[8], t[8];
      ld8f((const T *)buf.p[rank] + offset + i * 8, acc);
#pragma unroll
      for (int k = 1; k < MAX_RANKS; ++k) {
        if (k < world) {
          int peer = (rank + k) % world;
          ld8f((const T *)buf.p[peer] + offset + i * 8, t);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += t[j];
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] *= scale;
      if (UPDATE) {
        fused_update8(upd, alpha_t, offset + i * 8, acc, rank, world);
      } else {
#pragma unroll
        for (int k = 0; k < MAX_RANKS; ++k)
          if (k < world) st8f((T *)buf.p[(rank + k) % world] + offset + i * 8, acc);
      }
    }
    // tail (n % 8 elements) is handled by rank 0 (the fused update requires n % 8 == 0)
    if (!UPDATE && rank == 0 && blockIdx.x == 0) {
      for (long long i = nvec * 8 + threadIdx.x; i < n; i += blockDim.x) {
        float a = 0.f;
        for (int k = 0; k < world; ++k) a += (float)((const T *)buf.p[k])[offset + i];
        for (int k = 0; k < world; ++k) ((T *)buf.p[k])[offset + i] = (T)(a * scale);
      }
    }
  }
  // ---- end barrier: the last block to finish tells the peers and waits for theirs
  __threadfence_system();
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) last = (atomicAdd(sync.blocks_done, 1u) == gridDim.x - 1);
  __syncthreads();
  if (last) {
    if ((int)threadIdx.x < world) {
      st_release_sys((unsigned long long *)flags.p[threadIdx.x] + flag_base + rank, epoch + 1);
      wait_flag((const unsigned long long *)flags.p[rank] + flag_base + threadIdx.x, epoch + 1, status);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      *sync.epoch_ctr = epoch + 1;
      *sync.blocks_done = 0;
    }
  }
}

// ---------------------------------------------------------------- all-gather as a push (F2 producer side)
// Every rank copies its `rows x row_bytes` shard into slot `rank` of each peer's staging buffer and then
// raises flag[flag_base + rank] on that peer to `epoch`.  The last block to finish raises the flags.
__global__ void push_rows_kernel(const uint4 *__restrict__ src, PeerPtrs dst, long long dst_offset_vec, long long nvec, PeerPtrs flags,
                                 int flag_base, int rank, int world, unsigned long long *epoch_ctr, unsigned int *blocks_done, int skip_self) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    uint4 v = src[i];
#pragma unroll
    for (int k = 0; k < MAX_RANKS; ++k) {
      if (k < world) {
        int peer = (rank + k) % world;
        if (skip_self && peer == rank) continue;
        ((uint4 *)dst.p[peer])[dst_offset_vec + i] = v;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) last = (atomicAdd(blocks_done, 1u) == gridDim.x - 1);
  __syncthreads();
  if (last) {
    unsigned long long epoch = *epoch_ctr + 1;
    if ((int)threadIdx.x < world) st_release_sys((unsigned long long *)flags.p[threadIdx.x] + flag_base + rank, epoch);
    __syncthreads();
    if (threadIdx.x == 0) {
      *epoch_ctr = epoch;
      *blocks_done = 0;
    }
  }
}

// ---------------------------------------------------------------- reduce-scatter, sending half
// src holds `world` consecutive pieces of nvec vectors; piece p goes into slot `rank` of peer p's staging buffer
// [world][nvec] (the layout reduce_partials_kernel sums), then flag[flag_base + rank] is raised on every peer.
__global__ void scatter_pieces_kernel(const uint4 *__restrict__ src, PeerPtrs dst, long long nvec, PeerPtrs flags, int flag_base, int rank, int world,
                                      unsigned long long *epoch_ctr, unsigned int *blocks_done) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
#pragma unroll
    for (int k = 0; k < MAX_RANKS; ++k) {
      if (k < world) {
        const int peer = (rank + k) % world;
        ((uint4 *)dst.p[peer])[(long long)rank * nvec + i] = src[(long long)peer * nvec + i];
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) last = (atomicAdd(blocks_done, 1u) == gridDim.x - 1);
  __syncthreads();
  if (last) {
    unsigned long long epoch = *epoch_ctr + 1;
    if ((int)threadIdx.x < world) st_release_sys((unsigned long long *)flags.p[threadIdx.x] + flag_base + rank, epoch);
    __syncthreads();
    if (threadIdx.x == 0) {
      *epoch_ctr = epoch;
      *blocks_done = 0;
    }
  }
}

// ---------------------------------------------------------------- reduce staged partials (F1 consumer side)
// stage holds `nsrc` partial copies [nsrc][n] written by the peers' GEMM epilogues; out = sum (+ residual).
// Waits for flag[flag_base + s] >= *epoch_ctr + 1 for every source first.
template <typename T>
__global__ void reduce_partials_kernel(const T *__restrict__ stage, const T *__restrict__ residual, T *__restrict__ out, long long n, int nsrc,
                                       const unsigned long long *flags, int flag_base, unsigned long long *epoch_ctr, unsigned int *blocks_done,
                                       int *status) {
  __shared__ int go;
  if (threadIdx.x == 0) go = 1;
  __syncthreads();
  if ((int)threadIdx.x < nsrc) {
    if (!wait_flag(flags + flag_base + threadIdx.x, *epoch_ctr + 1, status)) go = 0;
  }
  __syncthreads();
  if (go) {
    const long long nvec = n / 8;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
      float acc[8], t[8];
      ld8f(stage + i * 8, acc);
      for (int s = 1; s < nsrc; ++s) {
        ld8f(stage + (long long)s * n + i * 8, t);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += t[j];
      }
      if (residual) {
        ld8f(residual + i * 8, t);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += t[j];
      }
      st8f(out + i * 8, acc);
    }
  }
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) last = (atomicAdd(blocks_done, 1u) == gridDim.x - 1);
  __syncthreads();
  if (last && threadIdx.x == 0) {
    *epoch_ctr = *epoch_ctr + 1;
    *blocks_done = 0;
  }
}

// ---------------------------------------------------------------- all-to-all fused with the embedding gather (F4)
// Rank `rank` holds `tables_local` tables (table t of the model is local table t / world when t % world == rank).
// idx: [global_batch, num_tables] indices for ALL samples (every rank has them).  For each local table and
// every sample b, the row is read from the local table and written into the owner of sample b
// (b / local_batch) at out[owner][(b % local_batch), t, :].  Output rows are `dim` elements of T.
template <typename W, typename T, typename I>
__global__ void alltoall_embedding_fwd_kernel(const W *const *__restrict__ tables, const long long *__restrict__ entries, const I *__restrict__ idx,
                                              PeerPtrs out, int global_batch, int local_batch, int num_tables, int dim, int rank, int world) {
  const int tables_local = (num_tables - rank + world - 1) / world;
  const long long total = (long long)tables_local * global_batch * dim;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int c = (int)(i % dim);
    long long rest = i / dim;
    int b = (int)(rest % global_batch);
    int lt = (int)(rest / global_batch);
    int t = lt * world + rank;
    long long e = (long long)idx[(long long)b * num_tables + t];
    float v = (e >= 0 && e < entries[lt]) ? (float)tables[lt][e * dim + c] : 0.f;
    int owner = b / local_batch;
    ((T *)out.p[owner])[((long long)(b - owner * local_batch) * num_tables + t) * dim + c] = (T)v;
  }
}
// backward: for its local tables, each rank pulls d(out) rows for all samples from the owners and applies
// the sparse SGD update (or accumulates into a dense gradient when lr == 0 and dgrad != null).
template <typename T, typename I>
__global__ void alltoall_embedding_bwd_kernel(float *const *__restrict__ tables, float *const *__restrict__ dgrad, const long long *__restrict__ entries,
                                              const I *__restrict__ idx, PeerPtrs dout, int global_batch, int local_batch, int num_tables,
                                              int dim, int rank, int world, float lr) {
  const int tables_local = (num_tables - rank + world - 1) / world;
  const long long total = (long long)tables_local * global_batch * dim;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int c = (int)(i % dim);
    long long rest = i / dim;
    int b = (int)(rest % global_batch);
    int lt = (int)(rest / global_batch);
    int t = lt * world + rank;
    long long e = (long long)idx[(long long)b * num_tables + t];
    if (e < 0 || e >= entries[lt]) continue;
    int owner = b / local_batch;
    float g = (float)((const T *)dout.p[owner])[((long long)(b - owner * local_batch) * num_tables + t) * dim + c];
    if (dgrad) atomicAdd(dgrad[lt] + e * dim + c, g);
    else atomicAdd(tables[lt] + e * dim + c, -lr * g);
  }
}

// The same two kernels for dim % 4 == 0 (every table and staging row then starts on a 16-byte boundary): one thread
// moves four consecutive elements of a row -- one 16-byte table read, one 8- or 16-byte remote store; backward adds with
// one 16-byte vector atomic -- and the flat index is split with 32-bit arithmetic (the launcher checks that it fits).
template <typename T>
__device__ __forceinline__ void st4(T *dst, float4 v);
template <>
__device__ __forceinline__ void st4<float>(float *dst, float4 v) { *reinterpret_cast<float4 *>(dst) = v; }
template <>
__device__ __forceinline__ void st4<bf16>(bf16 *dst, float4 v) { *reinterpret_cast<uint2 *>(dst) = make_uint2(pack_bf162(v.x, v.y), pack_bf162(v.z, v.w)); }
template <typename T>
__device__ __forceinline__ float4 ld4(const T *src);
template <>
__device__ __forceinline__ float4 ld4<float>(const float *src) { return *reinterpret_cast<const float4 *>(src); }
template <>
__device__ __forceinline__ float4 ld4<bf16>(const bf16 *src) {
  const uint2 u = *reinterpret_cast<const uint2 *>(src);
  const float2 a = unpack_bf162(u.x), b = unpack_bf162(u.y);
  return make_float4(a.x, a.y, b.x, b.y);
}

template <typename T, typename I>
__global__ void alltoall_embedding_fwd_vec_kernel(const float *const *__restrict__ tables, const long long *__restrict__ entries,
                                                  const I *__restrict__ idx, PeerPtrs out, int global_batch, int local_batch, int num_tables, int dim,
                                                  int rank, int world, unsigned total_vec) {
  const unsigned dv = (unsigned)dim >> 2;
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total_vec; i += stride) {
    const unsigned c4 = i % dv;
    const unsigned rest = i / dv;
    const unsigned b = rest % (unsigned)global_batch;
    const unsigned lt = rest / (unsigned)global_batch;
    const int t = (int)lt * world + rank;
    const long long e = (long long)idx[(long long)b * num_tables + t];
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (e >= 0 && e < entries[lt]) v = *reinterpret_cast<const float4 *>(tables[lt] + e * dim + c4 * 4);
    const unsigned owner = b / (unsigned)local_batch;
    st4<T>((T *)out.p[owner] + ((long long)(b - owner * (unsigned)local_batch) * num_tables + t) * dim + c4 * 4, v);
  }
}
template <typename T, typename I>
__global__ void alltoall_embedding_bwd_vec_kernel(float *const *__restrict__ tables, float *const *__restrict__ dgrad, const long long *__restrict__ entries,
                                                  const I *__restrict__ idx, PeerPtrs dout, int global_batch, int local_batch, int num_tables,
                                                  int dim, int rank, int world, float lr, unsigned total_vec) {
  const unsigned dv = (unsigned)dim >> 2;
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total_vec; i += stride) {
    const unsigned c4 = i % dv;
    const unsigned rest = i / dv;
    const unsigned b = rest % (unsigned)global_batch;
    const unsigned lt = rest / (unsigned)global_batch;
    const int t = (int)lt * world + rank;
    const long long e = (long long)idx[(long long)b * num_tables + t];
    if (e < 0 || e >= entries[lt]) continue;
    const unsigned owner = b / (unsigned)local_batch;
    float4 g = ld4<T>((const T *)dout.p[owner] + ((long long)(b - owner * (unsigned)local_batch) * num_tables + t) * dim + c4 * 4);
    if (dgrad) {
      atomicAdd(reinterpret_cast<float4 *>(dgrad[lt] + e * dim + c4 * 4), g);
    } else {
      g.x *= -lr; g.y *= -lr; g.z *= -lr; g.w *= -lr;
      atomicAdd(reinterpret_cast<float4 *>(tables[lt] + e * dim + c4 * 4), g);
    }
  }
}

PeerPtrs make_ptrs(void *const *p, int world) {
  PeerPtrs r;
  for (int i = 0; i < MAX_RANKS; ++i) r.p[i] = i < world ? p[i] : nullptr;
  return r;
}

}  // namespace

// All entry points: `peers` arrays hold `world` device pointers (this rank's own pointer at index rank).
// `sync_words` is a small local device buffer owned by the caller: [0..1] epoch counter (u64), [2] started,
// [3] blocks_done (u32 each, zero-initialised once).

FFK_API int ffk_comm_barrier(void *const *flag_peers, int flag_base, int rank, int world, void *sync_words, int *status, cudaStream_t st) {
  if (world > MAX_RANKS) return -2;
  signal_wait_kernel<<<1, 32, 0, st>>>(make_ptrs(flag_peers, world), flag_base, rank, world, (unsigned long long *)sync_words, status);
  return (int)cudaGetLastError();
}

// In-place sum over ranks of buf[offset .. offset+n) times `scale`.  dt: 0 = fp32, 1 = bf16.  offset and the
// arena base must keep 16-byte alignment.  `blocks` bounds the SMs the collective takes from overlapping compute.
FFK_API int ffk_grad_allreduce_scale(void *const *buf_peers, void *const *flag_peers, int flag_base, long long offset, long long n, float scale,
                                     int rank, int world, void *sync_words, int *status, int dt, int blocks, cudaStream_t st) {
  if (world > MAX_RANKS || n <= 0) return world > MAX_RANKS ? -2 : 0;
  AllReduceSync s;
  s.epoch_ctr = (unsigned long long *)sync_words;
  s.started = (unsigned int *)sync_words + 2;
  s.blocks_done = (unsigned int *)sync_words + 3;
  if (blocks <= 0) blocks = 32;
  UpdateArgs none = {};
  if (dt == 1)
    allreduce_scale_kernel<bf16, false><<<blocks, 512, 0, st>>>(make_ptrs(buf_peers, world), make_ptrs(flag_peers, world), flag_base, offset, n, scale,
                                                                rank, world, s, status, none);
  else if (dt == 0)
    allreduce_scale_kernel<float, false><<<blocks, 512, 0, st>>>(make_ptrs(buf_peers, world), make_ptrs(flag_peers, world), flag_base, offset, n, scale,
                                                                 rank, world, s, status, none);
  else return -2;
  return (int)cudaGetLastError();
}

// Gradient reduce-scatter + optimizer update of the owned slice + all-gather of the new bf16 weights, one kernel.
// grads: bf16 arenas (symmetric), shadow: bf16 weight arenas (symmetric), w/m/v: local fp32 arenas.  offset and n
// are in elements, multiples of 8.  kind: 0 Adam (alpha_ptr = device pointer to the step size), 1 SGD.
FFK_API int ffk_grad_allreduce_update(void *const *grad_peers, void *const *shadow_peers, float *w, float *m, float *v, void *const *flag_peers,
                                      int flag_base, long long offset, long long n, float scale, int rank, int world, void *sync_words,
                                      int *status, int kind, float lr, const float *alpha_ptr, float beta1, float beta2, float eps, float wd,
                                      float momentum, int nesterov, int blocks, cudaStream_t st) {
  if (world > MAX_RANKS || (n & 7) || (offset & 7)) return -2;
  if (n <= 0) return 0;
  AllReduceSync s;
  s.epoch_ctr = (unsigned long long *)sync_words;
  s.started = (unsigned int *)sync_words + 2;
  s.blocks_done = (unsigned int *)sync_words + 3;
  if (blocks <= 0) blocks = 32;
  UpdateArgs u;
  u.w = w; u.m = m; u.v = v; u.shadow = make_ptrs(shadow_peers, world); u.alpha_ptr = alpha_ptr; u.kind = kind; u.lr = lr;
  u.beta1 = beta1; u.beta2 = beta2; u.eps = eps; u.wd = wd; u.momentum = momentum; u.nesterov = nesterov;
  allreduce_scale_kernel<bf16, true><<<blocks, 512, 0, st>>>(make_ptrs(grad_peers, world), make_ptrs(flag_peers, world), flag_base, offset, n, scale,
                                                             rank, world, s, status, u);
  return (int)cudaGetLastError();
}

// Push `nbytes` (multiple of 16) from src into every peer's buffer at byte offset dst_offset, then raise
// flag[flag_base + rank] on every peer.  sync_words: [0..1] epoch (u64), [3] blocks_done.
FFK_API int ffk_push_rows(const void *src, void *const *dst_peers, long long dst_offset, long long nbytes, void *const *flag_peers, int flag_base,
                          int rank, int world, void *sync_words, int skip_self, int blocks, cudaStream_t st) {
  if (world > MAX_RANKS || (nbytes & 15) || (dst_offset & 15)) return -2;
  if (blocks <= 0) blocks = 32;
  push_rows_kernel<<<blocks, 512, 0, st>>>((const uint4 *)src, make_ptrs(dst_peers, world), dst_offset / 16, nbytes / 16, make_ptrs(flag_peers, world),
                                           flag_base, rank, world, (unsigned long long *)sync_words, (unsigned int *)sync_words + 3, skip_self);
  return (int)cudaGetLastError();
}

// Piece p (piece_bytes each) of src goes into slot `rank` of peer p's staging buffer; then this rank's flag is raised on
// every peer.  Together with ffk_reduce_partials on the receiving side this is a reduce-scatter over peer memory.
FFK_API int ffk_scatter_pieces(const void *src, void *const *dst_peers, long long piece_bytes, void *const *flag_peers, int flag_base, int rank,
                               int world, void *sync_words, int blocks, cudaStream_t st) {
  if (world > MAX_RANKS || (piece_bytes & 15) || (((uintptr_t)src) & 15)) return -2;
  if (blocks <= 0) blocks = 32;
  scatter_pieces_kernel<<<blocks, 512, 0, st>>>((const uint4 *)src, make_ptrs(dst_peers, world), piece_bytes / 16, make_ptrs(flag_peers, world),
                                                flag_base, rank, world, (unsigned long long *)sync_words, (unsigned int *)sync_words + 3);
  return (int)cudaGetLastError();
}

// out[n] = sum_{s<nsrc} stage[s][n] (+ residual); waits for the nsrc source flags of the next epoch first.
FFK_API int ffk_reduce_partials(const void *stage, const void *residual, void *out, long long n, int nsrc, const void *flags_local, int flag_base,
                                void *sync_words, int *status, int dt, int blocks, cudaStream_t st) {
  if (nsrc > MAX_RANKS || (n & 7)) return -2;
  if (blocks <= 0) blocks = 148 * 2;
  if (dt == 1)
    reduce_partials_kernel<bf16><<<blocks, 256, 0, st>>>((const bf16 *)stage, (const bf16 *)residual, (bf16 *)out, n, nsrc,
                                                         (const unsigned long long *)flags_local, flag_base, (unsigned long long *)sync_words,
                                                         (unsigned int *)sync_words + 3, status);
  else if (dt == 0)
    reduce_partials_kernel<float><<<blocks, 256, 0, st>>>((const float *)stage, (const float *)residual, (float *)out, n, nsrc,
                                                          (const unsigned long long *)flags_local, flag_base, (unsigned long long *)sync_words,
                                                          (unsigned int *)sync_words + 3, status);
  else return -2;
  return (int)cudaGetLastError();
}

// tables: device array of `tables_local` pointers (fp32 tables); entries: device array of their row counts.
// out_dt: 0 = fp32, 1 = bf16; idx_dt: 2 = int32, 3 = int64.
FFK_API int ffk_alltoall_embedding_fwd(const void *tables, const void *entries, const void *idx, void *const *out_peers, int global_batch,
                                       int local_batch, int num_tables, int dim, int rank, int world, int out_dt, int idx_dt, cudaStream_t st) {
  if (world > MAX_RANKS) return -2;
  int tl = (num_tables - rank + world - 1) / world;
  long long total = (long long)tl * global_batch * dim;
  if (total <= 0) return 0;
  PeerPtrs o = make_ptrs(out_peers, world);
  if (dim % 4 == 0 && total / 4 < 0x7fffffffll) {
    // rows start on 16-byte boundaries (tables and staging buffers come from cudaMalloc / the symmetric allocator)
    const unsigned tv = (unsigned)(total / 4);
    const int gridv = ffk_blocks(tv, 256);
#define A2A_FWDV(T, I) alltoall_embedding_fwd_vec_kernel<T, I><<<gridv, 256, 0, st>>>((const float *const *)tables, (const long long *)entries, (const I *)idx, o, global_batch, local_batch, num_tables, dim, rank, world, tv)
    if (out_dt == 1 && idx_dt == 3) A2A_FWDV(bf16, long long);
    else if (out_dt == 1 && idx_dt == 2) A2A_FWDV(bf16, int);
    else if (out_dt == 0 && idx_dt == 3) A2A_FWDV(float, long long);
    else if (out_dt == 0 && idx_dt == 2) A2A_FWDV(float, int);
    else return -2;
#undef A2A_FWDV
    return (int)cudaGetLastError();
  }
  int grid = ffk_blocks(total, 256);
#define A2A_FWD(T, I) alltoall_embedding_fwd_kernel<float, T, I><<<grid, 256, 0, st>>>((const float *const *)tables, (const long long *)entries, (const I *)idx, o, global_batch, local_batch, num_tables, dim, rank, world)
  if (out_dt == 1 && idx_dt == 3) A2A_FWD(bf16, long long);
  else if (out_dt == 1 && idx_dt == 2) A2A_FWD(bf16, int);
  else if (out_dt == 0 && idx_dt == 3) A2A_FWD(float, long long);
  else if (out_dt == 0 && idx_dt == 2) A2A_FWD(float, int);
  else return -2;
#undef A2A_FWD
  return (int)cudaGetLastError();
}
FFK_API int ffk_alltoall_embedding_bwd(const void *tables, const void *dgrad, const void *entries, const void *idx, void *const *dout_peers,
                                       int global_batch, int local_batch, int num_tables, int dim, int rank, int world, float lr, int out_dt,
                                       int idx_dt, cudaStream_t st) {
  if (world > MAX_RANKS) return -2;
  int tl = (num_tables - rank + world - 1) / world;
  long long total = (long long)tl * global_batch * dim;
  if (total <= 0) return 0;
  PeerPtrs o = make_ptrs(dout_peers, world);
  if (dim % 4 == 0 && total / 4 < 0x7fffffffll) {
    const unsigned tv = (unsigned)(total / 4);
    const int gridv = ffk_blocks(tv, 256);
#define A2A_BWDV(T, I) alltoall_embedding_bwd_vec_kernel<T, I><<<gridv, 256, 0, st>>>((float *const *)tables, (float *const *)dgrad, (const long long *)entries, (const I *)idx, o, global_batch, local_batch, num_tables, dim, rank, world, lr, tv)
    if (out_dt == 1 && idx_dt == 3) A2A_BWDV(bf16, long long);
    else if (out_dt == 1 && idx_dt == 2) A2A_BWDV(bf16, int);
    else if (out_dt == 0 && idx_dt == 3) A2A_BWDV(float, long long);
    else if (out_dt == 0 && idx_dt == 2) A2A_BWDV(float, int);
    else return -2;
#undef A2A_BWDV
    return (int)cudaGetLastError();
  }
  int grid = ffk_blocks(total, 256);
#define A2A_BWD(T, I) alltoall_embedding_bwd_kernel<T, I><<<grid, 256, 0, st>>>((float *const *)tables, (float *const *)dgrad, (const long long *)entries, (const I *)idx, o, global_batch, local_batch, num_tables, dim, rank, world, lr)
  if (out_dt == 1 && idx_dt == 3) A2A_BWD(bf16, long long);
  else if (out_dt == 1 && idx_dt == 2) A2A_BWD(bf16, int);
  else if (out_dt == 0 && idx_dt == 3) A2A_BWD(float, long long);
  else if (out_dt == 0 && idx_dt == 2) A2A_BWD(float, int);
  else return -2;
#undef A2A_BWD
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- symmetric memory set-up (called once, not per step)
// A symmetric buffer is a plain cudaMalloc region whose CUDA IPC handle every peer opens; the peers'
// mappings are ordinary device pointers that kernels dereference over NVLink.
FFK_API void *ffk_symm_alloc(long long nbytes) {
  void *p = nullptr;
  if (cudaMalloc(&p, (size_t)nbytes) != cudaSuccess) return nullptr;
  cudaMemset(p, 0, (size_t)nbytes);
  return p;
}
FFK_API int ffk_symm_free(void *p) { return (int)cudaFree(p); }
FFK_API int ffk_ipc_get_handle(void *ptr, void *out64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return (int)e;
  memcpy(out64, &h, sizeof(h));
  return 0;
}
FFK_API void *ffk_ipc_open(const void *handle64) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void *p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return nullptr;
  return p;
}
FFK_API int ffk_ipc_close(void *p) { return (int)cudaIpcCloseMemHandle(p); }
