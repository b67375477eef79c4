// gemm_sm100.cu -- Blackwell (sm_100a) GEMM: TMA -> shared memory -> tcgen05.mma
// with fp32 accumulators in tensor memory (TMEM), persistent over output tiles.
//
// Replaces the cuBLAS GemmEx calls the reference makes for Linear forward /
// dgrad / wgrad (lib/kernels/src/cuda/ops/linear_kernels.cu:121-341) and supplies
// the BatchMatmul the reference only declares
// (lib/pcg/include/pcg/computation_graph_builder.h:129).
//
//   D[b][m][n] = epilogue( alpha * sum_k A[b][m][k] * B[b][n][k] )
//
// Operand layouts.  A is logically [M,K], B is logically [N,K] (so a Linear's
// weight [out,in] is used as stored).  Either operand may be "K-major" (k is the
// contiguous index) or "MN-major" (m resp. n is the contiguous index); this is
// what lets forward, dgrad (dX = dY * W) and wgrad (dW = dY^T * X) all run
// without a transpose pass.  Two batch dimensions (inner `nh`, outer `nb`)
// with independent strides cover attention's [batch, seq, head, dim] views.
//
// CTA layout (320 threads): warp 0 issues TMA loads, warp 1 allocates TMEM and
// issues tcgen05.mma from one thread, warps 2..9 are the epilogue (TMEM ->
// registers -> bias/activation/addend -> global).  Two TMEM accumulator stages
// let the epilogue of tile i overlap the main loop of tile i+1.
//
// Every mbarrier wait is bounded: after ~2 s without progress the waiting thread
// records an error code, raises a CTA-wide abort flag and every role leaves its
// loop; TMEM is then freed and the kernel returns normally.
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128;
constexpr int GEMM_THREADS = 384;  // TMA warp, MMA warp, 8 epilogue warps, 2 copy warps (all-gather push)
constexpr int COPY_THREADS = 64;

struct GemmArgs {
  int M, N, K;
  int nh, nb;  // inner / outer batch extents
  void *C;
  long long ldc, c_sh, c_sb;
  void *C2;  // optional second output: pre-activation value, bf16, same layout as C
  const void *bias;    // [N] or null
  const void *addend;  // optional, added after activation (residual), layout of C
  long long ld_add, add_sh, add_sb;
  float alpha;
  int act;
  int out_fp32;    // C is float instead of bf16
  int accumulate;  // C += result
  int aux_fp32;    // bias / addend / C2 are float (fp32 activations) instead of bf16
  int tiles_m, tiles_n;
  long long num_tiles;
  // Split-K: a problem with few output tiles and a very long K (the weight gradient of a convolution:
  // [OC, KH*KW*C] accumulated over N*OH*OW rows) is cut into split_k ranges of kb_per_split k-blocks; the work
  // items are (tile, split) pairs and every split adds its partial into the fp32 output with atomics.
  int split_k;
  int kb_per_split;
  // Dropout fused into the epilogue (after the activation): element (row, col) is kept when the counter-based
  // generator says so for flat index row * ldc + col -- the same function of (seed, index) as the stand-alone
  // dropout kernel, so backward regenerates the mask.  drop_seed_ptr (device memory) holds the per-step seed.
  float drop_p;
  float drop_scale;
  unsigned long long drop_salt;
  const unsigned long long *drop_seed_ptr;
  // Output through TMA stores (bf16 output, bias + ReLU/none only): each epilogue warp converts its 32 x 32 chunk
  // into a swizzled bf16 tile in shared memory and one lane issues a bulk tensor store; rows and columns past the
  // matrix edge are clipped by the tensor map.
  int tma_store;
  int *err;
  // --- fused collectives (all optional) ---
  // Scatter epilogue (GEMM -> reduce-scatter): when scatter_rows > 0 the output rows are split into blocks of
  // scatter_rows rows owned by rank (row / scatter_rows); a tile is written into its owner's staging buffer
  // scatter[owner] (a peer pointer over NVLink) at row  scatter_src * scatter_rows + row % scatter_rows, i.e.
  // into slot `scatter_src` of the owner's [world][scatter_rows][N] partial-sum stage.
  void *scatter[8];
  int scatter_rows;
  int scatter_src;
  // Gated A operand (all-gather -> GEMM): rows of A arrive in blocks of gate_rows rows pushed by the peers;
  // block s may be read once gate_flags[s] >= *gate_sync + 1.  mb_rotate starts the tile order at the
  // m-blocks of the local shard so that math begins before any remote data has landed.
  const unsigned long long *gate_flags;
  unsigned long long *gate_sync;  // [0] epoch (u64), word 3 (u32) = CTAs finished
  int gate_rows;
  int mb_rotate;
  // Push (the sending half of all-gather -> GEMM, in the same kernel): two warps of every CTA copy this rank's
  // row shard (push_nvec 16-byte vectors at push_src) into every peer's staging buffer push_dst[p] at vector
  // offset push_off, while the other warps already multiply the local shard; the last CTA to finish raises
  // push_flag[p] (this rank's flag on peer p) to *push_sync + 1.  Because the copy warps live in the GEMM's own
  // CTAs, the transfer can never be starved of SMs by the GEMM that waits for it.
  const uint4 *push_src;
  long long push_nvec;
  long long push_off;
  void *push_dst[8];
  unsigned long long *push_flag[8];
  unsigned long long *push_sync;  // [0] epoch (u64), word 3 (u32) = CTAs finished copying
  int push_world;
  int push_rank;
};

// ----------------------------------------------------------------------------
// Kernel
// ----------------------------------------------------------------------------
// ES = operand element size (2: bf16 via kind::f16, 4: fp32 storage via kind::tf32).
// A 128-byte swizzle row holds 128/ES elements, which is also the K extent of a
// pipeline stage for K-major operands and the MN extent of one TMA box for
// MN-major operands.
// CTA2: a pair of CTAs (cluster of 2, tcgen05 cta_group::2) computes a 256 x BN tile: each CTA stages its own 128 rows of
// A and its own BN / 2 rows of B, the even CTA issues the MMAs for both and each CTA drains the 128 x BN accumulator in its own
// tensor memory.  Per SM and k-block this halves the B traffic into shared memory, which leaves room for a deeper ring.
template <int ES, int BN, bool A_MN, bool B_MN, bool CTA2 = false>
struct GemmCfg {
  static constexpr int ROW_ELEMS = 128 / ES;       // elements per 128-byte row
  static constexpr int BK = ROW_ELEMS;             // k extent per stage
  static constexpr int UMMA_K = 32 / ES;           // k per tcgen05.mma
  static constexpr int BN_CTA = CTA2 ? BN / 2 : BN;  // rows of B staged by one CTA
  static constexpr int A_BYTES = BM * BK * ES;     // 16 KB
  static constexpr int B_BYTES = BN_CTA * BK * ES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (STAGE_BYTES <= 32768) ? 6 : (STAGE_BYTES <= 49152 ? 4 : 3);
  static constexpr int TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 512 /*barriers*/ + 8 * 32 * 32 * 4 /*epilogue staging*/;
  // K-major: one 8-row group is 8*128 B apart (SBO), LBO is the fixed 16 B.
  // MN-major: 8 k-rows of one 64-wide chunk are 128 B apart, 8-row groups are
  // 1024 B apart (SBO) and the next MN chunk starts BK*128 B later (LBO).
  static constexpr uint32_t A_LBO = A_MN ? BK * 128 : 16;
  static constexpr uint32_t B_LBO = B_MN ? BK * 128 : 16;
  static constexpr uint32_t SBO = 1024;
  static constexpr uint32_t A_KADV = A_MN ? UMMA_K * 128 : UMMA_K * ES;  // bytes per UMMA k-step
  static constexpr uint32_t B_KADV = B_MN ? UMMA_K * 128 : UMMA_K * ES;
  static constexpr uint32_t IDESC = (1u << 4)                                  // D = f32
                                    | ((ES == 2 ? 1u : 2u) << 7)               // A: bf16 / tf32
                                    | ((ES == 2 ? 1u : 2u) << 10)              // B
                                    | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16)
                                    | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((CTA2 ? 2 * BM : BM) >> 4) << 24);
};

__device__ __forceinline__ float ld_aux(const void *p, long long i, int fp32) {
  return fp32 ? ((const float *)p)[i] : bf2f(((const bf16 *)p)[i]);
}
__device__ __forceinline__ void st_aux(void *p, long long i, int fp32, float v) {
  if (fp32) ((float *)p)[i] = v;
  else ((bf16 *)p)[i] = f2bf(v);
}
__device__ __forceinline__ void tile_coords(long long tile, const GemmArgs &p, int &mb, int &nb_, int &bh, int &bb) {
  long long per_batch = (long long)p.tiles_m * p.tiles_n;
  long long batch = tile / per_batch;
  int t = (int)(tile - batch * per_batch);
  bh = (int)(batch % p.nh);
  bb = (int)(batch / p.nh);
  // grouped rasterisation: 8 m-blocks share the same B panel while it is hot in L2
  const int GROUP = 8;
  int per_group = GROUP * p.tiles_n;
  int g = t / per_group;
  int first_m = g * GROUP;
  int gsize = min(p.tiles_m - first_m, GROUP);
  int r = t - g * per_group;
  mb = first_m + (r % gsize);
  nb_ = r / gsize;
  if (p.mb_rotate) mb = (mb + p.mb_rotate) % p.tiles_m;
}

// Output maps of the scatter epilogue: one per owning rank's staging buffer (peer memory).
struct ScatterMaps {
  CUtensorMap m[8];
};

template <int ES, int BN, bool A_MN, bool B_MN, bool CTA2>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_sm100_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
                  const __grid_constant__ CUtensorMap tmapC, const __grid_constant__ ScatterMaps smaps, const GemmArgs p) {
  using Cfg = GemmCfg<ES, BN, A_MN, B_MN, CTA2>;
  static_assert(!CTA2 || ES == 2, "CTA pairs are built for bf16 operands");
  // worker = the unit that owns output tiles: a CTA, or a CTA pair (rank 0 = the CTA that issues the MMAs)
  const uint32_t pair_rank = CTA2 ? cluster_ctarank() : 0u;
  const unsigned worker = CTA2 ? blockIdx.x >> 1 : blockIdx.x;
  const unsigned num_workers = CTA2 ? gridDim.x >> 1 : gridDim.x;
  constexpr int TILE_M = CTA2 ? 2 * BM : BM;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is what the 128-byte swizzle pattern is anchored to.
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *tiles = smem;
  uint64_t *bars = (uint64_t *)(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t *full_bar = bars;                 // [STAGES]
  uint64_t *empty_bar = bars + STAGES;       // [STAGES]
  uint64_t *tmem_full = bars + 2 * STAGES;   // [2]
  uint64_t *tmem_empty = bars + 2 * STAGES + 2;  // [2]
  uint32_t *tmem_slot = (uint32_t *)(bars + 2 * STAGES + 4);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
  float *epi_stage = (float *)(smem + STAGES * Cfg::STAGE_BYTES + 512);  // 8 epilogue warps x 4 KB, 512-byte aligned (TMA store source)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + Cfg::BK - 1) / Cfg::BK;
  const long long num_items = p.num_tiles * p.split_k;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tmem_full[s], 1);
      mbar_init(&tmem_empty[s], CTA2 ? 16 : 8);  // the epilogue warps of both CTAs of a pair report to the even CTA
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (CTA2) {  // the same warp of both CTAs allocates for the pair
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"((uint32_t)Cfg::TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"((uint32_t)Cfg::TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CTA2) cluster_sync_all();  // the partner's barriers exist before anything is signalled across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t gate_seen = 0;
      for (long long item = worker; item < num_items && ok; item += num_workers) {
        const long long tile = item % p.num_tiles;
        const int kb0 = (int)(item / p.num_tiles) * p.kb_per_split;
        const int kb1 = kb0 + p.kb_per_split < num_kb ? kb0 + p.kb_per_split : num_kb;
        int mb, nb_, bh, bb;
        tile_coords(tile, p, mb, nb_, bh, bb);
        const int a_row = mb * TILE_M + (int)pair_rank * BM;            // this CTA's 128 rows of A
        const int b_row = nb_ * BN + (int)pair_rank * Cfg::BN_CTA;      // and its rows of B
        if (p.gate_flags) {
          // rows of this m-block come from rank src's push: wait (bounded) until its flag reaches this call's epoch
          const int src = (mb * BM) / p.gate_rows;
          if (!((gate_seen >> src) & 1u)) {
            const unsigned long long want = *p.gate_sync + 1;
            uint64_t t0 = ffk_globaltimer();
            while (true) {
              unsigned long long v;
              asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p.gate_flags + src) : "memory");
              if (v >= want) break;
              if (*abort_flag || ffk_globaltimer() - t0 > WAIT_LIMIT_NS) {
                *abort_flag = 1;
                if (p.err) atomicCAS(p.err, 0, (int)FFK_ERR_TIMEOUT_PEER);
                ok = false;
                break;
              }
              __nanosleep(100);
            }
            if (!ok) break;
            gate_seen |= 1u << src;
            // the pushed rows were written by a peer through the generic proxy; order them before the
            // async-proxy (TMA) reads that follow
            asm volatile("fence.proxy.async.global;" ::: "memory");
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err, FFK_ERR_TIMEOUT_PRODUCER);
          if (!ok) break;
          uint32_t sa = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
          uint32_t sb = sa + Cfg::A_BYTES;
          int k0 = kb * Cfg::BK;
          if constexpr (CTA2) {
            // both CTAs' loads are counted on the even CTA's barrier, which expects the bytes of the whole pair
            if (pair_rank == 0) mbar_expect_tx(&full_bar[stage], 2 * Cfg::STAGE_BYTES);
            const uint32_t fb = mapa_u32(smem_u32(&full_bar[stage]), 0);
            if constexpr (!A_MN) {
              tma_load_4d_pair(sa, &tmapA, fb, k0, a_row, bh, bb);
            } else {
#pragma unroll
              for (int c = 0; c < BM / Cfg::ROW_ELEMS; ++c) tma_load_4d_pair(sa + c * Cfg::BK * 128, &tmapA, fb, a_row + c * Cfg::ROW_ELEMS, k0, bh, bb);
            }
            if constexpr (!B_MN) {
              tma_load_4d_pair(sb, &tmapB, fb, k0, b_row, bh, bb);
            } else {
#pragma unroll
              for (int c = 0; c < Cfg::BN_CTA / Cfg::ROW_ELEMS; ++c)
                tma_load_4d_pair(sb + c * Cfg::BK * 128, &tmapB, fb, b_row + c * Cfg::ROW_ELEMS, k0, bh, bb);
            }
          } else {
            mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
            if constexpr (!A_MN) {
              tma_load_4d(sa, &tmapA, &full_bar[stage], k0, a_row, bh, bb);
            } else {
#pragma unroll
              for (int c = 0; c < BM / Cfg::ROW_ELEMS; ++c)
                tma_load_4d(sa + c * Cfg::BK * 128, &tmapA, &full_bar[stage], a_row + c * Cfg::ROW_ELEMS, k0, bh, bb);
            }
            if constexpr (!B_MN) {
              tma_load_4d(sb, &tmapB, &full_bar[stage], k0, b_row, bh, bb);
            } else {
#pragma unroll
              for (int c = 0; c < BN / Cfg::ROW_ELEMS; ++c)
                tma_load_4d(sb + c * Cfg::BK * 128, &tmapB, &full_bar[stage], b_row + c * Cfg::ROW_ELEMS, k0, bh, bb);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      // Drain: every load that was issued must land before the CTA may exit.
      // The consumer releases each stage only after using it, so waiting for all
      // stages to be empty again covers every load in flight.
      for (int s = 0; s < STAGES && ok; ++s) {
        ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err, FFK_ERR_TIMEOUT_PRODUCER);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && pair_rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (long long item = worker; item < num_items && ok; item += num_workers) {
        const int kb0 = (int)(item / p.num_tiles) * p.kb_per_split;
        const int kb1 = kb0 + p.kb_per_split < num_kb ? kb0 + p.kb_per_split : num_kb;
        ok = mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          uint32_t sa = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
          uint32_t sb = sa + Cfg::A_BYTES;
          uint64_t adesc = make_smem_desc(sa, Cfg::A_LBO, Cfg::SBO);
          uint64_t bdesc = make_smem_desc(sb, Cfg::B_LBO, Cfg::SBO);
#pragma unroll
          for (int k = 0; k < Cfg::BK / Cfg::UMMA_K; ++k) {
            if constexpr (CTA2)
              tc_mma_pair_bf16(d_tmem, adesc + (uint64_t)((k * Cfg::A_KADV) >> 4), bdesc + (uint64_t)((k * Cfg::B_KADV) >> 4), Cfg::IDESC,
                               ((kb - kb0) | k) != 0 ? 1u : 0u);
            else
              tc_mma<ES == 4>(d_tmem, adesc + (uint64_t)((k * Cfg::A_KADV) >> 4), bdesc + (uint64_t)((k * Cfg::B_KADV) >> 4),
                              Cfg::IDESC, ((kb - kb0) | k) != 0 ? 1u : 0u);
          }
          // frees the smem stage (in both CTAs of a pair) once these MMAs retire
          if constexpr (CTA2) tc_commit_pair(&empty_bar[stage]);
          else tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if constexpr (CTA2) tc_commit_pair(&tmem_full[acc]);
        else tc_commit(&tmem_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (warp >= 10) {
    // ------------------------------------------------------------ all-gather push (two warps)
    if (p.push_src) {
      const int t = (int)threadIdx.x - 10 * 32;
      const long long stride = (long long)gridDim.x * COPY_THREADS;
      unsigned int *done = (unsigned int *)p.push_sync + 2;  // [2]: local copy, [3]: remote copies
      // phase 0 copies the shard into this rank's own staging slot (the GEMM reads every row from the staging
      // buffer) and raises the local flag; phase 1 sends it to the peers and raises this rank's flag there
      for (int phase = 0; phase < 2; ++phase) {
        const int k0 = phase, k1 = phase ? p.push_world : 1;
        if (k0 < k1) {
          long long i = (long long)blockIdx.x * COPY_THREADS + t;
          for (; i + 3 * stride < p.push_nvec; i += 4 * stride) {  // four loads in flight per thread
            uint4 v0 = p.push_src[i], v1 = p.push_src[i + stride], v2 = p.push_src[i + 2 * stride], v3 = p.push_src[i + 3 * stride];
            for (int k = k0; k < k1; ++k) {
              uint4 *d = (uint4 *)p.push_dst[(p.push_rank + k) % p.push_world] + p.push_off;
              d[i] = v0; d[i + stride] = v1; d[i + 2 * stride] = v2; d[i + 3 * stride] = v3;
            }
          }
          for (; i < p.push_nvec; i += stride) {
            uint4 v = p.push_src[i];
            for (int k = k0; k < k1; ++k) ((uint4 *)p.push_dst[(p.push_rank + k) % p.push_world] + p.push_off)[i] = v;
          }
        }
        __threadfence_system();
        asm volatile("bar.sync 1, %0;" ::"n"(COPY_THREADS) : "memory");
        if (t == 0) {
          if (atomicAdd(done + phase, 1u) == gridDim.x - 1) {
            __threadfence_system();
            const unsigned long long epoch = *p.push_sync + 1;
            for (int k = k0; k < k1; ++k)
              asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p.push_flag[(p.push_rank + k) % p.push_world]), "l"(epoch)
                           : "memory");
            done[phase] = 0;
            if (phase == 1) *p.push_sync = epoch;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    // Eight warps: warp w reads TMEM lane quarter (w & 3) -- the hardware ties a warp to the lanes
    // 32*(warp%4)..+31 -- and column half (w - 2) / 4 of the accumulator.  The epilogue of a tile must fit
    // under the main loop of the next one, and with so few warps per SM it is bound by instruction latency,
    // not bandwidth: the common case (bf16 output, bias + ReLU/none) therefore takes a branch-free path with
    // all address arithmetic hoisted out of the inner loops.
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int HALF_COLS = BN / 2;
    const int unit = lane & 7;
    const int rsub = lane >> 3;
    float *stg = epi_stage + (warp - 2) * (32 * 32);
    // staging offsets: write = my row, 8 units; read = rows rsub, rsub+4, ... of unit `unit`
    const uint32_t wr_base = smem_u32(stg + lane * 32);
    const uint32_t rd_even = smem_u32(stg + rsub * 32 + ((unit ^ rsub) << 2));            // rows with (rr & 7) == rsub
    const uint32_t rd_odd = smem_u32(stg + (rsub + 4) * 32 + ((unit ^ (rsub + 4)) << 2));  // rows with (rr & 7) == rsub + 4
    const bool simple = p.split_k == 1 && p.drop_p == 0.f && !p.out_fp32 && !p.accumulate && !p.C2 && !p.addend && !p.aux_fp32 &&
                        (p.act == ACT_NONE || p.act == ACT_RELU) && (p.ldc % 4 == 0) && (((uintptr_t)p.C) & 7) == 0 &&
                        (p.c_sh % 4 == 0) && (p.c_sb % 4 == 0);
    const float relu_floor = p.act == ACT_RELU ? 0.f : -INFINITY;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t store_it = 0;  // TMA-store chunks issued by this warp (selects the staging buffer)
    bool ok = true;
    for (long long item = worker; item < num_items && ok; item += num_workers) {
      const long long tile = item % p.num_tiles;
      const bool first_split = item < p.num_tiles;  // the bias is added once
      int mb, nb_, bh, bb;
      tile_coords(tile, p, mb, nb_, bh, bb);
      ok = mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      long long c_base = (long long)bh * p.c_sh + (long long)bb * p.c_sb;
      void *Cout = p.C;
      if (p.scatter_rows) {  // this tile belongs to rank `owner`: write it into slot scatter_src of the owner's stage
        const int owner = (mb * BM) / p.scatter_rows;
        Cout = p.scatter[owner];
        c_base = (long long)(p.scatter_src - owner) * p.scatter_rows * p.ldc;
      }
      const long long a_base = (long long)bh * p.add_sh + (long long)bb * p.add_sb;
      const int row0 = mb * TILE_M + (int)pair_rank * BM + q * 32;  // first row of this warp's quarter
      const int rows_left = p.M - row0 - rsub;     // iteration i is valid iff 4*i < rows_left
      const uint32_t t_base = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + half * HALF_COLS);
      uint32_t r[32];
      tmem_ld32(t_base, r);
      if (p.tma_store) {
        // lane = row of this warp's 32-row quarter, r[j] = column c0 + j: the lane writes its row (32 bf16 = 64 B,
        // as four 16-byte pieces at SWIZZLE_64B positions) and lane 0 stores the 32 x 32 tile
        const uint32_t sbase = smem_u32(stg);
        const bool bias_vec = p.bias && ((((uintptr_t)p.bias) & 15) == 0);
#pragma unroll 1
        for (int c0 = 0; c0 < HALF_COLS; c0 += 32) {
          tmem_ld_wait();
          const uint32_t buf = sbase + (store_it & 1u) * 2048u;
          if (store_it >= 2) {  // the store issued two chunks ago has finished reading this buffer
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            __syncwarp();
          }
          const int col = nb_ * BN + half * HALF_COLS + c0;
#pragma unroll
          for (int qd = 0; qd < 4; ++qd) {
            float b8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            const int cq = col + qd * 8;
            if (p.bias) {
              if (bias_vec && cq + 8 <= p.N) {
                uint4 u = *reinterpret_cast<const uint4 *>((const bf16 *)p.bias + cq);
                float2 x0 = unpack_bf162(u.x), x1 = unpack_bf162(u.y), x2 = unpack_bf162(u.z), x3 = unpack_bf162(u.w);
                b8[0] = x0.x; b8[1] = x0.y; b8[2] = x1.x; b8[3] = x1.y; b8[4] = x2.x; b8[5] = x2.y; b8[6] = x3.x; b8[7] = x3.y;
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (cq + j < p.N) b8[j] = bf2f(((const bf16 *)p.bias)[cq + j]);
              }
            }
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = fmaxf(fmaf(__uint_as_float(r[qd * 8 + j]), p.alpha, b8[j]), relu_floor);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(buf + (uint32_t)(lane * 64) + (uint32_t)((qd ^ ((lane >> 1) & 3)) << 4)),
                         "r"(pack_bf162(v[0], v[1])), "r"(pack_bf162(v[2], v[3])), "r"(pack_bf162(v[4], v[5])), "r"(pack_bf162(v[6], v[7]))
                         : "memory");
          }
          if (c0 + 32 < HALF_COLS) tmem_ld32(t_base + (uint32_t)(c0 + 32), r);  // overlaps the store below
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            if (p.scatter_rows) {  // the tile goes into slot scatter_src of its owner's stage (a peer's memory)
              const int owner = (mb * BM) / p.scatter_rows;
              tma_store_4d(buf, &smaps.m[owner], col, row0 + (p.scatter_src - owner) * p.scatter_rows, 0, 0);
            } else {
              tma_store_4d(buf, &tmapC, col, row0, bh, bb);
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          ++store_it;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CTA2) mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty[acc]), 0));
          else mbar_arrive(&tmem_empty[acc]);
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        continue;
      }
#pragma unroll 1
      for (int c0 = 0; c0 < HALF_COLS; c0 += 32) {
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 8; ++u)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(wr_base + (uint32_t)(((u ^ (lane & 7)) << 4))), "r"(r[4 * u]),
                       "r"(r[4 * u + 1]), "r"(r[4 * u + 2]), "r"(r[4 * u + 3])
                       : "memory");
        __syncwarp();
        if (c0 + 32 < HALF_COLS) tmem_ld32(t_base + (uint32_t)(c0 + 32), r);  // overlaps the stores below
        const int col = nb_ * BN + half * HALF_COLS + c0 + unit * 4;
        const bool col_ok = col < p.N;
        const bool vec4 = col + 4 <= p.N;
        float b4[4] = {0.f, 0.f, 0.f, 0.f};
        if (p.bias && col_ok && first_split) {
          if (vec4 && !p.aux_fp32 && ((((uintptr_t)p.bias) & 7) == 0)) {
            uint2 u = *reinterpret_cast<const uint2 *>((const bf16 *)p.bias + col);
            float2 x0 = unpack_bf162(u.x), x1 = unpack_bf162(u.y);
            b4[0] = x0.x; b4[1] = x0.y; b4[2] = x1.x; b4[3] = x1.y;
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (col + j < p.N) b4[j] = ld_aux(p.bias, col + j, p.aux_fp32);
          }
        }
        if (simple && vec4) {
          bf16 *cp = (bf16 *)Cout + c_base + (long long)(row0 + rsub) * p.ldc + col;
          const long long step = 4 * p.ldc;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float4 f;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(f.x), "=f"(f.y), "=f"(f.z), "=f"(f.w)
                         : "r"(((i & 1) ? rd_odd : rd_even) + (uint32_t)((i >> 1) * 8 * 32 * 4)));
            if (4 * i < rows_left) {
              float v0 = fmaxf(fmaf(f.x, p.alpha, b4[0]), relu_floor), v1 = fmaxf(fmaf(f.y, p.alpha, b4[1]), relu_floor);
              float v2 = fmaxf(fmaf(f.z, p.alpha, b4[2]), relu_floor), v3 = fmaxf(fmaf(f.w, p.alpha, b4[3]), relu_floor);
              *reinterpret_cast<uint2 *>(cp) = make_uint2(pack_bf162(v0, v1), pack_bf162(v2, v3));
            }
            cp += step;
          }
        } else {
#pragma unroll 1
          for (int i = 0; i < 8; ++i) {
            const int rr = i * 4 + rsub;
            const int row = row0 + rr;
            float4 f = *reinterpret_cast<const float4 *>(stg + rr * 32 + ((unit ^ (rr & 7)) << 2));
            if (row >= p.M || !col_ok) continue;
            float v[4] = {f.x * p.alpha + b4[0], f.y * p.alpha + b4[1], f.z * p.alpha + b4[2], f.w * p.alpha + b4[3]};
            const long long coff = c_base + (long long)row * p.ldc + col;
            if (p.C2) {
              if (!p.aux_fp32 && vec4 && (((uintptr_t)((bf16 *)p.C2 + coff)) & 7) == 0)
                *reinterpret_cast<uint2 *>((bf16 *)p.C2 + coff) = make_uint2(pack_bf162(v[0], v[1]), pack_bf162(v[2], v[3]));
              else
                for (int j = 0; j < 4; ++j) if (col + j < p.N) st_aux(p.C2, coff + j, p.aux_fp32, v[j]);
            }
            if (p.act != ACT_NONE) {
#pragma unroll
              for (int j = 0; j < 4; ++j) v[j] = act_fwd(v[j], p.act);
            }
            if (p.drop_p > 0.f) {
              const unsigned long long seed = p.drop_seed_ptr ? p.drop_salt * 0x9E3779B97F4A7C15ull + *p.drop_seed_ptr : p.drop_salt;
              const uint32_t thr = ffk_drop_threshold(p.drop_p);
              if (vec4 && (coff & 3) == 0) {
                const uint32_t keep = ffk_keep4(seed, (unsigned long long)(coff >> 2), thr);
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = ((keep >> j) & 1u) ? v[j] * p.drop_scale : 0.f;
              } else {
                for (int j = 0; j < 4; ++j) v[j] = ffk_keep(seed, (unsigned long long)(coff + j), thr) ? v[j] * p.drop_scale : 0.f;
              }
            }
            if (p.addend) {
              const long long aoff = a_base + (long long)row * p.ld_add + col;
              if (!p.aux_fp32 && vec4 && (((uintptr_t)((const bf16 *)p.addend + aoff)) & 7) == 0) {
                uint2 u = *reinterpret_cast<const uint2 *>((const bf16 *)p.addend + aoff);
                float2 a0 = unpack_bf162(u.x), a1 = unpack_bf162(u.y);
                v[0] += a0.x; v[1] += a0.y; v[2] += a1.x; v[3] += a1.y;
              } else {
                for (int j = 0; j < 4; ++j) if (col + j < p.N) v[j] += ld_aux(p.addend, aoff + j, p.aux_fp32);
              }
            }
            if (p.out_fp32) {
              float *c = (float *)Cout + coff;
              if (p.split_k > 1) {  // partial sum of one K range: the output was cleared (or holds the accumuland)
                for (int j = 0; j < 4; ++j) if (col + j < p.N) atomicAdd(c + j, v[j]);
              } else if (vec4 && (((uintptr_t)c) & 15) == 0) {
                float4 o = make_float4(v[0], v[1], v[2], v[3]);
                if (p.accumulate) {
                  float4 old = *reinterpret_cast<float4 *>(c);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4 *>(c) = o;
              } else {
                for (int j = 0; j < 4; ++j) if (col + j < p.N) c[j] = p.accumulate ? c[j] + v[j] : v[j];
              }
            } else {
              bf16 *c = (bf16 *)Cout + coff;
              if (vec4 && (((uintptr_t)c) & 7) == 0) {
                if (p.accumulate) {
                  uint2 u = *reinterpret_cast<uint2 *>(c);
                  float2 o0 = unpack_bf162(u.x), o1 = unpack_bf162(u.y);
                  v[0] += o0.x; v[1] += o0.y; v[2] += o1.x; v[3] += o1.y;
                }
                *reinterpret_cast<uint2 *>(c) = make_uint2(pack_bf162(v[0], v[1]), pack_bf162(v[2], v[3]));
              } else {
                for (int j = 0; j < 4; ++j) if (col + j < p.N) c[j] = f2bf(p.accumulate ? bf2f(c[j]) + v[j] : v[j]);
              }
            }
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
          if constexpr (CTA2) mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty[acc]), 0));
          else mbar_arrive(&tmem_empty[acc]);
        }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    // every bulk store this warp issued must have completed before the CTA's shared memory goes away
    if (p.tma_store && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  tc_fence_before();
  __syncthreads();
  if constexpr (CTA2) cluster_sync_all();  // neither CTA's shared or tensor memory goes away while its partner may still use it
  if (warp == 1) {
    tc_fence_after();
    if constexpr (CTA2)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS)
                   : "memory");
  }
  if (p.gate_sync && threadIdx.x == 0) {
    // the last CTA to leave advances the epoch the next call will wait for
    unsigned int *done = (unsigned int *)p.gate_sync + 3;
    __threadfence();
    if (atomicAdd(done, 1u) == gridDim.x - 1) {
      *p.gate_sync = *p.gate_sync + 1;
      *done = 0;
    }
  }
}

// ----------------------------------------------------------------------------
// General-shape fallback.  TMA needs 16-byte aligned bases and row pitches; operands that cannot offer
// that (a 10-class classifier head, odd feature counts) take this shared-memory-tiled CUDA-core kernel.
// Same semantics and epilogue as the tensor-core kernel.
// ----------------------------------------------------------------------------
struct SimtOperands {
  const void *A, *B;
  long long lda, a_sh, a_sb, ldb, b_sh, b_sb;
  int a_mn, b_mn;
  int kw;           // warps sharing one tile (splitting k): 1, 2, 4 or 8
  int group_batch;  // the block's 8 / kw tiles are consecutive batch entries (else consecutive row tiles)
};
// alpha, bias, pre-activation copy, activation, addend, accumulate, store: the tensor-core kernel's epilogue for one value
__device__ __forceinline__ void simt_epilogue(const GemmArgs &p, float v, int bh, int bb, int m, int n) {
  v *= p.alpha;
  if (p.bias) v += ld_aux(p.bias, n, p.aux_fp32);
  const long long coff = (long long)bh * p.c_sh + (long long)bb * p.c_sb + (long long)m * p.ldc + n;
  if (p.C2) st_aux(p.C2, coff, p.aux_fp32, v);
  v = act_fwd(v, p.act);
  if (p.addend) v += ld_aux(p.addend, (long long)bh * p.add_sh + (long long)bb * p.add_sb + (long long)m * p.ld_add + n, p.aux_fp32);
  if (p.out_fp32) {
    float *c = (float *)p.C + coff;
    *c = p.accumulate ? *c + v : v;
  } else {
    bf16 *c = (bf16 *)p.C + coff;
    *c = f2bf(p.accumulate ? bf2f(*c) + v : v);
  }
}

// A block has 8 warps and works on 32x32 output tiles.  `kw` warps (1, 2, 4 or 8) share one tile and split its
// k range in chunks of 32 (chunk c goes to k-slot c % kw); the block's 8 / kw tiles are consecutive batch
// entries (small batched problems) or consecutive row tiles.  Warps work without block-wide barriers: a warp
// loads its next chunk of A and B into registers (all 64 loads in flight, coalesced along whichever dim is
// contiguous) while it computes on the chunk staged in its own shared-memory region, every lane accumulating
// one output row of 32 values.  The partial tiles of the warps sharing a tile are summed through shared memory
// at the end.  A weight-gradient GEMM with a small output and a long reduction dim (the batch) thereby still has
// 8 warps per tile in flight, a GEMM with a tiny k costs one chunk, and a batch of tiny problems fills its blocks.
constexpr int ST = 32;
constexpr int SIMT_WARPS = 8;
constexpr int SA_LD = 33;  // lane-indexed reads and transposed writes without bank conflicts
constexpr int SB_LD = 36;  // rows read as float4
constexpr int SIMT_WARP_FLOATS = ST * SA_LD + ST * SB_LD;
constexpr int SIMT_SMEM_BYTES = SIMT_WARPS * SIMT_WARP_FLOATS * 4;

template <typename T>
__device__ __forceinline__ void simt_fetch(float (&r)[ST], const T *X, long long ld, int mn_major, int k0, int x0, int lane, int K, int X_extent) {
  if (mn_major) {  // X[k][x]: lanes along x, registers along k
    const int x = x0 + lane;
#pragma unroll
    for (int i = 0; i < ST; ++i) {
      const int k = k0 + i;
      r[i] = (k < K && x < X_extent) ? (float)X[(long long)k * ld + x] : 0.f;
    }
  } else {         // X[x][k]: lanes along k, registers along x
    const int k = k0 + lane;
#pragma unroll
    for (int i = 0; i < ST; ++i) {
      const int x = x0 + i;
      r[i] = (k < K && x < X_extent) ? (float)X[(long long)x * ld + k] : 0.f;
    }
  }
}
// stage as s[k][x] with row pitch LD
template <int LD>
__device__ __forceinline__ void simt_stage(float *s, const float (&r)[ST], int mn_major, int lane) {
  if (mn_major) {
#pragma unroll
    for (int i = 0; i < ST; ++i) s[i * LD + lane] = r[i];
  } else {
#pragma unroll
    for (int i = 0; i < ST; ++i) s[lane * LD + i] = r[i];
  }
}

template <typename T>
__global__ void __launch_bounds__(SIMT_WARPS * 32, 2) gemm_simt_kernel(SimtOperands o, GemmArgs p) {
  extern __shared__ __align__(16) float simt_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float *sa = simt_smem + warp * SIMT_WARP_FLOATS, *sb = sa + ST * SA_LD;
  const int kw = o.kw, ti = warp / kw, ks = warp % kw, tpb = SIMT_WARPS / kw;
  int batch = blockIdx.z, tile_m = blockIdx.y;
  if (o.group_batch) batch = blockIdx.z * tpb + ti;
  else tile_m = blockIdx.y * tpb + ti;
  const int m0 = tile_m * ST, n0 = blockIdx.x * ST;
  const bool active = batch < p.nh * p.nb && m0 < p.M;
  const int bh = batch % p.nh, bb = batch / p.nh;
  const T *A = (const T *)o.A + (long long)bh * o.a_sh + (long long)bb * o.a_sb;
  const T *B = (const T *)o.B + (long long)bh * o.b_sh + (long long)bb * o.b_sb;
  float acc[ST];
#pragma unroll
  for (int i = 0; i < ST; ++i) acc[i] = 0.f;
  if (active) {
    const int chunks = (p.K + ST - 1) / ST;
    float ra[ST], rb[ST];
    if (ks < chunks) {
      simt_fetch<T>(ra, A, o.lda, o.a_mn, ks * ST, m0, lane, p.K, p.M);
      simt_fetch<T>(rb, B, o.ldb, o.b_mn, ks * ST, n0, lane, p.K, p.N);
    }
    for (int c = ks; c < chunks; c += kw) {
      simt_stage<SA_LD>(sa, ra, o.a_mn, lane);
      simt_stage<SB_LD>(sb, rb, o.b_mn, lane);
      __syncwarp();
      if (c + kw < chunks) {  // next chunk's loads fly while this one is computed
        simt_fetch<T>(ra, A, o.lda, o.a_mn, (c + kw) * ST, m0, lane, p.K, p.M);
        simt_fetch<T>(rb, B, o.ldb, o.b_mn, (c + kw) * ST, n0, lane, p.K, p.N);
      }
      const int kmax = min(ST, p.K - c * ST);  // a short (last) chunk costs only its own k steps
#pragma unroll 2
      for (int k = 0; k < kmax; ++k) {
        const float a = sa[k * SA_LD + lane];
        const float4 *bv = reinterpret_cast<const float4 *>(sb + k * SB_LD);
#pragma unroll
        for (int j = 0; j < ST / 4; ++j) {
          const float4 b = bv[j];
          acc[4 * j + 0] += a * b.x;
          acc[4 * j + 1] += a * b.y;
          acc[4 * j + 2] += a * b.z;
          acc[4 * j + 3] += a * b.w;
        }
      }
      __syncwarp();
    }
  }
  __syncthreads();  // every warp is done with its staging region: reuse the memory for the partial tiles
  float *red = simt_smem;  // [warp][m][SA_LD]
#pragma unroll
  for (int n = 0; n < ST; ++n) red[(warp * ST + lane) * SA_LD + n] = acc[n];
  __syncthreads();
  if (!active) return;
  const int n = n0 + lane;
  for (int ml = ks; ml < ST; ml += kw) {
    const int m = m0 + ml;
    if (m >= p.M || n >= p.N) continue;
    float v = 0.f;
    for (int w = ti * kw; w < ti * kw + kw; ++w) v += red[(w * ST + ml) * SA_LD + lane];
    simt_epilogue(p, v, bh, bb, m, n);
  }
}

// Batches of small problems (an interaction layer's 9x9x64 products): one warp per batch entry.  The warp
// stages its A[M,K] and B[N,K] panels in shared memory (row pitch K+1, so rows start in different banks), then
// every lane computes whole outputs, lane l the outputs l, l+32, ... in row-major order.  Index arithmetic is
// incremental (no divisions), so a 9x9x64 product costs a few hundred instructions per warp.
constexpr int SB_WARPS = 8;
constexpr int SB_FLOATS = 2304;  // per warp: (M + N) * (K + 1) floats
constexpr int SB_SMEM_BYTES = SB_WARPS * SB_FLOATS * 4;

// advance a (slow, fast) index pair by 32 positions in fast-dim-first order
__device__ __forceinline__ void small_advance(int &slow, int &fast, int extent) {
  fast += 32;
  while (fast >= extent) { fast -= extent; ++slow; }
}
// Panel X (rows x K, either layout) -> s[x * (K + 1) + k]; four independent loads in flight per lane.
template <typename T>
__device__ __forceinline__ void small_stage(float *s, const T *X, int rows, int K, long long ld, int mn_major, int lane) {
  const int ldk = K + 1, total = rows * K;
  const int fast_extent = mn_major ? rows : K;   // the dim that is contiguous in memory
  int slow = lane / fast_extent, fast = lane - slow * fast_extent;
  for (int e = lane; e < total; e += 128) {
    int sl[4], fa[4];
    T v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      sl[j] = slow; fa[j] = fast;
      small_advance(slow, fast, fast_extent);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (e + 32 * j < total) v[j] = X[(long long)sl[j] * ld + fa[j]];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (e + 32 * j < total) {
        const int x = mn_major ? fa[j] : sl[j], k = mn_major ? sl[j] : fa[j];
        s[x * ldk + k] = (float)v[j];
      }
  }
}

template <typename T>
__global__ void __launch_bounds__(SB_WARPS * 32) gemm_small_batched_kernel(SimtOperands o, GemmArgs p) {
  extern __shared__ __align__(16) float simt_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int batch = blockIdx.x * SB_WARPS + warp;
  if (batch >= p.nh * p.nb) return;  // warps never meet at a block-wide barrier
  const int bh = batch % p.nh, bb = batch / p.nh;
  const T *A = (const T *)o.A + (long long)bh * o.a_sh + (long long)bb * o.a_sb;
  const T *B = (const T *)o.B + (long long)bh * o.b_sh + (long long)bb * o.b_sb;
  const int ldk = p.K + 1;
  float *sa = simt_smem + warp * ((p.M + p.N) * ldk), *sb = sa + p.M * ldk;
  small_stage<T>(sa, A, p.M, p.K, o.lda, o.a_mn, lane);
  small_stage<T>(sb, B, p.N, p.K, o.ldb, o.b_mn, lane);
  __syncwarp();
  int m = 0, n = lane;
  while (n >= p.N) { n -= p.N; ++m; }
  while (m < p.M) {
    const float *ar = sa + m * ldk, *br = sb + n * ldk;
    float acc = 0.f;
#pragma unroll 4
    for (int k = 0; k < p.K; ++k) acc += ar[k] * br[k];
    simt_epilogue(p, acc, bh, bb, m, n);
    n += 32;
    while (n >= p.N) { n -= p.N; ++m; }
  }
}

// ----------------------------------------------------------------------------
// Host side
// ----------------------------------------------------------------------------
// Build the 4-D map {contiguous, rows, inner batch, outer batch} of one operand.
// K-major operand: contiguous = k, rows = m|n, box {128/ES, box_rows}.
// MN-major operand: contiguous = m|n, rows = k, box {128/ES, BK}.
int make_operand_map(CUtensorMap *map, const void *ptr, int es, long long contiguous, long long rows, long long ld,
                     int nh, long long sh, int nb, long long sb, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)contiguous, (cuuint64_t)rows, (cuuint64_t)nh, (cuuint64_t)nb};
  // a batch extent of 1 still needs a legal (multiple of 16 B, non-zero) stride
  long long sh_b = (nh > 1 ? sh : ld * rows) * es, sb_b = (nb > 1 ? sb : (nh > 1 ? sh * nh : ld * rows)) * es;
  if (sh_b <= 0) sh_b = 16;
  if (sb_b <= 0) sb_b = 16;
  cuuint64_t strides[3] = {(cuuint64_t)(ld * es), (cuuint64_t)sh_b, (cuuint64_t)sb_b};
  cuuint32_t box[4] = {(cuuint32_t)(128 / es), (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, es == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void *)ptr,
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// Output map for the TMA-store epilogue: boxes of 32 rows x 32 bf16 columns (64 bytes, SWIZZLE_64B).
int make_store_map(CUtensorMap *map, void *ptr, long long cols, long long rows, long long ld, int nh, long long sh, int nb, long long sb) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)nh, (cuuint64_t)nb};
  long long sh_b = (nh > 1 ? sh : ld * rows) * 2, sb_b = (nb > 1 ? sb : (nh > 1 ? sh * nh : ld * rows)) * 2;
  if (sh_b <= 0) sh_b = 16;
  if (sb_b <= 0) sb_b = 16;
  cuuint64_t strides[3] = {(cuuint64_t)(ld * 2), (cuuint64_t)sh_b, (cuuint64_t)sb_b};
  cuuint32_t box[4] = {32, 32, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

__device__ int g_gemm_err = 0;

// The CTA-pair kernel: same arguments; the grid is a whole number of clusters of 2 and tiles are 256 rows tall.
template <int BN, bool A_MN, bool B_MN>
int launch_pair(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tc, const ScatterMaps &sm, GemmArgs &args, int max_ctas,
                cudaStream_t stream) {
  using Cfg = GemmCfg<2, BN, A_MN, B_MN, true>;
  static bool attr_done = false;
  auto kern = gemm_sm100_kernel<2, BN, A_MN, B_MN, true>;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  args.tiles_m = (args.M + 2 * BM - 1) / (2 * BM);
  args.tiles_n = (args.N + BN - 1) / BN;
  args.num_tiles = (long long)args.tiles_m * args.tiles_n * args.nh * args.nb;
  args.split_k = 1;
  args.kb_per_split = (args.K + Cfg::BK - 1) / Cfg::BK;
  long long pairs = max_ctas / 2;
  if (args.num_tiles < pairs) pairs = args.num_tiles;
  if (pairs < 1) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, sm, args);
  return (int)e;
}

template <int ES, int BN, bool A_MN, bool B_MN>
int launch_cfg(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tc, const ScatterMaps &sm, GemmArgs &args, int max_ctas,
               cudaStream_t stream) {
  using Cfg = GemmCfg<ES, BN, A_MN, B_MN>;
  static bool attr_done = false;
  auto kern = gemm_sm100_kernel<ES, BN, A_MN, B_MN, false>;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  args.tiles_m = (args.M + BM - 1) / BM;
  args.tiles_n = (args.N + BN - 1) / BN;
  args.num_tiles = (long long)args.tiles_m * args.tiles_n * args.nh * args.nb;
  args.split_k = 1;
  const int num_kb = (args.K + Cfg::BK - 1) / Cfg::BK;
  args.kb_per_split = num_kb;
  const bool plain = args.out_fp32 && !args.C2 && !args.addend && args.act == ACT_NONE && !args.scatter_rows && !args.gate_flags &&
                     args.nh * args.nb == 1 && args.alpha == 1.0f;
  if (plain && args.num_tiles * 2 <= max_ctas && num_kb >= 16) {
    int want = (int)(max_ctas / args.num_tiles);
    if (want > num_kb / 8) want = num_kb / 8;
    if (want > 1) {
      args.kb_per_split = (num_kb + want - 1) / want;
      args.split_k = (num_kb + args.kb_per_split - 1) / args.kb_per_split;
      if (!args.accumulate) {
        cudaError_t e = cudaMemset2DAsync(args.C, (size_t)args.ldc * 4, 0, (size_t)args.N * 4, (size_t)args.M, stream);
        if (e != cudaSuccess) return (int)e;
      }
    }
  }
  long long items = args.num_tiles * args.split_k;
  long long grid = items < max_ctas ? items : max_ctas;
  if (grid < 1) return 0;
  if (args.split_k > 1) args.tma_store = 0;
  kern<<<(unsigned)grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(ta, tb, tc, sm, args);
  return (int)cudaGetLastError();
}

template <int ES, int BN>
int launch_major(bool a_mn, bool b_mn, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tc, const ScatterMaps &sm,
                 GemmArgs &args, int max_ctas, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch_cfg<ES, BN, false, false>(ta, tb, tc, sm, args, max_ctas, stream);
  if (!a_mn && b_mn) return launch_cfg<ES, BN, false, true>(ta, tb, tc, sm, args, max_ctas, stream);
  if (a_mn && !b_mn) return launch_cfg<ES, BN, true, false>(ta, tb, tc, sm, args, max_ctas, stream);
  return launch_cfg<ES, BN, true, true>(ta, tb, tc, sm, args, max_ctas, stream);
}

int launch_pair_major(bool a_mn, bool b_mn, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tc, const ScatterMaps &sm,
                      GemmArgs &args, int max_ctas, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch_pair<256, false, false>(ta, tb, tc, sm, args, max_ctas, stream);
  if (!a_mn && b_mn) return launch_pair<256, false, true>(ta, tb, tc, sm, args, max_ctas, stream);
  if (a_mn && !b_mn) return launch_pair<256, true, false>(ta, tb, tc, sm, args, max_ctas, stream);
  return launch_pair<256, true, true>(ta, tb, tc, sm, args, max_ctas, stream);
}

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace

// Descriptor of one GEMM call.  Plain C struct so ctypes can fill it.
struct FfkGemmDesc {
  int M, N, K;
  int nh, nb;             // batch extents (1,1 for a plain GEMM)
  int es;                 // operand element size: 2 = bf16, 4 = fp32 storage run as tf32
  int a_mn, b_mn;         // 1 = operand is MN-major (m resp. n contiguous)
  const void *A;
  long long lda, a_sh, a_sb;  // leading dimension and batch strides, in elements
  const void *B;
  long long ldb, b_sh, b_sb;
  void *C;
  long long ldc, c_sh, c_sb;
  void *C2;
  const void *bias;
  const void *addend;
  long long ld_add, add_sh, add_sb;
  float alpha;
  int act;
  int out_fp32;
  int accumulate;
  int bn;                 // tile N: 0 = choose, else 64/128/256
  int max_ctas;           // 0 = one per SM
  // fused collectives, see GemmArgs
  void *scatter[8];
  int scatter_rows;
  int scatter_src;
  const void *gate_flags;
  void *gate_sync;
  int gate_rows;
  int mb_rotate;
  // in-kernel push of this rank's shard to the peers (see GemmArgs)
  const void *push_src;
  long long push_bytes;
  long long push_dst_offset;
  void *push_dst[8];
  void *push_flag[8];
  void *push_sync;
  int push_world;
  int push_rank;
  // dropout in the epilogue (see GemmArgs); drop_p = 0 disables it
  float drop_p;
  unsigned long long drop_salt;
  const void *drop_seed_ptr;
};

static int g_pair_mode = 1;  // 1: CTA pairs where they apply, 0: never
// CTA-pair (tcgen05 cta_group::2) kernel on (1) or off (0) process-wide; for A/B measurements.
FFK_API void ffk_gemm_set_cta_pairs(int enabled) { g_pair_mode = enabled ? 1 : 0; }
static int g_disable_tma_store = 0;
static int g_disable_scatter_tma = 0;
// Scatter epilogue (GEMM -> reduce-scatter) through TMA stores into the peers' stages (1) or per-lane stores (0).
FFK_API void ffk_gemm_set_scatter_tma_store(int enabled) { g_disable_scatter_tma = enabled ? 0 : 1; }
// Switches the TMA-store epilogue off (1) or on (0) process-wide; for A/B measurements.
FFK_API void ffk_gemm_set_tma_store(int enabled) { g_disable_tma_store = enabled ? 0 : 1; }

// Returns 0 on success, a CUDA/driver error code otherwise, -2 for an
// argument the TMA path cannot express (unaligned base or stride).
FFK_API int ffk_gemm(const FfkGemmDesc *d, cudaStream_t stream) {
  const int es = d->es;
  if (es != 2 && es != 4) return -2;
  if (d->M <= 0 || d->N <= 0 || d->K <= 0) return 0;
  bool tma_ok = !(((uintptr_t)d->A & 15) || ((uintptr_t)d->B & 15)) && !((d->lda * es) % 16 || (d->ldb * es) % 16) &&
                !((d->nh > 1 && ((d->a_sh * es) % 16 || (d->b_sh * es) % 16)) || (d->nb > 1 && ((d->a_sb * es) % 16 || (d->b_sb * es) % 16))) &&
                !(es == 4 && (d->a_mn || d->b_mn));  // tf32 operands must be K-major
  const bool fused = d->scatter_rows || d->gate_flags || d->push_src || d->drop_p > 0.f;
  // many small problems: one warp each on the CUDA cores beats one mostly empty 128-row tensor-core tile each
  const long long nbatch = (long long)(d->nh < 1 ? 1 : d->nh) * (d->nb < 1 ? 1 : d->nb);
  const bool small_batched = !fused && nbatch >= 32 && (long long)d->M * d->N <= 1024 &&
                             (long long)(d->M + d->N) * (d->K + 1) <= SB_FLOATS;
  if (!tma_ok || small_batched) {
    GemmArgs a;
    a.M = d->M; a.N = d->N; a.K = d->K; a.nh = d->nh < 1 ? 1 : d->nh; a.nb = d->nb < 1 ? 1 : d->nb;
    a.C = d->C; a.ldc = d->ldc; a.c_sh = d->c_sh; a.c_sb = d->c_sb;
    a.C2 = d->C2; a.bias = d->bias; a.addend = d->addend;
    a.ld_add = d->ld_add; a.add_sh = d->add_sh; a.add_sb = d->add_sb;
    a.alpha = d->alpha; a.act = d->act; a.out_fp32 = d->out_fp32; a.accumulate = d->accumulate; a.aux_fp32 = es == 4;
    a.tiles_m = a.tiles_n = 0; a.num_tiles = 0; a.err = nullptr; a.split_k = 1; a.kb_per_split = 0; a.push_src = nullptr; a.drop_p = 0.f; a.tma_store = 0;
    if (fused) return -2;  // the fused-collective paths need TMA-addressable operands
    if (small_batched) {
      static bool sb_attr = false;
      if (!sb_attr) {
        if (cudaFuncSetAttribute(gemm_small_batched_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SB_SMEM_BYTES) != cudaSuccess ||
            cudaFuncSetAttribute(gemm_small_batched_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, SB_SMEM_BYTES) != cudaSuccess)
          return (int)cudaGetLastError();
        sb_attr = true;
      }
      SimtOperands so{d->A, d->B, d->lda, d->a_sh, d->a_sb, d->ldb, d->b_sh, d->b_sb, d->a_mn, d->b_mn, 1, 1};
      const int blocks = (int)((nbatch + SB_WARPS - 1) / SB_WARPS);
      // only the panels' own size: more resident warps per SM hide the staging loads
      const int smem = SB_WARPS * (d->M + d->N) * (d->K + 1) * 4;
      if (es == 2) gemm_small_batched_kernel<bf16><<<blocks, SB_WARPS * 32, smem, stream>>>(so, a);
      else gemm_small_batched_kernel<float><<<blocks, SB_WARPS * 32, smem, stream>>>(so, a);
      return (int)cudaGetLastError();
    }
    const int chunks = (d->K + ST - 1) / ST, tiles_m = (d->M + ST - 1) / ST, nbatch = a.nh * a.nb;
    int kw = 1;
    while (kw < SIMT_WARPS && kw < chunks) kw *= 2;
    const int tpb = SIMT_WARPS / kw;
    const int group_batch = tiles_m == 1 && nbatch > 1;
    SimtOperands o{d->A, d->B, d->lda, d->a_sh, d->a_sb, d->ldb, d->b_sh, d->b_sb, d->a_mn, d->b_mn, kw, group_batch};
    static bool simt_attr = false;
    if (!simt_attr) {
      if (cudaFuncSetAttribute(gemm_simt_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SIMT_SMEM_BYTES) != cudaSuccess ||
          cudaFuncSetAttribute(gemm_simt_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, SIMT_SMEM_BYTES) != cudaSuccess)
        return (int)cudaGetLastError();
      simt_attr = true;
    }
    const int gy = group_batch ? tiles_m : (tiles_m + tpb - 1) / tpb, gz = group_batch ? (nbatch + tpb - 1) / tpb : nbatch;
    if (gy > 65535 || gz > 65535) return -2;
    dim3 grid((d->N + ST - 1) / ST, gy, gz), block(SIMT_WARPS * 32);
    if (es == 2) gemm_simt_kernel<bf16><<<grid, block, SIMT_SMEM_BYTES, stream>>>(o, a);
    else gemm_simt_kernel<float><<<grid, block, SIMT_SMEM_BYTES, stream>>>(o, a);
    return (int)cudaGetLastError();
  }
  int bn = d->bn;
  if (bn == 0) {
    // Prefer the widest tile that still gives every SM work.
    long long t256 = (long long)((d->M + 127) / 128) * ((d->N + 255) / 256) * d->nh * d->nb;
    if (d->N > 128 && t256 >= sm_count()) bn = 256;
    else if (d->N > 64) bn = 128;
    else bn = 64;
    if (es == 4 && bn == 256) bn = 128;
  }
  // A CTA pair per 256 x 256 tile when the problem has at least one such tile per pair of SMs and none of the fused-collective
  // or split-K machinery is involved (those stay on the single-CTA kernel).
  bool pair = false;
  if (g_pair_mode && es == 2 && bn == 256 && !fused && d->M >= 256) {
    const long long t = (long long)((d->M + 255) / 256) * ((d->N + 255) / 256) * nbatch;
    pair = t >= sm_count() / 2;
  }
  const int BK = 128 / es;
  CUtensorMap ta, tb;
  int r;
  if (!d->a_mn) r = make_operand_map(&ta, d->A, es, d->K, d->M, d->lda, d->nh, d->a_sh, d->nb, d->a_sb, BM);
  else r = make_operand_map(&ta, d->A, es, d->M, d->K, d->lda, d->nh, d->a_sh, d->nb, d->a_sb, BK);
  if (r) return r;
  if (!d->b_mn) r = make_operand_map(&tb, d->B, es, d->K, d->N, d->ldb, d->nh, d->b_sh, d->nb, d->b_sb, pair ? bn / 2 : bn);
  else r = make_operand_map(&tb, d->B, es, d->N, d->K, d->ldb, d->nh, d->b_sh, d->nb, d->b_sb, BK);
  if (r) return r;

  GemmArgs a;
  a.M = d->M; a.N = d->N; a.K = d->K; a.nh = d->nh < 1 ? 1 : d->nh; a.nb = d->nb < 1 ? 1 : d->nb;
  a.C = d->C; a.ldc = d->ldc; a.c_sh = d->c_sh; a.c_sb = d->c_sb;
  a.C2 = d->C2; a.bias = d->bias; a.addend = d->addend;
  a.ld_add = d->ld_add; a.add_sh = d->add_sh; a.add_sb = d->add_sb;
  a.alpha = d->alpha; a.act = d->act; a.out_fp32 = d->out_fp32; a.accumulate = d->accumulate; a.aux_fp32 = es == 4;
  for (int i = 0; i < 8; ++i) a.scatter[i] = d->scatter[i];
  a.scatter_rows = d->scatter_rows; a.scatter_src = d->scatter_src;
  a.gate_flags = (const unsigned long long *)d->gate_flags; a.gate_sync = (unsigned long long *)d->gate_sync;
  a.gate_rows = d->gate_rows; a.mb_rotate = d->mb_rotate;
  if (a.scatter_rows && (a.scatter_rows % BM != 0 || a.nh * a.nb != 1)) return -2;
  if (a.gate_flags && (a.gate_rows % BM != 0 || a.nh * a.nb != 1 || d->a_mn)) return -2;
  a.drop_p = d->drop_p; a.drop_scale = d->drop_p > 0.f ? 1.0f / (1.0f - d->drop_p) : 1.f; a.drop_salt = d->drop_salt;
  a.drop_seed_ptr = (const unsigned long long *)d->drop_seed_ptr;
  if (a.drop_p > 0.f && (a.nh * a.nb != 1 || d->out_fp32 || d->accumulate)) return -2;
  a.push_src = (const uint4 *)d->push_src;
  a.push_nvec = d->push_bytes / 16; a.push_off = d->push_dst_offset / 16;
  for (int i = 0; i < 8; ++i) { a.push_dst[i] = d->push_dst[i]; a.push_flag[i] = (unsigned long long *)d->push_flag[i]; }
  a.push_sync = (unsigned long long *)d->push_sync; a.push_world = d->push_world; a.push_rank = d->push_rank;
  if (a.push_src && ((d->push_bytes & 15) || (d->push_dst_offset & 15) || ((uintptr_t)d->push_src & 15) || a.push_world > 8 || !a.push_sync))
    return -2;
  void *errp = nullptr;
  cudaGetSymbolAddress(&errp, g_gemm_err);
  a.err = (int *)errp;
  int max_ctas = d->max_ctas > 0 ? d->max_ctas : sm_count();
  // TMA-store epilogue for the plain bf16 case (bias + ReLU/none) when the output can be described by a tensor map
  CUtensorMap tc = ta;
  a.tma_store = 0;
  static ScatterMaps sm_zero = {};
  ScatterMaps sm = sm_zero;
  const bool store_ok = es == 2 && !d->out_fp32 && !d->accumulate && !d->C2 && !d->addend && (d->act == ACT_NONE || d->act == ACT_RELU) &&
                        d->drop_p == 0.f && (((uintptr_t)d->C) & 15) == 0 && (d->ldc * 2) % 16 == 0 &&
                        (a.nh == 1 || (d->c_sh * 2) % 16 == 0) && (a.nb == 1 || (d->c_sb * 2) % 16 == 0) && !g_disable_tma_store;
  if (store_ok && !d->scatter_rows) {
    if (make_store_map(&tc, d->C, d->N, d->M, d->ldc, a.nh, d->c_sh, a.nb, d->c_sb) == 0) a.tma_store = 1;
  } else if (store_ok && !g_disable_scatter_tma) {
    // one map per owner: its stage is [world][scatter_rows][N]; M / scatter_rows owners
    const int owners = (d->M + d->scatter_rows - 1) / d->scatter_rows;
    bool ok = owners <= 8;
    for (int o = 0; ok && o < owners; ++o)
      ok = d->scatter[o] && (((uintptr_t)d->scatter[o]) & 15) == 0 &&
           make_store_map(&sm.m[o], d->scatter[o], d->N, (long long)owners * d->scatter_rows, d->ldc, 1, 0, 1, 0) == 0;
    if (ok) a.tma_store = 1;
  }
  if (pair) return launch_pair_major(d->a_mn, d->b_mn, ta, tb, tc, sm, a, max_ctas, stream);
  if (es == 2) {
    if (bn == 256) return launch_major<2, 256>(d->a_mn, d->b_mn, ta, tb, tc, sm, a, max_ctas, stream);
    if (bn == 128) return launch_major<2, 128>(d->a_mn, d->b_mn, ta, tb, tc, sm, a, max_ctas, stream);
    return launch_major<2, 64>(d->a_mn, d->b_mn, ta, tb, tc, sm, a, max_ctas, stream);
  } else {
    if (bn == 128) return launch_major<4, 128>(d->a_mn, d->b_mn, ta, tb, tc, sm, a, max_ctas, stream);
    return launch_major<4, 64>(d->a_mn, d->b_mn, ta, tb, tc, sm, a, max_ctas, stream);
  }
}

// Reads (and clears) the device-side error word written by a bounded wait that
// ran out.  Synchronises the device.
FFK_API int ffk_gemm_last_error() {
  int v = 0, z = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  cudaMemcpyFromSymbol(&v, g_gemm_err, sizeof(int));
  cudaMemcpyToSymbol(g_gemm_err, &z, sizeof(int));
  return v;
}
