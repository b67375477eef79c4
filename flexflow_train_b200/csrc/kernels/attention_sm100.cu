// attention_sm100.cu -- fused multi-head attention core for Blackwell (sm_100a), forward and backward.
//
//   O = dropout(softmax(scale * Q K^T [+ causal mask])) V          per (batch, head)
//
// Replaces the cuDNN multi-head-attention calls of the reference
// (lib/kernels/src/cuda/ops/attention_kernels.cu:224-285: cudnnMultiHeadAttnForward / BackwardData /
// BackwardWeights) for the score / softmax / context part; the projections stay GEMMs.  The [Sq, Sk] score
// matrix never exists in global memory: scores are produced by tcgen05.mma into tensor memory (TMEM), turned into
// probabilities by one thread per query row, written as bf16 into shared memory and multiplied with V by the
// tensor core again.  Only the row log-sum-exp is kept for backward, which recomputes the scores tile by tile.
//
// Layouts.  Q, K, V, O, dO, dQ, dK, dV are [batch * seq, ld] bf16 matrices in which head h occupies the D
// columns starting at h * D (so the packed output of one QKV projection GEMM is used as it lies); D is 64 or 128.
//
// Dropout is counter based: element (b, h, q, k) is kept when 16 bits of hash(seed, row * ceil(Sk / 4) + k / 4),
// row = (b * H + h) * Sq + q, selected by k % 4, are >= p * 65536 (common.cuh: ffk_rand16x4), so backward
// regenerates the mask.  The 1 / (1 - p) factor is applied once per output row / gradient tile.
//
// Forward CTA (320 threads) = one 128-query block of one (batch, head):
//   warp 0      TMA producer: Q once, then K and V tiles of 128 keys through a two-stage ring
//   warp 1      MMA issuer:   S[t] = Q K_j^T   (TMEM, two stages)   and   Opart[t] = P_j V_j   (TMEM, two stages)
//   warps 2-9   softmax and output: thread = query row x half of the tile's keys (and half of the output columns);
//               running max / sum, P_j -> shared memory (bf16, 128-byte swizzle), O = O * alpha_j + Opart[t] in registers
//
// Backward CTA (448 threads) = one 128-query block of one (batch, head), looping over tiles of 64 keys:
//   S = Q K_j^T, dP = dO V_j^T (TMEM, two stages) -> eight warps (thread = query row x 32 keys) compute P and
//   dS = P o (dP - delta) -> shared memory -> dV_j^T = dO^T P, dK_j^T = Q^T dS (TMEM, read out and added to fp32
//   accumulators in global memory by four read-out warps) and dQ += dS K_j (TMEM accumulator, stored once at the end).
//
// Every mbarrier wait is bounded (tcgen05.cuh); on expiry the CTA records a code in the library's error word,
// frees its TMEM and returns.
#include <cstdlib>

#include "tcgen05.cuh"

namespace {

constexpr int ATT_THREADS = 320;
constexpr int BQ = 128;    // query rows per CTA
constexpr int BKF = 128;   // keys per forward tile
constexpr int BKB = 64;    // keys per backward tile
constexpr float LOG2E = 1.4426950408889634f;

struct AttnArgs {
  int B, H, Sq, Sk;
  float scale;            // applied to Q K^T
  int causal;             // 1: key k is visible to query q iff k <= q (Sq == Sk)
  float drop_p;
  unsigned long long drop_salt;
  const unsigned long long *drop_seed_ptr;
  bf16 *O;                // forward output [B*Sq, ldo]
  long long ldo;
  float *lse;             // [B, H, Sq] log2-domain log-sum-exp of the scaled scores
  // backward only
  const float *delta;     // [B, H, Sq] rowsum(dO o O)
  bf16 *dQ;
  long long lddq;
  float *dK_acc, *dV_acc; // [B, H, Sk, D] fp32, zeroed by the caller
  int *err;
  int dbg;                // experiment switches (FFK_ATTN_DBG): parts of the kernel left out to time the rest
};

// Timeline of one CTA (experiment switch 4096): SM clock at event `ev` (0..31) of step `j` (0..63), one slot each, written
// with a plain store by the roles' first lanes.
__device__ long long g_attn_trace[32 * 64];
__device__ __forceinline__ void attn_trace(const AttnArgs &p, int ev, int j) {
  if ((p.dbg & 4096) && blockIdx.x == 0 && (threadIdx.x & 31) == 0 && j < 64) g_attn_trace[ev * 64 + j] = clock64();
}

__device__ __forceinline__ unsigned long long attn_seed(const AttnArgs &p) {
  return p.drop_seed_ptr ? p.drop_salt * 0x9E3779B97F4A7C15ull + *p.drop_seed_ptr : p.drop_salt;
}

// instruction descriptor: D f32, A/B bf16, majors, N, M
__host__ __device__ constexpr uint32_t attn_idesc(int M, int N, int a_mn, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) | ((uint32_t)(N >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void warp_arrive(uint64_t *bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

// keep bits of the four keys 4*g4 .. 4*g4+3 of one row
__device__ __forceinline__ uint64_t attn_rand4(unsigned long long seed, unsigned long long row_groups_base, int g4) {
  return ffk_rand16x4(seed, row_groups_base + (unsigned long long)g4);
}

// ================================================================================================ forward
template <int D>
struct FwdCfg {
  static constexpr int PANELS = D / 64;              // 64-column (128-byte) panels per row of Q / K / V
  static constexpr int Q_BYTES = BQ * D * 2;
  static constexpr int KV_BYTES = BKF * D * 2;       // one K or one V tile
  static constexpr int P_BYTES = BQ * BKF * 2;       // 32 KB
  // A K tile is free again once the scores of its step are computed, a V tile only at the end of its step: the V ring
  // is one stage deeper so that its loads also run a full step ahead.
  static constexpr int NK = 2, NV = 3;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + NK * KV_BYTES;
  static constexpr int OFF_P = OFF_V + NV * KV_BYTES;
  static constexpr int OFF_XCHG = OFF_P + P_BYTES;           // [2 tile parities][2 column halves][128 rows] floats
  static constexpr int OFF_BAR = OFF_XCHG + 4 * 128 * 4;
  static constexpr int SLACK = D == 128 ? 768 : 1024;        // room to align the base to 1024 bytes (checked in the kernel)
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + SLACK;
  static constexpr int TMEM_S = 0;                           // S[t] at columns t * 128
  static constexpr int TMEM_O = 256;                         // Opart[t] at columns 256 + t * D
  static constexpr uint32_t IDESC_S = attn_idesc(128, BKF, 0, 0);
  static constexpr uint32_t IDESC_PV = attn_idesc(128, D, 0, 1);
};

// named barrier of the two warps that share a TMEM lane quarter (ids 1..4; 0 is __syncthreads)
__device__ __forceinline__ void pair_sync(int quarter) { asm volatile("bar.sync %0, 64;" ::"r"(quarter + 1) : "memory"); }

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnArgs p) {
  using C = FwdCfg<D>;
  constexpr int DH = D / 2;                          // output columns owned by one thread
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float *xchg = (float *)(smem + C::OFF_XCHG);       // [2][2][128]
  uint64_t *bars = (uint64_t *)(smem + C::OFF_BAR);
  uint64_t *q_full = bars;            // 1
  uint64_t *k_full = bars + 1;        // [2]
  uint64_t *k_empty = bars + 5;       // [2]
  uint64_t *v_full = bars + 19;       // [NV]
  uint64_t *v_empty = bars + 22;      // [NV]
  uint64_t *s_full = bars + 9;        // [2]
  uint64_t *s_empty = bars + 11;      // [2] 8 warps
  uint64_t *p_full = bars + 13;       // 8 warps
  uint64_t *p_empty = bars + 14;      // commit
  uint64_t *o_full = bars + 15;       // [2] commit
  uint64_t *o_empty = bars + 17;      // [2] 8 warps
  uint32_t *tmem_slot = (uint32_t *)(bars + 25);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
  if ((uintptr_t)(smem - smem_raw) > (uintptr_t)C::SLACK) {  // the launch did not leave room to align the tiles: refuse
    if (threadIdx.x == 0 && p.err) atomicCAS(p.err, 0, (int)FFK_ERR_BAD_ARG);
    return;
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.Sq + BQ - 1) / BQ;
  const int qb = blockIdx.x % nqb;
  const int bh = blockIdx.x / nqb;
  const int h = bh % p.H, b = bh / p.H;
  const int q0 = qb * BQ;
  int n_tiles = (p.Sk + BKF - 1) / BKF;
  if (p.causal) {
    const int last = (min(q0 + BQ, p.Sq) - 1) / BKF + 1;   // tiles that contain a key <= the block's last query
    n_tiles = min(n_tiles, last);
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 8); mbar_init(&o_full[s], 1); mbar_init(&o_empty[s], 8);
    }
    for (int s = 0; s < C::NV; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    mbar_init(p_full, 8); mbar_init(p_empty, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, C::Q_BYTES);
#pragma unroll
      for (int c = 0; c < C::PANELS; ++c) tma_load_4d(smem_u32(smem + C::OFF_Q + c * BQ * 128), &tmQ, q_full, c * 64, q0, h, b);
      // the K and V rings advance independently; the wait for progress on either is bounded
      int kj = 0, vj = 0;
      uint64_t t0 = ffk_globaltimer();
      uint32_t spins = 0;
      while (kj < n_tiles || vj < n_tiles) {
        bool progress = false;
        if (kj < n_tiles) {
          const int t = kj % C::NK;
          if (mbar_try_wait(&k_empty[t], ((uint32_t)(kj / C::NK) & 1u) ^ 1u)) {
            mbar_expect_tx(&k_full[t], C::KV_BYTES);
#pragma unroll
            for (int c = 0; c < C::PANELS; ++c)
              tma_load_4d(smem_u32(smem + C::OFF_K + t * C::KV_BYTES + c * BKF * 128), &tmK, &k_full[t], c * 64, kj * BKF, h, b);
            ++kj;
            progress = true;
          }
        }
        if (vj < n_tiles) {
          const int t = vj % C::NV;
          if (mbar_try_wait(&v_empty[t], ((uint32_t)(vj / C::NV) & 1u) ^ 1u)) {
            mbar_expect_tx(&v_full[t], C::KV_BYTES);
#pragma unroll
            for (int c = 0; c < C::PANELS; ++c)
              tma_load_4d(smem_u32(smem + C::OFF_V + t * C::KV_BYTES + c * BKF * 128), &tmV, &v_full[t], c * 64, vj * BKF, h, b);
            ++vj;
            progress = true;
          }
        }
        if (progress) {
          t0 = ffk_globaltimer();
        } else if ((++spins & 63u) == 0) {
          if (*abort_flag) break;
          if (ffk_globaltimer() - t0 > WAIT_LIMIT_NS) {
            *abort_flag = 1;
            if (p.err) atomicCAS(p.err, 0, (int)FFK_ERR_TIMEOUT_PRODUCER);
            break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA);
      // descriptors are built once; an MMA then costs two adds
      const uint64_t dq = make_smem_desc(smem_u32(smem + C::OFF_Q), 16, 1024);
      const uint64_t dk0 = make_smem_desc(smem_u32(smem + C::OFF_K), 16, 1024);
      const uint64_t dp = make_smem_desc(smem_u32(smem + C::OFF_P), 16, 1024);
      const uint64_t dv0 = make_smem_desc(smem_u32(smem + C::OFF_V), BKF * 128, 1024);
      auto issue_s = [&](int j) -> bool {
        const int t = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        if (!mbar_wait(&k_full[t], ph, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA)) return false;
        if (!mbar_wait(&s_empty[t], ph ^ 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint64_t dk = desc_advance(dk0, (uint32_t)(t * C::KV_BYTES));
        const uint32_t d_tmem = tmem_base + (uint32_t)(C::TMEM_S + t * 128);
        if (!(p.dbg & 16)) {
          tc_mma_bf16<false>(d_tmem, dq, dk, C::IDESC_S);
#pragma unroll
          for (int ks = 1; ks < D / 16; ++ks) {
            const uint32_t off = (uint32_t)((ks >> 2) * (BQ * 128) + (ks & 3) * 32);   // panel, then 32 bytes per k-step
            tc_mma_bf16<true>(d_tmem, desc_advance(dq, off), desc_advance(dk, off), C::IDESC_S);
          }
        }
        tc_commit(&s_full[t]);
        tc_commit(&k_empty[t]);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int t = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        if (j + 1 < n_tiles) { ok = issue_s(j + 1); if (!ok) break; }
        const int vt = j % C::NV;
        ok = mbar_wait(&v_full[vt], (uint32_t)(j / C::NV) & 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA) &&
             mbar_wait(p_full, (uint32_t)j & 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA) &&
             mbar_wait(&o_empty[t], ph ^ 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        const uint64_t dv = desc_advance(dv0, (uint32_t)(vt * C::KV_BYTES));
        const uint32_t d_tmem = tmem_base + (uint32_t)(C::TMEM_O + t * D);
        if (!(p.dbg & 2)) {
          // A = P (K-major, two panels of 64 keys); B = V (N = head dim contiguous: MN-major, 16 key rows per step)
          tc_mma_bf16<false>(d_tmem, dp, dv, C::IDESC_PV);
#pragma unroll
          for (int ks = 1; ks < BKF / 16; ++ks) {
            const uint32_t a_off = (uint32_t)((ks >> 2) * (BQ * 128) + (ks & 3) * 32);
            const uint32_t b_off = (uint32_t)(ks * 16 * 128);
            tc_mma_bf16<true>(d_tmem, desc_advance(dp, a_off), desc_advance(dv, b_off), C::IDESC_PV);
          }
        }
        tc_commit(&o_full[t]);
        tc_commit(&v_empty[vt]);
        tc_commit(p_empty);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + output accumulation
    // Eight warps: warp w works on TMEM lane quarter w % 4 (a hardware rule) and on column half (w - 2) / 4, so a thread is
    // one query row and 64 of the tile's 128 keys (and D / 2 of the output columns).  Two warps per scheduler hide each
    // other's TMEM-load and special-function latencies; the row maximum is the only thing the two halves must agree on
    // per tile and goes through a two-float exchange in shared memory.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const int q = q0 + r;
    const float sl2 = p.scale * LOG2E;
    float m = -INFINITY, l = 0.f;
    const bool drop = p.drop_p > 0.f;
    const uint32_t thr = ffk_drop_threshold(p.drop_p);
    const unsigned long long seed = drop ? attn_seed(p) : 0ull;
    const unsigned long long groups_per_row = (unsigned long long)((p.Sk + 3) >> 2);
    const unsigned long long row_base = ((unsigned long long)(b * p.H + h) * p.Sq + (unsigned long long)q) * groups_per_row;
    const uint32_t prow = smem_u32(smem + C::OFF_P + half * (BQ * 128) + r * 128);   // this row in this half's 64-key panel
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    float o[DH];
#pragma unroll
    for (int i = 0; i < DH; ++i) o[i] = 0.f;
    float alpha_pending = 1.f;
    bool ok = true;
    // O += Opart of tile jj (rescaled by the factor that tile's softmax produced)
    auto accumulate = [&](int jj, float alpha) -> bool {
      const int t = jj & 1;
      bool k_ = mbar_wait(&o_full[t], (uint32_t)(jj >> 1) & 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      k_ = __all_sync(0xffffffffu, k_);
      if (!k_) return false;
      tc_fence_after();
      const uint32_t t_o = lane_base + (uint32_t)(C::TMEM_O + t * D + half * DH);
      uint32_t ra[32];
      if (p.dbg & 8) { tc_fence_before(); warp_arrive(&o_empty[t], lane); return true; }
      tmem_ld32(t_o, ra);
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) {
        tmem_ld_wait();
        uint32_t rb[32];
        if (c + 1 < DH / 32) tmem_ld32(t_o + (uint32_t)((c + 1) * 32), rb);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha, __uint_as_float(ra[i]));
        if (c + 1 < DH / 32) {
#pragma unroll
          for (int i = 0; i < 32; ++i) ra[i] = rb[i];
        }
      }
      tc_fence_before();
      warp_arrive(&o_empty[t], lane);
      return true;
    };
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int t = j & 1;
      const uint32_t ph = (uint32_t)(j >> 1) & 1u;
      ok = mbar_wait(&s_full[t], ph, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_s = lane_base + (uint32_t)(C::TMEM_S + t * 128 + half * 64);
      uint32_t rs[64];
      tmem_ld32(t_s, *reinterpret_cast<uint32_t(*)[32]>(&rs[0]));
      tmem_ld32(t_s + 32u, *reinterpret_cast<uint32_t(*)[32]>(&rs[32]));
      tmem_ld_wait();
      tc_fence_before();
      warp_arrive(&s_empty[t], lane);     // the scores are in registers: the next-but-one tile may overwrite them
      const int k0 = j * BKF + half * 64;
      // columns of this half that exist / are visible to this row
      int kmax = p.Sk - k0;
      if (p.causal) kmax = min(kmax, q - k0 + 1);
      const bool full = kmax >= 64;
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
      if (full) {
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
          mx0 = fmaxf(mx0, __uint_as_float(rs[i])); mx1 = fmaxf(mx1, __uint_as_float(rs[i + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(rs[i + 2])); mx3 = fmaxf(mx3, __uint_as_float(rs[i + 3]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) mx0 = fmaxf(mx0, i < kmax ? __uint_as_float(rs[i]) : -INFINITY);
      }
      const float mine = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      xchg[(t * 2 + half) * 128 + r] = mine;
      pair_sync(quarter);
      const float other = xchg[(t * 2 + (half ^ 1)) * 128 + r];
      float m_new = fmaxf(m, fmaxf(mine, other) * sl2);
      if (m_new == -INFINITY) m_new = 0.f;        // nothing visible yet (padding rows only)
      const float alpha = exp2f(m - m_new);
      float ls0 = 0.f, ls1 = 0.f, ls2 = 0.f, ls3 = 0.f;
      if (!(p.dbg & 1))
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
        float e0 = exp2f(fmaf(__uint_as_float(rs[i]), sl2, -m_new)), e1 = exp2f(fmaf(__uint_as_float(rs[i + 1]), sl2, -m_new));
        float e2 = exp2f(fmaf(__uint_as_float(rs[i + 2]), sl2, -m_new)), e3 = exp2f(fmaf(__uint_as_float(rs[i + 3]), sl2, -m_new));
        if (!full) {
          if (i >= kmax) e0 = 0.f;
          if (i + 1 >= kmax) e1 = 0.f;
          if (i + 2 >= kmax) e2 = 0.f;
          if (i + 3 >= kmax) e3 = 0.f;
        }
        ls0 += e0; ls1 += e1; ls2 += e2; ls3 += e3;
        if (drop) {
          const uint64_t z = attn_rand4(seed, row_base, (k0 + i) >> 2);
          if ((uint32_t)(z & 0xFFFFu) < thr) e0 = 0.f;
          if ((uint32_t)((z >> 16) & 0xFFFFu) < thr) e1 = 0.f;
          if ((uint32_t)((z >> 32) & 0xFFFFu) < thr) e2 = 0.f;
          if ((uint32_t)(z >> 48) < thr) e3 = 0.f;
        }
        rs[i >> 1] = pack_bf162(e0, e1);            // probabilities packed in place (pair i/2, i/2 + 1 are already consumed)
        rs[(i >> 1) + 1] = pack_bf162(e2, e3);
      }
      ok = mbar_wait(p_empty, ((uint32_t)j & 1u) ^ 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      // 64 probabilities = 128 bytes = the eight 16-byte chunks of this row in this half's panel; chunk index XOR (row % 8)
      // is the 128-byte swizzle the MMA descriptor expects
      if (!(p.dbg & 4))
#pragma unroll
      for (int u = 0; u < 8; ++u)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + (uint32_t)((u ^ (r & 7)) << 4)), "r"(rs[4 * u]), "r"(rs[4 * u + 1]),
                     "r"(rs[4 * u + 2]), "r"(rs[4 * u + 3])
                     : "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      warp_arrive(p_full, lane);
      l = l * alpha + ((ls0 + ls1) + (ls2 + ls3));
      m = m_new;
      // the previous tile's P.V has had this tile's softmax to finish under
      if (j > 0) ok = accumulate(j - 1, alpha_pending);
      alpha_pending = alpha;
    }
    if (ok && n_tiles > 0) ok = accumulate(n_tiles - 1, alpha_pending);
    if (ok) {
      // row sum over both halves, then out = O / (sum * keep probability); the half-0 thread stores the log-sum-exp
      xchg[half * 128 + r] = l;
      pair_sync(quarter);
      const float lt = l + xchg[(half ^ 1) * 128 + r];
      const float inv_keep = p.drop_p > 0.f ? 1.f / (1.f - p.drop_p) : 1.f;
      const float f = lt > 0.f ? inv_keep / lt : 0.f;
      if (q < p.Sq) {
        if (half == 0 && p.lse) p.lse[((long long)(b * p.H + h)) * p.Sq + q] = lt > 0.f ? m + log2f(lt) : INFINITY;
        bf16 *orow = p.O + ((long long)b * p.Sq + q) * p.ldo + (long long)h * D + half * DH;
#pragma unroll
        for (int c = 0; c < DH / 8; ++c) {
          uint4 v = make_uint4(pack_bf162(o[8 * c] * f, o[8 * c + 1] * f), pack_bf162(o[8 * c + 2] * f, o[8 * c + 3] * f),
                               pack_bf162(o[8 * c + 4] * f, o[8 * c + 5] * f), pack_bf162(o[8 * c + 6] * f, o[8 * c + 7] * f));
          *reinterpret_cast<uint4 *>(orow + 8 * c) = v;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ================================================================================================ backward
// delta[b, h, q] = sum_c dO[b, q, h, c] * O[b, q, h, c]; one warp per (row, head)
template <int D>
__global__ void attn_delta_kernel(const bf16 *__restrict__ dO, long long lddo, const bf16 *__restrict__ O, long long ldo,
                                  float *__restrict__ delta, int B, int H, int Sq) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long total = (long long)B * Sq * H;
  if (w >= total) return;
  const int h = (int)(w % H);
  const long long row = w / H;   // b * Sq + q
  const bf16 *a = dO + row * lddo + (long long)h * D, *c = O + row * ldo + (long long)h * D;
  float s = 0.f;
  constexpr int PER = D / 32;    // 2 or 4 elements per lane
  if constexpr (PER == 4) {
    uint2 ua = *reinterpret_cast<const uint2 *>(a + lane * 4), uc = *reinterpret_cast<const uint2 *>(c + lane * 4);
    float2 a0 = unpack_bf162(ua.x), a1 = unpack_bf162(ua.y), c0 = unpack_bf162(uc.x), c1 = unpack_bf162(uc.y);
    s = a0.x * c0.x + a0.y * c0.y + a1.x * c1.x + a1.y * c1.y;
  } else {
    uint32_t ua = *reinterpret_cast<const uint32_t *>(a + lane * 2), uc = *reinterpret_cast<const uint32_t *>(c + lane * 2);
    float2 a0 = unpack_bf162(ua), c0 = unpack_bf162(uc);
    s = a0.x * c0.x + a0.y * c0.y;
  }
  s = warp_sum(s);
  if (lane == 0) {
    const long long b = row / Sq, q = row - b * Sq;
    delta[(b * H + h) * Sq + q] = s;
  }
}

// fp32 accumulators [B, H, Sk, D] -> bf16 [B*Sk, ld] (head h at columns h*D)
template <int D>
__global__ void attn_acc_to_bf16_kernel(const float *__restrict__ acc, bf16 *__restrict__ out, long long ld, int B, int H, int Sk) {
  const long long total = (long long)B * H * Sk * (D / 4);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c4 = (int)(i % (D / 4));
    long long rest = i / (D / 4);
    const int k = (int)(rest % Sk);
    rest /= Sk;
    const int h = (int)(rest % H);
    const long long b = rest / H;
    const float4 v = *reinterpret_cast<const float4 *>(acc + i * 4);
    *reinterpret_cast<uint2 *>(out + (b * Sk + k) * ld + (long long)h * D + c4 * 4) = make_uint2(pack_bf162(v.x, v.y), pack_bf162(v.z, v.w));
  }
}

struct BwdCfg {
  static constexpr int D = 128;
  static constexpr int Q_BYTES = BQ * D * 2;          // 32 KB (also dO)
  static constexpr int KV_BYTES = BKB * D * 2;        // 16 KB: two panels of [64 keys x 128 B]
  static constexpr int PS_BYTES = BQ * BKB * 2;       // 16 KB: P or dS tile, [128 rows x 128 B]
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = OFF_Q + Q_BYTES;
  // A K tile is needed from the first MMA of its step (S) to the last (dQ), a V tile only by the second (dP): with the
  // step's shared-memory budget the K ring gets four stages and the V ring two, so that a K load is issued three steps
  // before its first use and the load latency stays off the critical path.
  static constexpr int NK = 4, NV = 2;
  static constexpr int OFF_K = OFF_DO + Q_BYTES;       // [NK]
  static constexpr int OFF_V = OFF_K + NK * KV_BYTES;  // [NV]
  static constexpr int OFF_P = OFF_V + NV * KV_BYTES;  // [2]
  static constexpr int OFF_DS = OFF_P + 2 * PS_BYTES; // [2]
  static constexpr int OFF_BAR = OFF_DS + 2 * PS_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  // Tensor memory.  S and dP are copied into registers the moment they are complete, so one stage each is enough; dV^T and
  // dK^T stay until four warps have added them to global memory, so they get two stages and the tensor core never waits
  // for that read-out.
  static constexpr int TMEM_S = 0;      // 64 columns
  static constexpr int TMEM_DP = 64;    // 64 columns
  static constexpr int TMEM_DVT = 128;  // dV^T[u] at 128 + u * 128 (64 columns)
  static constexpr int TMEM_DKT = 192;  // dK^T[u] at 192 + u * 128 (64 columns)
  static constexpr int TMEM_DQ = 384;   // 128 columns
  static constexpr uint32_t IDESC_S = attn_idesc(128, BKB, 0, 0);     // Q K^T, dO V^T
  static constexpr uint32_t IDESC_T = attn_idesc(128, BKB, 1, 1);     // dO^T P, Q^T dS   (both operands MN-major)
  static constexpr uint32_t IDESC_DQ = attn_idesc(128, D, 0, 1);      // dS K
};

constexpr int BWD_THREADS = 576;  // TMA warp, MMA warp, 8 dS warps, 8 read-out warps

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const AttnArgs p) {
  using C = BwdCfg;
  constexpr int D = C::D;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t *bars = (uint64_t *)(smem + C::OFF_BAR);
  uint64_t *q_full = bars;            // Q and dO
  uint64_t *v_full = bars + 1;        // [2]
  uint64_t *v_empty = bars + 3;       // [2] commit
  uint64_t *sdp_full = bars + 5;      // commit
  uint64_t *sdp_empty = bars + 6;     // 8 warps
  uint64_t *pds_full = bars + 7;      // [2] 8 warps
  uint64_t *pds_empty = bars + 9;     // [2] commit
  uint64_t *dkv_full = bars + 11;     // [2] commit
  uint64_t *dkv_empty = bars + 13;    // [2] 4 warps
  uint64_t *dq_full = bars + 15;      // commit
  uint64_t *k_full = bars + 16;       // [NK]
  uint64_t *k_empty = bars + 20;      // [NK] commit
  uint32_t *tmem_slot = (uint32_t *)(bars + 24);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.Sq + BQ - 1) / BQ;
  const int qb = blockIdx.x % nqb;
  const int bh = blockIdx.x / nqb;
  const int h = bh % p.H, b = bh / p.H;
  const int q0 = qb * BQ;
  int n_tiles = (p.Sk + BKB - 1) / BKB;
  if (p.causal) n_tiles = min(n_tiles, (min(q0 + BQ, p.Sq) - 1) / BKB + 1);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
      mbar_init(&pds_full[s], 8); mbar_init(&pds_empty[s], 1); mbar_init(&dkv_full[s], 1); mbar_init(&dkv_empty[s], 8);
    }
    for (int s = 0; s < C::NK; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    mbar_init(sdp_full, 1); mbar_init(sdp_empty, 8); mbar_init(dq_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * C::Q_BYTES);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        tma_load_4d(smem_u32(smem + C::OFF_Q + c * BQ * 128), &tmQ, q_full, c * 64, q0, h, b);
        tma_load_4d(smem_u32(smem + C::OFF_DO + c * BQ * 128), &tmDO, q_full, c * 64, q0, h, b);
      }
      // the K and V rings advance independently: whichever has a free stage gets its next tile; the wait for progress
      // on either is bounded like every other wait
      int kj = 0, vj = 0;
      uint64_t t0 = ffk_globaltimer();
      uint32_t spins = 0;
      while (kj < n_tiles || vj < n_tiles) {
        bool progress = false;
        if (kj < n_tiles) {
          const int t = kj % C::NK;
          if (mbar_try_wait(&k_empty[t], ((uint32_t)(kj / C::NK) & 1u) ^ 1u)) {
            mbar_expect_tx(&k_full[t], C::KV_BYTES);
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tma_load_4d(smem_u32(smem + C::OFF_K + t * C::KV_BYTES + c * BKB * 128), &tmK, &k_full[t], c * 64, kj * BKB, h, b);
            ++kj;
            progress = true;
          }
        }
        if (vj < n_tiles) {
          const int t = vj % C::NV;
          if (mbar_try_wait(&v_empty[t], ((uint32_t)(vj / C::NV) & 1u) ^ 1u)) {
            mbar_expect_tx(&v_full[t], C::KV_BYTES);
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tma_load_4d(smem_u32(smem + C::OFF_V + t * C::KV_BYTES + c * BKB * 128), &tmV, &v_full[t], c * 64, vj * BKB, h, b);
            ++vj;
            progress = true;
          }
        }
        if (progress) {
          t0 = ffk_globaltimer();
        } else if ((++spins & 63u) == 0) {
          if (*abort_flag) break;
          if (ffk_globaltimer() - t0 > WAIT_LIMIT_NS) {
            *abort_flag = 1;
            if (p.err) atomicCAS(p.err, 0, (int)FFK_ERR_TIMEOUT_PRODUCER);
            break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA);
      // descriptors are built once; an MMA then costs two adds
      const uint64_t dqA = make_smem_desc(smem_u32(smem + C::OFF_Q), 16, 1024), ddoA = make_smem_desc(smem_u32(smem + C::OFF_DO), 16, 1024);
      const uint64_t dqT = make_smem_desc(smem_u32(smem + C::OFF_Q), BQ * 128, 1024), ddoT = make_smem_desc(smem_u32(smem + C::OFF_DO), BQ * 128, 1024);
      const uint64_t dkB0 = make_smem_desc(smem_u32(smem + C::OFF_K), 16, 1024), dkN0 = make_smem_desc(smem_u32(smem + C::OFF_K), BKB * 128, 1024);
      const uint64_t dvB0 = make_smem_desc(smem_u32(smem + C::OFF_V), 16, 1024);
      const uint64_t dpN0 = make_smem_desc(smem_u32(smem + C::OFF_P), BQ * 128, 1024), ddsN0 = make_smem_desc(smem_u32(smem + C::OFF_DS), BQ * 128, 1024);
      const uint64_t ddsA0 = make_smem_desc(smem_u32(smem + C::OFF_DS), 16, 1024);
      // S = Q K_j^T and dP = dO V_j^T : K-major operands, k-steps of 16 head-dim columns
      auto issue_sdp = [&](int j) -> bool {
        const int t = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        const int kt = j % C::NK;
        if (!mbar_wait(&k_full[kt], (uint32_t)(j / C::NK) & 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA)) return false;
        if (!mbar_wait(sdp_empty, ((uint32_t)j & 1u) ^ 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint64_t dkB = desc_advance(dkB0, (uint32_t)(kt * C::KV_BYTES)), dvB = desc_advance(dvB0, (uint32_t)(t * C::KV_BYTES));
        if (!(p.dbg & 32)) {
          tc_mma_bf16<false>(tmem_base + (uint32_t)C::TMEM_S, dqA, dkB, C::IDESC_S);
#pragma unroll
          for (int ks = 1; ks < D / 16; ++ks) {
            const uint32_t a_off = (uint32_t)((ks >> 2) * (BQ * 128) + (ks & 3) * 32);
            const uint32_t b_off = (uint32_t)((ks >> 2) * (BKB * 128) + (ks & 3) * 32);
            tc_mma_bf16<true>(tmem_base + (uint32_t)C::TMEM_S, desc_advance(dqA, a_off), desc_advance(dkB, b_off), C::IDESC_S);
          }
        }
        if (!mbar_wait(&v_full[t], ph, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA)) return false;
        if (!(p.dbg & 32)) {
          tc_mma_bf16<false>(tmem_base + (uint32_t)C::TMEM_DP, ddoA, dvB, C::IDESC_S);
#pragma unroll
          for (int ks = 1; ks < D / 16; ++ks) {
            const uint32_t a_off = (uint32_t)((ks >> 2) * (BQ * 128) + (ks & 3) * 32);
            const uint32_t b_off = (uint32_t)((ks >> 2) * (BKB * 128) + (ks & 3) * 32);
            tc_mma_bf16<true>(tmem_base + (uint32_t)C::TMEM_DP, desc_advance(ddoA, a_off), desc_advance(dvB, b_off), C::IDESC_S);
          }
        }
        tc_commit(sdp_full);
        tc_commit(&v_empty[t]);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_sdp(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int t = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        attn_trace(p, 0, j);
        if (j + 1 < n_tiles) { ok = issue_sdp(j + 1); if (!ok) break; }
        attn_trace(p, 1, j);
        ok = mbar_wait(&pds_full[t], ph, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA);
        attn_trace(p, 2, j);
        ok = ok && mbar_wait(&dkv_empty[t], ph ^ 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA);
        attn_trace(p, 3, j);
        if (!ok) break;
        tc_fence_after();
        const uint64_t dpN = desc_advance(dpN0, (uint32_t)(t * C::PS_BYTES)), ddsN = desc_advance(ddsN0, (uint32_t)(t * C::PS_BYTES));
        const uint64_t ddsA = desc_advance(ddsA0, (uint32_t)(t * C::PS_BYTES));
        const uint64_t dkN = desc_advance(dkN0, (uint32_t)((j % C::NK) * C::KV_BYTES));
        // dV_j^T [D x 64] = dO^T P and dK_j^T = Q^T dS: A = dO / Q read M-major (M = head dim: two 64-column panels, LBO = panel
        // stride), B = P / dS read N-major (N = 64 keys, one panel); every k-step is 16 query rows = 2048 bytes
        if (!(p.dbg & 64)) {
          const uint32_t dvt = tmem_base + (uint32_t)(C::TMEM_DVT + t * 128), dkt = tmem_base + (uint32_t)(C::TMEM_DKT + t * 128);
          tc_mma_bf16<false>(dvt, ddoT, dpN, C::IDESC_T);
#pragma unroll
          for (int ks = 1; ks < BQ / 16; ++ks) tc_mma_bf16<true>(dvt, desc_advance(ddoT, ks * 2048u), desc_advance(dpN, ks * 2048u), C::IDESC_T);
          tc_mma_bf16<false>(dkt, dqT, ddsN, C::IDESC_T);
#pragma unroll
          for (int ks = 1; ks < BQ / 16; ++ks) tc_mma_bf16<true>(dkt, desc_advance(dqT, ks * 2048u), desc_advance(ddsN, ks * 2048u), C::IDESC_T);
        }
        tc_commit(&dkv_full[t]);
        // dQ += dS K_j: A = dS K-major (64 keys = one panel, 32 bytes per k-step), B = K_j N-major (N = head dim, 16 key rows per step)
        if (!(p.dbg & 128)) {
          const uint32_t dqt = tmem_base + (uint32_t)C::TMEM_DQ;
          if (j == 0) tc_mma_bf16<false>(dqt, ddsA, dkN, C::IDESC_DQ);
          else tc_mma_bf16<true>(dqt, ddsA, dkN, C::IDESC_DQ);
#pragma unroll
          for (int ks = 1; ks < BKB / 16; ++ks) tc_mma_bf16<true>(dqt, desc_advance(ddsA, ks * 32u), desc_advance(dkN, ks * 2048u), C::IDESC_DQ);
        }
        tc_commit(&k_empty[j % C::NK]);
        tc_commit(&pds_empty[t]);
        attn_trace(p, 4, j);
      }
      if (ok) tc_commit(dq_full);
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------------ P and dS: thread = query row x 32 of the tile's 64 keys
    // Eight warps, two per TMEM lane quarter (w % 4), each on one half of the key columns, so that every scheduler has two
    // warps to switch between while tensor-memory loads and exponentials are in flight.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const int q = q0 + r;
    const float sl2 = p.scale * LOG2E;
    const bool row_ok = q < p.Sq;
    const long long stat = ((long long)(b * p.H + h)) * p.Sq + q;
    const float lse = row_ok ? p.lse[stat] : INFINITY;
    const float dlt = row_ok ? p.delta[stat] : 0.f;
    const bool drop = p.drop_p > 0.f;
    const float inv_keep = drop ? 1.f / (1.f - p.drop_p) : 1.f;
    const uint32_t thr = ffk_drop_threshold(p.drop_p);
    const unsigned long long seed = drop ? attn_seed(p) : 0ull;
    const unsigned long long groups_per_row = (unsigned long long)((p.Sk + 3) >> 2);
    const unsigned long long row_base = ((unsigned long long)(b * p.H + h) * p.Sq + (unsigned long long)q) * groups_per_row;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int t = j & 1;
      const uint32_t ph = (uint32_t)(j >> 1) & 1u;
      ok = mbar_wait(sdp_full, (uint32_t)j & 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (warp == 2) attn_trace(p, 10, j);
      tc_fence_after();
      uint32_t rs[32], rd[32];
      tmem_ld32(lane_base + (uint32_t)(C::TMEM_S + half * 32), rs);
      tmem_ld32(lane_base + (uint32_t)(C::TMEM_DP + half * 32), rd);
      tmem_ld_wait();
      tc_fence_before();
      if (warp == 2) attn_trace(p, 11, j);
      warp_arrive(sdp_empty, lane);       // scores and dP are in registers
      const int k0 = j * BKB + half * 32;
      int kmax = p.Sk - k0;
      if (p.causal) kmax = min(kmax, q - k0 + 1);
      const bool full = kmax >= 32;
      // rs <- packed P (dropped entries zeroed: the operand of dV), rd <- packed dS = P o (dP o mask / keep - delta)
      if (!(p.dbg & 256))
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        float e[4], g[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          e[u] = exp2f(fmaf(__uint_as_float(rs[i + u]), sl2, -lse));
          if (!full && i + u >= kmax) e[u] = 0.f;
          g[u] = __uint_as_float(rd[i + u]) * inv_keep;
        }
        if (drop) {
          const uint64_t z = attn_rand4(seed, row_base, (k0 + i) >> 2);
          const bool d0 = (uint32_t)(z & 0xFFFFu) < thr, d1 = (uint32_t)((z >> 16) & 0xFFFFu) < thr;
          const bool d2 = (uint32_t)((z >> 32) & 0xFFFFu) < thr, d3 = (uint32_t)(z >> 48) < thr;
          g[0] = e[0] * ((d0 ? 0.f : g[0]) - dlt); g[1] = e[1] * ((d1 ? 0.f : g[1]) - dlt);
          g[2] = e[2] * ((d2 ? 0.f : g[2]) - dlt); g[3] = e[3] * ((d3 ? 0.f : g[3]) - dlt);
          if (d0) e[0] = 0.f;
          if (d1) e[1] = 0.f;
          if (d2) e[2] = 0.f;
          if (d3) e[3] = 0.f;
        } else {
#pragma unroll
          for (int u = 0; u < 4; ++u) g[u] = e[u] * (g[u] - dlt);
        }
        rs[i >> 1] = pack_bf162(e[0], e[1]); rs[(i >> 1) + 1] = pack_bf162(e[2], e[3]);
        rd[i >> 1] = pack_bf162(g[0], g[1]); rd[(i >> 1) + 1] = pack_bf162(g[2], g[3]);
      }
      if (warp == 2) attn_trace(p, 12, j);
      ok = mbar_wait(&pds_empty[t], ph ^ 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (warp == 2) attn_trace(p, 13, j);
      const uint32_t prow = smem_u32(smem + C::OFF_P + t * C::PS_BYTES + r * 128);
      const uint32_t dsrow = smem_u32(smem + C::OFF_DS + t * C::PS_BYTES + r * 128);
      if (!(p.dbg & 512))
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t sw = (uint32_t)(((half * 4 + u) ^ (r & 7)) << 4);   // 16-byte chunk index XOR row % 8: the 128-byte swizzle
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + sw), "r"(rs[4 * u]), "r"(rs[4 * u + 1]), "r"(rs[4 * u + 2]),
                     "r"(rs[4 * u + 3])
                     : "memory");
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dsrow + sw), "r"(rd[4 * u]), "r"(rd[4 * u + 1]), "r"(rd[4 * u + 2]),
                     "r"(rd[4 * u + 3])
                     : "memory");
      }
      if (warp == 2) attn_trace(p, 14, j);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      warp_arrive(&pds_full[t], lane);
      if (warp == 2) attn_trace(p, 15, j);
    }
    // dQ of this block: scale * accumulator -> bf16; each half stores 64 of the 128 columns
    if (ok) {
      ok = mbar_wait(dq_full, 0, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      bf16 *dqrow = p.dQ + ((long long)b * p.Sq + q) * p.lddq + (long long)h * D + half * (D / 2);
#pragma unroll 1
      for (int c = 0; c < D / 64; ++c) {
        uint32_t rr[32];
        tmem_ld32(lane_base + (uint32_t)(C::TMEM_DQ + half * (D / 2) + c * 32), rr);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 v = make_uint4(pack_bf162(__uint_as_float(rr[8 * u]) * p.scale, __uint_as_float(rr[8 * u + 1]) * p.scale),
                                 pack_bf162(__uint_as_float(rr[8 * u + 2]) * p.scale, __uint_as_float(rr[8 * u + 3]) * p.scale),
                                 pack_bf162(__uint_as_float(rr[8 * u + 4]) * p.scale, __uint_as_float(rr[8 * u + 5]) * p.scale),
                                 pack_bf162(__uint_as_float(rr[8 * u + 6]) * p.scale, __uint_as_float(rr[8 * u + 7]) * p.scale));
            *reinterpret_cast<uint4 *>(dqrow + c * 32 + 8 * u) = v;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ read-out of dV_j^T / dK_j^T: thread = head-dim index
    // Eight warps: TMEM lane quarter w % 4 (= 32 head-dim indices) and 32 of the tile's 64 keys each.  A warp-wide add
    // covers 32 consecutive floats of one key's row in the fp32 accumulators.
    const int quarter = warp & 3;
    const int half = (warp - 10) >> 2;
    const int dcol = quarter * 32 + lane;
    const float inv_keep = p.drop_p > 0.f ? 1.f / (1.f - p.drop_p) : 1.f;
    float *dv_base = p.dV_acc + ((long long)(b * p.H + h) * p.Sk) * D + dcol;
    float *dk_base = p.dK_acc + ((long long)(b * p.H + h) * p.Sk) * D + dcol;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int t = j & 1;
      ok = mbar_wait(&dkv_full[t], (uint32_t)(j >> 1) & 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (warp == 10) attn_trace(p, 20, j);
      tc_fence_after();
      const int k0 = j * BKB + half * 32;
      const int kn = (p.dbg & 1024) ? 0 : min(32, p.Sk - k0);
      uint32_t ra[32], rb[32];
      tmem_ld32(lane_base + (uint32_t)(C::TMEM_DVT + t * 128 + half * 32), ra);
      tmem_ld32(lane_base + (uint32_t)(C::TMEM_DKT + t * 128 + half * 32), rb);
      tmem_ld_wait();
      tc_fence_before();
      warp_arrive(&dkv_empty[t], lane);
      if (warp == 10) attn_trace(p, 21, j);
      float *dvp = dv_base + (long long)k0 * D, *dkp = dk_base + (long long)k0 * D;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < kn) {
          atomicAdd(dvp + i * D, __uint_as_float(ra[i]) * inv_keep);
          atomicAdd(dkp + i * D, __uint_as_float(rb[i]) * p.scale);
        }
      if (warp == 10) attn_trace(p, 22, j);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ host side
// 4-D map {head-dim column, row within the sequence, head, batch} of a [B*S, ld] matrix; box = 64 columns x box_rows rows
int make_head_map(CUtensorMap *map, const void *ptr, int D, int S, long long ld, int H, int B, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)(ld * 2), (cuuint64_t)(D * 2), (cuuint64_t)((long long)S * ld * 2)};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, (void *)ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

__device__ int g_attn_err = 0;

bool aligned16(const void *p, long long ld) { return (((uintptr_t)p) & 15) == 0 && (ld * 2) % 16 == 0; }

}  // namespace

// One attention call.  Plain C struct so ctypes can fill it.
struct FfkAttnDesc {
  int B, H, Sq, Sk, D;
  float scale;
  int causal;
  float drop_p;
  unsigned long long drop_salt;
  const void *drop_seed_ptr;   // device u64 (per-step seed) or null
  const void *Q; long long ldq;
  const void *K; long long ldk;
  const void *V; long long ldv;
  void *O; long long ldo;
  void *lse;                   // [B, H, Sq] float
  // backward
  const void *dO; long long lddo;
  void *delta;                 // [B, H, Sq] float scratch
  void *dQ; long long lddq;
  void *dK; long long lddk;
  void *dV; long long lddv;
  void *acc;                   // 2 * B*H*Sk*D floats of scratch (dK and dV accumulators)
};

// 1 when the fused kernels cover this head dimension / direction
FFK_API int ffk_attention_supported(int D, int backward) { return backward ? (D == 128) : (D == 64 || D == 128); }
FFK_API long long ffk_attention_bwd_scratch_floats(int B, int H, int Sk, int D) { return 2ll * B * H * Sk * D; }

FFK_API int ffk_attention_fwd(const FfkAttnDesc *d, cudaStream_t stream) {
  if (d->D != 64 && d->D != 128) return -2;
  if (d->B <= 0 || d->H <= 0 || d->Sq <= 0 || d->Sk <= 0) return 0;
  if (!aligned16(d->Q, d->ldq) || !aligned16(d->K, d->ldk) || !aligned16(d->V, d->ldv) || !aligned16(d->O, d->ldo)) return -2;
  if (d->causal && d->Sq != d->Sk) return -2;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_head_map(&tq, d->Q, d->D, d->Sq, d->ldq, d->H, d->B, BQ))) return r;
  if ((r = make_head_map(&tk, d->K, d->D, d->Sk, d->ldk, d->H, d->B, BKF))) return r;
  if ((r = make_head_map(&tv, d->V, d->D, d->Sk, d->ldv, d->H, d->B, BKF))) return r;
  AttnArgs a = {};
  a.B = d->B; a.H = d->H; a.Sq = d->Sq; a.Sk = d->Sk; a.scale = d->scale; a.causal = d->causal;
  a.drop_p = d->drop_p; a.drop_salt = d->drop_salt; a.drop_seed_ptr = (const unsigned long long *)d->drop_seed_ptr;
  a.O = (bf16 *)d->O; a.ldo = d->ldo; a.lse = (float *)d->lse;
  void *errp = nullptr;
  cudaGetSymbolAddress(&errp, g_attn_err);
  a.err = (int *)errp;
  { const char *e = getenv("FFK_ATTN_DBG"); a.dbg = e ? atoi(e) : 0; }
  const long long grid = (long long)((d->Sq + BQ - 1) / BQ) * d->H * d->B;
  if (grid > 0x7fffffffll) return -2;
  if (d->D == 128) {
    static bool attr = false;
    if (!attr) {
      cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdCfg<128>::SMEM_BYTES);
      if (e != cudaSuccess) return (int)e;
      attr = true;
    }
    attn_fwd_kernel<128><<<(unsigned)grid, ATT_THREADS, FwdCfg<128>::SMEM_BYTES, stream>>>(tq, tk, tv, a);
  } else {
    static bool attr = false;
    if (!attr) {
      cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdCfg<64>::SMEM_BYTES);
      if (e != cudaSuccess) return (int)e;
      attr = true;
    }
    attn_fwd_kernel<64><<<(unsigned)grid, ATT_THREADS, FwdCfg<64>::SMEM_BYTES, stream>>>(tq, tk, tv, a);
  }
  return (int)cudaGetLastError();
}

FFK_API int ffk_attention_bwd(const FfkAttnDesc *d, cudaStream_t stream) {
  if (d->D != 128) return -2;
  if (d->B <= 0 || d->H <= 0 || d->Sq <= 0 || d->Sk <= 0) return 0;
  if (!aligned16(d->Q, d->ldq) || !aligned16(d->K, d->ldk) || !aligned16(d->V, d->ldv) || !aligned16(d->O, d->ldo) ||
      !aligned16(d->dO, d->lddo) || !aligned16(d->dQ, d->lddq) || !aligned16(d->dK, d->lddk) || !aligned16(d->dV, d->lddv) ||
      (((uintptr_t)d->acc) & 15))
    return -2;
  if (d->causal && d->Sq != d->Sk) return -2;
  constexpr int D = 128;
  CUtensorMap tq, tk, tv, tdo;
  int r;
  if ((r = make_head_map(&tq, d->Q, D, d->Sq, d->ldq, d->H, d->B, BQ))) return r;
  if ((r = make_head_map(&tdo, d->dO, D, d->Sq, d->lddo, d->H, d->B, BQ))) return r;
  if ((r = make_head_map(&tk, d->K, D, d->Sk, d->ldk, d->H, d->B, BKB))) return r;
  if ((r = make_head_map(&tv, d->V, D, d->Sk, d->ldv, d->H, d->B, BKB))) return r;
  const long long n_acc = (long long)d->B * d->H * d->Sk * D;
  cudaError_t e = cudaMemsetAsync(d->acc, 0, (size_t)(2 * n_acc) * sizeof(float), stream);
  if (e != cudaSuccess) return (int)e;
  {
    const long long warps = (long long)d->B * d->Sq * d->H;
    attn_delta_kernel<D><<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>((const bf16 *)d->dO, d->lddo, (const bf16 *)d->O, d->ldo,
                                                                           (float *)d->delta, d->B, d->H, d->Sq);
  }
  AttnArgs a = {};
  a.B = d->B; a.H = d->H; a.Sq = d->Sq; a.Sk = d->Sk; a.scale = d->scale; a.causal = d->causal;
  a.drop_p = d->drop_p; a.drop_salt = d->drop_salt; a.drop_seed_ptr = (const unsigned long long *)d->drop_seed_ptr;
  a.lse = (float *)d->lse; a.delta = (const float *)d->delta;
  a.dQ = (bf16 *)d->dQ; a.lddq = d->lddq;
  a.dK_acc = (float *)d->acc; a.dV_acc = (float *)d->acc + n_acc;
  void *errp = nullptr;
  cudaGetSymbolAddress(&errp, g_attn_err);
  a.err = (int *)errp;
  { const char *e = getenv("FFK_ATTN_DBG"); a.dbg = e ? atoi(e) : 0; }
  static bool attr = false;
  if (!attr) {
    e = cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdCfg::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  const long long grid = (long long)((d->Sq + BQ - 1) / BQ) * d->H * d->B;
  if (grid > 0x7fffffffll) return -2;
  attn_bwd_kernel<<<(unsigned)grid, BWD_THREADS, BwdCfg::SMEM_BYTES, stream>>>(tq, tk, tv, tdo, a);
  const int cblocks = ffk_blocks(n_acc / 4, 256);
  attn_acc_to_bf16_kernel<D><<<cblocks, 256, 0, stream>>>(a.dK_acc, (bf16 *)d->dK, d->lddk, d->B, d->H, d->Sk);
  attn_acc_to_bf16_kernel<D><<<cblocks, 256, 0, stream>>>(a.dV_acc, (bf16 *)d->dV, d->lddv, d->B, d->H, d->Sk);
  return (int)cudaGetLastError();
}

// Copies out the timeline recorded under experiment switch 4096: 32 events x 64 steps of SM clock values (0 = not reached).
// Synchronises the device.
FFK_API int ffk_attention_trace(long long *host_out) {
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  static long long zeros[32 * 64] = {};
  cudaMemcpyFromSymbol(host_out, g_attn_trace, sizeof(long long) * 32 * 64);
  cudaMemcpyToSymbol(g_attn_trace, zeros, sizeof(zeros));
  return 32 * 64;
}

// Reads (and clears) the error word of the attention kernels' bounded waits.  Synchronises the device.
FFK_API int ffk_attention_last_error() {
  int v = 0, z = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  cudaMemcpyFromSymbol(&v, g_attn_err, sizeof(int));
  cudaMemcpyToSymbol(g_attn_err, &z, sizeof(int));
  return v;
}
