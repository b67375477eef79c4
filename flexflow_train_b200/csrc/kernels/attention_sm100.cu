// attention_sm100.cu -- fused multi-head attention core for Blackwell (sm_100a), forward and backward.
//
//   O = dropout(softmax(scale * Q K^T [+ causal mask])) V          per (batch, head)
//
// Replaces the cuDNN multi-head-attention calls of the reference
// (lib/kernels/src/cuda/ops/attention_kernels.cu:224-285: cudnnMultiHeadAttnForward / BackwardData /
// BackwardWeights) for the score / softmax / context part; the projections stay GEMMs.  The [Sq, Sk] score
// matrix never exists in global memory: scores are produced by tcgen05.mma into tensor memory (TMEM), turned into
// probabilities by two threads per query row and multiplied with V by the tensor core again (forward: the bf16
// probabilities go back into tensor memory and are the A operand of the second product from there; backward: through
// shared memory).  Only the row log-sum-exp is kept for backward, which recomputes the scores tile by tile.
//
// Layouts.  Q, K, V, O, dO, dQ, dK, dV are [batch * seq, ld] bf16 matrices in which head h occupies the D
// columns starting at h * D (so the packed output of one QKV projection GEMM is used as it lies); D is 64 or 128.
//
// Dropout is counter based: element (b, h, q, k) is kept when word(seed, row, k / 4) * RC[k % 4] (mod 2^32) is at least
// p * 2^32, row = (b * H + h) * Sq + q (attn_group_word below), so backward regenerates the mask.  The 1 / (1 - p) factor is
// applied once per output row / gradient tile.
//
// Forward CTA (320 threads) = one 128-query block of one (batch, head):
//   warp 0      TMA producer: Q once, then K and V tiles of 128 keys through three-stage rings
//   warp 1      MMA issuer:   S[j % 3] = Q K_j^T, issued two key tiles ahead (TMEM, three buffers), and O += P_j V_j (TMEM)
//   warps 2-9   softmax: thread = query row x half of the tile's keys; the row maximum is exchanged between the two halves,
//               P_j (bf16) overwrites the first 64 columns of S[j % 3]; the exponentials are taken against a reference
//               maximum that only moves when the true maximum has grown by more than 2^8, in which case the thread rescales
//               its half of the row of O in tensor memory; at the end O / sum is written out
//
// Backward CTA (576 threads) = one 128-key block of one (batch, head), walking over the query blocks that see it (see the
// comment at the backward kernel): dK and dV accumulate in tensor memory and are written once; the dQ contributions of the
// key blocks are added into an fp32 accumulator in global memory and converted to bf16 by a last small kernel.
//
// Every mbarrier wait is bounded (tcgen05.cuh); on expiry the CTA records a code in the library's error word,
// frees its TMEM and returns.
#include <cstdlib>

#include "tcgen05.cuh"

namespace {

constexpr int ATT_THREADS = 320;
constexpr int BQ = 128;    // query rows per CTA
constexpr int BKF = 128;   // keys per forward tile
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
  bf16 *dK, *dV;          // [B*Sk, ld] outputs, written once per key block
  long long lddk, lddv;
  float *dQ_acc;          // [B, H, Sq, D] fp32, zeroed by the caller: the key blocks of a head add into it
  int *err;
  int dbg;                // FFK_ATTN_DBG: 4096 records the timeline of one CTA (ffk_attention_trace)
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

// 2^x on the special-function unit, one instruction (exp2f() adds range handling for results below the normal range,
// which a probability does not need: those flush to zero)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void warp_arrive(uint64_t *bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

// Dropout draws of the attention kernels: one 32-bit word per (query row, group of four keys) from two multiply-fold steps,
// then one odd multiplier per key of the group; key j is dropped iff word * ATT_RC[j] (mod 2^32) < p * 2^32.  Sixteen
// instructions per four keys (the generic 64-bit generator of the element-wise kernels costs about forty); the forward and
// the backward kernel and ops/kernels.py::attention_keep_mask (the host restatement the tests use) share this definition.
__device__ __forceinline__ uint32_t attn_row_mix(unsigned long long seed, unsigned long long row) {
  return (uint32_t)seed + (uint32_t)row * 0x9E3779B9u;
}
__device__ __forceinline__ uint32_t attn_group_word(uint32_t row_mix, uint32_t seed_hi, uint32_t group) {
  const uint32_t a = group * 0xB5297A4Du + row_mix;
  const uint64_t m = (uint64_t)a * 0xCC9E2D51u;
  return (uint32_t)m ^ (uint32_t)(m >> 32) ^ seed_hi;
}
constexpr uint32_t ATT_RC0 = 0x9E3779B1u, ATT_RC1 = 0x85EBCA6Bu, ATT_RC2 = 0xC2B2AE35u, ATT_RC3 = 0x27D4EB2Fu;
__device__ __forceinline__ uint32_t attn_drop_threshold(float p) {
  const float t = p * 4294967296.0f;
  return t >= 4294967040.0f ? 0xFFFFFF00u : (uint32_t)t;
}

// Probabilities of one thread's 64 scores when there is no dropout: rs[i] (raw fp32 bits of s_i) becomes the bf16 pair
// (p_2i, p_2i+1) in rs[0..31], p_i = 2^(s_i * sl2 - m), zero from column kmax on; returns the sum of the p_i.  The work goes
// in chunks of 16 scores whose sixteen special-function instructions are issued back to back (volatile keeps them in source
// order).  A warp issues in order: an exponential followed directly by the add that consumes it stalls the warp for the
// unit's latency each time, which held this phase at 0.4 of the unit's rate (0.641 -> 0.573 ms at batch 32 x 16 heads x 1024
// x 128; with dropout, after the mask generator became cheap, 0.604 -> 0.551 ms).  In the backward kernel, which has 96
// registers per thread, the chunked form spills and is slower.
__device__ __forceinline__ float fast_exp2_ordered(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x on the FMA pipe: x = n + f with n = round(x), f in [-0.5, 0.5]; a cubic for 2^f (relative error 8e-5, well below a
// bf16 ulp), then n is added to the exponent field.  Nine instructions against two for the special-function path, used for
// a quarter of the scores so that the two pipes finish together.
__device__ __forceinline__ float poly_exp2(float x) {
  const float MAGIC = 12582912.f;                  // 1.5 * 2^23: adding it rounds x to an integer in the low mantissa bits
  x = fmaxf(x, -126.f);
  const float t = x + MAGIC;
  const float f = x - (t - MAGIC);
  float pz = fmaf(f, 0.05508868396282196f, 0.24260404706001282f);
  pz = fmaf(pz, f, 0.6932762265205383f);
  pz = fmaf(pz, f, 0.9999289512634277f);
  return __uint_as_float(__float_as_uint(pz) + (__float_as_uint(t) << 23));   // the low bits of t hold n; MAGIC's own bits shift out
}
__device__ __forceinline__ float softmax_exp64(uint32_t (&rs)[64], float sl2, float m, bool full, int kmax) {
  float ls0 = 0.f, ls1 = 0.f, ls2 = 0.f, ls3 = 0.f;
  const float neg_m = -m;
#pragma unroll
  for (int c = 0; c < 64; c += 16) {
    float e[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) e[i] = fmaf(__uint_as_float(rs[c + i]), sl2, neg_m);
#pragma unroll
    for (int i = 0; i < 12; ++i) e[i] = fast_exp2_ordered(e[i]);
#pragma unroll
    for (int i = 12; i < 16; ++i) e[i] = poly_exp2(e[i]);
    if (!full) {
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (c + i >= kmax) e[i] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
      ls0 += e[i]; ls1 += e[i + 1]; ls2 += e[i + 2]; ls3 += e[i + 3];
    }
#pragma unroll
    for (int i = 0; i < 16; i += 2) rs[(c + i) >> 1] = pack_bf162(e[i], e[i + 1]);   // registers (c + i) / 2 are already consumed
  }
  return (ls0 + ls1) + (ls2 + ls3);
}

// The same with dropout: the four group words of a chunk are drawn before its exponentials are issued (integer work that
// runs under the special-function unit's latency), the mask is applied after the row sum has taken the undropped values.
__device__ __forceinline__ float softmax_exp64_drop(uint32_t (&rs)[64], float sl2, float m, bool full, int kmax, uint32_t thr, uint32_t row_mix,
                                                    uint32_t seed_hi, int k0) {
  float ls0 = 0.f, ls1 = 0.f, ls2 = 0.f, ls3 = 0.f;
  const float neg_m = -m;
#pragma unroll
  for (int c = 0; c < 64; c += 16) {
    float e[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) e[i] = fmaf(__uint_as_float(rs[c + i]), sl2, neg_m);
    uint32_t z[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) z[g] = attn_group_word(row_mix, seed_hi, (uint32_t)((k0 + c + 4 * g) >> 2));
#pragma unroll
    for (int i = 0; i < 16; ++i) e[i] = fast_exp2_ordered(e[i]);
    if (!full) {
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (c + i >= kmax) e[i] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
      ls0 += e[i]; ls1 += e[i + 1]; ls2 += e[i + 2]; ls3 += e[i + 3];
    }
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (z[g] * ATT_RC0 < thr) e[4 * g] = 0.f;
      if (z[g] * ATT_RC1 < thr) e[4 * g + 1] = 0.f;
      if (z[g] * ATT_RC2 < thr) e[4 * g + 2] = 0.f;
      if (z[g] * ATT_RC3 < thr) e[4 * g + 3] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < 16; i += 2) rs[(c + i) >> 1] = pack_bf162(e[i], e[i + 1]);
  }
  return (ls0 + ls1) + (ls2 + ls3);
}

// ================================================================================================ forward
constexpr float RESCALE_GAP = 8.f;      // log2 units the true row maximum may exceed the one in use
template <int D>
struct FwdCfg {
  static constexpr int PANELS = D / 64;              // 64-column (128-byte) panels per row of Q / K / V
  static constexpr int Q_BYTES = BQ * D * 2;
  static constexpr int KV_BYTES = BKF * D * 2;       // one K or one V tile
  // Three stages each: the score product runs two key tiles ahead of the softmax, a V tile is needed one step after its K tile
  static constexpr int NK = 3, NV = 3;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + NK * KV_BYTES;
  static constexpr int OFF_XCHG = OFF_V + NV * KV_BYTES;     // [2 tile parities][2 column halves][128 rows] floats
  static constexpr int OFF_BAR = OFF_XCHG + 4 * 128 * 4;
  static constexpr int SLACK = D == 128 ? 768 : 1024;        // room to align the base to 1024 bytes (checked in the kernel)
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + SLACK;
  static constexpr int NS = 3;                               // score buffers S[j % 3] at tensor-memory columns (j % 3) * 128;
  static constexpr int TMEM_S = 0;                           // P(j) overwrites the first 64 columns of its own buffer
  static constexpr int TMEM_O = 384;                         // O, D columns
  static_assert(SMEM_BYTES <= 232448, "forward tiles exceed the shared memory of one CTA");
  static constexpr uint32_t IDESC_S = attn_idesc(128, BKF, 0, 0);
  static constexpr uint32_t IDESC_PV = attn_idesc(128, D, 0, 1);
};

// named barrier of the two warps that share a TMEM lane quarter (ids 1..4; 0 is __syncthreads)
__device__ __forceinline__ void pair_sync(int quarter) { asm volatile("bar.sync %0, 64;" ::"r"(quarter + 1) : "memory"); }

template <int D, bool DROP>
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
  uint64_t *k_full = bars + 1;        // [NK]
  uint64_t *k_empty = bars + 5;       // [NK]
  uint64_t *v_full = bars + 19;       // [NV]
  uint64_t *v_empty = bars + 22;      // [NV]
  uint64_t *s_full = bars + 9;        // [NS]
  uint64_t *s_empty = bars + 15;      // [NS] 8 warps
  // The softmax warps may run up to two key tiles apart (the score products are issued two tiles ahead), so the barriers
  // they arrive on or wait for by parity exist once per score buffer: a single one could count an early arrival into the
  // previous phase, or answer a wait for product j - 1 with the completion of product j - 3.
  uint64_t *p_full = bars + 26;       // [NS] 8 warps: P(j) is in tensor memory
  uint64_t *pv_done = bars + 29;      // [NS] commit: P(j) has been read and O holds key tiles 0..j
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
    for (int s = 0; s < C::NK; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < C::NS; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 8); }
    for (int s = 0; s < C::NV; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    for (int s = 0; s < C::NS; ++s) { mbar_init(&p_full[s], 8); mbar_init(&pv_done[s], 1); }
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
      const uint64_t dv0 = make_smem_desc(smem_u32(smem + C::OFF_V), BKF * 128, 1024);
      // S(j) = Q K_j^T into buffer j % 3.  That buffer held S(j - 3) and then P(j - 3): the softmax warps have read the former
      // (s_empty) and the product that reads the latter was issued before this one, and products run in issue order.
      auto issue_s = [&](int j) -> bool {
        const int t = j % C::NS;
        const uint32_t ph = (uint32_t)(j / C::NS) & 1u;
        if (!mbar_wait(&k_full[t], ph, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA)) return false;
        if (!mbar_wait(&s_empty[t], ph ^ 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint64_t dk = desc_advance(dk0, (uint32_t)(t * C::KV_BYTES));
        const uint32_t d_tmem = tmem_base + (uint32_t)(C::TMEM_S + t * 128);
        {
          tc_mma_bf16<false>(d_tmem, dq, dk, C::IDESC_S);
#pragma unroll
          for (int ks = 1; ks < D / 16; ++ks) {
            const uint32_t off = (uint32_t)((ks >> 2) * (BQ * 128) + (ks & 3) * 32);   // panel, then 32 bytes per k-step
            tc_mma_bf16<true>(d_tmem, desc_advance(dq, off), desc_advance(dk, off), C::IDESC_S);
          }
        }
        tc_commit(&s_full[t]);
        tc_commit(&k_empty[t]);
        attn_trace(p, 20, j);
        return true;
      };
      // the score products run two key tiles ahead, so the softmax of tile j + 1 never waits for the tensor core
      if (ok && n_tiles > 0) ok = issue_s(0);
      if (ok && n_tiles > 1) ok = issue_s(1);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 2 < n_tiles) { ok = issue_s(j + 2); if (!ok) break; }
        const int vt = j % C::NV;
        ok = mbar_wait(&v_full[vt], (uint32_t)(j / C::NV) & 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA) &&
             mbar_wait(&p_full[j % C::NS], (uint32_t)(j / C::NS) & 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA);
        if (!ok) break;
        attn_trace(p, 21, j);
        tc_fence_after();
        const uint64_t dv = desc_advance(dv0, (uint32_t)(vt * C::KV_BYTES));
        const uint32_t d_tmem = tmem_base + (uint32_t)C::TMEM_O;
        {
          // O += P V.  A = P (K-major, two panels of 64 keys); B = V (N = head dim contiguous: MN-major, 16 key rows per step)
          // P(j) lies in the first 64 columns of the tensor-memory buffer its scores came from (bf16 pairs, 8 columns per
          // step of 16 keys)
          const uint32_t a_tmem = tmem_base + (uint32_t)(C::TMEM_S + (j % C::NS) * 128);
          if (j == 0) tc_mma_ts_bf16<false>(d_tmem, a_tmem, dv, C::IDESC_PV);
          else tc_mma_ts_bf16<true>(d_tmem, a_tmem, dv, C::IDESC_PV);
#pragma unroll
          for (int ks = 1; ks < BKF / 16; ++ks)
            tc_mma_ts_bf16<true>(d_tmem, a_tmem + (uint32_t)(ks * 8), desc_advance(dv, (uint32_t)(ks * 16 * 128)), C::IDESC_PV);
        }
        tc_commit(&v_empty[vt]);
        tc_commit(&pv_done[j % C::NS]);
        attn_trace(p, 22, j);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax, rescale and read-out of O
    // Eight warps: warp w works on TMEM lane quarter w % 4 (a hardware rule) and on column half (w - 2) / 4, so a thread is
    // one query row and 64 of the tile's 128 keys (and D / 2 of the output columns).  Two warps per scheduler hide each
    // other's TMEM-load and special-function latencies; the row maximum is the only thing the two halves must agree on
    // per tile and goes through a two-float exchange in shared memory.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const int q = q0 + r;
    const float sl2 = p.scale * LOG2E;
    float m = 0.f, l = 0.f;     // m: the maximum the row's exponentials are taken against (see RESCALE_GAP)
    const uint32_t thr = attn_drop_threshold(p.drop_p);
    const unsigned long long seed = DROP ? attn_seed(p) : 0ull;
    const uint32_t seed_hi = (uint32_t)(seed >> 32);
    const uint32_t row_mix = attn_row_mix(seed, (unsigned long long)(b * p.H + h) * p.Sq + (unsigned long long)q);
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t t_o = lane_base + (uint32_t)(C::TMEM_O + half * DH);   // this thread's half of its row of O
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int t = j % C::NS;
      const uint32_t ph = (uint32_t)(j / C::NS) & 1u;
      const int xp = j & 1;              // parity of the exchange slots
      ok = mbar_wait(&s_full[t], ph, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const bool tr = warp == 2;
      if (tr) attn_trace(p, 0, j);
      tc_fence_after();
      const uint32_t t_s = lane_base + (uint32_t)(C::TMEM_S + t * 128 + half * 64);
      uint32_t rs[64];
      tmem_ld32(t_s, *reinterpret_cast<uint32_t(*)[32]>(&rs[0]));
      tmem_ld32(t_s + 32u, *reinterpret_cast<uint32_t(*)[32]>(&rs[32]));
      tmem_ld_wait();
      tc_fence_before();
      warp_arrive(&s_empty[t], lane);
      if (tr) attn_trace(p, 1, j);     // the scores are in registers: the next-but-one tile may overwrite them
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
      xchg[(xp * 2 + half) * 128 + r] = mine;
      pair_sync(quarter);
      const float other = xchg[(xp * 2 + (half ^ 1)) * 128 + r];
      if (tr) attn_trace(p, 2, j);
      // The reference maximum only moves when the true maximum has grown past it by more than RESCALE_GAP (a factor 256,
      // harmless in fp32 / bf16); then this thread rescales its columns of O in tensor memory before it publishes P, so the
      // common step has no correction pass.  Both threads of a row see the same two maxima and take the same decision.
      const float m_row = fmaxf(mine, other) * sl2;
      bool need = false;
      if (j == 0) m = m_row == -INFINITY ? 0.f : m_row;
      else need = m_row > m + RESCALE_GAP;
      if (__any_sync(0xffffffffu, need)) {
        // O is complete up to tile j - 1 once the previous product has finished (the same event that frees the P buffer)
        ok = mbar_wait(&pv_done[(j - 1) % C::NS], (uint32_t)((j - 1) / C::NS) & 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const float alpha = need ? fast_exp2(m - m_row) : 1.f;
#pragma unroll 1
        for (int c = 0; c < DH / 32; ++c) {
          uint32_t ro[32];
          tmem_ld32(t_o + (uint32_t)(c * 32), ro);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * alpha);
          tmem_st32(t_o + (uint32_t)(c * 32), ro);
        }
        tmem_st_wait();
        tc_fence_before();
        l *= alpha;
        if (need) m = m_row;
      }
      const float m_new = m;
      float lsum;
      if constexpr (DROP) lsum = softmax_exp64_drop(rs, sl2, m_new, full, kmax, thr, row_mix, seed_hi, k0);
      else lsum = softmax_exp64(rs, sl2, m_new, full, kmax);
      if (tr) attn_trace(p, 3, j);
      if (tr) attn_trace(p, 4, j);
      // 64 probabilities = 32 columns of bf16 pairs: half 0 writes columns 0-31, half 1 columns 32-63 of this row of S(j)'s
      // buffer.  Those columns held half 0's scores, which are in registers since the exchange above.
      tmem_st32(lane_base + (uint32_t)(C::TMEM_S + t * 128 + half * 32), *reinterpret_cast<uint32_t(*)[32]>(&rs[0]));
      tmem_st_wait();
      tc_fence_before();
      warp_arrive(&p_full[t], lane);
      if (tr) attn_trace(p, 5, j);
      l += lsum;
    }
    if (ok && n_tiles > 0) {     // the last product has finished: O is complete
      ok = mbar_wait(&pv_done[(n_tiles - 1) % C::NS], (uint32_t)((n_tiles - 1) / C::NS) & 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
    }
    if (ok) {
      // row sum over both halves, then out = O / (sum * keep probability); the half-0 thread stores the log-sum-exp
      xchg[half * 128 + r] = l;
      pair_sync(quarter);
      const float lt = l + xchg[(half ^ 1) * 128 + r];
      const float inv_keep = p.drop_p > 0.f ? 1.f / (1.f - p.drop_p) : 1.f;
      const float f = lt > 0.f ? inv_keep / lt : 0.f;
      if (q < p.Sq) {
        if (half == 0 && p.lse) p.lse[((long long)(b * p.H + h)) * p.Sq + q] = lt > 0.f ? m + log2f(lt) : INFINITY;
      }
      bf16 *orow = p.O + ((long long)b * p.Sq + q) * p.ldo + (long long)h * D + half * DH;
#pragma unroll 1
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t ro[32];
        if (n_tiles > 0) {
          tmem_ld32(t_o + (uint32_t)(c * 32), ro);     // warp-wide: rows past the end read too and store nothing
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) ro[i] = 0u;
        }
        if (q < p.Sq) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 v = make_uint4(pack_bf162(__uint_as_float(ro[8 * u]) * f, __uint_as_float(ro[8 * u + 1]) * f),
                                 pack_bf162(__uint_as_float(ro[8 * u + 2]) * f, __uint_as_float(ro[8 * u + 3]) * f),
                                 pack_bf162(__uint_as_float(ro[8 * u + 4]) * f, __uint_as_float(ro[8 * u + 5]) * f),
                                 pack_bf162(__uint_as_float(ro[8 * u + 6]) * f, __uint_as_float(ro[8 * u + 7]) * f));
            *reinterpret_cast<uint4 *>(orow + c * 32 + 8 * u) = v;
          }
        }
      }
      tc_fence_before();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ================================================================================================ forward, two query tiles per CTA
// One CTA = 256 queries of one (batch, head) as two independent 128-row tiles that share every K and V tile brought into
// shared memory (half the L2 -> shared-memory traffic of one tile per CTA, which bounded the one-tile kernel).  The
// output accumulates in tensor memory: O_t += P_t V_j.  The running maximum a row's exponentials are taken against is
// only moved when the true maximum has grown past it by more than 8 (a factor 256, harmless in fp32 / bf16); then the
// row's softmax threads rescale their columns of O_t in tensor memory before they publish P_t, so the common step has no
// correction pass at all.  While one tile's softmax runs, the tensor core works on the other tile.
//   warp 0       TMA: Q (both tiles) once, then K / V tiles through rings
//   warp 1       MMA: S_t = Q_t K_j^T; O_t += P_t V_j
//   warps 2-17   softmax: tile t = (w - 2) / 8; thread = query row x 64 of the 128 keys
// P_TMEM: the probabilities go back into the first 64 columns of S_t (bf16 pairs) and the second product reads its A
// operand from tensor memory; otherwise they go through shared memory.
template <int D, bool P_TMEM>
struct Fwd2Cfg {
  static constexpr int PANELS = D / 64;
  static constexpr int QT_BYTES = 128 * D * 2;
  static constexpr int KV_BYTES = BKF * D * 2;
  static constexpr int P_BYTES = 128 * BKF * 2;
  static constexpr int NK = P_TMEM ? 3 : 2;
  static constexpr int NV = P_TMEM ? 2 : 1;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + 2 * QT_BYTES;
  static constexpr int OFF_V = OFF_K + NK * KV_BYTES;
  static constexpr int OFF_P = OFF_V + NV * KV_BYTES;
  static constexpr int OFF_XCHG = OFF_P + (P_TMEM ? 0 : 2 * P_BYTES);   // [2 tiles][2 halves][128 rows] floats
  static constexpr int OFF_BAR = OFF_XCHG + 2 * 2 * 128 * 4;
  static constexpr int SLACK = 512;                                     // room to align the base (checked in the kernel)
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + SLACK;
  static constexpr int TMEM_S = 0;      // S_t at t * 128
  static constexpr int TMEM_O = 256;    // O_t at 256 + t * D
  static constexpr uint32_t IDESC_S = attn_idesc(128, BKF, 0, 0);
  static constexpr uint32_t IDESC_PV = attn_idesc(128, D, 0, 1);
  static_assert(SMEM_BYTES <= 232448, "forward tiles exceed the shared memory of one CTA");
};

constexpr int FWD2_THREADS = 576;

template <int D, bool P_TMEM>
__global__ void __launch_bounds__(FWD2_THREADS, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnArgs p) {
  using C = Fwd2Cfg<D, P_TMEM>;
  constexpr int DH = D / 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float *xchg = (float *)(smem + C::OFF_XCHG);
  uint64_t *bars = (uint64_t *)(smem + C::OFF_BAR);
  uint64_t *q_full = bars;
  uint64_t *k_full = bars + 1;        // [NK]
  uint64_t *k_empty = bars + 4;       // [NK] commit
  uint64_t *v_full = bars + 7;        // [NV]
  uint64_t *v_empty = bars + 9;       // [NV] commit
  uint64_t *s_full = bars + 11;       // [2] commit
  uint64_t *p_full = bars + 13;       // [2] 8 warps
  uint64_t *pv_done = bars + 15;      // [2] commit
  uint32_t *tmem_slot = (uint32_t *)(bars + 17);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
  if ((uintptr_t)(smem - smem_raw) > (uintptr_t)C::SLACK) {
    if (threadIdx.x == 0 && p.err) atomicCAS(p.err, 0, (int)FFK_ERR_BAD_ARG);
    return;
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.Sq + 255) / 256;
  const int qb = blockIdx.x % nqb;
  const int bh = blockIdx.x / nqb;
  const int h = bh % p.H, b = bh / p.H;
  const int q0 = qb * 256;
  // key tiles each query tile needs: all of them, or under the causal mask those with a key <= the tile's last query
  int n_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int first = q0 + t * 128;
    int n = first < p.Sq ? (p.Sk + BKF - 1) / BKF : 0;
    if (p.causal && n > 0) n = min(n, (min(first + 128, p.Sq) - 1) / BKF + 1);
    n_t[t] = n;
  }
  const int n_tiles = max(n_t[0], n_t[1]);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < C::NK; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < C::NV; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    for (int t = 0; t < 2; ++t) { mbar_init(&s_full[t], 1); mbar_init(&p_full[t], 8); mbar_init(&pv_done[t], 1); }
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
      mbar_expect_tx(q_full, 2 * C::QT_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int c = 0; c < C::PANELS; ++c)
          tma_load_4d(smem_u32(smem + C::OFF_Q + t * C::QT_BYTES + c * 128 * 128), &tmQ, q_full, c * 64, q0 + t * 128, h, b);
      int kj = 0, vj = 0;
      uint64_t t0 = ffk_globaltimer();
      uint32_t spins = 0;
      while (kj < n_tiles || vj < n_tiles) {
        bool progress = false;
        if (kj < n_tiles) {
          const int s = kj % C::NK;
          if (mbar_try_wait(&k_empty[s], ((uint32_t)(kj / C::NK) & 1u) ^ 1u)) {
            mbar_expect_tx(&k_full[s], C::KV_BYTES);
#pragma unroll
            for (int c = 0; c < C::PANELS; ++c)
              tma_load_4d(smem_u32(smem + C::OFF_K + s * C::KV_BYTES + c * BKF * 128), &tmK, &k_full[s], c * 64, kj * BKF, h, b);
            ++kj;
            progress = true;
          }
        }
        if (vj < n_tiles) {
          const int s = vj % C::NV;
          if (mbar_try_wait(&v_empty[s], ((uint32_t)(vj / C::NV) & 1u) ^ 1u)) {
            mbar_expect_tx(&v_full[s], C::KV_BYTES);
#pragma unroll
            for (int c = 0; c < C::PANELS; ++c)
              tma_load_4d(smem_u32(smem + C::OFF_V + s * C::KV_BYTES + c * BKF * 128), &tmV, &v_full[s], c * 64, vj * BKF, h, b);
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
      const uint64_t dq0 = make_smem_desc(smem_u32(smem + C::OFF_Q), 16, 1024);
      const uint64_t dk0 = make_smem_desc(smem_u32(smem + C::OFF_K), 16, 1024);
      const uint64_t dv0 = make_smem_desc(smem_u32(smem + C::OFF_V), BKF * 128, 1024);
      const uint64_t dp0 = make_smem_desc(smem_u32(smem + C::OFF_P), 16, 1024);
      auto issue_s = [&](int t, int j) {        // S_t = Q_t K_j^T (the caller has waited for K_j)
        const uint64_t dq = desc_advance(dq0, (uint32_t)(t * C::QT_BYTES));
        const uint64_t dk = desc_advance(dk0, (uint32_t)((j % C::NK) * C::KV_BYTES));
        const uint32_t d = tmem_base + (uint32_t)(C::TMEM_S + t * 128);
        tc_mma_bf16<false>(d, dq, dk, C::IDESC_S);
#pragma unroll
        for (int ks = 1; ks < D / 16; ++ks) {
          const uint32_t off = (uint32_t)((ks >> 2) * (128 * 128) + (ks & 3) * 32);
          tc_mma_bf16<true>(d, desc_advance(dq, off), desc_advance(dk, off), C::IDESC_S);
        }
        tc_commit(&s_full[t]);
      };
      if (ok && n_tiles > 0) {
        ok = mbar_wait(&k_full[0], 0, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA);
        if (ok) {
          tc_fence_after();
          for (int t = 0; t < 2; ++t)
            if (n_t[t] > 0) issue_s(t, 0);
          tc_commit(&k_empty[0]);
        }
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const uint32_t ph = (uint32_t)j & 1u;
        const int vs = j % C::NV;
        ok = mbar_wait(&v_full[vs], (uint32_t)(j / C::NV) & 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA);
        if (!ok) break;
        const uint64_t dv = desc_advance(dv0, (uint32_t)(vs * C::KV_BYTES));
        bool k_ready = false;
        for (int t = 0; t < 2 && ok; ++t) {
          if (j < n_t[t]) {
            attn_trace(p, 20 + 4 * t, j);
            ok = mbar_wait(&p_full[t], ph, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA);
            if (!ok) break;
            attn_trace(p, 21 + 4 * t, j);
            tc_fence_after();
            const uint32_t d = tmem_base + (uint32_t)(C::TMEM_O + t * D);
            if constexpr (P_TMEM) {
              const uint32_t a = tmem_base + (uint32_t)(C::TMEM_S + t * 128);
              if (j == 0) tc_mma_ts_bf16<false>(d, a, dv, C::IDESC_PV);
              else tc_mma_ts_bf16<true>(d, a, dv, C::IDESC_PV);
#pragma unroll
              for (int ks = 1; ks < BKF / 16; ++ks) tc_mma_ts_bf16<true>(d, a + (uint32_t)(ks * 8), desc_advance(dv, (uint32_t)(ks * 2048)), C::IDESC_PV);
            } else {
              const uint64_t dp = desc_advance(dp0, (uint32_t)(t * C::P_BYTES));
              if (j == 0) tc_mma_bf16<false>(d, dp, dv, C::IDESC_PV);
              else tc_mma_bf16<true>(d, dp, dv, C::IDESC_PV);
#pragma unroll
              for (int ks = 1; ks < BKF / 16; ++ks) {
                const uint32_t a_off = (uint32_t)((ks >> 2) * (128 * 128) + (ks & 3) * 32);
                tc_mma_bf16<true>(d, desc_advance(dp, a_off), desc_advance(dv, (uint32_t)(ks * 2048)), C::IDESC_PV);
              }
            }
            tc_commit(&pv_done[t]);
            attn_trace(p, 22 + 4 * t, j);
          }
          if (j + 1 < n_t[t]) {
            if (!k_ready) {
              ok = mbar_wait(&k_full[(j + 1) % C::NK], (uint32_t)((j + 1) / C::NK) & 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA);
              if (!ok) break;
              tc_fence_after();
              k_ready = true;
            }
            issue_s(t, j + 1);
            attn_trace(p, 23 + 4 * t, j);
          }
        }
        if (!ok) break;
        tc_commit(&v_empty[vs]);
        if (j + 1 < n_tiles) tc_commit(&k_empty[(j + 1) % C::NK]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax: tile t, thread = query row x 64 keys
    const int t = (warp - 2) >> 3;
    const int quarter = warp & 3;
    const int half = ((warp - 2) >> 2) & 1;
    const int r = quarter * 32 + lane;
    const int q = q0 + t * 128 + r;
    const int n_mine = n_t[t];
    const float sl2 = p.scale * LOG2E;
    const bool drop = p.drop_p > 0.f;
    const uint32_t thr = attn_drop_threshold(p.drop_p);
    const unsigned long long seed = drop ? attn_seed(p) : 0ull;
    const uint32_t seed_hi = (uint32_t)(seed >> 32);
    const uint32_t row_mix = attn_row_mix(seed, (unsigned long long)(b * p.H + h) * p.Sq + (unsigned long long)q);
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t t_s = lane_base + (uint32_t)(C::TMEM_S + t * 128);
    const uint32_t t_o = lane_base + (uint32_t)(C::TMEM_O + t * D + half * DH);
    const uint32_t prow = smem_u32(smem + C::OFF_P + t * C::P_BYTES + half * (128 * 128) + r * 128);
    float *my_x = xchg + (t * 2 + half) * 128 + r, *other_x = xchg + (t * 2 + (half ^ 1)) * 128 + r;
    const int pair_bar = 1 + t * 4 + quarter;     // named barrier of the two warps that share these 32 rows
    float m_ref = 0.f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_mine && ok; ++j) {
      const uint32_t ph = (uint32_t)j & 1u;
      const bool tr = warp == 2 || warp == 10;
      const int te = t * 6;
      ok = mbar_wait(&s_full[t], ph, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (tr) attn_trace(p, te + 0, j);
      tc_fence_after();
      uint32_t rs[64];
      tmem_ld32(t_s + (uint32_t)(half * 64), *reinterpret_cast<uint32_t(*)[32]>(&rs[0]));
      tmem_ld32(t_s + (uint32_t)(half * 64 + 32), *reinterpret_cast<uint32_t(*)[32]>(&rs[32]));
      tmem_ld_wait();
      if (tr) attn_trace(p, te + 1, j);
      const int k0 = j * BKF + half * 64;
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
      *my_x = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");   // both halves hold their scores in registers from here on
      if (tr) attn_trace(p, te + 2, j);
      const float m_row = fmaxf(*my_x, *other_x) * sl2;
      bool need = false;
      if (j == 0) m_ref = m_row == -INFINITY ? 0.f : m_row;
      else need = m_row > m_ref + RESCALE_GAP;
      const bool any = __any_sync(0xffffffffu, need);
      bool waited = false;
      if (any) {
        // O_t (complete up to tile j - 1) and the row sum move to the new reference maximum
        ok = mbar_wait(&pv_done[t], ph ^ 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        waited = true;
        tc_fence_after();
        const float alpha = need ? fast_exp2(m_ref - m_row) : 1.f;
#pragma unroll 1
        for (int c = 0; c < DH / 32; ++c) {
          uint32_t ro[32];
          tmem_ld32(t_o + (uint32_t)(c * 32), ro);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * alpha);
          tmem_st32(t_o + (uint32_t)(c * 32), ro);
        }
        tmem_st_wait();
        l *= alpha;
        if (need) m_ref = m_row;
      }
      float ls0 = 0.f, ls1 = 0.f, ls2 = 0.f, ls3 = 0.f;
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
        float e0 = fast_exp2(fmaf(__uint_as_float(rs[i]), sl2, -m_ref)), e1 = fast_exp2(fmaf(__uint_as_float(rs[i + 1]), sl2, -m_ref));
        float e2 = fast_exp2(fmaf(__uint_as_float(rs[i + 2]), sl2, -m_ref)), e3 = fast_exp2(fmaf(__uint_as_float(rs[i + 3]), sl2, -m_ref));
        if (!full) {
          if (i >= kmax) e0 = 0.f;
          if (i + 1 >= kmax) e1 = 0.f;
          if (i + 2 >= kmax) e2 = 0.f;
          if (i + 3 >= kmax) e3 = 0.f;
        }
        ls0 += e0; ls1 += e1; ls2 += e2; ls3 += e3;
        if (drop) {
          const uint32_t z = attn_group_word(row_mix, seed_hi, (uint32_t)((k0 + i) >> 2));
          if (z * ATT_RC0 < thr) e0 = 0.f;
          if (z * ATT_RC1 < thr) e1 = 0.f;
          if (z * ATT_RC2 < thr) e2 = 0.f;
          if (z * ATT_RC3 < thr) e3 = 0.f;
        }
        rs[i >> 1] = pack_bf162(e0, e1);          // packed in place (registers i / 2, i / 2 + 1 are already consumed)
        rs[(i >> 1) + 1] = pack_bf162(e2, e3);
      }
      l += (ls0 + ls1) + (ls2 + ls3);
      if (tr) attn_trace(p, te + 3, j);
      if constexpr (P_TMEM) {
        // 64 probabilities = 32 columns of bf16 pairs at the start of S_t (this half's own scores or the other half's,
        // all of which are in registers since the barrier above)
        tmem_st32(t_s + (uint32_t)(half * 32), *reinterpret_cast<uint32_t(*)[32]>(&rs[0]));
        tmem_st_wait();
        tc_fence_before();
      } else {
        if (j > 0 && !waited) {   // the previous product has finished reading this tile's P buffer
          ok = mbar_wait(&pv_done[t], ph ^ 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + (uint32_t)((u ^ (r & 7)) << 4)), "r"(rs[4 * u]), "r"(rs[4 * u + 1]),
                       "r"(rs[4 * u + 2]), "r"(rs[4 * u + 3])
                       : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        tc_fence_before();   // orders the tensor-memory traffic of a rescale before the arrival
      }
      warp_arrive(&p_full[t], lane);
      if (tr) attn_trace(p, te + 4, j);
    }
    if (ok && n_mine > 0) {
      ok = mbar_wait(&pv_done[t], (uint32_t)(n_mine - 1) & 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && n_mine > 0) {
      tc_fence_after();
      *my_x = l;
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      const float lt = l + *other_x;
      const float inv_keep = drop ? 1.f / (1.f - p.drop_p) : 1.f;
      const float f = lt > 0.f ? inv_keep / lt : 0.f;
      if (q < p.Sq && half == 0 && p.lse) p.lse[((long long)(b * p.H + h)) * p.Sq + q] = lt > 0.f ? m_ref + log2f(lt) : INFINITY;
      bf16 *orow = p.O + ((long long)b * p.Sq + q) * p.ldo + (long long)h * D + half * DH;
#pragma unroll 1
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t ro[32];
        tmem_ld32(t_o + (uint32_t)(c * 32), ro);
        tmem_ld_wait();
        if (q < p.Sq) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 v = make_uint4(pack_bf162(__uint_as_float(ro[8 * u]) * f, __uint_as_float(ro[8 * u + 1]) * f),
                                 pack_bf162(__uint_as_float(ro[8 * u + 2]) * f, __uint_as_float(ro[8 * u + 3]) * f),
                                 pack_bf162(__uint_as_float(ro[8 * u + 4]) * f, __uint_as_float(ro[8 * u + 5]) * f),
                                 pack_bf162(__uint_as_float(ro[8 * u + 6]) * f, __uint_as_float(ro[8 * u + 7]) * f));
            *reinterpret_cast<uint4 *>(orow + c * 32 + 8 * u) = v;
          }
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

// Backward main kernel.  One CTA owns a block of 128 keys of one (batch, head) and walks over the blocks of 128 queries
// that can see it.  K and V stay in shared memory; dK and dV accumulate in tensor memory for the whole walk and are
// written once, as bf16, at the end.  Per query block i:
//   S = Q_i K^T, dP = dO_i V^T                      (tensor memory; S and dP one stage each)
//   P = exp2(S * scale * log2 e - lse), dS = P o (dP o keep / keep_prob - delta)   (eight warps, thread = query row x 64 keys)
//   dV += P^T dO_i, dK += dS^T Q_i                  (A operand = P / dS in shared memory read M-major)
//   dQ_i^T = K^T dS^T                               (into the columns dP just left; eight warps add it to the fp32 dQ
//                                                    accumulator in global memory: lanes = head-dim index, so one warp-wide
//                                                    add covers 128 contiguous bytes of one query's row)
// The tensor core sees the five products of a step in the order dV, dQ^T, dK, S(next), dP(next): the read-out of dQ^T
// overlaps the dK and S products, and the next step's softmax overlaps the dP product.
template <int D_>
struct BwdCfg {
  static constexpr int D = D_;                            // head dim: 128, or 64 (then dQ is produced untransposed, see the kernel)
  static constexpr int BK = 128;                          // keys per CTA
  static constexpr int PANEL = 128 * 128;                 // bytes of one 64-column panel: [128 rows x 128 B]
  static constexpr int TILE_BYTES = 128 * D * 2;          // a [128 x D] bf16 tile = D / 64 panels
  static constexpr int PS_BYTES = 128 * 128 * 2;          // P or dS: [128 queries x 128 keys] = two panels
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + TILE_BYTES;
  static constexpr int OFF_Q = OFF_V + TILE_BYTES;        // [2]
  static constexpr int OFF_DO = OFF_Q + 2 * TILE_BYTES;   // one stage: free again after the step's second product
  static constexpr int OFF_P = OFF_DO + TILE_BYTES;
  static constexpr int OFF_DS = OFF_P + PS_BYTES;
  static constexpr int OFF_BAR = OFF_DS + PS_BYTES;       // 224 KB of tiles at head dim 128
  static constexpr int SLACK = 1024;                      // room to align the base to 1024 bytes (checked in the kernel)
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + SLACK;
  static constexpr int TMEM_S = 0;
  static constexpr int TMEM_DPQ = 128;                    // dP, then dQ^T of the same step
  static constexpr int TMEM_DK = 256;                     // D columns
  static constexpr int TMEM_DV = 256 + D;
  static constexpr uint32_t IDESC_SS = attn_idesc(128, 128, 0, 0);    // Q K^T, dO V^T
  static constexpr uint32_t IDESC_T = attn_idesc(128, D, 1, 1);       // P^T dO, dS^T Q
  static constexpr uint32_t IDESC_DQT = attn_idesc(128, 128, 1, 0);   // K^T dS^T (head dim 128)
  static constexpr uint32_t IDESC_DQ = attn_idesc(128, D, 0, 1);      // dS K (head dim 64)
  static_assert(SMEM_BYTES <= 232448, "backward tiles exceed the shared memory of one CTA");
};

constexpr int BWD_THREADS = 576;  // TMA warp, MMA warp, 8 softmax / dS warps, 8 dQ read-out warps

template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const AttnArgs p) {
  using C = BwdCfg<D>;
  constexpr int PANELS = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t *bars = (uint64_t *)(smem + C::OFF_BAR);
  uint64_t *kv_full = bars;
  uint64_t *q_full = bars + 1;        // [2]
  uint64_t *q_empty = bars + 3;       // [2] commit
  uint64_t *do_full = bars + 5;
  uint64_t *do_empty = bars + 6;      // commit
  uint64_t *s_full = bars + 7;        // commit
  uint64_t *s_empty = bars + 8;       // 8 warps
  uint64_t *dp_full = bars + 9;       // commit
  uint64_t *p_full = bars + 10;       // 8 warps
  uint64_t *p_empty = bars + 11;      // commit
  uint64_t *ds_full = bars + 12;      // 8 warps
  uint64_t *ds_empty = bars + 13;     // commit
  uint64_t *dq_full = bars + 14;      // commit
  uint64_t *dq_empty = bars + 15;     // 8 warps
  uint64_t *dkv_full = bars + 16;     // commit
  uint32_t *tmem_slot = (uint32_t *)(bars + 17);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
  if ((uintptr_t)(smem - smem_raw) > (uintptr_t)C::SLACK) {  // the launch did not leave room to align the tiles: refuse
    if (threadIdx.x == 0 && p.err) atomicCAS(p.err, 0, (int)FFK_ERR_BAD_ARG);
    return;
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = (p.Sk + C::BK - 1) / C::BK;
  const int kb = blockIdx.x % nkb;
  const int bh = blockIdx.x / nkb;
  const int h = bh % p.H, b = bh / p.H;
  const int k0 = kb * C::BK;
  const int nqb = (p.Sq + BQ - 1) / BQ;
  const int i0 = p.causal ? k0 / BQ : 0;     // first query block with a row that sees a key of this block (Sq == Sk)
  const int n_it = nqb - i0;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
    mbar_init(do_full, 1); mbar_init(do_empty, 1);
    mbar_init(s_full, 1); mbar_init(s_empty, 8); mbar_init(dp_full, 1);
    mbar_init(p_full, 8); mbar_init(p_empty, 1); mbar_init(ds_full, 8); mbar_init(ds_empty, 1);
    mbar_init(dq_full, 1); mbar_init(dq_empty, 8); mbar_init(dkv_full, 1);
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
      mbar_expect_tx(kv_full, 2 * C::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < PANELS; ++c) {
        tma_load_4d(smem_u32(smem + C::OFF_K + c * C::PANEL), &tmK, kv_full, c * 64, k0, h, b);
        tma_load_4d(smem_u32(smem + C::OFF_V + c * C::PANEL), &tmV, kv_full, c * 64, k0, h, b);
      }
      // the Q ring (two stages) and the dO stage advance independently; the wait for progress on either is bounded
      int qi = 0, di = 0;
      uint64_t t0 = ffk_globaltimer();
      uint32_t spins = 0;
      while (qi < n_it || di < n_it) {
        bool progress = false;
        if (qi < n_it) {
          const int s = qi & 1;
          if (mbar_try_wait(&q_empty[s], ((uint32_t)(qi >> 1) & 1u) ^ 1u)) {
            mbar_expect_tx(&q_full[s], C::TILE_BYTES);
#pragma unroll
            for (int c = 0; c < PANELS; ++c)
              tma_load_4d(smem_u32(smem + C::OFF_Q + s * C::TILE_BYTES + c * C::PANEL), &tmQ, &q_full[s], c * 64, (i0 + qi) * BQ, h, b);
            ++qi;
            progress = true;
          }
        }
        if (di < n_it) {
          if (mbar_try_wait(do_empty, ((uint32_t)di & 1u) ^ 1u)) {
            mbar_expect_tx(do_full, C::TILE_BYTES);
#pragma unroll
            for (int c = 0; c < PANELS; ++c) tma_load_4d(smem_u32(smem + C::OFF_DO + c * C::PANEL), &tmDO, do_full, c * 64, (i0 + di) * BQ, h, b);
            ++di;
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
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA);
      // descriptors are built once; "K-major" = the reduction runs along a row (16 / 1024), "M-major" or "N-major" = the
      // reduction runs down the rows of the two 64-column panels (panel stride / 1024, 2048 bytes per step of 16 rows)
      const uint64_t dK_kmaj = make_smem_desc(smem_u32(smem + C::OFF_K), 16, 1024);
      const uint64_t dK_mmaj = make_smem_desc(smem_u32(smem + C::OFF_K), C::PANEL, 1024);
      const uint64_t dV_kmaj = make_smem_desc(smem_u32(smem + C::OFF_V), 16, 1024);
      const uint64_t dQ_kmaj0 = make_smem_desc(smem_u32(smem + C::OFF_Q), 16, 1024);
      const uint64_t dQ_nmaj0 = make_smem_desc(smem_u32(smem + C::OFF_Q), C::PANEL, 1024);
      const uint64_t dDO_kmaj = make_smem_desc(smem_u32(smem + C::OFF_DO), 16, 1024);
      const uint64_t dDO_nmaj = make_smem_desc(smem_u32(smem + C::OFF_DO), C::PANEL, 1024);
      const uint64_t dP_mmaj = make_smem_desc(smem_u32(smem + C::OFF_P), C::PANEL, 1024);
      const uint64_t dDS_mmaj = make_smem_desc(smem_u32(smem + C::OFF_DS), C::PANEL, 1024);
      const uint64_t dDS_kmaj = make_smem_desc(smem_u32(smem + C::OFF_DS), 16, 1024);
      // byte offset of k-step ks inside a K-major tile: 64-column panel, then 32 bytes per step
      auto koff = [](int ks) -> uint32_t { return (uint32_t)((ks >> 2) * C::PANEL + (ks & 3) * 32); };
      // S = Q_it K^T.  `try_only`: issue only if the Q tile has arrived and the previous scores have been read, without waiting.
      auto issue_s = [&](int it, bool try_only) -> int {      // 1 issued, 0 not yet (try_only), -1 a wait ran out
        const int s = it & 1;
        if (try_only) {
          if (!mbar_try_wait(&q_full[s], (uint32_t)(it >> 1) & 1u) || !mbar_try_wait(s_empty, ((uint32_t)it & 1u) ^ 1u)) return 0;
        } else {
          if (!mbar_wait(&q_full[s], (uint32_t)(it >> 1) & 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA)) return -1;
          if (!mbar_wait(s_empty, ((uint32_t)it & 1u) ^ 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA)) return -1;
        }
        tc_fence_after();
        const uint64_t a = desc_advance(dQ_kmaj0, (uint32_t)(s * C::TILE_BYTES));
        const uint32_t d = tmem_base + (uint32_t)C::TMEM_S;
        tc_mma_bf16<false>(d, a, dK_kmaj, C::IDESC_SS);
#pragma unroll
        for (int ks = 1; ks < D / 16; ++ks) tc_mma_bf16<true>(d, desc_advance(a, koff(ks)), desc_advance(dK_kmaj, koff(ks)), C::IDESC_SS);
        tc_commit(s_full);
        attn_trace(p, 23, it);
        return 1;
      };
      // Waits for `bar` like mbar_wait; while it waits, the next step's S is issued as soon as it can be (pending_s is then
      // cleared): the probability warps can work on step it + 1 while the tensor core still runs the products of step it.
      bool pending_s = false;
      int next_it = 0;
      auto wait_issuing_s = [&](uint64_t *bar, uint32_t parity) -> bool {
        uint64_t t0 = ffk_globaltimer();
        uint32_t spins = 0;
        while (true) {
          if (pending_s) {
            const int r = issue_s(next_it, true);
            if (r > 0) pending_s = false;
          }
          if (mbar_try_wait(bar, parity)) return true;
          if ((++spins & 63u) == 0) {
            if (*abort_flag) return false;
            if (ffk_globaltimer() - t0 > WAIT_LIMIT_NS) {
              *abort_flag = 1;
              if (p.err) atomicCAS(p.err, 0, (int)FFK_ERR_TIMEOUT_MMA);
              return false;
            }
          }
        }
      };
      auto issue_dp = [&](int it) -> bool {     // dP = dO_it V^T, into the columns the previous step's dQ^T has left
        if (!mbar_wait(do_full, (uint32_t)it & 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA)) return false;
        if (!mbar_wait(dq_empty, ((uint32_t)it & 1u) ^ 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint32_t d = tmem_base + (uint32_t)C::TMEM_DPQ;
        tc_mma_bf16<false>(d, dDO_kmaj, dV_kmaj, C::IDESC_SS);
#pragma unroll
        for (int ks = 1; ks < D / 16; ++ks) tc_mma_bf16<true>(d, desc_advance(dDO_kmaj, koff(ks)), desc_advance(dV_kmaj, koff(ks)), C::IDESC_SS);
        tc_commit(dp_full);
        attn_trace(p, 24, it);
        return true;
      };
      if (ok && n_it > 0) ok = issue_s(0, false) > 0 && issue_dp(0);
      for (int it = 0; it < n_it && ok; ++it) {
        const uint32_t ph = (uint32_t)it & 1u;
        pending_s = it + 1 < n_it;
        next_it = it + 1;
        // dV += P^T dO_it
        ok = wait_issuing_s(p_full, ph);
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t d = tmem_base + (uint32_t)C::TMEM_DV;
          if (it == 0) tc_mma_bf16<false>(d, dP_mmaj, dDO_nmaj, C::IDESC_T);
          else tc_mma_bf16<true>(d, dP_mmaj, dDO_nmaj, C::IDESC_T);
#pragma unroll
          for (int ks = 1; ks < BQ / 16; ++ks) tc_mma_bf16<true>(d, desc_advance(dP_mmaj, ks * 2048u), desc_advance(dDO_nmaj, ks * 2048u), C::IDESC_T);
        }
        tc_commit(p_empty);
        tc_commit(do_empty);
        attn_trace(p, 20, it);
        // dQ_it^T = K^T dS^T (the dS warps have read dP out of these columns before they wrote dS)
        ok = wait_issuing_s(ds_full, ph);
        if (!ok) break;
        attn_trace(p, 21, it);
        tc_fence_after();
        {
          const uint32_t d = tmem_base + (uint32_t)C::TMEM_DPQ;
          if constexpr (D == 128) {   // transposed: lanes = head-dim index
            tc_mma_bf16<false>(d, dK_mmaj, dDS_kmaj, C::IDESC_DQT);
#pragma unroll
            for (int ks = 1; ks < C::BK / 16; ++ks)
              tc_mma_bf16<true>(d, desc_advance(dK_mmaj, ks * 2048u), desc_advance(dDS_kmaj, koff(ks)), C::IDESC_DQT);
          } else {                    // dQ_it = dS K: lanes = query rows, 64 columns (a 64-row product would not fill the tensor core)
            tc_mma_bf16<false>(d, dDS_kmaj, dK_mmaj, C::IDESC_DQ);
#pragma unroll
            for (int ks = 1; ks < C::BK / 16; ++ks)
              tc_mma_bf16<true>(d, desc_advance(dDS_kmaj, koff(ks)), desc_advance(dK_mmaj, ks * 2048u), C::IDESC_DQ);
          }
        }
        tc_commit(dq_full);
        // dK += dS^T Q_it
        {
          const uint32_t d = tmem_base + (uint32_t)C::TMEM_DK;
          const uint64_t bq = desc_advance(dQ_nmaj0, (uint32_t)((it & 1) * C::TILE_BYTES));
          if (it == 0) tc_mma_bf16<false>(d, dDS_mmaj, bq, C::IDESC_T);
          else tc_mma_bf16<true>(d, dDS_mmaj, bq, C::IDESC_T);
#pragma unroll
          for (int ks = 1; ks < BQ / 16; ++ks) tc_mma_bf16<true>(d, desc_advance(dDS_mmaj, ks * 2048u), desc_advance(bq, ks * 2048u), C::IDESC_T);
        }
        tc_commit(ds_empty);
        tc_commit(&q_empty[it & 1]);
        attn_trace(p, 22, it);
        if (it + 1 < n_it) ok = (!pending_s || issue_s(it + 1, false) > 0) && issue_dp(it + 1);
      }
      if (ok) tc_commit(dkv_full);
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------------ P and dS: thread = query row x 64 of the block's 128 keys
    // Eight warps, two per TMEM lane quarter (w % 4), each on one half of the key columns.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const float sl2 = p.scale * LOG2E;
    const bool drop = p.drop_p > 0.f;
    const float inv_keep = drop ? 1.f / (1.f - p.drop_p) : 1.f;
    const uint32_t thr = attn_drop_threshold(p.drop_p);
    const unsigned long long seed = drop ? attn_seed(p) : 0ull;
    const uint32_t seed_hi = (uint32_t)(seed >> 32);
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t prow = smem_u32(smem + C::OFF_P + half * C::PANEL + r * 128);     // this row in this half's 64-key panel
    const uint32_t dsrow = smem_u32(smem + C::OFF_DS + half * C::PANEL + r * 128);
    const int kbase = k0 + half * 64;
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const uint32_t ph = (uint32_t)it & 1u;
      const int q = (i0 + it) * BQ + r;
      const bool row_ok = q < p.Sq;
      const long long stat = ((long long)(b * p.H + h)) * p.Sq + q;
      const float lse = row_ok ? p.lse[stat] : INFINITY;
      const float dlt = row_ok ? p.delta[stat] : 0.f;
      const uint32_t row_mix = attn_row_mix(seed, (unsigned long long)(b * p.H + h) * p.Sq + (unsigned long long)q);
      int kmax = p.Sk - kbase;
      if (p.causal) kmax = min(kmax, q - kbase + 1);
      const bool full = kmax >= 64;     // every key of this half exists and is visible to this row
      ok = mbar_wait(s_full, ph, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE) &&
           mbar_wait(p_empty, ph ^ 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (warp == 2) attn_trace(p, 0, it);
      tc_fence_after();
      uint32_t pe[32];          // the row's 64 probabilities before dropout, packed bf16 (dS needs them again)
      uint32_t dropped[2] = {0u, 0u};
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rs[32];
        tmem_ld32(lane_base + (uint32_t)(C::TMEM_S + half * 64 + c * 32), rs);
        tmem_ld_wait();
        if (c == 1) {           // the scores are in registers: the next step's S may overwrite them
          tc_fence_before();
          warp_arrive(s_empty, lane);
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          float e[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            e[u] = fast_exp2(fmaf(__uint_as_float(rs[i + u]), sl2, -lse));
            if (!full && c * 32 + i + u >= kmax) e[u] = 0.f;
          }
          pe[c * 16 + (i >> 1)] = pack_bf162(e[0], e[1]);
          pe[c * 16 + (i >> 1) + 1] = pack_bf162(e[2], e[3]);
          if (drop) {
            const uint32_t z = attn_group_word(row_mix, seed_hi, (uint32_t)((kbase + c * 32 + i) >> 2));
            const uint32_t m = (z * ATT_RC0 < thr ? 1u : 0u) | (z * ATT_RC1 < thr ? 2u : 0u) | (z * ATT_RC2 < thr ? 4u : 0u) |
                               (z * ATT_RC3 < thr ? 8u : 0u);
            dropped[c] |= m << i;
            if (m & 1u) e[0] = 0.f;
            if (m & 2u) e[1] = 0.f;
            if (m & 4u) e[2] = 0.f;
            if (m & 8u) e[3] = 0.f;
          }
          pk[i >> 1] = pack_bf162(e[0], e[1]);
          pk[(i >> 1) + 1] = pack_bf162(e[2], e[3]);
        }
        // 32 probabilities = 64 bytes = four 16-byte chunks; chunk index XOR (row % 8) is the 128-byte swizzle
#pragma unroll
        for (int u = 0; u < 4; ++u)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + (uint32_t)(((c * 4 + u) ^ (r & 7)) << 4)), "r"(pk[4 * u]),
                       "r"(pk[4 * u + 1]), "r"(pk[4 * u + 2]), "r"(pk[4 * u + 3])
                       : "memory");
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      warp_arrive(p_full, lane);
      if (warp == 2) attn_trace(p, 1, it);
      // dS = P o (dP o keep / keep_prob - delta)
      ok = mbar_wait(dp_full, ph, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE) &&
           mbar_wait(ds_empty, ph ^ 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (warp == 2) attn_trace(p, 2, it);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rd[32];
        tmem_ld32(lane_base + (uint32_t)(C::TMEM_DPQ + half * 64 + c * 32), rd);
        tmem_ld_wait();
        if (c == 1) tc_fence_before();   // ordered before the arrival below, which lets dQ^T overwrite these columns
        uint32_t gk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 e = unpack_bf162(pe[c * 16 + (i >> 1)]);
          float g0 = fmaf(__uint_as_float(rd[i]), inv_keep, -dlt), g1 = fmaf(__uint_as_float(rd[i + 1]), inv_keep, -dlt);
          if (drop) {
            if ((dropped[c] >> i) & 1u) g0 = -dlt;
            if ((dropped[c] >> (i + 1)) & 1u) g1 = -dlt;
          }
          gk[i >> 1] = pack_bf162(e.x * g0, e.y * g1);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dsrow + (uint32_t)(((c * 4 + u) ^ (r & 7)) << 4)), "r"(gk[4 * u]),
                       "r"(gk[4 * u + 1]), "r"(gk[4 * u + 2]), "r"(gk[4 * u + 3])
                       : "memory");
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      warp_arrive(ds_full, lane);
      if (warp == 2) attn_trace(p, 3, it);
    }
    // dK and dV of this key block: thread = key row x 64 of the 128 head-dim columns
    if (ok && n_it > 0) {
      ok = mbar_wait(dkv_full, 0, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const int key = k0 + r;
      constexpr int DH = D / 2;               // head-dim columns per thread
      bf16 *dkrow = p.dK + ((long long)b * p.Sk + key) * p.lddk + (long long)h * D + half * DH;
      bf16 *dvrow = p.dV + ((long long)b * p.Sk + key) * p.lddv + (long long)h * D + half * DH;
#pragma unroll 1
      for (int w = 0; w < 2; ++w) {            // 0: dK (times the score scale), 1: dV (times 1 / keep_prob)
        const float f = w == 0 ? p.scale : inv_keep;
        bf16 *orow = w == 0 ? dkrow : dvrow;
#pragma unroll 1
        for (int c = 0; c < DH / 32; ++c) {
          uint32_t rr[32];
          if (n_it > 0) {
            tmem_ld32(lane_base + (uint32_t)((w == 0 ? C::TMEM_DK : C::TMEM_DV) + half * DH + c * 32), rr);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) rr[i] = 0u;
          }
          if (key < p.Sk) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint4 v = make_uint4(pack_bf162(__uint_as_float(rr[8 * u]) * f, __uint_as_float(rr[8 * u + 1]) * f),
                                   pack_bf162(__uint_as_float(rr[8 * u + 2]) * f, __uint_as_float(rr[8 * u + 3]) * f),
                                   pack_bf162(__uint_as_float(rr[8 * u + 4]) * f, __uint_as_float(rr[8 * u + 5]) * f),
                                   pack_bf162(__uint_as_float(rr[8 * u + 6]) * f, __uint_as_float(rr[8 * u + 7]) * f));
              *reinterpret_cast<uint4 *>(orow + c * 32 + 8 * u) = v;
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ read-out of dQ_it
    // Eight warps.  Head dim 128: dQ_it^T, thread = head-dim index (TMEM lane quarter w % 4) x 64 of the block's 128 queries; a
    // warp-wide add covers 32 consecutive floats of one query's row in the fp32 accumulator.  Head dim 64: dQ_it, thread =
    // query row x 32 of the 64 columns, added with 16-byte vector atomics.
    const int quarter = warp & 3;
    const int qhalf = (warp - 10) >> 2;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    float *acc_head = p.dQ_acc + ((long long)(b * p.H + h) * p.Sq) * D;
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      ok = mbar_wait(dq_full, (uint32_t)it & 1u, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (warp == 10) attn_trace(p, 10, it);
      tc_fence_after();
      if constexpr (D == 128) {
        const int dcol = quarter * 32 + lane;
        uint32_t ra[32], rb[32];
        tmem_ld32(lane_base + (uint32_t)(C::TMEM_DPQ + qhalf * 64), ra);
        tmem_ld32(lane_base + (uint32_t)(C::TMEM_DPQ + qhalf * 64 + 32), rb);
        tmem_ld_wait();
        tc_fence_before();
        warp_arrive(dq_empty, lane);
        if (warp == 10) attn_trace(p, 11, it);
        const int qb0 = (i0 + it) * BQ + qhalf * 64;
        const int qn = p.Sq - qb0;               // queries of this half that exist
        float *dst = acc_head + (long long)qb0 * D + dcol;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < qn) atomicAdd(dst + i * D, __uint_as_float(ra[i]) * p.scale);
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (32 + i < qn) atomicAdd(dst + (32 + i) * D, __uint_as_float(rb[i]) * p.scale);
        if (warp == 10) attn_trace(p, 12, it);
      } else {
        uint32_t ra[32];
        tmem_ld32(lane_base + (uint32_t)(C::TMEM_DPQ + qhalf * 32), ra);
        tmem_ld_wait();
        tc_fence_before();
        warp_arrive(dq_empty, lane);
        const int q = (i0 + it) * BQ + quarter * 32 + lane;
        if (q < p.Sq) {
          float4 *dst = reinterpret_cast<float4 *>(acc_head + (long long)q * D + qhalf * 32);
#pragma unroll
          for (int u = 0; u < 8; ++u)
            atomicAdd(dst + u, make_float4(__uint_as_float(ra[4 * u]) * p.scale, __uint_as_float(ra[4 * u + 1]) * p.scale,
                                           __uint_as_float(ra[4 * u + 2]) * p.scale, __uint_as_float(ra[4 * u + 3]) * p.scale));
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

template <int D, bool P_TMEM>
int launch_fwd2(const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv, const AttnArgs &a, long long grid, cudaStream_t stream) {
  using C = Fwd2Cfg<D, P_TMEM>;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd2_kernel<D, P_TMEM>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  attn_fwd2_kernel<D, P_TMEM><<<(unsigned)grid, FWD2_THREADS, C::SMEM_BYTES, stream>>>(tq, tk, tv, a);
  return (int)cudaGetLastError();
}

// forward kernel in use: 1 = one query tile per CTA, 2 = two tiles per CTA with P through shared memory, 3 = two tiles with
// P through tensor memory.  All three give the same results; on B200 they also take the same time (the softmax warps, not
// the tensor core or the K / V traffic, bound them), so 1 stays the default.  FFK_ATTN_FWD or ffk_attention_set_fwd_variant
// choose another.
int g_fwd_variant = 0;
int fwd_variant() {
  if (!g_fwd_variant) {
    const char *e = getenv("FFK_ATTN_FWD");
    g_fwd_variant = e ? atoi(e) : 1;
    if (g_fwd_variant < 1 || g_fwd_variant > 3) g_fwd_variant = 1;
  }
  return g_fwd_variant;
}

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
  void *acc;                   // B*H*Sq*D floats of scratch (the dQ accumulator the key blocks add into)
};

template <int D, bool DROP>
static int launch_fwd1(const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv, const AttnArgs &a, long long grid, cudaStream_t stream) {
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<D, DROP>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdCfg<D>::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  attn_fwd_kernel<D, DROP><<<(unsigned)grid, ATT_THREADS, FwdCfg<D>::SMEM_BYTES, stream>>>(tq, tk, tv, a);
  return (int)cudaGetLastError();
}

// 1 when the fused kernels cover this head dimension / direction
FFK_API void ffk_attention_set_fwd_variant(int v) { g_fwd_variant = (v >= 1 && v <= 3) ? v : 1; }
FFK_API int ffk_attention_supported(int D, int backward) { (void)backward; return D == 64 || D == 128; }
FFK_API long long ffk_attention_bwd_scratch_floats(int B, int H, int Sq, int D) { return 1ll * B * H * Sq * D; }

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
  const int variant = fwd_variant();
  if (variant >= 2) {
    const long long grid2 = (long long)((d->Sq + 255) / 256) * d->H * d->B;
    if (grid2 > 0x7fffffffll) return -2;
    if (d->D == 128) return variant == 3 ? launch_fwd2<128, true>(tq, tk, tv, a, grid2, stream) : launch_fwd2<128, false>(tq, tk, tv, a, grid2, stream);
    return variant == 3 ? launch_fwd2<64, true>(tq, tk, tv, a, grid2, stream) : launch_fwd2<64, false>(tq, tk, tv, a, grid2, stream);
  }
  const long long grid = (long long)((d->Sq + BQ - 1) / BQ) * d->H * d->B;
  if (grid > 0x7fffffffll) return -2;
  const bool drop = d->drop_p > 0.f;
  if (d->D == 128) return drop ? launch_fwd1<128, true>(tq, tk, tv, a, grid, stream) : launch_fwd1<128, false>(tq, tk, tv, a, grid, stream);
  return drop ? launch_fwd1<64, true>(tq, tk, tv, a, grid, stream) : launch_fwd1<64, false>(tq, tk, tv, a, grid, stream);
}

template <int D>
static int launch_bwd(const FfkAttnDesc *d, AttnArgs &a, cudaStream_t stream) {
  using C = BwdCfg<D>;
  CUtensorMap tq, tk, tv, tdo;
  int r;
  if ((r = make_head_map(&tq, d->Q, D, d->Sq, d->ldq, d->H, d->B, BQ))) return r;
  if ((r = make_head_map(&tdo, d->dO, D, d->Sq, d->lddo, d->H, d->B, BQ))) return r;
  if ((r = make_head_map(&tk, d->K, D, d->Sk, d->ldk, d->H, d->B, C::BK))) return r;
  if ((r = make_head_map(&tv, d->V, D, d->Sk, d->ldv, d->H, d->B, C::BK))) return r;
  const long long n_acc = (long long)d->B * d->H * d->Sq * D;
  cudaError_t e = cudaMemsetAsync(d->acc, 0, (size_t)n_acc * sizeof(float), stream);
  if (e != cudaSuccess) return (int)e;
  {
    const long long warps = (long long)d->B * d->Sq * d->H;
    attn_delta_kernel<D><<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>((const bf16 *)d->dO, d->lddo, (const bf16 *)d->O, d->ldo,
                                                                           (float *)d->delta, d->B, d->H, d->Sq);
  }
  static bool attr = false;
  if (!attr) {
    e = cudaFuncSetAttribute(attn_bwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  const long long grid = (long long)((d->Sk + C::BK - 1) / C::BK) * d->H * d->B;
  if (grid > 0x7fffffffll) return -2;
  attn_bwd_kernel<D><<<(unsigned)grid, BWD_THREADS, C::SMEM_BYTES, stream>>>(tq, tk, tv, tdo, a);
  attn_acc_to_bf16_kernel<D><<<ffk_blocks(n_acc / 4, 256), 256, 0, stream>>>(a.dQ_acc, (bf16 *)d->dQ, d->lddq, d->B, d->H, d->Sq);
  return (int)cudaGetLastError();
}

FFK_API int ffk_attention_bwd(const FfkAttnDesc *d, cudaStream_t stream) {
  if (d->D != 128 && d->D != 64) return -2;
  if (d->B <= 0 || d->H <= 0 || d->Sq <= 0 || d->Sk <= 0) return 0;
  if (!aligned16(d->Q, d->ldq) || !aligned16(d->K, d->ldk) || !aligned16(d->V, d->ldv) || !aligned16(d->O, d->ldo) ||
      !aligned16(d->dO, d->lddo) || !aligned16(d->dQ, d->lddq) || !aligned16(d->dK, d->lddk) || !aligned16(d->dV, d->lddv) ||
      (((uintptr_t)d->acc) & 15))
    return -2;
  if (d->causal && d->Sq != d->Sk) return -2;
  AttnArgs a = {};
  a.B = d->B; a.H = d->H; a.Sq = d->Sq; a.Sk = d->Sk; a.scale = d->scale; a.causal = d->causal;
  a.drop_p = d->drop_p; a.drop_salt = d->drop_salt; a.drop_seed_ptr = (const unsigned long long *)d->drop_seed_ptr;
  a.lse = (float *)d->lse; a.delta = (const float *)d->delta;
  a.dK = (bf16 *)d->dK; a.lddk = d->lddk; a.dV = (bf16 *)d->dV; a.lddv = d->lddv;
  a.dQ_acc = (float *)d->acc;
  void *errp = nullptr;
  cudaGetSymbolAddress(&errp, g_attn_err);
  a.err = (int *)errp;
  { const char *e = getenv("FFK_ATTN_DBG"); a.dbg = e ? atoi(e) : 0; }
  return d->D == 128 ? launch_bwd<128>(d, a, stream) : launch_bwd<64>(d, a, stream);
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
