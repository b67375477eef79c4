// conv_sm100.cu -- stride-1 2-D convolution as an implicit GEMM on tcgen05 (sm_100a): forward, data gradient and
// weight gradient read the channels-last activation itself; no im2col / col2im matrix is ever written.
//
// Idea: over channels-last data [N, H, W, C], the rows of the im2col matrix that belong to one filter tap (r, s) and a
// box of bw x bh x bn output pixels are exactly the same box of the activation shifted by (r - pad_h, s - pad_w).  A tiled
// TMA load of that shifted box (64 channels deep) lands in shared memory as a K-major operand tile with one 128-byte
// row per pixel, and what falls outside the image is filled with zeros by the TMA unit -- which is the convolution's
// zero padding.  The reduction over K = KH * KW * C becomes a loop over (tap, 64-channel chunk).
//
//   forward        Y[p, oc]  = sum_{tap, c}  X[p + shift(tap), c]   * Wp[oc, tap * C + c]     M = pixels, N = OC
//   data gradient  dX[p, c]  = sum_{tap, oc} dY[p - shift(tap), oc] * Wp[oc, tap * C + c]     M = pixels, N = C
//   weight grad    dWp[oc, tap * C + c] = sum_p X[p + shift(tap), c] * dY[p, oc]              M = C, N = OC, K = pixels
//
// Wp is the packed filter [OC, KH * KW * C] the GEMM path already uses.  The weight gradient stages both operands with
// pixels as the reduction rows ("MN-major" operands), splits the pixel range over the CTAs and adds its partial sums into
// the fp32 packed gradient with warp-wide coalesced atomics.
//
// Roles per CTA (persistent, one CTA per SM): warp 0 issues TMA loads, warp 1 issues the MMAs, eight warps drain the
// accumulator (double-buffered in tensor memory) and write the output.  Every wait is bounded (see tcgen05.cuh).
//
// Reference counterpart: lib/kernels/src/cuda/ops/conv_2d_kernels.cu (cudnnConvolutionForward / BackwardData /
// BackwardFilter, algorithm chosen by cudnnFind*).
#include "tcgen05.cuh"

namespace {

constexpr int CONV_THREADS = 320;  // TMA warp, MMA warp, 8 epilogue warps
enum ConvMode : int { CONV_FPROP = 0, CONV_DGRAD = 1, CONV_WGRAD = 2 };

struct ConvArgs {
  // pixel grid the tiles walk over (output pixels for forward, input pixels for the data gradient, dY pixels for the
  // weight gradient) and the pixel box of one tile
  int PN, PH, PW;
  int bn, bh, bw, rows;          // rows = bn * bh * bw <= 128
  int tiles_n, tiles_h, tiles_w;
  int KH, KW;
  // operand box of tap (r, s) starts at pixel origin + (off_h + sgn * r, off_w + sgn * s)
  int off_h, off_w, sgn;
  int CK;                        // reduction channels per tap (forward: C, data gradient: OC)
  int chunks;                    // ceil(CK / 64)
  int Cf;                        // channels of the filter = columns of Wp per tap
  int Nout;                      // output columns (forward: OC, data gradient: C, weight gradient: OC)
  int Mw;                        // weight gradient: rows of the product = C
  int tiles_nb;                  // output column tiles
  int tiles_mb;                  // weight gradient: 128-row tiles over C
  long long num_items;
  int split, k_per_split;        // weight gradient: pixel tiles per split
  // output
  void *out; long long ldo;      // bf16 [pixels, Nout] (forward / data gradient); float [OC, ldo] (weight gradient)
  void *pre;                     // optional pre-activation copy (bf16, layout of out)
  const void *bias;              // bf16 [Nout] or null
  int act;
  int accumulate;
  int *err;
};

template <int BN, int MODE>
struct ConvCfg {
  static constexpr bool WG = MODE == CONV_WGRAD;
  static constexpr bool B_MN = MODE != CONV_FPROP;
  // forward / data gradient: A = 128 pixel rows x 64 channels (K-major).  weight gradient: A = X box, two 64-channel
  // chunks of 128 pixel rows each (MN-major: channels contiguous, pixels are the reduction)
  static constexpr int A_BYTES = WG ? 2 * 128 * 128 : 128 * 128;
  // forward: B = BN filter rows x 64 k (K-major).  data gradient: B = BN / 64 chunks of 64 k-rows (MN-major).
  // weight gradient: B = dY box, BN / 64 chunks of 128 pixel rows.
  static constexpr int B_BYTES = WG ? (BN / 64) * 128 * 128 : BN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = STAGE_BYTES <= 24576 ? 8 : (STAGE_BYTES <= 32768 ? 6 : (STAGE_BYTES <= 49152 ? 4 : 3));
  static constexpr int TMEM_COLS = 2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512);
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
  static constexpr uint32_t A_LBO = WG ? 128 * 128 : 16;
  static constexpr uint32_t B_LBO = WG ? 128 * 128 : (B_MN ? 64 * 128 : 16);
  static constexpr uint32_t A_KADV = WG ? 16 * 128 : 32;
  static constexpr uint32_t B_KADV = B_MN ? 16 * 128 : 32;
  static constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((WG ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                                    ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
};

struct ConvItem {
  int n0, h0, w0;   // pixel tile origin (forward / data gradient)
  int nb;           // output column tile
  int mb, tap;      // weight gradient: row tile over C, filter tap
  int k0, k1;       // reduction range: (tap, chunk) blocks or pixel tiles
};

template <int MODE>
__device__ __forceinline__ ConvItem decode_item(long long item, const ConvArgs &p) {
  ConvItem it;
  if (MODE != CONV_WGRAD) {
    it.nb = (int)(item % p.tiles_nb);
    long long t = item / p.tiles_nb;
    it.w0 = (int)(t % p.tiles_w) * p.bw;
    t /= p.tiles_w;
    it.h0 = (int)(t % p.tiles_h) * p.bh;
    it.n0 = (int)(t / p.tiles_h) * p.bn;
    it.mb = 0; it.tap = 0;
    it.k0 = 0; it.k1 = p.KH * p.KW * p.chunks;
  } else {
    it.nb = (int)(item % p.tiles_nb);
    long long t = item / p.tiles_nb;
    it.mb = (int)(t % p.tiles_mb);
    t /= p.tiles_mb;
    it.tap = (int)(t % (p.KH * p.KW));
    const int s = (int)(t / (p.KH * p.KW));
    const int total = p.tiles_n * p.tiles_h * p.tiles_w;
    it.k0 = s * p.k_per_split;
    it.k1 = min(it.k0 + p.k_per_split, total);
    it.n0 = it.h0 = it.w0 = 0;
  }
  return it;
}

template <int BN, int MODE>
__global__ void __launch_bounds__(CONV_THREADS, 1)
conv_sm100_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB, const ConvArgs p) {
  using Cfg = ConvCfg<BN, MODE>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr bool WG = Cfg::WG;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *tiles = smem;
  uint64_t *bars = (uint64_t *)(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t *full_bar = bars;
  uint64_t *empty_bar = bars + STAGES;
  uint64_t *tmem_full = bars + 2 * STAGES;
  uint64_t *tmem_empty = bars + 2 * STAGES + 2;
  uint32_t *tmem_slot = (uint32_t *)(bars + 2 * STAGES + 4);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&tmem_full[s], 1); mbar_init(&tmem_empty[s], 8); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)Cfg::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (WG && p.rows < 128) {
    // pixel rows past the box are never written by the loads; as reduction rows of the weight gradient they must be zero
    uint4 *z = (uint4 *)tiles;
    const int n16 = STAGES * Cfg::STAGE_BYTES / 16;
    for (int i = threadIdx.x; i < n16; i += CONV_THREADS) z[i] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t box_bytes = (uint32_t)p.rows * 128u;   // one 64-channel box of the pixel tile

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long item = blockIdx.x; item < p.num_items && ok; item += gridDim.x) {
        const ConvItem it = decode_item<MODE>(item, p);
        for (int kb = it.k0; kb < it.k1; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err, FFK_ERR_TIMEOUT_PRODUCER);
          if (!ok) break;
          const uint32_t sa = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
          if constexpr (!WG) {
            const int tap = kb / p.chunks, cc = kb - tap * p.chunks;
            const int r = tap / p.KW, s = tap - r * p.KW;
            mbar_expect_tx(&full_bar[stage], box_bytes + (uint32_t)Cfg::B_BYTES);
            tma_load_4d(sa, &tmapA, &full_bar[stage], cc * 64, it.w0 + p.off_w + p.sgn * s, it.h0 + p.off_h + p.sgn * r, it.n0);
            if constexpr (MODE == CONV_FPROP) {
              // BN filter rows, 64 reduction columns of this tap and chunk (columns past the tap's C meet zero channels)
              tma_load_4d(sb, &tmapB, &full_bar[stage], tap * p.Cf + cc * 64, it.nb * BN, 0, 0);
            } else {
#pragma unroll
              for (int c = 0; c < BN / 64; ++c)
                tma_load_4d(sb + c * 64 * 128, &tmapB, &full_bar[stage], tap * p.Cf + it.nb * BN + c * 64, cc * 64, 0, 0);
            }
          } else {
            int t = kb;
            const int w0 = (t % p.tiles_w) * p.bw;
            t /= p.tiles_w;
            const int h0 = (t % p.tiles_h) * p.bh;
            const int n0 = (t / p.tiles_h) * p.bn;
            const int r = it.tap / p.KW, s = it.tap - r * p.KW;
            mbar_expect_tx(&full_bar[stage], box_bytes * (uint32_t)(2 + BN / 64));
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tma_load_4d(sa + c * 128 * 128, &tmapA, &full_bar[stage], it.mb * 128 + c * 64, w0 + p.off_w + s, h0 + p.off_h + r, n0);
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_4d(sb + c * 128 * 128, &tmapB, &full_bar[stage], it.nb * BN + c * 64, w0, h0, n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      for (int s = 0; s < STAGES && ok; ++s) {   // every load issued has landed and been consumed before the CTA exits
        ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err, FFK_ERR_TIMEOUT_PRODUCER);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      const int wg_ksteps = (p.rows + 15) / 16;
      for (long long item = blockIdx.x; item < p.num_items && ok; item += gridDim.x) {
        const ConvItem it = decode_item<MODE>(item, p);
        ok = mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = it.k0; kb < it.k1; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.err, FFK_ERR_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
          const uint64_t adesc = make_smem_desc(sa, Cfg::A_LBO, 1024);
          const uint64_t bdesc = make_smem_desc(sa + Cfg::A_BYTES, Cfg::B_LBO, 1024);
          int ksteps = wg_ksteps;
          if constexpr (!WG) {   // the last chunk of a tap may hold fewer than 64 channels: skip the all-zero k-steps
            const int left = p.CK - (kb % p.chunks) * 64;
            ksteps = left >= 64 ? 4 : (left + 15) / 16;
          }
          for (int k = 0; k < ksteps; ++k)
            tc_mma<false>(d_tmem, desc_advance(adesc, (uint32_t)k * Cfg::A_KADV), desc_advance(bdesc, (uint32_t)k * Cfg::B_KADV), Cfg::IDESC,
                          ((kb - it.k0) | k) != 0 ? 1u : 0u);
          tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&tmem_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: thread = accumulator row
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;       // column half
    constexpr int HALF = BN / 2;
    const int row = q * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (long long item = blockIdx.x; item < p.num_items && ok; item += gridDim.x) {
      const ConvItem it = decode_item<MODE>(item, p);
      ok = mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.err, FFK_ERR_TIMEOUT_EPILOGUE);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_base = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + half * HALF);
      if constexpr (!WG) {
        // row -> pixel of the box (image, row, column innermost)
        const int pw = row % p.bw;
        const int t = row / p.bw;
        const int ph = t % p.bh;
        const int pn = t / p.bh;
        const int n = it.n0 + pn, h = it.h0 + ph, w = it.w0 + pw;
        const bool row_ok = row < p.rows && n < p.PN && h < p.PH && w < p.PW;
        const long long orow = ((long long)n * p.PH + h) * p.PW + w;
        bf16 *op = (bf16 *)p.out + orow * p.ldo;
        bf16 *pp = p.pre ? (bf16 *)p.pre + orow * p.ldo : nullptr;
#pragma unroll 1
        for (int c0 = 0; c0 < HALF; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(t_base + (uint32_t)c0, r);
          tmem_ld_wait();
          const int col0 = it.nb * BN + half * HALF + c0;
          if (row_ok) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int col = col0 + u * 8;
              if (col >= p.Nout) break;   // Nout is a multiple of 8
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[u * 8 + j]);
              if (p.bias) {
                const uint4 bv = *reinterpret_cast<const uint4 *>((const bf16 *)p.bias + col);
                const float2 b0 = unpack_bf162(bv.x), b1 = unpack_bf162(bv.y), b2 = unpack_bf162(bv.z), b3 = unpack_bf162(bv.w);
                v[0] += b0.x; v[1] += b0.y; v[2] += b1.x; v[3] += b1.y; v[4] += b2.x; v[5] += b2.y; v[6] += b3.x; v[7] += b3.y;
              }
              if (pp)
                *reinterpret_cast<uint4 *>(pp + col) =
                    make_uint4(pack_bf162(v[0], v[1]), pack_bf162(v[2], v[3]), pack_bf162(v[4], v[5]), pack_bf162(v[6], v[7]));
              if (p.act == ACT_RELU) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = fmaxf(v[j], 0.f);
              } else if (p.act != ACT_NONE) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = act_fwd(v[j], p.act);
              }
              if (p.accumulate) {
                const uint4 ov = *reinterpret_cast<const uint4 *>(op + col);
                const float2 o0 = unpack_bf162(ov.x), o1 = unpack_bf162(ov.y), o2 = unpack_bf162(ov.z), o3 = unpack_bf162(ov.w);
                v[0] += o0.x; v[1] += o0.y; v[2] += o1.x; v[3] += o1.y; v[4] += o2.x; v[5] += o2.y; v[6] += o3.x; v[7] += o3.y;
              }
              *reinterpret_cast<uint4 *>(op + col) =
                  make_uint4(pack_bf162(v[0], v[1]), pack_bf162(v[2], v[3]), pack_bf162(v[4], v[5]), pack_bf162(v[6], v[7]));
            }
          }
        }
      } else {
        // row = filter channel c, registers = output channels: a warp-wide add covers 32 consecutive floats of one
        // output channel's row in the packed fp32 gradient
        const int c = it.mb * 128 + row;
        const bool row_ok = c < p.Mw;
        float *gp = (float *)p.out + (long long)it.tap * p.Cf + c;
#pragma unroll 1
        for (int c0 = 0; c0 < HALF; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(t_base + (uint32_t)c0, r);
          tmem_ld_wait();
          const int oc0 = it.nb * BN + half * HALF + c0;
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (oc0 + j < p.Nout) atomicAdd(gp + (long long)(oc0 + j) * p.ldo, __uint_as_float(r[j]));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
  }
}

__device__ int g_conv_err = 0;

// channels-last activation [N, H, W, C] as a 4-D map {C, W, H, N}; box = 64 channels x bw x bh x bn pixels
int make_act_map(CUtensorMap *map, const void *ptr, int N, int H, int W, int C, int bn, int bh, int bw) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
  cuuint64_t strides[3] = {(cuuint64_t)C * 2, (cuuint64_t)W * C * 2, (cuuint64_t)H * W * C * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)bw, (cuuint32_t)bh, (cuuint32_t)bn};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, (void *)ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
// packed filter [OC, cols] (row pitch ld elements) as {cols, OC, 1, 1}; box = 64 columns x box_rows rows
int make_filter_map(CUtensorMap *map, const void *ptr, int OC, long long cols, long long ld, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)OC, 1, 1};
  cuuint64_t strides[3] = {(cuuint64_t)ld * 2, (cuuint64_t)ld * 2 * (cuuint64_t)OC, (cuuint64_t)ld * 2 * (cuuint64_t)OC};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, (void *)ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

int conv_sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

// the pixel box with the fewest tiles over a PN x PH x PW grid: bw * bh * bn <= 128; several images share a tile only
// when one image fits whole
void choose_box(int PN, int PH, int PW, int &bn, int &bh, int &bw) {
  long long best = -1;
  bn = bh = bw = 1;
  for (int w = 1; w <= PW && w <= 128; ++w) {
    for (int h = 1; h <= PH && w * h <= 128; ++h) {
      int n = 1;
      if (w == PW && h == PH) n = 128 / (w * h) < PN ? 128 / (w * h) : PN;
      if (n < 1) n = 1;
      const long long tiles = (long long)((PW + w - 1) / w) * ((PH + h - 1) / h) * ((PN + n - 1) / n);
      // fewer tiles first; among equals the wider box (longer contiguous runs per row of pixels)
      if (best < 0 || tiles < best || (tiles == best && w > bw)) { best = tiles; bn = n; bh = h; bw = w; }
    }
  }
}

template <int BN, int MODE>
int launch_conv(const CUtensorMap &ta, const CUtensorMap &tb, const ConvArgs &a, cudaStream_t st) {
  using Cfg = ConvCfg<BN, MODE>;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(conv_sm100_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  const long long grid = a.num_items < conv_sm_count() ? a.num_items : conv_sm_count();
  conv_sm100_kernel<BN, MODE><<<(unsigned)grid, CONV_THREADS, Cfg::SMEM_BYTES, st>>>(ta, tb, a);
  return (int)cudaGetLastError();
}

template <int MODE>
int launch_conv_bn(int bn_tile, const CUtensorMap &ta, const CUtensorMap &tb, const ConvArgs &a, cudaStream_t st) {
  if (bn_tile == 64) return launch_conv<64, MODE>(ta, tb, a, st);
  if (bn_tile == 128) return launch_conv<128, MODE>(ta, tb, a, st);
  if constexpr (MODE != CONV_WGRAD) return launch_conv<256, MODE>(ta, tb, a, st);
  return -2;
}

}  // namespace

// One stride-1 convolution over channels-last bf16 data.  Plain C struct so ctypes can fill it.
struct FfkConvDesc {
  int N, H, W, C;          // input activation [N, H, W, C]
  int OC, KH, KW;
  int pad_h, pad_w;
  int OH, OW;              // = H + 2 pad - K + 1
  const void *x;           // [N, H, W, C] bf16 (forward, weight gradient)
  const void *wp;          // packed filter [OC, ldw] bf16, column (r * KW + s) * C + c
  long long ldw;
  void *y;                 // forward: [N, OH, OW, OC] bf16 out
  void *pre;               // forward: optional pre-activation copy
  const void *bias;        // forward: bf16 [OC] or null
  int act;
  const void *dy;          // gradients: [N, OH, OW, OC] bf16
  void *dx;                // data gradient: [N, H, W, C] bf16
  int accumulate;          // data gradient: dx += ; weight gradient: dwp += (else dwp is cleared first)
  void *dwp;               // weight gradient: [OC, ldw] fp32
};

// Which convolutions this kernel takes (everything else keeps the im2col + GEMM path): stride 1 (the caller checks),
// channel counts that keep every TMA row pitch and every vector store 16-byte aligned.
FFK_API int ffk_conv_implicit_supported(int C, int OC, int KH, int KW) {
  return C % 8 == 0 && OC % 8 == 0 && C >= 8 && OC >= 8 && KH >= 1 && KW >= 1 && KH * KW <= 64;
}

static int conv_common(const FfkConvDesc *d, ConvArgs &a, int PN, int PH, int PW) {
  if (!ffk_conv_implicit_supported(d->C, d->OC, d->KH, d->KW)) return -2;
  if (d->OH != d->H + 2 * d->pad_h - d->KH + 1 || d->OW != d->W + 2 * d->pad_w - d->KW + 1 || d->OH <= 0 || d->OW <= 0) return -2;
  if (d->ldw % 8 != 0 || d->ldw < (long long)d->KH * d->KW * d->C) return -2;
  a = ConvArgs{};
  a.PN = PN; a.PH = PH; a.PW = PW;
  choose_box(PN, PH, PW, a.bn, a.bh, a.bw);
  a.rows = a.bn * a.bh * a.bw;
  a.tiles_n = (PN + a.bn - 1) / a.bn; a.tiles_h = (PH + a.bh - 1) / a.bh; a.tiles_w = (PW + a.bw - 1) / a.bw;
  a.KH = d->KH; a.KW = d->KW;
  a.Cf = d->C;
  void *errp = nullptr;
  cudaGetSymbolAddress(&errp, g_conv_err);
  a.err = (int *)errp;
  return 0;
}

static int pick_bn(int n) { return n <= 64 ? 64 : (n <= 128 ? 128 : 256); }

FFK_API int ffk_conv_fprop(const FfkConvDesc *d, cudaStream_t st) {
  if (d->N <= 0) return 0;
  ConvArgs a;
  int r = conv_common(d, a, d->N, d->OH, d->OW);
  if (r) return r;
  if ((((uintptr_t)d->x) | ((uintptr_t)d->wp) | ((uintptr_t)d->y) | ((uintptr_t)d->pre) | ((uintptr_t)d->bias)) & 15) return -2;
  a.off_h = -d->pad_h; a.off_w = -d->pad_w; a.sgn = 1;
  a.CK = d->C; a.chunks = (d->C + 63) / 64;
  a.Nout = d->OC;
  const int bn_tile = pick_bn(d->OC);
  a.tiles_nb = (d->OC + bn_tile - 1) / bn_tile;
  a.num_items = (long long)a.tiles_n * a.tiles_h * a.tiles_w * a.tiles_nb;
  a.out = d->y; a.ldo = d->OC; a.pre = d->pre; a.bias = d->bias; a.act = d->act; a.accumulate = 0;
  CUtensorMap ta, tb;
  if ((r = make_act_map(&ta, d->x, d->N, d->H, d->W, d->C, a.bn, a.bh, a.bw))) return r;
  if ((r = make_filter_map(&tb, d->wp, d->OC, (long long)d->KH * d->KW * d->C, d->ldw, bn_tile))) return r;
  return launch_conv_bn<CONV_FPROP>(bn_tile, ta, tb, a, st);
}

FFK_API int ffk_conv_dgrad(const FfkConvDesc *d, cudaStream_t st) {
  if (d->N <= 0) return 0;
  ConvArgs a;
  int r = conv_common(d, a, d->N, d->H, d->W);
  if (r) return r;
  if ((((uintptr_t)d->dy) | ((uintptr_t)d->wp) | ((uintptr_t)d->dx)) & 15) return -2;
  // dX[h, w] takes dY[h + pad_h - r, w + pad_w - s] through filter tap (r, s)
  a.off_h = d->pad_h; a.off_w = d->pad_w; a.sgn = -1;
  a.CK = d->OC; a.chunks = (d->OC + 63) / 64;
  a.Nout = d->C;
  const int bn_tile = pick_bn(d->C);
  a.tiles_nb = (d->C + bn_tile - 1) / bn_tile;
  a.num_items = (long long)a.tiles_n * a.tiles_h * a.tiles_w * a.tiles_nb;
  a.out = d->dx; a.ldo = d->C; a.pre = nullptr; a.bias = nullptr; a.act = ACT_NONE; a.accumulate = d->accumulate;
  CUtensorMap ta, tb;
  if ((r = make_act_map(&ta, d->dy, d->N, d->OH, d->OW, d->OC, a.bn, a.bh, a.bw))) return r;
  if ((r = make_filter_map(&tb, d->wp, d->OC, (long long)d->KH * d->KW * d->C, d->ldw, 64))) return r;
  return launch_conv_bn<CONV_DGRAD>(bn_tile, ta, tb, a, st);
}

FFK_API int ffk_conv_wgrad(const FfkConvDesc *d, cudaStream_t st) {
  if (d->N <= 0) return 0;
  ConvArgs a;
  int r = conv_common(d, a, d->N, d->OH, d->OW);
  if (r) return r;
  if ((((uintptr_t)d->dy) | ((uintptr_t)d->x) | ((uintptr_t)d->dwp)) & 15) return -2;
  a.off_h = -d->pad_h; a.off_w = -d->pad_w; a.sgn = 1;
  a.Mw = d->C;
  a.Nout = d->OC;
  const int bn_tile = d->OC <= 64 ? 64 : 128;
  a.tiles_nb = (d->OC + bn_tile - 1) / bn_tile;
  a.tiles_mb = (d->C + 127) / 128;
  const long long base = (long long)a.tiles_nb * a.tiles_mb * d->KH * d->KW;
  const int ptiles = a.tiles_n * a.tiles_h * a.tiles_w;
  // enough splits of the pixel range to give every SM about two work items, at least 4 pixel tiles each
  long long want = (2LL * conv_sm_count() + base - 1) / base;
  if (want > ptiles / 4) want = ptiles / 4;
  if (want < 1) want = 1;
  a.k_per_split = (int)((ptiles + want - 1) / want);
  a.split = (ptiles + a.k_per_split - 1) / a.k_per_split;
  a.num_items = base * a.split;
  a.out = d->dwp; a.ldo = d->ldw;
  if (!d->accumulate) {
    cudaError_t e = cudaMemsetAsync(d->dwp, 0, (size_t)d->OC * (size_t)d->ldw * sizeof(float), st);
    if (e != cudaSuccess) return (int)e;
  }
  CUtensorMap ta, tb;
  if ((r = make_act_map(&ta, d->x, d->N, d->H, d->W, d->C, a.bn, a.bh, a.bw))) return r;
  if ((r = make_act_map(&tb, d->dy, d->N, d->OH, d->OW, d->OC, a.bn, a.bh, a.bw))) return r;
  return launch_conv_bn<CONV_WGRAD>(bn_tile, ta, tb, a, st);
}

// Reads (and clears) the error word of the convolution kernel's bounded waits.  Synchronises the device.
FFK_API int ffk_conv_last_error() {
  int v = 0, z = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  cudaMemcpyFromSymbol(&v, g_conv_err, sizeof(int));
  cudaMemcpyToSymbol(g_conv_err, &z, sizeof(int));
  return v;
}
