// Gated half of the GLU MLP on CTA pairs:  h[:, k q + n] = gelu(x_k . wg[k][n, :]) * (x_{k+nb/2} . wg[k+nb/2][n, :])
// for K = d_model / nblocks <= 192 per block (the 80M and large shapes: 192 and 384 -> the latter stays on the
// single-CTA kernels).
//
// A pair of CTAs (the two SMs of a TPC) owns 256 rows: each CTA keeps ITS 128 rows of the two x slices a block pair
// needs resident in shared memory (2 x 48 KB) while the pair walks the block pair's column tiles; only wg rows stream
// through a ring, and each CTA fetches just HALF of them -- `tcgen05.mma.cta_group::2` (M = 256, N = 128, K = 16)
// reads 64 of the 128 rows of a column tile from each CTA's shared memory.  Per 128-column tile and CTA that is 48 KB
// of TMA traffic for two 128 x 128 x 192 products, against 96 KB for the single-CTA kernel with resident x and 196 KB
// without -- and the L2 -> shared-memory rate is what paces these GEMMs.  Gate and linear accumulators sit side by
// side in tensor memory (columns [0,128) and [128,256) of one of two buffers); the epilogue applies GELU and the
// product with the reference's bf16 rounding points and never writes the pre-activation.
//
// Roles per CTA (608 threads): warp 0 TMA producer, warps 1-2 MMA issue (leader CTA only; one thread per accumulator),
// warps 3-18 epilogue.  Loads of both CTAs count on the LEADER's barriers; commits multicast to both CTAs; the peer's
// epilogue returns accumulators with a remote mbarrier arrive.  Every wait is bounded.
//
// Computation replaced: gated_layers + slice + GELU + product of BertGatedLinearUnitMLP.forward,
// bert/src/bert_layers.py:492-501, on BlockdiagMultiply (bert/src/mm/blockdiag_multiply.py:49-60).
#include "tc_common.cuh"

namespace m2 {
namespace glup {

constexpr int BM = 128, BK = 64, BN = 128;              // rows per CTA, K step, gate columns per tile (+ as many linear)
constexpr int MAX_KS = 3, NSTB = 6;
constexpr int A_BYTES = BM * BK * 2;                    // 16 KB: one K step of one x slice
constexpr int BH = BN / 2;                              // wg rows of a column tile each CTA stages
constexpr int B_HALF = BH * BK * 2;                     // 8 KB
constexpr int B_STAGE = 2 * B_HALF;                     // gate + linear rows of one K step
constexpr int OFF_B = 2 * MAX_KS * A_BYTES;             // after the resident x tiles: 96 KB
constexpr int OFF_BAR = OFF_B + NSTB * B_STAGE;
constexpr int NBARS = 2 * NSTB + MAX_KS + 4;
constexpr int EPI_WARPS = 16, EPI_WARP0 = 3, THREADS = 32 * (EPI_WARP0 + EPI_WARPS);
constexpr int CW = BN / (EPI_WARPS / 4);                // gate columns per epilogue warp: 32
constexpr int SMEM = OFF_BAR + NBARS * 8 + 16 + 1024;
static_assert(SMEM <= 227 * 1024, "shared memory budget");

struct Params {
  int M, p, q, nb_half, ksteps, ntn, gs, ngroups, total_units, wide_out;
  void* out; long long ldo;
};

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
glu_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params P) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* b_full = bars;                   // [NSTB] leader's: wg rows (and, on a unit's first tile, x tiles) of both CTAs landed
  uint64_t* b_empty = b_full + NSTB;         // [NSTB] each CTA's: both issuers' MMAs have read the stage
  uint64_t* a_empty = b_empty + NSTB;        // [MAX_KS] each CTA's: both issuers are done with the x tiles of K step ks
  uint64_t* tfull = a_empty + MAX_KS;        // [2] each CTA's: both accumulators of the buffer complete
  uint64_t* tempty = tfull + 2;              // [2] leader's: both CTAs' epilogues have drained the buffer
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = tc::cluster_ctarank();
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTB; ++s) { tc::mbar_init(b_full + s, 1); tc::mbar_init(b_empty + s, 2); }
    for (int k = 0; k < MAX_KS; ++k) tc::mbar_init(a_empty + k, 2);
    for (int b = 0; b < 2; ++b) { tc::mbar_init(tfull + b, 2); tc::mbar_init(tempty + b, 2 * EPI_WARPS); }
    *abort_flag = 0;
    tc::mbar_fence_init();
    tc::tma_prefetch_desc(&tmA);
    tc::tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tc::tmem_alloc2(tmem_slot, 512);
    tc::tmem_relinquish2();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::cluster_sync();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // this pair's contiguous range of units; unit = (x pair = 256-row tile x block pair, group of column tiles)
  const int u0 = (int)((long long)pair * P.total_units / npairs);
  const int u1 = (int)((long long)(pair + 1) * P.total_units / npairs);
  auto decode = [&](int unit, int& xp, int& mp, int& kb, int& nt0, int& ntiles) {
    xp = unit / P.ngroups;
    const int g = unit % P.ngroups;
    mp = xp / P.nb_half; kb = xp % P.nb_half;
    nt0 = g * P.gs;
    ntiles = P.ntn - nt0 < P.gs ? P.ntn - nt0 : P.gs;
  };

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) -------------------------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int epoch = -1, prev_xp = -1;
      bool ok = true;
      for (int unit = u0; unit < u1 && ok; ++unit) {
        int xp, mp, kb, nt0, ntiles;
        decode(unit, xp, mp, kb, nt0, ntiles);
        const int row0 = (2 * mp + (int)rank) * BM;
        const bool new_x = xp != prev_xp;
        if (new_x) { ++epoch; prev_xp = xp; }
        for (int t = 0; t < ntiles && ok; ++t) {
          const bool load_x = new_x && t == 0;
          for (int ks = 0; ks < P.ksteps; ++ks) {
            if (!tc::mbar_wait(b_empty + stage, phase ^ 1, abort_flag, tc::ST_TIMEOUT_EMPTY)) { ok = false; break; }
            if (load_x && epoch > 0 &&
                !tc::mbar_wait(a_empty + ks, (uint32_t)(epoch - 1) & 1u, abort_flag, tc::ST_TIMEOUT_EMPTY)) { ok = false; break; }
            unsigned char* st = smem + OFF_B + stage * B_STAGE;
            const uint32_t fb = tc::mapa_shared(tc::smem_u32(b_full + stage), 0);
            if (rank == 0) tc::mbar_expect_tx(b_full + stage, 2 * (B_STAGE + (load_x ? 2 * A_BYTES : 0)));
            if (load_x) {
              tc::tma_load_2d_2sm(smem + ks * A_BYTES, &tmA, fb, kb * P.p + ks * BK, row0);
              tc::tma_load_2d_2sm(smem + (MAX_KS + ks) * A_BYTES, &tmA, fb, (kb + P.nb_half) * P.p + ks * BK, row0);
            }
            const int row_g = kb * P.q + (nt0 + t) * BN + (int)rank * BH;
            tc::tma_load_2d_2sm(st, &tmB, fb, ks * BK, row_g);
            tc::tma_load_2d_2sm(st + B_HALF, &tmB, fb, ks * BK, row_g + P.nb_half * P.q);
            if (++stage == NSTB) { stage = 0; phase ^= 1; }
          }
        }
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ------------------------------- MMA issuers (leader CTA): warp 1 gate, warp 2 linear -------------------------------
    // Each thread issues every tile's MMAs of its accumulator in order, so its commit to `a_empty` after the last
    // tile that reads the old x covers all of its earlier MMAs as well.
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = tc::make_idesc(2 * BM, BN, 1);
      const int chain = warp - 1;
      const uint64_t dA0 = tc::smem_desc_k_sw128(tc::smem_u32(smem + chain * MAX_KS * A_BYTES));
      const uint64_t dB0 = tc::smem_desc_k_sw128(tc::smem_u32(smem + OFF_B + chain * B_HALF));
      int stage = 0; uint32_t phase = 0;
      int buf = 0; uint32_t bphase = 0;
      bool ok = true;
      for (int unit = u0; unit < u1 && ok; ++unit) {
        int xp, mp, kb, nt0, ntiles;
        decode(unit, xp, mp, kb, nt0, ntiles);
        const bool x_changes = unit + 1 < u1 && (unit + 1) / P.ngroups != xp;
        for (int t = 0; t < ntiles && ok; ++t) {
          if (!tc::mbar_wait(tempty + buf, bphase ^ 1, abort_flag, tc::ST_TIMEOUT_MMA)) { ok = false; break; }
          tc::tc_fence_after();
          const uint32_t acc = tmem_base + buf * 2 * BN + chain * BN;
          const bool release_x = x_changes && t == ntiles - 1;
          for (int ks = 0; ks < P.ksteps; ++ks) {
            if (!tc::mbar_wait(b_full + stage, phase, abort_flag, tc::ST_TIMEOUT_TMA)) { ok = false; break; }
            tc::tc_fence_after();
            const uint64_t dA = dA0 + (uint64_t)(ks * (A_BYTES >> 4)), dB = dB0 + (uint64_t)(stage * (B_STAGE >> 4));
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) tc::mma_ss2(acc, dA + 2 * kk, dB + 2 * kk, idesc, (ks | kk) ? 1u : 0u);
            tc::mma_commit2_mc(b_empty + stage, 3);
            if (release_x) tc::mma_commit2_mc(a_empty + ks, 3);
            if (++stage == NSTB) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          tc::mma_commit2_mc(tfull + buf, 3);
          if ((buf ^= 1) == 0) bphase ^= 1;
        }
      }
    }
  } else if (warp >= EPI_WARP0) {
    // ------------------------------- epilogue (both CTAs) -------------------------------
    const int quarter = warp & 3;
    const int cs = (warp - EPI_WARP0) >> 2;                 // which 32 gate columns (and their 32 linear partners)
    const uint32_t tempty_leader = tc::mapa_shared(tc::smem_u32(tempty), 0);
    int buf = 0; uint32_t bphase = 0;
    bool ok = true;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(P.out);
    for (int unit = u0; unit < u1 && ok; ++unit) {
      int xp, mp, kb, nt0, ntiles;
      decode(unit, xp, mp, kb, nt0, ntiles);
      const int row = (2 * mp + (int)rank) * BM + quarter * 32 + lane;
      for (int t = 0; t < ntiles; ++t) {
        if (!tc::mbar_wait(tfull + buf, bphase, abort_flag, tc::ST_TIMEOUT_EPI)) { ok = false; break; }
        tc::tc_fence_after();
        const uint32_t tacc = tmem_base + buf * 2 * BN + ((uint32_t)(quarter * 32) << 16) + cs * CW;
        // all of the warp's columns go to registers and the buffer is handed back before any arithmetic
        uint32_t a[CW / 16][16], b[CW / 16][16];
#pragma unroll
        for (int ch = 0; ch < CW / 16; ++ch) {
          tc::tmem_ld16(tacc + 16 * ch, a[ch]);
          tc::tmem_ld16(tacc + BN + 16 * ch, b[ch]);
        }
        tc::tmem_ld_wait();
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive_cluster(tempty_leader + 8 * buf);
        __nv_bfloat16* orow = out + (long long)row * P.ldo + kb * P.q + (nt0 + t) * BN + cs * CW;
#pragma unroll
        for (int ch = 0; ch < CW / 16; ++ch) {
          uint32_t packed[8];
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            const uint32_t g = pack_bf16(__uint_as_float(a[ch][j]), __uint_as_float(a[ch][j + 1]));
            const uint32_t n = pack_bf16(__uint_as_float(b[ch][j]), __uint_as_float(b[ch][j + 1]));
            float a0, a1;
            gelu_pair(__uint_as_float(g << 16), __uint_as_float(g & 0xFFFF0000u), a0, a1);
            packed[j >> 1] = bf2_mul(pack_bf16(a0, a1), n);   // GELU output cast to bf16, times the linear half
          }
          if (row < P.M) {
            if (P.wide_out) {                   // one full 32-byte sector per thread
              stg256(orow + 16 * ch, packed[0], packed[1], packed[2], packed[3], packed[4], packed[5], packed[6], packed[7]);
            } else {
              uint4* dst = reinterpret_cast<uint4*>(orow + 16 * ch);
              dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
              dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            }
          }
        }
        if ((buf ^= 1) == 0) bphase ^= 1;
      }
    }
  }

  // ------------------------------- teardown -------------------------------------
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0 && rank == 0) {
    for (int s = 0; s < NSTB; ++s)
      for (uint32_t i = 0; i < 4096 && !tc::mbar_try_wait(b_full + s, 0) && !tc::mbar_try_wait(b_full + s, 1); ++i) {}
  }
  tc::tc_fence_before();
  tc::cluster_sync();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc2(tmem_base, 512);
  }
}

}  // namespace glup

bool glu_pair_supported(const m2_glu_args* a) {
  const int p = a->d_model / a->nblocks, q = 2 * a->inter / a->nblocks;
  return a->dtype == M2_BF16 && a->nblocks % 2 == 0 && p % 64 == 0 && p / 64 <= glup::MAX_KS && q % 128 == 0 &&
         a->ldx % 8 == 0 && a->ldh % 8 == 0 && m2_aligned(a->x, 16) && m2_aligned(a->wg, 16) && m2_aligned(a->h, 16) && a->m >= 1;
}

int glu_pair_launch(const m2_glu_args* a, cudaStream_t st) {
  using namespace glup;
  const int p = a->d_model / a->nblocks, q = 2 * a->inter / a->nblocks;
  CUtensorMap tmA, tmB;
  int rc = m2_make_tmap_bf16_2d(&tmA, a->x, a->m, a->d_model, a->ldx, BM);
  if (rc) return rc;
  rc = m2_make_tmap_bf16_2d(&tmB, a->wg, (uint64_t)a->nblocks * q, p, p, BH);
  if (rc) return rc;
  static int pairs_cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  M2_CUDA(cudaFuncSetAttribute(glu_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
  if (!pairs_cached[dev]) {
    int sms = 148, n = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (sms / 2)); cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = SMEM;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at; cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&n, reinterpret_cast<const void*>(glu_pair_kernel), &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sms / 2;
    }
    pairs_cached[dev] = n;
  }
  Params R;
  R.M = a->m; R.p = p; R.q = q; R.nb_half = a->nblocks / 2; R.ksteps = p / BK; R.ntn = q / BN;
  // column tiles per unit: about 6 units per pair, so that the contiguous ranges balance
  const long long xpairs = (long long)((a->m + 2 * BM - 1) / (2 * BM)) * R.nb_half;
  int gs = R.ntn;
  while (gs > 1 && xpairs * ((R.ntn + gs - 1) / gs) < 6LL * pairs_cached[dev]) gs = (gs + 1) / 2;
  R.gs = gs; R.ngroups = (R.ntn + gs - 1) / gs;
  R.total_units = (int)(xpairs * R.ngroups);
  R.wide_out = m2_aligned(a->h, 32) && a->ldh % 16 == 0 && q % 16 == 0;
  R.out = a->h; R.ldo = a->ldh;
  const int pairs = R.total_units < pairs_cached[dev] ? R.total_units : pairs_cached[dev];
  glu_pair_kernel<<<2 * pairs, THREADS, SMEM, st>>>(tmA, tmB, R);
  M2_LAUNCH_CHECK("glu_pair_kernel");
  return M2_OK;
}

}  // namespace m2
