// Dense linear layers of the sequence mixer (in_linear, out_linear) as bf16 GEMMs on the 5th-generation
// tensor cores, issued for CTA PAIRS: one `tcgen05.mma.cta_group::2` multiplies a 256 x 256 x 16 block whose
// M side is split over the two SMs of a pair (128 rows each, accumulators in each SM's own tensor memory) and
// whose N-side operand is split the other way (each CTA stages 128 of the 256 rows).  A pair therefore moves
// 64 KB through TMA per 64-deep K step for 256 x 256 outputs -- half of what two independent 128 x 256 tiles
// would -- which is what keeps the kernel under the L2 -> shared-memory rate that paces single-CTA tiles.
//
//   y[b, t, n] = sum_k x[b, t, k] * w[n, k] + bias[n]        (nn.Linear, bias added in float32, one rounding)
//
// Three operand arrangements, chosen from the strides of x and out:
//   ROWS      x rows of features (k contiguous), out rows of features: tokens on the M side.
//   CHANNELS  x rows of features, out time-contiguous ((b, n, t) or channel-major (n, b*t)): the WEIGHT rows go
//             on the M side, so a TMEM lane is an output channel and its columns are consecutive tokens --
//             the transposed layout is written with 32-byte stores and nothing is ever transposed in memory.
//   TIMEIN    x time-contiguous ((b, k, t)): the M-side operand is read "MN-major" (tokens contiguous, K strided)
//             straight from that layout through 3-D TMA boxes; out rows of features.
//
// Roles per CTA (640 threads): warp 0 TMA producer, warp 1 MMA issue (leader CTA of the pair only) and tensor-
// memory allocation, warps 4-19 epilogue (TMEM -> registers -> bias -> bf16 -> global).  Two 256-column
// accumulators alternate, so the epilogue of one tile overlaps the MMAs of the next.  Loads of both CTAs
// signal the LEADER's `full` barrier; `tcgen05.commit` multicasts stage-free and accumulator-ready arrivals to
// both CTAs; the peer's epilogue hands accumulators back through a remote mbarrier arrive.  Every wait is
// bounded (tc::mbar_wait); a wait that runs out sets the device status word and the pair winds down.
//
// Computation replaced: nn.Linear at bert/src/mm/monarch_mixer_sequence_mixer.py:81-82, :108 (in_linear,
// followed by the transpose of :109) and :152 (out_linear, after the transpose of :150).
#include "tc_common.cuh"

namespace m2 {
namespace lin {

constexpr int BM = 128;                    // M-side rows per CTA (256 per pair)
constexpr int BNH = 128;                   // N-side rows staged per CTA (UMMA N = 256 per pair)
constexpr int BK = 64;                     // one 128-byte swizzle row of bf16
constexpr int NST = 6;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BNH * BK * 2, STAGE = A_BYTES + B_BYTES;
constexpr int ACC_COLS = 2 * BNH;          // TMEM columns of one accumulator
constexpr int EPI_WARPS = 16, EPI_WARP0 = 4, THREADS = 32 * (EPI_WARP0 + EPI_WARPS);
constexpr int CW = ACC_COLS / (EPI_WARPS / 4);   // accumulator columns per epilogue warp: 64
constexpr int OFF_BAR = NST * STAGE;
constexpr int NBARS = 2 * NST + 4;
constexpr int OFF_BIAS = OFF_BAR + 256;    // float32 copy of the (bf16-rounded) column bias, read by every epilogue thread
constexpr int BIAS_MAX = 6144;
constexpr int SMEM = OFF_BIAS + BIAS_MAX * 4 + 1024;
static_assert(NBARS * 8 + 16 <= 256, "barrier block");
static_assert(SMEM <= 227 * 1024, "shared memory budget");

enum Mode { ROWS = 0, CHANNELS = 1, TIMEIN = 2 };

struct Params {
  int m_rows, n_rows;            // extents of the M-side / N-side operands (rows of the GEMM's A / B)
  int ksteps, m_pairs, n_tiles, total_tiles;
  int L, batch;                  // tokens are (b, t), b < batch, t < L
  int tiles_per_batch, m_tiles;  // TIMEIN: 128-token tiles per batch row, and in all
  int nb, p, q;                  // ROWS only: block-diagonal weight, nb blocks of q outputs x p inputs (dense: nb = 1)
  int n_tile, bh;                // UMMA N of the pair (<= 256) and the N-side rows each CTA stages (n_tile / 2)
  int round_first;               // BlockdiagLinear's arithmetic: the product is rounded to bf16 before the bias is added
  uint32_t idesc;
  int vec;                       // 32-byte stores are legal for every full 16-element chunk
  int flat;                      // CHANNELS: token m lives at m * 1 from the channel's row start (osb == L)
  __nv_bfloat16* out; long long osb, ost, osc;
  const float* bias;
};

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
linear_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params P) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* full = bars;                  // [NST] leader's: both CTAs' loads of the stage have landed
  uint64_t* empty = full + NST;           // [NST] each CTA's: the pair's MMAs have read the stage
  uint64_t* tfull = empty + NST;          // [2]   each CTA's: accumulator complete
  uint64_t* tempty = tfull + 2;           // [2]   leader's: both CTAs' epilogues have drained the accumulator
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = tc::cluster_ctarank();          // 0 = leader of the pair
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) { tc::mbar_init(full + s, 1); tc::mbar_init(empty + s, 1); }
    for (int b = 0; b < 2; ++b) { tc::mbar_init(tfull + b, 1); tc::mbar_init(tempty + b, 2 * EPI_WARPS); }
    *abort_flag = 0;
    tc::mbar_fence_init();
    tc::tma_prefetch_desc(&tmA);
    tc::tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tc::tmem_alloc2(tmem_slot, 512);
    tc::tmem_relinquish2();
  }
  float* sbias = reinterpret_cast<float*>(smem + OFF_BIAS);
  const bool bias_smem = MODE != CHANNELS && P.bias != nullptr && P.n_rows <= BIAS_MAX;
  if (bias_smem)
    for (int i = threadIdx.x; i < ((P.n_rows + 15) & ~15); i += THREADS) sbias[i] = i < P.n_rows ? bf16r(__ldg(P.bias + i)) : 0.f;
  tc::tc_fence_before();
  __syncthreads();
  tc::cluster_sync();                       // the peer's barriers and tensor memory exist before anything touches them
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto decode = [&](int tile, int& mp, int& nt, int& kb) {
    // the weight-side tile index runs fastest, so the pairs working at the same moment share one token tile
    kb = 0;
    if (MODE == CHANNELS) { mp = tile % P.m_pairs; nt = tile / P.m_pairs; }
    else if (MODE == ROWS) { nt = tile % P.n_tiles; const int r = tile / P.n_tiles; kb = r % P.nb; mp = r / P.nb; }
    else { nt = tile % P.n_tiles; mp = tile / P.n_tiles; }
  };

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) -------------------------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < P.total_tiles && ok; tile += npairs) {
        int mp, nt, kb;
        decode(tile, mp, nt, kb);
        const int mt = 2 * mp + (int)rank;
        const int n0 = kb * P.q + nt * P.n_tile + (int)rank * P.bh;
        const int ka = kb * P.p;
        int tb = 0, t0 = 0;
        if (MODE == TIMEIN) {
          tb = mt < P.m_tiles ? mt / P.tiles_per_batch : P.batch;     // past the end: an all-zero (out-of-range) box
          t0 = (mt % P.tiles_per_batch) * BM;
        }
        for (int ks = 0; ks < P.ksteps; ++ks) {
          if (!tc::mbar_wait(empty + stage, phase ^ 1, abort_flag, tc::ST_TIMEOUT_EMPTY)) { ok = false; break; }
          unsigned char* st = smem + stage * STAGE;
          const uint32_t fb = tc::mapa_shared(tc::smem_u32(full + stage), 0);
          if (rank == 0) tc::mbar_expect_tx(full + stage, 2 * (A_BYTES + P.bh * (BK * 2)));
          if (MODE == TIMEIN) {
            tc::tma_load_3d_2sm(st, &tmA, fb, t0, ks * BK, tb);
            tc::tma_load_3d_2sm(st + A_BYTES / 2, &tmA, fb, t0 + 64, ks * BK, tb);
          } else {
            tc::tma_load_2d_2sm(st, &tmA, fb, ka + ks * BK, mt * BM);
          }
          tc::tma_load_2d_2sm(st + A_BYTES, &tmB, fb, ks * BK, n0);
          if (++stage == NST) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issue (leader CTA only) -------------------------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = P.idesc;
      // M-side operand: K-major rows of 128 bytes, or (TIMEIN) MN-major: 64-token chunks 8 KB apart, 8-K groups 1 KB apart
      const uint64_t dA0 = MODE == TIMEIN ? tc::smem_desc_sw128(tc::smem_u32(smem), A_BYTES / 2, 1024)
                                          : tc::smem_desc_k_sw128(tc::smem_u32(smem));
      const uint64_t dB0 = tc::smem_desc_k_sw128(tc::smem_u32(smem + A_BYTES));
      constexpr uint64_t a_step = MODE == TIMEIN ? (16 * 128) >> 4 : 2;      // 16 K rows of 128 bytes, or 32 bytes along a row
      int stage = 0; uint32_t phase = 0;
      int buf = 0; uint32_t bphase = 0;
      bool ok = true;
      for (int tile = pair; tile < P.total_tiles && ok; tile += npairs) {
        if (!tc::mbar_wait(tempty + buf, bphase ^ 1, abort_flag, tc::ST_TIMEOUT_MMA)) break;
        tc::tc_fence_after();
        const uint32_t acc = tmem_base + buf * ACC_COLS;
        for (int ks = 0; ks < P.ksteps; ++ks) {
          if (!tc::mbar_wait(full + stage, phase, abort_flag, tc::ST_TIMEOUT_TMA)) { ok = false; break; }
          tc::tc_fence_after();
          const uint64_t off = (uint64_t)(stage * (STAGE >> 4));
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)
            tc::mma_ss2(acc, dA0 + off + a_step * kk, dB0 + off + 2 * kk, idesc, (ks | kk) ? 1u : 0u);
          tc::mma_commit2_mc(empty + stage, 3);        // both CTAs' stage is free once these MMAs have read it
          if (++stage == NST) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc::mma_commit2_mc(tfull + buf, 3);            // accumulator complete, in both CTAs
        if ((buf ^= 1) == 0) bphase ^= 1;
      }
    }
  } else if (warp >= EPI_WARP0) {
    // ------------------------------- epilogue (both CTAs) -------------------------------
    const int quarter = warp & 3;                 // TMEM lanes 32*quarter .. +31
    const int cs = (warp - EPI_WARP0) >> 2;       // which 64 columns of the accumulator
    const uint32_t tempty_leader = tc::mapa_shared(tc::smem_u32(tempty), 0);
    int buf = 0; uint32_t bphase = 0;
    for (int tile = pair; tile < P.total_tiles; tile += npairs) {
      int mp, nt, kb;
      decode(tile, mp, nt, kb);
      const int mt = 2 * mp + (int)rank;
      if (!tc::mbar_wait(tfull + buf, bphase, abort_flag, tc::ST_TIMEOUT_EPI)) break;
      tc::tc_fence_after();
      const uint32_t tacc = tmem_base + buf * ACC_COLS + ((uint32_t)(quarter * 32) << 16) + cs * CW;
      const bool cols_live = cs * CW < P.n_tile;                 // narrower tiles leave the last column slices idle
      uint32_t acc_r[CW / 16][16];
      if (cols_live) {
#pragma unroll
        for (int ch = 0; ch < CW / 16; ++ch) tc::tmem_ld16(tacc + 16 * ch, acc_r[ch]);
      }
      tc::tmem_ld_wait();
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive_cluster(tempty_leader + 8 * buf);
      const int lrow = mt * BM + quarter * 32 + lane;          // index on the M side
      const int c0 = kb * P.q + nt * P.n_tile + cs * CW;       // first index on the N side
      // columns of this tile that exist: up to the end of the tile, of the block and of the tensor
      int lim = kb * P.q + (nt + 1) * P.n_tile;
      if (MODE == ROWS && lim > (kb + 1) * P.q) lim = (kb + 1) * P.q;
      if (lim > P.n_rows) lim = P.n_rows;
      if (!cols_live) lim = 0;
      if (MODE == CHANNELS) {
        // lane = output channel, columns = consecutive tokens
        const bool live = lrow < P.m_rows;
        const float bv = (live && P.bias) ? bf16r(__ldg(P.bias + lrow)) : 0.f;
#pragma unroll
        for (int ch = 0; ch < CW / 16; ++ch) {
          const int m0 = c0 + 16 * ch;                         // first token of the chunk
          if (!live || m0 >= lim) continue;
          uint32_t packed[8];
#pragma unroll
          for (int j = 0; j < 16; j += 2)
            packed[j >> 1] = pack_bf16(__uint_as_float(acc_r[ch][j]) + bv, __uint_as_float(acc_r[ch][j + 1]) + bv);
          const int b = P.flat ? 0 : m0 / P.L;
          const int t = P.flat ? m0 : m0 - b * P.L;
          __nv_bfloat16* dst = P.out + (long long)b * P.osb + (long long)lrow * P.osc + t;
          if (P.vec && m0 + 16 <= lim) {
            stg256(dst, packed[0], packed[1], packed[2], packed[3], packed[4], packed[5], packed[6], packed[7]);
          } else {
            for (int j = 0; j < 16 && m0 + j < lim; ++j) {
              const int mj = m0 + j, bj = P.flat ? 0 : mj / P.L, tj = P.flat ? mj : mj - bj * P.L;
              const uint32_t w = packed[j >> 1];
              reinterpret_cast<uint16_t*>(P.out)[(long long)bj * P.osb + (long long)lrow * P.osc + tj] =
                  (uint16_t)((j & 1) ? (w >> 16) : (w & 0xffffu));
            }
          }
        }
      } else {
        // lane = token, columns = output features
        int b, t;
        bool live;
        if (MODE == TIMEIN) {
          b = mt / P.tiles_per_batch;
          t = (mt % P.tiles_per_batch) * BM + quarter * 32 + lane;
          live = mt < P.m_tiles && t < P.L;
        } else {
          b = lrow / P.L;
          t = lrow - b * P.L;
          live = lrow < P.m_rows;
        }
        __nv_bfloat16* orow = P.out + (long long)b * P.osb + (long long)t * P.ost;
#pragma unroll
        for (int ch = 0; ch < CW / 16; ++ch) {
          const int n0 = c0 + 16 * ch;
          if (!live || n0 >= lim) continue;
          const bool fullc = n0 + 16 <= lim;
          uint32_t packed[8];
          if (bias_smem) {
            // the staged bias is padded with zeros to a multiple of 16 entries: whole-chunk vector reads
            const float4* bp = reinterpret_cast<const float4*>(sbias + n0);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 bq = bp[q];
              float v0 = __uint_as_float(acc_r[ch][4 * q]), v1 = __uint_as_float(acc_r[ch][4 * q + 1]);
              float v2 = __uint_as_float(acc_r[ch][4 * q + 2]), v3 = __uint_as_float(acc_r[ch][4 * q + 3]);
              if (P.round_first) { v0 = bf16r(v0); v1 = bf16r(v1); v2 = bf16r(v2); v3 = bf16r(v3); }
              packed[2 * q] = pack_bf16(v0 + bq.x, v1 + bq.y);
              packed[2 * q + 1] = pack_bf16(v2 + bq.z, v3 + bq.w);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
              float v0 = __uint_as_float(acc_r[ch][j]), v1 = __uint_as_float(acc_r[ch][j + 1]);
              if (P.round_first) { v0 = bf16r(v0); v1 = bf16r(v1); }
              if (P.bias) {
                if (fullc || n0 + j < lim) v0 += bf16r(__ldg(P.bias + n0 + j));
                if (fullc || n0 + j + 1 < lim) v1 += bf16r(__ldg(P.bias + n0 + j + 1));
              }
              packed[j >> 1] = pack_bf16(v0, v1);
            }
          }
          if (P.vec && fullc) {
            stg256(orow + n0, packed[0], packed[1], packed[2], packed[3], packed[4], packed[5], packed[6], packed[7]);
          } else {
            for (int j = 0; j < 16 && n0 + j < lim; ++j) {
              const uint32_t w = packed[j >> 1];
              reinterpret_cast<uint16_t*>(orow)[n0 + j] = (uint16_t)((j & 1) ? (w >> 16) : (w & 0xffffu));
            }
          }
        }
      }
      if ((buf ^= 1) == 0) bphase ^= 1;
    }
  }

  // ------------------------------- teardown -------------------------------------
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0 && rank == 0) {
    // give loads that were issued before the abort a bounded time to land
    for (int s = 0; s < NST; ++s)
      for (uint32_t i = 0; i < 4096 && !tc::mbar_try_wait(full + s, 0) && !tc::mbar_try_wait(full + s, 1); ++i) {}
  }
  tc::tc_fence_before();
  tc::cluster_sync();                       // nobody leaves while the peer may still signal it or read its operands
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc2(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------
// CUDA-core fallback with float32 accumulation: float32 tensors (the 1e-4 mode) and bf16 shapes the TMA
// path does not take (strides that are not multiples of 8 elements).  Arbitrary element strides.
// ---------------------------------------------------------------------------------------
template <typename T, bool ROUND>
__global__ void __launch_bounds__(256)
linear_simt_kernel(const T* __restrict__ x, long long xsb, long long xst, long long xsc, const T* __restrict__ w,
                   const float* __restrict__ bias, T* __restrict__ out, long long osb, long long ost, long long osc,
                   int batch, int L, int K, int N) {
  constexpr int TS = 64, KC = 16;
  __shared__ float sX[KC][TS + 4], sW[KC][TS + 4];
  const long long tokens = (long long)batch * L;
  const long long r0 = (long long)blockIdx.y * TS;
  const int n0 = blockIdx.x * TS;
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int lr = tid / 4, lk = (tid % 4) * 4;
  float acc[4][4] = {};
  const long long xr = r0 + lr;
  const long long xoff = xr < tokens ? (xr / L) * xsb + (xr % L) * xst : 0;
  for (int k0 = 0; k0 < K; k0 += KC) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      float xv = 0.f, wv = 0.f;
      if (k < K) {
        if (xr < tokens) xv = ld_as_float(x + xoff + (long long)k * xsc);
        if (n0 + lr < N) wv = ld_as_float(w + (long long)(n0 + lr) * K + k);
      }
      sX[lk + e][lr] = xv;
      sW[lk + e][lr] = wv;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = sX[k][ty * 4 + i]; b[i] = sW[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long r = r0 + ty * 4 + i;
    if (r >= tokens) continue;
    const long long ooff = (r / L) * osb + (r % L) * ost;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += rnd<ROUND>(__ldg(bias + n));
      st_from_float(out + ooff + (long long)n * osc, rnd<ROUND>(v));
    }
  }
}

static int max_pairs(const void* kern) {
  // CTA pairs that can be resident at once (one pair per two SMs); cached per device
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!cached[dev]) {
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int n = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (sms / 2));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at; cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = sms / 2; }
    cached[dev] = n;
  }
  return cached[dev];
}

template <int MODE>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const Params& P, cudaStream_t st) {
  auto kern = linear_pair_kernel<MODE>;
  M2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
  const int mp = max_pairs(reinterpret_cast<const void*>(kern));
  const int pairs = P.total_tiles < mp ? P.total_tiles : mp;
  kern<<<2 * pairs, THREADS, SMEM, st>>>(tmA, tmB, P);
  M2_LAUNCH_CHECK("linear_pair_kernel");
  return M2_OK;
}

}  // namespace lin

// 3-D bf16 tensor {d0 (contiguous), d1, d2} with strides s1, s2 in elements, box 64 x 64 x 1, 128-byte swizzle,
// out-of-range elements read as zero: the time-contiguous operand of linear_pair_kernel<TIMEIN>.
static int make_tmap_bf16_3d(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2) {
  m2_encode_tiled_fn enc;
  int rc = m2_get_encode_fn(&enc);
  if (rc) return rc;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1 * 2, s2 * 2};
  cuuint32_t box[3] = {64, 64, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return m2_set_error(M2_ERR_CUDA, "cuTensorMapEncodeTiled (3-D) failed with code %d", (int)r);
  return M2_OK;
}

}  // namespace m2

extern "C" int m2_linear_fwd(const m2_linear_args* a, void* stream) {
  using namespace m2;
  M2_REQUIRE(a != nullptr, M2_ERR_ARG, "m2_linear_fwd: args is NULL");
  M2_REQUIRE(a->batch >= 0 && a->seq_len > 0 && a->in_features > 0 && a->out_features > 0, M2_ERR_ARG,
             "m2_linear_fwd: bad sizes batch=%d seq_len=%d in=%d out=%d", a->batch, a->seq_len, a->in_features, a->out_features);
  if (a->batch == 0) return M2_OK;
  M2_REQUIRE(a->x && a->w && a->out, M2_ERR_ARG, "m2_linear_fwd: NULL tensor pointer");
  M2_REQUIRE(a->dtype == M2_BF16 || a->dtype == M2_F32, M2_ERR_UNSUPPORTED, "m2_linear_fwd: dtype must be float32 or bf16");
  const long long tokens = (long long)a->batch * a->seq_len;
  M2_REQUIRE(tokens < (1LL << 31) - 512, M2_ERR_UNSUPPORTED, "m2_linear_fwd: more than 2^31 tokens");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int L = a->seq_len, K = a->in_features, N = a->out_features;
  const bool x_rows = a->x_sc == 1, x_time = a->x_st == 1 && !x_rows;
  const bool o_rows = a->out_sc == 1, o_time = a->out_st == 1 && !o_rows;
  // what the TMA / tensor-core path needs: 16-byte aligned bases, strides that are multiples of 8 elements
  bool tc_ok = a->dtype == M2_BF16 && !a->force_simt && m2_aligned(a->x, 16) && m2_aligned(a->w, 16) && K % 8 == 0 &&
               (x_rows || x_time) && (o_rows || o_time) && !(x_time && o_time);
  if (tc_ok && x_rows) tc_ok = a->x_st % 8 == 0 && a->x_st >= K && (a->batch == 1 || a->x_sb == (long long)L * a->x_st);
  if (tc_ok && x_time) tc_ok = a->x_sc % 8 == 0 && a->x_sb % 8 == 0 && a->x_sc >= L;
  if (!tc_ok) {
    dim3 grid((N + 63) / 64, (unsigned)((tokens + 63) / 64));
    M2_REQUIRE(grid.y <= 65535, M2_ERR_UNSUPPORTED, "m2_linear_fwd: too many tokens for the CUDA-core kernel");
    if (a->dtype == M2_BF16)
      lin::linear_simt_kernel<__nv_bfloat16, true><<<grid, 256, 0, st>>>(
          (const __nv_bfloat16*)a->x, a->x_sb, a->x_st, a->x_sc, (const __nv_bfloat16*)a->w, a->bias, (__nv_bfloat16*)a->out,
          a->out_sb, a->out_st, a->out_sc, a->batch, L, K, N);
    else
      lin::linear_simt_kernel<float, false><<<grid, 256, 0, st>>>(
          (const float*)a->x, a->x_sb, a->x_st, a->x_sc, (const float*)a->w, a->bias, (float*)a->out,
          a->out_sb, a->out_st, a->out_sc, a->batch, L, K, N);
    M2_LAUNCH_CHECK("linear_simt_kernel");
    return M2_OK;
  }
  using namespace lin;
  Params P;
  memset(&P, 0, sizeof(P));
  P.L = L; P.batch = a->batch; P.ksteps = (K + BK - 1) / BK;
  P.out = (__nv_bfloat16*)a->out; P.osb = a->out_sb; P.ost = a->out_st; P.osc = a->out_sc; P.bias = a->bias;
  CUtensorMap tmA, tmB;
  int rc;
  if (x_rows && o_time) {                                     // CHANNELS: weight rows on the M side
    P.m_rows = N; P.n_rows = (int)tokens;
    if ((rc = m2_make_tmap_bf16_2d(&tmA, a->w, (uint64_t)N, (uint64_t)K, (uint64_t)K, BM))) return rc;
    if ((rc = m2_make_tmap_bf16_2d(&tmB, a->x, (uint64_t)tokens, (uint64_t)K, (uint64_t)a->x_st, BNH))) return rc;
    P.flat = a->batch == 1 || a->out_sb == L;
    P.vec = m2_aligned(a->out, 32) && a->out_sc % 16 == 0 && (P.flat || (L % 16 == 0 && a->out_sb % 16 == 0));
  } else {
    P.n_rows = N;
    if ((rc = m2_make_tmap_bf16_2d(&tmB, a->w, (uint64_t)N, (uint64_t)K, (uint64_t)K, BNH))) return rc;
    if (x_rows) {                                             // ROWS
      P.m_rows = (int)tokens;
      if ((rc = m2_make_tmap_bf16_2d(&tmA, a->x, (uint64_t)tokens, (uint64_t)K, (uint64_t)a->x_st, BM))) return rc;
    } else {                                                  // TIMEIN
      P.tiles_per_batch = (L + BM - 1) / BM;
      P.m_tiles = P.tiles_per_batch * a->batch;
      P.m_rows = P.m_tiles * BM;
      if ((rc = make_tmap_bf16_3d(&tmA, a->x, (uint64_t)L, (uint64_t)K, (uint64_t)a->batch, (uint64_t)a->x_sc,
                                  (uint64_t)(a->batch == 1 ? a->x_sc * (long long)K : a->x_sb)))) return rc;
    }
    P.vec = m2_aligned(a->out, 32) && a->out_st % 16 == 0 && a->out_sb % 16 == 0;
  }
  P.nb = 1; P.p = K; P.q = P.n_rows; P.n_tile = 2 * BNH; P.bh = BNH; P.round_first = 0;
  P.idesc = tc::make_idesc_major(2 * BM, P.n_tile, 1, x_time ? 1 : 0, 0);
  P.m_pairs = (P.m_rows + 2 * BM - 1) / (2 * BM);
  P.n_tiles = (P.n_rows + P.n_tile - 1) / P.n_tile;
  P.total_tiles = P.m_pairs * P.n_tiles;
  if (x_rows && o_time) return launch<CHANNELS>(tmA, tmB, P, st);
  if (x_rows) return launch<ROWS>(tmA, tmB, P, st);
  return launch<TIMEIN>(tmA, tmB, P, st);
}

namespace m2 {
// BlockdiagLinear on the CTA-pair kernel: out[:, k q + n] = x[:, k p : (k+1) p] . w[k][n, :] (+ bias), the product
// rounded to bf16 before the (bf16-rounded) bias is added, as BlockdiagMultiply + StructuredLinear do under autocast
// (bert/src/mm/blockdiag_multiply.py:49-60, bert/src/mm/structured_linear.py:67-70).
bool blockdiag_pair_supported(const m2_blockdiag_args* a) {
  return a->dtype == M2_BF16 && a->p % 64 == 0 && a->q % 16 == 0 && a->in_features == a->nblocks * a->p &&
         a->out_features == a->nblocks * a->q && a->out_features <= lin::BIAS_MAX && a->ldx % 8 == 0 && a->ldo % 8 == 0 &&
         m2_aligned(a->x, 16) && m2_aligned(a->w, 16) && m2_aligned(a->out, 16) && a->m >= 1;
}

int blockdiag_pair_launch(const m2_blockdiag_args* a, cudaStream_t st) {
  using namespace lin;
  Params P;
  memset(&P, 0, sizeof(P));
  P.L = a->m; P.batch = 1; P.ksteps = a->p / BK;
  P.out = (__nv_bfloat16*)a->out; P.osb = 0; P.ost = a->ldo; P.osc = 1; P.bias = a->bias;
  P.m_rows = a->m; P.n_rows = a->out_features;
  P.nb = a->nblocks; P.p = a->p; P.q = a->q; P.round_first = 1;
  P.n_tile = a->q >= 2 * BNH ? 2 * BNH : ((a->q + 31) / 32) * 32;
  P.bh = P.n_tile / 2;
  P.idesc = tc::make_idesc_major(2 * BM, P.n_tile, 1, 0, 0);
  P.vec = m2_aligned(a->out, 32) && a->ldo % 16 == 0;
  CUtensorMap tmA, tmB;
  int rc;
  if ((rc = m2_make_tmap_bf16_2d(&tmA, a->x, (uint64_t)a->m, (uint64_t)a->in_features, (uint64_t)a->ldx, BM))) return rc;
  if ((rc = m2_make_tmap_bf16_2d(&tmB, a->w, (uint64_t)a->nblocks * a->q, (uint64_t)a->p, (uint64_t)a->p, (uint32_t)P.bh))) return rc;
  P.m_pairs = (P.m_rows + 2 * BM - 1) / (2 * BM);
  P.n_tiles = (a->q + P.n_tile - 1) / P.n_tile;
  P.total_tiles = P.m_pairs * P.nb * P.n_tiles;
  return launch<ROWS>(tmA, tmB, P, st);
}
}  // namespace m2
