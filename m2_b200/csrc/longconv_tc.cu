// Fused gated long convolution on tcgen05 tensor cores, sequence lengths 64 < L <= 128
// (transform length N = 256), bf16 activations (kernel family 1).
//
// The length-256 real FFT is evaluated at the odd frequencies k + 1/2 (which turns the
// circular convolution into a negacyclic one -- the wrapped half of the filter is negated
// when its spectrum is built -- and leaves no self-paired DC/Nyquist bins), factored
// Monarch style as N = 32 x 8 with n = 8 n1 + n2, k = k1 + 32 k2:
//
//   F1  B1[k1, n2] = sum_{n1<16} W32^{n1 (k1+1/2)} a[8 n1 + n2]          real -> complex,
//       only k1 < 16 (the other half is the complex conjugate) and n1 < 16 (zero padding)
//   F2  Z[k1, k2]  = sum_{n2} w^{n2 (k1+1/2)} W8^{n2 k2} B1[k1, n2]      twiddle folded in
//   x   Y = Z * (G + bias)                                                filter spectrum
//   I2  D[k1, n2]  = w^{-n2 (k1+1/2)} sum_{k2} W8^{-n2 k2} Y[k1, k2]
//   I1  y[8 n1+n2] = (2/N) Re sum_{k1<16} W32^{-n1 (k1+1/2)} D[k1, n2]   n1 < 16 only
//
// Each stage is a batch of small real GEMMs with M = 128 channels (one row per TMEM lane),
// K = 16 and N = 16 or 32: the data (fp16, exact for bf16 inputs) is the A operand in
// shared memory, the constant DFT matrices are the B operands, accumulators live in tensor
// memory.  Between stages each channel's row stays with the same thread, which re-lays it
// out for the next stage (TMEM -> registers -> shared memory), so no cross-thread transpose
// and no bit reversal exist.  The conv bias term u*D is folded into the spectrum (+bias on
// every bin).  A CTA processes one (batch row, 128-channel tile) at a time; two CTAs share
// an SM so one's CUDA-core phases overlap the other's MMAs and memory traffic.
//
// Computation replaced: bert/src/mm/monarch_mixer_sequence_mixer.py:109-149 and
// bert/src/mm/hyena_utils.py:16-42, :219-248 of the reference.
#include "tc_common.cuh"

namespace m2 {
namespace lc {

constexpr int NFFT = 256;
constexpr int CT = 128;                    // channels per unit
constexpr int THREADS = 256;
constexpr int TILE = 4096;                 // one [128 x 16] fp16 A-operand tile
constexpr int H_BYTES = 16 * TILE;         // 64 KB: operand tiles, later the float32 y tile
constexpr int F1_OFF = 0, F2_OFF = 1024, I2_OFF = F2_OFF + 8192, I1_OFF = I2_OFF + 8192;
constexpr int MAT_BYTES = I1_OFF + 1024;   // 18 KB of constant DFT matrices (fp16)
constexpr int MAT_FLOATS = MAT_BYTES / 4;
constexpr float S1 = 0.25f, S2 = 0.5f, S3 = 0.5f, S4 = 0.25f;   // per-stage scalings (exact powers of two)
constexpr float KAPPA = (2.0f / NFFT) / (S1 * S2 * S3 * S4);     // folded into the filter table
// core-matrix strides of every operand tile: LBO between the two K halves, SBO between 8-row groups
constexpr uint32_t LBO = 128, SBO = 256;

// byte offset of element (row, k) in a K-major un-swizzled tile with 16 K columns
__host__ __device__ constexpr int tile_off(int row, int k) {
  return (row >> 3) * 256 + (k >> 3) * 128 + (row & 7) * 16 + (k & 7) * 2;
}

// ---------------------------------------------------------------------------------------
// Spectrum table (kind 1): [MAT_FLOATS floats: the fp16 matrices] then per channel
// G[k1][k2] as half2 (re, im), k1 < 16, k2 < 8, already multiplied by KAPPA.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
spectrum_kind1_kernel(const float* __restrict__ kfilt, float* __restrict__ spec, int D, int L) {
  const int tid = threadIdx.x;
  if (blockIdx.x == (unsigned)D) {
    __half* m = reinterpret_cast<__half*>(spec);
    // F1: row j = 16h + 8g + 4ri + kq  <->  k1 = 8h + 4g + kq ; column n1
    for (int idx = tid; idx < 32 * 16; idx += blockDim.x) {
      const int j = idx / 16, n1 = idx % 16;
      const int h = j >> 4, g = (j >> 3) & 1, ri = (j >> 2) & 1, kq = j & 3;
      const int k1 = 8 * h + 4 * g + kq;
      double sn, cs;
      sincospi(2.0 * n1 * (k1 + 0.5) / 32.0, &sn, &cs);          // W32^{n1(k1+1/2)} = cs - i sn
      m[(F1_OFF + tile_off(j, n1)) / 2] = __double2half((double)S1 * (ri ? -sn : cs));
    }
    // F2[k1] / I2[k1]: 16 x 16 real forms of the twiddled 8-point complex DFTs
    for (int idx = tid; idx < 16 * 8 * 8; idx += blockDim.x) {
      const int k1 = idx / 64, k2 = (idx / 8) % 8, n2 = idx % 8;
      double sn, cs;
      sincospi(2.0 * (n2 * (k1 + 0.5) / 256.0 + n2 * k2 / 8.0), &sn, &cs);   // forward coefficient c + i s, s = -sn
      const double c = cs, s = -sn;
      __half* f2 = m + (F2_OFF + k1 * 512) / 2;
      f2[tile_off(k2, n2) / 2] = __double2half(S2 * c);
      f2[tile_off(k2, 8 + n2) / 2] = __double2half(-S2 * s);
      f2[tile_off(8 + k2, n2) / 2] = __double2half(S2 * s);
      f2[tile_off(8 + k2, 8 + n2) / 2] = __double2half(S2 * c);
      const double ci = cs, si = sn;                               // conjugate coefficient
      __half* i2 = m + (I2_OFF + k1 * 512) / 2;
      i2[tile_off(n2, k2) / 2] = __double2half(S3 * ci);
      i2[tile_off(n2, 8 + k2) / 2] = __double2half(-S3 * si);
      i2[tile_off(8 + n2, k2) / 2] = __double2half(S3 * si);
      i2[tile_off(8 + n2, 8 + k2) / 2] = __double2half(S3 * ci);
    }
    // I1[ri]: rows n1, columns k1:  cos, then -sin, of 2 pi n1 (k1+1/2) / 32
    for (int idx = tid; idx < 2 * 16 * 16; idx += blockDim.x) {
      const int ri = idx / 256, n1 = (idx / 16) % 16, k1 = idx % 16;
      double sn, cs;
      sincospi(2.0 * n1 * (k1 + 0.5) / 32.0, &sn, &cs);
      m[(I1_OFF + ri * 512 + tile_off(n1, k1)) / 2] = __double2half((double)S4 * (ri ? -sn : cs));
    }
    return;
  }
  // one bin per thread: G[k] = KAPPA * sum_n g[n] w^{n (k + 1/2)}, g = filter with its wrapped half negated
  const int c = blockIdx.x;
  const int k1 = tid >> 3, k2 = tid & 7;
  const int k = k1 + 32 * k2;
  const float* row = kfilt + (size_t)c * NFFT;
  double re = 0.0, im = 0.0;
  for (int n = 0; n < NFFT; ++n) {
    double sn, cs;
    sincospi(2.0 * n * (k + 0.5) / NFFT, &sn, &cs);
    const double g = (n < NFFT / 2) ? (double)row[n] : -(double)row[n];
    re += g * cs;
    im -= g * sn;
  }
  __half2* G = reinterpret_cast<__half2*>(spec + MAT_FLOATS) + (size_t)c * 128;
  G[k1 * 8 + k2] = __floats2half2_rn((float)(re * KAPPA), (float)(im * KAPPA));
}

// ---------------------------------------------------------------------------------------
struct Params {
  int B, L, D, nf, units, ctiles;
  int prefetch_ok;   // rows are 16-byte aligned, so bulk L2 prefetches are legal
  const __nv_bfloat16* xin; long long xsb, xst;
  const void* u; long long usb, ust;
  __nv_bfloat16* out; long long osb, ost;
  const float* sw; const float* sb;
  const float* spec[2]; const float* bias[2];
};

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}

// depthwise 3-tap conv of a channel pair at one time step, both channels at once in packed
// float32 pairs; wa, wb hold x[t-2], x[t-1]
struct Taps { f32x2 w0, w1, w2, b; };
__device__ __forceinline__ void load_taps(Taps& T, const float* sw, const float* sb, int ch) {
  T.w0 = f2_pack(bf16r(__ldg(sw + 3 * ch)), bf16r(__ldg(sw + 3 * ch + 3)));
  T.w1 = f2_pack(bf16r(__ldg(sw + 3 * ch + 1)), bf16r(__ldg(sw + 3 * ch + 4)));
  T.w2 = f2_pack(bf16r(__ldg(sw + 3 * ch + 2)), bf16r(__ldg(sw + 3 * ch + 5)));
  T.b = f2_pack(bf16r(__ldg(sb + ch)), bf16r(__ldg(sb + ch + 1)));
}
__device__ __forceinline__ f32x2 bf2_to_f2(uint32_t u) { return f2_pack(bf_lo(u), bf_hi(u)); }
__device__ __forceinline__ uint32_t f2_to_bf2(f32x2 v) {
  float lo, hi;
  f2_unpack(v, lo, hi);
  return pack_bf2(lo, hi);
}
// returns the bf16-rounded conv outputs of both channels packed as bf16x2 and slides the window
__device__ __forceinline__ uint32_t conv_step(const Taps& T, f32x2& wa, f32x2& wb, uint32_t xpair) {
  const f32x2 x = bf2_to_f2(xpair);
  const f32x2 c = f2_fma(T.w2, x, f2_fma(T.w1, wb, f2_fma(T.w0, wa, T.b)));
  wa = wb; wb = x;
  return f2_to_bf2(c);
}

// MMAs of one stage, issued by a single thread once every operand tile is in shared memory.
__device__ __forceinline__ void issue_stage(int stage, uint32_t tmem, uint32_t Hs, uint32_t Ms) {
  constexpr uint32_t id32 = tc::make_idesc(128, 32, 0), id16 = tc::make_idesc(128, 16, 0);
  // every tile lies within the first 256 KB of shared memory, so adding a tile offset (in
  // 16-byte units) to the descriptor never carries out of its 14-bit address field
  const uint64_t dH = tc::smem_desc_k_nosw(Hs, LBO, SBO);
  const uint64_t dM = tc::smem_desc_k_nosw(Ms, LBO, SBO);
  if (stage == 0) {
#pragma unroll
    for (int n2 = 0; n2 < 8; ++n2)
      tc::mma_ss(tmem + 32 * n2, dH + n2 * (TILE >> 4), dM + (F1_OFF >> 4), id32, 0);
  } else if (stage == 1 || stage == 2) {
    const uint64_t dB = dM + ((stage == 1 ? F2_OFF : I2_OFF) >> 4);
#pragma unroll
    for (int k1 = 0; k1 < 16; ++k1)
      tc::mma_ss(tmem + 16 * k1, dH + k1 * (TILE >> 4), dB + k1 * (512 >> 4), id16, 0);
  } else {
#pragma unroll
    for (int n2 = 0; n2 < 8; ++n2) {
      tc::mma_ss(tmem + 16 * n2, dH + (2 * n2) * (TILE >> 4), dM + (I1_OFF >> 4), id16, 0);
      tc::mma_ss(tmem + 16 * n2, dH + (2 * n2 + 1) * (TILE >> 4), dM + ((I1_OFF + 512) >> 4), id16, 1);
    }
  }
}

template <typename TU>
__global__ void __launch_bounds__(THREADS, 2)
longconv_tc128_kernel(const Params P) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
  unsigned char* Hb = smem;                            // operand tiles / y tile
  unsigned char* Mb = smem + H_BYTES;                  // DFT matrices
  uint64_t* bar_ops = reinterpret_cast<uint64_t*>(Mb + MAT_BYTES);   // operand tiles written (256 arrivals)
  uint64_t* bar_mma = bar_ops + 1;                                    // stage's MMAs complete (commit)
  uint64_t* bar_w = bar_ops + 2;                                      // workers <-> workers (256)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_ops + 3);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    tc::mbar_init(bar_ops, THREADS);
    tc::mbar_init(bar_mma, 1);
    tc::mbar_init(bar_w, THREADS);
    *abort_flag = 0;
    tc::mbar_fence_init();
  }
  {  // constant matrices: global (spectrum header of filter 0) -> shared
    const uint4* src = reinterpret_cast<const uint4*>(P.spec[0]);
    uint4* dst = reinterpret_cast<uint4*>(Mb);
    for (int i = tid; i < MAT_BYTES / 16; i += THREADS) dst[i] = __ldg(src + i);
    tc::fence_proxy_async_smem();
  }
  if (warp == 0) {
    tc::tmem_alloc(tmem_slot, 256);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t Hs = tc::smem_u32(Hb), Ms = tc::smem_u32(Mb);

  const int quarter = warp & 3, half = warp >> 2;
  const int r = quarter * 32 + lane;                         // TMEM lane = channel within the tile
  const uint32_t tlane = tmem + ((uint32_t)(quarter * 32) << 16);
  const uint32_t rowoff = (uint32_t)((r >> 3) * 256 + (r & 7) * 16);
  const int pi = tid & 63, tq = tid >> 6;                    // channel pair, quarter of the time axis
  const int t_begin = 32 * tq;
  const uint32_t prow0 = (uint32_t)(((2 * pi) >> 3) * 256 + ((2 * pi) & 7) * 16);   // row 2pi; row 2pi+1 is +16
  const uint32_t pkoff = (uint32_t)((tq >> 1) * 128 + (tq & 1) * 8);                 // n1 = 4 tq + i
  uint32_t ph_ops = 0, ph_mma = 0, ph_w = 0;
  bool ok = true;

  // operand tiles are complete: thread 0 issues the stage's MMAs, everybody waits for them
#define LC_STAGE(stage_)                                                                              \
  tc::fence_proxy_async_smem();                                                                       \
  tc::mbar_arrive(bar_ops);                                                                           \
  if (tid == 0) {                                                                                     \
    if (tc::mbar_wait(bar_ops, ph_ops, abort_flag, tc::ST_TIMEOUT_MMA)) {                             \
      tc::tc_fence_after();                                                                           \
      issue_stage(stage_, tmem, Hs, Ms);                                                    \
      tc::mma_commit(bar_mma);                                                                        \
    }                                                                                                 \
    ph_ops ^= 1;                                                                                      \
  }                                                                                                   \
  if (!__all_sync(0xffffffffu, tc::mbar_wait(bar_mma, ph_mma, abort_flag, tc::ST_TIMEOUT_EPI))) { ok = false; break; } \
  ph_mma ^= 1;                                                                                        \
  tc::tc_fence_after();

#define LC_WORKER_BARRIER()                                                                           \
  tc::mbar_arrive(bar_w);                                                                             \
  if (!__all_sync(0xffffffffu, tc::mbar_wait(bar_w, ph_w, abort_flag, tc::ST_TIMEOUT_EPI))) { ok = false; break; } \
  ph_w ^= 1;

  for (int unit = blockIdx.x; unit < P.units && ok; unit += gridDim.x) {
    const int ct = unit % P.ctiles, b = unit / P.ctiles;
    const int c0 = ct * CT;
    const int ch = c0 + 2 * pi;
    const __nv_bfloat16* xb = P.xin + (long long)b * P.xsb + ch;
    __nv_bfloat16* ob = P.out + (long long)b * P.osb + ch;

    // pull the next unit's input rows into L2 while this one is computed
    if (P.prefetch_ok && unit + (int)gridDim.x < P.units) {
      const int nxt = unit + gridDim.x;
      const int nct = nxt % P.ctiles, nb = nxt / P.ctiles;
      const __nv_bfloat16* nx = P.xin + (long long)nb * P.xsb + nct * CT;
      const char* nu = reinterpret_cast<const char*>(P.u) + ((long long)nb * P.usb + nct * CT) * (long long)sizeof(TU);
      for (int i = tid; i < P.L * 4; i += THREADS) {
        const int t = i >> 2, which = i & 3;
        if (which < 3) {
          const void* ptr = nx + (long long)t * P.xst + which * P.D;
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ptr), "r"(CT * 2) : "memory");
        } else if (P.nf == 2) {
          const void* ptr = nu + (long long)t * P.ust * (long long)sizeof(TU);
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ptr), "r"((int)(CT * sizeof(TU))) : "memory");
        }
      }
    }

    for (int f = 0; f < P.nf && ok; ++f) {
      // ---------------- operand tiles of stage F1: a[t] as fp16, tile n2 = t % 8, k = t / 8 ----------------
      {
        uint32_t hv[2][8][2];                              // [row][n2][two packed pairs over i]
        if (f == 0) {
          Taps Tx, Tv;
          load_taps(Tx, P.sw, P.sb, ch);
          load_taps(Tv, P.sw, P.sb, 2 * P.D + ch);
          // every load of the pass is issued before the first is consumed
          uint32_t lx[34], lv[34];
#pragma unroll
          for (int j = 0; j < 34; ++j) {
            const int t = t_begin - 2 + j;
            lx[j] = lv[j] = 0;
            if (t >= 0 && t < P.L) {
              lx[j] = __ldg(reinterpret_cast<const uint32_t*>(xb + (long long)t * P.xst));
              lv[j] = __ldg(reinterpret_cast<const uint32_t*>(xb + 2 * P.D + (long long)t * P.xst));
            }
          }
          f32x2 xa = bf2_to_f2(lx[0]), xbw = bf2_to_f2(lx[1]), va = bf2_to_f2(lv[0]), vbw = bf2_to_f2(lv[1]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t cx = conv_step(Tx, xa, xbw, lx[2 + 8 * i + j]);
              const uint32_t cv = conv_step(Tv, va, vbw, lv[2 + 8 * i + j]);
              const uint32_t pr = f2_to_bf2(f2_mul(bf2_to_f2(cv), bf2_to_f2(cx)));
              const bool live = (t_begin + 8 * i + j) < P.L;
              const float a0 = live ? bf_lo(pr) : 0.f, a1 = live ? bf_hi(pr) : 0.f;
              if ((i & 1) == 0) {
                hv[0][j][i >> 1] = __float_as_uint(a0);
                hv[1][j][i >> 1] = __float_as_uint(a1);
              } else {
                hv[0][j][i >> 1] = pack_h2(__uint_as_float(hv[0][j][i >> 1]), a0);
                hv[1][j][i >> 1] = pack_h2(__uint_as_float(hv[1][j][i >> 1]), a1);
              }
            }
          }
        } else {
          const TU* up = reinterpret_cast<const TU*>(P.u) + (long long)b * P.usb + ch;
#pragma unroll
          for (int ii = 0; ii < 4; ii += 2) {
            float u0[16], u1[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = t_begin + 8 * ii + j;
              u0[j] = u1[j] = 0.f;
              if (t < P.L) {
                if (sizeof(TU) == 4) {
                  const float2 v = __ldg(reinterpret_cast<const float2*>(up + (long long)t * P.ust));
                  u0[j] = v.x; u1[j] = v.y;
                } else {
                  const uint32_t v = __ldg(reinterpret_cast<const uint32_t*>(up + (long long)t * P.ust));
                  u0[j] = bf_lo(v); u1[j] = bf_hi(v);
                }
              }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {                  // elements i = ii (t = 8 ii + j) and i = ii + 1
              hv[0][j][ii >> 1] = pack_h2(u0[j], u0[8 + j]);
              hv[1][j][ii >> 1] = pack_h2(u1[j], u1[8 + j]);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          sts64(Hs + j * TILE + prow0 + pkoff, hv[0][j][0], hv[0][j][1]);
          sts64(Hs + j * TILE + prow0 + 16 + pkoff, hv[1][j][0], hv[1][j][1]);
        }
      }
      LC_STAGE(0)

      // ---------------- hop 1: F1 result -> operand tiles of F2 ----------------
#pragma unroll 1
      for (int g = 0; g < 2; ++g) {
        uint32_t pk[8][4];                                  // [ri*4+kq][n2 pair]
#pragma unroll
        for (int np = 0; np < 4; np += 2) {
          uint32_t e[8], o[8], e2[8], o2[8];
          tmem_ld8(tlane + 32 * (2 * np) + 16 * half + 8 * g, e);
          tmem_ld8(tlane + 32 * (2 * np + 1) + 16 * half + 8 * g, o);
          tmem_ld8(tlane + 32 * (2 * np + 2) + 16 * half + 8 * g, e2);
          tmem_ld8(tlane + 32 * (2 * np + 3) + 16 * half + 8 * g, o2);
          tc::tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            pk[q][np] = pack_h2(__uint_as_float(e[q]), __uint_as_float(o[q]));
            pk[q][np + 1] = pack_h2(__uint_as_float(e2[q]), __uint_as_float(o2[q]));
          }
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int ri = q >> 2, kq = q & 3;
          const int k1 = 8 * half + 4 * g + kq;
          sts128(Hs + k1 * TILE + rowoff + ri * 128, pk[q][0], pk[q][1], pk[q][2], pk[q][3]);
        }
      }
      // filter values of hop 2 are independent of the data: fetch them before waiting on the MMAs
      const uint4* G = reinterpret_cast<const uint4*>(P.spec[f] + MAT_FLOATS) + ((size_t)(c0 + r) * 16 + 8 * half) * 2;
      uint4 gq[4][2];
#pragma unroll
      for (int kl = 0; kl < 4; ++kl) { gq[kl][0] = __ldg(G + 2 * kl); gq[kl][1] = __ldg(G + 2 * kl + 1); }
      const float bk = __ldg(P.bias[f] + c0 + r) * KAPPA;
      tc::tc_fence_before();
      LC_STAGE(1)

      // ---------------- hop 2: spectrum x filter -> operand tiles of I2 ----------------
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) {
        if (kb == 1) {
#pragma unroll
          for (int kl = 0; kl < 4; ++kl) { gq[kl][0] = __ldg(G + 8 + 2 * kl); gq[kl][1] = __ldg(G + 8 + 2 * kl + 1); }
        }
#pragma unroll
        for (int kl = 0; kl < 4; ++kl) {
          const int k1 = 8 * half + 4 * kb + kl;
          uint32_t z[16];
          tc::tmem_ld16(tlane + 16 * k1, z);
          tc::tmem_ld_wait();
          const uint32_t gw[8] = {gq[kl][0].x, gq[kl][0].y, gq[kl][0].z, gq[kl][0].w,
                                  gq[kl][1].x, gq[kl][1].y, gq[kl][1].z, gq[kl][1].w};
          float yr[8], yi[8];
#pragma unroll
          for (int k2 = 0; k2 < 8; ++k2) {
            const float2 gg = __half22float2(*reinterpret_cast<const __half2*>(&gw[k2]));
            const float gr = gg.x + bk, gi = gg.y;
            const float zr = __uint_as_float(z[k2]), zi = __uint_as_float(z[8 + k2]);
            yr[k2] = zr * gr - zi * gi;
            yi[k2] = zr * gi + zi * gr;
          }
          sts128(Hs + k1 * TILE + rowoff, pack_h2(yr[0], yr[1]), pack_h2(yr[2], yr[3]), pack_h2(yr[4], yr[5]),
                 pack_h2(yr[6], yr[7]));
          sts128(Hs + k1 * TILE + rowoff + 128, pack_h2(yi[0], yi[1]), pack_h2(yi[2], yi[3]),
                 pack_h2(yi[4], yi[5]), pack_h2(yi[6], yi[7]));
        }
      }
      tc::tc_fence_before();
      LC_STAGE(2)

      // ---------------- hop 3: I2 result -> operand tiles of I1 (tile 2 n2 + ri, k = k1) ----------------
#pragma unroll 1
      for (int ri = 0; ri < 2; ++ri) {
        uint32_t pk[8][4];                                  // [n2][k1 pair]
#pragma unroll
        for (int kp = 0; kp < 4; kp += 2) {
          uint32_t e[8], o[8], e2[8], o2[8];
          tmem_ld8(tlane + 16 * (8 * half + 2 * kp) + 8 * ri, e);
          tmem_ld8(tlane + 16 * (8 * half + 2 * kp + 1) + 8 * ri, o);
          tmem_ld8(tlane + 16 * (8 * half + 2 * kp + 2) + 8 * ri, e2);
          tmem_ld8(tlane + 16 * (8 * half + 2 * kp + 3) + 8 * ri, o2);
          tc::tmem_ld_wait();
#pragma unroll
          for (int n2 = 0; n2 < 8; ++n2) {
            pk[n2][kp] = pack_h2(__uint_as_float(e[n2]), __uint_as_float(o[n2]));
            pk[n2][kp + 1] = pack_h2(__uint_as_float(e2[n2]), __uint_as_float(o2[n2]));
          }
        }
#pragma unroll
        for (int n2 = 0; n2 < 8; ++n2)
          sts128(Hs + (2 * n2 + ri) * TILE + rowoff + half * 128, pk[n2][0], pk[n2][1], pk[n2][2], pk[n2][3]);
      }
      tc::tc_fence_before();
      LC_STAGE(3)

      // ---------------- hop 4: y (float32) -> shared [t][channel] ----------------
      {
        float* Y = reinterpret_cast<float*>(Hb);
#pragma unroll 1
        for (int nn = 0; nn < 4; nn += 2) {
          const int n2 = 4 * half + nn;
          uint32_t v[16], w[16];
          tc::tmem_ld16(tlane + 16 * n2, v);
          tc::tmem_ld16(tlane + 16 * (n2 + 1), w);
          tc::tmem_ld_wait();
#pragma unroll
          for (int n1 = 0; n1 < 16; ++n1) {
            Y[(8 * n1 + n2) * CT + r] = __uint_as_float(v[n1]);
            Y[(8 * n1 + n2 + 1) * CT + r] = __uint_as_float(w[n1]);
          }
        }
      }
      // the gate's inputs (f == 0) or the partial result (f == 1) can be fetched while the others finish
      uint32_t gl[34];
      if (f == 0) {
#pragma unroll
        for (int j = 0; j < 34; ++j) {
          const int t = t_begin - 2 + j;
          gl[j] = 0;
          if (t >= 0 && t < P.L) gl[j] = __ldg(reinterpret_cast<const uint32_t*>(xb + P.D + (long long)t * P.xst));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int t = t_begin + j;
          gl[j] = 0;
          if (t < P.L) gl[j] = *reinterpret_cast<const uint32_t*>(ob + (long long)t * P.ost);   // written by this thread
        }
      }
      tc::tc_fence_before();
      LC_WORKER_BARRIER()

      // ---------------- epilogue: gate / residual add, coalesced bf16 stores ----------------
      {
        const float2* Y2 = reinterpret_cast<const float2*>(Hb);
        if (f == 0) {
          Taps T2;
          load_taps(T2, P.sw, P.sb, P.D + ch);
          f32x2 ga = bf2_to_f2(gl[0]), gb = bf2_to_f2(gl[1]);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int t = t_begin + j;
            const uint32_t c2 = conv_step(T2, ga, gb, gl[j + 2]);
            const float2 y = Y2[t * (CT / 2) + pi];
            const uint32_t yr = pack_bf2(y.x, y.y);          // conv + bias term, cast to bf16
            const uint32_t res = f2_to_bf2(f2_mul(bf2_to_f2(yr), bf2_to_f2(c2)));
            if (t < P.L) *reinterpret_cast<uint32_t*>(ob + (long long)t * P.ost) = res;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int t = t_begin + j;
            float2 y = Y2[t * (CT / 2) + pi];
            if (sizeof(TU) == 2) {                           // bf16 layer input: yu is cast to bf16 first
              const uint32_t yr = pack_bf2(y.x, y.y);
              y.x = bf_lo(yr); y.y = bf_hi(yr);
            }
            if (t < P.L)
              *reinterpret_cast<uint32_t*>(ob + (long long)t * P.ost) = pack_bf2(bf_lo(gl[j]) + y.x, bf_hi(gl[j]) + y.y);
          }
        }
      }
      LC_WORKER_BARRIER()                                    // the y tile is free again
    }
  }
#undef LC_STAGE
#undef LC_WORKER_BARRIER

  __syncthreads();
  if (warp == 0) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, 256);
  }
}

constexpr size_t SMEM_BYTES = H_BYTES + MAT_BYTES + 64 + 128;

}  // namespace lc


int longconv_tc_supported(int seq_len, m2_dtype act_dtype, int d_model) {
  return act_dtype == M2_BF16 && seq_len > 64 && seq_len <= 128 && d_model % lc::CT == 0;
}

size_t spectrum_kind1_floats(int D, int L) {
  (void)L;
  return (size_t)lc::MAT_FLOATS + (size_t)128 * D;
}

int spectrum_kind1_launch(int D, int L, const float* k, float* spec, cudaStream_t st) {
  M2_REQUIRE(L > 64 && L <= 128, M2_ERR_UNSUPPORTED, "m2_filter_spectrum: kind 1 covers 64 < seq_len <= 128");
  lc::spectrum_kind1_kernel<<<D + 1, 128, 0, st>>>(k, spec, D, L);
  M2_LAUNCH_CHECK("spectrum_kind1_kernel");
  return M2_OK;
}

int longconv_tc_launch(const m2_longconv_args* a, cudaStream_t st) {
  using namespace lc;
  M2_REQUIRE(longconv_tc_supported(a->seq_len, a->act_dtype, a->d_model), M2_ERR_UNSUPPORTED,
             "m2_longconv_fwd: kind 1 needs bf16 activations, 64 < seq_len <= 128 and d_model %% 128 == 0");
  M2_REQUIRE(a->xin_sc == 1 && a->out_sc == 1 && (a->n_filters == 1 || a->u_sc == 1), M2_ERR_UNSUPPORTED,
             "m2_longconv_fwd: kind 1 needs channel-contiguous tensors");
  M2_REQUIRE(a->xin_st % 2 == 0 && a->xin_sb % 2 == 0 && a->out_st % 2 == 0 && a->out_sb % 2 == 0 &&
             m2_aligned(a->xin, 4) && m2_aligned(a->out, 4), M2_ERR_ALIGN,
             "m2_longconv_fwd: kind 1 needs 4-byte aligned rows of xin and out");
  Params P;
  P.B = a->batch; P.L = a->seq_len; P.D = a->d_model; P.nf = a->n_filters;
  P.ctiles = a->d_model / CT; P.units = P.B * P.ctiles;
  P.xin = (const __nv_bfloat16*)a->xin; P.xsb = a->xin_sb; P.xst = a->xin_st;
  P.u = a->u; P.usb = a->u_sb; P.ust = a->u_st;
  P.out = (__nv_bfloat16*)a->out; P.osb = a->out_sb; P.ost = a->out_st;
  P.sw = a->short_w; P.sb = a->short_b;
  for (int f = 0; f < 2; ++f) { P.spec[f] = a->spec[f]; P.bias[f] = a->bias[f]; }
  P.prefetch_ok = m2_aligned(a->xin, 16) && a->xin_st % 8 == 0 && a->xin_sb % 8 == 0 &&
                  (a->n_filters == 1 || (m2_aligned(a->u, 16) && a->u_st % 8 == 0 && a->u_sb % 8 == 0));
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = P.units < 2 * sms ? P.units : 2 * sms;
  const bool ubf = (a->n_filters == 2) && a->u_dtype == M2_BF16;
  if (a->n_filters == 2) {
    const size_t ua = ubf ? 4 : 8;
    M2_REQUIRE(m2_aligned(a->u, ua) && a->u_st % 2 == 0 && a->u_sb % 2 == 0, M2_ERR_ALIGN,
               "m2_longconv_fwd: kind 1 needs channel pairs of u aligned to their size");
  }
  if (ubf) {
    auto kern = longconv_tc128_kernel<__nv_bfloat16>;
    M2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    kern<<<grid, THREADS, SMEM_BYTES, st>>>(P);
  } else {
    auto kern = longconv_tc128_kernel<float>;
    M2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    kern<<<grid, THREADS, SMEM_BYTES, st>>>(P);
  }
  M2_LAUNCH_CHECK("longconv_tc128_kernel");
  return M2_OK;
}

}  // namespace m2
