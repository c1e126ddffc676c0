// Fused gated long convolution as Toeplitz GEMMs on tcgen05 tensor cores, sequence lengths
// L <= 128 (a multiple of 8), bf16 activations, time-contiguous tensors (kernel family 3).
//
// For a short sequence the bidirectional long convolution of one channel is a product with an
// L x L Toeplitz matrix, y[b, t] = sum_s a[b, s] T_c[t, s],  T_c[t, s] = k_c[(t - s) mod R]
// (+ bias on the diagonal), and the batch supplies the GEMM's M dimension: per channel
// D[128 batch rows x 128 t] = A[128 x 128 s] . T_c^T in eight K = 16 steps.  That is
// 2 B D L^2 flops per filter -- a few microseconds of tensor time for M2-BERT-base at L = 128
// -- instead of four FFT stages whose re-layouts run on CUDA cores.  The 128 x 16 B operand of
// K step kk is T_c[n, 16 kk + j] = h(16 kk + j - n), h(d) = k_c[(-d) mod R]: consecutive K steps
// are the same 16-column Toeplitz strip S[m, j] = h(j - m) shifted by 16 rows, so one strip of
// 240 rows (7.5 KB, fp16, power-of-two scaled per channel) serves all eight steps through the
// start address of the shared-memory descriptor.
//
// A persistent CTA (one per SM) walks units of (channel, 128 batch rows), time in four stages
// of 32 steps:
//   warp 0      TMA: raw x1 / v rows (with an 8-column halo so the 3-tap conv sees t-2, t-1; the
//               halo of the first stage starts at t = -8 and reads the causal zeros), filter strips
//   warp 2      TMA: the fp16 residual input in 64-step tiles (128-byte swizzled rows, the MMA's
//               K-major operand layout) and raw x2 rows for the epilogue
//   warps 11-18 short conv on x1 and v, v*x1 with the reference's bf16 rounding points, fp16
//               A-operand tile (generic proxy -> fence -> mbarrier)
//   warp 1      one thread issues the MMAs of both filters into one of two TMEM accumulator sets
//   warps 3-10  epilogue: TMEM -> registers, short conv on x2, gate, residual add, bf16 stores
// Every mbarrier wait is bounded; a wait that runs out sets the device status word and the CTA
// winds down.
//
// Computation replaced: bert/src/mm/monarch_mixer_sequence_mixer.py:109-149 and
// bert/src/mm/hyena_utils.py:16-42, :219-248 of the reference.
#include "tc_common.cuh"

namespace m2 {
namespace tz {

constexpr int TB = 128;                        // batch rows per unit (MMA M)
constexpr int TW = 32;                         // time steps per pipeline stage
constexpr int HALO = 8;                        // leading columns of a raw tile (16 bytes)
constexpr int RAW_ROW = (TW + HALO) * 2;       // 80 bytes: rows 16 (mod 128) apart -> no bank conflicts
constexpr int RAW_BYTES = TB * RAW_ROW;        // 10 KB
constexpr int OP_BYTES = TB * TW * 2;          // 8 KB: [128 x 32] fp16 operand in core-matrix order
constexpr int OP_LBO = TB * 16, OP_SBO = 128;  // K-adjacent core matrices 2 KB apart, row groups 128 B
constexpr int STAGE_BYTES = 2 * RAW_BYTES;     // raw x1 and v rows of one stage
constexpr int U_BYTES = TB * 128;              // [128 rows x 64 steps] fp16, 128-byte swizzled rows (TMA box)
constexpr int NST = 4, NA1 = 3, XSETS = 1, NX2 = 4 * XSETS, NU = 3;   // x2 slots: XSETS units of four
constexpr int STRIP_ROWS = 240;
constexpr int STRIP_BYTES = STRIP_ROWS * 32;   // 16 fp16 per row
constexpr int STRIP_FLOATS = STRIP_BYTES / 4;
constexpr int STRIP_LBO = 128, STRIP_SBO = 256;

constexpr int OFF_U = NST * STAGE_BYTES;       // every offset is a multiple of 1024 (swizzle anchor of the U tiles)
constexpr int OFF_A1 = OFF_U + NU * U_BYTES;
constexpr int OFF_X2 = OFF_A1 + NA1 * OP_BYTES;
constexpr int OFF_STRIP = OFF_X2 + NX2 * RAW_BYTES;
constexpr int OFF_BAR = OFF_STRIP + 4 * STRIP_BYTES;
constexpr int NBARS = 2 * NST + 2 * NU + 2 * NA1 + 2 * NX2 + 4 + 4;
constexpr int SMEM_BYTES = OFF_BAR + NBARS * 8 + 16 + 1024;
static_assert(OFF_U % 1024 == 0 && U_BYTES % 1024 == 0, "U tiles must sit on 1024-byte boundaries");
static_assert(SMEM_BYTES <= 232448, "shared memory budget");

constexpr int CTRL_WARPS = 3, EPI_WARPS = 8, P_WARPS = 8;
constexpr int THREADS = 32 * (CTRL_WARPS + EPI_WARPS + P_WARPS);

// byte offset of strip element (row m, column j)
__host__ __device__ constexpr int strip_off(int m, int j) {
  return (m >> 3) * STRIP_SBO + (j >> 3) * STRIP_LBO + (m & 7) * 16 + (j & 7) * 2;
}

// ---------------------------------------------------------------------------------------
// Spectrum table (kind 3): per channel the Toeplitz strip (STRIP_FLOATS floats holding fp16
// pairs), then d_model floats: the inverse of each channel's power-of-two scale.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
spectrum_kind3_kernel(const float* __restrict__ kfilt, const float* __restrict__ bias, float* __restrict__ spec,
                      int D, int L, int R) {
  __shared__ float h[256];
  __shared__ float red[8];
  const int c = blockIdx.x, tid = threadIdx.x;
  const float* row = kfilt + (size_t)c * R;
  float v = 0.f;
  if (tid < 255) {
    const int d = tid - 127;                                  // h(d) multiplies a[t + d]
    if (d > -L && d < L) v = row[((-d) % R + R) % R];          // taps beyond the sequence do not exist
    if (d == 0 && bias) v += bias[c];
  }
  h[tid] = v;
  float m = fabsf(v);
  if (!(m < 3.0e38f)) m = 0.f;                                // non-finite taps do not pick the scale
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((tid & 31) == 0) red[tid >> 5] = m;
  __syncthreads();
  m = red[0];
  for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
  int e = 0;
  if (m > 0.f) {
    int ex;
    frexpf(m, &ex);                                           // m = f * 2^ex, f in [0.5, 1)
    e = 14 - ex;                                              // m * 2^e in [2^13, 2^14)
    e = e < -60 ? -60 : (e > 60 ? 60 : e);
  }
  const float scale = ldexpf(1.0f, e);
  __half* S = reinterpret_cast<__half*>(spec + (size_t)c * STRIP_FLOATS);
  for (int idx = tid; idx < STRIP_ROWS * 16; idx += blockDim.x) {
    const int mrow = idx >> 4, j = idx & 15;
    S[strip_off(mrow, j) / 2] = __float2half_rn(h[j - mrow + 112 + 127] * scale);
  }
  if (tid == 0) spec[(size_t)D * STRIP_FLOATS + c] = ldexpf(1.0f, -e);
}

// ---------------------------------------------------------------------------------------
// (b, t, c) tensor of float32 / bf16 -> fp16 copy with time contiguous (the layout the
// residual filter's A operand is loaded from)
// ---------------------------------------------------------------------------------------
template <typename TS>
__global__ void __launch_bounds__(256)
time_major_f16_kernel(const TS* __restrict__ src, long long ssb, long long sst, long long ssc,
                      __half* __restrict__ dst, long long dsb, long long dsc, int L, int D) {
  __shared__ __half tile[64][66];
  const int t0 = blockIdx.x * 64, c0 = blockIdx.y * 64, b = blockIdx.z;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  float v[16];                                             // all loads of the thread in flight at once
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int tl = ty + 4 * i;
    v[i] = 0.f;
    if (t0 + tl < L && c0 + tx < D) v[i] = ld_as_float(src + b * ssb + (long long)(t0 + tl) * sst + (long long)(c0 + tx) * ssc);
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) tile[ty + 4 * i][tx] = __float2half_rn(fminf(fmaxf(v[i], -65504.f), 65504.f));
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int cl = ty + 4 * i;
    if (t0 + tx < L && c0 + cl < D) dst[(long long)(c0 + cl) * dsc + b * dsb + t0 + tx] = tile[tx][cl];
  }
}

// ---------------------------------------------------------------------------------------
struct Params {
  int B, L, D, nf, nbt, units, nsub, yu_bf16, wide_out;
  const float* sw; const float* sb;
  const float* spec[2];
  __nv_bfloat16* out; long long osb, osc;
};

__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_h2_sat(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// warp-uniform bounded wait: every lane polls, the warp leaves together
#define TZ_WAIT(bar, parity, why) \
  if (!__all_sync(0xffffffffu, tc::mbar_wait((bar), (parity), abort_flag, (why)))) break

__global__ void __launch_bounds__(THREADS, 1)
longconv_tz_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmU, const Params P) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* full_main = bars;                  // raw x1 / v rows of the stage landed (TMA bytes)
  uint64_t* empty_main = full_main + NST;      // raw rows consumed: 8 worker warps
  uint64_t* u_full = empty_main + NST;         // 64 steps of the residual operand landed (only the MMA thread waits)
  uint64_t* u_empty = u_full + NU;             // ... consumed: 1 MMA commit
  uint64_t* a1_full = u_empty + NU;            // 8 worker warps
  uint64_t* a1_empty = a1_full + NA1;          // 1 MMA commit
  uint64_t* x2_full = a1_empty + NA1;          // TMA bytes
  uint64_t* x2_empty = x2_full + NX2;          // 4 epilogue warps
  uint64_t* strip_full = x2_empty + NX2;       // TMA bytes
  uint64_t* strip_empty = strip_full + 2;      // 1 MMA commit
  uint64_t* tmem_full = strip_empty + 2;       // 1 MMA commit
  uint64_t* tmem_empty = tmem_full + 2;        // 8 epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) { tc::mbar_init(full_main + s, 1); tc::mbar_init(empty_main + s, P_WARPS); }
    for (int s = 0; s < NU; ++s) { tc::mbar_init(u_full + s, 1); tc::mbar_init(u_empty + s, 1); }
    for (int a = 0; a < NA1; ++a) { tc::mbar_init(a1_full + a, P_WARPS); tc::mbar_init(a1_empty + a, 1); }
    for (int j = 0; j < NX2; ++j) { tc::mbar_init(x2_full + j, 1); tc::mbar_init(x2_empty + j, EPI_WARPS / 2); }
    for (int p = 0; p < 2; ++p) {
      tc::mbar_init(strip_full + p, 1); tc::mbar_init(strip_empty + p, 1);
      tc::mbar_init(tmem_full + p, 1); tc::mbar_init(tmem_empty + p, EPI_WARPS);
    }
    *abort_flag = 0;
    tc::mbar_fence_init();
    tc::tma_prefetch_desc(&tmX);
    tc::tma_prefetch_desc(&tmU);
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, 512);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // contiguous range of units: consecutive units share the channel, so its strips stay put
  const int u_first = (int)(((long long)blockIdx.x * P.units) / gridDim.x);
  const int u_last = (int)(((long long)(blockIdx.x + 1) * P.units) / gridDim.x);

  if (warp == 0) {
    // ------------------------- TMA: strips, raw x1 / v, residual operand -------------------------
    if (lane == 0) {
      int it = 0, epoch = -1, prev_c = -1;
      bool ok = true;
      for (int unit = u_first; unit < u_last && ok; ++unit) {
        const int c = unit / P.nbt, b0 = (unit % P.nbt) * TB;
        if (c != prev_c) {
          prev_c = c; ++epoch;
          const int p = epoch & 1;
          if (!tc::mbar_wait(strip_empty + p, ((epoch >> 1) & 1) ^ 1, abort_flag, tc::ST_TIMEOUT_EMPTY)) break;
          tc::mbar_expect_tx(strip_full + p, P.nf * STRIP_BYTES);
          for (int f = 0; f < P.nf; ++f)
            tc::bulk_load(smem + OFF_STRIP + (2 * p + f) * STRIP_BYTES, (f ? P.spec[1] : P.spec[0]) + (size_t)c * STRIP_FLOATS,
                          STRIP_BYTES, strip_full + p);
        }
        for (int j = 0; j < P.nsub; ++j, ++it) {
          const int s = it % NST;
          if (!tc::mbar_wait(empty_main + s, ((it / NST) & 1) ^ 1, abort_flag, tc::ST_TIMEOUT_EMPTY)) { ok = false; break; }
          unsigned char* st = smem + s * STAGE_BYTES;
          tc::mbar_expect_tx(full_main + s, 2 * RAW_BYTES);
          tc::tma_load_3d(st, &tmX, full_main + s, TW * j - HALO, b0, c);
          tc::tma_load_3d(st + RAW_BYTES, &tmX, full_main + s, TW * j - HALO, b0, 2 * P.D + c);
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------- TMA: raw x2 rows for the epilogue -------------------------
    if (lane == 0) {
      bool ok = true;
      int ui = 0, it = 0;
      for (int unit = u_first; unit < u_last && ok; ++unit, ++ui) {
        const int c = unit / P.nbt, b0 = (unit % P.nbt) * TB;
        // the residual operand of the unit in tiles of 64 steps, rows of 128 bytes (a 16-byte-row
        // box in core-matrix order would cost the TMA unit eight times the requests) ...
        for (int k = 0; k < (P.nsub + 1) / 2 && P.nf == 2; ++k, ++it) {
          const int s = it % NU;
          if (!tc::mbar_wait(u_empty + s, ((it / NU) & 1) ^ 1, abort_flag, tc::ST_TIMEOUT_EMPTY)) { ok = false; break; }
          tc::mbar_expect_tx(u_full + s, U_BYTES);
          tc::tma_load_3d(smem + OFF_U + s * U_BYTES, &tmU, u_full + s, 64 * k, b0, c);
        }
        if (!ok) break;
        // ... then the x2 rows its epilogue reads
        for (int j = 0; j < P.nsub; ++j) {
          const int sl = 4 * (ui % XSETS) + j;             // units rotate through the slot sets
          if (!tc::mbar_wait(x2_empty + sl, ((ui / XSETS) & 1) ^ 1, abort_flag, tc::ST_TIMEOUT_EMPTY)) { ok = false; break; }
          tc::mbar_expect_tx(x2_full + sl, RAW_BYTES);
          tc::tma_load_3d(smem + OFF_X2 + sl * RAW_BYTES, &tmX, x2_full + sl, TW * j - HALO, b0, P.D + c);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------- MMA issuer -------------------------
    if (lane == 0) {
      // both operands fp16: kind::f16 with a bf16 A and an fp16 B is an illegal instruction on
      // sm_100a, so v*x1 (bf16 by the reference's arithmetic) is converted, exactly, to fp16
      constexpr uint32_t idesc = tc::make_idesc(TB, 128, 0);
      int it = 0, ut = 0, epoch = -1, prev_c = -1, ui = 0;
      bool ok = true;
      for (int unit = u_first; unit < u_last && ok; ++unit, ++ui) {
        const int c = unit / P.nbt;
        if (c != prev_c) {
          prev_c = c; ++epoch;
          if (!tc::mbar_wait(strip_full + (epoch & 1), (epoch >> 1) & 1, abort_flag, tc::ST_TIMEOUT_TMA)) break;
        }
        const int p = epoch & 1, acc = ui & 1;
        if (!tc::mbar_wait(tmem_empty + acc, ((ui >> 1) & 1) ^ 1, abort_flag, tc::ST_TIMEOUT_MMA)) break;
        tc::tc_fence_after();
        const uint32_t tacc = tmem_base + acc * 256;
        const uint32_t strip0 = tc::smem_u32(smem + OFF_STRIP + (2 * p) * STRIP_BYTES);
        for (int j = 0; j < P.nsub; ++j, ++it) {
          const int s = it % NST, a = it % NA1;
          if (P.nf == 2 && (j & 1) == 0 &&
              !tc::mbar_wait(u_full + ut % NU, (ut / NU) & 1, abort_flag, tc::ST_TIMEOUT_TMA)) { ok = false; break; }
          if (!tc::mbar_wait(a1_full + a, (it / NA1) & 1, abort_flag, tc::ST_TIMEOUT_MMA)) { ok = false; break; }
          tc::tc_fence_after();
          const uint32_t a1 = tc::smem_u32(smem + OFF_A1 + a * OP_BYTES);
          // 64-step tile of the residual operand: K step q of it starts 32 q bytes into the swizzled rows
          const uint64_t udesc = tc::smem_desc_k_sw128(tc::smem_u32(smem + OFF_U + (ut % NU) * U_BYTES)) + 4 * (j & 1);
#pragma unroll
          for (int ks = 0; ks < TW / 16; ++ks) {
            const int kk = (TW / 16) * j + ks;
            const uint32_t boff = (uint32_t)(14 - 2 * kk) * STRIP_SBO;       // strip rows 112 - 16 kk ..
            tc::mma_ss(tacc, tc::smem_desc_k_nosw(a1 + ks * 2 * OP_LBO, OP_LBO, OP_SBO),
                       tc::smem_desc_k_nosw(strip0 + boff, STRIP_LBO, STRIP_SBO), idesc, kk ? 1u : 0u);
            if (P.nf == 2)
              tc::mma_ss(tacc + 128, udesc + 2 * ks,
                         tc::smem_desc_k_nosw(strip0 + STRIP_BYTES + boff, STRIP_LBO, STRIP_SBO), idesc, kk ? 1u : 0u);
          }
          if (P.nf == 2 && ((j & 1) || j == P.nsub - 1)) { tc::mma_commit(u_empty + ut % NU); ++ut; }
          tc::mma_commit(a1_empty + a);
        }
        if (!ok) break;
        tc::mma_commit(tmem_full + acc);
        if (unit + 1 >= u_last || (unit + 1) / P.nbt != c) tc::mma_commit(strip_empty + p);
      }
    }
  } else if (warp < CTRL_WARPS + EPI_WARPS) {
    // ------------------------- epilogue -------------------------
    const int quarter = warp & 3;                        // TMEM lanes this warp may touch
    const int hh = (warp - CTRL_WARPS) >> 2;             // which half of the time axis
    const int r = quarter * 32 + lane;
    int ui = 0;
    for (int unit = u_first; unit < u_last; ++unit, ++ui) {
      const int c = unit / P.nbt, b = (unit % P.nbt) * TB + r;
      const int acc = ui & 1;
      const float is1 = __ldg(P.spec[0] + (size_t)P.D * STRIP_FLOATS + c);
      const float is2 = P.nf == 2 ? __ldg(P.spec[1] + (size_t)P.D * STRIP_FLOATS + c) : 0.f;
      const int ch = P.D + c;
      const float w0 = bf16r(__ldg(P.sw + 3 * ch)), w1 = bf16r(__ldg(P.sw + 3 * ch + 1)),
                  w2 = bf16r(__ldg(P.sw + 3 * ch + 2)), wb = bf16r(__ldg(P.sb + ch));
      TZ_WAIT(tmem_full + acc, (ui >> 1) & 1, tc::ST_TIMEOUT_EPI);
      tc::tc_fence_after();
      const uint32_t tacc = tmem_base + acc * 256 + ((uint32_t)(quarter * 32) << 16);
      __nv_bfloat16* orow = P.out + (long long)c * P.osc + (long long)b * P.osb;
      bool ok = true;
#pragma unroll 1
      for (int k = 0; k < 4; ++k) {
        const int t0 = 64 * hh + 16 * k;
        if (t0 >= P.L) break;
        const int j = 4 * (ui % XSETS) + t0 / TW, toff = t0 % TW;   // x2 slot
        if ((k & 1) == 0) {
          if (!__all_sync(0xffffffffu, tc::mbar_wait(x2_full + j, (ui / XSETS) & 1, abort_flag, tc::ST_TIMEOUT_TMA))) { ok = false; break; }
        }
        uint32_t d1[16], d2[16];
        tc::tmem_ld16(tacc + t0, d1);
        if (P.nf == 2) tc::tmem_ld16(tacc + 128 + t0, d2);
        // raw x2: columns toff + 6 .. toff + 23 of the slot's row (halo included)
        const uint32_t xrow = tc::smem_u32(smem + OFF_X2 + j * RAW_BYTES) + r * RAW_ROW + toff * 2;
        const uint32_t hw = lds32(xrow + 12);
        const uint4 q0 = lds128(xrow + 16), q1 = lds128(xrow + 32);
        const uint32_t xw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        tc::tmem_ld_wait();
        float xa = bf_lo(hw), xb = bf_hi(hw);
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float x0 = bf_lo(xw[i]), x1 = bf_hi(xw[i]);
          const float c0 = fmaf(w2, x0, fmaf(w1, xb, fmaf(w0, xa, wb)));
          const float c1 = fmaf(w2, x1, fmaf(w1, x0, fmaf(w0, xb, wb)));
          xa = x0; xb = x1;
          const uint32_t g = pack_bf2(c0, c1);                                          // short conv output, bf16
          const uint32_t y = pack_bf2(__uint_as_float(d1[2 * i]) * is1, __uint_as_float(d1[2 * i + 1]) * is1);
          const uint32_t res = bf2_mul(y, g);                                           // y * x2, bf16
          if (P.nf == 2) {
            float u0 = __uint_as_float(d2[2 * i]) * is2, u1 = __uint_as_float(d2[2 * i + 1]) * is2;
            if (P.yu_bf16) { const uint32_t ur = pack_bf2(u0, u1); u0 = bf_lo(ur); u1 = bf_hi(ur); }
            o[i] = pack_bf2(bf_lo(res) + u0, bf_hi(res) + u1);
          } else {
            o[i] = res;
          }
        }
        if (b < P.B) {
          if (t0 + 16 <= P.L) {
            if (P.wide_out) {
              stg256(orow + t0, o[0], o[1], o[2], o[3], o[4], o[5], o[6], o[7]);
            } else {
              uint4* dst = reinterpret_cast<uint4*>(orow + t0);
              dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
              dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
            }
          } else {                                        // L is a multiple of 8: one full half remains
            *reinterpret_cast<uint4*>(orow + t0) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
        if (k & 1) {
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(x2_empty + j);
        } else if (t0 + 16 >= P.L) {                      // the slot's second half does not exist
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(x2_empty + j);
        }
      }
      if (!ok) break;
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(tmem_empty + acc);
    }
  } else {
    // ------------------------- workers: short conv on x1 and v, gate, A operand -------------------------
    const int pw = warp - CTRL_WARPS - EPI_WARPS;
    const int r = (pw & 3) * 32 + lane, h = pw >> 2;      // batch row, which 16 of the stage's 32 steps
    int it = 0;
    bool ok = true;
    for (int unit = u_first; unit < u_last && ok; ++unit) {
      const int c = unit / P.nbt;
      const int cv = 2 * P.D + c;
      // packed pairs (x1, v): both short convolutions advance in one f32x2 FMA chain
      const f32x2 w0 = f2_pack(bf16r(__ldg(P.sw + 3 * c)), bf16r(__ldg(P.sw + 3 * cv)));
      const f32x2 w1 = f2_pack(bf16r(__ldg(P.sw + 3 * c + 1)), bf16r(__ldg(P.sw + 3 * cv + 1)));
      const f32x2 w2 = f2_pack(bf16r(__ldg(P.sw + 3 * c + 2)), bf16r(__ldg(P.sw + 3 * cv + 2)));
      const f32x2 wb = f2_pack(bf16r(__ldg(P.sb + c)), bf16r(__ldg(P.sb + cv)));
      for (int j = 0; j < P.nsub; ++j, ++it) {
        const int s = it % NST, a = it % NA1;
        if (!__all_sync(0xffffffffu, tc::mbar_wait(full_main + s, (it / NST) & 1, abort_flag, tc::ST_TIMEOUT_TMA))) { ok = false; break; }
        const uint32_t xrow = tc::smem_u32(smem + s * STAGE_BYTES) + r * RAW_ROW + h * 32;
        const uint32_t hx = lds32(xrow + 12), hv = lds32(xrow + RAW_BYTES + 12);
        const uint4 x0 = lds128(xrow + 16), x1 = lds128(xrow + 32);
        const uint4 v0 = lds128(xrow + RAW_BYTES + 16), v1 = lds128(xrow + RAW_BYTES + 32);
        const uint32_t xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        const uint32_t vw[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        f32x2 pa = f2_pack(bf_lo(hx), bf_lo(hv)), pb = f2_pack(bf_hi(hx), bf_hi(hv));
        const int tbase = TW * j + 16 * h;
        uint32_t aw[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const f32x2 e0 = f2_pack(bf_lo(xw[i]), bf_lo(vw[i])), e1 = f2_pack(bf_hi(xw[i]), bf_hi(vw[i]));
          const f32x2 c0 = f2_fma(w2, e0, f2_fma(w1, pb, f2_fma(w0, pa, wb)));
          const f32x2 c1 = f2_fma(w2, e1, f2_fma(w1, e0, f2_fma(w0, pb, wb)));
          pa = e0; pb = e1;
          float cx0, cv0, cx1, cv1;
          f2_unpack(c0, cx0, cv0);
          f2_unpack(c1, cx1, cv1);
          const uint32_t pr = bf2_mul(pack_bf2(cx0, cx1), pack_bf2(cv0, cv1));   // bf16 conv outputs, v * x1 in bf16
          aw[i] = pack_h2_sat(bf_lo(pr), bf_hi(pr));
        }
        if (tbase + 16 > P.L) {                           // the long convolution sees zeros past L
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (tbase + 2 * i >= P.L) aw[i] = 0u;
            else if (tbase + 2 * i + 1 >= P.L) aw[i] &= 0x0000ffffu;
          }
        }
        if (!__all_sync(0xffffffffu, tc::mbar_wait(a1_empty + a, ((it / NA1) & 1) ^ 1, abort_flag, tc::ST_TIMEOUT_EMPTY))) { ok = false; break; }
        const uint32_t dst = tc::smem_u32(smem + OFF_A1 + a * OP_BYTES) + (2 * h) * OP_LBO + r * 16;
        sts128(dst, aw[0], aw[1], aw[2], aw[3]);
        sts128(dst + OP_LBO, aw[4], aw[5], aw[6], aw[7]);
        tc::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tc::mbar_arrive(a1_full + a);
          tc::mbar_arrive(empty_main + s);
        }
      }
    }
  }

  // ------------------------- teardown -------------------------
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // give loads that were issued before the abort a bounded time to land
    for (int s = 0; s < NST; ++s)
      for (uint32_t i = 0; i < 4096 && !tc::mbar_try_wait(full_main + s, 0) && !tc::mbar_try_wait(full_main + s, 1); ++i) {}
    for (int s = 0; s < NU; ++s)
      for (uint32_t i = 0; i < 4096 && !tc::mbar_try_wait(u_full + s, 0) && !tc::mbar_try_wait(u_full + s, 1); ++i) {}
    for (int j = 0; j < NX2; ++j)
      for (uint32_t i = 0; i < 4096 && !tc::mbar_try_wait(x2_full + j, 0) && !tc::mbar_try_wait(x2_full + j, 1); ++i) {}
  }
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, 512);
  }
}
#undef TZ_WAIT

}  // namespace tz


int longconv_tz_supported(int batch, int seq_len, m2_dtype act_dtype) {
  return act_dtype == M2_BF16 && seq_len >= 16 && seq_len <= 128 && seq_len % 8 == 0 && batch >= 64;
}

size_t spectrum_kind3_floats(int D, int L) {
  (void)L;
  return (size_t)D * tz::STRIP_FLOATS + (size_t)D;
}

int spectrum_kind3_launch(int D, int L, const float* k, const float* bias, float* spec, cudaStream_t st) {
  M2_REQUIRE(L >= 1 && L <= 128, M2_ERR_UNSUPPORTED, "m2_filter_spectrum: kind 3 covers seq_len <= 128");
  tz::spectrum_kind3_kernel<<<D, 256, 0, st>>>(k, bias, spec, D, L, m2_filter_row_len(L));
  M2_LAUNCH_CHECK("spectrum_kind3_kernel");
  return M2_OK;
}

static int tz_encode(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base, const cuuint64_t* dims,
                     const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_NONE) {
  m2_encode_tiled_fn enc;
  int rc = m2_get_encode_fn(&enc);
  if (rc) return rc;
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, dt, rank, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return m2_set_error(M2_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return M2_OK;
}

int longconv_tz_launch(const m2_longconv_args* a, cudaStream_t st) {
  using namespace tz;
  M2_REQUIRE(a->act_dtype == M2_BF16 && a->seq_len >= 16 && a->seq_len <= 128 && a->seq_len % 8 == 0, M2_ERR_UNSUPPORTED,
             "m2_longconv_fwd: kind 3 needs bf16 activations and 16 <= seq_len <= 128, a multiple of 8");
  M2_REQUIRE(a->xin_st == 1 && a->out_st == 1 && (a->n_filters == 1 || a->u_st == 1), M2_ERR_UNSUPPORTED,
             "m2_longconv_fwd: kind 3 needs time-contiguous tensors");
  M2_REQUIRE(a->n_filters == 1 || a->u_dtype == M2_F16, M2_ERR_UNSUPPORTED,
             "m2_longconv_fwd: kind 3 reads the residual input as fp16 (m2_time_major_f16)");
  M2_REQUIRE(!a->bias[0] && !a->bias[1], M2_ERR_ARG,
             "m2_longconv_fwd: kind 3 takes the bias folded into the spectrum (m2_filter_spectrum_bias); pass bias = NULL");
  M2_REQUIRE(m2_aligned(a->xin, 16) && a->xin_sb % 8 == 0 && a->xin_sc % 8 == 0 && m2_aligned(a->out, 16) &&
             a->out_sb % 8 == 0 && a->out_sc % 8 == 0 && a->xin_sb > 0 && a->xin_sc > 0, M2_ERR_ALIGN,
             "m2_longconv_fwd: kind 3 needs 16-byte aligned rows of xin and out");
  M2_REQUIRE(a->n_filters == 1 || (m2_aligned(a->u, 16) && a->u_sb % 8 == 0 && a->u_sc % 8 == 0 && a->u_sb > 0 && a->u_sc > 0),
             M2_ERR_ALIGN, "m2_longconv_fwd: kind 3 needs 16-byte aligned rows of u");
  Params P;
  P.B = a->batch; P.L = a->seq_len; P.D = a->d_model; P.nf = a->n_filters;
  P.nbt = (P.B + TB - 1) / TB;
  M2_REQUIRE((long long)P.nbt * P.D < (1LL << 30), M2_ERR_UNSUPPORTED, "m2_longconv_fwd: too many units");
  P.units = P.nbt * P.D;
  P.nsub = (P.L + TW - 1) / TW;
  P.yu_bf16 = a->yu_bf16 ? 1 : 0;
  P.sw = a->short_w; P.sb = a->short_b;
  P.spec[0] = a->spec[0]; P.spec[1] = a->spec[1];
  P.out = (__nv_bfloat16*)a->out; P.osb = a->out_sb; P.osc = a->out_sc;
  P.wide_out = m2_aligned(a->out, 32) && a->out_sb % 16 == 0 && a->out_sc % 16 == 0;   // 32-byte stores are legal

  CUtensorMap tmX, tmU;
  {
    const cuuint64_t dims[3] = {(cuuint64_t)P.L, (cuuint64_t)P.B, (cuuint64_t)3 * P.D};
    const cuuint64_t strides[2] = {(cuuint64_t)a->xin_sb * 2, (cuuint64_t)a->xin_sc * 2};
    const cuuint32_t box[3] = {TW + HALO, TB, 1};
    int rc = tz_encode(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a->xin, dims, strides, box);
    if (rc) return rc;
  }
  if (P.nf == 2) {
    // rows of 64 steps (128 bytes) with the 128-byte swizzle: the K-major operand layout of the MMA
    const cuuint64_t dims[3] = {(cuuint64_t)P.L, (cuuint64_t)P.B, (cuuint64_t)P.D};
    const cuuint64_t strides[2] = {(cuuint64_t)a->u_sb * 2, (cuuint64_t)a->u_sc * 2};
    const cuuint32_t box[3] = {64, TB, 1};
    int rc = tz_encode(&tmU, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, a->u, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  } else {
    tmU = tmX;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = P.units < sms ? P.units : sms;
  auto kern = longconv_tz_kernel;
  M2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
  kern<<<grid, THREADS, SMEM_BYTES, st>>>(tmX, tmU, P);
  M2_LAUNCH_CHECK("longconv_tz_kernel");
  return M2_OK;
}

int time_major_f16_launch(const m2_time_major_args* a, cudaStream_t st) {
  dim3 grid((a->seq_len + 63) / 64, (a->d_model + 63) / 64, a->batch);
  if (a->src_dtype == M2_F32)
    tz::time_major_f16_kernel<float><<<grid, 256, 0, st>>>((const float*)a->src, a->src_sb, a->src_st, a->src_sc,
                                                            (__half*)a->dst, a->dst_sb, a->dst_sc, a->seq_len, a->d_model);
  else
    tz::time_major_f16_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)a->src, a->src_sb, a->src_st,
                                                                    a->src_sc, (__half*)a->dst, a->dst_sb, a->dst_sc,
                                                                    a->seq_len, a->d_model);
  M2_LAUNCH_CHECK("time_major_f16_kernel");
  return M2_OK;
}

}  // namespace m2
