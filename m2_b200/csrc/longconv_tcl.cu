// Fused gated long convolution on tcgen05 tensor cores for long rows (kernel family 2):
// bf16 activations stored time-contiguous ((B, channels, L) layout), transform length
// N = 32 * N2 * N3 = 4096 (1024 < L <= 2048), 16384 (4096 < L <= 8192) or 65536
// (16384 < L <= 32768).
//
// One (batch row, channel) sequence is processed at a time by a "slot" of four warps (sixteen
// for N = 65536, where one sequence fills the SM); a CTA holds several slots that run independently (own barriers, own TMEM columns, own shared-
// memory region) so that one slot's loads and stage hand-offs overlap the others' work.
//
// The real FFT of length N is evaluated at the odd frequencies k + 1/2 (negacyclic form,
// no DC/Nyquist specials, Hermitian half = k1 < 16) and factored Monarch style with
// n = R n1 + N3 n2 + n3 (R = N2 N3), k = k1 + 32 k2 + 32 N2 k3:
//
//   F1  rows r = (n2, n3):  B1[r, k1]   = sum_{n1 < 16} W32^{n1 (k1 + 1/2)} a[R n1 + r]
//   x T1[r, k1] = w^{r (k1 + 1/2)}, rows -> (k1, n3)
//   F2  rows (k1, n3):      B2[., k2]   = sum_{n2} W_N2^{n2 k2} B1
//   x T2[n3, k2] = w^{32 n3 k2}, rows -> (k1, k2)
//   F3  rows (k1, k2):      Z[., k3]    = sum_{n3} W_N3^{n3 k3} B2
//   x (G + bias), then the three inverse stages in mirror order; I1 yields only the L kept
//   outputs y[R n1 + r], n1 < 16.  The inverse DFT stages reuse the forward matrices on
//   conjugated data (IDFT(x) = conj DFT(conj x)), so each radix needs one matrix only.
//
// Every stage is a batched real GEMM with M = 128 rows per tile taken from inside the
// sequence itself, fp16 operands in un-swizzled core-matrix shared memory, constant DFT
// matrices as B operands and float32 accumulators in tensor memory.  Between stages the
// thread that owns a TMEM lane applies the twiddle and scatters its row into the next
// stage's operand layout (the row <-> column exchange of the four-step FFT happens in
// these stores).
//
// Computation replaced: bert/src/mm/monarch_mixer_sequence_mixer.py:109-149 and
// bert/src/mm/hyena_utils.py:16-42, :219-248 of the reference.
#include "tc_common.cuh"
#include <cooperative_groups.h>

namespace m2 {
namespace lcl {

constexpr float S1 = 0.25f;
__host__ __device__ constexpr float stage_scale(int n) {   // 2^-ceil(log2(n)/2)
  return n >= 32 ? 0.125f : n >= 8 ? 0.25f : 0.5f;
}
__host__ __device__ constexpr int cmax(int a, int b) { return a > b ? a : b; }

// N2, N3: radices of the second and third stage (the first is 32); SLOTS: independent
// sequences in flight per CTA; TS: warps per TMEM lane quarter inside a slot (they split
// the row tiles of every stage among themselves).
template <int N2_, int N3_, int SLOTS_, int TS_>
struct Geo {
  static constexpr int N2 = N2_, N3 = N3_, SLOTS = SLOTS_, TS = TS_;
  static constexpr int R = N2 * N3;             // rows of stage 1 = N / 32
  static constexpr int N = 32 * R;
  static constexpr int LG = (N == 4096) ? 12 : (N == 16384) ? 14 : 16;
  static constexpr int K2 = 2 * N2, K3 = 2 * N3;
  static constexpr int TR = R / 128;            // row tiles of the first / last stage
  static constexpr int T2T = 16 * N3 / 128;     // row tiles of the DFT_N2 stages
  static constexpr int T3T = 16 * N2 / 128;     // row tiles of the DFT_N3 stages
  static constexpr int G2 = N2 / 8, G3 = N3 / 8;             // 8-row groups per k1
  static constexpr int TPS = 128 * TS;          // threads per slot
  static constexpr int THREADS = SLOTS * TPS;
  static constexpr bool SPLIT_T1 = R > 512;     // twiddle table of stage 1 as a product of two small ones
  // operand layouts: core matrices of 8 rows x 16 bytes; LBO = stride between K chunks,
  // SBO = stride between 8-row groups, TILE = 128 rows.  The padded strides spread the
  // scattered 4-byte stores of the re-layout steps over the shared-memory banks.
  static constexpr int A1_LBO = 128, A1_SBO = 2 * 128 + 16, A1_TILE = 16 * A1_SBO;            // K = 16
  static constexpr int A2_LBO = 144, A2_SBO = (K2 / 8) * 144, A2_TILE = 16 * A2_SBO;          // K = K2
  static constexpr int A3_LBO = 144, A3_SBO = (K3 / 8) * 144 + 16, A3_TILE = 16 * A3_SBO;     // K = K3
  static constexpr int A6_LBO = 128, A6_SBO = 4 * 128, A6_TILE = 16 * A6_SBO;                 // K = 32
  static constexpr int DATA_BYTES =
      ((cmax(cmax(TR * A1_TILE, T2T * A2_TILE), cmax(cmax(T3T * A3_TILE, TR * A6_TILE), 64 * R)) + 127) / 128) * 128;
  static constexpr int COLS = cmax(TR * 32, cmax(T2T * K2, T3T * K3));
  static constexpr int TCOLS = (SLOTS * COLS <= 32) ? 32 : (SLOTS * COLS <= 64) ? 64 : (SLOTS * COLS <= 128) ? 128
                               : (SLOTS * COLS <= 256) ? 256 : 512;
  static constexpr float S2 = stage_scale(N2), S3 = stage_scale(N3);
  static constexpr float KAPPA = (2.0f / N) / ((S1 * S2 * S3) * (S1 * S2 * S3));
  // header of the spectrum table (bytes): constant matrices (un-padded core-matrix layout)
  // and twiddle tables
  static constexpr int F1_OFF = 0;                       // [32 x 16]
  static constexpr int I1_OFF = F1_OFF + 1024;           // [16 x 32]
  static constexpr int F2_OFF = I1_OFF + 1024;           // [K2 x K2]
  static constexpr int F3_OFF = F2_OFF + K2 * K2 * 2;    // [K3 x K3]
  static constexpr int T1_OFF = F3_OFF + K3 * K3 * 2;    // half2 [16][R], or [16][N2] then [16][N3] when split
  static constexpr int T1_BYTES = SPLIT_T1 ? 64 * (N2 + N3) : 64 * R;
  static constexpr int T2A_OFF = T1_OFF + T1_BYTES;      // half2 [N2][N3]  (k2 major)
  static constexpr int T2B_OFF = T2A_OFF + 4 * R;        // half2 [N3][N2]  (n3 major)
  static constexpr int HDR_BYTES = T2B_OFF + 4 * R;
  static constexpr int HDR_FLOATS = HDR_BYTES / 4;
  static constexpr int SMEM = SLOTS * DATA_BYTES + HDR_BYTES + 3 * SLOTS * 8 + 64 + 128;
  static_assert(R % 128 == 0 && (16 * N3) % 128 == 0 && (16 * N2) % 128 == 0, "row tiles must be full");
  static_assert(SLOTS * COLS <= 512, "accumulators exceed tensor memory");
  static_assert(TR % TS == 0 && T2T % TS == 0 && T3T % TS == 0, "tile split must divide every stage");
  static_assert((R / 4) % TPS == 0 || TPS % (R / 4) == 0, "load mapping");
  static_assert(SMEM <= 227 * 1024, "shared memory");
};

// byte offset of element (row, k) of a constant matrix with K columns (un-padded layout)
template <int K>
__host__ __device__ constexpr int mat_off(int row, int k) {
  return (row >> 3) * (K * 16) + (k >> 3) * 128 + (row & 7) * 16 + (k & 7) * 2;
}

// ---------------------------------------------------------------------------------------
// Spectrum table (kind 2): [HDR_FLOATS floats: matrices + twiddles] then per channel
// G[(k1 N2 + k2)][k3] as half2, multiplied by KAPPA * 2^e, then one float 2^-e per channel.
// ---------------------------------------------------------------------------------------
template <typename G>
__device__ void write_header(float* spec, int tid, int nt) {
  constexpr int N = G::N, N2 = G::N2, N3 = G::N3, R = G::R, K2 = G::K2, K3 = G::K3;
  __half* m = reinterpret_cast<__half*>(spec);
  for (int idx = tid; idx < 16 * 16; idx += nt) {
    // F1 rows 2k1+ri: W32^{n1 (k1+1/2)}.  I1 columns 2k1+ri act on the CONJUGATE of the last
    // inverse stage's input: y = sum cos * Qr + sin * Qi.
    const int k1 = idx / 16, n1 = idx % 16;
    double sn, cs;
    sincospi(2.0 * n1 * (k1 + 0.5) / 32.0, &sn, &cs);
    m[(G::F1_OFF + mat_off<16>(2 * k1, n1)) / 2] = __double2half(S1 * cs);
    m[(G::F1_OFF + mat_off<16>(2 * k1 + 1, n1)) / 2] = __double2half(-S1 * sn);
    m[(G::I1_OFF + mat_off<32>(n1, 2 * k1)) / 2] = __double2half(S1 * cs);
    m[(G::I1_OFF + mat_off<32>(n1, 2 * k1 + 1)) / 2] = __double2half(S1 * sn);
  }
  for (int idx = tid; idx < N2 * N2; idx += nt) {            // forward DFT_N2 in real form
    const int ko = idx / N2, ni = idx % N2;
    double sn, cs;
    sincospi(2.0 * ((ko * ni) % N2) / N2, &sn, &cs);
    const double c = G::S2 * cs, s = G::S2 * sn;             // w = c - i s
    __half* f = m + G::F2_OFF / 2;
    f[mat_off<K2>(2 * ko, 2 * ni) / 2] = __double2half(c);
    f[mat_off<K2>(2 * ko, 2 * ni + 1) / 2] = __double2half(s);
    f[mat_off<K2>(2 * ko + 1, 2 * ni) / 2] = __double2half(-s);
    f[mat_off<K2>(2 * ko + 1, 2 * ni + 1) / 2] = __double2half(c);
  }
  for (int idx = tid; idx < N3 * N3; idx += nt) {            // forward DFT_N3
    const int ko = idx / N3, ni = idx % N3;
    double sn, cs;
    sincospi(2.0 * ((ko * ni) % N3) / N3, &sn, &cs);
    const double c = G::S3 * cs, s = G::S3 * sn;
    __half* f = m + G::F3_OFF / 2;
    f[mat_off<K3>(2 * ko, 2 * ni) / 2] = __double2half(c);
    f[mat_off<K3>(2 * ko, 2 * ni + 1) / 2] = __double2half(s);
    f[mat_off<K3>(2 * ko + 1, 2 * ni) / 2] = __double2half(-s);
    f[mat_off<K3>(2 * ko + 1, 2 * ni + 1) / 2] = __double2half(c);
  }
  __half2* t1 = reinterpret_cast<__half2*>(reinterpret_cast<unsigned char*>(spec) + G::T1_OFF);
  if (G::SPLIT_T1) {
    for (int idx = tid; idx < 16 * N2; idx += nt) {          // Ta[k1][n2] = w^{N3 n2 (k1 + 1/2)}
      const int k1 = idx / N2, n2 = idx % N2;
      double sn, cs;
      sincospi(2.0 * N3 * n2 * (k1 + 0.5) / N, &sn, &cs);
      t1[idx] = __floats2half2_rn((float)cs, (float)(-sn));
    }
    for (int idx = tid; idx < 16 * N3; idx += nt) {          // Tb[k1][n3] = w^{n3 (k1 + 1/2)}
      const int k1 = idx / N3, n3 = idx % N3;
      double sn, cs;
      sincospi(2.0 * n3 * (k1 + 0.5) / N, &sn, &cs);
      t1[16 * N2 + idx] = __floats2half2_rn((float)cs, (float)(-sn));
    }
  } else {
    for (int idx = tid; idx < 16 * R; idx += nt) {           // T1[k1][r] = w^{r (k1 + 1/2)}
      const int k1 = idx / R, r = idx % R;
      double sn, cs;
      sincospi(2.0 * r * (k1 + 0.5) / N, &sn, &cs);
      t1[idx] = __floats2half2_rn((float)cs, (float)(-sn));
    }
  }
  __half2* t2a = reinterpret_cast<__half2*>(reinterpret_cast<unsigned char*>(spec) + G::T2A_OFF);
  __half2* t2b = reinterpret_cast<__half2*>(reinterpret_cast<unsigned char*>(spec) + G::T2B_OFF);
  for (int idx = tid; idx < R; idx += nt) {                  // T2 = w^{32 n3 k2} in both index orders
    const int k2 = idx / N3, n3 = idx % N3;
    double sn, cs;
    sincospi(2.0 * 32.0 * n3 * k2 / N, &sn, &cs);
    const __half2 v = __floats2half2_rn((float)cs, (float)(-sn));
    t2a[k2 * N3 + n3] = v;
    t2b[n3 * N2 + k2] = v;
  }
}

// The spectrum of a long filter has a large dynamic range (its DC gain grows with the length) and fp16
// tops out at 65504, so every channel's bins are stored multiplied by a power of two 2^e that brings the
// largest component just below 1; the convolution kernel multiplies its float32 result by 2^-e (stored
// per channel after the bins).  Power-of-two factors change no mantissa bit.
__device__ __forceinline__ float gain_scale(float gmax) {
  if (!(gmax > 0.f) || !isfinite(gmax)) return 1.f;
  int e;
  frexpf(gmax, &e);                      // gmax = m * 2^e, m in [0.5, 1)
  return ldexpf(1.f, -e);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
    for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
    if (threadIdx.x == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

// One CTA per channel: N-point complex FFT (decimation in frequency) in shared memory of
// g[n] w^{n/2}, g = the filter with its wrapped half negated; bins gathered in table order.
template <typename G>
__global__ void __launch_bounds__(512)
spectrum_kind2_kernel(const float* __restrict__ kfilt, float* __restrict__ spec, int D, int R) {
  constexpr int N = G::N, N2 = G::N2, N3 = G::N3;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x, nt = blockDim.x;
  if (blockIdx.x == (unsigned)D) { write_header<G>(spec, tid, nt); return; }
  float2* s = reinterpret_cast<float2*>(smem_raw);
  const int c = blockIdx.x;
  // the filter row has period R <= N ([forward taps | zeros | reversed backward taps]): its first half
  // stays at the start, its wrapped half moves to the end of the length-N period
  const float* row = kfilt + (size_t)c * R;
  for (int n = tid; n < N; n += nt) {
    double sn, cs;
    sincospi((double)n / N, &sn, &cs);                         // w^{n/2} = cos(pi n / N) - i sin(pi n / N)
    const double tap = n < R / 2 ? (double)row[n] : (n >= N - R / 2 ? (double)row[n - N + R] : 0.0);
    const double g = (n < N / 2) ? tap : -tap;
    s[n] = make_float2((float)(g * cs), (float)(-g * sn));
  }
  __syncthreads();
  for (int h = N / 2; h >= 1; h >>= 1) {
    for (int j = tid; j < N / 2; j += nt) {
      const int g = j / h, pos = j % h;
      float2* base = s + g * 2 * h + pos;
      float sn, cs;
      sincospif((float)pos / (float)h, &sn, &cs);              // W_{2h}^{pos}
      const float2 a = base[0], b = base[h];
      const float dx = a.x - b.x, dy = a.y - b.y;
      base[0] = make_float2(a.x + b.x, a.y + b.y);
      base[h] = make_float2(dx * cs + dy * sn, dy * cs - dx * sn);
    }
    __syncthreads();
  }
  // largest |Re|, |Im| over the stored half of the spectrum decides the channel's scale 2^e (see gain_scale)
  float gmax = 0.f;
  for (int idx = tid; idx < N / 2; idx += nt) {
    const int k3 = idx % N3, k2 = (idx / N3) % N2, k1 = idx / (N3 * N2);
    const int p = (int)(__brev((unsigned)(k1 + 32 * k2 + 32 * N2 * k3)) >> (32 - G::LG));
    gmax = fmaxf(gmax, fmaxf(fabsf(s[p].x), fabsf(s[p].y)));
  }
  __shared__ float red[32];
  gmax = block_max(gmax, red);
  const float sc = gain_scale(gmax * G::KAPPA);
  if (tid == 0) spec[G::HDR_FLOATS + (size_t)D * (N / 2) + c] = 1.0f / sc;
  __half2* Gt = reinterpret_cast<__half2*>(spec + G::HDR_FLOATS) + (size_t)c * (N / 2);
  for (int idx = tid; idx < N / 2; idx += nt) {
    const int k3 = idx % N3, k2 = (idx / N3) % N2, k1 = idx / (N3 * N2);
    const int k = k1 + 32 * k2 + 32 * N2 * k3;
    const int p = (int)(__brev((unsigned)k) >> (32 - G::LG));
    Gt[idx] = __floats2half2_rn(s[p].x * (G::KAPPA * sc), s[p].y * (G::KAPPA * sc));
  }
}

// N = 65536: the transform no longer fits one CTA.  The real filter is packed as
// z[m] = g[2m] + i g[2m+1] (M = N/2 points), transformed at odd frequencies by a cluster of
// two CTAs (each holds half of the M points; only the first decimation-in-frequency stage
// crosses halves and it reads its inputs straight from global memory), and un-packed with
//   E[k] = (Z[k] + conj Z[M-1-k]) / 2,  O[k] = (Z[k] - conj Z[M-1-k]) / 2i,
//   G[k] = E[k] + w^{k+1/2} O[k],   G[k+M] = E[k] - w^{k+1/2} O[k],
// where the partner bin M-1-k always lives in the other CTA (read through distributed
// shared memory).
template <typename G>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(512)
spectrum_kind2_cluster_kernel(const float* __restrict__ kfilt, float* __restrict__ spec, int D, int R) {
  namespace cg = cooperative_groups;
  constexpr int N = G::N, M = N / 2, Mh = M / 2, N2 = G::N2, N3 = G::N3, LGM = G::LG - 1;
  cg::cluster_group cluster = cg::this_cluster();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float2* s = reinterpret_cast<float2*>(smem_raw);            // local half: positions q*Mh + [0, Mh)
  const int tid = threadIdx.x, nt = blockDim.x;
  const int q = (int)cluster.block_rank();
  const int c = blockIdx.x >> 1;
  if (c == D) {
    if (q == 0) write_header<G>(spec, tid, nt);
    cluster.sync();
    cluster.sync();
    cluster.sync();
    return;
  }
  const float* row = kfilt + (size_t)c * R;                    // period R <= N, see spectrum_kind2_kernel
  auto tap = [&](int n) -> double {
    return n < R / 2 ? (double)row[n] : (n >= N - R / 2 ? (double)row[n - N + R] : 0.0);
  };
  // packed, pre-twisted input x[m] = z[m] W_M^{m/2}; first stage pairs m and m + Mh
  for (int i = tid; i < Mh; i += nt) {
    float2 x[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int m = i + e * Mh;
      const double sg = (2 * m < N / 2) ? 1.0 : -1.0;          // wrapped half of the filter negated
      const double zr = sg * tap(2 * m), zi = sg * tap(2 * m + 1);
      double sn, cs;
      sincospi((double)m / M, &sn, &cs);                       // W_M^{m/2} = cos(pi m / M) - i sin(pi m / M)
      x[e] = make_float2((float)(zr * cs + zi * sn), (float)(zi * cs - zr * sn));
    }
    if (q == 0) {
      s[i] = make_float2(x[0].x + x[1].x, x[0].y + x[1].y);
    } else {
      float sn, cs;
      sincospif((float)i / (float)Mh, &sn, &cs);               // W_M^{i}
      const float dx = x[0].x - x[1].x, dy = x[0].y - x[1].y;
      s[i] = make_float2(dx * cs + dy * sn, dy * cs - dx * sn);
    }
  }
  __syncthreads();
  for (int h = Mh / 2; h >= 1; h >>= 1) {
    for (int j = tid; j < Mh / 2; j += nt) {
      const int g = j / h, pos = j % h;
      float2* base = s + g * 2 * h + pos;
      float sn, cs;
      sincospif((float)pos / (float)h, &sn, &cs);
      const float2 a = base[0], b = base[h];
      const float dx = a.x - b.x, dy = a.y - b.y;
      base[0] = make_float2(a.x + b.x, a.y + b.y);
      base[h] = make_float2(dx * cs + dy * sn, dy * cs - dx * sn);
    }
    __syncthreads();
  }
  cluster.sync();
  // bin kappa of the M-point transform sits at global position rev_M(kappa): CTA = kappa & 1
  const float2* other = cluster.map_shared_rank(s, q ^ 1);
  __half2* Gt = reinterpret_cast<__half2*>(spec + G::HDR_FLOATS) + (size_t)c * (N / 2);
  __shared__ float red[32];
  __shared__ float cta_max;
  // two passes over this CTA's bins: the first finds the channel's largest component (combined with the
  // other CTA's through distributed shared memory), the second stores the scaled bins
  float sc = 1.f;
  for (int pass = 0; pass < 2; ++pass) {
    float gmax = 0.f;
    for (int idx = tid; idx < N / 2; idx += nt) {
      const int k3 = idx % N3, k2 = (idx / N3) % N2, k1 = idx / (N3 * N2);
      const int k = k1 + 32 * k2 + 32 * N2 * k3;
      const int kap = k & (M - 1);
      if ((kap & 1) != q) continue;
      const int pk = (int)(__brev((unsigned)kap) >> (32 - LGM)) - q * Mh;
      const int pm = (int)(__brev((unsigned)(M - 1 - kap)) >> (32 - LGM)) - (q ^ 1) * Mh;
      const float2 Zk = s[pk], Zp = other[pm];
      const float2 E = make_float2(0.5f * (Zk.x + Zp.x), 0.5f * (Zk.y - Zp.y));
      const float2 O = make_float2(0.5f * (Zk.y + Zp.y), -0.5f * (Zk.x - Zp.x));     // (Zk - conj Zp) / 2i
      double snd, csd;
      sincospi(2.0 * (kap + 0.5) / N, &snd, &csd);               // w^{kap + 1/2} = cos - i sin
      const float cs = (float)csd, sn = (float)snd;
      const float2 wO = make_float2(O.x * cs + O.y * sn, O.y * cs - O.x * sn);
      const float sg = (k >= M) ? -1.f : 1.f;
      const float gr = E.x + sg * wO.x, gi = E.y + sg * wO.y;
      if (pass == 0) gmax = fmaxf(gmax, fmaxf(fabsf(gr), fabsf(gi)));
      else Gt[idx] = __floats2half2_rn(gr * (G::KAPPA * sc), gi * (G::KAPPA * sc));
    }
    if (pass == 0) {
      gmax = block_max(gmax, red);
      if (tid == 0) cta_max = gmax;
      cluster.sync();
      const float om = *cluster.map_shared_rank(&cta_max, q ^ 1);
      sc = gain_scale(fmaxf(gmax, om) * G::KAPPA);
      if (tid == 0 && q == 0) spec[G::HDR_FLOATS + (size_t)D * (N / 2) + c] = 1.0f / sc;
    }
  }
  cluster.sync();
}

// ---------------------------------------------------------------------------------------
struct Params {
  int B, L, D, nf, rows;
  int u_f16, yu_bf16;                               // 2-byte u holds fp16 (not bf16); round the residual conv to bf16
  const __nv_bfloat16* xin; long long xsb, xsc;      // (b, channel) row start = xin + b*xsb + ch*xsc, time stride 1
  const void* u; long long usb, usc;
  __nv_bfloat16* out; long long osb, osc;
  const float* sw; const float* sb;
  const float* spec[2]; const float* bias[2];
};

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_h2(uint32_t u) { return __half22float2(*reinterpret_cast<__half2*>(&u)); }
__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t a) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(a) : "memory");
}
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float2 cmulf(float2 x, float2 w) { return make_float2(x.x * w.x - x.y * w.y, x.x * w.y + x.y * w.x); }

// depthwise 3-tap conv over 4 consecutive time steps of one channel
struct Taps { float w0, w1, w2, b; };
__device__ __forceinline__ Taps load_taps(const float* sw, const float* sb, int ch) {
  Taps T;
  T.w0 = bf16r(__ldg(sw + 3 * ch)); T.w1 = bf16r(__ldg(sw + 3 * ch + 1)); T.w2 = bf16r(__ldg(sw + 3 * ch + 2));
  T.b = bf16r(__ldg(sb + ch));
  return T;
}
// x6 = {x[t0-2], x[t0-1], x[t0], .., x[t0+3]} -> bf16-rounded conv outputs at t0..t0+3
__device__ __forceinline__ void conv4(const Taps& T, const float (&x6)[6], float (&y)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) y[j] = bf16r(fmaf(T.w2, x6[j + 2], fmaf(T.w1, x6[j + 1], fmaf(T.w0, x6[j], T.b))));
}
// loads x[t0-2 .. t0+3] of a time-contiguous bf16 row (t0 % 4 == 0); positions outside [0, L) read as 0
__device__ __forceinline__ void load6(const __nv_bfloat16* row, int t0, int L, float (&x6)[6]) {
  uint32_t h = 0;
  uint2 v = make_uint2(0u, 0u);
  if (t0 >= 2 && t0 - 2 < L) h = __ldg(reinterpret_cast<const uint32_t*>(row + t0 - 2));
  if (t0 < L) v = __ldg(reinterpret_cast<const uint2*>(row + t0));
  x6[0] = bf_lo(h); x6[1] = bf_hi(h);
  x6[2] = bf_lo(v.x); x6[3] = bf_hi(v.x); x6[4] = bf_lo(v.y); x6[5] = bf_hi(v.y);
}

// MMAs of one stage: 0 F1, 1 DFT_N2, 2 DFT_N3, 3 DFT_N3 (on conjugated data = inverse),
// 4 DFT_N2 (inverse), 5 I1
template <typename G>
__device__ __forceinline__ void issue_stage(int stage, uint32_t tm, uint32_t data, uint32_t hdr) {
  constexpr int K2 = G::K2, K3 = G::K3;
  if (stage == 0) {
    constexpr uint32_t id = tc::make_idesc(128, 32, 0);
    const uint64_t dB = tc::smem_desc_k_nosw(hdr + G::F1_OFF, 128, 16 * 16);
#pragma unroll
    for (int t = 0; t < G::TR; ++t)
      tc::mma_ss(tm + 32 * t, tc::smem_desc_k_nosw(data + t * G::A1_TILE, G::A1_LBO, G::A1_SBO), dB, id, 0);
  } else if (stage == 1 || stage == 4) {
    constexpr uint32_t id = tc::make_idesc(128, K2, 0);
#pragma unroll
    for (int t = 0; t < G::T2T; ++t)
#pragma unroll
      for (int s = 0; s < K2 / 16; ++s)
        tc::mma_ss(tm + K2 * t, tc::smem_desc_k_nosw(data + t * G::A2_TILE + s * 2 * G::A2_LBO, G::A2_LBO, G::A2_SBO),
                   tc::smem_desc_k_nosw(hdr + G::F2_OFF + s * 256, 128, K2 * 16), id, s ? 1u : 0u);
  } else if (stage == 2 || stage == 3) {
    constexpr uint32_t id = tc::make_idesc(128, K3, 0);
#pragma unroll
    for (int t = 0; t < G::T3T; ++t)
#pragma unroll
      for (int s = 0; s < K3 / 16; ++s)
        tc::mma_ss(tm + K3 * t, tc::smem_desc_k_nosw(data + t * G::A3_TILE + s * 2 * G::A3_LBO, G::A3_LBO, G::A3_SBO),
                   tc::smem_desc_k_nosw(hdr + G::F3_OFF + s * 256, 128, K3 * 16), id, s ? 1u : 0u);
  } else {
    constexpr uint32_t id = tc::make_idesc(128, 16, 0);
#pragma unroll
    for (int t = 0; t < G::TR; ++t)
#pragma unroll
      for (int s = 0; s < 2; ++s)
        tc::mma_ss(tm + 16 * t, tc::smem_desc_k_nosw(data + t * G::A6_TILE + s * 2 * G::A6_LBO, G::A6_LBO, G::A6_SBO),
                   tc::smem_desc_k_nosw(hdr + G::I1_OFF + s * 256, 128, 32 * 16), id, s ? 1u : 0u);
  }
}

template <typename G, typename TU>
__global__ void __launch_bounds__(G::THREADS, 1)
longconv_tcl_kernel(const Params P) {
  constexpr int N2 = G::N2, N3 = G::N3, R = G::R, K2 = G::K2, K3 = G::K3, TS = G::TS, TPS = G::TPS;
  constexpr int CH = R / 4;                                  // 4-wide time chunks per n1 block
  constexpr int GROUPS = (TPS > CH) ? TPS / CH : 1;          // n1 groups when a slot has more threads than chunks
  constexpr int NP = 16 / GROUPS;                            // n1 values per thread and chunk in the load / store phases
  constexpr int CPT = (CH > TPS) ? CH / TPS : 1;             // chunks per thread
  static_assert(NP >= 4 && NP % 4 == 0, "n1 group must be a multiple of 4");
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
  unsigned char* hdrb = smem + G::SLOTS * G::DATA_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(hdrb + G::HDR_BYTES);       // per slot: ops, mma, w
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * G::SLOTS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slot = tid / TPS;
  const int sl = tid % TPS;                      // thread index inside the slot
  const int l = sl & 127;                        // TMEM lane = row within every 128-row tile
  const int ts = sl >> 7;                        // which share of the row tiles this thread handles
  if (tid == 0) {
    for (int s = 0; s < G::SLOTS; ++s) {
      tc::mbar_init(bars + 3 * s, TPS);
      tc::mbar_init(bars + 3 * s + 1, 1);
      tc::mbar_init(bars + 3 * s + 2, TPS);
    }
    *abort_flag = 0;
    tc::mbar_fence_init();
  }
  {
    const uint4* src = reinterpret_cast<const uint4*>(P.spec[0]);
    uint4* dst = reinterpret_cast<uint4*>(hdrb);
    for (int i = tid; i < G::HDR_BYTES / 16; i += G::THREADS) dst[i] = __ldg(src + i);
    tc::fence_proxy_async_smem();
  }
  if (warp == 0) {
    tc::tmem_alloc(tmem_slot, G::TCOLS);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  uint64_t* bar_ops = bars + 3 * slot;
  uint64_t* bar_mma = bar_ops + 1;
  uint64_t* bar_w = bar_ops + 2;
  const uint32_t tm = *tmem_slot + slot * G::COLS;
  const uint32_t tml = tm + ((uint32_t)((warp & 3) * 32) << 16);
  const uint32_t data = tc::smem_u32(smem + slot * G::DATA_BYTES);
  float* Y = reinterpret_cast<float*>(smem + slot * G::DATA_BYTES);
  const uint32_t hdr = tc::smem_u32(hdrb);
  const uint32_t t1s = hdr + G::T1_OFF, t2a = hdr + G::T2A_OFF, t2b = hdr + G::T2B_OFF;
  const uint32_t lrow = (uint32_t)((l >> 3) * 1 /* x SBO */), lsub = (uint32_t)((l & 7) * 16);
  uint32_t ph_ops = 0, ph_mma = 0, ph_w = 0;
  bool ok = true;

#define LCL_STAGE(stage_)                                                                             \
  tc::fence_proxy_async_smem();                                                                       \
  tc::mbar_arrive(bar_ops);                                                                           \
  if (sl == 0) {                                                                                      \
    if (tc::mbar_wait(bar_ops, ph_ops, abort_flag, tc::ST_TIMEOUT_MMA)) {                             \
      tc::tc_fence_after();                                                                           \
      issue_stage<G>(stage_, tm, data, hdr);                                                          \
      tc::mma_commit(bar_mma);                                                                        \
    }                                                                                                 \
    ph_ops ^= 1;                                                                                      \
  }                                                                                                   \
  if (!__all_sync(0xffffffffu, tc::mbar_wait(bar_mma, ph_mma, abort_flag, tc::ST_TIMEOUT_EPI))) { ok = false; break; } \
  ph_mma ^= 1;                                                                                        \
  tc::tc_fence_after();
#define LCL_BARRIER()                                                                                 \
  tc::mbar_arrive(bar_w);                                                                             \
  if (!__all_sync(0xffffffffu, tc::mbar_wait(bar_w, ph_w, abort_flag, tc::ST_TIMEOUT_EPI))) { ok = false; break; } \
  ph_w ^= 1;

  for (int rowid = blockIdx.x * G::SLOTS + slot; rowid < P.rows && ok; rowid += gridDim.x * G::SLOTS) {
    const int ch = rowid % P.D, b = rowid / P.D;
    const __nv_bfloat16* x1row = P.xin + (long long)b * P.xsb + (long long)ch * P.xsc;
    const __nv_bfloat16* x2row = x1row + (long long)P.D * P.xsc;
    const __nv_bfloat16* vrow = x2row + (long long)P.D * P.xsc;
    __nv_bfloat16* orow = P.out + (long long)b * P.osb + (long long)ch * P.osc;
    const TU* urow = reinterpret_cast<const TU*>(P.u) + (long long)b * P.usb + (long long)ch * P.usc;

    for (int f = 0; f < P.nf && ok; ++f) {
      // ---------------- F1 operands: a[R n1 + r] as fp16 at (row r, k = n1) ----------------
#pragma unroll 1
      for (int cc = 0; cc < CPT; ++cc) {
        const int pc = (sl % CH) + cc * TPS, pg = (CH >= TPS) ? 0 : sl / CH;
        const int r0 = 4 * pc, n1_0 = pg * NP;
        uint32_t hv[4][NP / 2];                              // [j = r - r0][n1 pair]
        if (f == 0) {
          const Taps Tx = load_taps(P.sw, P.sb, ch), Tv = load_taps(P.sw, P.sb, 2 * P.D + ch);
#pragma unroll
          for (int i = 0; i < NP; i += 2) {
            float a[2][4];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int t0 = R * (n1_0 + i + e) + r0;
              float x6[6], v6[6], cx[4], cv[4];
              load6(x1row, t0, P.L, x6);
              load6(vrow, t0, P.L, v6);
              conv4(Tx, x6, cx);
              conv4(Tv, v6, cv);
#pragma unroll
              for (int j = 0; j < 4; ++j) a[e][j] = (t0 < P.L) ? bf16r(cv[j] * cx[j]) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) hv[j][i >> 1] = pack_h2(a[0][j], a[1][j]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < NP; i += 2) {
            float a[2][4];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int t0 = R * (n1_0 + i + e) + r0;
              a[e][0] = a[e][1] = a[e][2] = a[e][3] = 0.f;
              if (t0 < P.L) {
                if (sizeof(TU) == 4) {
                  const float4 v = __ldg(reinterpret_cast<const float4*>(urow + t0));
                  a[e][0] = v.x; a[e][1] = v.y; a[e][2] = v.z; a[e][3] = v.w;
                } else {
                  const uint2 v = __ldg(reinterpret_cast<const uint2*>(urow + t0));
                  if (P.u_f16) {
                    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
                    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
                    a[e][0] = lo.x; a[e][1] = lo.y; a[e][2] = hi.x; a[e][3] = hi.y;
                  } else {
                    a[e][0] = bf_lo(v.x); a[e][1] = bf_hi(v.x); a[e][2] = bf_lo(v.y); a[e][3] = bf_hi(v.y);
                  }
                }
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) hv[j][i >> 1] = pack_h2(a[0][j], a[1][j]);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = r0 + j;
          const uint32_t ro = data + (r >> 7) * G::A1_TILE + ((r & 127) >> 3) * G::A1_SBO + (r & 7) * 16;
#pragma unroll
          for (int q = 0; q < NP / 4; ++q) {
            const int k = n1_0 + 4 * q;
            sts64(ro + (k >> 3) * G::A1_LBO + (k & 7) * 2, hv[j][2 * q], hv[j][2 * q + 1]);
          }
        }
      }
      LCL_STAGE(0)

      // ---------------- hop 1: x T1, rows (n2, n3) -> rows (k1, n3), k = (n2, ri) ----------------
#pragma unroll 1
      for (int t = ts; t < G::TR; t += TS) {
        const int r = 128 * t + l, n2 = r / N3, n3 = r % N3;
        // thread part of the destination: row group / row of n3, K position of n2
        const uint32_t dst = data + (n3 >> 3) * G::A2_SBO + (n3 & 7) * 16 + (n2 >> 2) * G::A2_LBO + (n2 & 3) * 4;
        const uint32_t tw = G::SPLIT_T1 ? 0u : t1s + r * 4;
#pragma unroll
        for (int hq = 0; hq < 2; ++hq) {
          uint32_t z[16];
          tc::tmem_ld16(tml + 32 * t + 16 * hq, z);
          tc::tmem_ld_wait();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            constexpr int KPT = 128 / N3;                    // k1 values per 128-row tile of the destination
            const int k1 = 8 * hq + kk;
            float2 w;
            if (G::SPLIT_T1) w = cmulf(unpack_h2(lds32(t1s + (k1 * N2 + n2) * 4)), unpack_h2(lds32(t1s + (16 * N2 + k1 * N3 + n3) * 4)));
            else w = unpack_h2(lds32(tw + k1 * R * 4));
            const float2 y = cmulf(make_float2(__uint_as_float(z[2 * kk]), __uint_as_float(z[2 * kk + 1])), w);
            sts32(dst + (k1 / KPT) * G::A2_TILE + (k1 % KPT) * G::G3 * G::A2_SBO, pack_h2(y.x, y.y));
          }
        }
      }
      tc::tc_fence_before();
      LCL_STAGE(1)

      // ---------------- hop 2: x T2, rows (k1, n3) -> rows (k1, k2), k = (n3, ri) ----------------
#pragma unroll 1
      for (int t = ts; t < G::T2T; t += TS) {
        constexpr int KPT = 128 / N2 > 0 ? 128 / N2 : 1;     // k1 values per 128-row tile of the destination (N2 <= 128)
        const int rho = 128 * t + l, k1 = rho / N3, n3 = rho % N3;
        const uint32_t dst = data + (k1 / KPT) * G::A3_TILE + (k1 % KPT) * G::G2 * G::A3_SBO +
                             (n3 >> 2) * G::A3_LBO + (n3 & 3) * 4;
        const uint32_t tw = t2a + n3 * 4;
#pragma unroll
        for (int c0 = 0; c0 < K2; c0 += 16) {
          uint32_t z[16];
          tc::tmem_ld16(tml + K2 * t + c0, z);
          tc::tmem_ld_wait();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const int k2 = c0 / 2 + kk;
            const float2 w = unpack_h2(lds32(tw + k2 * N3 * 4));
            const float2 y = cmulf(make_float2(__uint_as_float(z[2 * kk]), __uint_as_float(z[2 * kk + 1])), w);
            sts32(dst + (k2 >> 3) * G::A3_SBO + (k2 & 7) * 16, pack_h2(y.x, y.y));
          }
        }
      }
      tc::tc_fence_before();
      LCL_STAGE(2)

      // ---------------- hop 3: conj(Z (G + bias)); rows (k1, k2) keep their place, k = (k3, ri) ----------------
      {
        const uint32_t* Gt = reinterpret_cast<const uint32_t*>(P.spec[f] + G::HDR_FLOATS) + (size_t)ch * (G::N / 2);
        const float inv_gain = __ldg(P.spec[f] + G::HDR_FLOATS + (size_t)P.D * (G::N / 2) + ch);   // 2^-e of this channel
        const float bk = __ldg(P.bias[f] + ch) * G::KAPPA / inv_gain;
#pragma unroll 1
        for (int t = ts; t < G::T3T; t += TS) {
          const int rho = 128 * t + l;
          const uint32_t dst = data + t * G::A3_TILE + (l >> 3) * G::A3_SBO + (l & 7) * 16;
#pragma unroll
          for (int c0 = 0; c0 < K3; c0 += 16) {
            uint32_t z[16];
            tc::tmem_ld16(tml + K3 * t + c0, z);
            const uint4 g0 = __ldg(reinterpret_cast<const uint4*>(Gt + rho * N3 + c0 / 2));
            const uint4 g1 = __ldg(reinterpret_cast<const uint4*>(Gt + rho * N3 + c0 / 2 + 4));
            tc::tmem_ld_wait();
            const uint32_t gw[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            uint32_t o[8];
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              float2 g = unpack_h2(gw[kk]);
              g.x += bk;
              const float2 y = cmulf(make_float2(__uint_as_float(z[2 * kk]), __uint_as_float(z[2 * kk + 1])), g);
              o[kk] = pack_h2(y.x, -y.y);
            }
            sts128(dst + (c0 >> 3) * G::A3_LBO, o[0], o[1], o[2], o[3]);
            sts128(dst + ((c0 >> 3) + 1) * G::A3_LBO, o[4], o[5], o[6], o[7]);
          }
        }
      }
      tc::tc_fence_before();
      LCL_STAGE(3)

      // ---------------- hop 4: x T2, rows (k1, k2) -> rows (k1, n3), k = (k2, ri) ----------------
#pragma unroll 1
      for (int t = ts; t < G::T3T; t += TS) {
        constexpr int KPT = 128 / N3;
        const int rho = 128 * t + l, k1 = rho / N2, k2 = rho % N2;
        const uint32_t dst = data + (k1 / KPT) * G::A2_TILE + (k1 % KPT) * G::G3 * G::A2_SBO +
                             (k2 >> 2) * G::A2_LBO + (k2 & 3) * 4;
        const uint32_t tw = t2b + k2 * 4;
#pragma unroll
        for (int c0 = 0; c0 < K3; c0 += 16) {
          uint32_t z[16];
          tc::tmem_ld16(tml + K3 * t + c0, z);
          tc::tmem_ld_wait();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const int n3 = c0 / 2 + kk;
            const float2 w = unpack_h2(lds32(tw + n3 * N2 * 4));
            const float2 y = cmulf(make_float2(__uint_as_float(z[2 * kk]), __uint_as_float(z[2 * kk + 1])), w);
            sts32(dst + (n3 >> 3) * G::A2_SBO + (n3 & 7) * 16, pack_h2(y.x, y.y));
          }
        }
      }
      tc::tc_fence_before();
      LCL_STAGE(4)

      // ---------------- hop 5: x T1, rows (k1, n3) -> rows r = (n2, n3), k = (k1, ri) ----------------
#pragma unroll 1
      for (int t = ts; t < G::T2T; t += TS) {
        constexpr int NPT = 128 / N3;                        // n2 values per 128-row tile of the destination
        const int rho = 128 * t + l, k1 = rho / N3, n3 = rho % N3;
        const uint32_t dst = data + (n3 >> 3) * G::A6_SBO + (n3 & 7) * 16 + (k1 >> 2) * G::A6_LBO + (k1 & 3) * 4;
        const uint32_t tw = G::SPLIT_T1 ? t1s + (k1 * N2) * 4 : t1s + (k1 * R + n3) * 4;
        float2 wb = make_float2(1.f, 0.f);
        if (G::SPLIT_T1) wb = unpack_h2(lds32(t1s + (16 * N2 + k1 * N3 + n3) * 4));
#pragma unroll
        for (int c0 = 0; c0 < K2; c0 += 16) {
          uint32_t z[16];
          tc::tmem_ld16(tml + K2 * t + c0, z);
          tc::tmem_ld_wait();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const int n2 = c0 / 2 + kk;
            float2 w;
            if (G::SPLIT_T1) w = cmulf(unpack_h2(lds32(tw + n2 * 4)), wb);
            else w = unpack_h2(lds32(tw + n2 * N3 * 4));
            const float2 y = cmulf(make_float2(__uint_as_float(z[2 * kk]), __uint_as_float(z[2 * kk + 1])), w);
            sts32(dst + (n2 / NPT) * G::A6_TILE + (n2 % NPT) * G::G3 * G::A6_SBO, pack_h2(y.x, y.y));
          }
        }
      }
      tc::tc_fence_before();
      LCL_STAGE(5)

      // ---------------- hop 6: y[R n1 + r] (float32) into shared memory in time order ----------------
#pragma unroll 1
      for (int t = ts; t < G::TR; t += TS) {
        uint32_t z[16];
        tc::tmem_ld16(tml + 16 * t, z);
        tc::tmem_ld_wait();
#pragma unroll
        for (int n1 = 0; n1 < 16; ++n1) Y[R * n1 + 128 * t + l] = __uint_as_float(z[n1]);
      }
      tc::tc_fence_before();
      LCL_BARRIER()

      // ---------------- epilogue: gate / residual add; 8-byte stores along time ----------------
      const float inv_gain = __ldg(P.spec[f] + G::HDR_FLOATS + (size_t)P.D * (G::N / 2) + ch);     // undo the table's 2^e
#pragma unroll 1
      for (int cc = 0; cc < CPT; ++cc) {
        const int pc = (sl % CH) + cc * TPS, pg = (CH >= TPS) ? 0 : sl / CH;
        const int r0 = 4 * pc, n1_0 = pg * NP;
        if (f == 0) {
          const Taps T2 = load_taps(P.sw, P.sb, P.D + ch);
#pragma unroll
          for (int i = 0; i < NP; ++i) {
            const int t0 = R * (n1_0 + i) + r0;
            if (t0 < P.L) {
              float x6[6], c2[4];
              load6(x2row, t0, P.L, x6);
              conv4(T2, x6, c2);
              const float4 y = *reinterpret_cast<const float4*>(Y + t0);
              const float yv[4] = {y.x * inv_gain, y.y * inv_gain, y.z * inv_gain, y.w * inv_gain};
              float o[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) o[j] = bf16r(yv[j]) * c2[j];      // (conv + bias term) cast, then the gate
              *reinterpret_cast<uint2*>(orow + t0) = make_uint2(pack_bf2(o[0], o[1]), pack_bf2(o[2], o[3]));
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < NP; ++i) {
            const int t0 = R * (n1_0 + i) + r0;
            if (t0 < P.L) {
              const float4 y = *reinterpret_cast<const float4*>(Y + t0);
              float yv[4] = {y.x * inv_gain, y.y * inv_gain, y.z * inv_gain, y.w * inv_gain};
              if (P.yu_bf16) {                                 // bf16 layer input: yu is cast to bf16 first
#pragma unroll
                for (int j = 0; j < 4; ++j) yv[j] = bf16r(yv[j]);
              }
              uint2* po = reinterpret_cast<uint2*>(orow + t0);
              const uint2 prev = *po;                          // y * x2 written by this thread for f == 0
              *po = make_uint2(pack_bf2(bf_lo(prev.x) + yv[0], bf_hi(prev.x) + yv[1]),
                               pack_bf2(bf_lo(prev.y) + yv[2], bf_hi(prev.y) + yv[3]));
            }
          }
        }
      }
      LCL_BARRIER()                                          // the y buffer is free again
    }
  }
#undef LCL_STAGE
#undef LCL_BARRIER
  (void)lrow; (void)lsub;

  __syncthreads();
  if (warp == 0) {
    tc::tc_fence_after();
    tc::tmem_dealloc(*tmem_slot, G::TCOLS);
  }
}

using Geo4k = Geo<16, 8, 4, 1>;
using Geo16k = Geo<32, 16, 4, 2>;
using Geo64k = Geo<64, 32, 1, 4>;

template <typename G>
static int launch_spectrum(int D, int R, const float* k, float* spec, cudaStream_t st) {
  if (G::N <= 16384) {
    auto kern = spectrum_kind2_kernel<G>;
    const size_t smem = (size_t)G::N * sizeof(float2);
    M2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<D + 1, 512, smem, st>>>(k, spec, D, R);
  } else {
    auto kern = spectrum_kind2_cluster_kernel<G>;
    const size_t smem = (size_t)(G::N / 4) * sizeof(float2);
    M2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<2 * (D + 1), 512, smem, st>>>(k, spec, D, R);
  }
  M2_LAUNCH_CHECK("spectrum_kind2_kernel");
  return M2_OK;
}

template <typename G, typename TU>
static int launch_conv(const Params& P, cudaStream_t st) {
  auto kern = longconv_tcl_kernel<G, TU>;
  M2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM));
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int need = (P.rows + G::SLOTS - 1) / G::SLOTS;
  const int grid = need < sms ? need : sms;
  kern<<<grid, G::THREADS, G::SMEM, st>>>(P);
  M2_LAUNCH_CHECK("longconv_tcl_kernel");
  return M2_OK;
}

}  // namespace lcl

// 2 when the long-row tensor-core family covers (seq_len, dtype); the caller must then
// supply time-contiguous tensors
int longconv_tcl_supported(int seq_len, m2_dtype act_dtype) {
  if (act_dtype != M2_BF16 || seq_len % 4 != 0) return 0;
  return seq_len > 512 && seq_len <= 32768;      // transform length 4096 up to 2048, 16384 up to 8192, else 65536
}

// header + per channel N/2 half2 bins + per channel one float (2^-e, see gain_scale)
size_t spectrum_kind2_floats(int D, int L) {
  if (L <= 2048) return (size_t)lcl::Geo4k::HDR_FLOATS + (size_t)(lcl::Geo4k::N / 2 + 1) * D;
  if (L <= 8192) return (size_t)lcl::Geo16k::HDR_FLOATS + (size_t)(lcl::Geo16k::N / 2 + 1) * D;
  return (size_t)lcl::Geo64k::HDR_FLOATS + (size_t)(lcl::Geo64k::N / 2 + 1) * D;
}

int spectrum_kind2_launch(int D, int L, const float* k, float* spec, cudaStream_t st) {
  M2_REQUIRE(longconv_tcl_supported(L, M2_BF16), M2_ERR_UNSUPPORTED,
             "m2_filter_spectrum: kind 2 covers 512 < seq_len <= 32768, multiples of 4");
  const int R = m2_filter_row_len(L);
  if (L <= 2048) return lcl::launch_spectrum<lcl::Geo4k>(D, R, k, spec, st);
  if (L <= 8192) return lcl::launch_spectrum<lcl::Geo16k>(D, R, k, spec, st);
  return lcl::launch_spectrum<lcl::Geo64k>(D, R, k, spec, st);
}

int longconv_tcl_launch(const m2_longconv_args* a, cudaStream_t st) {
  using namespace lcl;
  M2_REQUIRE(longconv_tcl_supported(a->seq_len, a->act_dtype), M2_ERR_UNSUPPORTED,
             "m2_longconv_fwd: kind 2 needs bf16 activations and 512 < seq_len <= 32768, a multiple of 4");
  M2_REQUIRE(a->xin_st == 1 && a->out_st == 1 && (a->n_filters == 1 || a->u_st == 1), M2_ERR_UNSUPPORTED,
             "m2_longconv_fwd: kind 2 needs time-contiguous tensors ((batch, channel, time) layout)");
  M2_REQUIRE(a->xin_sc % 4 == 0 && a->xin_sb % 4 == 0 && a->out_sc % 4 == 0 && a->out_sb % 4 == 0 &&
             m2_aligned(a->xin, 8) && m2_aligned(a->out, 8), M2_ERR_ALIGN,
             "m2_longconv_fwd: kind 2 needs 8-byte aligned rows of xin and out");
  Params P;
  P.B = a->batch; P.L = a->seq_len; P.D = a->d_model; P.nf = a->n_filters;
  P.rows = a->batch * a->d_model;
  P.xin = (const __nv_bfloat16*)a->xin; P.xsb = a->xin_sb; P.xsc = a->xin_sc;
  P.u = a->u; P.usb = a->u_sb; P.usc = a->u_sc;
  P.out = (__nv_bfloat16*)a->out; P.osb = a->out_sb; P.osc = a->out_sc;
  P.sw = a->short_w; P.sb = a->short_b;
  for (int f = 0; f < 2; ++f) { P.spec[f] = a->spec[f]; P.bias[f] = a->bias[f]; }
  // 2-byte residual input: bf16, or the fp16 time-major copy a LayerNorm / m2_time_major_f16 wrote
  const bool ubf = a->n_filters == 2 && (a->u_dtype == M2_BF16 || a->u_dtype == M2_F16);
  P.u_f16 = a->n_filters == 2 && a->u_dtype == M2_F16;
  P.yu_bf16 = a->n_filters == 2 && (a->u_dtype == M2_BF16 || (a->u_dtype == M2_F16 && a->yu_bf16));
  if (a->n_filters == 2) {
    const size_t ua = ubf ? 8 : 16;
    M2_REQUIRE(m2_aligned(a->u, ua) && a->u_sc % 4 == 0 && a->u_sb % 4 == 0, M2_ERR_ALIGN,
               "m2_longconv_fwd: kind 2 needs rows of u aligned to four elements");
  }
  if (a->seq_len <= 2048) return ubf ? launch_conv<Geo4k, __nv_bfloat16>(P, st) : launch_conv<Geo4k, float>(P, st);
  if (a->seq_len <= 8192) return ubf ? launch_conv<Geo16k, __nv_bfloat16>(P, st) : launch_conv<Geo16k, float>(P, st);
  return ubf ? launch_conv<Geo64k, __nv_bfloat16>(P, st) : launch_conv<Geo64k, float>(P, st);
}

}  // namespace m2
