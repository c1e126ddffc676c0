// Fused gated long convolution on tcgen05 tensor cores for long rows (kernel family 2):
// bf16 activations stored time-contiguous ((B, channels, L) layout), transform length
// N = 32 * N2 * N3 = 4096 (128 < L <= 2048), 16384 (L <= 8192) or 65536 (L <= 32768).
//
// One (batch row, channel) sequence is processed at a time by a "slot" of 128 * TS threads; a CTA holds several
// slots that run independently (own barriers, own TMEM columns, own shared-memory region) so that one slot's loads
// and stage hand-offs overlap the others' work.
//
// The real FFT of length N is evaluated at the odd frequencies k + 1/2 (negacyclic form, no DC/Nyquist specials,
// Hermitian half = k1 < 16) and factored Monarch style with n = R n1 + N3 n2 + n3 (R = N2 N3),
// k = k1 + 32 k2 + 32 N2 k3:
//
//   F1  B1[r, k1]       = sum_{n1 < 16} W32^{n1 (k1 + 1/2)} a[R n1 + r],   r = (n2, n3)
//   x   w^{r (k1 + 1/2)}                      (as the product of an n2 part and an n3 part)
//   F2  B2[k1, n3, k2]  = sum_{n2} W_N2^{n2 k2} B1
//   x   w^{32 n3 k2}
//   F3  Z[k1, k2, k3]   = sum_{n3} W_N3^{n3 k3} B2
//   x   (G + bias), then the three inverse stages in mirror order on conjugated data (IDFT(x) = conj DFT(conj x),
//   so every radix needs one matrix only); the last stage yields only the L kept outputs y[R n1 + r], n1 < 16.
//
// Every stage is a batched real GEMM with M = 128 rows per tile, fp16 operands in un-swizzled core-matrix shared
// memory, constant DFT matrices as B operands and float32 accumulators in tensor memory.  Complex data is PLANAR:
// a TMEM row holds [Re of all columns | Im of all columns], so the thread that owns the row has both parts of
// every element, applies the twiddle with packed half2 arithmetic and writes its row as 16-byte chunks of 8
// consecutive columns.  What makes this possible is the operand view: a stage that contracts over the index held
// in the PREVIOUS stage's rows reads those chunks as an "MN-major" A operand (the 8 columns of a chunk become 8
// consecutive M rows, the row index becomes K), so the row <-> column exchange of the four-step FFT happens inside
// the MMA's operand fetch -- never as scattered stores.  Only the spectrum stage (Z -> inverse F3), which
// contracts over its own columns, uses the ordinary K-major view.  All chunk stores are bank-conflict free
// (row groups are padded by 16 bytes where consecutive lanes write to consecutive groups).
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

// N2, N3: radices of the second and third stage (the first is 32); SLOTS: independent sequences in flight per
// CTA; TS: groups of 128 threads inside a slot (they split the row tiles of every stage among themselves).
template <int N2_, int N3_, int SLOTS_, int TS_>
struct Geo {
  static constexpr int N2 = N2_, N3 = N3_, SLOTS = SLOTS_, TS = TS_;
  static constexpr int R = N2 * N3;             // rows of stage 1 = N / 32
  static constexpr int N = 32 * R;
  static constexpr int LG = (N == 4096) ? 12 : (N == 16384) ? 14 : 16;
  static constexpr int K2 = 2 * N2, K3 = 2 * N3;
  static constexpr int T1T = R / 128;           // row tiles of the first / last stage (rows r)
  static constexpr int T2T = N3 / 8;            // row tiles of the DFT_N2 stages (rows (k1, n3), 16 N3 of them)
  static constexpr int T3T = N2 / 8;            // row tiles of the DFT_N3 stages (rows (k1, k2), 16 N2 of them)
  static constexpr int TPS = 128 * TS;          // threads per slot
  static constexpr int THREADS = SLOTS * TPS;
  // operand regions (byte strides): a row GROUP is 8 rows of the MMA's M; its K extent is contiguous in 128-byte
  // core matrices (LBO = 128); groups follow each other at the SBO below (+16 where lanes hit consecutive groups)
  static constexpr int SBO1 = 256;                          // F1 operand: K = 16 (n1)
  static constexpr int SBO2 = K2 * 16 + 16;                 // DFT_N2 forward operand: K = (ri, n2)
  static constexpr int SBO3 = K3 * 16 + 16;                 // DFT_N3 forward operand: K = (ri, n3)
  static constexpr int SBO3K = K3 * 16, TILE3 = 16 * SBO3K; // DFT_N3 inverse operand (K-major rows): K = (ri, k3)
  static constexpr int SBO4 = K2 * 16;                      // DFT_N2 inverse operand: K = (ri, k2)
  static constexpr int SBO5 = 32 * 16 + 16;                 // last stage operand: K = (ri, k1)
  static constexpr int YF = 16 * R + 4 * (16 * R / 32);     // floats of the padded output buffer (4 after every 32)
  static constexpr int DATA_BYTES =
      ((cmax(cmax(cmax(R * 32, 2 * N3 * SBO2), cmax(2 * N2 * SBO3, T3T * TILE3)),
             cmax(cmax(2 * N3 * SBO4, (R / 8) * SBO5), 4 * YF)) + 127) / 128) * 128;
  // Variant with asynchronous staging of the global rows (see the kernel): per slot
  //   [0, A_RA)        the operand regions' first part / the bf16 output buffer (16-byte pad after every 128 bytes)
  //   [A_RA, +32 R)    one raw row (x1, then u): overlaps the operand regions, used only between passes
  //   [A_SB, +32 R)    one raw row beyond every operand region (v; x2 and the gated result during the passes)
  static constexpr int DEXT =
      ((cmax(cmax(cmax(R * 32, 2 * N3 * SBO2), cmax(2 * N2 * SBO3, T3T * TILE3)),
             cmax(2 * N3 * SBO4, (R / 8) * SBO5)) + 127) / 128) * 128;
  static constexpr int A_RA = 36 * R;
  static constexpr int A_SB = cmax(DEXT, A_RA + 32 * R);
  static constexpr int A_SLOT = A_SB + 32 * R;
  static constexpr int COLS = cmax(T1T * 32, cmax(T2T * K2, T3T * K3));
  static constexpr int TCOLS = (SLOTS * COLS <= 32) ? 32 : (SLOTS * COLS <= 64) ? 64 : (SLOTS * COLS <= 128) ? 128
                               : (SLOTS * COLS <= 256) ? 256 : 512;
  static constexpr float S2 = stage_scale(N2), S3 = stage_scale(N3);
  static constexpr float KAPPA = (2.0f / N) / ((S1 * S2 * S3) * (S1 * S2 * S3));
  // header of the spectrum table (bytes): constant matrices (core-matrix layout, K-major B operands) and
  // twiddle tables (fp16, planar: 16-byte runs of Re then of Im)
  static constexpr int F1_OFF = 0;                       // [32 (ri, k1)] x [16 n1]
  static constexpr int I1_OFF = F1_OFF + 1024;           // [16 n1] x [32 (ri, k1)]
  static constexpr int F2_OFF = I1_OFF + 1024;           // [K2 (ri', k2)] x [K2 (ri, n2)]
  static constexpr int F3_OFF = F2_OFF + K2 * K2 * 2;    // [K3] x [K3]
  static constexpr int TA1_OFF = F3_OFF + K3 * K3 * 2;   // [n2][Re k1 x16 | Im k1 x16]: w^{N3 n2 (k1 + 1/2)}
  static constexpr int TB1_PITCH = 64 + 16;              // rows read by 8 lanes at once are padded by 16 bytes: no two
  static constexpr int T2B_PITCH = K3 * 2 + 16;          // of the 8 rows start in the same 16-byte bank group
  static constexpr int TB1_OFF = TA1_OFF + N2 * 64;      // [n3][Re k1 x16 | Im k1 x16 | pad]: w^{n3 (k1 + 1/2)}
  static constexpr int TA5_OFF = TB1_OFF + N3 * TB1_PITCH;   // [k1][Re n2 x N2 | Im n2 x N2]
  static constexpr int TB5_OFF = TA5_OFF + 16 * K2 * 2;  // [k1][n3] half2 (Re, Im)
  static constexpr int T2A_OFF = TB5_OFF + 16 * N3 * 4;  // [n3][Re k2 x N2 | Im k2 x N2]: w^{32 n3 k2}
  static constexpr int T2B_OFF = T2A_OFF + 4 * R;        // [k2][Re n3 x N3 | Im n3 x N3 | pad]
  static constexpr int HDR_BYTES = T2B_OFF + N2 * T2B_PITCH;
  static constexpr int HDR_FLOATS = HDR_BYTES / 4;
  static constexpr int SMEM = SLOTS * DATA_BYTES + HDR_BYTES + 3 * SLOTS * 8 + 64 + 128;
  static constexpr int SMEM_A = SLOTS * A_SLOT + HDR_BYTES + 3 * SLOTS * 8 + 64 + 128 + SLOTS * 64;   // + per-slot scalars
  static constexpr bool CAN_ASYNC = TS == 1 && SMEM_A <= 227 * 1024;
  // Where that does not fit (N = 65536: one sequence fills the SM) rows are staged inside the phase that uses them:
  //   [32 R, +32 R)    halves of the raw x1 and v rows, then the raw u row, while the F1 operand [0, 32 R) is built
  //   [36 R, +32 R)    x2 / the first pass's gated result, copied once the last stage's MMAs are done
  static constexpr int B_LR = 32 * R;
  static constexpr int B_SB = 36 * R;
  static constexpr int B_SLOT = cmax(DEXT, 68 * R);
  static constexpr int SMEM_B = SLOTS * B_SLOT + HDR_BYTES + 3 * SLOTS * 8 + 64 + 128 + SLOTS * 64;
  static constexpr bool CAN_STAGE_IN_PHASE = !CAN_ASYNC && SMEM_B <= 227 * 1024 && (2 * R / TPS) % 2 == 0;
  static_assert(R % 128 == 0 && N3 % 8 == 0 && N2 % 8 == 0, "row tiles must be full");
  static_assert(SLOTS * COLS <= 512, "accumulators exceed tensor memory");
  static_assert(T1T % TS == 0 && T2T % TS == 0 && T3T % TS == 0, "tile split must divide every stage");
  static_assert((2 * R) % TPS == 0 && (4 * R) % TPS == 0, "load / store mapping");
  static_assert(HDR_BYTES % 16 == 0, "header is copied in 16-byte pieces");
  static_assert(SMEM <= 227 * 1024, "shared memory");
};

// byte offset of element (row, k) of a constant matrix with K columns (K-major B operand, un-padded)
template <int K>
__host__ __device__ constexpr int mat_off(int row, int k) {
  return (row >> 3) * (K * 16) + (k >> 3) * 128 + (row & 7) * 16 + (k & 7) * 2;
}

// ---------------------------------------------------------------------------------------
// Spectrum table (kind 2): [HDR_FLOATS floats: matrices + twiddles], then per channel N fp16 values -- for
// row tile t3 = k2 / 8: 16-byte chunks [j][m], j = 0 .. K3 / 8 - 1, row m = 8 k1 + (k2 % 8) of the tile; chunk j
// of a row holds Re G[k3] for k3 = 8 j .. 8 j + 7 (j < N3 / 8), then Im G[k3] the same way; bins
// k = k1 + 32 k2 + 32 N2 k3, multiplied by KAPPA * 2^e -- then one float 2^-e per channel.  Chunk-major tiles:
// the 32 lanes of a warp (32 consecutive rows) read one chunk each from 512 contiguous bytes.
// ---------------------------------------------------------------------------------------
template <typename G>
__device__ void write_header(float* spec, int tid, int nt) {
  constexpr int N = G::N, N2 = G::N2, N3 = G::N3, K2 = G::K2, K3 = G::K3;
  unsigned char* base = reinterpret_cast<unsigned char*>(spec);
  __half* m = reinterpret_cast<__half*>(spec);
  for (int idx = tid; idx < 16 * 16; idx += nt) {
    // F1 rows (ri, k1): W32^{n1 (k1+1/2)} = cos - i sin.  I1 acts on the CONJUGATE of the last inverse stage's
    // input: y = sum cos * Qr + sin * Qi.
    const int k1 = idx / 16, n1 = idx % 16;
    double sn, cs;
    sincospi(2.0 * n1 * (k1 + 0.5) / 32.0, &sn, &cs);
    m[(G::F1_OFF + mat_off<16>(k1, n1)) / 2] = __double2half(S1 * cs);
    m[(G::F1_OFF + mat_off<16>(16 + k1, n1)) / 2] = __double2half(-S1 * sn);
    m[(G::I1_OFF + mat_off<32>(n1, k1)) / 2] = __double2half(S1 * cs);
    m[(G::I1_OFF + mat_off<32>(n1, 16 + k1)) / 2] = __double2half(S1 * sn);
  }
  for (int idx = tid; idx < N2 * N2; idx += nt) {            // forward DFT_N2, planar real form
    const int ko = idx / N2, ni = idx % N2;
    double sn, cs;
    sincospi(2.0 * ((ko * ni) % N2) / N2, &sn, &cs);
    const double c = G::S2 * cs, s = G::S2 * sn;             // w = c - i s
    __half* f = m + G::F2_OFF / 2;
    f[mat_off<K2>(ko, ni) / 2] = __double2half(c);
    f[mat_off<K2>(ko, N2 + ni) / 2] = __double2half(s);
    f[mat_off<K2>(N2 + ko, ni) / 2] = __double2half(-s);
    f[mat_off<K2>(N2 + ko, N2 + ni) / 2] = __double2half(c);
  }
  for (int idx = tid; idx < N3 * N3; idx += nt) {            // forward DFT_N3
    const int ko = idx / N3, ni = idx % N3;
    double sn, cs;
    sincospi(2.0 * ((ko * ni) % N3) / N3, &sn, &cs);
    const double c = G::S3 * cs, s = G::S3 * sn;
    __half* f = m + G::F3_OFF / 2;
    f[mat_off<K3>(ko, ni) / 2] = __double2half(c);
    f[mat_off<K3>(ko, N3 + ni) / 2] = __double2half(s);
    f[mat_off<K3>(N3 + ko, ni) / 2] = __double2half(-s);
    f[mat_off<K3>(N3 + ko, N3 + ni) / 2] = __double2half(c);
  }
  __half* ta1 = reinterpret_cast<__half*>(base + G::TA1_OFF);
  __half* ta5 = reinterpret_cast<__half*>(base + G::TA5_OFF);
  for (int idx = tid; idx < 16 * N2; idx += nt) {            // w^{N3 n2 (k1 + 1/2)} in both index orders
    const int k1 = idx / N2, n2 = idx % N2;
    double sn, cs;
    sincospi(2.0 * N3 * n2 * (k1 + 0.5) / N, &sn, &cs);
    ta1[n2 * 32 + k1] = __double2half(cs);  ta1[n2 * 32 + 16 + k1] = __double2half(-sn);
    ta5[k1 * K2 + n2] = __double2half(cs);  ta5[k1 * K2 + N2 + n2] = __double2half(-sn);
  }
  __half* tb1 = reinterpret_cast<__half*>(base + G::TB1_OFF);
  __half2* tb5 = reinterpret_cast<__half2*>(base + G::TB5_OFF);
  for (int idx = tid; idx < 16 * N3; idx += nt) {            // w^{n3 (k1 + 1/2)}
    const int k1 = idx / N3, n3 = idx % N3;
    double sn, cs;
    sincospi(2.0 * n3 * (k1 + 0.5) / N, &sn, &cs);
    tb1[n3 * (G::TB1_PITCH / 2) + k1] = __double2half(cs);  tb1[n3 * (G::TB1_PITCH / 2) + 16 + k1] = __double2half(-sn);
    tb5[k1 * N3 + n3] = __floats2half2_rn((float)cs, (float)(-sn));
  }
  __half* t2a = reinterpret_cast<__half*>(base + G::T2A_OFF);
  __half* t2b = reinterpret_cast<__half*>(base + G::T2B_OFF);
  for (int idx = tid; idx < N2 * N3; idx += nt) {            // w^{32 n3 k2} in both index orders
    const int k2 = idx / N3, n3 = idx % N3;
    double sn, cs;
    sincospi(2.0 * 32.0 * n3 * k2 / N, &sn, &cs);
    t2a[n3 * K2 + k2] = __double2half(cs);  t2a[n3 * K2 + N2 + k2] = __double2half(-sn);
    t2b[k2 * (G::T2B_PITCH / 2) + n3] = __double2half(cs);  t2b[k2 * (G::T2B_PITCH / 2) + N3 + n3] = __double2half(-sn);
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
// position idx of a channel's table (complex entry (t3, m, k3)) -> bin k
template <typename G>
__device__ __forceinline__ int table_bin(int idx) {
  const int k3 = idx % G::N3, m = (idx / G::N3) % 128, t3 = idx / (G::N3 * 128);
  return (m >> 3) + 32 * (8 * t3 + (m & 7)) + 32 * G::N2 * k3;
}
// where its real part goes, in fp16 units from the channel's start (the imaginary part follows TABLE_IM entries on)
template <typename G>
__device__ __forceinline__ int table_pos(int idx) {
  const int k3 = idx % G::N3, m = (idx / G::N3) % 128, t3 = idx / (G::N3 * 128);
  return t3 * (128 * G::K3) + (k3 >> 3) * (128 * 8) + m * 8 + (k3 & 7);
}
template <typename G>
constexpr int TABLE_IM = (G::N3 / 8) * 128 * 8;

// One CTA per channel: N-point complex FFT (decimation in frequency) in shared memory of
// g[n] w^{n/2}, g = the filter with its wrapped half negated; bins gathered in table order.
template <typename G>
__global__ void __launch_bounds__(512)
spectrum_kind2_kernel(const float* __restrict__ kfilt, float* __restrict__ spec, int D, int R) {
  constexpr int N = G::N;
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
    const int p = (int)(__brev((unsigned)table_bin<G>(idx)) >> (32 - G::LG));
    gmax = fmaxf(gmax, fmaxf(fabsf(s[p].x), fabsf(s[p].y)));
  }
  __shared__ float red[32];
  gmax = block_max(gmax, red);
  const float sc = gain_scale(gmax * G::KAPPA);
  if (tid == 0) spec[G::HDR_FLOATS + (size_t)D * (N / 2) + c] = 1.0f / sc;
  __half* Gt = reinterpret_cast<__half*>(spec + G::HDR_FLOATS) + (size_t)c * N;
  for (int idx = tid; idx < N / 2; idx += nt) {
    const int p = (int)(__brev((unsigned)table_bin<G>(idx)) >> (32 - G::LG));
    const int o = table_pos<G>(idx);
    Gt[o] = __float2half_rn(s[p].x * (G::KAPPA * sc));
    Gt[o + TABLE_IM<G>] = __float2half_rn(s[p].y * (G::KAPPA * sc));
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
  constexpr int N = G::N, M = N / 2, Mh = M / 2, LGM = G::LG - 1;
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
  __half* Gt = reinterpret_cast<__half*>(spec + G::HDR_FLOATS) + (size_t)c * N;
  __shared__ float red[32];
  __shared__ float cta_max;
  // two passes over this CTA's bins: the first finds the channel's largest component (combined with the
  // other CTA's through distributed shared memory), the second stores the scaled bins
  float sc = 1.f;
  for (int pass = 0; pass < 2; ++pass) {
    float gmax = 0.f;
    for (int idx = tid; idx < N / 2; idx += nt) {
      const int k = table_bin<G>(idx);
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
      if (pass == 0) {
        gmax = fmaxf(gmax, fmaxf(fabsf(gr), fabsf(gi)));
      } else {
        const int o = table_pos<G>(idx);
        Gt[o] = __float2half_rn(gr * (G::KAPPA * sc));
        Gt[o + TABLE_IM<G>] = __float2half_rn(gi * (G::KAPPA * sc));
      }
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
  int al16;                                         // rows of xin / u / out start on 16-byte boundaries
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
__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}
// packed half2 arithmetic on 32-bit registers
__device__ __forceinline__ uint32_t h2_mul(uint32_t a, uint32_t b) {
  uint32_t d; asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
__device__ __forceinline__ uint32_t h2_neg(uint32_t a) {
  uint32_t d; asm("neg.f16x2 %0, %1;" : "=r"(d) : "r"(a)); return d;
}
__device__ __forceinline__ uint32_t h2_add(uint32_t a, uint32_t b) {
  uint32_t d; asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
}
// (re + i im) * (tr + i ti) for two packed complex numbers
__device__ __forceinline__ void cmul_h2(uint32_t re, uint32_t im, uint32_t tr, uint32_t ti, uint32_t& ore, uint32_t& oim) {
  ore = h2_fma(h2_neg(im), ti, h2_mul(re, tr));
  oim = h2_fma(re, ti, h2_mul(im, tr));
}
// One re-layout step ("hop") of a thread: for each of its NT row tiles (tile index t = ts + TS i, accumulator at
// column tile_cols * t of the thread's TMEM lane) and each group g of 8 complex columns of that row -- planar: Re in
// columns [8g, 8g+8), Im in columns [NC + 8g, ...) -- calls body(t, g, re, im) with the values as half2 pairs.
// Columns are fetched 16 complex at a time (8 when NC = 8) and the fetch of the next batch is issued before the
// current one is processed, so the TMEM latency is exposed once per hop instead of once per batch.
template <int NC, int NT, int TS, typename F>
__device__ __forceinline__ void hop_rows(uint32_t tml, int tile_cols, int ts, F&& body) {
  constexpr int W = NC >= 16 ? 16 : 8;                  // complex columns per batch
  constexpr int BPT = NC / W;                           // batches per tile
  constexpr int NB = NT * BPT;
  uint32_t a[2][W], b[2][W];
  auto issue = [&](int buf, int i) {
    const uint32_t tl = tml + tile_cols * (ts + TS * (i / BPT)) + W * (i % BPT);
    if constexpr (W == 16) { tc::tmem_ld16(tl, a[buf]); tc::tmem_ld16(tl + NC, b[buf]); }
    else { tmem_ld8(tl, a[buf]); tmem_ld8(tl + NC, b[buf]); }
  };
  issue(0, 0);
#pragma unroll
  for (int i = 0; i < NB; ++i) {
    tc::tmem_ld_wait();
    if (i + 1 < NB) issue((i + 1) & 1, i + 1);
    const int t = ts + TS * (i / BPT);
#pragma unroll
    for (int h = 0; h < W / 8; ++h) {
      uint32_t re[4], im[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        re[k] = pack_h2(__uint_as_float(a[i & 1][8 * h + 2 * k]), __uint_as_float(a[i & 1][8 * h + 2 * k + 1]));
        im[k] = pack_h2(__uint_as_float(b[i & 1][8 * h + 2 * k]), __uint_as_float(b[i & 1][8 * h + 2 * k + 1]));
      }
      body(t, (W / 8) * (i % BPT) + h, re, im);
    }
  }
}
// 16-byte asynchronous copy global -> shared (L2 only), and the group bookkeeping of the issuing thread
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
  unsigned short v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts16(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"((unsigned short)v) : "memory");
}

// depthwise 3-tap conv taps of one channel, rounded to bf16 as autocast rounds the conv's parameters
struct Taps { float w0, w1, w2, b; };
__device__ __forceinline__ Taps load_taps(const float* sw, const float* sb, int ch) {
  Taps T;
  T.w0 = bf16r(__ldg(sw + 3 * ch)); T.w1 = bf16r(__ldg(sw + 3 * ch + 1)); T.w2 = bf16r(__ldg(sw + 3 * ch + 2));
  T.b = bf16r(__ldg(sb + ch));
  return T;
}
// raw words of x[t0-2 .. t0+NV-1] of a time-contiguous bf16 row (w[0] = the two steps before t0; t0 % 8 == 0 for
// NV = 8, % 4 for NV = 4); positions outside [0, L) read as 0.  L % 4 == 0, rows 8-byte aligned (16-byte when al16).
// Split from the unpacking so that a caller can issue the loads of several chunks before using any of them.
template <int NV>
__device__ __forceinline__ void load_raw(const __nv_bfloat16* row, int t0, int L, bool al16, uint32_t (&w)[NV / 2 + 1]) {
#pragma unroll
  for (int i = 0; i <= NV / 2; ++i) w[i] = 0u;
  if (t0 < L) {
    if (t0 >= 2) w[0] = __ldg(reinterpret_cast<const uint32_t*>(row + t0 - 2));
    if (NV == 8 && al16 && t0 + 8 <= L) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(row + t0));
      w[1] = v.x; w[2] = v.y; w[NV / 2 - 1] = v.z; w[NV / 2] = v.w;
    } else {
#pragma unroll
      for (int q = 0; q < NV / 4; ++q)
        if (t0 + 4 * q < L) {
          const uint2 v = __ldg(reinterpret_cast<const uint2*>(row + t0 + 4 * q));
          w[1 + 2 * q] = v.x; w[2 + 2 * q] = v.y;
        }
    }
  }
}
template <int NV>
__device__ __forceinline__ void unpack_raw(const uint32_t (&w)[NV / 2 + 1], float (&x)[NV + 2]) {
#pragma unroll
  for (int i = 0; i <= NV / 2; ++i) { x[2 * i] = bf_lo(w[i]); x[2 * i + 1] = bf_hi(w[i]); }
}
// The depthwise 3-tap conv on NV consecutive steps from the raw words of load_raw, two outputs per packed float32
// FMA: out[p] = bf16x2 of (y[2p], y[2p+1]), y[t] = b + w0 x[t-2] + w1 x[t-1] + w2 x[t] accumulated in float32 and
// rounded to bf16 once, as the reference's conv1d under autocast.
struct Taps2 { f32x2 w0, w1, w2, b; };
__device__ __forceinline__ Taps2 load_taps2(const float* sw, const float* sb, int ch) {
  const Taps T = load_taps(sw, sb, ch);
  Taps2 P;
  P.w0 = f2_splat(T.w0); P.w1 = f2_splat(T.w1); P.w2 = f2_splat(T.w2); P.b = f2_splat(T.b);
  return P;
}
template <int NV>
__device__ __forceinline__ void conv_packed(const Taps2& T, const uint32_t (&w)[NV / 2 + 1], uint32_t (&out)[NV / 2]) {
  float f[NV + 2];
  unpack_raw<NV>(w, f);
#pragma unroll
  for (int p = 0; p < NV / 2; ++p) {
    f32x2 acc = f2_fma(f2_pack(f[2 * p], f[2 * p + 1]), T.w0, T.b);
    acc = f2_fma(f2_pack(f[2 * p + 1], f[2 * p + 2]), T.w1, acc);
    acc = f2_fma(f2_pack(f[2 * p + 2], f[2 * p + 3]), T.w2, acc);
    float lo, hi;
    f2_unpack(acc, lo, hi);
    out[p] = pack_bf2(lo, hi);
  }
}
// bf16x2 -> fp16x2 (exact for values inside fp16's range)
__device__ __forceinline__ uint32_t bf2_to_h2(uint32_t v) { return pack_h2(bf_lo(v), bf_hi(v)); }

// MMAs of one stage: 0 F1, 1 DFT_N2, 2 DFT_N3, 3 DFT_N3 on conjugated data (= inverse), 4 DFT_N2 (inverse), 5 I1.
// A operands: MN-major (row groups `sbo` apart, K core matrices 128 bytes apart) except stage 3 (K-major rows).
// The issuing thread is on every stage's critical path, so descriptors are not rebuilt per MMA: an un-swizzled
// descriptor is {start address >> 4 | LBO field, SBO field | version}, the two high parts are compile-time
// constants per operand and moving to another tile or K step adds a constant to the 14-bit address field
// (shared-memory addresses stay below 2^18, so the field cannot overflow into its neighbour).
__device__ __forceinline__ uint64_t desc_at(uint32_t lo_base, uint32_t byte_off, uint32_t lbo, uint32_t sbo) {
  const uint32_t lo = lo_base + (byte_off >> 4) + ((lbo >> 4) << 16);
  const uint32_t hi = (sbo >> 4) | (1u << 14);          // bits 32..45 SBO, bit 46 descriptor version
  return ((uint64_t)hi << 32) | lo;
}
template <typename G>
__device__ __forceinline__ void issue_stage(int stage, uint32_t tm, uint32_t data, uint32_t hdr) {
  constexpr int K2 = G::K2, K3 = G::K3;
  const uint32_t dlo = data >> 4, hlo = hdr >> 4;        // both bases are 16-byte aligned and below 2^18
  if (stage == 0) {
    constexpr uint32_t id = tc::make_idesc_major(128, 32, 0, 1, 0);
    const uint64_t dB = desc_at(hlo, G::F1_OFF, 128, 16 * 16);
#pragma unroll
    for (int t = 0; t < G::T1T; ++t)
      tc::mma_ss(tm + 32 * t, desc_at(dlo, t * 16 * G::SBO1, 128, G::SBO1), dB, id, 0);
  } else if (stage == 1) {
    constexpr uint32_t id = tc::make_idesc_major(128, K2, 0, 1, 0);
#pragma unroll
    for (int t = 0; t < G::T2T; ++t)
#pragma unroll
      for (int s = 0; s < K2 / 16; ++s)
        tc::mma_ss(tm + K2 * t, desc_at(dlo, t * 16 * G::SBO2 + s * 256, 128, G::SBO2),
                   desc_at(hlo, G::F2_OFF + s * 256, 128, K2 * 16), id, s ? 1u : 0u);
  } else if (stage == 4) {
    constexpr uint32_t id = tc::make_idesc_major(128, K2, 0, 1, 0);
#pragma unroll
    for (int t = 0; t < G::T2T; ++t)
#pragma unroll
      for (int s = 0; s < K2 / 16; ++s)
        tc::mma_ss(tm + K2 * t, desc_at(dlo, t * 16 * G::SBO4 + s * 256, 128, G::SBO4),
                   desc_at(hlo, G::F2_OFF + s * 256, 128, K2 * 16), id, s ? 1u : 0u);
  } else if (stage == 2) {
    constexpr uint32_t id = tc::make_idesc_major(128, K3, 0, 1, 0);
#pragma unroll
    for (int t = 0; t < G::T3T; ++t)
#pragma unroll
      for (int s = 0; s < K3 / 16; ++s)
        tc::mma_ss(tm + K3 * t, desc_at(dlo, t * 16 * G::SBO3 + s * 256, 128, G::SBO3),
                   desc_at(hlo, G::F3_OFF + s * 256, 128, K3 * 16), id, s ? 1u : 0u);
  } else if (stage == 3) {
    constexpr uint32_t id = tc::make_idesc(128, K3, 0);
#pragma unroll
    for (int t = 0; t < G::T3T; ++t)
#pragma unroll
      for (int s = 0; s < K3 / 16; ++s)
        tc::mma_ss(tm + K3 * t, desc_at(dlo, t * G::TILE3 + s * 256, 128, G::SBO3K),
                   desc_at(hlo, G::F3_OFF + s * 256, 128, K3 * 16), id, s ? 1u : 0u);
  } else {
    constexpr uint32_t id = tc::make_idesc_major(128, 16, 0, 1, 0);
#pragma unroll
    for (int t = 0; t < G::T1T; ++t)
#pragma unroll
      for (int s = 0; s < 2; ++s)
        tc::mma_ss(tm + 16 * t, desc_at(dlo, t * 16 * G::SBO5 + s * 256, 128, G::SBO5),
                   desc_at(hlo, G::I1_OFF + s * 256, 128, 32 * 16), id, s ? 1u : 0u);
  }
}

// ASYNC (geometries with room for it; 2-byte u, 16-byte aligned rows, L % 8 == 0):
// no thread ever waits for a global load it has just issued.  Every row this slot reads is copied into the slot's
// shared memory with cp.async one phase ahead -- x2 while the first filter's transform runs, u during the first
// epilogue, the next sequence's x1 / v during and after the second epilogue -- the output buffer holds bf16, and the
// first filter's gated result stays in shared memory until the residual pass's last re-layout adds its conv to it;
// the output is written once.
template <typename G, typename TU, bool ASYNC>
__global__ void __launch_bounds__(G::THREADS, 1)
longconv_tcl_kernel(const Params P) {
  static_assert(!ASYNC || ((G::CAN_ASYNC || G::CAN_STAGE_IN_PHASE) && sizeof(TU) == 2), "asynchronous staging: geometry / element size");
  // XP: rows cross phases (copied one phase ahead); BIG: one sequence fills the SM, rows are copied inside the phase
  // that uses them -- still as 512-byte runs with every piece of a phase in flight at once, instead of 64-byte runs
  // fetched a few registers at a time -- and the first pass's gated result takes the way through global memory
  constexpr bool XP = ASYNC && G::CAN_ASYNC, BIG = ASYNC && !G::CAN_ASYNC;
  constexpr int SLOT_BYTES = XP ? G::A_SLOT : BIG ? G::B_SLOT : G::DATA_BYTES;
  constexpr int N2 = G::N2, N3 = G::N3, R = G::R, K2 = G::K2, K3 = G::K3, TS = G::TS, TPS = G::TPS;
  constexpr int LIT = 2 * R / TPS;                 // 8-step chunks per thread in the load phase
  constexpr int LB = LIT < 4 ? LIT : 4;            // ... of which this many have their global loads in flight together
  constexpr int EIT = 4 * R / TPS;                 // 4-step chunks per thread in the epilogue
  constexpr int EB = EIT < 8 ? EIT : 8;
  static_assert(LIT % LB == 0 && EIT % EB == 0, "batching of the memory phases");
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
  unsigned char* hdrb = smem + G::SLOTS * SLOT_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(hdrb + G::HDR_BYTES);       // per slot: ops, mma, w
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * G::SLOTS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
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
  const uint32_t data = tc::smem_u32(smem + slot * SLOT_BYTES);
  float* Y = reinterpret_cast<float*>(smem + slot * SLOT_BYTES);
  const uint32_t RA = data + G::A_RA, SB = data + (BIG ? G::B_SB : G::A_SB);     // raw-row regions of the asynchronous variants
  const uint32_t LR = data + G::B_LR;
  const int lane = tid & 31;
  // ASYNC: the sequence's scalars, copied ahead like its rows: [4 g + k] short-conv taps w0 w1 w2 b of x1, x2, v
  // (g = 0, 1, 2); [12 + f] 2^-e of filter f's channel; [14 + f] its bias
  volatile float* prm = reinterpret_cast<volatile float*>(tmem_slot + 4) + 16 * slot;
  const uint32_t hdr = tc::smem_u32(hdrb);
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

  // position of chunk q of the load phase: a warp covers 8 n1 x 4 row groups -- 64 contiguous bytes per n1 from
  // global memory, and each quarter warp fills one 128-byte core matrix of the F1 operand
  auto chunk_of = [&](int q, int& n1, int& rg) {
    n1 = ((q >> 5) & 1) * 8 + (q & 7);
    rg = (q >> 6) * 4 + ((q >> 3) & 3);
  };
  const int stride = gridDim.x * G::SLOTS;
  constexpr int CPN = R / 8;                       // 16-byte chunks per n1 of a raw 2-byte row
  // ASYNC: copies of the steps below L of a raw row.  Swizzled: chunk c = (R / 8) n1 + rg lands at chunk
  // c ^ (n1 & 7), so that a quarter warp of the load phase (8 values of n1, one rg) reads 8 different bank groups.
  auto stage_swz = [&](uint32_t dst, const void* row) {
    const unsigned char* src = reinterpret_cast<const unsigned char*>(row);
    for (int c = sl; 8 * c < P.L; c += TPS) cp_async16(dst + 16 * (c ^ ((c / CPN) & 7)), src + 16 * c);
  };
  // ... in time order, chunk c at c ^ ((c >> 3) & 1): the epilogue's quarter warps (8 consecutive chunks) and the
  // last re-layout's 2-byte reads (lanes 32 bytes apart, 8 of them) both find 8 different bank groups
  auto stage_lin = [&](uint32_t dst, const void* row) {
    const unsigned char* src = reinterpret_cast<const unsigned char*>(row);
    for (int c = sl; 8 * c < P.L; c += TPS) cp_async16(dst + 16 * (c ^ ((c >> 3) & 1)), src + 16 * c);
  };
  auto stage_scalars = [&](int rid) {
    if (sl < 16) {
      const int c = rid / P.B, g = sl >> 2, k = sl & 3, f = sl & 1;
      const float* src = sl < 12 ? (k < 3 ? P.sw + 3 * (g * P.D + c) + k : P.sb + g * P.D + c)
                       : sl < 14 ? P.spec[f] + G::HDR_FLOATS + (size_t)P.D * (G::N / 2) + c : P.bias[f] + c;
      if (sl < 12 || f < P.nf) cp_async4(tc::smem_u32(const_cast<float*>(prm + sl)), src);
    }
  };
  auto taps_of = [&](int g) {
    Taps2 T;
    T.w0 = f2_splat(bf16r(prm[4 * g])); T.w1 = f2_splat(bf16r(prm[4 * g + 1])); T.w2 = f2_splat(bf16r(prm[4 * g + 2]));
    T.b = f2_splat(bf16r(prm[4 * g + 3]));
    return T;
  };
  auto x1_of = [&](int rid) { return P.xin + (long long)(rid % P.B) * P.xsb + (long long)(rid / P.B) * P.xsc; };
  if constexpr (ASYNC) {
    const int r0 = blockIdx.x * G::SLOTS + slot;
    if (r0 < P.rows) {
      stage_scalars(r0);
      if (XP) {
        stage_swz(RA, x1_of(r0));
        stage_swz(SB, x1_of(r0) + 2 * (long long)P.D * P.xsc);
      }
    }
    cp_async_commit();
  }
  // rows of one channel are neighbours in the walk (batch index fastest): the slots working at the same time share
  // a few channels' spectrum tables, which then come from L2
  for (int rowid = blockIdx.x * G::SLOTS + slot; rowid < P.rows && ok; rowid += stride) {
    const int ch = rowid / P.B, b = rowid % P.B;
    const __nv_bfloat16* x1row = P.xin + (long long)b * P.xsb + (long long)ch * P.xsc;
    const __nv_bfloat16* x2row = x1row + (long long)P.D * P.xsc;
    const __nv_bfloat16* vrow = x2row + (long long)P.D * P.xsc;
    __nv_bfloat16* orow = P.out + (long long)b * P.osb + (long long)ch * P.osc;
    const TU* urow = reinterpret_cast<const TU*>(P.u) + (long long)b * P.usb + (long long)ch * P.usc;
    if constexpr (ASYNC) {
      cp_async_wait<0>();                          // this sequence's scalars; XP: its x1 (RA) and v (SB) as well
      LCL_BARRIER()
    }

    for (int f = 0; f < P.nf && ok; ++f) {
      // 2^-e of this channel and the bias term of the spectrum product
      const float ig = ASYNC ? prm[12 + f] : __ldg(P.spec[f] + G::HDR_FLOATS + (size_t)P.D * (G::N / 2) + ch);
      const float bkf = (ASYNC ? prm[14 + f] : __ldg(P.bias[f] + ch)) * G::KAPPA / ig;
      // ---------------- F1 operand: a[R n1 + r] as fp16, one 16-byte chunk = 8 consecutive r of one n1 ----------------
      if (BIG && f == 0) {
        const Taps2 Tx = taps_of(0), Tv = taps_of(2);
        constexpr int HI = LIT / 2, HC = CPN / 2;          // iterations / chunks per n1 of one half
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          // this half's chunks of x1 (LR) and v (LR + 16 R): chunk (n1, rg) at index HC n1 + rg - HC half, low bits ^ n1
          for (int j = sl; j < 16 * HC; j += TPS) {
            const int n1 = j / HC, c = n1 * CPN + half * HC + j % HC;
            if (8 * c < P.L) {
              cp_async16(LR + 16 * (j ^ (n1 & 7)), x1row + 8 * c);
              cp_async16(LR + 16 * R + 16 * (j ^ (n1 & 7)), vrow + 8 * c);
            }
          }
          cp_async_commit();
          // the two steps before a chunk: by shuffle from the lane 8 below; the first quarter warp asks global memory
          uint32_t gx[HI], gw[HI];
#pragma unroll
          for (int i = 0; i < HI; ++i) {
            int n1, rg;
            chunk_of((half * HI + i) * TPS + sl, n1, rg);
            const int t0 = R * n1 + 8 * rg;
            gx[i] = gw[i] = 0u;
            if (lane < 8 && t0 >= 2 && t0 < P.L) {
              gx[i] = __ldg(reinterpret_cast<const uint32_t*>(x1row + t0 - 2));
              gw[i] = __ldg(reinterpret_cast<const uint32_t*>(vrow + t0 - 2));
            }
          }
          cp_async_wait<0>();
          LCL_BARRIER()
#pragma unroll
          for (int i = 0; i < HI; ++i) {
            int n1, rg;
            chunk_of((half * HI + i) * TPS + sl, n1, rg);
            const int t0 = R * n1 + 8 * rg;
            const bool in = t0 < P.L;
            uint4 x = make_uint4(0u, 0u, 0u, 0u), v = x;
            if (in) {
              const uint32_t o = 16 * ((n1 * HC + rg - half * HC) ^ (n1 & 7));
              x = lds128(LR + o); v = lds128(LR + 16 * R + o);
            }
            uint32_t hx = __shfl_up_sync(0xffffffffu, x.w, 8), hv = __shfl_up_sync(0xffffffffu, v.w, 8);
            if (lane < 8) { hx = gx[i]; hv = gw[i]; }
            const uint32_t wx[5] = {hx, x.x, x.y, x.z, x.w}, wv[5] = {hv, v.x, v.y, v.z, v.w};
            uint32_t cx[4], cv[4], h[4];
            conv_packed<8>(Tx, wx, cx);
            conv_packed<8>(Tv, wv, cv);
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = in ? bf2_to_h2(bf2_mul(cv[j], cx[j])) : 0u;
            sts128(data + rg * G::SBO1 + n1 * 16, h[0], h[1], h[2], h[3]);
          }
          if (half == 0) { LCL_BARRIER() }                 // every thread is done with this half before the next lands
        }
      } else if (BIG) {
        // the raw u row (LR, swizzled like the cross-phase variant's rows), all of it in flight at once
        stage_swz(LR, urow);
        cp_async_commit();
        cp_async_wait<0>();
        LCL_BARRIER()
#pragma unroll 2
        for (int it = 0; it < LIT; ++it) {
          int n1, rg;
          chunk_of(it * TPS + sl, n1, rg);
          const int t0 = R * n1 + 8 * rg, c = t0 >> 3;
          uint4 w = make_uint4(0u, 0u, 0u, 0u);
          if (t0 < P.L) w = lds128(LR + 16 * (c ^ (n1 & 7)));
          if (!P.u_f16) {
            w.x = bf2_to_h2(w.x); w.y = bf2_to_h2(w.y); w.z = bf2_to_h2(w.z); w.w = bf2_to_h2(w.w);
          }
          sts128(data + rg * G::SBO1 + n1 * 16, w.x, w.y, w.z, w.w);
        }
      } else if (ASYNC && f == 0) {
        const Taps2 Tx = taps_of(0), Tv = taps_of(2);
#pragma unroll 2
        for (int it = 0; it < LIT; ++it) {
          int n1, rg;
          chunk_of(it * TPS + sl, n1, rg);
          const int t0 = R * n1 + 8 * rg, c = t0 >> 3;
          const bool in = t0 < P.L;
          uint4 x = make_uint4(0u, 0u, 0u, 0u), v = x;
          if (in) {
            const uint32_t o = 16 * (c ^ (n1 & 7));
            x = lds128(RA + o); v = lds128(SB + o);
          }
          // the two steps before the chunk: the lane 8 below holds chunk (n1, rg - 1); the first quarter warp reads them
          uint32_t hx = __shfl_up_sync(0xffffffffu, x.w, 8), hv = __shfl_up_sync(0xffffffffu, v.w, 8);
          if (lane < 8) {
            hx = hv = 0u;
            if (in && c > 0) {
              const int pc = c - 1;
              const uint32_t o = 16 * (pc ^ ((pc / CPN) & 7)) + 12;
              hx = lds32(RA + o); hv = lds32(SB + o);
            }
          }
          const uint32_t wx[5] = {hx, x.x, x.y, x.z, x.w}, wv[5] = {hv, v.x, v.y, v.z, v.w};
          uint32_t cx[4], cv[4], h[4];
          conv_packed<8>(Tx, wx, cx);
          conv_packed<8>(Tv, wv, cv);
#pragma unroll
          for (int j = 0; j < 4; ++j) h[j] = in ? bf2_to_h2(bf2_mul(cv[j], cx[j])) : 0u;   // steps from L on are zero padding
          sts128(data + rg * G::SBO1 + n1 * 16, h[0], h[1], h[2], h[3]);
        }
      } else if (ASYNC) {
#pragma unroll 2
        for (int it = 0; it < LIT; ++it) {
          int n1, rg;
          chunk_of(it * TPS + sl, n1, rg);
          const int t0 = R * n1 + 8 * rg, c = t0 >> 3;
          uint4 w = make_uint4(0u, 0u, 0u, 0u);
          if (t0 < P.L) w = lds128(RA + 16 * (c ^ (n1 & 7)));
          if (!P.u_f16) {
            w.x = bf2_to_h2(w.x); w.y = bf2_to_h2(w.y); w.z = bf2_to_h2(w.z); w.w = bf2_to_h2(w.w);
          }
          sts128(data + rg * G::SBO1 + n1 * 16, w.x, w.y, w.z, w.w);
        }
      } else if (f == 0) {
        const Taps2 Tx = load_taps2(P.sw, P.sb, ch), Tv = load_taps2(P.sw, P.sb, 2 * P.D + ch);
#pragma unroll 1
        for (int it0 = 0; it0 < LIT; it0 += LB) {
          uint32_t xr[LB][5], vr[LB][5];
#pragma unroll
          for (int i = 0; i < LB; ++i) {
            int n1, rg;
            chunk_of((it0 + i) * TPS + sl, n1, rg);
            load_raw<8>(x1row, R * n1 + 8 * rg, P.L, P.al16, xr[i]);
            load_raw<8>(vrow, R * n1 + 8 * rg, P.L, P.al16, vr[i]);
          }
#pragma unroll
          for (int i = 0; i < LB; ++i) {
            int n1, rg;
            chunk_of((it0 + i) * TPS + sl, n1, rg);
            const int t0 = R * n1 + 8 * rg;
            uint32_t cx[4], cv[4], h[4];
            conv_packed<8>(Tx, xr[i], cx);
            conv_packed<8>(Tv, vr[i], cv);
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = bf2_to_h2(bf2_mul(cv[j], cx[j]));     // v * x1: the exact product, rounded to bf16
            if (t0 + 8 > P.L) {                                                     // steps at and beyond L are zero padding
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (t0 + 2 * j >= P.L) h[j] = 0u;
                else if (t0 + 2 * j + 1 >= P.L) h[j] &= 0xffffu;
              }
            }
            sts128(data + rg * G::SBO1 + n1 * 16, h[0], h[1], h[2], h[3]);
          }
        }
      } else {
#pragma unroll 1
        for (int it0 = 0; it0 < LIT; it0 += LB) {
          uint32_t w[LB][sizeof(TU) == 4 ? 8 : 4];
#pragma unroll
          for (int i = 0; i < LB; ++i) {
            int n1, rg;
            chunk_of((it0 + i) * TPS + sl, n1, rg);
            const int t0 = R * n1 + 8 * rg;
#pragma unroll
            for (int j = 0; j < (sizeof(TU) == 4 ? 8 : 4); ++j) w[i][j] = 0u;
            if (sizeof(TU) == 4) {
#pragma unroll
              for (int q4 = 0; q4 < 2; ++q4)
                if (t0 + 4 * q4 < P.L) {
                  const uint4 v = __ldg(reinterpret_cast<const uint4*>(urow + t0 + 4 * q4));
                  w[i][4 * q4] = v.x; w[i][4 * q4 + 1] = v.y; w[i][4 * q4 + 2] = v.z; w[i][4 * q4 + 3] = v.w;
                }
            } else if (P.al16 && t0 + 8 <= P.L) {
              const uint4 v = __ldg(reinterpret_cast<const uint4*>(urow + t0));
              w[i][0] = v.x; w[i][1] = v.y; w[i][2] = v.z; w[i][3] = v.w;
            } else {
#pragma unroll
              for (int q4 = 0; q4 < 2; ++q4)
                if (t0 + 4 * q4 < P.L) {
                  const uint2 v = __ldg(reinterpret_cast<const uint2*>(urow + t0 + 4 * q4));
                  w[i][2 * q4] = v.x; w[i][2 * q4 + 1] = v.y;
                }
            }
          }
#pragma unroll
          for (int i = 0; i < LB; ++i) {
            int n1, rg;
            chunk_of((it0 + i) * TPS + sl, n1, rg);
            uint32_t h[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (sizeof(TU) == 4) h[j] = pack_h2(__uint_as_float(w[i][2 * j]), __uint_as_float(w[i][2 * j + 1]));
              else h[j] = P.u_f16 ? w[i][j] : pack_h2(bf_lo(w[i][j]), bf_hi(w[i][j]));
            }
            sts128(data + rg * G::SBO1 + n1 * 16, h[0], h[1], h[2], h[3]);
          }
        }
      }
      LCL_STAGE(0)
      if constexpr (XP) {
        if (f == 0) {                              // every thread of the slot is done with the raw x1 / v rows
          stage_lin(SB, x2row);
          cp_async_commit();
        }
      }

      // ---------------- hop 1: x w^{r (k1 + 1/2)}; rows r = (n2, n3) -> operand rows (k1, n3), K = (ri, n2) ----------------
      hop_rows<16, G::T1T / TS, TS>(tml, 32, ts, [&](int t, int g, const uint32_t (&re)[4], const uint32_t (&im)[4]) {   // k1 = 8 g ..
        const int r = 128 * t + l, n2 = r / N3, n3 = r % N3;
        const uint32_t ta = hdr + G::TA1_OFF + n2 * 64, tb = hdr + G::TB1_OFF + n3 * G::TB1_PITCH;
        const uint4 ar = lds128(ta + 16 * g), ai = lds128(ta + 32 + 16 * g);
        const uint4 br = lds128(tb + 16 * g), bi = lds128(tb + 32 + 16 * g);
        const uint32_t arr[4] = {ar.x, ar.y, ar.z, ar.w}, aii[4] = {ai.x, ai.y, ai.z, ai.w};
        const uint32_t brr[4] = {br.x, br.y, br.z, br.w}, bii[4] = {bi.x, bi.y, bi.z, bi.w};
        uint32_t orr[4], oi[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t wr, wi;
          cmul_h2(arr[i], aii[i], brr[i], bii[i], wr, wi);
          cmul_h2(re[i], im[i], wr, wi, orr[i], oi[i]);
        }
        // row group j = k1hi N3 + n3, K index n2 (real plane) and N2 + n2 (imaginary plane)
        const uint32_t d = data + (g * N3 + n3) * G::SBO2 + (n2 >> 3) * 128 + (n2 & 7) * 16;
        sts128(d, orr[0], orr[1], orr[2], orr[3]);
        sts128(d + (N2 / 8) * 128, oi[0], oi[1], oi[2], oi[3]);
      });
      tc::tc_fence_before();
      LCL_STAGE(1)

      // ---------------- hop 2: x w^{32 n3 k2}; rows (k1, n3) -> operand rows (k1, k2), K = (ri, n3) ----------------
      hop_rows<N2, G::T2T / TS, TS>(tml, K2, ts, [&](int t, int g, const uint32_t (&re)[4], const uint32_t (&im)[4]) {   // k2 = 8 g ..
        const int j = 16 * t + (l >> 3), k1 = 8 * (j / N3) + (l & 7), n3 = j % N3;
        const uint32_t tw = hdr + G::T2A_OFF + n3 * (K2 * 2);
        const uint4 wr4 = lds128(tw + 16 * g), wi4 = lds128(tw + N2 * 2 + 16 * g);
        const uint32_t wr[4] = {wr4.x, wr4.y, wr4.z, wr4.w}, wi[4] = {wi4.x, wi4.y, wi4.z, wi4.w};
        uint32_t orr[4], oi[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) cmul_h2(re[i], im[i], wr[i], wi[i], orr[i], oi[i]);
        // row group j3 = k2hi 16 + k1, K index n3 / N3 + n3
        const uint32_t d = data + (g * 16 + k1) * G::SBO3 + (n3 >> 3) * 128 + (n3 & 7) * 16;
        sts128(d, orr[0], orr[1], orr[2], orr[3]);
        sts128(d + (N3 / 8) * 128, oi[0], oi[1], oi[2], oi[3]);
      });
      // this row's slice of the spectrum comes from global memory (L2 for all but the first sequence of a channel):
      // the first tile's slice is requested before the wait for stage 2's MMAs, every further tile's while the
      // one before it is being multiplied
      constexpr int NG = K3 / 8;
      const __half* Gc = reinterpret_cast<const __half*>(P.spec[f] + G::HDR_FLOATS) + (size_t)ch * G::N;
      uint4 gv[NG], gn[NG];
      {
        const uint4* gp = reinterpret_cast<const uint4*>(Gc) + (size_t)ts * NG * 128 + l;   // chunk i of row l of tile ts
#pragma unroll
        for (int i = 0; i < NG; ++i) gv[i] = __ldg(gp + i * 128);
      }
      tc::tc_fence_before();
      LCL_STAGE(2)

      // ---------------- hop 3: conj(Z (G + bias)); rows (k1, k2) keep their place (K-major), K = (ri, k3) ----------------
      {
        const uint32_t bk = pack_h2(bkf, bkf);
        hop_rows<N3, G::T3T / TS, TS>(tml, K3, ts, [&](int t, int g, const uint32_t (&re)[4], const uint32_t (&im)[4]) {   // k3 = 8 g ..
          if (g == 0 && t + TS < G::T3T) {
            const uint4* gp = reinterpret_cast<const uint4*>(Gc) + (size_t)(t + TS) * NG * 128 + l;
#pragma unroll
            for (int i = 0; i < NG; ++i) gn[i] = __ldg(gp + i * 128);
          }
          const uint32_t gr[4] = {gv[g].x, gv[g].y, gv[g].z, gv[g].w};
          const uint32_t gi[4] = {gv[N3 / 8 + g].x, gv[N3 / 8 + g].y, gv[N3 / 8 + g].z, gv[N3 / 8 + g].w};
          uint32_t orr[4], oi[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            cmul_h2(re[i], im[i], h2_add(gr[i], bk), gi[i], orr[i], oi[i]);
            oi[i] = h2_neg(oi[i]);
          }
          const uint32_t dst = data + t * G::TILE3 + (l >> 3) * G::SBO3K + (l & 7) * 16;
          sts128(dst + g * 128, orr[0], orr[1], orr[2], orr[3]);
          sts128(dst + (N3 / 8 + g) * 128, oi[0], oi[1], oi[2], oi[3]);
          if (g == N3 / 8 - 1) {
#pragma unroll
            for (int i = 0; i < NG; ++i) gv[i] = gn[i];
          }
        });
      }
      tc::tc_fence_before();
      LCL_STAGE(3)

      // ---------------- hop 4: x w^{32 n3 k2}; rows (k1, k2) -> operand rows (k1, n3), K = (ri, k2) ----------------
      hop_rows<N3, G::T3T / TS, TS>(tml, K3, ts, [&](int t, int g, const uint32_t (&re)[4], const uint32_t (&im)[4]) {   // n3 = 8 g ..
        const int k1 = l >> 3, k2 = 8 * t + (l & 7);
        const uint32_t tw = hdr + G::T2B_OFF + k2 * G::T2B_PITCH;
        const uint4 wr4 = lds128(tw + 16 * g), wi4 = lds128(tw + N3 * 2 + 16 * g);
        const uint32_t wr[4] = {wr4.x, wr4.y, wr4.z, wr4.w}, wi[4] = {wi4.x, wi4.y, wi4.z, wi4.w};
        uint32_t orr[4], oi[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) cmul_h2(re[i], im[i], wr[i], wi[i], orr[i], oi[i]);
        // row group j4 = n3hi 16 + k1, K index k2 / N2 + k2
        const uint32_t d = data + (g * 16 + k1) * G::SBO4 + (k2 >> 3) * 128 + (k2 & 7) * 16;
        sts128(d, orr[0], orr[1], orr[2], orr[3]);
        sts128(d + (N2 / 8) * 128, oi[0], oi[1], oi[2], oi[3]);
      });
      tc::tc_fence_before();
      LCL_STAGE(4)

      // ---------------- hop 5: x w^{r (k1 + 1/2)}; rows (k1, n3) -> operand rows r = (n2, n3), K = (ri, k1) ----------------
      hop_rows<N2, G::T2T / TS, TS>(tml, K2, ts, [&](int t, int g, const uint32_t (&re)[4], const uint32_t (&im)[4]) {   // n2 = 8 g ..
        const int k1 = l >> 3, n3 = 8 * t + (l & 7);
        const uint32_t ta = hdr + G::TA5_OFF + k1 * (K2 * 2);
        const uint32_t tbs = lds32(hdr + G::TB5_OFF + (k1 * N3 + n3) * 4);          // (Re, Im) of the n3 part
        const uint32_t tbr = __byte_perm(tbs, tbs, 0x1010), tbi = __byte_perm(tbs, tbs, 0x3232);
        const uint4 ar4 = lds128(ta + 16 * g), ai4 = lds128(ta + N2 * 2 + 16 * g);
        const uint32_t ar[4] = {ar4.x, ar4.y, ar4.z, ar4.w}, ai[4] = {ai4.x, ai4.y, ai4.z, ai4.w};
        uint32_t orr[4], oi[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t wr, wi;
          cmul_h2(ar[i], ai[i], tbr, tbi, wr, wi);
          cmul_h2(re[i], im[i], wr, wi, orr[i], oi[i]);
        }
        // row group j5 = n2hi N3 + n3, K index k1 / 16 + k1
        const uint32_t d = data + (g * N3 + n3) * G::SBO5 + (k1 >> 3) * 128 + (k1 & 7) * 16;
        sts128(d, orr[0], orr[1], orr[2], orr[3]);
        sts128(d + 2 * 128, oi[0], oi[1], oi[2], oi[3]);
      });
      tc::tc_fence_before();
      LCL_STAGE(5)

      if constexpr (ASYNC) {
        const bool last = f + 1 == P.nf;
        if (XP) {
          // the operand regions are free: the next raw row goes into RA while this pass finishes
          if (!last) stage_swz(RA, urow);
          else if (rowid + stride < P.rows) stage_swz(RA, x1_of(rowid + stride));
        } else {
          // ... x2, or the gated result this slot's threads wrote to the output a pass ago, goes into SB
          stage_lin(SB, f == 0 ? (const void*)x2row : (const void*)orow);
        }
        cp_async_commit();
        // x2's two steps before each chunk come from the lane below; lane 0 fetches its own (L2: the row was just copied)
        uint32_t hh[LIT];
#pragma unroll
        for (int it = 0; it < LIT; ++it) {
          const int c = it * TPS + sl;
          hh[it] = 0u;
          if (f == 0 && lane == 0 && c > 0 && 8 * c < P.L) hh[it] = __ldg(reinterpret_cast<const uint32_t*>(x2row + 8 * c - 2));
        }
        if (XP && f == 0) cp_async_wait<1>();      // this thread's pieces of x2 (all but the newest group)
        if (BIG && f == 1) {                       // the last re-layout adds to the gated result: it has to be there
          cp_async_wait<0>();
          LCL_BARRIER()
        }
        // ---- hop 6: time R n1 + r gets bf16(y 2^-e) -- in the residual pass added to the first pass's gated result,
        // which waits in SB -- at element t + 8 (t / 64) of the output buffer: neither these 2-byte scattered
        // accesses nor the epilogue's 16-byte reads meet bank conflicts
#pragma unroll 1
        for (int t = ts; t < G::T1T; t += TS) {
          uint32_t z[16];
          tc::tmem_ld16(tml + 16 * t, z);
          tc::tmem_ld_wait();
          const int j5 = 16 * t + (l >> 3), n2 = 8 * (j5 / N3) + (l & 7), n3 = j5 % N3;
          const int r = N3 * n2 + n3;
          const uint32_t yp = data + 2 * (r + 8 * (r >> 6));
          float y[16];
#pragma unroll
          for (int n1 = 0; n1 < 16; ++n1) y[n1] = __uint_as_float(z[n1]) * ig;
          if (f == 1) {
            const uint32_t op = SB + 16 * ((r >> 3) ^ ((r >> 6) & 1)) + 2 * (r & 7);     // (R / 8) n1 is a multiple of 16 chunks
#pragma unroll
            for (int n1 = 0; n1 < 16; ++n1) {
              const float o = __uint_as_float(lds16(op + n1 * 2 * R) << 16);
              y[n1] = o + (P.yu_bf16 ? bf16r(y[n1]) : y[n1]);
            }
          }
#pragma unroll
          for (int n1 = 0; n1 < 16; n1 += 2) {
            const uint32_t pk = pack_bf2(y[n1], y[n1 + 1]);
            sts16(yp + n1 * (2 * (R + R / 8)), pk & 0xffffu);
            sts16(yp + (n1 + 1) * (2 * (R + R / 8)), pk >> 16);
          }
        }
        if (BIG && f == 0) cp_async_wait<0>();     // x2 came in behind the re-layout
        tc::tc_fence_before();
        LCL_BARRIER()
        // after a residual pass SB (the gated result) and the scalars are done with: the next sequence's v and scalars
        // start their way here; after a single-filter pass SB holds x2 for the epilogue below and they start after it
        auto stage_next_v = [&]() {
          if (rowid + stride < P.rows) {
            stage_scalars(rowid + stride);
            if (XP) stage_swz(SB, x1_of(rowid + stride) + 2 * (long long)P.D * P.xsc);
          }
          cp_async_commit();
        };
        if (last && f == 1) stage_next_v();
        if (f == 0) {
          // ---- first epilogue: (conv + bias term as bf16) x short conv of x2; kept in SB when a residual pass follows
          const Taps2 T2 = taps_of(1);
#pragma unroll
          for (int it = 0; it < LIT; ++it) {
            const int c = it * TPS + sl, t0 = 8 * c;
            const bool in = t0 < P.L;
            uint4 x = make_uint4(0u, 0u, 0u, 0u);
            const uint32_t sbc = SB + 16 * (c ^ ((c >> 3) & 1));
            if (in) x = lds128(sbc);
            uint32_t h = __shfl_up_sync(0xffffffffu, x.w, 1);
            if (lane == 0) h = hh[it];
            if (in) {
              const uint32_t wx[5] = {h, x.x, x.y, x.z, x.w};
              uint32_t c2[4];
              conv_packed<8>(T2, wx, c2);
              const uint4 y = lds128(data + 16 * c + 16 * (c >> 3));
              const uint4 o = make_uint4(bf2_mul(y.x, c2[0]), bf2_mul(y.y, c2[1]), bf2_mul(y.z, c2[2]), bf2_mul(y.w, c2[3]));
              if (last || BIG) *reinterpret_cast<uint4*>(orow + t0) = o;
              else sts128(sbc, o.x, o.y, o.z, o.w);
            }
          }
        } else {
          // ---- second epilogue: the sums are in the output buffer; one 16-byte store per 8 steps
#pragma unroll
          for (int it = 0; it < LIT; ++it) {
            const int c = it * TPS + sl, t0 = 8 * c;
            if (t0 < P.L) *reinterpret_cast<uint4*>(orow + t0) = lds128(data + 16 * c + 16 * (c >> 3));
          }
        }
        if (XP && !last) cp_async_wait<0>();       // u has had the whole epilogue to arrive
        LCL_BARRIER()                              // output buffer, SB (after the last pass) and RA's copy are settled
        if (last && f == 0) stage_next_v();
      } else {
      // ---------------- hop 6: y[R n1 + r] (float32) into shared memory in time order, 4 floats of padding after every 32
      // (position t lives at t + 4 (t / 32): the scattered writes below and the float4 reads of the epilogue are both
      // free of bank conflicts) ----------------
#pragma unroll 1
      for (int t = ts; t < G::T1T; t += TS) {
        uint32_t z[16];
        tc::tmem_ld16(tml + 16 * t, z);
        tc::tmem_ld_wait();
        const int j5 = 16 * t + (l >> 3), n2 = 8 * (j5 / N3) + (l & 7), n3 = j5 % N3;
        const int r = N3 * n2 + n3;
        float* yp = Y + r + 4 * (r >> 5);
#pragma unroll
        for (int n1 = 0; n1 < 16; ++n1) yp[n1 * (R + R / 8)] = __uint_as_float(z[n1]);
      }
      tc::tc_fence_before();
      LCL_BARRIER()

      // ---------------- epilogue: gate / residual add; 8-byte stores along time ----------------
      const f32x2 gain2 = f2_splat(ig);                                                             // undo the table's 2^e
      if (f == 0) {
        const Taps2 T2 = load_taps2(P.sw, P.sb, P.D + ch);
#pragma unroll 1
        for (int it0 = 0; it0 < EIT; it0 += EB) {
          uint32_t xr[EB][3];
#pragma unroll
          for (int i = 0; i < EB; ++i) load_raw<4>(x2row, 4 * ((it0 + i) * TPS + sl), P.L, false, xr[i]);
#pragma unroll
          for (int i = 0; i < EB; ++i) {
            const int t0 = 4 * ((it0 + i) * TPS + sl);
            if (t0 < P.L) {
              uint32_t c2[2], o[2];
              conv_packed<4>(T2, xr[i], c2);
              const float4 y = *reinterpret_cast<const float4*>(Y + t0 + 4 * (t0 >> 5));
              float a0, a1, a2, a3;
              f2_unpack(f2_mul(f2_pack(y.x, y.y), gain2), a0, a1);
              f2_unpack(f2_mul(f2_pack(y.z, y.w), gain2), a2, a3);
              o[0] = bf2_mul(pack_bf2(a0, a1), c2[0]);                  // (conv + bias term) cast to bf16, then the gate
              o[1] = bf2_mul(pack_bf2(a2, a3), c2[1]);
              *reinterpret_cast<uint2*>(orow + t0) = make_uint2(o[0], o[1]);
            }
          }
        }
      } else {
#pragma unroll 1
        for (int it0 = 0; it0 < EIT; it0 += EB) {
          uint2 prev[EB];                                    // y * x2 written by this thread for f == 0
#pragma unroll
          for (int i = 0; i < EB; ++i) {
            const int t0 = 4 * ((it0 + i) * TPS + sl);
            prev[i] = t0 < P.L ? *reinterpret_cast<const uint2*>(orow + t0) : make_uint2(0u, 0u);
          }
#pragma unroll
          for (int i = 0; i < EB; ++i) {
            const int t0 = 4 * ((it0 + i) * TPS + sl);
            if (t0 < P.L) {
              const float4 y = *reinterpret_cast<const float4*>(Y + t0 + 4 * (t0 >> 5));
              float yv[4];
              f2_unpack(f2_mul(f2_pack(y.x, y.y), gain2), yv[0], yv[1]);
              f2_unpack(f2_mul(f2_pack(y.z, y.w), gain2), yv[2], yv[3]);
              if (P.yu_bf16) {                                 // bf16 layer input: yu is cast to bf16 first
#pragma unroll
                for (int j = 0; j < 4; ++j) yv[j] = bf16r(yv[j]);
              }
              *reinterpret_cast<uint2*>(orow + t0) =
                  make_uint2(pack_bf2(bf_lo(prev[i].x) + yv[0], bf_hi(prev[i].x) + yv[1]),
                             pack_bf2(bf_lo(prev[i].y) + yv[2], bf_hi(prev[i].y) + yv[3]));
            }
          }
        }
      }
      LCL_BARRIER()                                          // the y buffer is free again
      }
    }
  }
#undef LCL_STAGE
#undef LCL_BARRIER

  if constexpr (ASYNC) cp_async_wait<0>();         // nothing may still be landing when the block gives its memory back
  __syncthreads();
  if (warp == 0) {
    tc::tc_fence_after();
    tc::tmem_dealloc(*tmem_slot, G::TCOLS);
  }
}

using Geo4k = Geo<16, 8, 8, 1>;
using Geo16k = Geo<32, 16, 4, 1>;
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

template <typename G, typename TU, bool ASYNC = false>
static int launch_conv(const Params& P, cudaStream_t st) {
  auto kern = longconv_tcl_kernel<G, TU, ASYNC>;
  constexpr int SMEM = !ASYNC ? G::SMEM : G::CAN_ASYNC ? G::SMEM_A : G::SMEM_B;
  M2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int need = (P.rows + G::SLOTS - 1) / G::SLOTS;
  const int grid = need < sms ? need : sms;
  kern<<<grid, G::THREADS, SMEM, st>>>(P);
  M2_LAUNCH_CHECK("longconv_tcl_kernel");
  return M2_OK;
}

}  // namespace lcl

// 2 when the long-row tensor-core family covers (seq_len, dtype); the caller must then
// supply time-contiguous tensors
int longconv_tcl_supported(int seq_len, m2_dtype act_dtype) {
  if (act_dtype != M2_BF16 || seq_len % 4 != 0) return 0;
  // transform length 4096 up to 2048, 16384 up to 8192, else 65536; lengths from 129 on run the 4096-point
  // transform with more zero padding (still several times faster than the float32 CUDA-core family)
  return seq_len > 128 && seq_len <= 32768;
}

// header + per channel N/2 half2 bins + per channel one float (2^-e, see gain_scale)
size_t spectrum_kind2_floats(int D, int L) {
  if (L <= 2048) return (size_t)lcl::Geo4k::HDR_FLOATS + (size_t)(lcl::Geo4k::N / 2 + 1) * D;
  if (L <= 8192) return (size_t)lcl::Geo16k::HDR_FLOATS + (size_t)(lcl::Geo16k::N / 2 + 1) * D;
  return (size_t)lcl::Geo64k::HDR_FLOATS + (size_t)(lcl::Geo64k::N / 2 + 1) * D;
}

int spectrum_kind2_launch(int D, int L, const float* k, float* spec, cudaStream_t st) {
  M2_REQUIRE(longconv_tcl_supported(L, M2_BF16), M2_ERR_UNSUPPORTED,
             "m2_filter_spectrum: kind 2 covers 128 < seq_len <= 32768, multiples of 4");
  const int R = m2_filter_row_len(L);
  if (L <= 2048) return lcl::launch_spectrum<lcl::Geo4k>(D, R, k, spec, st);
  if (L <= 8192) return lcl::launch_spectrum<lcl::Geo16k>(D, R, k, spec, st);
  return lcl::launch_spectrum<lcl::Geo64k>(D, R, k, spec, st);
}

int longconv_tcl_launch(const m2_longconv_args* a, cudaStream_t st) {
  using namespace lcl;
  M2_REQUIRE(longconv_tcl_supported(a->seq_len, a->act_dtype), M2_ERR_UNSUPPORTED,
             "m2_longconv_fwd: kind 2 needs bf16 activations and 128 < seq_len <= 32768, a multiple of 4");
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
  // 16-byte row starts allow one 16-byte load per 8 time steps; otherwise two 8-byte loads
  P.al16 = a->xin_sc % 8 == 0 && a->xin_sb % 8 == 0 && m2_aligned(a->xin, 16) &&
           (a->n_filters == 1 || a->u_dtype == M2_F32 || (a->u_sc % 8 == 0 && a->u_sb % 8 == 0 && m2_aligned(a->u, 16)));
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
  // rows staged through shared memory ahead of their use: 16-byte pieces of every row, bf16 output buffer
  const bool staged = P.al16 && a->seq_len % 8 == 0 && a->out_sc % 8 == 0 && a->out_sb % 8 == 0 && m2_aligned(a->out, 16) &&
                      (a->n_filters == 1 || ubf);
  if (a->seq_len <= 2048) {
    if (staged) return launch_conv<Geo4k, __nv_bfloat16, true>(P, st);
    return ubf ? launch_conv<Geo4k, __nv_bfloat16>(P, st) : launch_conv<Geo4k, float>(P, st);
  }
  if (a->seq_len <= 8192) {
    if (staged) return launch_conv<Geo16k, __nv_bfloat16, true>(P, st);
    return ubf ? launch_conv<Geo16k, __nv_bfloat16>(P, st) : launch_conv<Geo16k, float>(P, st);
  }
  if (staged) return launch_conv<Geo64k, __nv_bfloat16, true>(P, st);
  return ubf ? launch_conv<Geo64k, __nv_bfloat16>(P, st) : launch_conv<Geo64k, float>(P, st);
}

}  // namespace m2
