// Fused gated long convolution on tcgen05 tensor cores for long rows (kernel family 2):
// bf16 activations stored time-contiguous ((B, channels, L) layout), transform length
// N = 32 * N2 * N3 = 4096 (1024 < L <= 2048) or 16384 (4096 < L <= 8192).
//
// One (batch row, channel) sequence is processed at a time by a "slot" of four warps; a CTA
// holds several slots that run independently (own barriers, own TMEM columns, own shared-
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
//   outputs y[R n1 + r], n1 < 16.
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

namespace m2 {
namespace lcl {

constexpr float S1 = 0.25f;
__host__ __device__ constexpr float stage_scale(int n) {   // 2^-ceil(log2(n)/2)
  return n >= 64 ? 0.125f : n >= 32 ? 0.125f : n >= 16 ? 0.25f : n >= 8 ? 0.25f : 0.5f;
}

template <int N2_, int N3_>
struct Geo {
  static constexpr int N2 = N2_, N3 = N3_;
  static constexpr int R = N2 * N3;             // rows of stage 1 = N / 32
  static constexpr int N = 32 * R;
  static constexpr int K2 = 2 * N2, K3 = 2 * N3;
  static constexpr int TR = R / 128;            // row tiles of F1 / I1
  static constexpr int T2T = 16 * N3 / 128;     // row tiles of F2 / I2
  static constexpr int T3T = 16 * N2 / 128;     // row tiles of F3 / I3
  static constexpr int DATA_BYTES = 64 * R;     // half spectrum as fp16 complex = every stage's operand set
  static constexpr int COLS = (TR * 32 > T2T * K2 ? (TR * 32 > T3T * K3 ? TR * 32 : T3T * K3)
                                                  : (T2T * K2 > T3T * K3 ? T2T * K2 : T3T * K3));
  static constexpr int SLOTS = (R >= 512) ? 4 : 4;
  static constexpr int TCOLS = (SLOTS * COLS <= 32) ? 32 : (SLOTS * COLS <= 64) ? 64 : (SLOTS * COLS <= 128) ? 128
                               : (SLOTS * COLS <= 256) ? 256 : 512;
  static constexpr float S2 = stage_scale(N2), S3 = stage_scale(N3);
  static constexpr float KAPPA = (2.0f / N) / ((S1 * S2 * S3) * (S1 * S2 * S3));
  // header of the spectrum table (bytes): constant matrices and twiddle tables
  static constexpr int F1_OFF = 0;                       // [32 x 16]
  static constexpr int I1_OFF = F1_OFF + 1024;           // [16 x 32]
  static constexpr int F2_OFF = I1_OFF + 1024;           // [K2 x K2]
  static constexpr int I2_OFF = F2_OFF + K2 * K2 * 2;
  static constexpr int F3_OFF = I2_OFF + K2 * K2 * 2;    // [K3 x K3]
  static constexpr int I3_OFF = F3_OFF + K3 * K3 * 2;
  static constexpr int T1_OFF = I3_OFF + K3 * K3 * 2;    // half2 [16][R]
  static constexpr int T2A_OFF = T1_OFF + 64 * R;        // half2 [N2][N3]  (k2 major)
  static constexpr int T2B_OFF = T2A_OFF + 4 * R;        // half2 [N3][N2]  (n3 major)
  static constexpr int HDR_BYTES = T2B_OFF + 4 * R;
  static constexpr int HDR_FLOATS = HDR_BYTES / 4;
  static constexpr int THREADS = SLOTS * 128;
  static constexpr int SMEM = SLOTS * DATA_BYTES + HDR_BYTES + 16 * SLOTS * 8 + 64 + 128;
  static_assert(R % 128 == 0 && (16 * N3) % 128 == 0 && (16 * N2) % 128 == 0, "row tiles must be full");
  static_assert(SLOTS * COLS <= 512, "accumulators exceed tensor memory");
};

// byte offset of element (row, k) in a K-major un-swizzled tile set with K columns:
// 128-row tiles, 8-row groups of K/8 core matrices, 16 bytes per row of a core matrix
template <int K>
__host__ __device__ constexpr int op_off(int row, int k) {
  return (row >> 7) * (128 * K * 2) + ((row & 127) >> 3) * (K * 16) + (k >> 3) * 128 + (row & 7) * 16 + (k & 7) * 2;
}

// ---------------------------------------------------------------------------------------
// Spectrum table (kind 2): [HDR_FLOATS floats: matrices + twiddles] then per channel
// G[(k1 N2 + k2)][k3] as half2, multiplied by KAPPA.  Built with an N-point complex FFT in
// shared memory of g[n] w^{n/2} (g = the filter with its wrapped half negated).
// ---------------------------------------------------------------------------------------
template <typename G>
__global__ void __launch_bounds__(512)
spectrum_kind2_kernel(const float* __restrict__ kfilt, float* __restrict__ spec, int D) {
  constexpr int N = G::N, N2 = G::N2, N3 = G::N3, R = G::R, K2 = G::K2, K3 = G::K3;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x, nt = blockDim.x;
  if (blockIdx.x == (unsigned)D) {
    __half* m = reinterpret_cast<__half*>(spec);
    for (int idx = tid; idx < 16 * 16; idx += nt) {            // F1 rows 2k1+ri, I1 columns 2k1+ri
      const int k1 = idx / 16, n1 = idx % 16;
      double sn, cs;
      sincospi(2.0 * n1 * (k1 + 0.5) / 32.0, &sn, &cs);
      m[(G::F1_OFF + op_off<16>(2 * k1, n1)) / 2] = __double2half(S1 * cs);
      m[(G::F1_OFF + op_off<16>(2 * k1 + 1, n1)) / 2] = __double2half(-S1 * sn);
      m[(G::I1_OFF + op_off<32>(n1, 2 * k1)) / 2] = __double2half(S1 * cs);
      m[(G::I1_OFF + op_off<32>(n1, 2 * k1 + 1)) / 2] = __double2half(-S1 * sn);
    }
    for (int idx = tid; idx < N2 * N2; idx += nt) {            // DFT_N2, forward and inverse, real form
      const int ko = idx / N2, ni = idx % N2;
      double sn, cs;
      sincospi(2.0 * ((ko * ni) % N2) / N2, &sn, &cs);
      const double c = G::S2 * cs, s = G::S2 * sn;             // forward w = c - i s, inverse w = c + i s
      __half* f = m + G::F2_OFF / 2;
      f[op_off<K2>(2 * ko, 2 * ni) / 2] = __double2half(c);
      f[op_off<K2>(2 * ko, 2 * ni + 1) / 2] = __double2half(s);
      f[op_off<K2>(2 * ko + 1, 2 * ni) / 2] = __double2half(-s);
      f[op_off<K2>(2 * ko + 1, 2 * ni + 1) / 2] = __double2half(c);
      __half* g = m + G::I2_OFF / 2;
      g[op_off<K2>(2 * ko, 2 * ni) / 2] = __double2half(c);
      g[op_off<K2>(2 * ko, 2 * ni + 1) / 2] = __double2half(-s);
      g[op_off<K2>(2 * ko + 1, 2 * ni) / 2] = __double2half(s);
      g[op_off<K2>(2 * ko + 1, 2 * ni + 1) / 2] = __double2half(c);
    }
    for (int idx = tid; idx < N3 * N3; idx += nt) {            // DFT_N3
      const int ko = idx / N3, ni = idx % N3;
      double sn, cs;
      sincospi(2.0 * ((ko * ni) % N3) / N3, &sn, &cs);
      const double c = G::S3 * cs, s = G::S3 * sn;
      __half* f = m + G::F3_OFF / 2;
      f[op_off<K3>(2 * ko, 2 * ni) / 2] = __double2half(c);
      f[op_off<K3>(2 * ko, 2 * ni + 1) / 2] = __double2half(s);
      f[op_off<K3>(2 * ko + 1, 2 * ni) / 2] = __double2half(-s);
      f[op_off<K3>(2 * ko + 1, 2 * ni + 1) / 2] = __double2half(c);
      __half* g = m + G::I3_OFF / 2;
      g[op_off<K3>(2 * ko, 2 * ni) / 2] = __double2half(c);
      g[op_off<K3>(2 * ko, 2 * ni + 1) / 2] = __double2half(-s);
      g[op_off<K3>(2 * ko + 1, 2 * ni) / 2] = __double2half(s);
      g[op_off<K3>(2 * ko + 1, 2 * ni + 1) / 2] = __double2half(c);
    }
    __half2* t1 = reinterpret_cast<__half2*>(reinterpret_cast<unsigned char*>(spec) + G::T1_OFF);
    for (int idx = tid; idx < 16 * R; idx += nt) {             // T1[k1][r] = w^{r (k1 + 1/2)}
      const int k1 = idx / R, r = idx % R;
      double sn, cs;
      sincospi(2.0 * r * (k1 + 0.5) / N, &sn, &cs);
      t1[idx] = __floats2half2_rn((float)cs, (float)(-sn));
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
    return;
  }
  // ---- one channel: N-point complex FFT (decimation in frequency) of g[n] w^{n/2} ----
  float2* s = reinterpret_cast<float2*>(smem_raw);
  const int c = blockIdx.x;
  const float* row = kfilt + (size_t)c * N;
  constexpr int lg = (N == 4096) ? 12 : (N == 16384) ? 14 : 16;
  for (int n = tid; n < N; n += nt) {
    double sn, cs;
    sincospi((double)n / N, &sn, &cs);                         // w^{n/2} = cos(pi n / N) - i sin(pi n / N)
    const double g = (n < N / 2) ? (double)row[n] : -(double)row[n];
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
  __half2* Gt = reinterpret_cast<__half2*>(spec + G::HDR_FLOATS) + (size_t)c * (N / 2);
  for (int idx = tid; idx < N / 2; idx += nt) {
    const int k3 = idx % N3, k2 = (idx / N3) % N2, k1 = idx / (N3 * N2);
    const int k = k1 + 32 * k2 + 32 * N2 * k3;
    const int p = (int)(__brev((unsigned)k) >> (32 - lg));
    Gt[idx] = __floats2half2_rn(s[p].x * G::KAPPA, s[p].y * G::KAPPA);
  }
}

// ---------------------------------------------------------------------------------------
struct Params {
  int B, L, D, nf, rows;
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
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}

// (a + i b)(c + i d) and (a + i b) conj(c + i d)
__device__ __forceinline__ float2 cmulf(float2 x, float2 w) { return make_float2(x.x * w.x - x.y * w.y, x.x * w.y + x.y * w.x); }
__device__ __forceinline__ float2 cmulcf(float2 x, float2 w) { return make_float2(x.x * w.x + x.y * w.y, x.y * w.x - x.x * w.y); }

// depthwise 3-tap conv over 4 consecutive time steps of one channel; in[0..1] = x[t0-2], x[t0-1]
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

template <typename G>
__device__ __forceinline__ void issue_stage(int stage, uint32_t tm, uint32_t data, uint32_t hdr) {
  constexpr int K2 = G::K2, K3 = G::K3;
  if (stage == 0) {
    constexpr uint32_t id = tc::make_idesc(128, 32, 0);
    const uint64_t dB = tc::smem_desc_k_nosw(hdr + G::F1_OFF, 128, 16 * 16);
#pragma unroll
    for (int t = 0; t < G::TR; ++t)
      tc::mma_ss(tm + 32 * t, tc::smem_desc_k_nosw(data + t * 4096, 128, 16 * 16), dB, id, 0);
  } else if (stage == 1 || stage == 4) {
    constexpr uint32_t id = tc::make_idesc(128, K2, 0);
    const uint32_t mb = hdr + (stage == 1 ? G::F2_OFF : G::I2_OFF);
#pragma unroll
    for (int t = 0; t < G::T2T; ++t)
#pragma unroll
      for (int s = 0; s < K2 / 16; ++s)
        tc::mma_ss(tm + K2 * t, tc::smem_desc_k_nosw(data + t * (128 * K2 * 2) + s * 256, 128, K2 * 16),
                   tc::smem_desc_k_nosw(mb + s * 256, 128, K2 * 16), id, s ? 1u : 0u);
  } else if (stage == 2 || stage == 3) {
    constexpr uint32_t id = tc::make_idesc(128, K3, 0);
    const uint32_t mb = hdr + (stage == 2 ? G::F3_OFF : G::I3_OFF);
#pragma unroll
    for (int t = 0; t < G::T3T; ++t)
#pragma unroll
      for (int s = 0; s < K3 / 16; ++s)
        tc::mma_ss(tm + K3 * t, tc::smem_desc_k_nosw(data + t * (128 * K3 * 2) + s * 256, 128, K3 * 16),
                   tc::smem_desc_k_nosw(mb + s * 256, 128, K3 * 16), id, s ? 1u : 0u);
  } else {
    constexpr uint32_t id = tc::make_idesc(128, 16, 0);
#pragma unroll
    for (int t = 0; t < G::TR; ++t)
#pragma unroll
      for (int s = 0; s < 2; ++s)
        tc::mma_ss(tm + 16 * t, tc::smem_desc_k_nosw(data + t * 8192 + s * 256, 128, 32 * 16),
                   tc::smem_desc_k_nosw(hdr + G::I1_OFF + s * 256, 128, 32 * 16), id, s ? 1u : 0u);
  }
}

template <typename G, typename TU>
__global__ void __launch_bounds__(G::THREADS, 1)
longconv_tcl_kernel(const Params P) {
  constexpr int N2 = G::N2, N3 = G::N3, R = G::R, K2 = G::K2, K3 = G::K3;
  constexpr int CH = R / 4;                      // 4-wide time chunks per n1 block
  constexpr int GROUPS = (128 * 4) / R > 0 ? (128 * 4) / R : 1;   // n1 groups when R < 512
  constexpr int NP = 16 / GROUPS;                // n1 values per thread in the load / store phases
  constexpr int CPT = (CH * GROUPS) / 128;       // chunks per thread (1 unless R > 512)
  static_assert(CPT == 1, "this kernel covers R <= 512");
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
  unsigned char* hdrb = smem + G::SLOTS * G::DATA_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(hdrb + G::HDR_BYTES);       // per slot: ops, mma, w
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * G::SLOTS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slot = warp >> 2;
  const int l = (warp & 3) * 32 + lane;          // TMEM lane = row within every 128-row tile
  if (tid == 0) {
    for (int s = 0; s < G::SLOTS; ++s) {
      tc::mbar_init(bars + 3 * s, 128);
      tc::mbar_init(bars + 3 * s + 1, 1);
      tc::mbar_init(bars + 3 * s + 2, 128);
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
  // load / store phase mapping: chunk of 4 consecutive r, NP consecutive n1
  const int pc = l % CH, pg = l / CH;
  const int r0 = 4 * pc, n1_0 = pg * NP;
  uint32_t ph_ops = 0, ph_mma = 0, ph_w = 0;
  bool ok = true;

#define LCL_STAGE(stage_)                                                                             \
  tc::fence_proxy_async_smem();                                                                       \
  tc::mbar_arrive(bar_ops);                                                                           \
  if (l == 0) {                                                                                       \
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
      {
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
                  a[e][0] = bf_lo(v.x); a[e][1] = bf_hi(v.x); a[e][2] = bf_lo(v.y); a[e][3] = bf_hi(v.y);
                }
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) hv[j][i >> 1] = pack_h2(a[0][j], a[1][j]);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int q = 0; q < NP / 4; ++q)
            sts64(data + op_off<16>(r0 + j, n1_0 + 4 * q), hv[j][2 * q], hv[j][2 * q + 1]);
      }
      LCL_STAGE(0)

      // ---------------- hop 1: x T1, rows (n2, n3) -> rows (k1, n3), k = (n2, ri) ----------------
#pragma unroll 1
      for (int t = 0; t < G::TR; ++t) {
        const int r = 128 * t + l, n2 = r / N3, n3 = r % N3;
#pragma unroll
        for (int hq = 0; hq < 2; ++hq) {
          uint32_t z[16];
          tc::tmem_ld16(tml + 32 * t + 16 * hq, z);
          tc::tmem_ld_wait();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const int k1 = 8 * hq + kk;
            const float2 w = unpack_h2(lds32(t1s + (k1 * R + r) * 4));
            const float2 y = cmulf(make_float2(__uint_as_float(z[2 * kk]), __uint_as_float(z[2 * kk + 1])), w);
            sts32(data + op_off<K2>(k1 * N3 + n3, 2 * n2), pack_h2(y.x, y.y));
          }
        }
      }
      tc::tc_fence_before();
      LCL_STAGE(1)

      // ---------------- hop 2: x T2, rows (k1, n3) -> rows (k1, k2), k = (n3, ri) ----------------
#pragma unroll 1
      for (int t = 0; t < G::T2T; ++t) {
        const int rho = 128 * t + l, k1 = rho / N3, n3 = rho % N3;
#pragma unroll 1
        for (int c0 = 0; c0 < K2; c0 += 16) {
          uint32_t z[16];
          tc::tmem_ld16(tml + K2 * t + c0, z);
          tc::tmem_ld_wait();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const int k2 = c0 / 2 + kk;
            const float2 w = unpack_h2(lds32(t2a + (k2 * N3 + n3) * 4));
            const float2 y = cmulf(make_float2(__uint_as_float(z[2 * kk]), __uint_as_float(z[2 * kk + 1])), w);
            sts32(data + op_off<K3>(k1 * N2 + k2, 2 * n3), pack_h2(y.x, y.y));
          }
        }
      }
      tc::tc_fence_before();
      LCL_STAGE(2)

      // ---------------- hop 3: x (G + bias); rows (k1, k2) keep their place, k = (k3, ri) ----------------
      {
        const uint32_t* Gt = reinterpret_cast<const uint32_t*>(P.spec[f] + G::HDR_FLOATS) + (size_t)ch * (G::N / 2);
        const float bk = __ldg(P.bias[f] + ch) * G::KAPPA;
#pragma unroll 1
        for (int t = 0; t < G::T3T; ++t) {
          const int rho = 128 * t + l;
#pragma unroll 1
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
              o[kk] = pack_h2(y.x, y.y);
            }
            sts128(data + op_off<K3>(rho, c0), o[0], o[1], o[2], o[3]);
            sts128(data + op_off<K3>(rho, c0 + 8), o[4], o[5], o[6], o[7]);
          }
        }
      }
      tc::tc_fence_before();
      LCL_STAGE(3)

      // ---------------- hop 4: x conj T2, rows (k1, k2) -> rows (k1, n3), k = (k2, ri) ----------------
#pragma unroll 1
      for (int t = 0; t < G::T3T; ++t) {
        const int rho = 128 * t + l, k1 = rho / N2, k2 = rho % N2;
#pragma unroll 1
        for (int c0 = 0; c0 < K3; c0 += 16) {
          uint32_t z[16];
          tc::tmem_ld16(tml + K3 * t + c0, z);
          tc::tmem_ld_wait();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const int n3 = c0 / 2 + kk;
            const float2 w = unpack_h2(lds32(t2b + (n3 * N2 + k2) * 4));
            const float2 y = cmulcf(make_float2(__uint_as_float(z[2 * kk]), __uint_as_float(z[2 * kk + 1])), w);
            sts32(data + op_off<K2>(k1 * N3 + n3, 2 * k2), pack_h2(y.x, y.y));
          }
        }
      }
      tc::tc_fence_before();
      LCL_STAGE(4)

      // ---------------- hop 5: x conj T1, rows (k1, n3) -> rows r = (n2, n3), k = (k1, ri) ----------------
#pragma unroll 1
      for (int t = 0; t < G::T2T; ++t) {
        const int rho = 128 * t + l, k1 = rho / N3, n3 = rho % N3;
#pragma unroll 1
        for (int c0 = 0; c0 < K2; c0 += 16) {
          uint32_t z[16];
          tc::tmem_ld16(tml + K2 * t + c0, z);
          tc::tmem_ld_wait();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const int n2 = c0 / 2 + kk;
            const int r = n2 * N3 + n3;
            const float2 w = unpack_h2(lds32(t1s + (k1 * R + r) * 4));
            const float2 y = cmulcf(make_float2(__uint_as_float(z[2 * kk]), __uint_as_float(z[2 * kk + 1])), w);
            sts32(data + op_off<32>(r, 2 * k1), pack_h2(y.x, y.y));
          }
        }
      }
      tc::tc_fence_before();
      LCL_STAGE(5)

      // ---------------- hop 6: y[R n1 + r] (float32) into shared memory in time order ----------------
#pragma unroll 1
      for (int t = 0; t < G::TR; ++t) {
        uint32_t z[16];
        tc::tmem_ld16(tml + 16 * t, z);
        tc::tmem_ld_wait();
#pragma unroll
        for (int n1 = 0; n1 < 16; ++n1) Y[R * n1 + 128 * t + l] = __uint_as_float(z[n1]);
      }
      tc::tc_fence_before();
      LCL_BARRIER()

      // ---------------- epilogue: gate / residual add; 8-byte stores along time ----------------
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
            const float yv[4] = {y.x, y.y, y.z, y.w};
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
            float yv[4] = {y.x, y.y, y.z, y.w};
            if (sizeof(TU) == 2) {                           // bf16 layer input: yu is cast to bf16 first
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
      LCL_BARRIER()                                          // the y buffer is free again
    }
  }
#undef LCL_STAGE
#undef LCL_BARRIER

  __syncthreads();
  if (warp == 0) {
    tc::tc_fence_after();
    tc::tmem_dealloc(*tmem_slot, G::TCOLS);
  }
}

using Geo4k = Geo<16, 8>;
using Geo16k = Geo<32, 16>;

template <typename G>
static int launch_spectrum(int D, const float* k, float* spec, cudaStream_t st) {
  auto kern = spectrum_kind2_kernel<G>;
  const size_t smem = (size_t)G::N * sizeof(float2);
  M2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<D + 1, 512, smem, st>>>(k, spec, D);
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
  return (seq_len > 1024 && seq_len <= 2048) || (seq_len > 4096 && seq_len <= 8192);
}

size_t spectrum_kind2_floats(int D, int L) {
  if (L <= 2048) return (size_t)lcl::Geo4k::HDR_FLOATS + (size_t)(lcl::Geo4k::N / 2) * D;
  return (size_t)lcl::Geo16k::HDR_FLOATS + (size_t)(lcl::Geo16k::N / 2) * D;
}

int spectrum_kind2_launch(int D, int L, const float* k, float* spec, cudaStream_t st) {
  M2_REQUIRE(longconv_tcl_supported(L, M2_BF16), M2_ERR_UNSUPPORTED,
             "m2_filter_spectrum: kind 2 covers 1024 < seq_len <= 2048 and 4096 < seq_len <= 8192 (multiples of 4)");
  if (L <= 2048) return lcl::launch_spectrum<lcl::Geo4k>(D, k, spec, st);
  return lcl::launch_spectrum<lcl::Geo16k>(D, k, spec, st);
}

int longconv_tcl_launch(const m2_longconv_args* a, cudaStream_t st) {
  using namespace lcl;
  M2_REQUIRE(longconv_tcl_supported(a->seq_len, a->act_dtype), M2_ERR_UNSUPPORTED,
             "m2_longconv_fwd: kind 2 needs bf16 activations and 1024 < seq_len <= 2048 or 4096 < seq_len <= 8192");
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
  const bool ubf = a->n_filters == 2 && a->u_dtype == M2_BF16;
  if (a->n_filters == 2) {
    const size_t ua = ubf ? 8 : 16;
    M2_REQUIRE(m2_aligned(a->u, ua) && a->u_sc % 4 == 0 && a->u_sb % 4 == 0, M2_ERR_ALIGN,
               "m2_longconv_fwd: kind 2 needs rows of u aligned to four elements");
  }
  const bool small = a->seq_len <= 2048;
  if (small) return ubf ? launch_conv<Geo4k, __nv_bfloat16>(P, st) : launch_conv<Geo4k, float>(P, st);
  return ubf ? launch_conv<Geo16k, __nv_bfloat16>(P, st) : launch_conv<Geo16k, float>(P, st);
}

}  // namespace m2
