// Implicit Hyena filter generation and the filter-spectrum tables of the long convolution.
//
// Computation replaced (reference paths relative to the HazyResearch/m2 checkout):
//   bert/src/mm/hyena_utils.py:201-217  HyenaFilter.filter / filter_rev
//   bert/src/mm/hyena_utils.py:62-63    Sin.forward
//   bert/src/mm/hyena_utils.py:109-112  ExponentialModulation.forward
//   bert/src/mm/hyena_utils.py:231-234  bidirectional merge (pad + flip + add)
//   bert/src/mm/hyena_utils.py:23-24    rfft of the kernel, scaled by 1/(2L)
#include "common.cuh"

namespace m2 {

constexpr int FILT_TL = 8;         // sequence positions per CTA
constexpr int FILT_THREADS = 128;
constexpr int FILT_MAX_ORDER = 256;
constexpr int FILT_MAX_EMB = 16;

struct FilterParams {
  int D, L, order, emb, bidir, row_len;
  float w_mod, shift;
  const float* z; const float* t;
  const float* w[2][4]; const float* b[2][3];
  const float* freq; const float* deltas;
  float* k_out;
};

// ACC = float reproduces a bf16 GEMM with float32 accumulation (ROUND = true);
// ACC = double is the float32 mode: sums and sin/exp in double so that the result is
// limited by the float32 output format only.
template <bool ROUND, typename ACC>
__global__ void __launch_bounds__(FILT_THREADS)
hyena_filter_kernel(FilterParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  ACC* hA = reinterpret_cast<ACC*>(smem_raw);          // [FILT_TL][order]
  ACC* hB = hA + FILT_TL * p.order;                     // [FILT_TL][order]
  const int net = blockIdx.y;                            // 0 forward net, 1 reverse net
  const int l0 = blockIdx.x * FILT_TL;
  const int tid = threadIdx.x;
  const int order = p.order, emb = p.emb;
  const float* const* W = p.w[net];
  const float* const* Bv = p.b[net];

  // layer 0: (emb -> order), Sin
  for (int idx = tid; idx < FILT_TL * order; idx += FILT_THREADS) {
    const int li = idx / order, j = idx % order;
    const int l = l0 + li;
    ACC acc = 0;
    if (l < p.L) {
      for (int i = 0; i < emb; ++i)
        acc += (ACC)rnd<ROUND>(p.z[(size_t)l * emb + i]) * (ACC)rnd<ROUND>(W[0][j * emb + i]);
      acc += (ACC)rnd<ROUND>(Bv[0][j]);
      if (ROUND) {
        float x = bf16r((float)acc);
        float arg = (p.w_mod * p.freq[j]) * x;
        acc = (ACC)sinf(arg);
      } else {
        acc = (ACC)sin((double)(p.w_mod * p.freq[j]) * (double)acc);
      }
    }
    hA[idx] = acc;
  }
  __syncthreads();

  // layers 1, 2: (order -> order), Sin
  ACC* src = hA; ACC* dst = hB;
  for (int layer = 1; layer <= 2; ++layer) {
    for (int idx = tid; idx < FILT_TL * order; idx += FILT_THREADS) {
      const int li = idx / order, j = idx % order;
      const float* wrow = W[layer] + (size_t)j * order;
      ACC acc = 0;
      for (int i = 0; i < order; ++i) {
        const ACC hv = ROUND ? (ACC)bf16r((float)src[li * order + i]) : src[li * order + i];
        const ACC wv = ROUND ? (ACC)bf16r(wrow[i]) : (ACC)wrow[i];
        acc += hv * wv;
      }
      acc += (ACC)rnd<ROUND>(Bv[layer][j]);
      if (ROUND) {
        float x = bf16r((float)acc);
        float arg = (p.w_mod * p.freq[j]) * x;
        acc = (ACC)sinf(arg);
      } else {
        acc = (ACC)sin((double)(p.w_mod * p.freq[j]) * (double)acc);
      }
      dst[idx] = acc;
    }
    __syncthreads();
    ACC* tmp = src; src = dst; dst = tmp;
  }

  // output layer (order -> D, no bias), modulation, merged store
  const int twoL = p.row_len;   // row = [k_fwd | zeros | reversed k_rev]
  for (int c = tid; c < p.D; c += FILT_THREADS) {
    const float* wrow = W[3] + (size_t)c * order;
    ACC acc[FILT_TL];
#pragma unroll
    for (int li = 0; li < FILT_TL; ++li) acc[li] = 0;
    for (int i = 0; i < order; ++i) {
      const ACC wv = ROUND ? (ACC)bf16r(wrow[i]) : (ACC)wrow[i];
#pragma unroll
      for (int li = 0; li < FILT_TL; ++li) {
        const ACC hv = ROUND ? (ACC)bf16r((float)src[li * order + i]) : src[li * order + i];
        acc[li] += hv * wv;
      }
    }
    const float ad = fabsf(p.deltas[c]);
#pragma unroll
    for (int li = 0; li < FILT_TL; ++li) {
      const int l = l0 + li;
      if (l >= p.L) continue;
      float kv;
      if (ROUND) {
        const float decay = expf(-p.t[l] * ad);
        kv = bf16r((float)acc[li]) * (decay + p.shift);
      } else {
        const double decay = exp(-(double)p.t[l] * (double)ad);
        kv = (float)((double)acc[li] * (decay + (double)p.shift));
      }
      const int pos = (net == 0) ? l : (twoL - 1 - l);
      p.k_out[(size_t)c * twoL + pos] = kv;
    }
  }
}

// ---- spectrum tables for the shared-memory FFT convolution (kind 0) -----------------
//
// With M = the power of two >= L, the convolution kernel packs a zero-padded real row of
// 2M samples as M complex
// points z[n] = x[2n] + i x[2n+1], transforms with a radix-2 decimation-in-frequency FFT
// (spectrum left in bit-reversed order), and needs per bin
//     Zy[k] = alpha[k] Z[k] + beta[k] conj(Z[(M-k) mod M])
// so that the decimation-in-time inverse of Zy is the packed convolution result.  With
// K = DFT_2M(k), S = (K[k]+K[k+M])/2, Dk = (K[k]-K[k+M])/2, theta = 2 pi k / 2M:
//     alpha = (S - Dk sin(theta)) / M,   beta = i Dk cos(theta) / M.
// Layout of one filter's table (float32): [ M floats: twiddles W_M^j, j < M/2, as (re,im) ]
// followed by, per channel, alpha (M complex) then beta (M complex), both stored at the
// bit-reversed position of their bin.
template <typename R> struct Cplx { R x, y; };

// alpha/beta of bin k from Z[k] and conj(Z[M-k])
__device__ __forceinline__ void alpha_beta(double2 Zk, double2 Zm, int k, int N, double invM, float2* alpha, float2* beta) {
  const double2 Xe = make_double2(0.5 * (Zk.x + Zm.x), 0.5 * (Zk.y + Zm.y));
  const double2 Xo = make_double2(0.5 * (Zk.y - Zm.y), -0.5 * (Zk.x - Zm.x));   // (Zk - Zm) / (2i)
  double sn, cs;
  sincospi(2.0 * k / N, &sn, &cs);                                            // theta = 2 pi k / N
  const double2 Dk = make_double2(Xo.x * cs + Xo.y * sn, Xo.y * cs - Xo.x * sn);   // W^k Xo, W^k = cos - i sin
  *alpha = make_float2((float)((Xe.x - Dk.x * sn) * invM), (float)((Xe.y - Dk.y * sn) * invM));
  *beta = make_float2((float)(-Dk.y * cs * invM), (float)(Dk.x * cs * invM));
}

// R: scalar type of the work array.  GLOBAL = false keeps the M work points in shared
// memory; GLOBAL = true (rows too long for shared memory) works in place in the channel's
// own beta region of the output table, which is overwritten pair by pair at the end.
template <typename R, bool GLOBAL>
__global__ void __launch_bounds__(256)
spectrum_kind0_kernel(const float* __restrict__ k2, float* __restrict__ spec, int D, int M) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int N = 2 * M;
  const int lg = 31 - __clz(M);
  const int tid = threadIdx.x, nt = blockDim.x;
  if (blockIdx.x == (unsigned)D) {   // one extra CTA writes the twiddle table
    for (int j = tid; j < M / 2; j += nt) {
      double sn, cs;
      sincospi(2.0 * j / M, &sn, &cs);
      spec[2 * j] = (float)cs;
      spec[2 * j + 1] = (float)(-sn);
    }
    return;
  }
  const int c = blockIdx.x;
  float2* alpha = reinterpret_cast<float2*>(spec + M + (size_t)c * 4 * M);
  float2* beta = alpha + M;
  Cplx<R>* s = GLOBAL ? reinterpret_cast<Cplx<R>*>(beta) : reinterpret_cast<Cplx<R>*>(smem_raw);
  static_assert(!GLOBAL || sizeof(Cplx<R>) == sizeof(float2), "in-place work array must match the table's element size");
  const float* row = k2 + (size_t)c * N;
  for (int n = tid; n < M; n += nt) s[n] = Cplx<R>{(R)row[2 * n], (R)row[2 * n + 1]};
  __syncthreads();
  for (int h = M / 2; h >= 1; h >>= 1) {
    for (int j = tid; j < M / 2; j += nt) {
      const int g = j / h, pos = j % h;
      const int i0 = g * 2 * h + pos, i1 = i0 + h;
      double sn, cs;
      sincospi(2.0 * pos / (2.0 * h), &sn, &cs);   // W_{2h}^{pos} = cos - i sin
      const Cplx<R> u = s[i0], v = s[i1];
      const double dx = (double)u.x - (double)v.x, dy = (double)u.y - (double)v.y;
      s[i0] = Cplx<R>{(R)(u.x + v.x), (R)(u.y + v.y)};
      s[i1] = Cplx<R>{(R)(dx * cs + dy * sn), (R)(dy * cs - dx * sn)};
    }
    __syncthreads();
  }
  const double invM = 1.0 / M;
  // bins are finished in pairs (k, M-k): both inputs are read before either output is written
  for (int k = tid; k <= M / 2; k += nt) {
    const int km = (M - k) % M;
    const int pk = (lg == 0) ? 0 : (int)(__brev((unsigned)k) >> (32 - lg));
    const int pm = (lg == 0) ? 0 : (int)(__brev((unsigned)km) >> (32 - lg));
    const double2 Zk = make_double2((double)s[pk].x, (double)s[pk].y);
    const double2 Zq = make_double2((double)s[pm].x, (double)s[pm].y);
    float2 a1, b1, a2, b2;
    alpha_beta(Zk, make_double2(Zq.x, -Zq.y), k, N, invM, &a1, &b1);
    alpha_beta(Zq, make_double2(Zk.x, -Zk.y), km, N, invM, &a2, &b2);
    alpha[pk] = a1; beta[pk] = b1;
    if (pm != pk) { alpha[pm] = a2; beta[pm] = b2; }
  }
}

int spectrum_kind0_launch(int D, int L, const float* k, float* spec, cudaStream_t st) {
  int M = 2;
  while (M < L) M <<= 1;
  if (M <= 8192) {
    const size_t smem = (size_t)M * sizeof(Cplx<double>);
    auto kern = spectrum_kind0_kernel<double, false>;
    M2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<D + 1, 256, smem, st>>>(k, spec, D, M);
  } else if (M <= 16384) {
    const size_t smem = (size_t)M * sizeof(Cplx<float>);
    auto kern = spectrum_kind0_kernel<float, false>;
    M2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<D + 1, 256, smem, st>>>(k, spec, D, M);
  } else {
    M2_REQUIRE(M <= 32768, M2_ERR_UNSUPPORTED, "m2_filter_spectrum: seq_len %d too long for kind 0", L);
    spectrum_kind0_kernel<float, true><<<D + 1, 256, 0, st>>>(k, spec, D, M);
  }
  M2_LAUNCH_CHECK("spectrum_kind0_kernel");
  return M2_OK;
}

}  // namespace m2

extern "C" int m2_filter_row_len(int seq_len) {
  int M = 2;
  while (M < seq_len) M <<= 1;
  return 2 * M;
}

extern "C" int m2_hyena_filter(const m2_filter_args* a, void* stream) {
  using namespace m2;
  M2_REQUIRE(a != nullptr, M2_ERR_ARG, "m2_hyena_filter: args is NULL");
  M2_REQUIRE(a->d_model > 0 && a->seq_len > 0 && a->order > 0 && a->emb_dim > 0, M2_ERR_ARG,
             "m2_hyena_filter: sizes must be positive (d_model=%d seq_len=%d order=%d emb_dim=%d)",
             a->d_model, a->seq_len, a->order, a->emb_dim);
  M2_REQUIRE(a->order <= FILT_MAX_ORDER && a->emb_dim <= FILT_MAX_EMB, M2_ERR_UNSUPPORTED,
             "m2_hyena_filter: order <= %d and emb_dim <= %d supported", FILT_MAX_ORDER, FILT_MAX_EMB);
  M2_REQUIRE(a->z && a->t && a->freq && a->deltas && a->k_out, M2_ERR_ARG,
             "m2_hyena_filter: NULL tensor pointer");
  const int nets = a->bidirectional ? 2 : 1;
  FilterParams p;
  p.D = a->d_model; p.L = a->seq_len; p.order = a->order; p.emb = a->emb_dim;
  p.bidir = a->bidirectional; p.w_mod = a->w_mod; p.shift = a->shift;
  p.z = a->z; p.t = a->t; p.freq = a->freq; p.deltas = a->deltas; p.k_out = a->k_out;
  for (int i = 0; i < 4; ++i) {
    M2_REQUIRE(a->w[i] != nullptr, M2_ERR_ARG, "m2_hyena_filter: w[%d] is NULL", i);
    p.w[0][i] = a->w[i];
    p.w[1][i] = a->bidirectional ? a->w_rev[i] : a->w[i];
    M2_REQUIRE(p.w[1][i] != nullptr, M2_ERR_ARG, "m2_hyena_filter: w_rev[%d] is NULL", i);
  }
  for (int i = 0; i < 3; ++i) {
    M2_REQUIRE(a->b[i] != nullptr, M2_ERR_ARG, "m2_hyena_filter: b[%d] is NULL", i);
    p.b[0][i] = a->b[i];
    p.b[1][i] = a->bidirectional ? a->b_rev[i] : a->b[i];
    M2_REQUIRE(p.b[1][i] != nullptr, M2_ERR_ARG, "m2_hyena_filter: b_rev[%d] is NULL", i);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  p.row_len = m2_filter_row_len(a->seq_len);
  M2_CUDA(cudaMemsetAsync(a->k_out, 0, (size_t)a->d_model * p.row_len * sizeof(float), st));
  dim3 grid((a->seq_len + FILT_TL - 1) / FILT_TL, nets);
  if (a->bf16_rounding) {
    size_t smem = 2 * FILT_TL * a->order * sizeof(float);
    hyena_filter_kernel<true, float><<<grid, FILT_THREADS, smem, st>>>(p);
  } else {
    size_t smem = 2 * FILT_TL * a->order * sizeof(double);
    hyena_filter_kernel<false, double><<<grid, FILT_THREADS, smem, st>>>(p);
  }
  M2_LAUNCH_CHECK("hyena_filter_kernel");
  return M2_OK;
}
