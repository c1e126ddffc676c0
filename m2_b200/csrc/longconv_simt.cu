// Fused gated long convolution, float32 arithmetic on CUDA cores (kernel family 0).
//
// One CTA owns a tile of CT channels of one batch row and keeps their packed spectra in
// shared memory for the whole computation: short depthwise conv + pre-gate -> radix-2
// decimation-in-frequency FFT -> per-bin filter multiply -> decimation-in-time inverse ->
// bias, post-gate and (optionally) the residual long convolution on the raw layer input.
// Inputs are read in the layout in_linear wrote them and the result is written in the
// layout out_linear reads, so no transposed copy of an activation ever exists.
//
// This family does all arithmetic in float32 and is the path for float32 activations (and
// for any length not covered by the tensor-core family).
//
// Computation replaced: bert/src/mm/monarch_mixer_sequence_mixer.py:109-149 and
// bert/src/mm/hyena_utils.py:16-42, :219-248 of the reference.
#include "common.cuh"

namespace m2 {

struct ConvParams {
  int B, L, D, M, lgM, CT, nf, plain;
  const void* xin; long long xsb, xst, xsc;
  const void* u;   long long usb, ust, usc;
  void* out;       long long osb, ost, osc;
  const float* sw; const float* sb;
  const float* spec[2]; const float* bias[2];
};

// conv output of channel `ch` (index into the 3D projected channels) at time t, rounded as
// the reference's conv1d output is:  y[t] = b + w0 x[t-2] + w1 x[t-1] + w2 x[t]
template <typename TA, bool ROUND>
__device__ __forceinline__ float short_conv_at(const TA* xb, long long st, long long sc, int ch, int t,
                                               const float* sw, const float* sb) {
  const TA* px = xb + (long long)ch * sc + (long long)t * st;
  const float w0 = rnd<ROUND>(__ldg(sw + 3 * ch)), w1 = rnd<ROUND>(__ldg(sw + 3 * ch + 1)),
              w2 = rnd<ROUND>(__ldg(sw + 3 * ch + 2));
  float acc = rnd<ROUND>(__ldg(sb + ch));
  if (t >= 2) acc = fmaf(w0, ld_as_float(px - 2 * st), acc);
  if (t >= 1) acc = fmaf(w1, ld_as_float(px - st), acc);
  acc = fmaf(w2, ld_as_float(px), acc);
  return rnd<ROUND>(acc);
}

template <typename TA, typename TU, bool ROUND>
__global__ void __launch_bounds__(256)
longconv_simt_kernel(ConvParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float2* s = reinterpret_cast<float2*>(smem_raw);   // [CT][M]
  const int M = p.M, L = p.L, D = p.D, CT = p.CT;
  const int halfM = M >> 1;
  const int tid = threadIdx.x, nt = blockDim.x;
  const int c0 = blockIdx.x * CT;
  const int b = blockIdx.y;
  const bool ch_fast = (p.xsc == 1);
  const TA* xb = reinterpret_cast<const TA*>(p.xin) + (long long)b * p.xsb;
  const TU* ub = reinterpret_cast<const TU*>(p.u) + (long long)b * p.usb;
  TA* ob = reinterpret_cast<TA*>(p.out) + (long long)b * p.osb;
  const int npair = (L + 1) >> 1;                     // packed points that hold data

  // plain mode runs only the un-gated convolution (the f == 1 code path) on spec[1]/bias[1]
  const int f_begin = p.plain ? 1 : 0, f_end = p.plain ? 2 : p.nf;
  for (int f = f_begin; f < f_end; ++f) {
    const float2* tw = reinterpret_cast<const float2*>(p.spec[f]);
    const float2* tab = reinterpret_cast<const float2*>(p.spec[f] + M);   // per channel: alpha[M], beta[M]

    // ---- load + short conv + pre-gate, packed as z[n] = a[2n] + i a[2n+1] ----
    for (int idx = tid; idx < CT * M; idx += nt) {
      int ci, n;
      if (ch_fast) { ci = idx % CT; n = idx / CT; } else { n = idx % M; ci = idx / M; }
      const int c = c0 + ci;
      float2 zv = make_float2(0.f, 0.f);
      if (n < npair && c < D) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int t = 2 * n + e;
          float a = 0.f;
          if (t < L) {
            if (f == 0) {
              const float x1 = short_conv_at<TA, ROUND>(xb, p.xst, p.xsc, c, t, p.sw, p.sb);
              const float v = short_conv_at<TA, ROUND>(xb, p.xst, p.xsc, 2 * D + c, t, p.sw, p.sb);
              a = rnd<ROUND>(v * x1);
            } else {
              a = ld_as_float(ub + (long long)t * p.ust + (long long)c * p.usc);
            }
          }
          if (e == 0) zv.x = a; else zv.y = a;
        }
      }
      s[ci * M + n] = zv;
    }
    __syncthreads();

    // ---- forward FFT, decimation in frequency, result in bit-reversed order ----
    for (int h = halfM; h >= 1; h >>= 1) {
      const int tstep = halfM / h;
      for (int idx = tid; idx < CT * halfM; idx += nt) {
        const int ci = idx / halfM, j = idx % halfM;
        const int g = j / h, pos = j % h;
        float2* base = s + ci * M + g * 2 * h + pos;
        const float2 a = base[0], bb = base[h];
        const float2 w = __ldg(tw + pos * tstep);
        base[0] = make_float2(a.x + bb.x, a.y + bb.y);
        base[h] = cmul(make_float2(a.x - bb.x, a.y - bb.y), w);
      }
      __syncthreads();
    }

    // ---- per-bin filter multiply: Zy[k] = alpha Z[k] + beta conj(Z[M-k]) ----
    // work item = bin pair (k, M-k), k in [0, M/2]; k = 0 and k = M/2 pair with themselves
    for (int idx = tid; idx < CT * (halfM + 1); idx += nt) {
      const int ci = idx / (halfM + 1), k = idx % (halfM + 1);
      const int c = c0 + ci;
      if (c >= D) continue;
      const int km = (M - k) & (M - 1);
      const int pk = (p.lgM == 0) ? 0 : (int)(__brev((unsigned)k) >> (32 - p.lgM));
      const int pm = (p.lgM == 0) ? 0 : (int)(__brev((unsigned)km) >> (32 - p.lgM));
      const float2* al = tab + (size_t)c * 2 * M;
      const float2* be = al + M;
      const float2 Zk = s[ci * M + pk], Zm = s[ci * M + pm];
      const float2 a1 = __ldg(al + pk), b1 = __ldg(be + pk);
      float2 r1 = cmul(a1, Zk);
      const float2 t1 = cmul_conj(b1, Zm);
      r1.x += t1.x; r1.y += t1.y;
      if (pm != pk) {
        const float2 a2 = __ldg(al + pm), b2 = __ldg(be + pm);
        float2 r2 = cmul(a2, Zm);
        const float2 t2 = cmul_conj(b2, Zk);
        r2.x += t2.x; r2.y += t2.y;
        s[ci * M + pm] = r2;
      }
      s[ci * M + pk] = r1;
    }
    __syncthreads();

    // ---- inverse FFT, decimation in time from bit-reversed input, natural-order output ----
    for (int h = 1; h <= halfM; h <<= 1) {
      const int tstep = halfM / h;
      for (int idx = tid; idx < CT * halfM; idx += nt) {
        const int ci = idx / halfM, j = idx % halfM;
        const int g = j / h, pos = j % h;
        float2* base = s + ci * M + g * 2 * h + pos;
        const float2 w = __ldg(tw + pos * tstep);
        const float2 a = base[0];
        const float2 bb = cmul_conj(base[h], w);       // times conj(W) = W^{-1}
        base[0] = make_float2(a.x + bb.x, a.y + bb.y);
        base[h] = make_float2(a.x - bb.x, a.y - bb.y);
      }
      __syncthreads();
    }

    // ---- bias, gates, residual; write out in the (b, t, c) layout ----
    const float* biasv = p.bias[f];
    for (int idx = tid; idx < CT * npair; idx += nt) {
      int ci, n;
      if (ch_fast) { ci = idx % CT; n = idx / CT; } else { n = idx % npair; ci = idx / npair; }
      const int c = c0 + ci;
      if (c >= D) continue;
      const float2 zy = s[ci * M + n];
      const float bc = __ldg(biasv + c);
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int t = 2 * n + e;
        if (t >= L) continue;
        const float y = (e == 0) ? zy.x : zy.y;
        TA* po = ob + (long long)t * p.ost + (long long)c * p.osc;
        if (f == 0) {
          const float x1 = short_conv_at<TA, ROUND>(xb, p.xst, p.xsc, c, t, p.sw, p.sb);
          const float v = short_conv_at<TA, ROUND>(xb, p.xst, p.xsc, 2 * D + c, t, p.sw, p.sb);
          const float x2 = short_conv_at<TA, ROUND>(xb, p.xst, p.xsc, D + c, t, p.sw, p.sb);
          const float a = rnd<ROUND>(v * x1);
          const float yc = rnd<ROUND>(fmaf(a, bc, y));     // conv + u*bias, cast to the activation dtype
          st_from_float(po, rnd<ROUND>(yc * x2));
        } else {
          const float uo = ld_as_float(ub + (long long)t * p.ust + (long long)c * p.usc);
          float yu = fmaf(uo, bc, y);
          // a bf16 layer input makes the reference cast yu back to bf16 before the add; a
          // float32 layer input keeps yu and the sum in float32
          if (ROUND && sizeof(TU) == 2) yu = bf16r(yu);
          const float prev = p.plain ? 0.f : ld_as_float(po);   // y * x2, written by this thread for f == 0
          st_from_float(po, rnd<ROUND>(prev + yu));
        }
      }
    }
    __syncthreads();
  }
}

template <typename TA, typename TU, bool ROUND>
static int launch_simt(const ConvParams& p, size_t smem, cudaStream_t st) {
  auto kern = longconv_simt_kernel<TA, TU, ROUND>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return m2_set_error(M2_ERR_CUDA, "cudaFuncSetAttribute(longconv_simt): %s", cudaGetErrorString(e));
  dim3 grid((p.D + p.CT - 1) / p.CT, p.B);
  kern<<<grid, 256, smem, st>>>(p);
  M2_LAUNCH_CHECK("longconv_simt_kernel");
  return M2_OK;
}

static int next_pow2(int v) { int r = 2; while (r < v) r <<= 1; return r; }

constexpr size_t SIMT_SMEM_MAX = 200 * 1024;

int longconv_simt_launch(const m2_longconv_args* a, cudaStream_t st) {
  ConvParams p;
  p.B = a->batch; p.L = a->seq_len; p.D = a->d_model; p.nf = a->n_filters;
  p.M = next_pow2(a->seq_len); p.lgM = m2_ilog2(p.M);
  const size_t per_ch = (size_t)p.M * sizeof(float2);
  M2_REQUIRE(per_ch <= SIMT_SMEM_MAX, M2_ERR_UNSUPPORTED,
             "m2_longconv_fwd: seq_len %d exceeds the shared-memory FFT family (max 16384)", a->seq_len);
  // channels per CTA: enough for coalesced access in the channel-fastest layout, within
  // 64 KB so that several CTAs stay resident
  int ct = 32;
  while (ct > 1 && ct * per_ch > 64 * 1024) ct >>= 1;
  if (a->xin_sc != 1) ct = (per_ch >= 16 * 1024) ? 1 : ct;
  while (ct > 1 && ct > a->d_model) ct >>= 1;
  p.CT = ct;
  p.xin = a->xin; p.xsb = a->xin_sb; p.xst = a->xin_st; p.xsc = a->xin_sc;
  p.u = a->u; p.usb = a->u_sb; p.ust = a->u_st; p.usc = a->u_sc;
  p.out = a->out; p.osb = a->out_sb; p.ost = a->out_st; p.osc = a->out_sc;
  p.sw = a->short_w; p.sb = a->short_b;
  for (int f = 0; f < 2; ++f) { p.spec[f] = a->spec[f]; p.bias[f] = a->bias[f]; }
  p.plain = a->plain != 0;
  if (p.plain) {   // the input itself is the convolved signal
    p.u = a->xin; p.usb = a->xin_sb; p.ust = a->xin_st; p.usc = a->xin_sc;
    p.spec[1] = a->spec[0]; p.bias[1] = a->bias[0];
  } else if (p.nf == 1) { p.u = a->xin; p.usb = p.ust = p.usc = 0; }
  const size_t smem = (size_t)ct * per_ch;
  const bool round = a->bf16_rounding != 0;
  const bool abf = a->act_dtype == M2_BF16, ubf = (p.nf == 2 && !p.plain) ? (a->u_dtype == M2_BF16) : abf;
  if (abf && ubf) return round ? launch_simt<__nv_bfloat16, __nv_bfloat16, true>(p, smem, st)
                               : launch_simt<__nv_bfloat16, __nv_bfloat16, false>(p, smem, st);
  if (abf && !ubf) return round ? launch_simt<__nv_bfloat16, float, true>(p, smem, st)
                                : launch_simt<__nv_bfloat16, float, false>(p, smem, st);
  if (!abf && !ubf) return round ? launch_simt<float, float, true>(p, smem, st)
                                 : launch_simt<float, float, false>(p, smem, st);
  return m2_set_error(M2_ERR_UNSUPPORTED, "m2_longconv_fwd: float32 activations with a bf16 residual input are not supported");
}

int spectrum_kind0_launch(int D, int L, const float* k, float* spec, cudaStream_t st);

}  // namespace m2
