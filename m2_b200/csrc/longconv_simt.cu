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
#include <cooperative_groups.h>

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


// packed input point n of channel c for filter pass f: (a[2n], a[2n+1]) with a = the gated
// short-conv product (f == 0) or the raw residual input (f == 1)
template <typename TA, typename TU, bool ROUND>
__device__ __forceinline__ float2 load_point(const ConvParams& p, int f, const TA* xb, const TU* ub, int c, int n) {
  float2 zv = make_float2(0.f, 0.f);
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int t = 2 * n + e;
    float a = 0.f;
    if (t < p.L) {
      if (f == 0) {
        const float x1 = short_conv_at<TA, ROUND>(xb, p.xst, p.xsc, c, t, p.sw, p.sb);
        const float v = short_conv_at<TA, ROUND>(xb, p.xst, p.xsc, 2 * p.D + c, t, p.sw, p.sb);
        a = rnd<ROUND>(v * x1);
      } else {
        a = ld_as_float(ub + (long long)t * p.ust + (long long)c * p.usc);
      }
    }
    if (e == 0) zv.x = a; else zv.y = a;
  }
  return zv;
}

// bias, gates and residual add for the packed output point n of channel c; writes out[t]
template <typename TA, typename TU, bool ROUND>
__device__ __forceinline__ void store_point(const ConvParams& p, int f, const TA* xb, const TU* ub, TA* ob, int c, int n,
                                            float2 zy, float bc) {
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int t = 2 * n + e;
    if (t >= p.L) continue;
    const float y = (e == 0) ? zy.x : zy.y;
    TA* po = ob + (long long)t * p.ost + (long long)c * p.osc;
    if (f == 0) {
      const float x1 = short_conv_at<TA, ROUND>(xb, p.xst, p.xsc, c, t, p.sw, p.sb);
      const float v = short_conv_at<TA, ROUND>(xb, p.xst, p.xsc, 2 * p.D + c, t, p.sw, p.sb);
      const float x2 = short_conv_at<TA, ROUND>(xb, p.xst, p.xsc, p.D + c, t, p.sw, p.sb);
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

// Zy[k] = alpha Z[k] + beta conj(Z[M-k]) for the bin pair stored at positions pk, pm of s
__device__ __forceinline__ void filter_pair(float2* s, int lk, int lm, const float2* al, const float2* be, int pk, int pm) {
  const float2 Zk = s[lk], Zm = s[lm];
  const float2 a1 = __ldg(al + pk), b1 = __ldg(be + pk);
  float2 r1 = cmul(a1, Zk);
  const float2 t1 = cmul_conj(b1, Zm);
  r1.x += t1.x; r1.y += t1.y;
  if (pm != pk) {
    const float2 a2 = __ldg(al + pm), b2 = __ldg(be + pm);
    float2 r2 = cmul(a2, Zm);
    const float2 t2 = cmul_conj(b2, Zk);
    r2.x += t2.x; r2.y += t2.y;
    s[lm] = r2;
  }
  s[lk] = r1;
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
      if (n < npair && c < D) zv = load_point<TA, TU, ROUND>(p, f, xb, ub, c, n);
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
      filter_pair(s + ci * M, pk, pm, al, al + M, pk, pm);
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
      store_point<TA, TU, ROUND>(p, f, xb, ub, ob, c, n, s[ci * M + n], __ldg(biasv + c));
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


// ---------------------------------------------------------------------------------------
// Rows too long for one CTA's shared memory (L = 32768: 256 KB of packed float32 spectrum):
// a cluster of two CTAs holds one channel row, each CTA one half of the M packed points.
// The input lives entirely in the first half (the second is the zero padding), so the
// first decimation-in-frequency stage needs no exchange: CTA 0 keeps z, CTA 1 starts from
// z * W^n.  All later forward stages, the filter multiply (bins k and M-k have the same
// parity, hence the same CTA) and all but the last inverse stage are local.  The last
// inverse stage reads the partner's half through distributed shared memory, and only for
// the first M/2 outputs -- the ones that are kept.
// ---------------------------------------------------------------------------------------
template <typename TA, typename TU, bool ROUND>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(512)
longconv_simt_cluster2_kernel(ConvParams p) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float2* s = reinterpret_cast<float2*>(smem_raw);   // [M/2]
  const int M = p.M, Mh = M >> 1, L = p.L;
  const int tid = threadIdx.x, nt = blockDim.x;
  const int q = (int)cluster.block_rank();
  const int c = blockIdx.x >> 1;
  const int b = blockIdx.y;
  const TA* xb = reinterpret_cast<const TA*>(p.xin) + (long long)b * p.xsb;
  const TU* ub = reinterpret_cast<const TU*>(p.u) + (long long)b * p.usb;
  TA* ob = reinterpret_cast<TA*>(p.out) + (long long)b * p.osb;
  const int npair = (L + 1) >> 1;                     // <= Mh
  const float2* s0 = cluster.map_shared_rank(s, 0);
  const float2* s1 = cluster.map_shared_rank(s, 1);

  const int f_begin = p.plain ? 1 : 0, f_end = p.plain ? 2 : p.nf;
  for (int f = f_begin; f < f_end; ++f) {
    const float2* tw = reinterpret_cast<const float2*>(p.spec[f]);
    const float2* al = reinterpret_cast<const float2*>(p.spec[f] + M) + (size_t)c * 2 * M;
    const float2* be = al + M;

    // input + first forward stage
    for (int n = tid; n < Mh; n += nt) {
      float2 zv = make_float2(0.f, 0.f);
      if (n < npair) zv = load_point<TA, TU, ROUND>(p, f, xb, ub, c, n);
      s[n] = (q == 0) ? zv : cmul(zv, __ldg(tw + n));
    }
    __syncthreads();
    // remaining forward stages: an (M/2)-point decimation-in-frequency FFT of the local half
    for (int h = Mh >> 1; h >= 1; h >>= 1) {
      const int tstep = Mh / h;
      for (int j = tid; j < (Mh >> 1); j += nt) {
        const int g = j / h, pos = j % h;
        float2* base = s + g * 2 * h + pos;
        const float2 a = base[0], bb = base[h];
        const float2 w = __ldg(tw + pos * tstep);
        base[0] = make_float2(a.x + bb.x, a.y + bb.y);
        base[h] = cmul(make_float2(a.x - bb.x, a.y - bb.y), w);
      }
      __syncthreads();
    }
    // filter multiply on the local bins (global position = q * Mh + local position)
    for (int lp = tid; lp < Mh; lp += nt) {
      const int pk = q * Mh + lp;
      const int k = (int)(__brev((unsigned)pk) >> (32 - p.lgM));
      const int km = (M - k) & (M - 1);
      const int pm = (int)(__brev((unsigned)km) >> (32 - p.lgM));
      if (pm < pk) continue;                           // the pair is handled from its lower position
      filter_pair(s, lp, pm - q * Mh, al, be, pk, pm);
    }
    __syncthreads();
    // local inverse stages
    for (int h = 1; h <= (Mh >> 1); h <<= 1) {
      const int tstep = Mh / h;
      for (int j = tid; j < (Mh >> 1); j += nt) {
        const int g = j / h, pos = j % h;
        float2* base = s + g * 2 * h + pos;
        const float2 w = __ldg(tw + pos * tstep);
        const float2 a = base[0];
        const float2 bb = cmul_conj(base[h], w);
        base[0] = make_float2(a.x + bb.x, a.y + bb.y);
        base[h] = make_float2(a.x - bb.x, a.y - bb.y);
      }
      __syncthreads();
    }
    cluster.sync();
    // last inverse stage (kept outputs only) fused with the epilogue; each CTA takes half of them
    const float bc = __ldg(p.bias[f] + c);
    for (int n = q * (Mh >> 1) + tid; n < (q + 1) * (Mh >> 1) && n < npair; n += nt) {
      const float2 a = s0[n];
      const float2 bb = cmul_conj(s1[n], __ldg(tw + n));
      store_point<TA, TU, ROUND>(p, f, xb, ub, ob, c, n, make_float2(a.x + bb.x, a.y + bb.y), bc);
    }
    cluster.sync();                                    // both halves are free for the next pass
  }
}

template <typename TA, typename TU, bool ROUND>
static int launch_cluster2(const ConvParams& p, size_t smem, cudaStream_t st) {
  auto kern = longconv_simt_cluster2_kernel<TA, TU, ROUND>;
  M2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(2 * p.D, p.B);
  kern<<<grid, 512, smem, st>>>(p);
  M2_LAUNCH_CHECK("longconv_simt_cluster2_kernel");
  return M2_OK;
}

static int next_pow2(int v) { int r = 2; while (r < v) r <<= 1; return r; }

constexpr size_t SIMT_SMEM_MAX = 200 * 1024;

int longconv_simt_launch(const m2_longconv_args* a, cudaStream_t st) {
  ConvParams p;
  p.B = a->batch; p.L = a->seq_len; p.D = a->d_model; p.nf = a->n_filters;
  p.M = next_pow2(a->seq_len); p.lgM = m2_ilog2(p.M);
  const size_t per_ch = (size_t)p.M * sizeof(float2);
  const bool use_cluster = per_ch > SIMT_SMEM_MAX;
  M2_REQUIRE(per_ch <= 2 * SIMT_SMEM_MAX, M2_ERR_UNSUPPORTED,
             "m2_longconv_fwd: seq_len %d exceeds the shared-memory FFT family (max 32768)", a->seq_len);
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
  const size_t smem = use_cluster ? per_ch / 2 : (size_t)ct * per_ch;
  const bool round = a->bf16_rounding != 0;
  const bool abf = a->act_dtype == M2_BF16, ubf = (p.nf == 2 && !p.plain) ? (a->u_dtype == M2_BF16) : abf;
  if (use_cluster) {
    M2_REQUIRE(2LL * p.D <= 2147483647LL, M2_ERR_UNSUPPORTED, "m2_longconv_fwd: d_model too large");
    if (abf && ubf) return round ? launch_cluster2<__nv_bfloat16, __nv_bfloat16, true>(p, smem, st)
                                 : launch_cluster2<__nv_bfloat16, __nv_bfloat16, false>(p, smem, st);
    if (abf && !ubf) return round ? launch_cluster2<__nv_bfloat16, float, true>(p, smem, st)
                                  : launch_cluster2<__nv_bfloat16, float, false>(p, smem, st);
    if (!abf && !ubf) return round ? launch_cluster2<float, float, true>(p, smem, st)
                                   : launch_cluster2<float, float, false>(p, smem, st);
    return m2_set_error(M2_ERR_UNSUPPORTED, "m2_longconv_fwd: float32 activations with a bf16 residual input are not supported");
  }
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
