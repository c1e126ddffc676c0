// Block-diagonal linear layers and the GLU epilogue on CUDA cores with float32
// accumulation (the float32-activation path; bf16 activations use the tensor-core
// kernels), plus the residual-add + LayerNorm that closes the MLP.
//
// Computation replaced: bert/src/mm/blockdiag_multiply.py:49-60,
// bert/src/mm/structured_linear.py:52-70, bert/src/bert_layers.py:492-506.
#include "common.cuh"

namespace m2 {

constexpr int GT = 64;      // output tile edge
constexpr int GK = 16;      // k-chunk
constexpr int GPAD = 4;

// acc[4][4] += A[rows, K] * B[cols, K]^T for a 64x64 tile; A and B row-major with K
// contiguous; rows >= m_valid / cols >= n_valid / k >= k_valid read as zero.
template <typename T>
__device__ __forceinline__ void tile_mma(const T* __restrict__ A, long long lda, int m_valid,
                                         const T* __restrict__ Bm, long long ldb, int n_valid,
                                         int K, int k_valid, float (&acc)[4][4],
                                         float (*sA)[GT + GPAD], float (*sB)[GT + GPAD]) {
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int lr = tid / 4, lk = (tid % 4) * 4;
  for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      float av = 0.f, bv = 0.f;
      if (k < k_valid) {
        if (lr < m_valid) av = ld_as_float(A + (long long)lr * lda + k);
        if (lr < n_valid) bv = ld_as_float(Bm + (long long)lr * ldb + k);
      }
      sA[lk + e][lr] = av;
      sB[lk + e][lr] = bv;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = sA[k][ty * 4 + i]; b[i] = sB[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
}

template <typename T, bool ROUND>
__global__ void __launch_bounds__(256)
blockdiag_simt_kernel(const T* x, long long ldx, const T* w, const float* bias, T* out, long long ldo,
                      int m, int p, int q, int in_features, int out_features) {
  __shared__ float sA[GK][GT + GPAD], sB[GK][GT + GPAD];
  const int kb = blockIdx.z;
  const int row0 = blockIdx.y * GT, col0 = blockIdx.x * GT;
  float acc[4][4] = {};
  int k_valid = in_features - kb * p;
  k_valid = k_valid < 0 ? 0 : (k_valid > p ? p : k_valid);
  tile_mma<T>(x + (long long)row0 * ldx + (long long)kb * p, ldx, m - row0,
              w + ((long long)kb * q + col0) * p, p, q - col0, p, k_valid, acc, sA, sB);
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + ty * 4 + i;
    if (r >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int cq = col0 + tx * 4 + j;
      const int c = kb * q + cq;
      if (cq >= q || c >= out_features) continue;
      float v = rnd<ROUND>(acc[i][j]);
      if (bias) v = rnd<ROUND>(v + rnd<ROUND>(__ldg(bias + c)));
      st_from_float(out + (long long)r * ldo + c, v);
    }
  }
}

template <typename T, bool ROUND>
__global__ void __launch_bounds__(256)
blockdiag_glu_simt_kernel(const T* x, long long ldx, const T* wg, T* h, long long ldh,
                          int m, int p, int q, int half_blocks) {
  __shared__ float sA[GK][GT + GPAD], sB[GK][GT + GPAD];
  const int kb = blockIdx.z;            // gated block; its partner is kb + half_blocks
  const int kn = kb + half_blocks;
  const int row0 = blockIdx.y * GT, col0 = blockIdx.x * GT;
  float accg[4][4] = {}, accn[4][4] = {};
  tile_mma<T>(x + (long long)row0 * ldx + (long long)kb * p, ldx, m - row0,
              wg + ((long long)kb * q + col0) * p, p, q - col0, p, p, accg, sA, sB);
  tile_mma<T>(x + (long long)row0 * ldx + (long long)kn * p, ldx, m - row0,
              wg + ((long long)kn * q + col0) * p, p, q - col0, p, p, accn, sA, sB);
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + ty * 4 + i;
    if (r >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int cq = col0 + tx * 4 + j;
      if (cq >= q) continue;
      const float g = rnd<ROUND>(accg[i][j]), n = rnd<ROUND>(accn[i][j]);
      const float act = rnd<ROUND>(gelu_erf(g));
      st_from_float(h + (long long)r * ldh + (long long)kb * q + cq, rnd<ROUND>(act * n));
    }
  }
}

// out = LayerNorm(a + b); one CTA per row, the summed row cached in shared memory.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
add_layernorm_kernel(const TI* a, long long lda, const TI* b, long long ldb, const float* w,
                     const float* bias, float eps, TO* out, long long ldo, int n) {
  extern __shared__ float row[];
  __shared__ float red[32];
  const int r = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
  const TI* pa = a + (long long)r * lda;
  const TI* pb = b + (long long)r * ldb;
  float sum = 0.f;
  for (int i = tid; i < n; i += nt) {
    float v = ld_as_float(pa + i) + ld_as_float(pb + i);
    if (sizeof(TI) == 2) v = bf16r(v);
    row[i] = v;
    sum += v;
  }
  auto block_sum = [&](float v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    float t = (tid < (nt >> 5)) ? red[tid] : 0.f;
    if (tid < 32) for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (tid == 0) red[0] = t;
    __syncthreads();
    return red[0];
  };
  const float mean = block_sum(sum) / n;
  float sq = 0.f;
  for (int i = tid; i < n; i += nt) { const float d = row[i] - mean; sq += d * d; }
  const float var = block_sum(sq) / n;
  const float rstd = rsqrtf(var + eps);
  TO* po = out + (long long)r * ldo;
  for (int i = tid; i < n; i += nt)
    st_from_float(po + i, (row[i] - mean) * rstd * __ldg(w + i) + __ldg(bias + i));
}

// Vectorised variant: one warp per row, the row held in registers (n a multiple of 256 up to
// 2048, 16-byte aligned rows); optional second output rounded to bf16.
// Row selection for the embeddings' LayerNorm: addend a is row ids_a[r] of a table, addend b row
// ids_b[r] (or r % b_mod) of a second one, and a third float32 addend c (row ids_c[r], or row 0) joins
// as (a + c) + b -- the reference's word + token-type, then + position order.
// rows_a / rows_b / rows_c: row counts of the three tables; an id outside [0, rows) is clamped into the table
// and reported through the device status word (ST_BAD_INDEX) instead of being read out of bounds.
struct LnGather {
  const long long* ids_a; const long long* ids_b; int b_mod;
  const float* c; long long ldc; const long long* ids_c;
  long long rows_a, rows_b, rows_c;
};

constexpr int ST_BAD_INDEX = 16;   // bit of m2_dev_status_word: an embedding id was outside its table

__device__ __forceinline__ long long clamp_row(long long id, long long rows, bool& bad) {
  if (id < 0) { bad = true; return 0; }
  if (id >= rows) { bad = true; return rows - 1; }
  return id;
}

template <typename TI, typename TO, int VI>
__global__ void __launch_bounds__(512)
add_layernorm_warp_kernel(const TI* a, long long lda, const TI* b, long long ldb, const LnGather gt,
                          const float* __restrict__ w, const float* __restrict__ bias, float eps, TO* out,
                          long long ldo, __nv_bfloat16* out2, long long ld2, int m,
                          __half* out_tm, long long tm_sb, long long tm_sc, int seq_len, int rpw, int pad2) {
  extern __shared__ __half ln_tile[];   // [rows of the block][n] fp16, only with out_tm
  const int wib = threadIdx.x >> 5, nw = blockDim.x >> 5, lane = threadIdx.x & 31;
  constexpr int n = VI * 256;
  // a warp normalises rpw rows (rpw > 1 only with out_tm, where m is a multiple of the block's rows)
  for (int ri = 0; ri < rpw; ++ri) {
  const int trow = ri * nw + wib;                                   // row within the block
  const long long warp = (long long)blockIdx.x * nw * rpw + trow;   // row of the tensor
  if (warp >= m) break;
  float v[VI][8];
  float sum = 0.f;
  if constexpr (sizeof(TI) == 2) {
    const uint4* pa = reinterpret_cast<const uint4*>(a + (long long)warp * lda);
    const uint4* pb = b ? reinterpret_cast<const uint4*>(b + (long long)warp * ldb) : nullptr;
#pragma unroll
    for (int i = 0; i < VI; ++i) {
      const uint4 xa = __ldg(pa + i * 32 + lane), xb = pb ? __ldg(pb + i * 32 + lane) : make_uint4(0, 0, 0, 0);
      const uint32_t wa[4] = {xa.x, xa.y, xa.z, xa.w}, wb[4] = {xb.x, xb.y, xb.z, xb.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // bf16 + bf16 -> bf16 (the residual add of two bf16 tensors), then float32 statistics
        v[i][2 * j] = bf16r(__uint_as_float(wa[j] << 16) + __uint_as_float(wb[j] << 16));
        v[i][2 * j + 1] = bf16r(__uint_as_float(wa[j] & 0xffff0000u) + __uint_as_float(wb[j] & 0xffff0000u));
        sum += v[i][2 * j] + v[i][2 * j + 1];
      }
    }
  } else {
    bool bad = false;
    const long long ra = gt.ids_a ? clamp_row(gt.ids_a[warp], gt.rows_a, bad) : warp;
    const long long rb = gt.ids_b ? clamp_row(gt.ids_b[warp], gt.rows_b, bad) : (gt.b_mod > 0 ? warp % gt.b_mod : warp);
    const long long rc = gt.ids_c ? clamp_row(gt.ids_c[warp], gt.rows_c, bad) : 0;
    if (bad && lane == 0) atomicOr(&m2_dev_status_word, ST_BAD_INDEX);
    const float4* pa = reinterpret_cast<const float4*>(a + ra * lda);
    const float4* pb = b ? reinterpret_cast<const float4*>(b + rb * ldb) : nullptr;
    const float4* pc = gt.c ? reinterpret_cast<const float4*>(gt.c + rc * gt.ldc) : nullptr;
#pragma unroll
    for (int i = 0; i < VI; ++i) {
      const int q = (i * 32 + lane) * 2;
      const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
      float4 a0 = __ldg(pa + q), a1 = __ldg(pa + q + 1);
      if (pc) {
        const float4 c0 = __ldg(pc + q), c1 = __ldg(pc + q + 1);
        a0 = make_float4(a0.x + c0.x, a0.y + c0.y, a0.z + c0.z, a0.w + c0.w);
        a1 = make_float4(a1.x + c1.x, a1.y + c1.y, a1.z + c1.z, a1.w + c1.w);
      }
      const float4 b0 = pb ? __ldg(pb + q) : z, b1 = pb ? __ldg(pb + q + 1) : z;
      const float s8[8] = {a0.x + b0.x, a0.y + b0.y, a0.z + b0.z, a0.w + b0.w, a1.x + b1.x, a1.y + b1.y, a1.z + b1.z, a1.w + b1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) { v[i][j] = s8[j]; sum += s8[j]; }
    }
  }
  if (out2 && lane * 8 < pad2)      // columns n .. n + pad2 of the bf16 copy: [1, 0, 0, ...]
    *reinterpret_cast<uint4*>(out2 + (long long)warp * ld2 + n + lane * 8) = make_uint4(lane == 0 ? 0x3F80u : 0u, 0u, 0u, 0u);
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float mean = sum / n;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < VI; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) { const float d = v[i][j] - mean; sq += d * d; }
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  const float rstd = rsqrtf(sq / n + eps);
#pragma unroll
  for (int i = 0; i < VI; ++i) {
    const int c0 = (i * 32 + lane) * 8;
    const float4 w0 = __ldg(reinterpret_cast<const float4*>(w + c0)), w1 = __ldg(reinterpret_cast<const float4*>(w + c0 + 4));
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(bias + c0)), b1 = __ldg(reinterpret_cast<const float4*>(bias + c0 + 4));
    const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    float y[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = (v[i][j] - mean) * rstd * ww[j] + bb[j];
    uint32_t pk[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 h = __floats2bfloat162_rn(y[2 * j], y[2 * j + 1]);
      pk[j] = *reinterpret_cast<uint32_t*>(&h);
    }
    if (out == nullptr) {
      // only the copies are wanted
    } else if (sizeof(TO) == 4) {
      float4* po = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + (long long)warp * ldo + c0);
      po[0] = make_float4(y[0], y[1], y[2], y[3]);
      po[1] = make_float4(y[4], y[5], y[6], y[7]);
    } else {
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out) + (long long)warp * ldo + c0) =
          make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
    if (out2) *reinterpret_cast<uint4*>(out2 + (long long)warp * ld2 + c0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    if (out_tm) {
      uint32_t hk[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __half2 h = __floats2half2_rn(fminf(fmaxf(y[2 * j], -65504.f), 65504.f), fminf(fmaxf(y[2 * j + 1], -65504.f), 65504.f));
        hk[j] = *reinterpret_cast<uint32_t*>(&h);
      }
      *reinterpret_cast<uint4*>(ln_tile + (size_t)trow * n + c0) = make_uint4(hk[0], hk[1], hk[2], hk[3]);
    }
  }
  }
  if (out_tm) {
    // rows of the block are consecutive time steps of one sequence: write each channel's run
    // of them (16 to 128 contiguous bytes) into the time-major copy, two channels per thread
    __syncthreads();
    const int rows = nw * rpw;
    const long long row0 = (long long)blockIdx.x * rows;
    __half* dst = out_tm + (row0 / seq_len) * tm_sb + (row0 % seq_len);
    const uint32_t* tile32 = reinterpret_cast<const uint32_t*>(ln_tile);
    const bool wide = (rows % 16 == 0) && ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) && (tm_sc % 16 == 0);
    for (int cp = threadIdx.x; cp < n / 2; cp += blockDim.x) {
      __half* d0 = dst + (long long)(2 * cp) * tm_sc;
      __half* d1 = d0 + tm_sc;
      for (int r0 = 0; r0 < rows; r0 += 16) {
        uint32_t lo[8], hi[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (r0 + 2 * j < rows) {
            const uint32_t w0 = tile32[(size_t)(r0 + 2 * j) * (n / 2) + cp], w1 = tile32[(size_t)(r0 + 2 * j + 1) * (n / 2) + cp];
            lo[j] = __byte_perm(w0, w1, 0x5410);                    // channel 2 cp at rows r, r + 1
            hi[j] = __byte_perm(w0, w1, 0x7632);                    // channel 2 cp + 1
          }
        }
        if (wide) {                                                 // whole 32-byte sectors
          stg256(d0 + r0, lo[0], lo[1], lo[2], lo[3], lo[4], lo[5], lo[6], lo[7]);
          stg256(d1 + r0, hi[0], hi[1], hi[2], hi[3], hi[4], hi[5], hi[6], hi[7]);
        } else {
          *reinterpret_cast<uint4*>(d0 + r0) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
          *reinterpret_cast<uint4*>(d1 + r0) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
          if (r0 + 8 < rows) {
            *reinterpret_cast<uint4*>(d0 + r0 + 8) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
            *reinterpret_cast<uint4*>(d1 + r0 + 8) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
          }
        }
      }
    }
  }
}

int blockdiag_tc_launch(const m2_blockdiag_args* a, cudaStream_t st);   // gemm_tc.cu
int glu_tc_launch(const m2_glu_args* a, cudaStream_t st);
bool blockdiag_tc_supported(const m2_blockdiag_args* a);
bool glu_tc_supported(const m2_glu_args* a);
bool glu_pair_supported(const m2_glu_args* a);                            // glu_pair.cu
int glu_pair_launch(const m2_glu_args* a, cudaStream_t st);
bool blockdiag_pair_supported(const m2_blockdiag_args* a);               // linear_tc.cu
int blockdiag_pair_launch(const m2_blockdiag_args* a, cudaStream_t st);

}  // namespace m2

extern "C" int m2_blockdiag_fwd(const m2_blockdiag_args* a, void* stream) {
  using namespace m2;
  M2_REQUIRE(a != nullptr, M2_ERR_ARG, "m2_blockdiag_fwd: args is NULL");
  M2_REQUIRE(a->m >= 0 && a->nblocks > 0 && a->p > 0 && a->q > 0, M2_ERR_ARG,
             "m2_blockdiag_fwd: bad sizes m=%d nblocks=%d p=%d q=%d", a->m, a->nblocks, a->p, a->q);
  M2_REQUIRE(a->in_features > 0 && a->in_features <= a->nblocks * a->p && a->out_features > 0 &&
             a->out_features <= a->nblocks * a->q, M2_ERR_ARG,
             "m2_blockdiag_fwd: in_features=%d / out_features=%d do not fit %d blocks of (%d -> %d)",
             a->in_features, a->out_features, a->nblocks, a->p, a->q);
  if (a->m == 0) return M2_OK;
  M2_REQUIRE(a->x && a->w && a->out, M2_ERR_ARG, "m2_blockdiag_fwd: NULL tensor pointer");
  M2_REQUIRE(a->ldx >= a->in_features && a->ldo >= a->out_features, M2_ERR_ARG,
             "m2_blockdiag_fwd: row stride smaller than the row");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The MLP's block-diagonal GEMMs stream a wide activation once (wo: K = intermediate size) and are bound by
  // that read, not by operand re-use: the single-CTA kernel with its finer units (128-row tiles) is the faster
  // one there (52 vs 62 us at M = 32768, 3072 -> 768), so CTA-pair tiles run only on request or for shapes the
  // single-CTA kernel does not take (block widths that are not multiples of 64).
  if (a->variant == 2 && blockdiag_pair_supported(a)) return blockdiag_pair_launch(a, st);
  if (blockdiag_tc_supported(a)) return blockdiag_tc_launch(a, st);
  if (blockdiag_pair_supported(a)) return blockdiag_pair_launch(a, st);
  dim3 grid((a->q + GT - 1) / GT, (a->m + GT - 1) / GT, a->nblocks);
  M2_REQUIRE(grid.y <= 65535 && grid.z <= 65535, M2_ERR_UNSUPPORTED, "m2_blockdiag_fwd: too many row tiles");
  if (a->dtype == M2_BF16)
    blockdiag_simt_kernel<__nv_bfloat16, true><<<grid, 256, 0, st>>>(
        (const __nv_bfloat16*)a->x, a->ldx, (const __nv_bfloat16*)a->w, a->bias, (__nv_bfloat16*)a->out,
        a->ldo, a->m, a->p, a->q, a->in_features, a->out_features);
  else
    blockdiag_simt_kernel<float, false><<<grid, 256, 0, st>>>(
        (const float*)a->x, a->ldx, (const float*)a->w, a->bias, (float*)a->out, a->ldo, a->m, a->p,
        a->q, a->in_features, a->out_features);
  M2_LAUNCH_CHECK("blockdiag_simt_kernel");
  return M2_OK;
}

extern "C" int m2_blockdiag_glu_fwd(const m2_glu_args* a, void* stream) {
  using namespace m2;
  M2_REQUIRE(a != nullptr, M2_ERR_ARG, "m2_blockdiag_glu_fwd: args is NULL");
  M2_REQUIRE(a->m >= 0 && a->d_model > 0 && a->inter > 0 && a->nblocks > 0, M2_ERR_ARG,
             "m2_blockdiag_glu_fwd: bad sizes");
  M2_REQUIRE(a->nblocks % 2 == 0, M2_ERR_UNSUPPORTED, "m2_blockdiag_glu_fwd: nblocks must be even");
  M2_REQUIRE(a->d_model % a->nblocks == 0 && (2 * a->inter) % a->nblocks == 0, M2_ERR_UNSUPPORTED,
             "m2_blockdiag_glu_fwd: d_model and 2*inter must be multiples of nblocks");
  if (a->m == 0) return M2_OK;
  M2_REQUIRE(a->x && a->wg && a->h, M2_ERR_ARG, "m2_blockdiag_glu_fwd: NULL tensor pointer");
  M2_REQUIRE(a->ldx >= a->d_model && a->ldh >= a->inter, M2_ERR_ARG,
             "m2_blockdiag_glu_fwd: row stride smaller than the row");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // CTA pairs halve the wg traffic per tile but the GLU GEMM is paced by its GELU epilogue (K is only d_model /
  // nblocks): measured 108.7 us against 100.4 us for the single-CTA kernel with resident x slices at M = 32768,
  // so pairs run on request only
  if (a->variant == 3 && glu_pair_supported(a)) return glu_pair_launch(a, st);
  if (glu_tc_supported(a)) return glu_tc_launch(a, st);
  const int p = a->d_model / a->nblocks, q = 2 * a->inter / a->nblocks;
  dim3 grid((q + GT - 1) / GT, (a->m + GT - 1) / GT, a->nblocks / 2);
  M2_REQUIRE(grid.y <= 65535, M2_ERR_UNSUPPORTED, "m2_blockdiag_glu_fwd: too many row tiles");
  if (a->dtype == M2_BF16)
    blockdiag_glu_simt_kernel<__nv_bfloat16, true><<<grid, 256, 0, st>>>(
        (const __nv_bfloat16*)a->x, a->ldx, (const __nv_bfloat16*)a->wg, (__nv_bfloat16*)a->h, a->ldh,
        a->m, p, q, a->nblocks / 2);
  else
    blockdiag_glu_simt_kernel<float, false><<<grid, 256, 0, st>>>(
        (const float*)a->x, a->ldx, (const float*)a->wg, (float*)a->h, a->ldh, a->m, p, q, a->nblocks / 2);
  M2_LAUNCH_CHECK("blockdiag_glu_simt_kernel");
  return M2_OK;
}

static int add_layernorm_core(const m2_add_layernorm_args* a, const m2::LnGather& gather, void* stream);

extern "C" int m2_add_layernorm_fwd(const m2_add_layernorm_args* a, void* stream) {
  const m2::LnGather none = {nullptr, nullptr, 0, nullptr, 0, nullptr, 0, 0, 0};
  return add_layernorm_core(a, none, stream);
}

extern "C" int m2_embed_layernorm_fwd(const m2_embed_layernorm_args* e, void* stream) {
  M2_REQUIRE(e != nullptr, M2_ERR_ARG, "m2_embed_layernorm_fwd: args is NULL");
  M2_REQUIRE(e->m >= 0 && e->n > 0, M2_ERR_ARG, "m2_embed_layernorm_fwd: bad sizes");
  if (e->m == 0) return M2_OK;
  M2_REQUIRE(e->word_table && e->input_ids && e->type_table && e->weight && e->bias, M2_ERR_ARG,
             "m2_embed_layernorm_fwd: NULL pointer");
  M2_REQUIRE(!e->pos_table || e->position_ids || e->seq_len > 0, M2_ERR_ARG,
             "m2_embed_layernorm_fwd: position table without position_ids needs seq_len");
  M2_REQUIRE(e->vocab_rows > 0 && e->type_rows > 0 && (!e->pos_table || e->pos_rows > 0), M2_ERR_ARG,
             "m2_embed_layernorm_fwd: table row counts must be positive");
  M2_REQUIRE(!e->pos_table || e->position_ids || e->seq_len <= e->pos_rows, M2_ERR_ARG,
             "m2_embed_layernorm_fwd: seq_len %d exceeds the position table's %lld rows", e->seq_len, e->pos_rows);
  M2_REQUIRE(e->n % 256 == 0 && e->n <= 2048 && m2_aligned(e->word_table, 16) && m2_aligned(e->type_table, 16) &&
             m2_aligned(e->pos_table, 16), M2_ERR_UNSUPPORTED,
             "m2_embed_layernorm_fwd: needs hidden size a multiple of 256 up to 2048 and 16-byte aligned tables");
  m2_add_layernorm_args a;
  memset(&a, 0, sizeof(a));
  a.m = e->m; a.n = e->n; a.in_dtype = M2_F32; a.out_dtype = M2_F32;
  a.a = e->word_table; a.lda = e->n; a.b = e->pos_table; a.ldb = e->n;
  a.weight = e->weight; a.bias = e->bias; a.eps = e->eps;
  a.out = e->out; a.ldo = e->ldo; a.out_bf16 = e->out_bf16; a.ld_bf16 = e->ld_bf16; a.bf16_pad_cols = e->bf16_pad_cols;
  a.out_tm_f16 = e->out_tm_f16; a.tm_sb = e->tm_sb; a.tm_sc = e->tm_sc; a.seq_len = e->seq_len;
  const m2::LnGather g = {e->input_ids, e->pos_table ? e->position_ids : nullptr, e->pos_table && !e->position_ids ? e->seq_len : 0,
                          e->type_table, e->n, e->token_type_ids, e->vocab_rows, e->pos_rows, e->type_rows};
  return add_layernorm_core(&a, g, stream);
}

static int add_layernorm_core(const m2_add_layernorm_args* a, const m2::LnGather& gather, void* stream) {
  using namespace m2;
  M2_REQUIRE(a != nullptr, M2_ERR_ARG, "m2_add_layernorm_fwd: args is NULL");
  M2_REQUIRE(a->m >= 0 && a->n > 0, M2_ERR_ARG, "m2_add_layernorm_fwd: bad sizes m=%d n=%d", a->m, a->n);
  M2_REQUIRE(a->n <= 12288, M2_ERR_UNSUPPORTED, "m2_add_layernorm_fwd: n > 12288");
  if (a->m == 0) return M2_OK;
  M2_REQUIRE(a->a && a->weight && a->bias && (a->out || a->out_bf16), M2_ERR_ARG,
             "m2_add_layernorm_fwd: NULL tensor pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  M2_REQUIRE(a->out_bf16 == nullptr || a->ld_bf16 >= a->n, M2_ERR_ARG, "m2_add_layernorm_fwd: ld_bf16 smaller than the row");
  M2_REQUIRE(a->bf16_pad_cols >= 0 && a->bf16_pad_cols % 8 == 0 && a->bf16_pad_cols <= 256 &&
             (a->bf16_pad_cols == 0 || (a->out_bf16 && a->ld_bf16 >= a->n + a->bf16_pad_cols)), M2_ERR_ARG,
             "m2_add_layernorm_fwd: bf16_pad_cols must be a multiple of 8 (<= 256) that fits the rows of out_bf16");
  const int epv = a->in_dtype == M2_BF16 ? 8 : 4;        // elements per 16 bytes of input
  const bool vec = (a->in_dtype == M2_BF16 || (a->in_dtype == M2_F32 && a->out_dtype == M2_F32)) &&
                   a->n % 256 == 0 && a->n <= 2048 && a->lda % epv == 0 && (!a->b || a->ldb % epv == 0) &&
                   m2_aligned(a->a, 16) && m2_aligned(a->b, 16) && m2_aligned(a->out, 16) && a->ldo % 8 == 0 &&
                   m2_aligned(a->weight, 16) && m2_aligned(a->bias, 16) &&
                   (a->out_bf16 == nullptr || (m2_aligned(a->out_bf16, 16) && a->ld_bf16 % 8 == 0));
  if (a->out_tm_f16) {
    M2_REQUIRE(vec, M2_ERR_UNSUPPORTED,
               "m2_add_layernorm_fwd: the time-major copy needs n a multiple of 256 (<= 2048), 16-byte aligned rows and bf16 inputs (or float32 inputs with a float32 output)");
    M2_REQUIRE(a->seq_len > 0 && a->seq_len % 8 == 0 && a->m % a->seq_len == 0, M2_ERR_ARG,
               "m2_add_layernorm_fwd: the time-major copy needs m = batch * seq_len rows with seq_len a multiple of 8");
    M2_REQUIRE(m2_aligned(a->out_tm_f16, 16) && a->tm_sb % 8 == 0 && a->tm_sc % 8 == 0, M2_ERR_ALIGN,
               "m2_add_layernorm_fwd: the time-major copy needs 16-byte aligned rows");
  }
  if (vec) {
    // with the time-major copy a block covers 16 (or 8) consecutive steps of one sequence, so a
    // channel's run of them is one 32-byte sector
    int rows = 8, threads = 256, rpw = 1;
    if (a->out_tm_f16) {
      rows = a->seq_len % 32 == 0 && a->n <= 768 ? 32 : a->seq_len % 16 == 0 ? 16 : 8;   // 32 rows: 64-byte runs per channel
      threads = rows >= 16 ? 512 : 256;
      rpw = rows / (threads / 32);
    }
    const int blocks = (a->m + rows - 1) / rows;
    const size_t tile = a->out_tm_f16 ? (size_t)rows * a->n * 2 : 0;
#define M2_LNW(TO, VI) do { if (a->in_dtype == M2_F32) M2_LNW2(float, float, VI); else M2_LNW2(__nv_bfloat16, TO, VI); } while (0)
#define M2_LNW2(TI, TO, VI) do { \
      if (tile > 48 * 1024) M2_CUDA(cudaFuncSetAttribute(add_layernorm_warp_kernel<TI, TO, VI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile)); \
      add_layernorm_warp_kernel<TI, TO, VI><<<blocks, threads, tile, st>>>( \
      (const TI*)a->a, a->lda, (const TI*)a->b, a->ldb, gather, a->weight, a->bias, a->eps, \
      (TO*)a->out, a->ldo, (__nv_bfloat16*)a->out_bf16, a->ld_bf16, a->m, \
      (__half*)a->out_tm_f16, a->tm_sb, a->tm_sc, a->seq_len, rpw, a->bf16_pad_cols); } while (0)
#define M2_LNW_VI(TO) switch (a->n / 256) { case 1: M2_LNW(TO, 1); break; case 2: M2_LNW(TO, 2); break; \
      case 3: M2_LNW(TO, 3); break; case 4: M2_LNW(TO, 4); break; case 5: M2_LNW(TO, 5); break; \
      case 6: M2_LNW(TO, 6); break; case 7: M2_LNW(TO, 7); break; default: M2_LNW(TO, 8); break; }
    if (a->out_dtype == M2_F32) { M2_LNW_VI(float) } else { M2_LNW_VI(__nv_bfloat16) }
#undef M2_LNW_VI
#undef M2_LNW
#undef M2_LNW2
    M2_LAUNCH_CHECK("add_layernorm_warp_kernel");
    return M2_OK;
  }
  M2_REQUIRE(!gather.ids_a && !gather.c, M2_ERR_UNSUPPORTED, "m2_embed_layernorm_fwd: shape not covered by the vectorised kernel");
  M2_REQUIRE(a->out != nullptr && a->out_bf16 == nullptr && a->out_tm_f16 == nullptr, M2_ERR_UNSUPPORTED,
             "m2_add_layernorm_fwd: the copies need n a multiple of 256 (<= 2048) and 16-byte aligned rows");
  M2_REQUIRE(a->b != nullptr, M2_ERR_UNSUPPORTED, "m2_add_layernorm_fwd: b = NULL needs n a multiple of 256 (<= 2048) and 16-byte aligned rows");
  const size_t smem = (size_t)a->n * sizeof(float);
  const int threads = a->n >= 1024 ? 256 : 128;
#define M2_LN(TI, TO) add_layernorm_kernel<TI, TO><<<a->m, threads, smem, st>>>( \
      (const TI*)a->a, a->lda, (const TI*)a->b, a->ldb, a->weight, a->bias, a->eps, (TO*)a->out, a->ldo, a->n)
  if (a->in_dtype == M2_BF16 && a->out_dtype == M2_F32) M2_LN(__nv_bfloat16, float);
  else if (a->in_dtype == M2_BF16 && a->out_dtype == M2_BF16) M2_LN(__nv_bfloat16, __nv_bfloat16);
  else if (a->in_dtype == M2_F32 && a->out_dtype == M2_F32) M2_LN(float, float);
  else return m2_set_error(M2_ERR_UNSUPPORTED, "m2_add_layernorm_fwd: unsupported dtype combination");
#undef M2_LN
  M2_LAUNCH_CHECK("add_layernorm_kernel");
  return M2_OK;
}
