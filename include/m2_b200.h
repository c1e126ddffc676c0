/*
 * m2_b200 -- C ABI of the B200 (sm_100a) kernels behind the M2-BERT sequence mixer and
 * BlockdiagLinear GLU MLP forward path.
 *
 * Conventions
 *   - plain C: pointers, sizes and strides only; no framework types.
 *   - every pointer marked "device" is caller-owned device memory of the CURRENT device;
 *     the library never allocates or frees device memory in these calls.
 *   - calls are asynchronous on `stream` (a cudaStream_t passed as void*).
 *   - return value: M2_OK or an m2_status error; m2_last_error() gives a thread-local
 *     human-readable message.  Nothing aborts, nothing throws.
 *   - strides are in ELEMENTS of the tensor's dtype.
 *
 * The reference (HazyResearch/m2) has no C interface on this path: its default route is
 * PyTorch ops and its optional native route is a pybind11 module taking torch::Tensor
 * (csrc/flashmm/flash_mm.cpp:364-368).  Each entry point below cites the reference code
 * whose computation it replaces.
 */
#ifndef M2_B200_H
#define M2_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define M2_B200_ABI_VERSION 2

typedef enum { M2_F32 = 0, M2_BF16 = 1, M2_F16 = 2 /* only where an entry point says so */ } m2_dtype;

typedef enum {
  M2_OK = 0,
  M2_ERR_ARG = 1,          /* NULL pointer, non-positive size, inconsistent shapes */
  M2_ERR_UNSUPPORTED = 2,  /* shape or dtype outside what the kernels cover */
  M2_ERR_ALIGN = 3,        /* pointer or stride not aligned as documented */
  M2_ERR_CUDA = 4,         /* a CUDA runtime call or launch failed */
  M2_ERR_DEVICE = 5        /* a kernel gave up on a bounded wait (see m2_device_status) */
} m2_status;

/* Bits of the device status word read by m2_device_status(). */
#define M2_DEV_TIMEOUT_TMA   1   /* a wait for a TMA load ran out */
#define M2_DEV_TIMEOUT_MMA   2   /* a wait for tensor-core work or a free accumulator ran out */
#define M2_DEV_TIMEOUT_EPI   4   /* an epilogue's wait for an accumulator ran out */
#define M2_DEV_TIMEOUT_EMPTY 8   /* a producer's wait for a free shared-memory stage ran out */
#define M2_DEV_BAD_INDEX     16  /* m2_embed_layernorm_fwd met an id outside its table (clamped) */

/* ABI version of the loaded library (== M2_B200_ABI_VERSION it was built with). */
int m2_version(void);

/* Message of the last error returned on the calling thread ("" if none). */
const char* m2_last_error(void);

/* Reads and clears the device-side status word of the current device: 0 = no kernel has
 * given up on a bounded wait since the last call.  Synchronises the device. */
int m2_device_status(int* status_out);

/* Failure-path self-test (no counterpart in the reference): launches one thread that waits, for at most
 * limit_ns (1 ns .. 1 s) of the GPU's timer, on a barrier nothing arrives at.  The wait gives up exactly as
 * a stalled wait inside the kernels would: the launch completes, M2_DEV_TIMEOUT_TMA appears in
 * m2_device_status() and later launches run normally.  Nothing faults or hangs. */
int m2_selftest_wait_timeout(unsigned long long limit_ns, void* stream);

/* ---------------------------------------------------------------------------------------
 * Implicit long-convolution filter.
 * Replaces HyenaFilter.filter / filter_rev and the bidirectional merge
 *   bert/src/mm/hyena_utils.py:201-217 (MLP on the positional embedding, :62-63 Sin,
 *   :109-112 exponential modulation) and :231-234 (pad + flip + add).
 * k_out (device, float32): (d_model, R) with R = m2_filter_row_len(seq_len) = twice the
 *   power of two >= seq_len, the period of the circular convolution the kernels run:
 *   bidirectional: row c = [ k_fwd[c, 0..L) | zeros | k_rev[c, L-1..0] ]
 *   otherwise:     row c = [ k_fwd[c, 0..L) | zeros ]
 *   (for a power-of-two seq_len this is exactly the reference's length-2L kernel).
 * bf16_rounding != 0 reproduces the rounding points of the reference under
 * torch.autocast(bfloat16): every Linear on bf16-rounded operands with a bf16-rounded
 * result, Sin and the modulation in float32.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int d_model, seq_len, order, emb_dim;
  int bidirectional;
  int bf16_rounding;
  float w_mod, shift;
  const float* z;        /* device (seq_len, emb_dim): pos_emb.z[0, :seq_len] */
  const float* t;        /* device (seq_len): pos_emb.t[0, :seq_len, 0] */
  const float* w[4];     /* device implicit_filter.{0,2,4,6}.weight: (order,emb) (order,order) x2 (d_model,order) */
  const float* b[3];     /* device implicit_filter.{0,2,4}.bias */
  const float* w_rev[4]; /* implicit_filter_rev.*; ignored unless bidirectional */
  const float* b_rev[3];
  const float* freq;     /* device (order): the shared Sin.freq */
  const float* deltas;   /* device (d_model): modulation.deltas */
  float* k_out;
} m2_filter_args;

int m2_filter_row_len(int seq_len);
int m2_hyena_filter(const m2_filter_args* args, void* stream);

/* ---------------------------------------------------------------------------------------
 * Filter spectrum in the layout the long-convolution kernel consumes.
 * Replaces `k_f = torch.fft.rfft(k, n=2L) / (2L)`, bert/src/mm/hyena_utils.py:23-24.
 * m2_longconv_kind() names the kernel family used for (seq_len, act_dtype, d_model): 0 = float32
 * arithmetic on CUDA cores (any shape), 1 = tcgen05 tensor cores (bf16, 64 < seq_len <= 128,
 * d_model a multiple of 128, channel-contiguous tensors), 2 = tcgen05 tensor cores for long rows
 * (bf16, 128 < seq_len <= 32768, a multiple of 4, transform length 4096 / 16384 / 65536 for
 * seq_len up to 2048 / 8192 / 32768; needs time-contiguous tensors, i.e. xin_st == u_st ==
 * out_st == 1; when seq_len is a multiple of 8, u is a 2-byte type and every row of xin, u and out
 * starts on a 16-byte boundary, the kernel copies its rows into shared memory asynchronously, ahead
 * of their use -- same results bit for bit, 15-35 % less time);
 * 3 = tcgen05 Toeplitz GEMMs with the batch as the M dimension (bf16, 16 <= seq_len <= 128, a
 * multiple of 8, batch >= 64; time-contiguous tensors, the residual input as fp16 from
 * m2_time_major_f16).  m2_longconv_kind() never returns 3; m2_longconv_kind_batch() does when
 * the batch is large enough to fill the 128-row tiles.
 * m2_filter_spectrum_floats() is the number of float32 the spectrum of one filter takes.
 * m2_filter_spectrum_bias() is m2_filter_spectrum() with the convolution's bias term (the
 * `+ u * bias` of fftconv_ref, bert/src/mm/hyena_utils.py:35-36; float32 (d_model), device, or
 * NULL) folded into the table: required for kind 3, whose m2_longconv_fwd call then takes
 * bias = NULL; rejected for the other kinds, which take the bias in m2_longconv_fwd.
 * k (device, float32): (d_model, m2_filter_row_len(seq_len)) as written by m2_hyena_filter.
 * ------------------------------------------------------------------------------------- */
int    m2_longconv_kind(int seq_len, m2_dtype act_dtype, int d_model);
size_t m2_filter_spectrum_floats(int kind, int d_model, int seq_len);
int    m2_filter_spectrum(int kind, int d_model, int seq_len, const float* k, float* spec_out,
                          void* stream);
int    m2_longconv_kind_batch(int batch, int seq_len, m2_dtype act_dtype, int d_model);
int    m2_filter_spectrum_bias(int kind, int d_model, int seq_len, const float* k, const float* bias,
                               float* spec_out, void* stream);

/* ---------------------------------------------------------------------------------------
 * Dense linear layer  y[b, t, n] = sum_k x[b, t, k] * w[n, k] + bias[n]  with strided activations.
 * Replaces nn.Linear `in_linear` / `out_linear` of the sequence mixer together with the layout changes
 * around them: bert/src/mm/monarch_mixer_sequence_mixer.py:81-82 (definitions), :108-109 (in_linear and the
 * transpose to (B, 3D, L)), :150-152 (the transpose back and out_linear).
 *   x   : element (b, t, k) at x[b*x_sb + t*x_st + k*x_sc]; either x_sc == 1 (rows of features) or x_st == 1
 *         (time-contiguous, e.g. a (B, D, L) or channel-major (D, B*L) tensor).
 *   out : element (b, t, n) at out[b*out_sb + t*out_st + n*out_sc]; either out_sc == 1 or out_st == 1
 *         (time-contiguous: (B, N, L), or channel-major (N, B*L) with out_sb == seq_len).
 *   w   : (out_features, in_features) row-major, dtype of x; bias float32 (out_features) or NULL.
 * M2_BF16: float32 accumulation, the bias (rounded to bf16, as autocast casts it) added in float32, one
 * rounding to bf16 -- the arithmetic of F.linear under torch.autocast.  Runs on tcgen05 tensor cores when
 * bases are 16-byte aligned and strides are multiples of 8 elements (not both x and out time-contiguous);
 * otherwise, and for M2_F32 (float32 accumulation, no rounding), on CUDA cores.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int batch, seq_len, in_features, out_features;
  m2_dtype dtype;
  const void* x; long long x_sb, x_st, x_sc;
  const void* w;
  const float* bias;
  void* out; long long out_sb, out_st, out_sc;
  int force_simt;      /* != 0: always the CUDA-core kernel (cross-checks) */
} m2_linear_args;

int m2_linear_fwd(const m2_linear_args* args, void* stream);

/* ---------------------------------------------------------------------------------------
 * Fused gated long convolution: everything between in_linear and out_linear.
 * Replaces bert/src/mm/monarch_mixer_sequence_mixer.py:109-149 -- the layout change,
 * the depthwise 3-tap short_filter (:112), x1/x2/v split (:114), v*x1 (:116), the FFT
 * convolution + bias of HyenaFilter.forward / fftconv_ref (bert/src/mm/hyena_utils.py:16-42,
 * :219-248), y*x2 (:144) and the residual long convolution on the raw layer input
 * (:131-147).
 *   xin : device, in_linear output; element (b, t, ch), ch in [0, 3*d_model) ordered x1|x2|v,
 *         at xin[b*xin_sb + t*xin_st + ch*xin_sc]; either xin_st == 1 or xin_sc == 1.
 *   u   : device, raw layer input (b, t, c) with its own strides and dtype (float32 or bf16; kinds 2
 *         and 3 also take the fp16 copy written by m2_time_major_f16 / m2_add_layernorm_fwd); used
 *         only when n_filters == 2.
 *   out : device, (b, t, c) with its own strides, dtype act_dtype: the tensor out_linear
 *         consumes.
 * bf16_rounding != 0 rounds to bf16 where the reference under autocast does (conv output,
 * v*x1, the convolution result, y*x2, the final sum).
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int batch, seq_len, d_model;
  int n_filters;            /* 1, or 2 with residual_long_conv */
  int plain;                /* != 0: HyenaFilter.forward alone -- out = conv(xin, filter 0) + bias*xin
                               with xin (b, t, c) of d_model channels: no short conv, no gates,
                               n_filters must be 1 */
  int kind;                 /* from m2_longconv_kind() */
  m2_dtype act_dtype;       /* dtype of xin and out */
  m2_dtype u_dtype;         /* dtype of u */
  int bf16_rounding;
  const void* xin; long long xin_sb, xin_st, xin_sc;
  const void* u;   long long u_sb, u_st, u_sc;
  void* out;       long long out_sb, out_st, out_sc;
  const float* short_w;     /* device (3*d_model, 3): short_filter.weight */
  const float* short_b;     /* device (3*d_model):    short_filter.bias */
  const float* spec[2];     /* device, from m2_filter_spectrum (filter_fn, filter_fn2) */
  const float* bias[2];     /* device (d_model): filter_fn.bias, filter_fn2.bias (NULL for kind 3) */
  int yu_bf16;              /* with an fp16 u (kind 3 always, kind 2 optionally): != 0 rounds the residual
                               convolution to bf16 before the final add, as the reference does when the
                               layer input is bf16 (with a float32 / bf16 u this follows from u_dtype) */
} m2_longconv_args;

int m2_longconv_fwd(const m2_longconv_args* args, void* stream);

/* ---------------------------------------------------------------------------------------
 * dst[c, b, t] = fp16(src[b, t, c]) (saturating): the time-contiguous fp16 copy of the raw
 * layer input that kind 3 of m2_longconv_fwd loads as a tensor-core operand.  Part of the
 * `u.transpose(-1, -2)` layout change of bert/src/mm/monarch_mixer_sequence_mixer.py:109.
 *   src (batch, seq_len, d_model) of src_dtype (M2_F32 or M2_BF16) with strides in elements;
 *   dst fp16, element (c, b, t) at dst[c*dst_sc + b*dst_sb + t].
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int batch, seq_len, d_model;
  m2_dtype src_dtype;
  const void* src; long long src_sb, src_st, src_sc;
  void* dst;       long long dst_sb, dst_sc;
} m2_time_major_args;

int m2_time_major_f16(const m2_time_major_args* args, void* stream);

/* ---------------------------------------------------------------------------------------
 * Block-diagonal linear:  out[:, k*q:(k+1)*q] = x[:, k*p:(k+1)*p] @ w[k]^T (+ bias).
 * Replaces BlockdiagMultiply.forward, bert/src/mm/blockdiag_multiply.py:49-60, and the
 * bias add of StructuredLinear.forward, bert/src/mm/structured_linear.py:67-70.
 *   x (m, in_features) row stride ldx, in_features <= nblocks*p (missing columns read as
 *   zero: StructuredLinear.preprocess, structured_linear.py:52-56); w (nblocks, q, p)
 *   contiguous; out (m, out_features) row stride ldo, out_features <= nblocks*q (extra
 *   columns are cropped: postprocess, :58-62); x, w, out share `dtype`; bias float32
 *   (out_features) or NULL.  With M2_BF16 the product is rounded to bf16 before the
 *   (bf16-rounded) bias is added, as the reference does.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int m, nblocks, p, q;
  int in_features, out_features;
  m2_dtype dtype;
  const void* x; long long ldx;
  const void* w;
  const float* bias;
  void* out; long long ldo;
  int variant;   /* 0: the library picks the kernel; 2: CTA-pair tiles (the kernel of m2_linear_fwd) where they apply --
                    results are bit-identical, kept selectable for cross-checks */
} m2_blockdiag_args;

int m2_blockdiag_fwd(const m2_blockdiag_args* args, void* stream);

/* ---------------------------------------------------------------------------------------
 * Gated half of the GLU MLP: h = gelu(G[:, :I]) * G[:, I:],  G = blockdiag(x, wg).
 * Replaces gated_layers + the slice/GELU/multiply of BertGatedLinearUnitMLP.forward,
 * bert/src/bert_layers.py:492-501; G itself is never written.
 *   x (m, d_model); wg (nblocks, 2*inter/nblocks, d_model/nblocks); h (m, inter).
 *   nblocks must be even (column j of G pairs with column j + inter, which lies nblocks/2
 *   blocks further on and reads a different slice of x).
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int m, d_model, inter, nblocks;
  m2_dtype dtype;
  const void* x; long long ldx;
  const void* wg;
  void* h; long long ldh;
  int variant;   /* 0: the library picks the kernel (x slices resident in shared memory when d_model / nblocks <= 192);
                    1: always the kernel that streams x and wg tiles through shared memory (the general one);
                    3: CTA pairs with resident x slices where they apply.  Results are bit-identical; the variants are
                    selectable for cross-checks */
} m2_glu_args;

int m2_blockdiag_glu_fwd(const m2_glu_args* args, void* stream);

/* ---------------------------------------------------------------------------------------
 * out = LayerNorm(a + b) over the last dimension (float32 statistics).
 * Replaces `self.layernorm(hidden_states + residual_connection)`, bert/src/bert_layers.py:506.
 * a, b (m, n) of `in_dtype` (the sum is rounded to bf16 first when in_dtype is M2_BF16, as a
 * bf16 tensor add does); out (m, n) of `out_dtype`; weight/bias float32 (n).  b may be NULL
 * (plain LayerNorm(a), e.g. the embeddings' LayerNorm, bert/src/bert_layers.py:131-252) when n is
 * a multiple of 256 up to 2048 and rows are 16-byte aligned.
 * out_bf16 (optional, may be NULL): a second copy of the result rounded to bf16, row stride
 * ld_bf16 -- what the next layer's in_linear reads under autocast (its cast of the float32
 * LayerNorm output), written here instead of by a separate cast pass.  With out_bf16 given,
 * out may be NULL: only the copies are written (a caller that feeds the next mixer from them).
 * out_tm_f16 (optional, may be NULL): a third copy as fp16 laid out time-major, row r = b *
 * seq_len + t, column c at out_tm_f16[c*tm_sc + b*tm_sb + t] -- what m2_time_major_f16 would
 * make of `out`, the residual-filter operand of kind 3 of m2_longconv_fwd.  Needs the same
 * shapes as out_bf16, seq_len a multiple of 8 that divides m, tm_sb and tm_sc multiples of 8.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int m, n;
  m2_dtype in_dtype, out_dtype;
  const void* a; long long lda;
  const void* b; long long ldb;
  const float* weight; const float* bias;
  float eps;
  void* out; long long ldo;
  void* out_bf16; long long ld_bf16;
  void* out_tm_f16; long long tm_sb, tm_sc; int seq_len;
  int bf16_pad_cols;   /* > 0: also write columns n .. n+bf16_pad_cols of each out_bf16 row as
                          [1, 0, 0, ...] -- the constant column through which a following GEMM adds
                          its bias (a multiple of 8, at most 256) */
} m2_add_layernorm_args;

int m2_add_layernorm_fwd(const m2_add_layernorm_args* args, void* stream);

/* ---------------------------------------------------------------------------------------
 * Embeddings: out = LayerNorm((word_table[input_ids] + type_table[token_type_ids]) + pos_table[position_ids])
 * in float32 -- the gathers, the two adds and the LayerNorm of BertEmbeddings.forward,
 * bert/src/bert_layers.py:186-252 (dropout is the identity in eval mode) -- in one launch, with the
 * same optional copies for the first mixer as m2_add_layernorm_fwd.
 *   tables float32, row-major with n columns; ids int64 (m); token_type_ids NULL = type 0 everywhere;
 *   pos_table NULL = no position term; position_ids NULL = position r % seq_len for row r.
 *   n a multiple of 256 up to 2048.  out may be NULL when out_bf16 is given.
 *   vocab_rows / type_rows / pos_rows: row counts of the tables.  An id outside [0, rows) is never read
 *   out of bounds: it is clamped into the table and M2_DEV_BAD_INDEX is set in the device status word
 *   (torch's embedding would raise a device-side assert there); seq_len > pos_rows without explicit
 *   position_ids is refused on the host.
 * ------------------------------------------------------------------------------------- */
typedef struct {
  int m, n;
  const float* word_table; const long long* input_ids;
  const float* type_table; const long long* token_type_ids;
  const float* pos_table;  const long long* position_ids;
  const float* weight; const float* bias; float eps;
  float* out; long long ldo;
  void* out_bf16; long long ld_bf16; int bf16_pad_cols;
  void* out_tm_f16; long long tm_sb, tm_sc; int seq_len;
  long long vocab_rows, type_rows, pos_rows;
} m2_embed_layernorm_args;

int m2_embed_layernorm_fwd(const m2_embed_layernorm_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* M2_B200_H */
