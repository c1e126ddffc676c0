// Entry points of the fused gated long convolution: kernel-family selection, filter
// spectrum tables, argument validation.
#include "common.cuh"

namespace m2 {
int longconv_simt_launch(const m2_longconv_args* a, cudaStream_t st);
int spectrum_kind0_launch(int D, int L, const float* k, float* spec, cudaStream_t st);
int longconv_tc_supported(int seq_len, m2_dtype act_dtype, int d_model);
size_t spectrum_kind1_floats(int D, int L);
int spectrum_kind1_launch(int D, int L, const float* k, float* spec, cudaStream_t st);
int longconv_tc_launch(const m2_longconv_args* a, cudaStream_t st);
int longconv_tcl_supported(int seq_len, m2_dtype act_dtype);
size_t spectrum_kind2_floats(int D, int L);
int spectrum_kind2_launch(int D, int L, const float* k, float* spec, cudaStream_t st);
int longconv_tcl_launch(const m2_longconv_args* a, cudaStream_t st);
int longconv_tz_supported(int batch, int seq_len, m2_dtype act_dtype);
size_t spectrum_kind3_floats(int D, int L);
int spectrum_kind3_launch(int D, int L, const float* k, const float* bias, float* spec, cudaStream_t st);
int longconv_tz_launch(const m2_longconv_args* a, cudaStream_t st);
int time_major_f16_launch(const m2_time_major_args* a, cudaStream_t st);
}  // namespace m2

extern "C" int m2_longconv_kind(int seq_len, m2_dtype act_dtype, int d_model) {
  if (m2::longconv_tc_supported(seq_len, act_dtype, d_model)) return 1;
  if (m2::longconv_tcl_supported(seq_len, act_dtype)) return 2;
  return 0;
}

extern "C" int m2_longconv_kind_batch(int batch, int seq_len, m2_dtype act_dtype, int d_model) {
  if (m2::longconv_tz_supported(batch, seq_len, act_dtype)) return 3;
  return m2_longconv_kind(seq_len, act_dtype, d_model);
}

extern "C" size_t m2_filter_spectrum_floats(int kind, int d_model, int seq_len) {
  if (d_model <= 0 || seq_len <= 0) return 0;
  if (kind == 3) return m2::spectrum_kind3_floats(d_model, seq_len);
  if (kind == 1) return m2::spectrum_kind1_floats(d_model, seq_len);
  if (kind == 2) return m2::spectrum_kind2_floats(d_model, seq_len);
  const size_t M = (size_t)m2_filter_row_len(seq_len) / 2;
  return M + 4 * M * (size_t)d_model;
}

extern "C" int m2_filter_spectrum_bias(int kind, int d_model, int seq_len, const float* k, const float* bias,
                                       float* spec_out, void* stream) {
  if (kind != 3) {
    M2_REQUIRE(bias == nullptr, M2_ERR_ARG,
               "m2_filter_spectrum_bias: only kind 3 folds the bias into the table; kind %d takes it in m2_longconv_fwd", kind);
    return m2_filter_spectrum(kind, d_model, seq_len, k, spec_out, stream);
  }
  M2_REQUIRE(d_model > 0 && seq_len > 0, M2_ERR_ARG, "m2_filter_spectrum_bias: sizes must be positive");
  M2_REQUIRE(k && spec_out, M2_ERR_ARG, "m2_filter_spectrum_bias: NULL pointer");
  M2_REQUIRE(m2_aligned(spec_out, 16), M2_ERR_ALIGN, "m2_filter_spectrum_bias: spec_out must be 16-byte aligned");
  return m2::spectrum_kind3_launch(d_model, seq_len, k, bias, spec_out, static_cast<cudaStream_t>(stream));
}

extern "C" int m2_time_major_f16(const m2_time_major_args* a, void* stream) {
  M2_REQUIRE(a != nullptr, M2_ERR_ARG, "m2_time_major_f16: args is NULL");
  M2_REQUIRE(a->batch >= 0 && a->seq_len > 0 && a->d_model > 0, M2_ERR_ARG, "m2_time_major_f16: bad sizes");
  if (a->batch == 0) return M2_OK;
  M2_REQUIRE(a->src && a->dst, M2_ERR_ARG, "m2_time_major_f16: NULL tensor pointer");
  M2_REQUIRE(a->src_dtype == M2_F32 || a->src_dtype == M2_BF16, M2_ERR_UNSUPPORTED,
             "m2_time_major_f16: src must be float32 or bf16");
  M2_REQUIRE(a->batch <= 65535 && (a->d_model + 63) / 64 <= 65535, M2_ERR_UNSUPPORTED, "m2_time_major_f16: too large");
  return m2::time_major_f16_launch(a, static_cast<cudaStream_t>(stream));
}

extern "C" int m2_filter_spectrum(int kind, int d_model, int seq_len, const float* k, float* spec_out,
                                  void* stream) {
  M2_REQUIRE(d_model > 0 && seq_len > 0, M2_ERR_ARG, "m2_filter_spectrum: sizes must be positive");
  M2_REQUIRE(k && spec_out, M2_ERR_ARG, "m2_filter_spectrum: NULL pointer");
  M2_REQUIRE(m2_aligned(k, 8) && m2_aligned(spec_out, 16), M2_ERR_ALIGN,
             "m2_filter_spectrum: k must be 8-byte and spec_out 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (kind == 3) return m2::spectrum_kind3_launch(d_model, seq_len, k, nullptr, spec_out, st);
  if (kind == 0) return m2::spectrum_kind0_launch(d_model, seq_len, k, spec_out, st);
  if (kind == 1) return m2::spectrum_kind1_launch(d_model, seq_len, k, spec_out, st);
  if (kind == 2) return m2::spectrum_kind2_launch(d_model, seq_len, k, spec_out, st);
  return m2_set_error(M2_ERR_ARG, "m2_filter_spectrum: unknown kind %d", kind);
}

extern "C" int m2_longconv_fwd(const m2_longconv_args* a, void* stream) {
  M2_REQUIRE(a != nullptr, M2_ERR_ARG, "m2_longconv_fwd: args is NULL");
  M2_REQUIRE(a->batch >= 0 && a->seq_len > 0 && a->d_model > 0, M2_ERR_ARG,
             "m2_longconv_fwd: bad sizes batch=%d seq_len=%d d_model=%d", a->batch, a->seq_len, a->d_model);
  M2_REQUIRE(a->n_filters == 1 || a->n_filters == 2, M2_ERR_ARG, "m2_longconv_fwd: n_filters must be 1 or 2");
  M2_REQUIRE(!a->plain || a->n_filters == 1, M2_ERR_ARG, "m2_longconv_fwd: plain mode takes one filter");
  if (a->batch == 0) return M2_OK;
  const bool folded = a->kind == 3 && !a->plain;       // kind 3 has the bias inside its spectrum
  M2_REQUIRE(a->xin && a->out && (a->plain || (a->short_w && a->short_b)) && a->spec[0] && (folded || a->bias[0]), M2_ERR_ARG,
             "m2_longconv_fwd: NULL tensor pointer");
  M2_REQUIRE(a->n_filters == 1 || (a->u && a->spec[1] && (folded || a->bias[1])), M2_ERR_ARG,
             "m2_longconv_fwd: residual filter requested but u/spec[1]/bias[1] is NULL");
  M2_REQUIRE(a->xin_st == 1 || a->xin_sc == 1, M2_ERR_UNSUPPORTED,
             "m2_longconv_fwd: xin must be contiguous along time or along channels");
  M2_REQUIRE(a->batch <= 65535, M2_ERR_UNSUPPORTED, "m2_longconv_fwd: batch > 65535");
  M2_REQUIRE(m2_aligned(a->spec[0], 16) && (a->n_filters == 1 || m2_aligned(a->spec[1], 16)), M2_ERR_ALIGN,
             "m2_longconv_fwd: spectrum tables must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->kind == 0 || a->plain) return m2::longconv_simt_launch(a, st);
  if (a->kind == 1) return m2::longconv_tc_launch(a, st);
  if (a->kind == 2) return m2::longconv_tcl_launch(a, st);
  if (a->kind == 3) return m2::longconv_tz_launch(a, st);
  return m2_set_error(M2_ERR_ARG, "m2_longconv_fwd: unknown kind %d", a->kind);
}
