// Shared host/device helpers for the m2_b200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <string.h>
#include "../../include/m2_b200.h"

// ---- host side error plumbing -------------------------------------------------------
int m2_set_error(int code, const char* fmt, ...);   // stores a thread-local message, returns code

#define M2_REQUIRE(cond, code, ...) \
  do { if (!(cond)) return m2_set_error((code), __VA_ARGS__); } while (0)

#define M2_CUDA(call) \
  do { cudaError_t e_ = (call); \
       if (e_ != cudaSuccess) return m2_set_error(M2_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e_)); } while (0)

#define M2_LAUNCH_CHECK(name) \
  do { cudaError_t e_ = cudaGetLastError(); \
       if (e_ != cudaSuccess) return m2_set_error(M2_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e_)); } while (0)

static inline bool m2_is_pow2(long long v) { return v > 0 && (v & (v - 1)) == 0; }
static inline int m2_ilog2(long long v) { int l = 0; while ((1LL << l) < v) ++l; return l; }
static inline bool m2_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Per-device status word that kernels set when a bounded wait runs out (defined once; all
// parts are compiled as a single translation unit, see m2_b200.cu).
__device__ int m2_dev_status_word = 0;

// ---- device helpers -----------------------------------------------------------------
// Round a float to the nearest bf16 value (ties to even) and return it as a float.
__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

template <bool ROUND> __device__ __forceinline__ float rnd(float x) { return ROUND ? bf16r(x) : x; }

template <typename T> __device__ __forceinline__ float ld_as_float(const T* p);
template <> __device__ __forceinline__ float ld_as_float<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <typename T> __device__ __forceinline__ void st_from_float(T* p, float v);
template <> __device__ __forceinline__ void st_from_float<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st_from_float<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float2 cmul(float2 a, float2 b) {
  return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
}
__device__ __forceinline__ float2 cmul_conj(float2 a, float2 b) {  // a * conj(b)
  return make_float2(a.x * b.x + a.y * b.y, a.y * b.x - a.x * b.y);
}

// One 32-byte store per thread (a full DRAM/L2 sector; two 16-byte stores of the same thread
// reach L2 as two partial-sector writes).  p must be 32-byte aligned.
__device__ __forceinline__ void stg256(void* p, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t a4,
                                       uint32_t a5, uint32_t a6, uint32_t a7) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(p), "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(a4), "r"(a5), "r"(a6), "r"(a7) : "memory");
}

// ---- packed float32 pairs (sm_100 f32x2 arithmetic: two FMAs per instruction) ----------
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 f2_pack(float lo, float hi) {
  f32x2 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void f2_unpack(f32x2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 f2_fma(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 f2_mul(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 f2_splat(float v) { return f2_pack(v, v); }

// lane-wise product of two packed bf16 pairs, rounded to bf16 once (the exact product of two
// bf16 values fits a float32, so this equals multiplying in float32 and rounding)
__device__ __forceinline__ uint32_t bf2_mul(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// gelu(x) = x Phi(x) for two values at once.  With a = |x|:  x Phi(x) = max(x, 0) - a Phi(-a), and
// log2 Phi(-a) is smooth, so Phi(-a) = 2^P(a) with P the degree-7 least-squares Chebyshev fit of
// log2 Phi(-a) on [0, 6.5] (evaluated in u = 2a/6.5 - 1; relative error of Phi(-a) below 8e-6 over the
// whole range, tail included; a is clamped at 6.5, where a Phi(-a) = 2.6e-10).  One ex2 per value and
// packed f32x2 FMAs; the result is meant to be rounded to bf16 next: against the exact-erf value 0.05 %
// of bf16 results differ, by one bf16 step (2 M samples of N(0, 1.5) inputs).
__device__ __forceinline__ void gelu_pair(float x0, float x1, float& y0, float& y1) {
  const float n0 = -fabsf(x0), n1 = -fabsf(x1);                                // -a
  const f32x2 na = f2_pack(n0, n1);
  const f32x2 u = f2_fma(f2_pack(fmaxf(n0, -6.5f), fmaxf(n1, -6.5f)), f2_splat(-2.0f / 6.5f), f2_splat(-1.0f));
  f32x2 p = f2_fma(f2_splat(-6.778277458e-03f), u, f2_splat(2.354049963e-02f));
  p = f2_fma(p, u, f2_splat(-4.978999801e-02f));
  p = f2_fma(p, u, f2_splat(1.049118857e-01f));
  p = f2_fma(p, u, f2_splat(-2.236005766e-01f));
  p = f2_fma(p, u, f2_splat(-7.137094648e+00f));
  p = f2_fma(p, u, f2_splat(-1.648756080e+01f));
  p = f2_fma(p, u, f2_splat(-1.075908454e+01f));
  float p0, p1, q0, q1;
  f2_unpack(p, p0, p1);
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(q0) : "f"(p0));                    // Phi(-a)
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(q1) : "f"(p1));
  f2_unpack(f2_fma(na, f2_pack(q0, q1), f2_pack(fmaxf(x0, 0.f), fmaxf(x1, 0.f))), y0, y1);
}

__device__ __forceinline__ float gelu_erf(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
}
