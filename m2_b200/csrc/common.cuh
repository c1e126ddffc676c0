// Shared host/device helpers for the m2_b200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
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

__device__ __forceinline__ float gelu_erf(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
}
