// Shared definitions for the PSA sm_100a kernels: element-type traits, status codes, launch checks.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/psa_b200.h"

namespace psa {

// Last error text of this thread (returned by psa_last_error_string).
void set_error(const char* fmt, ...);

#define PSA_REQUIRE(cond, code, ...)          \
  do {                                        \
    if (!(cond)) {                            \
      ::psa::set_error(__VA_ARGS__);          \
      return (code);                          \
    }                                         \
  } while (0)

#define PSA_CHECK_LAUNCH(what)                                                       \
  do {                                                                               \
    cudaError_t e__ = cudaGetLastError();                                            \
    if (e__ != cudaSuccess) {                                                        \
      ::psa::set_error("%s: launch failed: %s", what, cudaGetErrorString(e__));      \
      return PSA_ERR_CUDA;                                                           \
    }                                                                                \
  } while (0)

template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_f(float x) { return x; }
  static __device__ __forceinline__ float from_f(float x) { return x; }
  static __device__ __forceinline__ float round(float x) { return x; }
};
template <> struct Elem<__half> {
  static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
  static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
  static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};

// Dispatch a templated launcher on the runtime dtype code.
#define PSA_DISPATCH_DTYPE(dtype, T, ...)                                   \
  switch (dtype) {                                                          \
    case PSA_F32: { using T = float; __VA_ARGS__; } break;                  \
    case PSA_F16: { using T = __half; __VA_ARGS__; } break;                 \
    case PSA_BF16: { using T = __nv_bfloat16; __VA_ARGS__; } break;         \
    default: ::psa::set_error("unsupported dtype code %d", (int)(dtype));   \
      return PSA_ERR_ARG;                                                   \
  }

static inline int64_t cdiv64(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace psa
