// Shared helpers of the sm_100a verify-step library: status codes, error capture,
// element-type traits and per-device immutable properties.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/rlt_verify.h"

namespace rlt {

// Records the text of a failed CUDA call for rlt_last_error() (thread-local).
void set_last_error(const char* what, cudaError_t err);
void set_last_error_text(const char* what);

#define RLT_CUDA_TRY(expr)                      \
  do {                                          \
    cudaError_t rlt_err__ = (expr);             \
    if (rlt_err__ != cudaSuccess) {             \
      ::rlt::set_last_error(#expr, rlt_err__);  \
      return RLT_ERR_CUDA;                      \
    }                                           \
  } while (0)

#define RLT_REQUIRE(cond, text)                 \
  do {                                          \
    if (!(cond)) {                              \
      ::rlt::set_last_error_text(text);         \
      return RLT_ERR_INVALID;                   \
    }                                           \
  } while (0)

// Checks the launch that was just issued without synchronising.
inline int launch_status(const char* what) {
  cudaError_t err = cudaPeekAtLastError();
  if (err != cudaSuccess) {
    cudaGetLastError();
    set_last_error(what, err);
    return RLT_ERR_CUDA;
  }
  return RLT_OK;
}

struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0;
  int cc_minor = 0;
  size_t smem_optin = 0;
};
// Properties of the current device, looked up once per device (safe during graph capture:
// attribute queries do not touch a stream).
int current_device_info(DeviceInfo* out);

inline size_t dtype_size(int dtype) { return dtype == RLT_F32 ? 4 : 2; }
inline bool dtype_valid(int dtype) { return dtype == RLT_F32 || dtype == RLT_F16 || dtype == RLT_BF16; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Element conversions used by the kernels that accept all three storage types.
template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int kCode = RLT_F32;
  __device__ __forceinline__ static float to_float(float x) { return x; }
  __device__ __forceinline__ static float from_float(float x) { return x; }
};
template <> struct Elem<__half> {
  static constexpr int kCode = RLT_F16;
  __device__ __forceinline__ static float to_float(__half x) { return __half2float(x); }
  __device__ __forceinline__ static __half from_float(float x) { return __float2half_rn(x); }
};
template <> struct Elem<__nv_bfloat16> {
  static constexpr int kCode = RLT_BF16;
  __device__ __forceinline__ static float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
  __device__ __forceinline__ static __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};

// Calls f.template operator()<T>() for the element type selected by `dtype`.
#define RLT_DISPATCH_DTYPE(dtype, T, ...)                        \
  do {                                                           \
    if ((dtype) == RLT_F32) { using T = float; __VA_ARGS__; }    \
    else if ((dtype) == RLT_F16) { using T = __half; __VA_ARGS__; } \
    else { using T = __nv_bfloat16; __VA_ARGS__; }               \
  } while (0)

}  // namespace rlt
