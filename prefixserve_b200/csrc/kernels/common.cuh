// Shared helpers for the sm_100a kernels: element types, error reporting, and
// the C ABI conventions.  Every entry point returns 0 on success; otherwise it
// has left a message for psb_last_error() and launched nothing (or the launch
// itself failed).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#define PSB_API extern "C" __attribute__((visibility("default")))

enum PsbDtype : int { PSB_F32 = 0, PSB_BF16 = 1 };

void psb_set_error(const char* fmt, ...);

#define PSB_REFUSE(...)          \
  do {                           \
    psb_set_error(__VA_ARGS__);  \
    return 1;                    \
  } while (0)

#define PSB_LAUNCH_CHECK(name)                                                   \
  do {                                                                           \
    cudaError_t e_ = cudaGetLastError();                                         \
    if (e_ != cudaSuccess) {                                                     \
      psb_set_error("%s: launch failed: %s", name, cudaGetErrorString(e_));      \
      return 2;                                                                  \
    }                                                                            \
  } while (0)

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Calls f.template operator()<T>() with T chosen by a PsbDtype code.
#define PSB_DISPATCH_DTYPE(code, T, ...)                       \
  if ((code) == PSB_F32) { using T = float; __VA_ARGS__ }      \
  else if ((code) == PSB_BF16) { using T = __nv_bfloat16; __VA_ARGS__ } \
  else PSB_REFUSE("unknown dtype code %d", (int)(code))
