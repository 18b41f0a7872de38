// Shared helpers of the kernels: element types, warp reductions, error reporting.
//
// Every entry point is `extern "C"`, takes raw device pointers, sizes and the stream to launch on,
// allocates nothing and returns 0 or a non-zero code after storing a message that
// `ember_last_error()` returns.  Arguments are checked on the host before any launch; no kernel
// traps, asserts or waits on another.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define EMBER_API extern "C" __attribute__((visibility("default")))

// element type codes shared with the Python side
enum : int { EMBER_F32 = 0, EMBER_BF16 = 1 };

// activation codes of the linear epilogues
enum : int { EMBER_ACT_NONE = 0, EMBER_ACT_GELU_TANH = 1, EMBER_ACT_GELU_ERF = 2 };

constexpr int kPage = 64;  // positions per cache page

int ember_fail(const char* fmt, ...);

#define EMBER_CHECK(cond, ...)                     \
  do {                                             \
    if (!(cond)) return ember_fail(__VA_ARGS__);   \
  } while (0)

#define EMBER_LAUNCH_OK(name)                                                        \
  do {                                                                               \
    cudaError_t e_ = cudaGetLastError();                                             \
    if (e_ != cudaSuccess) return ember_fail("%s: %s", name, cudaGetErrorString(e_)); \
  } while (0)

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

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

// GELU in both forms, every product in float32.
__device__ __forceinline__ float gelu_tanh(float v) {
  const float c = 0.7978845608028654f;  // sqrt(2/pi)
  return 0.5f * v * (1.0f + tanhf(c * (v + 0.044715f * v * v * v)));
}
__device__ __forceinline__ float gelu_erf(float v) { return 0.5f * v * (1.0f + erff(v * 0.7071067811865476f)); }

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == EMBER_ACT_GELU_TANH) return gelu_tanh(v);
  if (act == EMBER_ACT_GELU_ERF) return gelu_erf(v);
  return v;
}
