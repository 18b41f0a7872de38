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
#include <stdlib.h>

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

// Programmatic dependent launch.  A kernel launched with launch_pdl may begin while the kernel
// before it in the stream is still running; it must call pdl_wait() before it reads anything
// that kernel wrote and before it writes anything at all.  pdl_trigger() lets the kernel after
// this one begin early in the same way.  In a kernel that was launched the ordinary way both are
// no-ops.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// EMBER_PDL=0 in the environment launches these kernels the ordinary way (for measurements).
inline int pdl_allowed() {
  static const int on = [] {
    const char* v = getenv("EMBER_PDL");
    return (v && v[0] == '0') ? 0 : 1;
  }();
  return on;
}

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = pdl_allowed();
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
