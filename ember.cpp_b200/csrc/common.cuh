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
// no-ops.  What the kernel before wrote must not be read through the read-only data path
// (`ld.global.nc`, which the compiler may choose for a plain load through a const __restrict__
// pointer): that path is only right for data that does not change during the kernel's life, and
// this kernel's life begins before its producer's ends.  Such data is read with `__ldcg` (L2), by
// TMA, or with an explicit `ld.global.ca` where blocks of one SM share it (L1 is made coherent
// between dependent grids; the read-only path is not).  Seen once: a decode attention that moved
// its keys by TMA, so that nothing swept L1 any more, read q through the read-only path and got
// an earlier step's values in a replayed graph.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// Timeline of a step's kernels.  A library built with -DEMBER_TIMELINE (EMBER_TIMELINE=1 in the
// environment when it is built; it goes to a folder of its own) has every block of the decode
// step's kernels note the global timer when it starts, when its wait for the kernel before it
// returns, when it ends, and at a few places between.  Each source file keeps its own log (there is no relocatable device
// code to share one) and exports a reader; without the flag the marks compile to nothing.
#ifdef EMBER_TIMELINE
namespace timeline {
constexpr unsigned kMarks = 8;          // marks a block can leave
constexpr unsigned kCap = 1u << 18;     // entries of a file's log
enum Kernel { kEmbed = 1, kLayerNorm = 2, kLinearDecode = 3, kAttentionDecode = 4, kSample = 5, kLinearStream = 6 };
enum Mark { kStart = 0, kDependency = 1, kEnd = 2, kMerged = 3, kPhaseA = 4, kPhaseB = 5, kPhaseC = 6, kPhaseD = 7 };
struct Entry {
  unsigned long long t;  // nanoseconds of the global timer; 0: the block did not leave this mark
  unsigned what;         // kernel << 8 | mark
  unsigned block;        // linear block index
  unsigned grid;         // blocks of the launch
  unsigned sm;           // the SM the block runs on
};
static __device__ Entry g_log[kCap];
static __device__ unsigned g_n;
__device__ __forceinline__ unsigned long long now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void put(unsigned at, unsigned kernel, unsigned m) {
  if (at + m < kCap) {
    Entry e;
    e.t = now();
    e.what = kernel << 8 | m;
    e.block = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    e.grid = gridDim.x * gridDim.y * gridDim.z;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(e.sm));
    g_log[at + m] = e;
  }
}
// The block's first mark takes its kMarks places in the log (the only atomic: later marks wait
// for nothing); thread 0 keeps the place.
__device__ __forceinline__ unsigned start(unsigned kernel) {
  unsigned at = kCap;
  if (threadIdx.x == 0) {
    at = atomicAdd(&g_n, kMarks);
    put(at, kernel, kStart);
  }
  return at;
}
__device__ __forceinline__ void mark(unsigned at, unsigned kernel, unsigned m) {
  if (threadIdx.x == 0) put(at, kernel, m);
}
// Copies this file's log to dst (room for cap entries), empties it and returns how many places
// were taken (places whose time is 0 were not written).
inline int read(void* dst, unsigned cap) {
  unsigned n = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&n, g_n, sizeof(n)) != cudaSuccess) return -1;
  if (n > kCap) n = kCap;
  if (n > cap) n = cap;
  if (n && cudaMemcpyFromSymbol(dst, g_log, (size_t)n * sizeof(Entry)) != cudaSuccess) return -1;
  void* log_at = nullptr;
  if (cudaGetSymbolAddress(&log_at, g_log) != cudaSuccess) return -1;
  if (n && cudaMemset(log_at, 0, (size_t)n * sizeof(Entry)) != cudaSuccess) return -1;
  const unsigned zero = 0;
  if (cudaMemcpyToSymbol(g_n, &zero, sizeof(zero)) != cudaSuccess) return -1;
  return (int)n;
}
}  // namespace timeline
#define EMBER_MARK_START(kernel) const unsigned ember_tl = timeline::start(timeline::kernel)
#define EMBER_MARK(kernel, m) timeline::mark(ember_tl, timeline::kernel, timeline::m)
#define EMBER_TIMELINE_READER(file) \
  EMBER_API int ember_timeline_read_##file(void* dst, unsigned cap) { return timeline::read(dst, cap); }
#else
#define EMBER_MARK_START(kernel)
#define EMBER_MARK(kernel, m)
#define EMBER_TIMELINE_READER(file)
#endif

// Switches that the kernels' launch code reads; `ember_set_option(which, value)` sets them (the
// Python side does, from its RuntimeOptions).  Process-wide; all on by default.
//   EMBER_OPT_PDL             programmatic dependent launch between the kernels of a step (0: ordinary launches)
//   EMBER_OPT_DECODE_BULK     the CUDA-core decode attention brings pages in by bulk copies (0: by loads)
//   EMBER_OPT_DECODE_CLUSTER  the tensor-core decode attention merges its chunks in a cluster (0: scratch and a ticket)
enum : int { EMBER_OPT_PDL = 0, EMBER_OPT_DECODE_BULK = 1, EMBER_OPT_DECODE_CLUSTER = 2, EMBER_OPT_COUNT = 3 };
extern int g_ember_options[EMBER_OPT_COUNT];  // elementwise.cu
inline int pdl_allowed() { return g_ember_options[EMBER_OPT_PDL]; }

// The number of SMs of the current device (asked once per device; launch heuristics size grids by it).
inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    cached[dev] = n;
  }
  return cached[dev];
}

// A launch whose blocks all fit the chip at once is fastest with its blocks on as many SMs as can be (an
// SM takes in only some 50 KB a microsecond, and the block scheduler fills the SMs that are free first to
// the brim): a request for more shared memory than the block needs caps what an SM takes at
// ceil(blocks / SMs) blocks.
inline size_t spread_smem(size_t need, long long blocks) {
  const long long per_sm = (blocks + sm_count() - 1) / sm_count();
  const size_t room = (size_t)(227 * 1024) / (size_t)per_sm;
  const size_t want = room > 8192 ? room - 6144 : 0;  // less a block's own kilobyte of the SM's shared memory and its static variables
  return want > need ? want : need;
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
