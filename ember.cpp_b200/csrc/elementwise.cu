// Row kernels: token + position embedding, layer norm, row gather, and the error channel.
//
// ember.cpp runs these as separate float32 kernels (embedding and position add
// graph_ir_cuda.cu:19-32, layer norm :47-65 with sums in double).  Here the embedding and the
// position row are read and added in one kernel, and the norm keeps float32 statistics on the
// float32 residual stream; each row's arithmetic depends on that row alone.
#include <stdarg.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

int ember_fail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return 1;
}

EMBER_API const char* ember_last_error() { return g_error; }

int g_ember_options[EMBER_OPT_COUNT] = {1, 1, 1};

EMBER_API int ember_set_option(int which, int value) {
  EMBER_CHECK(which >= 0 && which < EMBER_OPT_COUNT, "set_option: there is no option %d", which);
  g_ember_options[which] = value != 0;
  return 0;
}

// ---------------------------------------------------------------------------- embedding
// x[t, :] = table[token_t, :] (+ pos_table[position_t, :]), in float32.  A token is tokens[t], or, where
// src is given and src[t] >= 0, ids[src[t]]: an id that an earlier step's sampler left on the device
// (clamped into the table: a sampler's id is always in range; nothing else may reach the table).  Rows
// whose width is a multiple of 8 are read 16 bytes a thread.
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const int* __restrict__ src, const int* ids, int n_ids,
                             int vocab, const int* __restrict__ positions, const T* __restrict__ table,
                             const T* __restrict__ pos_table, float* __restrict__ x, int d) {
  EMBER_MARK_START(kEmbed);
  const int t = blockIdx.x;
  int tok = tokens[t];
  if (src) {
    const int r = src[t];
    if (r >= 0 && r < n_ids) {
      const int v = __ldcg(ids + r);
      tok = (v >= 0 && v < vocab) ? v : 0;
    }
  }
  const T* row = table + (size_t)tok * d;
  const T* prow = pos_table ? pos_table + (size_t)positions[t] * d : nullptr;
  float* out = x + (size_t)t * d;
  constexpr int kVec = 16 / (int)sizeof(T);  // values in 16 bytes
  if (d % kVec == 0) {
    for (int i = threadIdx.x * kVec; i < d; i += blockDim.x * kVec) {
      const uint4 a = *reinterpret_cast<const uint4*>(row + i);
      uint4 b = make_uint4(0, 0, 0, 0);
      if (prow) b = *reinterpret_cast<const uint4*>(prow + i);
      const T* av = reinterpret_cast<const T*>(&a);
      const T* bv = reinterpret_cast<const T*>(&b);
      float v[kVec];
#pragma unroll
      for (int j = 0; j < kVec; ++j) v[j] = prow ? to_float(av[j]) + to_float(bv[j]) : to_float(av[j]);
#pragma unroll
      for (int j = 0; j < kVec; j += 4) *reinterpret_cast<float4*>(out + i + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      float v = to_float(row[i]);
      if (prow) v += to_float(prow[i]);
      out[i] = v;
    }
  }
  EMBER_MARK(kEmbed, kEnd);
}

// src, ids: both null, or the rows of `ids` (n_ids of them) that the tokens come from (see above).
EMBER_API int ember_embed(const int* tokens, const int* positions, const void* table, const void* pos_table, float* x,
                          int T, int d, int dtype, const int* src, const int* ids, int n_ids, int vocab,
                          cudaStream_t stream) {
  EMBER_CHECK(T > 0 && d > 0, "embed: T = %d, width = %d", T, d);
  EMBER_CHECK((src == nullptr) == (ids == nullptr) && (!ids || (n_ids > 0 && vocab > 0)),
              "embed: tokens from the device need their rows and the ids (%d of them), and the vocabulary (%d)", n_ids, vocab);
  if (dtype == EMBER_F32)
    embed_kernel<float><<<T, 128, 0, stream>>>(tokens, src, ids, n_ids, vocab, positions, (const float*)table,
                                               (const float*)pos_table, x, d);
  else if (dtype == EMBER_BF16)
    embed_kernel<__nv_bfloat16><<<T, 128, 0, stream>>>(tokens, src, ids, n_ids, vocab, positions, (const __nv_bfloat16*)table,
                                                       (const __nv_bfloat16*)pos_table, x, d);
  else
    return ember_fail("embed: element type %d", dtype);
  EMBER_LAUNCH_OK("embed");
  return 0;
}

// ---------------------------------------------------------------------------- layer norm
// One warp per row.  Two passes for mean and biased variance, a third to write.  A row of up to
// 2048 values is read once and held in registers (float4 per lane), so that its loads are in
// flight together; longer or oddly sized rows are read three times.
constexpr int kRowVecs = 16;

template <typename OutT>
__device__ __forceinline__ void store4(OutT* dst, float a, float b, float c, float d);
template <>
__device__ __forceinline__ void store4<float>(float* dst, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* dst, float a, float b, float c, float d) {
  __nv_bfloat162* d2 = reinterpret_cast<__nv_bfloat162*>(dst);
  d2[0] = __floats2bfloat162_rn(a, b);
  d2[1] = __floats2bfloat162_rn(c, d);
}

// The rows were written by the kernel in front, during this kernel's life (programmatic dependent
// launch): they are read with loads that go to L2 (`__ldcg`), never through the read-only data path.
// EARLY: the gain and the bias (constants of the model; in a decode step each layer's come from
// DRAM) are fetched into registers before the kernel in front is waited for, so that they are
// not a second trip to memory after the row's statistics.  Costs registers: for a decode step's rows only.
template <typename OutT, bool EARLY>
__global__ void layernorm_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                 OutT* __restrict__ out, int rows, int d, float eps) {
  EMBER_MARK_START(kLayerNorm);
  pdl_trigger();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  float4 gm_early[EARLY ? kRowVecs : 1], bt_early[EARLY ? kRowVecs : 1];
  if (EARLY && (d & 3) == 0 && d <= 128 * kRowVecs) {
#pragma unroll
    for (int j = 0; j < kRowVecs; ++j) {
      const int i = lane + 32 * j;
      if (i < (d >> 2)) {
        gm_early[j] = reinterpret_cast<const float4*>(w)[i];
        bt_early[j] = reinterpret_cast<const float4*>(b)[i];
      }
    }
  }
  pdl_wait();
  EMBER_MARK(kLayerNorm, kDependency);
  if (row >= rows) return;
  const float* r = x + (size_t)row * d;
  OutT* o = out + (size_t)row * d;
  if ((d & 3) == 0 && d <= 128 * kRowVecs) {
    const int nv = d >> 2;
    const float4* r4 = reinterpret_cast<const float4*>(r);
    float4 v[kRowVecs];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < kRowVecs; ++j) {
      const int i = lane + 32 * j;
      v[j] = i < nv ? __ldcg(r4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    }
    const float mean = warp_sum(s) / (float)d;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < kRowVecs; ++j) {
      if (lane + 32 * j < nv) {
        const float a0 = v[j].x - mean, a1 = v[j].y - mean, a2 = v[j].z - mean, a3 = v[j].w - mean;
        q += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
      }
    }
    const float inv = 1.0f / sqrtf(warp_sum(q) / (float)d + eps);
    EMBER_MARK(kLayerNorm, kPhaseA);  // statistics taken
#pragma unroll
    for (int j = 0; j < kRowVecs; ++j) {
      const int i = lane + 32 * j;
      if (i < nv) {
        const float4 gm = EARLY ? gm_early[j] : reinterpret_cast<const float4*>(w)[i];
        const float4 bt = EARLY ? bt_early[j] : reinterpret_cast<const float4*>(b)[i];
        store4<OutT>(o + 4 * i, (v[j].x - mean) * inv * gm.x + bt.x, (v[j].y - mean) * inv * gm.y + bt.y,
                     (v[j].z - mean) * inv * gm.z + bt.z, (v[j].w - mean) * inv * gm.w + bt.w);
      }
    }
    EMBER_MARK(kLayerNorm, kEnd);
    return;
  }
  float s = 0.f;
  for (int i = lane; i < d; i += 32) s += __ldcg(r + i);
  const float mean = warp_sum(s) / (float)d;
  float q = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float c = __ldcg(r + i) - mean;
    q += c * c;
  }
  const float var = warp_sum(q) / (float)d;
  const float inv = 1.0f / sqrtf(var + eps);
  for (int i = lane; i < d; i += 32) o[i] = from_float<OutT>((__ldcg(r + i) - mean) * inv * w[i] + b[i]);
}

EMBER_API int ember_layernorm(const float* x, const float* w, const float* b, void* out, int rows, int d, float eps,
                              int out_dtype, cudaStream_t stream) {
  EMBER_CHECK(rows > 0 && d > 0, "layernorm: rows = %d, width = %d", rows, d);
  const int warps = rows <= sm_count() ? 1 : 4;  // a decode step's rows: a block each, so that they run on different SMs
  const int grid = (rows + warps - 1) / warps;
  cudaError_t e;
  const bool early = rows <= 512;  // a decode step's rows: the gain and bias come from DRAM, once per layer
  // A decode step's few blocks ask for most of an SM's shared memory, which they do not use: each then has
  // an SM to itself, away from the blocks of the product that follows, which are resident by then and
  // have an SM's way in full of their weights (a step of GPT-2 XL at batch 8: 1.231 -> 1.199 ms).
  const size_t alone = rows <= sm_count() / 4 ? (size_t)200 * 1024 : 0;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(layernorm_kernel<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(layernorm_kernel<float, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    configured = true;
  }
  if (out_dtype == EMBER_F32)
    e = early ? launch_pdl(layernorm_kernel<float, true>, dim3(grid), dim3(warps * 32), alone, stream, x, w, b, (float*)out, rows,
                           d, eps)
              : launch_pdl(layernorm_kernel<float, false>, dim3(grid), dim3(warps * 32), 0, stream, x, w, b, (float*)out, rows,
                           d, eps);
  else if (out_dtype == EMBER_BF16)
    e = early ? launch_pdl(layernorm_kernel<__nv_bfloat16, true>, dim3(grid), dim3(warps * 32), alone, stream, x, w, b,
                           (__nv_bfloat16*)out, rows, d, eps)
              : launch_pdl(layernorm_kernel<__nv_bfloat16, false>, dim3(grid), dim3(warps * 32), 0, stream, x, w, b,
                           (__nv_bfloat16*)out, rows, d, eps);
  else
    return ember_fail("layernorm: element type %d", out_dtype);
  if (e != cudaSuccess) return ember_fail("layernorm: %s", cudaGetErrorString(e));
  return 0;
}

// ---------------------------------------------------------------------------- tokens sampled on the device
// A step whose tokens are the ids an earlier step's sampler drew takes them where they are:
// tokens[i] = ids[src[i]] where src[i] >= 0 (else the host's token stays).  The host can then
// queue the step before it has read those ids itself.
__global__ void take_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ src, const int* __restrict__ ids, int n,
                                   int n_ids, int vocab) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int r = src[i];
  if (r < 0 || r >= n_ids) return;
  const int t = ids[r];
  tokens[i] = (t >= 0 && t < vocab) ? t : 0;  // a sampler's id is always in range; nothing else may reach the table
}

EMBER_API int ember_take_tokens(int* tokens, const int* src, const int* ids, int n, int n_ids, int vocab,
                                cudaStream_t stream) {
  EMBER_CHECK(n > 0 && n_ids > 0 && vocab > 0, "take_tokens: %d tokens from %d ids, vocabulary %d", n, n_ids, vocab);
  take_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(tokens, src, ids, n, n_ids, vocab);
  EMBER_LAUNCH_OK("take_tokens");
  return 0;
}

// ---------------------------------------------------------------------------- row gather
__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, float* __restrict__ out,
                                   int d) {
  const float* src = x + (size_t)rows[blockIdx.x] * d;
  float* dst = out + (size_t)blockIdx.x * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = src[i];
}

EMBER_API int ember_gather_rows(const float* x, const int* rows, float* out, int n_rows, int d, cudaStream_t stream) {
  EMBER_CHECK(n_rows > 0 && d > 0, "gather_rows: rows = %d, width = %d", n_rows, d);
  gather_rows_kernel<<<n_rows, 128, 0, stream>>>(x, rows, out, d);
  EMBER_LAUNCH_OK("gather_rows");
  return 0;
}

// ---------------------------------------------------------------------------- activation in place
// For the activation that the library product has no epilogue for (the erf GELU on the bfloat16
// path): y = act(y), the bias already added by the product.
template <typename T>
__global__ void act_kernel(T* __restrict__ y, size_t n, int act) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = from_float<T>(apply_act(to_float(y[i]), act));
}

EMBER_API int ember_act_inplace(void* y, size_t n, int act, int dtype, cudaStream_t stream) {
  EMBER_CHECK(n > 0, "activation: no elements");
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (dtype == EMBER_F32)
    act_kernel<float><<<grid, 256, 0, stream>>>((float*)y, n, act);
  else if (dtype == EMBER_BF16)
    act_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((__nv_bfloat16*)y, n, act);
  else
    return ember_fail("activation: element type %d", dtype);
  EMBER_LAUNCH_OK("activation");
  return 0;
}

// y <- scale * y, then (cap > 0) cap * tanh(y / cap): a factor on the embedded rows, a cap on the logits.
__global__ void scale_cap_kernel(float* __restrict__ y, size_t n, float scale, float cap) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = y[i] * scale;
  if (cap > 0.f) v = cap * tanhf(v / cap);
  y[i] = v;
}

EMBER_API int ember_scale_cap_inplace(float* y, size_t n, float scale, float cap, cudaStream_t stream) {
  EMBER_CHECK(n > 0 && cap >= 0.f, "scale_cap: %zu values, cap %g", n, (double)cap);
  scale_cap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(y, n, scale, cap);
  EMBER_LAUNCH_OK("scale_cap");
  return 0;
}

EMBER_TIMELINE_READER(elementwise)
