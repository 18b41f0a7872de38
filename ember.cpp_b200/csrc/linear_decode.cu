// The linear layers of a decode step in bfloat16: Y[M,N] = X[M,K] . W[N,K]^T for a handful of rows
// (M <= 16), a kernel that streams the weight matrix once, with the layer norm before it and the
// bias, GELU and residual sum after it in the same launch.
//
// ember.cpp runs a decode step's products as cublasSgemm with one column and then separate bias,
// GELU and add kernels, about 17 launches a layer (graph_ir.cpp:3824-3834; graph_ir_cuda.cu:67-76,
// 230-242), each a full pass over its vector.  Here a layer's four products are four launches and
// nothing else touches the activations in between.
//
// The product runs on the tensor cores with the operands swapped: the 16 rows of an mma.sync
// m16n8k16 tile are 16 output features (weight rows), its 8 columns are 8 sequences of the batch.
// Each lane loads 16 bytes (8 consecutive k) of weight rows g and g+8 straight from global memory:
// those registers are the A fragments of two MMAs under a fixed relabelling of k inside a 32-wide
// slice, and the matching 8 values of X for sequence g, relabelled the same way, are the B
// fragment.
//
// Work is cut so that a few-megabyte matrix still occupies the whole chip: a tile is 16 weight
// rows; a thread-block cluster of 1, 2 or 4 blocks shares a tile and splits K between its blocks;
// inside a block 8 warps take interleaved slices.  Warps are summed in shared memory in warp order,
// the cluster's blocks are summed in block order through distributed shared memory into block 0,
// which applies the epilogue: no atomics, so a result does not depend on timing.
//
// The kernel is launched with programmatic stream serialization: it asks for its first weight
// slices at once and only then waits for the kernel before it (griddepcontrol.wait), so that
// weights stream while the producer of X is still finishing.  Nothing is written before the wait.
//
// Input modes: float32 rows with a layer norm (statistics in float32 per row, the normalised
// slice rounded to bfloat16 into shared memory, the values the separate norm kernel writes), or
// bfloat16 rows read as they are.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace {

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {  // weights are read once: do not keep them in L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

constexpr int kWarps = 8;
constexpr int kDepth = 4;  // weight slices a warp keeps in flight

// MT: batch tiles of 8 sequences (1 or 2).  LN: float32 input with a fused layer norm.
template <int MT, bool LN>
__global__ void __launch_bounds__(kWarps * 32, 3)
linear_decode_kernel(const void* __restrict__ xin, const float* __restrict__ gamma, const float* __restrict__ beta,
                     float eps, const __nv_bfloat16* __restrict__ W, const float* __restrict__ bias,
                     const float* residual, void* out, int M, int N, int K, int act, int out_f32, int k_split) {
  constexpr int U = kDepth;
  constexpr int kTile = 16 * 8 * MT;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int rank = blockIdx.x % k_split;  // this block's place in its cluster
  const int row0 = (blockIdx.x / k_split) * 16;
  // this block's share of the 32-wide slices of K
  const int all_steps = (K + 31) / 32;
  const int per_block = (all_steps + k_split - 1) / k_split;
  const int step_lo = rank * per_block, step_hi = min(all_steps, step_lo + per_block);
  const int k_lo = step_lo * 32;
  // shared memory: [red: kWarps x kTile][gather: k_split x kTile][xs: M x ldx bf16 (LN only)]
  float* red = reinterpret_cast<float*>(smem_raw);
  float* gather = red + kWarps * kTile;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(gather + k_split * kTile);
  const int ldx = per_block * 32 + 8;

  // weight rows of this lane; rows past N read row N-1 and are dropped at the end
  const __nv_bfloat16* w_lo = W + (size_t)min(row0 + g, N - 1) * K + c * 8;
  const __nv_bfloat16* w_hi = W + (size_t)min(row0 + g + 8, N - 1) * K + c * 8;

  // The first weight slices are asked for before anything else: they do not depend on the kernel
  // before this one, whose completion is awaited only after that.
  uint4 wl[U], wh[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int s = step_lo + warp + u * kWarps;
    const bool ok = s < step_hi && s * 32 + c * 8 < K;
    wl[u] = ok ? ldg_stream(w_lo + s * 32) : make_uint4(0, 0, 0, 0);
    wh[u] = ok ? ldg_stream(w_hi + s * 32) : make_uint4(0, 0, 0, 0);
  }
  if (LN) {
    // the norm's gain and bias are constants too: bring their lines into L1 now, so that the third
    // pass over a row finds them there
    const int lines = (K * (int)sizeof(float) + 127) / 128;
    for (int i = threadIdx.x; i < 2 * lines; i += kWarps * 32) {
      const float* p = (i < lines ? gamma : beta) + (size_t)(i % lines) * 32;
      asm volatile("prefetch.global.L1 [%0];\n" ::"l"(p));
    }
  }
  pdl_trigger();
  pdl_wait();

  uint4 xb[LN ? 1 : U][MT];
  if (!LN) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int s = step_lo + warp + u * kWarps;
      const int k = s * 32 + c * 8;
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        const int m = t * 8 + g;
        xb[u][t] = (s < step_hi && k < K && m < M)
                       ? *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(xin) + (size_t)m * K + k)
                       : make_uint4(0, 0, 0, 0);
      }
    }
  }
  // the element of the output tile that this thread finishes (block 0 of the cluster only)
  const int e_r = threadIdx.x % 16, e_m = threadIdx.x / 16;
  const int e_n = row0 + e_r;
  const bool e_ok = rank == 0 && threadIdx.x < kTile && e_m < M && e_n < N;
  const float e_bias = (e_ok && bias) ? bias[e_n] : 0.f;
  const float e_res = (e_ok && residual) ? residual[(size_t)e_m * N + e_n] : 0.f;

  if (LN) {
    const float* x = static_cast<const float*>(xin);
    const int k_hi = min(K, step_hi * 32);
    // One warp per row: mean, then biased variance over the whole row, then this block's slice of
    // the normalised row in bfloat16.  The row is read three times; after the first from L1.
    for (int m = warp; m < M; m += kWarps) {
      __nv_bfloat16* dst = xs + m * ldx;
      const float* r = x + (size_t)m * K;
      float mean, inv;
      if ((K & 3) == 0) {
        const int nv = K >> 2;
        const float4* r4 = reinterpret_cast<const float4*>(r);
        float sum = 0.f;
#pragma unroll 4
        for (int i = lane; i < nv; i += 32) {
          const float4 v = r4[i];
          sum += (v.x + v.y) + (v.z + v.w);
        }
        mean = warp_sum(sum) / (float)K;
        float sq = 0.f;
#pragma unroll 4
        for (int i = lane; i < nv; i += 32) {
          const float4 v = r4[i];
          const float a0 = v.x - mean, a1 = v.y - mean, a2 = v.z - mean, a3 = v.w - mean;
          sq += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
        }
        inv = 1.0f / sqrtf(warp_sum(sq) / (float)K + eps);
      } else {
        float sum = 0.f;
        for (int i = lane; i < K; i += 32) sum += r[i];
        mean = warp_sum(sum) / (float)K;
        float sq = 0.f;
        for (int i = lane; i < K; i += 32) {
          const float dlt = r[i] - mean;
          sq += dlt * dlt;
        }
        inv = 1.0f / sqrtf(warp_sum(sq) / (float)K + eps);
      }
      // k_lo is a multiple of 32 and K of 8, so the slice is whole groups of 4
      for (int i = k_lo + lane * 4; i < k_hi; i += 128) {
        const float4 v = *reinterpret_cast<const float4*>(r + i);
        const float4 gm = *reinterpret_cast<const float4*>(gamma + i), bt = *reinterpret_cast<const float4*>(beta + i);
        __nv_bfloat162* d2 = reinterpret_cast<__nv_bfloat162*>(dst + (i - k_lo));
        d2[0] = __floats2bfloat162_rn((v.x - mean) * inv * gm.x + bt.x, (v.y - mean) * inv * gm.y + bt.y);
        d2[1] = __floats2bfloat162_rn((v.z - mean) * inv * gm.z + bt.z, (v.w - mean) * inv * gm.w + bt.w);
      }
    }
    __syncthreads();
  }

  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[t][j] = 0.f;

  for (int s0 = step_lo + warp; s0 < step_hi; s0 += U * kWarps) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int s = s0 + u * kWarps;
      const int k = s * 32 + c * 8;
      const uint4 a_lo = wl[u], a_hi = wh[u];
      uint4 b[MT];
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        if (LN)
          b[t] = (s < step_hi && k < K && t * 8 + g < M)
                     ? *reinterpret_cast<const uint4*>(xs + (t * 8 + g) * ldx + (k - k_lo))
                     : make_uint4(0, 0, 0, 0);
        else
          b[t] = xb[u][t];
      }
      // refill this slot with the slice U rounds ahead
      const int sn = s + U * kWarps;
      const int kn = sn * 32 + c * 8;
      const bool okn = sn < step_hi && kn < K;
      wl[u] = okn ? ldg_stream(w_lo + sn * 32) : make_uint4(0, 0, 0, 0);
      wh[u] = okn ? ldg_stream(w_hi + sn * 32) : make_uint4(0, 0, 0, 0);
      if (!LN) {
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          const int m = t * 8 + g;
          xb[u][t] = (okn && m < M)
                         ? *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(xin) + (size_t)m * K + kn)
                         : make_uint4(0, 0, 0, 0);
        }
      }
      if (s >= step_hi) continue;  // uniform across the warp
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        mma_bf16(acc[t], a_lo.x, a_hi.x, a_lo.y, a_hi.y, b[t].x, b[t].y);
        mma_bf16(acc[t], a_lo.z, a_hi.z, a_lo.w, a_hi.w, b[t].z, b[t].w);
      }
    }
  }

  // warps -> block: tile element (weight row r, sequence m) at [r * 8*MT + m], summed in warp order
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    float* mine = red + warp * kTile + t * 8;
    mine[g * (8 * MT) + c * 2] = acc[t][0];
    mine[g * (8 * MT) + c * 2 + 1] = acc[t][1];
    mine[(g + 8) * (8 * MT) + c * 2] = acc[t][2];
    mine[(g + 8) * (8 * MT) + c * 2 + 1] = acc[t][3];
  }
  __syncthreads();
  float v = 0.f;
  const int e_at = e_r * (8 * MT) + e_m;
  if (threadIdx.x < kTile)
    for (int w = 0; w < kWarps; ++w) v += red[w * kTile + e_at];

  // blocks -> block 0 of the cluster, summed in block order
  if (k_split > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    if (rank != 0 && threadIdx.x < kTile) cluster.map_shared_rank(gather, 0)[rank * kTile + e_at] = v;
    cluster.sync();
    if (rank != 0) return;
    if (threadIdx.x < kTile)
      for (int b = 1; b < k_split; ++b) v += gather[b * kTile + e_at];
  }
  if (e_ok) {
    if (bias) v += e_bias;
    v = apply_act(v, act);
    if (residual) v = e_res + v;
    const size_t at = (size_t)e_m * N + e_n;
    if (out_f32)
      static_cast<float*>(out)[at] = v;
    else
      static_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(v);
  }
}

template <int MT, bool LN>
int launch(const void* xin, const float* gamma, const float* beta, float eps, const void* W, const float* bias,
           const float* residual, void* out, int M, int N, int K, int act, int out_dtype, cudaStream_t stream) {
  const int tiles = (N + 15) / 16;
  const int all_steps = (K + 31) / 32;
  // split K over a cluster while the blocks still fit the chip at once (three to an SM) and each
  // block keeps at least two slices per warp
  int k_split = 1;
  while (k_split < 4 && tiles * k_split * 2 <= 3 * 148 && all_steps / (k_split * 2) >= 2 * kWarps) k_split *= 2;
  const int per_block = (all_steps + k_split - 1) / k_split;
  size_t smem = (size_t)(kWarps + k_split) * 16 * 8 * MT * sizeof(float);
  if (LN) smem += (size_t)M * (per_block * 32 + 8) * sizeof(__nv_bfloat16);
  if (smem > 200 * 1024)
    return ember_fail("linear_decode: a fused norm over K = %d needs %zu bytes of shared memory", K, smem);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(linear_decode_kernel<MT, LN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return ember_fail("linear_decode: %s", cudaGetErrorString(e));
    configured = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * k_split);
  cfg.blockDim = dim3(kWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[0].val.programmaticStreamSerializationAllowed = pdl_allowed();
  attrs[1].id = cudaLaunchAttributeClusterDimension;
  attrs[1].val.clusterDim.x = k_split;
  attrs[1].val.clusterDim.y = 1;
  attrs[1].val.clusterDim.z = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 2;
  const int out_f32 = out_dtype == EMBER_F32;
  cudaError_t e = cudaLaunchKernelEx(&cfg, linear_decode_kernel<MT, LN>, xin, gamma, beta, eps,
                                     (const __nv_bfloat16*)W, bias, residual, out, M, N, K, act, out_f32, k_split);
  if (e != cudaSuccess) return ember_fail("linear_decode: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace

// xin: float32 [M,K] when gamma is given (layer norm fused), else bfloat16 [M,K].
// residual: float32 [M,N] or null; it may be the output buffer.  out: float32 or bfloat16 [M,N].
EMBER_API int ember_linear_decode(const void* xin, const float* gamma, const float* beta, float eps, const void* W,
                                  const float* bias, const float* residual, void* out, int M, int N, int K, int act,
                                  int out_dtype, cudaStream_t stream) {
  EMBER_CHECK(M > 0 && M <= 16 && N > 0 && K > 0, "linear_decode: M = %d (at most 16), N = %d, K = %d", M, N, K);
  EMBER_CHECK(K % 8 == 0, "linear_decode: K = %d is not a multiple of 8 (16-byte rows)", K);
  EMBER_CHECK(act >= 0 && act <= 2, "linear_decode: activation %d", act);
  EMBER_CHECK(out_dtype == EMBER_F32 || out_dtype == EMBER_BF16, "linear_decode: output type %d", out_dtype);
  EMBER_CHECK(!residual || out_dtype == EMBER_F32, "linear_decode: a residual sum needs a float32 output");
  EMBER_CHECK((gamma == nullptr) == (beta == nullptr), "linear_decode: give both norm parameters or neither");
  const bool ln = gamma != nullptr;
  if (M <= 8)
    return ln ? launch<1, true>(xin, gamma, beta, eps, W, bias, residual, out, M, N, K, act, out_dtype, stream)
              : launch<1, false>(xin, gamma, beta, eps, W, bias, residual, out, M, N, K, act, out_dtype, stream);
  return ln ? launch<2, true>(xin, gamma, beta, eps, W, bias, residual, out, M, N, K, act, out_dtype, stream)
            : launch<2, false>(xin, gamma, beta, eps, W, bias, residual, out, M, N, K, act, out_dtype, stream);
}
