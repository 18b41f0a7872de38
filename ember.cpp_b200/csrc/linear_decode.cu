// The linear layers of a decode step in bfloat16: Y[M,N] = X[M,K] . W[N,K]^T for a handful of rows
// (M <= 16), a kernel that streams the weight matrix once at memory speed, with the layer norm
// before it and the bias, GELU and residual sum after it in the same launch.
//
// ember.cpp runs a decode step's products as cublasSgemm with one column and then separate bias,
// GELU and add kernels, about 17 launches a layer (graph_ir.cpp:3824-3834; graph_ir_cuda.cu:67-76,
// 230-242), each a full pass over its vector.  Here a layer's four products are four launches and
// nothing else touches the activations in between.
//
// The product runs on the tensor cores with the operands swapped: the 16 rows of an mma.sync
// m16n8k16 tile are 16 output features (weight rows), its 8 columns are 8 sequences of the batch.
// A block owns 16 weight rows over the whole of K; its warps take interleaved 32-wide slices of K.
// Each lane loads 16 bytes (8 consecutive k) of weight rows g and g+8 straight from global memory:
// those registers are the A fragments of two MMAs under a fixed relabelling of k inside the slice,
// and the matching 8 values of X for sequence g, relabelled the same way, are the B fragment.  The
// warps' partial tiles are summed in shared memory in warp order, so a result does not depend on
// timing.
//
// Input modes: float32 rows with a layer norm (statistics in float32 per row, the normalised row
// rounded to bfloat16 into shared memory, exactly what the separate norm kernel writes), or
// bfloat16 rows read as they are.
#include "common.cuh"

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

constexpr int kUnroll = 4;
constexpr int kRowVecs = 16;  // float4 per lane that a row held in registers may take (K <= 2048)

// MT: batch tiles of 8 sequences (1 or 2).  LN: float32 input with a fused layer norm.
template <int MT, bool LN>
__global__ void __launch_bounds__(512)
linear_decode_kernel(const void* __restrict__ xin, const float* __restrict__ gamma, const float* __restrict__ beta,
                     float eps, const __nv_bfloat16* __restrict__ W, const float* __restrict__ bias,
                     const float* residual, void* out, int M, int N, int K, int act, int out_f32) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int n_warps = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int row0 = blockIdx.x * 16;
  const int n_steps = (K + 31) / 32;
  // shared memory: [red: n_warps x 16 x 8*MT floats][xs: 8*MT x (K + 8) bf16 (LN only)]
  float* red = reinterpret_cast<float*>(smem_raw);
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(red + n_warps * 16 * 8 * MT);
  const int ldx = K + 8;

  // weight rows of this lane; rows past N read row N-1 and are dropped at the end
  const __nv_bfloat16* w_lo = W + (size_t)min(row0 + g, N - 1) * K + c * 8;
  const __nv_bfloat16* w_hi = W + (size_t)min(row0 + g + 8, N - 1) * K + c * 8;

  // the first weight loads go out before anything else, so that they fly during the norm
  uint4 wl[kUnroll], wh[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int s = warp + u * n_warps;
    const bool ok = s < n_steps && s * 32 + c * 8 < K;
    wl[u] = ok ? ldg_stream(w_lo + s * 32) : make_uint4(0, 0, 0, 0);
    wh[u] = ok ? ldg_stream(w_hi + s * 32) : make_uint4(0, 0, 0, 0);
  }

  if (LN) {
    const float* x = static_cast<const float*>(xin);
    // one warp per row: mean and biased variance in two passes over the row, which is held in
    // registers when it fits, then the normalised row in bfloat16
    for (int m = warp; m < 8 * MT; m += n_warps) {
      __nv_bfloat16* dst = xs + m * ldx;
      if (m >= M) {
        for (int i = lane; i < K; i += 32) dst[i] = __float2bfloat16_rn(0.f);
        continue;
      }
      const float* r = x + (size_t)m * K;
      if ((K & 3) == 0 && K <= 128 * kRowVecs) {
        const int nv = K >> 2;
        const float4* r4 = reinterpret_cast<const float4*>(r);
        float4 v[kRowVecs];
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < kRowVecs; ++j) {
          const int i = lane + 32 * j;
          v[j] = i < nv ? r4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
          sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        }
        const float mean = warp_sum(sum) / (float)K;
        float sq = 0.f;
#pragma unroll
        for (int j = 0; j < kRowVecs; ++j) {
          if (lane + 32 * j < nv) {
            const float a0 = v[j].x - mean, a1 = v[j].y - mean, a2 = v[j].z - mean, a3 = v[j].w - mean;
            sq += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
          }
        }
        const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)K + eps);
#pragma unroll
        for (int j = 0; j < kRowVecs; ++j) {
          const int i = lane + 32 * j;
          if (i < nv) {
            const float4 gm = reinterpret_cast<const float4*>(gamma)[i], bt = reinterpret_cast<const float4*>(beta)[i];
            __nv_bfloat162* d2 = reinterpret_cast<__nv_bfloat162*>(dst + 4 * i);
            d2[0] = __floats2bfloat162_rn((v[j].x - mean) * inv * gm.x + bt.x, (v[j].y - mean) * inv * gm.y + bt.y);
            d2[1] = __floats2bfloat162_rn((v[j].z - mean) * inv * gm.z + bt.z, (v[j].w - mean) * inv * gm.w + bt.w);
          }
        }
      } else {
        float sum = 0.f;
        for (int i = lane; i < K; i += 32) sum += r[i];
        const float mean = warp_sum(sum) / (float)K;
        float sq = 0.f;
        for (int i = lane; i < K; i += 32) {
          const float dlt = r[i] - mean;
          sq += dlt * dlt;
        }
        const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)K + eps);
        for (int i = lane; i < K; i += 32) dst[i] = __float2bfloat16_rn((r[i] - mean) * inv * gamma[i] + beta[i]);
      }
    }
    __syncthreads();
  }

  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[t][j] = 0.f;

  for (int s0 = warp; s0 < n_steps; s0 += kUnroll * n_warps) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int s = s0 + u * n_warps;
      const int k = s * 32 + c * 8;
      const bool ok = s < n_steps && k < K;
      const uint4 a_lo = wl[u], a_hi = wh[u];
      // refill this slot with the slice four rounds ahead
      const int sn = s + kUnroll * n_warps;
      const bool okn = sn < n_steps && sn * 32 + c * 8 < K;
      wl[u] = okn ? ldg_stream(w_lo + sn * 32) : make_uint4(0, 0, 0, 0);
      wh[u] = okn ? ldg_stream(w_hi + sn * 32) : make_uint4(0, 0, 0, 0);
      if (s >= n_steps) continue;  // uniform across the warp
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        const int m = t * 8 + g;
        uint4 b = make_uint4(0, 0, 0, 0);
        if (ok) {
          if (LN)
            b = *reinterpret_cast<const uint4*>(xs + m * ldx + k);
          else if (m < M)
            b = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(xin) + (size_t)m * K + k);
        }
        mma_bf16(acc[t], a_lo.x, a_hi.x, a_lo.y, a_hi.y, b.x, b.y);
        mma_bf16(acc[t], a_lo.z, a_hi.z, a_lo.w, a_hi.w, b.z, b.w);
      }
    }
  }

  // partial tiles -> shared memory; tile element (weight row r, sequence m) at red[warp][r][m]
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    float* mine = red + (warp * 16) * (8 * MT) + t * 8;
    mine[g * (8 * MT) + c * 2] = acc[t][0];
    mine[g * (8 * MT) + c * 2 + 1] = acc[t][1];
    mine[(g + 8) * (8 * MT) + c * 2] = acc[t][2];
    mine[(g + 8) * (8 * MT) + c * 2 + 1] = acc[t][3];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < 16 * 8 * MT; e += blockDim.x) {
    const int r = e % 16, m = e / 16;  // consecutive threads: consecutive output features
    const int n = row0 + r;
    if (m >= M || n >= N) continue;
    float v = 0.f;
    for (int w = 0; w < n_warps; ++w) v += red[(w * 16 + r) * (8 * MT) + m];
    if (bias) v += bias[n];
    v = apply_act(v, act);
    const size_t at = (size_t)m * N + n;
    if (residual) v = residual[at] + v;
    if (out_f32)
      static_cast<float*>(out)[at] = v;
    else
      static_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(v);
  }
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
  const int mt = M <= 8 ? 1 : 2;
  const int tiles = (N + 15) / 16;
  const int n_warps = tiles < 2 * 148 ? 16 : 8;  // few row tiles: more warps each, to keep enough loads in flight
  size_t smem = (size_t)n_warps * 16 * 8 * mt * sizeof(float);
  if (ln) smem += (size_t)8 * mt * (K + 8) * sizeof(__nv_bfloat16);
  EMBER_CHECK(smem <= 200 * 1024, "linear_decode: a fused norm over K = %d needs %zu bytes of shared memory", K, smem);
#define EMBER_LD(MT, LN)                                                                                              \
  do {                                                                                                                \
    static size_t configured = 0;                                                                                     \
    if (smem > 48 * 1024 && smem > configured) {                                                                      \
      cudaError_t e = cudaFuncSetAttribute(linear_decode_kernel<MT, LN>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                                                \
      if (e != cudaSuccess) return ember_fail("linear_decode: %s", cudaGetErrorString(e));                            \
      configured = smem;                                                                                              \
    }                                                                                                                 \
    linear_decode_kernel<MT, LN><<<tiles, n_warps * 32, smem, stream>>>(                                              \
        xin, gamma, beta, eps, (const __nv_bfloat16*)W, bias, residual, out, M, N, K, act, out_dtype == EMBER_F32);   \
  } while (0)
  if (mt == 1 && ln) EMBER_LD(1, true);
  else if (mt == 1) EMBER_LD(1, false);
  else if (ln) EMBER_LD(2, true);
  else EMBER_LD(2, false);
#undef EMBER_LD
  EMBER_LAUNCH_OK("linear_decode");
  return 0;
}
