// The matrix product of the true 32-bit path: Y[M,N] = A[M,K] . W[N,K]^T (+ bias, activation,
// residual), float32 operands, FFMA on the CUDA cores, no reduced-precision matrix mode.
//
// ember.cpp's interpreter is float32 throughout (cublasSgemm in default math, then a bias kernel,
// graph_ir.cpp:3824-3834, cuda_kernels.cu:3617-3621), and its CPU form adds each dot product in a
// fixed order so that a row decoded alone equals the same row of a whole prompt
// (cpu_dot.h:13-21).  This kernel keeps that property on the GPU: every output element is one
// chain of fused multiply-adds over k = 0 .. K-1 in ascending order, whatever M, the tile or the
// batch, so logits do not depend on how tokens were cut into steps.  It is slow by design.
#include "common.cuh"

constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                const float* residual, float* out, int M, int N, int K, int act) {
  __shared__ float As[BK][BM + 1];
  __shared__ float Ws[BK][BN + 1];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int i = tid; i < BM * BK; i += 256) {
      const int r = i / BK, c = i % BK;
      const int m = m0 + r, k = k0 + c;
      As[c][r] = (m < M && k < K) ? A[(size_t)m * K + k] : 0.f;
      const int n = n0 + r;
      Ws[c][r] = (n < N && k < K) ? W[(size_t)n * K + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tn + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + tm + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tn + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      v = apply_act(v, act);
      if (residual) v = residual[(size_t)m * N + n] + v;
      out[(size_t)m * N + n] = v;
    }
  }
}

// residual may alias out (the residual stream is updated in place).
EMBER_API int ember_gemm_f32(const float* A, const float* W, const float* bias, const float* residual, float* out,
                             int M, int N, int K, int act, cudaStream_t stream) {
  EMBER_CHECK(M > 0 && N > 0 && K > 0, "gemm_f32: M = %d, N = %d, K = %d", M, N, K);
  EMBER_CHECK(act >= 0 && act <= 2, "gemm_f32: activation %d", act);
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  EMBER_CHECK(grid.y <= 65535, "gemm_f32: %d rows are more than one launch takes", M);
  gemm_f32_kernel<<<grid, 256, 0, stream>>>(A, W, bias, residual, out, M, N, K, act);
  EMBER_LAUNCH_OK("gemm_f32");
  return 0;
}
