// The linear layers of a decode step in bfloat16: Y[M,N] = X[M,K] . W[N,K]^T for a handful of rows
// (M <= 16), a kernel that streams the weight matrix once, with the bias, GELU and residual sum
// after it in the same launch.
//
// ember.cpp runs a decode step's products as cublasSgemm with one column and then separate bias,
// GELU and add kernels, about 17 launches a layer (graph_ir.cpp:3824-3834; graph_ir_cuda.cu:67-76,
// 230-242), each a full pass over its vector.  Here a layer's four products are four launches and
// nothing else touches the activations in between.
//
// The product runs on the tensor cores with the operands swapped: the 16 rows of an mma.sync
// m16n8k16 tile are 16 output features (weight rows), its 8 columns are 8 sequences of the batch.
// Under a fixed relabelling of k inside a 32-wide slice, 16 consecutive bytes of weight rows g and
// g+8 are the A fragments of two MMAs and the matching 8 values of X for sequence g are the B
// fragment, so no value is shuffled between lanes.
//
// Work is cut so that a few-megabyte matrix still occupies the whole chip: a tile is 16 weight
// rows; a thread-block cluster of 1, 2 or 4 blocks shares a tile and splits K between its blocks.
// A block asks for its whole share of the matrix at once (bulk copies into shared memory, a row of
// the tile each, about 50 KB, three blocks to an SM), so the matrix is in flight from the first instruction and the
// kernel runs at the speed of HBM, not of its own round trips.  Inside a block 8 warps take
// interleaved slices; warps are summed in shared memory in warp order, the cluster's blocks in
// block order through distributed shared memory into block 0, which applies the epilogue: no
// atomics, so a result does not depend on timing.
//
// The kernel is launched with programmatic stream serialization: the weight copies are issued
// first, and only then does it wait for the kernel before it (griddepcontrol.wait), so that
// weights stream while the producer of X is still finishing.  Nothing is written to global memory
// before the wait.  What that producer wrote (X, the residual) is read with loads that go to L2
// (`__ldcg`) or explicitly through L1 (`ld.global.ca`), never with plain loads that the compiler
// may send through the read-only data path: this kernel's life began before the producer's ended,
// and that path can hold what was there before.
//
// (Two ways of taking the layer norm out of the step's chain of launches were built and measured here
// and removed: the norm inside this kernel's prologue, every block norming all the rows again, 0.683
// against 0.586 ms for 12 layers; and the norm in this kernel's tail, by the block that finishes last,
// 2.08 against 1.44 ms a step.  While the separate norm kernel runs, the next product's blocks are all
// resident and their weights on the way; without it they wait for them later.)
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

__device__ int g_gave_up = 0;  // set when a block's wait for its weight copies ran out

// 16 bytes of what the kernel in front wrote, through L1 (blocks of one SM read the same rows) but
// never through the read-only data path.
__device__ __forceinline__ uint4 ld_ca(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

constexpr int kWarps = 8;

// Row stride of the weight tile in shared memory, in elements: the slice plus a pad that puts
// consecutive rows 64 bytes apart modulo 128, so that the 16-byte reads of a quarter warp (two rows,
// four chunks each) fall into distinct banks.
__host__ __device__ inline int tile_stride(int per_block) { return per_block * 32 + ((per_block & 1) ? 0 : 32); }

struct Warm {  // null / 0: nothing
  const char* at;            // constants of a kernel that runs soon (the next product's weights) ...
  unsigned long long bytes;  // ... a multiple of 16, which this launch's blocks ask into L2, a share each
};

// MT: batch tiles of 8 sequences (1 or 2).
template <int MT>
__global__ void __launch_bounds__(kWarps * 32, 3)
linear_decode_kernel(const __nv_bfloat16* __restrict__ xin, const __nv_bfloat16* __restrict__ W,
                     const float* __restrict__ bias, const float* residual, void* out, int M, int N, int K, int act,
                     int out_f32, int k_split, const Warm warm) {
  constexpr int kTile = 16 * 8 * MT;
  EMBER_MARK_START(kLinearDecode);
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
  const int ldw = tile_stride(per_block);
  // shared memory: [wt: 16 x ldw bf16][red: kWarps x kTile][gather: k_split x kTile]
  __nv_bfloat16* wt = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  float* red = reinterpret_cast<float*>(wt + 16 * ldw);
  float* gather = red + kWarps * kTile;

  // The block's whole share of the matrix is asked for before anything else: it does not depend
  // on the kernel before this one, whose completion is awaited only after that.  Sixteen bulk
  // copies, a row of the tile each, issued by sixteen lanes and counted on one mbarrier: no
  // per-16-byte address arithmetic, and the whole share is in flight a few cycles after the block
  // starts.  (Rows past N repeat the last row and are dropped at the end; values of K past the
  // matrix's width are zeroed by hand: a bulk copy cannot.)
  __shared__ unsigned long long s_bar;
  const unsigned bar = (unsigned)__cvta_generic_to_shared(&s_bar);
  const int k_hi = min(K, step_hi * 32);                      // one past the last value of K this block holds
  const unsigned row_bytes = (unsigned)max(0, k_hi - k_lo) * 2;  // a multiple of 16: K is a multiple of 8
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar));
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  if (warp == 0) {
    if (lane == 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(16u * row_bytes) : "memory");
    __syncwarp();
    if (lane < 16 && row_bytes) {
      const int row = min(row0 + lane, N - 1);
      const unsigned dst = (unsigned)__cvta_generic_to_shared(wt + lane * ldw);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
                   "l"(W + (size_t)row * K + k_lo), "r"(row_bytes), "r"(bar)
                   : "memory");
    }
  }
  {
    const int tail = (step_hi - step_lo) * 32 - (k_hi - k_lo);  // values past K in the block's last slice
    for (int i = threadIdx.x; i < 16 * tail; i += kWarps * 32)
      wt[(i / tail) * ldw + (k_hi - k_lo) + i % tail] = __float2bfloat16_rn(0.f);
  }
  pdl_trigger();
  // the element of the output tile that this thread finishes (block 0 of the cluster only); its
  // bias is a constant of the model and is fetched before the wait (in a decode step it comes from
  // DRAM: after the wait it would be the longest of the loads the epilogue waits for)
  const int e_r = threadIdx.x % 16, e_m = threadIdx.x / 16;
  const int e_n = row0 + e_r;
  const bool e_ok = rank == 0 && threadIdx.x < kTile && e_m < M && e_n < N;
  const float e_bias = (e_ok && bias) ? bias[e_n] : 0.f;
  if (warm.at && warp == 1) {
    // A product whose blocks cannot be resident beside this one's (shared memory) starts to stream
    // its weights only when these blocks leave.  Asked into L2 once this block's own weights have
    // landed (they are needed first, and DRAM is idle after them), they come from there.
    unsigned done = 0;
    for (unsigned spin = 0; !done && spin < (1u << 24); ++spin)
      asm volatile(
          "{\n.reg .pred p;\n"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n"
          "selp.u32 %0, 1, 0, p;\n}\n"
          : "=r"(done)
          : "r"(bar)
          : "memory");
    constexpr unsigned kPiece = 8192;
    const unsigned long long share = ((warm.bytes + gridDim.x - 1) / gridDim.x + 15) / 16 * 16;
    const unsigned long long lo = share * blockIdx.x, hi = min(warm.bytes, lo + share);
    for (unsigned long long at = lo + (unsigned long long)lane * kPiece; at < hi; at += 32ull * kPiece) {
      const unsigned n = (unsigned)min((unsigned long long)kPiece, hi - at);
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(warm.at + at), "r"(n) : "memory");
    }
  }
  pdl_wait();
  EMBER_MARK(kLinearDecode, kDependency);

  const float e_res = (e_ok && residual) ? __ldcg(residual + (size_t)e_m * N + e_n) : 0.f;

  // the weights have landed (a wait with a limit: a copy that never completes must not hang the GPU)
  auto wait_for_weights = [&]() {
    unsigned done = 0;
    for (unsigned spin = 0; !done && spin < (1u << 24); ++spin)
      asm volatile(
          "{\n.reg .pred p;\n"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n"
          "selp.u32 %0, 1, 0, p;\n}\n"
          : "=r"(done)
          : "r"(bar)
          : "memory");
    if (!done) g_gave_up = 1;  // the results of this launch are not valid; the host asks with ember_linear_decode_status
    __syncthreads();
    EMBER_MARK(kLinearDecode, kPhaseA);  // weights landed
  };

  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[t][j] = 0.f;

  constexpr int kMaxSlices = 7;
  if (MT == 1 && per_block <= kMaxSlices * kWarps) {
    // All of this warp's activations (8 values of row g for each of its slices) are asked for at
    // once, before the weights are waited for: one trip to L2 on the step's chain of dependent
    // waits instead of one for every two slices.  (Up to 56 slices a block, 7 a warp: every K up to
    // 6,912; wider matrices take the loop below.)
    uint4 xr[kMaxSlices];
#pragma unroll
    for (int j = 0; j < kMaxSlices; ++j) {
      const int k = (step_lo + warp + j * kWarps) * 32 + c * 8;
      xr[j] = make_uint4(0, 0, 0, 0);
      if (step_lo + warp + j * kWarps < step_hi && k < K && g < M)
        xr[j] = ld_ca(reinterpret_cast<const uint4*>(xin + (size_t)g * K + k));
    }
    wait_for_weights();
#pragma unroll
    for (int j = 0; j < kMaxSlices; ++j) {
      const int sl = step_lo + warp + j * kWarps;
      if (sl < step_hi) {
        const int kl = sl * 32 + c * 8 - k_lo;
        const uint4 a_lo = *reinterpret_cast<const uint4*>(wt + g * ldw + kl);
        const uint4 a_hi = *reinterpret_cast<const uint4*>(wt + (g + 8) * ldw + kl);
        mma_bf16(acc[0], a_lo.x, a_hi.x, a_lo.y, a_hi.y, xr[j].x, xr[j].y);
        mma_bf16(acc[0], a_lo.z, a_hi.z, a_lo.w, a_hi.w, xr[j].z, xr[j].w);
      }
    }
  } else {
    // (Two batch tiles, 9 to 16 rows, come here too: with all their activations asked for ahead as above, 56
    // registers of them a thread, a product took 1 to 2 microseconds longer than with this loop.)
    wait_for_weights();
  #pragma unroll 2
    for (int s = step_lo + warp; s < step_hi; s += kWarps) {
      const int k = s * 32 + c * 8;
      const bool ok = k < K;
      const uint4 a_lo = *reinterpret_cast<const uint4*>(wt + g * ldw + (k - k_lo));
      const uint4 a_hi = *reinterpret_cast<const uint4*>(wt + (g + 8) * ldw + (k - k_lo));
  #pragma unroll
      for (int t = 0; t < MT; ++t) {
        const int m = t * 8 + g;
        uint4 b = make_uint4(0, 0, 0, 0);
        if (ok && m < M) b = __ldcg(reinterpret_cast<const uint4*>(xin + (size_t)m * K + k));
        mma_bf16(acc[t], a_lo.x, a_hi.x, a_lo.y, a_hi.y, b.x, b.y);
        mma_bf16(acc[t], a_lo.z, a_hi.z, a_lo.w, a_hi.w, b.z, b.w);
      }
    }
  }

  EMBER_MARK(kLinearDecode, kPhaseB);  // products done
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
  EMBER_MARK(kLinearDecode, kEnd);
}

template <int MT>
int launch(const void* xin, const void* W, const float* bias, const float* residual, void* out, int M, int N, int K, int act,
           int out_dtype, const Warm& warm, cudaStream_t stream) {
  const int tiles = (N + 15) / 16;
  const int all_steps = (K + 31) / 32;
  // Split K over a cluster (1, 2 or 4 blocks) so that a block's share of the matrix fits the
  // shared memory three blocks can have on an SM (about 56 KB of weights each), and no further: a
  // matrix of few tiles (GPT-2 XL's output projection: 100) is faster as 100 blocks on 100 SMs than
  // as 200 that meet in pairs (a step at batch 8 1.3546 -> 1.3325 ms, at batch 1 1.1887 -> 1.1425).
  int k_split = 1;
  while (k_split < 4 && all_steps / k_split > 54) k_split *= 2;
  const int per_block = (all_steps + k_split - 1) / k_split;
  const size_t need = (size_t)16 * tile_stride(per_block) * sizeof(__nv_bfloat16) +
                      (size_t)(kWarps + k_split) * 16 * 8 * MT * sizeof(float);
  if (need > 200 * 1024)
    return ember_fail("linear_decode: K = %d needs %zu bytes of shared memory per block", K, need);
  // (the output projection's 200 blocks, three of which fit an SM, then run two to an SM on all of the chip
  // and not on some 94 SMs: a step of GPT-2 XL at batch 8 1.3621 -> 1.3545 ms, at batch 1 1.199 -> 1.1885)
  const size_t smem = spread_smem(need, (long long)tiles * k_split);
  static size_t configured = 0;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(linear_decode_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
    if (e != cudaSuccess) return ember_fail("linear_decode: %s", cudaGetErrorString(e));
    configured = 1;
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
  cudaError_t e = cudaLaunchKernelEx(&cfg, linear_decode_kernel<MT>, (const __nv_bfloat16*)xin, (const __nv_bfloat16*)W, bias,
                                     residual, out, M, N, K, act, out_f32, k_split, warm);
  if (e != cudaSuccess) return ember_fail("linear_decode: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace

// 0, or 1 if a block of some launch since the last call gave up waiting for its weight copies (its
// results are not valid); the flag is cleared.  Synchronizes with the device.
EMBER_API int ember_linear_decode_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gave_up, sizeof(int)) != cudaSuccess) return 0;
  if (v) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_gave_up, &zero, sizeof(int));
  }
  return v;
}

// xin: bfloat16 [M,K].  residual: float32 [M,N] or null; it may be the output buffer.  out: float32 or
// bfloat16 [M,N].  warm, warm_bytes: null and 0, or constants that a kernel soon after this one reads (the
// next product's weight matrix): this launch's blocks ask them into L2 before they wait for anything.
EMBER_API int ember_linear_decode(const void* xin, const void* W, const float* bias, const float* residual, void* out, int M,
                                  int N, int K, int act, int out_dtype, const void* warm, size_t warm_bytes,
                                  cudaStream_t stream) {
  EMBER_CHECK(M > 0 && M <= 16 && N > 0 && K > 0, "linear_decode: M = %d (at most 16), N = %d, K = %d", M, N, K);
  EMBER_CHECK(K % 8 == 0, "linear_decode: K = %d is not a multiple of 8 (16-byte rows)", K);
  EMBER_CHECK(act >= 0 && act <= 2, "linear_decode: activation %d", act);
  EMBER_CHECK(out_dtype == EMBER_F32 || out_dtype == EMBER_BF16, "linear_decode: output type %d", out_dtype);
  EMBER_CHECK(!residual || out_dtype == EMBER_F32, "linear_decode: a residual sum needs a float32 output");
  EMBER_CHECK(warm_bytes % 16 == 0 && (reinterpret_cast<size_t>(warm) & 15) == 0,
              "linear_decode: what is to be warmed is 16-byte aligned and a multiple of 16 bytes");
  const Warm w = {warm_bytes ? static_cast<const char*>(warm) : nullptr, warm_bytes};
  if (M <= 8) return launch<1>(xin, W, bias, residual, out, M, N, K, act, out_dtype, w, stream);
  return launch<2>(xin, W, bias, residual, out, M, N, K, act, out_dtype, w, stream);
}

EMBER_TIMELINE_READER(linear_decode)
