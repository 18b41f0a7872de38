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
// Tail norm: when the caller says that the sum this product adds into the residual stream is
// normed next, the block that finishes last (a ticket from an atomic counter, which it sets back to
// zero) norms all M rows of the stream and writes them in bfloat16: the values the separate norm
// kernel would write, one launch and one trip through the launch queue earlier.  Nothing waits:
// every block takes its ticket after its own stores and a fence, and only the last one goes on.
//
// Input modes: float32 rows with a layer norm (statistics in float32 per row, each value
// normalised and rounded to bfloat16 as it enters an MMA: the values the separate norm kernel
// writes), or bfloat16 rows read as they are.
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
constexpr int kRowVecs = 16;  // float4 per lane of a row held in registers (K <= 2048)

__device__ __forceinline__ unsigned pack2(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const unsigned*>(&v);
}

// Row stride of the weight tile in shared memory, in elements: the slice plus a pad that puts
// consecutive rows 64 bytes apart modulo 128, so that the 16-byte reads of a quarter warp (two rows,
// four chunks each) fall into distinct banks.
__host__ __device__ inline int tile_stride(int per_block) { return per_block * 32 + ((per_block & 1) ? 0 : 32); }

// Layer norm of rows of float32, written in bfloat16, by the whole block: two warps a row, four
// rows at a time.  The rows were written by other blocks of this launch: they are read from L2
// (`__ldcg`), never from this SM's L1.  Same order of operations inside a warp as the separate norm
// kernel (values in registers, mean, then the biased variance); the two warps' sums are added in
// warp order.  Every thread of the block must call it.
constexpr int kTailVecs = 8;  // float4 per lane: rows of up to 2 * 32 * 8 * 4 = 2048 values stay in registers
__device__ __noinline__ void tail_norm(const float* x, const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                                       __nv_bfloat16* out, int M, int K) {
  __shared__ float s_part[kWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nv = K >> 2;
  if ((K & 3) == 0 && nv <= 64 * kTailVecs) {
    for (int m0 = 0; m0 < M; m0 += kWarps / 2) {
      const int m = m0 + (warp >> 1);
      const int l64 = (warp & 1) * 32 + lane;
      const bool row_ok = m < M;
      const float4* r4 = reinterpret_cast<const float4*>(x + (size_t)(row_ok ? m : 0) * K);
      float4 v[kTailVecs];
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < kTailVecs; ++j) {
        const int i = l64 + 64 * j;
        v[j] = (row_ok && i < nv) ? __ldcg(r4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
      }
      s = warp_sum(s);
      __syncthreads();  // s_part is free again
      if (lane == 0) s_part[warp] = s;
      __syncthreads();
      const float mean = (s_part[warp & ~1] + s_part[warp | 1]) / (float)K;
      float q = 0.f;
#pragma unroll
      for (int j = 0; j < kTailVecs; ++j) {
        if (l64 + 64 * j < nv) {
          const float a0 = v[j].x - mean, a1 = v[j].y - mean, a2 = v[j].z - mean, a3 = v[j].w - mean;
          q += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
        }
      }
      q = warp_sum(q);
      __syncthreads();
      if (lane == 0) s_part[warp] = q;
      __syncthreads();
      const float inv = 1.0f / sqrtf((s_part[warp & ~1] + s_part[warp | 1]) / (float)K + eps);
      if (row_ok) {
        __nv_bfloat16* o = out + (size_t)m * K;
#pragma unroll
        for (int j = 0; j < kTailVecs; ++j) {
          const int i = l64 + 64 * j;
          if (i < nv) {
            const float4 gm = reinterpret_cast<const float4*>(gamma)[i], bt = reinterpret_cast<const float4*>(beta)[i];
            uint2 w;
            w.x = pack2((v[j].x - mean) * inv * gm.x + bt.x, (v[j].y - mean) * inv * gm.y + bt.y);
            w.y = pack2((v[j].z - mean) * inv * gm.z + bt.z, (v[j].w - mean) * inv * gm.w + bt.w);
            *reinterpret_cast<uint2*>(o + 4 * i) = w;
          }
        }
      }
    }
    return;
  }
  for (int m = warp; m < M; m += kWarps) {  // long or odd rows: a warp a row, three reads
    const float* r = x + (size_t)m * K;
    float s = 0.f;
    for (int i = lane; i < K; i += 32) s += __ldcg(r + i);
    const float mean = warp_sum(s) / (float)K;
    float q = 0.f;
    for (int i = lane; i < K; i += 32) {
      const float c = __ldcg(r + i) - mean;
      q += c * c;
    }
    const float inv = 1.0f / sqrtf(warp_sum(q) / (float)K + eps);
    for (int i = lane; i < K; i += 32)
      out[(size_t)m * K + i] = __float2bfloat16_rn((__ldcg(r + i) - mean) * inv * gamma[i] + beta[i]);
  }
}

struct TailNorm {  // all null / zero: no tail norm
  const float* gamma;
  const float* beta;
  float eps;
  __nv_bfloat16* out;  // [M, N]
  int* counter;        // zero between launches
};

struct Warm {  // null / 0: nothing
  const char* at;            // constants of a kernel that runs soon (the next product's weights) ...
  unsigned long long bytes;  // ... a multiple of 16, which this launch's blocks ask into L2, a share each
};

// MT: batch tiles of 8 sequences (1 or 2).  LN: float32 input with a fused layer norm.
template <int MT, bool LN>
__global__ void __launch_bounds__(kWarps * 32, 3)
linear_decode_kernel(const void* __restrict__ xin, const float* __restrict__ gamma, const float* __restrict__ beta,
                     float eps, const __nv_bfloat16* __restrict__ W, const float* __restrict__ bias,
                     const float* residual, void* out, int M, int N, int K, int act, int out_f32, int k_split,
                     const TailNorm tail, const Warm warm) {
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
  // shared memory: [wt: 16 x ldw bf16][red: kWarps x kTile][gather: k_split x kTile][stats: 2 x 16]
  __nv_bfloat16* wt = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  float* red = reinterpret_cast<float*>(wt + 16 * ldw);
  float* gather = red + kWarps * kTile;
  float* stats = gather + k_split * kTile;
  float* gain_s = stats + 2 * 16;                  // LN only: gamma[k_lo, k_hi) then beta[k_lo, k_hi)

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
    // with a fused norm, its gain and bias over the block's range of K come the same way
    const unsigned norm_bytes = LN ? 2u * row_bytes : 0u;  // float32: twice a weight row's bytes, each
    if (lane == 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(16u * row_bytes + 2u * norm_bytes)
                   : "memory");
    __syncwarp();
    if (LN && lane >= 16 && lane < 18 && norm_bytes) {
      const float* src = (lane == 16 ? gamma : beta) + k_lo;
      const unsigned dst = (unsigned)__cvta_generic_to_shared(gain_s + (lane == 16 ? 0 : k_hi - k_lo));
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
                   "l"(src), "r"(norm_bytes), "r"(bar)
                   : "memory");
    }
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

  if (LN) {
    const float* x = static_cast<const float*>(xin);
    // One warp per row: mean, then biased variance, over the whole row.  A row of up to 2048
    // values is read once into registers, all its loads in flight together (one trip to L2);
    // longer rows are read twice in pieces.
    for (int m = warp; m < M; m += kWarps) {
      const float* r = x + (size_t)m * K;
      const int nv = K >> 2;
      const float4* r4 = reinterpret_cast<const float4*>(r);
      float mean, var;
      if (nv <= 32 * kRowVecs) {
        float4 v[kRowVecs];
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < kRowVecs; ++j) {
          const int i = lane + 32 * j;
          v[j] = i < nv ? __ldcg(r4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < kRowVecs; ++j) sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        mean = warp_sum(sum) / (float)K;
        float sq = 0.f;
#pragma unroll
        for (int j = 0; j < kRowVecs; ++j) {
          if (lane + 32 * j < nv) {
            const float a0 = v[j].x - mean, a1 = v[j].y - mean, a2 = v[j].z - mean, a3 = v[j].w - mean;
            sq += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
          }
        }
        var = warp_sum(sq) / (float)K;
      } else {
        float sum = 0.f;
#pragma unroll 8
        for (int i = lane; i < nv; i += 32) {
          const float4 v = __ldcg(r4 + i);
          sum += (v.x + v.y) + (v.z + v.w);
        }
        mean = warp_sum(sum) / (float)K;
        float sq = 0.f;
#pragma unroll 8
        for (int i = lane; i < nv; i += 32) {
          const float4 v = __ldcg(r4 + i);
          const float a0 = v.x - mean, a1 = v.y - mean, a2 = v.z - mean, a3 = v.w - mean;
          sq += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
        }
        var = warp_sum(sq) / (float)K;
      }
      if (lane == 0) {
        stats[2 * m] = mean;
        stats[2 * m + 1] = 1.0f / sqrtf(var + eps);
      }
    }
  }
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
  if (MT == 1 && !LN && per_block <= kMaxSlices * kWarps) {
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
        xr[j] = ld_ca(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(xin) + (size_t)g * K + k));
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
  } else if (MT == 1 && LN && per_block <= kMaxSlices * kWarps) {
    // The same with the norm: this thread's values of row g (float32, 8 for each of its slices; the
    // warp that took the row's statistics has just read them, so most come from this SM's L1) are
    // asked for at once, then normalised with the gain and bias that came with the weights and
    // rounded to bfloat16 as they enter the MMAs.
    const float* x = static_cast<const float*>(xin);
    float4 xa[kMaxSlices], xb[kMaxSlices];
#pragma unroll
    for (int j = 0; j < kMaxSlices; ++j) {
      const int k = (step_lo + warp + j * kWarps) * 32 + c * 8;
      xa[j] = xb[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (step_lo + warp + j * kWarps < step_hi && k < K && g < M) {
        xa[j] = __ldcg(reinterpret_cast<const float4*>(x + (size_t)g * K + k));
        xb[j] = __ldcg(reinterpret_cast<const float4*>(x + (size_t)g * K + k + 4));
      }
    }
    wait_for_weights();  // and for the gain and bias; its barrier also publishes the statistics
    const float mean = g < M ? stats[2 * g] : 0.f, inv = g < M ? stats[2 * g + 1] : 0.f;
    const float* beta_s = gain_s + (k_hi - k_lo);
#pragma unroll
    for (int j = 0; j < kMaxSlices; ++j) {
      const int sl = step_lo + warp + j * kWarps;
      if (sl < step_hi) {
        const int kl = sl * 32 + c * 8 - k_lo;
        uint4 b = make_uint4(0, 0, 0, 0);
        if (kl + k_lo < K && g < M) {
          const float4 g0 = *reinterpret_cast<const float4*>(gain_s + kl), g1 = *reinterpret_cast<const float4*>(gain_s + kl + 4);
          const float4 b0 = *reinterpret_cast<const float4*>(beta_s + kl), b1 = *reinterpret_cast<const float4*>(beta_s + kl + 4);
          b.x = pack2((xa[j].x - mean) * inv * g0.x + b0.x, (xa[j].y - mean) * inv * g0.y + b0.y);
          b.y = pack2((xa[j].z - mean) * inv * g0.z + b0.z, (xa[j].w - mean) * inv * g0.w + b0.w);
          b.z = pack2((xb[j].x - mean) * inv * g1.x + b1.x, (xb[j].y - mean) * inv * g1.y + b1.y);
          b.w = pack2((xb[j].z - mean) * inv * g1.z + b1.z, (xb[j].w - mean) * inv * g1.w + b1.w);
        }
        const uint4 a_lo = *reinterpret_cast<const uint4*>(wt + g * ldw + kl);
        const uint4 a_hi = *reinterpret_cast<const uint4*>(wt + (g + 8) * ldw + kl);
        mma_bf16(acc[0], a_lo.x, a_hi.x, a_lo.y, a_hi.y, b.x, b.y);
        mma_bf16(acc[0], a_lo.z, a_hi.z, a_lo.w, a_hi.w, b.z, b.w);
      }
    }
  } else {
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
        if (ok && m < M) {
          if (LN) {
            const float* r = static_cast<const float*>(xin) + (size_t)m * K + k;
            const float4 v0 = __ldcg(reinterpret_cast<const float4*>(r)), v1 = __ldcg(reinterpret_cast<const float4*>(r + 4));
            const float* gs = gain_s + (k - k_lo);
            const float* bs = gs + (k_hi - k_lo);
            const float4 g0 = *reinterpret_cast<const float4*>(gs), g1 = *reinterpret_cast<const float4*>(gs + 4);
            const float4 b0 = *reinterpret_cast<const float4*>(bs), b1 = *reinterpret_cast<const float4*>(bs + 4);
            const float mean = stats[2 * m], inv = stats[2 * m + 1];
            b.x = pack2((v0.x - mean) * inv * g0.x + b0.x, (v0.y - mean) * inv * g0.y + b0.y);
            b.y = pack2((v0.z - mean) * inv * g0.z + b0.z, (v0.w - mean) * inv * g0.w + b0.w);
            b.z = pack2((v1.x - mean) * inv * g1.x + b1.x, (v1.y - mean) * inv * g1.y + b1.y);
            b.w = pack2((v1.z - mean) * inv * g1.z + b1.z, (v1.w - mean) * inv * g1.w + b1.w);
          } else {
            b = __ldcg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(xin) + (size_t)m * K + k));
          }
        }
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
  if (tail.out) {  // block 0 of every cluster comes here: one ticket a tile
    __shared__ int s_last;
    __threadfence();  // this thread's store is visible to the whole device before the ticket is taken
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(tail.counter, 1) == (int)(gridDim.x / k_split) - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    tail_norm(static_cast<const float*>(out), tail.gamma, tail.beta, tail.eps, tail.out, M, N);
    if (threadIdx.x == 0) *tail.counter = 0;
  }
}

template <int MT, bool LN>
int launch(const void* xin, const float* gamma, const float* beta, float eps, const void* W, const float* bias,
           const float* residual, void* out, int M, int N, int K, int act, int out_dtype, const TailNorm& tail,
           const Warm& warm, cudaStream_t stream) {
  const int tiles = (N + 15) / 16;
  const int all_steps = (K + 31) / 32;
  // Split K over a cluster (1, 2 or 4 blocks) so that a block's share of the matrix fits the
  // shared memory three blocks can have on an SM (about 56 KB of weights each), and further while
  // the blocks still fit the chip at once and keep at least two slices per warp.
  int k_split = 1;
  while (k_split < 4 && all_steps / k_split > 54) k_split *= 2;
  while (k_split < 4 && tiles * k_split * 2 <= 3 * sm_count() && all_steps / (k_split * 2) >= 2 * kWarps) k_split *= 2;
  const int per_block = (all_steps + k_split - 1) / k_split;
  const size_t smem = (size_t)16 * tile_stride(per_block) * sizeof(__nv_bfloat16) +
                      (size_t)(kWarps + k_split) * 16 * 8 * MT * sizeof(float) + 2 * 16 * sizeof(float) +
                      (LN ? (size_t)2 * per_block * 32 * sizeof(float) : 0);
  if (smem > 200 * 1024)
    return ember_fail("linear_decode: K = %d needs %zu bytes of shared memory per block", K, smem);
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
                                     (const __nv_bfloat16*)W, bias, residual, out, M, N, K, act, out_f32, k_split, tail,
                                     warm);
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

// xin: float32 [M,K] when gamma is given (layer norm fused), else bfloat16 [M,K].
// residual: float32 [M,N] or null; it may be the output buffer.  out: float32 or bfloat16 [M,N].
// warm, warm_bytes: null and 0, or constants that a kernel soon after this one reads (the next
// product's weight matrix): this launch's blocks ask them into L2 before they wait for anything.
// tail_*: all null, or the layer norm to apply to the float32 output's rows once they are complete
// (gain and bias float32 [N], result bfloat16 [M,N], a counter that is zero and is left zero).
EMBER_API int ember_linear_decode(const void* xin, const float* gamma, const float* beta, float eps, const void* W,
                                  const float* bias, const float* residual, void* out, int M, int N, int K, int act,
                                  int out_dtype, const float* tail_gamma, const float* tail_beta, float tail_eps,
                                  void* tail_out, int* tail_counter, const void* warm, size_t warm_bytes,
                                  cudaStream_t stream) {
  EMBER_CHECK(M > 0 && M <= 16 && N > 0 && K > 0, "linear_decode: M = %d (at most 16), N = %d, K = %d", M, N, K);
  EMBER_CHECK(K % 8 == 0, "linear_decode: K = %d is not a multiple of 8 (16-byte rows)", K);
  EMBER_CHECK(act >= 0 && act <= 2, "linear_decode: activation %d", act);
  EMBER_CHECK(out_dtype == EMBER_F32 || out_dtype == EMBER_BF16, "linear_decode: output type %d", out_dtype);
  EMBER_CHECK(!residual || out_dtype == EMBER_F32, "linear_decode: a residual sum needs a float32 output");
  EMBER_CHECK((gamma == nullptr) == (beta == nullptr), "linear_decode: give both norm parameters or neither");
  TailNorm tail = {tail_gamma, tail_beta, tail_eps, static_cast<__nv_bfloat16*>(tail_out), tail_counter};
  if (tail_out) {
    EMBER_CHECK(tail_gamma && tail_beta && tail_counter, "linear_decode: a tail norm needs its gain, bias and counter");
    EMBER_CHECK(out_dtype == EMBER_F32, "linear_decode: a tail norm reads a float32 output");
  } else {
    tail = TailNorm{nullptr, nullptr, 0.f, nullptr, nullptr};
  }
  EMBER_CHECK(warm_bytes % 16 == 0 && (reinterpret_cast<size_t>(warm) & 15) == 0,
              "linear_decode: what is to be warmed is 16-byte aligned and a multiple of 16 bytes");
  const Warm w = {warm_bytes ? static_cast<const char*>(warm) : nullptr, warm_bytes};
  const bool ln = gamma != nullptr;
  if (M <= 8)
    return ln ? launch<1, true>(xin, gamma, beta, eps, W, bias, residual, out, M, N, K, act, out_dtype, tail, w, stream)
              : launch<1, false>(xin, gamma, beta, eps, W, bias, residual, out, M, N, K, act, out_dtype, tail, w, stream);
  return ln ? launch<2, true>(xin, gamma, beta, eps, W, bias, residual, out, M, N, K, act, out_dtype, tail, w, stream)
            : launch<2, false>(xin, gamma, beta, eps, W, bias, residual, out, M, N, K, act, out_dtype, tail, w, stream);
}

EMBER_TIMELINE_READER(linear_decode)
