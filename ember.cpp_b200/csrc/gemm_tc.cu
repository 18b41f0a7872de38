// Y[M,N] = A[M,K] . W[N,K]^T (+ bias) (activation) (+ residual) on the fifth-generation tensor
// cores: the matrix product of the bfloat16 prefill path, with its epilogue in the same kernel.
//
// ember.cpp's engine makes these products with a library call and adds the bias, the GELU and the
// residual in separate kernels (cublasSgemm, cuda_kernels.cu:3617-3621; graph_ir_cuda.cu:67-76,
// 230-242).  Here one persistent kernel does all of it:
//
//   warp 0        TMA producer: `cp.async.bulk.tensor.2d` copies of a 128 x 64 tile of A and of this
//                 block's rows of the W tile into a ring of shared-memory stages (128-byte swizzle),
//                 completion counted on an mbarrier per stage;
//   warp 1        issues `tcgen05.mma.kind::f16` (operands read from shared memory through
//                 descriptors, float32 accumulator in tensor memory) and hands a stage back with
//                 `tcgen05.commit`;
//   warps 2 to 9  epilogue: `tcgen05.ld` of the accumulator (one row a thread), bias, activation,
//                 residual sum in float32, and the stores.
//
// Two forms.  `cta_group::2`: two blocks (a cluster of two SMs) make one 256 x BN tile.  Each block
// loads its own 128 rows of A and its half of the BN rows of W; the first block issues one
// instruction of M = 256 for both, which reads either half of W from the block that holds it, so a
// block fetches 32 KB for the products it would need 48 KB for alone: these products are bound by
// what shared memory can take in from L2.  Each block's tensor memory receives its own 128 rows.
// `cta_group::1`: one block makes a 128 x BN tile by itself (taken when M is at most 128).
//
// Tensor memory holds two accumulators (columns 0 and 256), so the epilogue of a tile runs under
// the products of the next one.  A block (pair) walks tiles i, i + pairs, ...; tiles that follow
// one another share their columns of W, so the weight tile is read from L2.
//
// Every wait on an mbarrier has a time limit.  A role whose wait runs out records a code in the
// status word (host-visible memory) and leaves; the block then waits, again with a limit, for its
// copies in flight, meets its partner, frees its tensor memory and returns.  The results of such a
// launch are not valid, and `ember_tc_status` says so.
#include <mutex>
#include <unordered_map>

#include "tc_common.cuh"

namespace {

constexpr int BM = 128;           // rows of A (tokens) a block holds: the lanes of its tensor memory
constexpr int BK = 64;            // values of K in a box: 128 bytes, the width of the swizzle
constexpr int KSUB = 2;           // boxes of each operand in a stage: a stage holds KSUB * BK values of K
constexpr int kMaxBN = 256;       // the most columns of a tile: the largest N of the instruction
constexpr int kAccStride = 256;   // tensor-memory columns between the two accumulators
constexpr int kTmemCols = 512;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr int kMaxStages = 16;
constexpr int kSmemLimit = 227 * 1024;
constexpr int kTurnBytes = kEpiWarps * 32 * 33 * 4;  // a 32 x 32 block (rows padded to 33) for each epilogue warp

using namespace tc;  // mbarriers with time-limited waits, descriptors, fences, tensor-memory loads (tc_common.cuh)

// the same barrier in the first block of the cluster (this block, when it is the first)
__device__ __forceinline__ unsigned leader_addr(unsigned bar) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, 0;\n" : "=r"(r) : "r"(bar));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_bar) : "memory");
}

// One box of a tensor map into this block's shared memory.  With two blocks the completion is
// counted on the first block's barrier (`bar` is a cluster address then): that block issues the
// products for both.  No multicast: every block fetches what it uses.
template <int CTAS>
__device__ __forceinline__ void load_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
  if constexpr (CTAS == 2)
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
            dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
  else
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// Issued by a whole, converged warp whose lanes all hold the same operands; one elected lane
// issues (tc_common.cuh has the measured cost of an instruction by shape and way of issuing).
template <int CTAS>
__device__ __forceinline__ void umma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc,
                                     unsigned accumulate) {
  if constexpr (CTAS == 2)
    asm volatile(
        "{\n.reg .pred p, e;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "elect.sync _|e, 0xffffffff;\n"
        "@e tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n.reg .pred p, e;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "elect.sync _|e, 0xffffffff;\n"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the barrier (at this offset in every block of the tile) once the products issued so
// far are complete.
template <int CTAS>
__device__ __forceinline__ void umma_commit(unsigned bar) {
  if constexpr (CTAS == 2)
    asm volatile(
        "{\n.reg .pred e;\n"
        "elect.sync _|e, 0xffffffff;\n"
        "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n}\n" ::"r"(bar),
        "h"((unsigned short)3)
        : "memory");
  else
    asm volatile(
        "{\n.reg .pred e;\n"
        "elect.sync _|e, 0xffffffff;\n"
        "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}\n" ::"r"(bar)
        : "memory");
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

// The tanh GELU as v / (1 + exp(-2u)), u = sqrt(2/pi) (v + 0.044715 v^3): the same function as
// 0.5 v (1 + tanh u), one exponential and one division in place of a tanh.
__device__ __forceinline__ float gelu_tanh_fast(float v) {
  const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
  return __fdividef(v, 1.0f + __expf(-2.0f * u));
}

struct TcArgs {
  const float* bias;
  const float* residual;
  void* out;
  int M, N, K, bn, stages, act, out_f32;
  int* status;
  int band;  // m-tiles whose tiles are walked together (all their n-tiles) before the next band
};

// status codes: which role gave up
enum : int { TC_OK = 0, TC_PRODUCER = 1, TC_MMA = 2, TC_EPILOGUE = 3, TC_DRAIN = 4 };

// Tile number -> (m-tile, n-tile).  Tiles are walked band by band: a band is `band` m-tiles with
// all their n-tiles, m fastest, so that the blocks running at one time share a few rows of tiles
// of A and every tile of W through L2 however large A is.
__device__ __forceinline__ void tile_coords(const TcArgs& p, int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_band = p.band * tiles_n;
  const int b = tile / per_band, idx = tile - b * per_band;
  const int here = min(p.band, tiles_m - b * p.band);
  tm = b * p.band + idx % here;
  tn = idx / here;
}

template <int CTAS>
__global__ void __launch_bounds__(kThreads, 1)
    linear_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const TcArgs p) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ unsigned long long bars[2 * kMaxStages + 4];  // full[stages], empty[stages], acc_full[2], acc_empty[2]
  __shared__ unsigned s_tmem;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = CTAS == 2 ? (int)(blockIdx.x & 1) : 0;  // a cluster is two consecutive blocks
  const int group = blockIdx.x / CTAS, groups = gridDim.x / CTAS;
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // stages start on 1,024 bytes
  const int bn_own = p.bn / CTAS;                                // the rows of the W tile this block holds
  const int a_bytes = BM * BK * 2, b_bytes = bn_own * BK * 2;  // one box of either operand
  const int stage_bytes = KSUB * (a_bytes + b_bytes);
  const unsigned full0 = smem_u32(bars), empty0 = full0 + 8 * p.stages;
  const unsigned acc_full0 = empty0 + 8 * p.stages, acc_empty0 = acc_full0 + 16;

  const int tile_rows = BM * CTAS;
  const int tiles_m = (p.M + tile_rows - 1) / tile_rows, tiles_n = (p.N + p.bn - 1) / p.bn;
  const int n_tiles = tiles_m * tiles_n;
  const int k_blocks = (p.K + KSUB * BK - 1) / (KSUB * BK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full0 + 8 * a, 1);
      mbar_init(acc_empty0 + 8 * a, kEpiWarps * CTAS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_w) : "memory");
  }
  if (warp == 1) {
    if constexpr (CTAS == 2) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem)),
                   "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem)),
                   "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
  }
  fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) cluster_sync();  // the partner's barriers exist before anything arrives on them
  fence_after();
  const unsigned tmem = s_tmem;
  // Everything above touched this block's own resources only and may run while the kernel before
  // this one still does; its results are read from here on.
  pdl_wait();
  pdl_trigger();

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    int it = 0;
    bool ok = true;
    for (int tile = group; tile < n_tiles && ok; tile += groups) {
      int tm, tn;
      tile_coords(p, tile, tiles_m, tiles_n, tm, tn);
      const int m0 = tm * tile_rows + rank * BM, n0 = tn * p.bn + rank * bn_own;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const int s = it % p.stages;
        ok = mbar_wait(empty0 + 8 * s, ((it / p.stages) & 1) ^ 1);
        if (!ok) break;
        if (lane == 0) {
          const unsigned dst = base + s * stage_bytes;
          unsigned bar = full0 + 8 * s;
          if (rank == 0) mbar_expect_tx(bar, stage_bytes * CTAS);
          if constexpr (CTAS == 2) bar = leader_addr(bar);
#pragma unroll
          for (int j = 0; j < KSUB; ++j) {  // a box past the end of K reads as zeros
            load_2d<CTAS>(dst + j * a_bytes, &map_a, (kb * KSUB + j) * BK, m0, bar);
            load_2d<CTAS>(dst + KSUB * a_bytes + j * b_bytes, &map_w, (kb * KSUB + j) * BK, n0, bar);
          }
        }
        __syncwarp();
      }
    }
    if (!ok && lane == 0) atomicCAS(p.status, TC_OK, TC_PRODUCER);
    // Copies still in flight land in this block's shared memory: the block may not end before
    // them.  Every stage that was filled is handed back (the empty barrier) only after its copies
    // landed and were used, so waiting for the last `stages` hand-backs covers them all; on the
    // way out after an error the wait simply runs out.
    for (int j = max(0, it - p.stages); j < it; ++j)
      if (!mbar_wait(empty0 + 8 * (j % p.stages), (j / p.stages) & 1)) {
        if (lane == 0) atomicCAS(p.status, TC_OK, TC_DRAIN);
        break;
      }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ products (first block only)
    if (rank == 0) {
      const unsigned idesc = instr_desc_bf16(BM * CTAS, p.bn, false);
      int it = 0, t = 0;
      bool ok = true;
      for (int tile = group; tile < n_tiles && ok; tile += groups, ++t) {
        const int as = t & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(acc_empty0 + 8 * as, ((t >> 1) & 1) ^ 1));
        if (!ok) break;
        fence_after();
        const unsigned acc = tmem + as * kAccStride;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % p.stages;
          ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, (it / p.stages) & 1));
          if (!ok) break;
          fence_after();
          const unsigned a_addr = base + s * stage_bytes;
#pragma unroll
          for (int j = 0; j < KSUB; ++j) {
            const unsigned long long da = smem_desc_sw128(a_addr + j * a_bytes), db = smem_desc_sw128(a_addr + KSUB * a_bytes + j * b_bytes);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) umma<CTAS>(acc, da + 2 * k, db + 2 * k, idesc, (kb | j | k) != 0);  // 32 bytes a step
          }
          umma_commit<CTAS>(empty0 + 8 * s);
        }
        if (ok) umma_commit<CTAS>(acc_full0 + 8 * as);
      }
      if (!ok && lane == 0) atomicCAS(p.status, TC_OK, TC_MMA);
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    // A warp reads 32 rows x 32 columns of the accumulator with a row in each thread, turns the
    // block through shared memory and finishes it with a column in each lane: the bias is one
    // value a lane, and every access to the residual and the output covers 32 consecutive
    // columns of one row.  The residual of a block is requested before its accumulator is read.
    // (Tried for the residual: a thread finishing the 32 columns of its own row, 128 bytes of residual and
    // of output a thread, with no turn.  The output projection gained, 167 -> 135 microseconds at 16,384
    // rows, but the down projection lost, 264 -> 294, and the form without a residual ran 8 % slower
    // for having the other beside it in the loop; taken out.)
    const int quarter = warp & 3;            // the 32 tensor-memory lanes this warp may read
    const int half = (warp - 2) >> 2;        // which of the two warps of this quarter: it takes every other 32 columns
    const bool vec_ok = p.out_f32 ? (p.N % 4 == 0) : (p.N % 8 == 0);
    float* turn = reinterpret_cast<float*>(smem_raw + (base - smem_u32(smem_raw)) + p.stages * stage_bytes) + (warp - 2) * (32 * 33);
    const unsigned acc_empty_leader = CTAS == 2 ? leader_addr(acc_empty0) : acc_empty0;
    int t = 0;
    bool ok = true;
    for (int tile = group; tile < n_tiles; tile += groups, ++t) {
      int tm, tn;
      tile_coords(p, tile, tiles_m, tiles_n, tm, tn);
      const int m0 = tm * tile_rows + rank * BM + quarter * 32, n0 = tn * p.bn;
      const int as = t & 1;
      const int rows = min(32, p.M - m0);  // may be <= 0: this warp's rows lie outside the matrix
      float res[32];
      auto fetch_residual = [&](int c0) {
        const int n = n0 + c0 + lane;
        const bool col_ok = c0 + lane < p.bn && n < p.N;
#pragma unroll
        for (int r = 0; r < 32; ++r)
          res[r] = (p.residual && col_ok && r < rows) ? __ldcs(p.residual + (size_t)(m0 + r) * p.N + n) : 0.f;
      };
      int c0 = half * 32;
      if (c0 < p.bn) fetch_residual(c0);
      ok = mbar_wait(acc_full0 + 8 * as, (t >> 1) & 1);
      if (!ok) break;
      fence_after();
      const unsigned taddr = tmem + ((unsigned)(quarter * 32) << 16) + as * kAccStride;
      for (; c0 < p.bn; c0 += 64) {
        unsigned acc[32];
        tmem_ld32(taddr + c0, acc);  // every lane of the warp takes part, whatever its row
        tmem_wait();
        if (!p.residual && vec_ok && c0 + 32 <= p.bn && n0 + c0 + 32 <= p.N) {
          // no residual to fetch: each thread finishes the 32 columns of its own row
          if (lane < rows) {
            const int n = n0 + c0;
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]);
            if (p.bias) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + n + j));
                v[j] += b.x, v[j + 1] += b.y, v[j + 2] += b.z, v[j + 3] += b.w;
              }
            }
            if (p.act == EMBER_ACT_GELU_TANH) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = gelu_tanh_fast(v[j]);
            } else if (p.act == EMBER_ACT_GELU_ERF) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
            }
            const size_t at = (size_t)(m0 + lane) * p.N + n;
            if (p.out_f32) {
              float4* o = reinterpret_cast<float4*>(static_cast<float*>(p.out) + at);
#pragma unroll
              for (int j = 0; j < 8; ++j) o[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            } else {
              uint4* o = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + at);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 h[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[8 * j + 2 * i], v[8 * j + 2 * i + 1]);
                o[j] = *reinterpret_cast<uint4*>(h);
              }
            }
          }
          continue;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) turn[lane * 33 + j] = __uint_as_float(acc[j]);
        __syncwarp();
        const int n = n0 + c0 + lane;
        const bool col_ok = c0 + lane < p.bn && n < p.N;
        const float b = (p.bias && col_ok) ? __ldg(p.bias + n) : 0.f;
        if (col_ok) {
#pragma unroll
          for (int r = 0; r < 32; ++r) {
            if (r < rows) {
              float v = turn[r * 33 + lane] + b;
              if (p.act == EMBER_ACT_GELU_TANH) v = gelu_tanh_fast(v);
              else if (p.act == EMBER_ACT_GELU_ERF) v = gelu_erf(v);
              v += res[r];
              const size_t at = (size_t)(m0 + r) * p.N + n;
              if (p.out_f32)
                static_cast<float*>(p.out)[at] = v;
              else
                static_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(v);
            }
          }
        }
        if (c0 + 64 < p.bn) fetch_residual(c0 + 64);
        __syncwarp();
      }
      fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CTAS == 2)
          mbar_arrive_cluster(acc_empty_leader + 8 * as);
        else
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(acc_empty0 + 8 * as) : "memory");
      }
    }
    if (!ok && lane == 0) atomicCAS(p.status, TC_OK, TC_EPILOGUE);
  }

  fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) cluster_sync();  // neither block ends, or frees tensor memory, while the other still uses it
  if (warp == 1) {
    fence_after();
    if constexpr (CTAS == 2)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------- host
std::mutex g_mutex;
int g_sms = 0;

int tc_setup() {
  if (g_sms) return 0;
  if (!tc::encoder()) return ember_fail("linear_tc: the driver has no cuTensorMapEncodeTiled");
  if (!tc::status().device) return ember_fail("linear_tc: no host-visible status word");
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaError_t e = cudaFuncSetAttribute(linear_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit - 1024);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(linear_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit - 1024);
  if (e != cudaSuccess) return ember_fail("linear_tc: shared memory: %s", cudaGetErrorString(e));
  g_sms = sms;
  return 0;
}

// The tile width: the one whose waves of tiles cost least, a tile costing its columns plus a
// fixed share (the first fill of the ring and the last epilogue, which nothing hides).  With few
// waves (up to 4,096 rows) only multiples of 64 are considered: the widths between them run a tile
// slower (GPT-2 XL's q|k|v product at 2,048 rows: 28.5 microseconds at 192 columns, 36.3 at 208,
// 32.2 at 160), which many waves make up for by a fuller last wave (the down projection at 16,384
// rows: 264 microseconds at 208 columns, 284 at 192) and few do not.
int pick_bn(int M, int N, int groups, int ctas) {
  const int tiles_m = (M + BM * ctas - 1) / (BM * ctas);
  const int step = tiles_m <= 16 ? 64 : 16;
  int best = 0;
  double best_cost = 0;
  for (int bn = kMaxBN; bn >= 64; bn -= step) {
    const int tiles = tiles_m * ((N + bn - 1) / bn);
    const double cost = (double)((tiles + groups - 1) / groups) * (bn + 32);
    if (!best || cost < best_cost - 1e-9) best = bn, best_cost = cost;
  }
  return best;
}

}  // namespace

// Tensor maps are kept by (address, shape, box): weights come back with every call, activations
// with every replay of a graph.  Declared in tc_common.cuh; shared by the kernels that use TMA.
namespace tc {
namespace map_cache {
struct MapKey {
  const void* ptr;
  int rows, cols, box_rows, kind;  // kind 0: bfloat16, 128-byte swizzle; 1: float32, unswizzled
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows && kind == o.kind;
  }
};
struct MapHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.ptr * 1099511628211ull;
    h = (h ^ (size_t)k.rows) * 1099511628211ull;
    h = (h ^ (size_t)k.cols) * 1099511628211ull;
    return (h ^ (size_t)(k.box_rows * 2 + k.kind)) * 1099511628211ull;
  }
};
std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapHash> g_maps;
}  // namespace map_cache

static int cached_map_kind(const void* ptr, int rows, int cols, int box_rows, int kind, CUtensorMap* out) {
  using namespace map_cache;
  std::lock_guard<std::mutex> lock(g_map_mutex);
  const MapKey key{ptr, rows, cols, box_rows, kind};
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return 0;
  }
  CUtensorMap m;
  const bool made = kind == 0 ? encode_bf16_sw128(&m, ptr, (size_t)rows, (size_t)cols, (size_t)cols * 2, box_rows)
                              : encode_f32_plain(&m, ptr, (size_t)rows, (size_t)cols, (size_t)cols * 4, box_rows);
  if (!made)
    return ember_fail("the driver refused a tensor map for a [%d, %d] %s matrix in boxes of %d rows", rows, cols,
                      kind == 0 ? "bfloat16" : "float32", box_rows);
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps.emplace(key, m);
  *out = m;
  return 0;
}
int cached_map(const void* ptr, int rows, int cols, int box_rows, CUtensorMap* out) {
  return cached_map_kind(ptr, rows, cols, box_rows, 0, out);
}
int cached_map_f32(const void* ptr, int rows, int cols, int box_rows, CUtensorMap* out) {
  return cached_map_kind(ptr, rows, cols, box_rows, 1, out);
}
}  // namespace tc

// 0 when every launch of the tcgen05 kernels so far ran to its end; else the code of the role
// whose wait ran out (linear_tc: 1 producer, 2 products, 3 epilogue, 4 copies that never landed;
// attention_prefill_tc: 11 loader, 12 products, 13 softmax), and the word is cleared.  Meaningful
// after the stream has been synchronized.
EMBER_API int ember_tc_status() {
  tc::Status& st = tc::status();
  if (!st.host) return 0;
  const int s = *reinterpret_cast<volatile int*>(st.host);
  if (s) *reinterpret_cast<volatile int*>(st.host) = 0;
  return s;
}

// A [M,K] and W [N,K] bfloat16 row-major, 16-byte aligned, K a multiple of 8.  bias: float32 [N] or
// null.  residual: float32 [M,N] or null (the output is float32 then and may be the same buffer).
// act: an EMBER_ACT code.  tile_n: 0 lets the kernel choose, else a multiple of 16 in [16, 256].
EMBER_API int ember_linear_tc(const void* A, const void* W, const float* bias, const float* residual, void* out, int M, int N,
                              int K, int act, int out_dtype, int tile_n, cudaStream_t stream) {
  EMBER_CHECK(M > 0 && N > 0 && K > 0, "linear_tc: M = %d, N = %d, K = %d", M, N, K);
  EMBER_CHECK(K % 8 == 0, "linear_tc: K = %d is not a multiple of 8 (rows of 16 bytes)", K);
  EMBER_CHECK(((uintptr_t)A | (uintptr_t)W) % 16 == 0, "linear_tc: operands are not 16-byte aligned");
  EMBER_CHECK(act >= EMBER_ACT_NONE && act <= EMBER_ACT_GELU_ERF, "linear_tc: activation %d", act);
  EMBER_CHECK(out_dtype == EMBER_F32 || out_dtype == EMBER_BF16, "linear_tc: output type %d", out_dtype);
  EMBER_CHECK(!residual || out_dtype == EMBER_F32, "linear_tc: a residual sum needs a float32 output");
  EMBER_CHECK((uintptr_t)out % 16 == 0 && (!residual || (uintptr_t)residual % 16 == 0) && (!bias || (uintptr_t)bias % 16 == 0),
              "linear_tc: output, residual and bias are 16-byte aligned");
  EMBER_CHECK(tile_n == 0 || (tile_n % 16 == 0 && tile_n >= 16 && tile_n <= kMaxBN), "linear_tc: tile width %d", tile_n);
  CUtensorMap map_a, map_w;
  const int ctas = M > BM ? 2 : 1;  // blocks that share a tile
  int bn, groups;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (int rc = tc_setup()) return rc;
    groups = g_sms / ctas;
    bn = tile_n ? tile_n : pick_bn(M, N, groups, ctas);
    if (int rc = tc::cached_map(A, M, K, BM, &map_a)) return rc;
    if (int rc = tc::cached_map(W, N, K, bn / ctas, &map_w)) return rc;
  }
  TcArgs p;
  p.bias = bias, p.residual = residual, p.out = out;
  p.M = M, p.N = N, p.K = K, p.bn = bn, p.act = act, p.out_f32 = out_dtype == EMBER_F32;
  p.status = tc::status().device;
  const int stage_bytes = KSUB * (BM + bn / ctas) * BK * 2;
  const int smem = kSmemLimit - 1024;
  p.stages = (smem - 1024 - kTurnBytes) / stage_bytes;
  if (p.stages > kMaxStages) p.stages = kMaxStages;
  const int tiles_m = (M + BM * ctas - 1) / (BM * ctas), tiles_n = (N + bn - 1) / bn;
  const int tiles = tiles_m * tiles_n;
  p.band = (groups + tiles_n - 1) / tiles_n;
  if (p.band > tiles_m) p.band = tiles_m;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((tiles < groups ? tiles : groups) * ctas);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ctas, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = pdl_allowed();
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  const cudaError_t e = ctas == 2 ? cudaLaunchKernelEx(&cfg, linear_tc_kernel<2>, map_a, map_w, p)
                                  : cudaLaunchKernelEx(&cfg, linear_tc_kernel<1>, map_a, map_w, p);
  if (e != cudaSuccess) return ember_fail("linear_tc: %s", cudaGetErrorString(e));
  EMBER_LAUNCH_OK("linear_tc");
  return 0;
}
