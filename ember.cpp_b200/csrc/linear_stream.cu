// The linear layers of a decode step in bfloat16 for up to 64 rows: Y[M,N] = X[M,K] . W[N,K]^T with
// bias, GELU and the float32 residual sum in the same launch, on the fifth-generation tensor cores
// with the operands swapped, streaming the weight matrix once.
//
// ember.cpp makes a decode step's products as a library SGEMM of one column per sequence and adds
// bias, GELU and residual in further kernels (cuda_kernels.cu:3617-3621 as called from
// graph_ir.cpp:3824-3834; graph_ir_cuda.cu:67-76, 230-242); its batch loop runs the sequences of a
// batch through that path together (api.cpp:1819-1845).  A product of 17 to 64 rows is bound by
// the bytes of W: a tile of a library kernel that puts the rows of X on the 128-row side of the
// instruction wastes most of it and leaves the matrix to a handful of blocks.
//
// Here the 128 rows of a `tcgen05.mma` tile are 128 output features (rows of W) and its N = 16, 32,
// 48 or 64 columns are the sequences of the batch.  A block owns 128 rows of W and a share of K; a
// thread-block cluster of 1 to 8 blocks shares a tile and splits K between its blocks, so that a
// matrix of a few megabytes still occupies the whole chip.
//
//   warp 0        requests boxes of 128 x 64 of W and M x 64 of X by TMA (128-byte swizzle) into a
//                 ring of stages, completion counted on an mbarrier per stage.  The boxes of W of
//                 the first turn of the ring are requested before the kernel waits for the kernel
//                 in front of it (programmatic dependent launch): weights are constants of the
//                 model and stream while the producer of X still runs.  X follows after the wait.
//   warp 1        issues the products (A = the box of W, B = the box of X, both K-major, float32
//                 accumulator [128, N] in tensor memory) and hands stages back with tcgen05.commit.
//   warps 2 to 5  the epilogue: a thread holds one row of the accumulator (one output feature, all
//                 sequences).  With K split, the cluster's blocks exchange their partial sums
//                 through distributed shared memory: the sequences are dealt out in groups of four
//                 among the blocks, every block sends each other block that block's columns and
//                 sums what it receives in block order (no atomics: a result does not depend on
//                 timing).  The stores into a partner's shared memory count their bytes on the
//                 partner's mbarrier as they land (st.async), so nobody meets at a barrier after
//                 the exchange.  Then all eight warps apply bias, activation and residual to the
//                 block's own columns and store them; stores of a warp cover 32 consecutive
//                 features of one sequence.
//
// Nothing is written to global memory before the dependency wait, and what the kernel in front
// wrote (X, the residual) is read by TMA or `__ldcg`, never through the read-only data path.
//
// Every wait on an mbarrier has a time limit; a role whose wait runs out records a code in the
// host-visible status word, the block still meets its cluster at the cluster's one barrier (nobody
// is left waiting there), frees its tensor memory and returns.  `ember_tc_status` reports it.
// A block leaves only after everything its partners send it has landed (it needs it), and it sends
// to a partner only what that partner waits for: no block's shared memory is written after it left.
#include <mutex>

#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int BM = 128;          // rows of W a block holds: the lanes of its tensor memory
constexpr int BK = 64;           // values of K in a box: 128 bytes, the width of the swizzle
constexpr int kMaxRows = 64;     // the most rows of X (the N of the instruction)
constexpr int kMaxStages = 10;
constexpr int kMaxSplit = 8;     // blocks of a cluster (the portable limit)
constexpr int kThreads = 256;      // warp 0 loads, warp 1 issues the products, warps 2 to 5 read tensor memory; all eight finish
constexpr int kWBox = BM * BK * 2;

struct StreamArgs {
  const float* bias;
  const float* residual;
  void* out;
  int M, N, K;
  int mp;        // M rounded up to a multiple of 16: columns of the accumulator
  int stages, act, out_f32, k_split;
  const char* warm;            // constants that a kernel soon after this one streams (the next product's weights), or null:
  unsigned long long warm_bytes;  // a multiple of 16; this launch's blocks ask them into L2, a share each
  int res_by_tma;  // the residual's tile comes as one TMA box (its rows are 16-byte aligned)
  int* status;
};

enum : int { ST_PRODUCER = 21, ST_MMA = 22, ST_EPILOGUE = 23, ST_DRAIN = 24 };

// (Relaxed: what the partners must see, this block's initialised barriers, was released at cluster scope by the
// initialising lanes' own fence, and every thread that fenced also arrives here.)
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }
__device__ __forceinline__ unsigned map_to_rank(unsigned addr, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// Four floats into a partner's shared memory; when they have landed there, 16 bytes are counted on
// the partner's mbarrier: the data's arrival is its own signal, no barrier of the cluster follows.
__device__ __forceinline__ void st_async_f4(unsigned addr, unsigned a, unsigned b, unsigned c, unsigned d, unsigned remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];\n" ::"r"(addr),
               "r"(a), "r"(b), "r"(c), "r"(d), "r"(remote_bar)
               : "memory");
}

// The columns of the accumulator in groups of four ("quads"); block r of a cluster of `split` owns
// the quads [quads * r / split, quads * (r + 1) / split).
__host__ __device__ inline int quad_lo(int quads, int split, int r) { return quads * r / split; }
__host__ __device__ inline int quad_owner(int quads, int split, int q) { return ((q + 1) * split - 1) / quads; }
__host__ __device__ inline int quads_most(int quads, int split) { return (quads + split - 1) / split; }

// The tanh GELU as v / (1 + exp(-2u)), u = sqrt(2/pi) (v + 0.044715 v^3): the same function as
// 0.5 v (1 + tanh u), one exponential and one division in place of a tanh (and a fraction of its code).
__device__ __forceinline__ float gelu_tanh_fast(float v) {
  const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
  return __fdividef(v, 1.0f + __expf(-2.0f * u));
}

// The kernel's code runs once per block, straight through: what is executed once costs a fetch from
// the instruction cache's backing store per 128 bytes, so everything that could be unrolled into a
// long line of code (the exchange, the epilogue) is a short loop over shared memory instead.
__global__ void __launch_bounds__(kThreads, 2)
    linear_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                         const __grid_constant__ CUtensorMap map_r, const StreamArgs p) {
  EMBER_MARK_START(kLinearStream);
  extern __shared__ unsigned char smem_raw[];
  __shared__ unsigned long long bars[2 * kMaxStages + 3];  // full[stages], empty[stages], done, residual, partial sums
  __shared__ unsigned s_tmem;
  __shared__ unsigned char s_owner[kMaxRows / 4], s_local[kMaxRows / 4];
  __shared__ int s_failed;  // a wait of this block ran out: nothing is stored

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = p.k_split;
  const int rank = (int)(blockIdx.x % (unsigned)split);  // a cluster is `split` consecutive blocks
  const int n0 = (int)(blockIdx.x / (unsigned)split) * BM;
  // The boxes of K are dealt out to the cluster's blocks in turn (block r takes r, r + split, ...):
  // blocks that run side by side then read neighbouring 128-byte pieces of the same rows of W.
  const int kb_all = (p.K + BK - 1) / BK;
  const int n_kb = (kb_all - rank + split - 1) / split;
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int stage_bytes = kWBox + p.mp * BK * 2;
  const int quads = p.mp >> 2;
  const int q_most = quads_most(quads, split);
  const unsigned recv = base + p.stages * stage_bytes;          // [source block][quad of mine][row 0..127] float4
  const unsigned res_s = recv + split * q_most * (BM * 16);     // [column of mine][row 0..127] float
  const unsigned full0 = smem_u32(bars), empty0 = full0 + 8 * p.stages, done = empty0 + 8 * p.stages, res_bar = done + 8,
                 recv_bar = res_bar + 8;
  const unsigned tmem_cols = p.mp <= 32 ? 32u : 64u;

  // The barriers are set up by the first warp's lanes side by side (one after the other they cost the block's
  // first thread a third of a microsecond before it can ask for anything).
  if (warp == 0) {
    if (lane < p.stages) {
      mbar_init(full0 + 8 * lane, 1);
      mbar_init(empty0 + 8 * lane, 1);
    }
    if (lane == 31) {
      mbar_init(done, 1);
      mbar_init(res_bar, 1);
      mbar_init(recv_bar, 1);
      if (split > 1)  // what the partners will send: every other block's partial sums of this block's quads
        mbar_expect_tx(recv_bar, (unsigned)((split - 1) * (quad_lo(quads, split, rank + 1) - quad_lo(quads, split, rank)) * BM * 16));
      s_failed = 0;
    }
    mbar_init_fence();
    __syncwarp();
  }
  if (threadIdx.x == 0) {
    // The weights of the ring's first turn are asked for at once: before the other warps are met,
    // before tensor memory is there, and before the kernel in front is waited for (programmatic
    // dependent launch).  Weights are constants of the model.
    const int first = min(n_kb, p.stages);
    for (int i = 0; i < first; ++i) {
      mbar_expect_tx(full0 + 8 * i, (unsigned)stage_bytes);
      tma_load_2d(base + i * stage_bytes, &map_w, (rank + i * split) * BK, n0, full0 + 8 * i);
    }
    prefetch_map(&map_x);
  }
  // which block owns each quad of columns, and where the quad lies among its owner's (no divisions later)
  if (threadIdx.x >= 32 && threadIdx.x < 32 + kMaxRows / 4) {
    const int q = threadIdx.x - 32;
    const int owner = q < quads ? quad_owner(quads, split, q) : 0;
    s_owner[q] = (unsigned char)owner;
    s_local[q] = (unsigned char)(q < quads ? q - quad_lo(quads, split, owner) : 0);
  }
#ifdef EMBER_TIMELINE
  __shared__ unsigned s_tl;  // the block's place in the log, for the marks that other threads than the first leave
  if (threadIdx.x == 0) s_tl = ember_tl;
#define STREAM_MARK(m) \
  if (lane == 0) timeline::put(s_tl, timeline::kLinearStream, timeline::m)
#else
#define STREAM_MARK(m)
#endif
  if (warp == 1) tmem_alloc_1cta(smem_u32(&s_tmem), tmem_cols);
  fence_before();
  __syncthreads();
  fence_after();
  const unsigned tmem = s_tmem;
  // every block of the cluster says that it runs (its shared memory and its barriers exist) long
  // before a partner writes into it; the wait for this phase comes just before the first such write
  if (split > 1) cluster_arrive();
  pdl_trigger();

  // the bias of the row this thread finishes at the end: a constant of the model, asked for now (in a
  // decode step it comes from DRAM; at its first use it would be the longest wait of the epilogue)
  const int my_n = n0 + (int)(threadIdx.x & (BM - 1));
  const float bias = (my_n < p.N && p.bias) ? __ldg(p.bias + my_n) : 0.f;

  bool ok = true;
  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    const int first = min(n_kb, p.stages);  // their boxes of W are on their way already
    pdl_wait();
    EMBER_MARK(kLinearStream, kDependency);
    if (lane == 0) {
      for (int i = 0; i < first; ++i) tma_load_2d(base + i * stage_bytes + kWBox, &map_x, (rank + i * split) * BK, 0, full0 + 8 * i);
      if (p.residual && p.res_by_tma) {  // the residual of this block's own columns and rows, one box
        mbar_expect_tx(res_bar, (unsigned)(q_most * 4 * BM * 4));
        tma_load_2d(res_s, &map_r, n0, 4 * quad_lo(quads, split, rank), res_bar);
      }
    }
    int it = first;
    for (; it < n_kb; ++it) {
      const int s = it % p.stages;
      ok = __all_sync(0xffffffffu, mbar_wait(empty0 + 8 * s, ((it / p.stages) & 1) ^ 1));
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(full0 + 8 * s, (unsigned)stage_bytes);
        tma_load_2d(base + s * stage_bytes, &map_w, (rank + it * split) * BK, n0, full0 + 8 * s);
        tma_load_2d(base + s * stage_bytes + kWBox, &map_x, (rank + it * split) * BK, 0, full0 + 8 * s);
      }
      __syncwarp();
    }
    if (!ok && lane == 0) atomicCAS(p.status, 0, ST_PRODUCER), s_failed = 1;
    // Copies in flight land in this block's shared memory: the block may not end before them.  The
    // `done` barrier covers them (the last product has read the last stage); on the way out after
    // an error the wait simply runs out.
    if (!mbar_wait(done, 0) && ok && lane == 0) atomicCAS(p.status, 0, ST_DRAIN);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ products
    // The whole warp runs the loop with the same values in every lane and one elected lane issues
    // (tc_common.cuh).  A product of N = 64 costs 48 cycles, a box of K four of them.
    const unsigned idesc = instr_desc_bf16(BM, p.mp, false);
    for (int it = 0; it < n_kb && ok; ++it) {
      const int s = it % p.stages;
      ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, (it / p.stages) & 1));
      if (!ok) break;
      fence_after();
      if (it == 0) STREAM_MARK(kPhaseA);  // (timeline only) the first stage has landed
      const unsigned long long dw = smem_desc_sw128(base + s * stage_bytes), dx = smem_desc_sw128(base + s * stage_bytes + kWBox);
#pragma unroll
      for (int k = 0; k < BK / 16; ++k) umma_1cta_elect(tmem, dw + 2 * k, dx + 2 * k, idesc, (it | k) != 0);  // 32 bytes a step
      // a stage is handed back only if it is filled again: a tcgen05.commit costs the issuing warp about
      // 200 cycles (bench.py --umma-issue), as much as the stage's four products
      if (it + p.stages < n_kb) umma_commit_1cta_elect(empty0 + 8 * s);
      if (it == n_kb - 1) umma_commit_1cta_elect(done);
    }
    if (!ok && lane == 0) atomicCAS(p.status, 0, ST_MMA), s_failed = 1;
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ the next product's weights, into L2
    // A product's ring holds three or four boxes of K; the boxes after those are asked for only as the ring
    // turns, and from DRAM each turn costs a microsecond and a half on the step's chain of dependent waits.
    // Asked into L2 one kernel early (by this launch, whose own weights were asked for by the launch before
    // it), they come from there.  Two warps, this block's share of the tensor, 8 KB a request.
    if (p.warm) {
      constexpr unsigned kPiece = 8192;
      const unsigned long long share = ((p.warm_bytes + gridDim.x - 1) / gridDim.x + 15) / 16 * 16;
      const unsigned long long lo = share * blockIdx.x, hi = min(p.warm_bytes, lo + share);
      for (unsigned long long at = lo + (unsigned long long)(threadIdx.x - 6 * 32) * kPiece; at < hi; at += 64ull * kPiece) {
        const unsigned n = (unsigned)min((unsigned long long)kPiece, hi - at);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(p.warm + at), "r"(n) : "memory");
      }
    }
  } else {
    // ------------------------------------------------------------------ the accumulator leaves tensor memory
    const int quarter = warp & 3;              // the 32 lanes of tensor memory this warp may read
    const int row = quarter * 32 + lane;       // row of the tile = output feature n0 + row
    ok = __all_sync(0xffffffffu, mbar_wait(done, 0));
    fence_after();
    if (warp == 2) STREAM_MARK(kPhaseB);  // accumulator complete
    if (!ok && lane == 0) atomicCAS(p.status, 0, ST_EPILOGUE), s_failed = 1;
    if (split > 1) cluster_wait();  // every block of the cluster runs: its shared memory may be written
    // Every quad of columns goes to the block that owns it: this block's own quads into its own shared
    // memory, the others into their owners' with a store that counts its bytes on the owner's barrier
    // when it lands.  16 columns of the accumulator at a time.
    if (ok) {
      const unsigned taddr = tmem + ((unsigned)(quarter * 32) << 16);
      const unsigned mine = recv + (unsigned)((rank * q_most * BM + row) * 16);
      // all of the row's columns are asked for before the first is waited for: one trip to tensor memory
      unsigned a[kMaxRows / 16][16];
#pragma unroll
      for (int i = 0; i < kMaxRows / 16; ++i)
        if (16 * i < p.mp) tmem_ld16(taddr + 16 * i, a[i]);
      tmem_wait();
#pragma unroll
      for (int i = 0; i < kMaxRows / 16; ++i) {
        if (16 * i < p.mp) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int q = 4 * i + j;
            const unsigned owner = s_owner[q], at = mine + (unsigned)(s_local[q] * (BM * 16));
            if ((int)owner == rank)
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(at), "r"(a[i][4 * j]), "r"(a[i][4 * j + 1]),
                           "r"(a[i][4 * j + 2]), "r"(a[i][4 * j + 3])
                           : "memory");
            else
              st_async_f4(map_to_rank(at, owner), a[i][4 * j], a[i][4 * j + 1], a[i][4 * j + 2], a[i][4 * j + 3],
                          map_to_rank(recv_bar, owner));
          }
        }
      }
    }
    if (warp == 2) STREAM_MARK(kMerged);  // (timeline only) partial sums sent
  }
  if ((warp < 2 || warp >= 6) && split > 1) cluster_wait();  // (every thread that arrived at the start also waits)
  __syncthreads();  // this block's own quads are in its shared memory
  bool landed = true;
  if (split > 1) landed = mbar_wait(recv_bar, 0);  // the partners' have landed
  if (warp == 2) STREAM_MARK(kPhaseC);  // partial sums exchanged
  // ------------------------------------------------------------------ all warps: sums, epilogue, stores
  // An item is a quad of this block's columns for one row: its partial sums are added in block order
  // (whichever block this is), then bias, activation and residual, and four stores; a warp's stores
  // cover 32 consecutive features of one sequence.  Thread t keeps row t % 128 in every item it takes.
  {
    const int row = threadIdx.x & (BM - 1);
    const int n = n0 + row;
    const bool n_ok = n < p.N;
    const int q_lo = quad_lo(quads, split, rank), q_n = quad_lo(quads, split, rank + 1) - q_lo;
    const bool res_box = p.residual && p.res_by_tma;
    // (The producer warp passed the dependency wait before anything reached this point, and every
    // thread has met it at a barrier since; only a residual read with plain loads waits itself.)
    if (p.residual && !res_box) pdl_wait();
    bool fine = true;
    if (res_box) fine = mbar_wait(res_bar, 0);  // (awaited in any case: the box lands in this block)
    const float4* part = reinterpret_cast<const float4*>(smem_raw + (recv - smem_u32(smem_raw)));
    const float* res_f = reinterpret_cast<const float*>(smem_raw + (res_s - smem_u32(smem_raw)));
    // One short loop, not unrolled and not specialised: this code runs once per block, and what it
    // costs is fetching it (unrolled twice, in a copy for every activation and every combination of
    // residual and output type, it was 49 KB of the kernel's 79 KB).
    if (!landed && threadIdx.x == 0) atomicCAS(p.status, 0, ST_EPILOGUE);
    if (fine && landed && n_ok && !*reinterpret_cast<volatile int*>(&s_failed)) {
      const int act = p.act;
      const bool with_res = p.residual != nullptr, out_f32 = p.out_f32 != 0;
#pragma unroll 1
      for (int ql = threadIdx.x >> 7; ql < q_n; ql += kThreads / BM) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (int src = 0; src < split; ++src) {
          const float4 r = part[(src * q_most + ql) * BM + row];
          v.x += r.x, v.y += r.y, v.z += r.z, v.w += r.w;
        }
        const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int m = 4 * (q_lo + ql) + j;
          if (m < p.M) {
            float y = vv[j] + bias;
            if (act == EMBER_ACT_GELU_TANH) y = gelu_tanh_fast(y);
            else if (act == EMBER_ACT_GELU_ERF) y = gelu_erf(y);
            const size_t at = (size_t)m * p.N + n;
            if (with_res) y = (res_box ? res_f[(4 * ql + j) * BM + row] : __ldcg(p.residual + at)) + y;
            if (out_f32)
              static_cast<float*>(p.out)[at] = y;
            else
              static_cast<__nv_bfloat16*>(p.out)[at] = __float2bfloat16_rn(y);
          }
        }
      }
    }
    if (warp == 2) STREAM_MARK(kPhaseD);  // (timeline only) this warp's outputs stored
  }
  fence_before();
  __syncthreads();
  EMBER_MARK(kLinearStream, kEnd);
  if (warp == 1) {
    fence_after();
    tmem_free_1cta(tmem, tmem_cols);
  }
}

// ---------------------------------------------------------------------------------------- host
std::mutex g_mutex;
int g_sms = 0;

int stream_setup() {
  if (g_sms) return 0;
  if (!tc::encoder()) return ember_fail("linear_stream: the driver has no cuTensorMapEncodeTiled");
  if (!tc::status().device) return ember_fail("linear_stream: no host-visible status word");
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaError_t e = cudaFuncSetAttribute(linear_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
  if (e != cudaSuccess) return ember_fail("linear_stream: shared memory: %s", cudaGetErrorString(e));
  g_sms = sms;
  return 0;
}

// How many blocks share a tile (split K between them): about one and a half blocks to an SM, which
// is where GPT-2 XL's products of 32 and 64 rows ran fastest as a chain of launches (tiles x blocks:
// 38 x 6, 13 x 8, 50 x 4, 13 x 8; the head's 393 tiles take no split).  Two blocks fit an SM, so
// the blocks of one launch leave room for the first blocks of the next.
int pick_split(int tiles, int kb_all, int sms) {
  int s = (3 * sms + tiles) / (2 * tiles);  // 1.5 sms / tiles, rounded
  if (s > kMaxSplit) s = kMaxSplit;
  if (s > kb_all) s = kb_all;
  return s < 1 ? 1 : s;
}

}  // namespace

// X [M,K] and W [N,K] bfloat16 row-major, 16-byte aligned, K a multiple of 8, 1 <= M <= 64.
// bias: float32 [N] or null.  residual: float32 [M,N] or null (the output is float32 then and may
// be the same buffer).  act: an EMBER_ACT code.  k_split: 0 lets the library choose how many
// blocks share a tile, else 1 to 8.  stages: 0 lets it choose the depth of the ring, else 2 to 10.
// warm, warm_bytes: null and 0, or constants that a kernel soon after this one reads (the next
// product's weight matrix; 16-byte aligned, a multiple of 16 bytes): this launch asks them into L2.
EMBER_API int ember_linear_stream(const void* X, const void* W, const float* bias, const float* residual, void* out, int M,
                                  int N, int K, int act, int out_dtype, int k_split, int stages, const void* warm,
                                  size_t warm_bytes, cudaStream_t stream) {
  EMBER_CHECK(M > 0 && M <= kMaxRows && N > 0 && K > 0, "linear_stream: M = %d (at most %d), N = %d, K = %d", M, kMaxRows, N, K);
  EMBER_CHECK(K % 8 == 0, "linear_stream: K = %d is not a multiple of 8 (rows of 16 bytes)", K);
  EMBER_CHECK(((uintptr_t)X | (uintptr_t)W) % 16 == 0, "linear_stream: operands are not 16-byte aligned");
  EMBER_CHECK(act >= EMBER_ACT_NONE && act <= EMBER_ACT_GELU_ERF, "linear_stream: activation %d", act);
  EMBER_CHECK(out_dtype == EMBER_F32 || out_dtype == EMBER_BF16, "linear_stream: output type %d", out_dtype);
  EMBER_CHECK(!residual || out_dtype == EMBER_F32, "linear_stream: a residual sum needs a float32 output");
  EMBER_CHECK(k_split >= 0 && k_split <= kMaxSplit, "linear_stream: k_split = %d (0 to %d)", k_split, kMaxSplit);
  EMBER_CHECK(stages == 0 || (stages >= 2 && stages <= kMaxStages), "linear_stream: stages = %d (0, or 2 to %d)", stages, kMaxStages);
  EMBER_CHECK(warm_bytes % 16 == 0 && (reinterpret_cast<size_t>(warm) & 15) == 0,
              "linear_stream: what is to be warmed is 16-byte aligned and a multiple of 16 bytes");
  const int tiles = (N + BM - 1) / BM, kb_all = (K + BK - 1) / BK;
  CUtensorMap map_w, map_x, map_r;
  StreamArgs p;
  p.mp = (M + 15) / 16 * 16;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (int rc = stream_setup()) return rc;
  }
  p.k_split = k_split ? (k_split < kb_all ? k_split : kb_all) : pick_split(tiles, kb_all, g_sms);
  if (int rc = tc::cached_map(W, N, K, BM, &map_w)) return rc;
  if (int rc = tc::cached_map(X, M, K, p.mp, &map_x)) return rc;
  const int share = (kb_all + p.k_split - 1) / p.k_split;
  const int stage_bytes = kWBox + p.mp * BK * 2;
  const int quads = p.mp / 4;
  const int q_most = quads_most(quads, p.k_split);
  p.res_by_tma = residual && N % 4 == 0 && (uintptr_t)residual % 16 == 0;
  map_r = map_x;  // a valid map in any case; read only when the residual comes by TMA
  if (p.res_by_tma)
    if (int rc = tc::cached_map_f32(residual, M, N, 4 * q_most, &map_r)) return rc;
  // partial sums (this block's own included) and the residual's box
  const int recv_bytes = p.k_split * q_most * BM * 16 + (p.res_by_tma ? q_most * 4 * BM * 4 : 0);
  // two blocks to an SM when there are more blocks than SMs, else the whole of it
  const int budget = (tiles * p.k_split > g_sms ? 112 : 224) * 1024 - 1024 - recv_bytes;
  int fit = budget / stage_bytes;
  if (fit < 2) fit = 2;
  p.stages = stages ? stages : (fit < share ? fit : share);
  if (p.stages > kMaxStages) p.stages = kMaxStages;
  if (p.stages < 2) p.stages = 2;
  const int smem = 1024 + p.stages * stage_bytes + recv_bytes;
  EMBER_CHECK(smem <= 226 * 1024, "linear_stream: %d stages of %d bytes and %d bytes of partial sums do not fit an SM", p.stages,
              stage_bytes, recv_bytes);
  p.bias = bias, p.residual = residual, p.out = out;
  p.M = M, p.N = N, p.K = K, p.act = act, p.out_f32 = out_dtype == EMBER_F32;
  p.status = tc::status().device;
  p.warm = warm_bytes ? static_cast<const char*>(warm) : nullptr;
  p.warm_bytes = warm_bytes;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * p.k_split);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.k_split, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = pdl_allowed();
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, linear_stream_kernel, map_w, map_x, map_r, p);
  if (e != cudaSuccess) return ember_fail("linear_stream: %s (k_split %d, %d stages)", cudaGetErrorString(e), p.k_split, p.stages);
  EMBER_LAUNCH_OK("linear_stream");
  return 0;
}

EMBER_TIMELINE_READER(linear_stream)
