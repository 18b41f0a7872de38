// Decode attention over the paged cache on the tensor cores (bfloat16, head size 64 or 128): one
// new token per sequence, split over chunks of pages like attention_decode.cu, whose scratch and
// merge it shares in form.
//
// The kernel of attention_decode.cu scores a key with eight lanes' multiply-adds and shuffles; with
// every key and value unpacked to float32 it issues about 40 instructions a key and lane, and at
// batch 8 and up that, not memory, is what its time goes to.  Here a warp takes a whole page of 64
// keys: S = Q K^T and O += P V are mma.sync m16n8k16 products (the rows of Q are the query heads
// that share the key/value head, up to 8; for plain multi-head attention one row of 16 is used,
// which wastes a tensor pipe that is idle anyway), about 150 instructions a page and warp.
//
// A block is two warps, a page each at a time, or four where chunks are three pages and longer and
// three such blocks an SM hold the whole launch (head size 64): every page of a short chunk is then
// on its way from the block's first instruction, and a context of up to four pages is one block with
// nothing to merge.  A page's keys and values for one head are one TMA box each (64 rows of 128
// bytes, 128-byte swizzle, so that ldmatrix reads them without bank conflicts), requested before the
// kernel in front is waited for; a warp that has more than one page in its chunk refills its own
// stage.  Every wait has a limit, after which the launch's results are marked invalid
// (ember_attention_decode_status).
#include <cooperative_groups.h>

#include <unordered_map>

#include "common.cuh"
#include "tc_common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int kMaxCluster = 8;      // chunks of a (token, head) that can merge through distributed shared memory
constexpr int kMaxChunkPages = 64;  // page numbers of a chunk kept in shared memory
constexpr int kMergeAtOnce = 8;     // chunks whose partial results the merging block fetches in one batch
constexpr int kMaxGroup = 8;        // query heads per key/value head that a block takes as rows

__device__ int g_gave_up = 0;  // set when a warp's wait for its page ran out

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const unsigned*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16(unsigned w) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
}
// exp2 of a difference that may be -inf - (-inf): what has seen no key weighs nothing
__device__ __forceinline__ float weight(float m, float top) { return m == -INFINITY ? 0.f : exp2f(m - top); }

// Byte offset of (row, 16-byte chunk) in a box of 64 rows of 128 bytes under the 128-byte swizzle.
__device__ __forceinline__ unsigned swz(int row, int chunk) { return (unsigned)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

// CLUSTER: the chunks of a (token, head) are the blocks of one thread-block cluster (plain multi-head
// attention, at most 8 chunks): each writes its partial result into the shared memory of the block
// that holds the token's own key and arrives at the cluster's barrier; that block waits for the
// barrier and merges.  No scratch in global memory, no ticket, no second trip to L2.  Every block
// of a cluster that is not padding arrives exactly once, whatever it finds to do.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }

// W: the block's warps (2 or 4), a page each at a time.
template <int HD, bool CLUSTER, int W>
__global__ void __launch_bounds__(W * 32, W == 2 ? 6 : 3)
attention_decode_mma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ out,
                            float* __restrict__ part_ml, float* __restrict__ part_acc, int* __restrict__ counters,
                            const int* __restrict__ positions, const int* __restrict__ seq_slot,
                            const int* __restrict__ pages, int max_blocks, int n_heads, int kv_heads, float scale_log2,
                            int window, int pages_per_chunk, int n_chunks, __nv_bfloat16* __restrict__ k_store,
                            __nv_bfloat16* __restrict__ v_store, const __nv_bfloat16* __restrict__ ahead_k,
                            const __nv_bfloat16* __restrict__ ahead_v) {
  constexpr int kWarps = W, kThreads = W * 32;
  static_assert(kMaxChunkPages <= kThreads, "a thread fetches at most one page number of its chunk");
  constexpr int KS = HD / 16;                   // 16-wide steps over the head's dims
  constexpr int kBoxes = HD / 64;               // TMA boxes (64 dims wide) of a page's keys
  constexpr unsigned kBox = kPage * 128;        // bytes of a box
  constexpr unsigned kStage = 2 * kBoxes * kBox;  // a page's keys, then its values
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_pages[kMaxChunkPages];
  __shared__ __align__(8) unsigned long long s_bar[kWarps];
  __shared__ int s_last;
  __shared__ float s_part[CLUSTER ? kMaxCluster : 1][HD + 2];  // CLUSTER: the chunks' results, in the merging block

  pdl_trigger();
  const int c = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
  const int s = t;  // one token per sequence: token t is sequence t of the step
  const int group = n_heads / kv_heads;  // query heads of this key/value head: rows of the products
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c2 = (lane & 3) * 2;
  // the step's description: three loads that do not depend on one another, one trip to L2
  const int* my_pages = pages + (size_t)s * max_blocks;
  const bool cached_pages = pages_per_chunk <= kMaxChunkPages;
  const int slot = seq_slot[s];
  const int p = positions[t];
  int my_page = -1;
  if (cached_pages && (int)threadIdx.x < pages_per_chunk) {
    const int blk = c * pages_per_chunk + threadIdx.x;
    if (blk < max_blocks) my_page = my_pages[blk];
  }
  if (slot < 0) {  // padding: a defined output, nothing read
    pdl_wait();
    if (c == 0)
      for (int i = threadIdx.x; i < group * HD; i += kThreads)
        out[((size_t)t * n_heads + (size_t)kvh * group) * HD + i] = __float2bfloat16_rn(0.f);
    return;
  }
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int chunk_keys = pages_per_chunk * kPage;
  const int first_chunk = lo / chunk_keys, last_chunk = p / chunk_keys;
  if (c < first_chunk || c > last_chunk) {
    if (CLUSTER) cluster_arrive();
    return;
  }
  EMBER_MARK_START(kAttentionDecode);
  const bool own = k_store != nullptr && c == last_chunk;  // this block also takes the token's own key
  const int begin = max(lo, c * chunk_keys);
  const int end = min(k_store ? p : p + 1, (c + 1) * chunk_keys);
  const int width = (n_heads + 2 * kv_heads) * HD;
  if (cached_pages && (int)threadIdx.x < pages_per_chunk) s_pages[threadIdx.x] = my_page;
  const unsigned bar = tc::smem_u32(&s_bar[warp]);
  if (lane == 0) {
    tc::mbar_init(bar, 1);
    tc::mbar_init_fence();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    tc::prefetch_map(&map_k);
    tc::prefetch_map(&map_v);
  }

  const unsigned stage = ((tc::smem_u32(smem_raw) + 1023u) & ~1023u) + (unsigned)warp * kStage;  // this warp's
  const int first_pg = begin / kPage, last_pg = end > begin ? (end - 1) / kPage : first_pg - 1;
  auto page_of = [&](int pg) { return cached_pages ? s_pages[pg - c * pages_per_chunk] : my_pages[pg]; };
  // lane 0: the whole page (rows past `end` are masked later), keys then values, 64 dims a box
  auto issue = [&](int pg) {
    const int page = page_of(pg);
    if (page < 0) {
      tc::mbar_arrive(bar);  // nothing comes: the phase completes at once
      return;
    }
    const int row = (page * kv_heads + kvh) * kPage;
    tc::mbar_expect_tx(bar, kStage);
#pragma unroll
    for (int b = 0; b < kBoxes; ++b) {
      tc::tma_load_2d(stage + b * kBox, &map_k, b * 64, row, bar);
      tc::tma_load_2d(stage + (kBoxes + b) * kBox, &map_v, b * 64, row, bar);
    }
  };
  // A cache that this launch stores into holds, below p, only rows of earlier steps: they can be
  // fetched while the kernels in front finish.  One that another layer stored into earlier in this
  // step may not be touched before the wait.
  if (!k_store) pdl_wait();
  if (lane == 0 && first_pg + warp <= last_pg) issue(first_pg + warp);
  if (ahead_k) {
    // The cache of the layer that attends next holds the same rows in the same pages: asked into L2
    // now, a layer early, that layer's boxes (above all those a warp fetches after its first) come
    // from there.  One bulk prefetch per page and tensor, a lane each.
    for (int i = threadIdx.x; i < 2 * (last_pg - first_pg + 1); i += kThreads) {
      const int page = page_of(first_pg + (i >> 1));
      if (page >= 0) {
        const __nv_bfloat16* at = ((i & 1) ? ahead_v : ahead_k) + ((size_t)page * kv_heads + kvh) * kPage * HD;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(at), "r"((unsigned)(kPage * HD * 2)) : "memory");
      }
    }
  }
  if (k_store) pdl_wait();
  EMBER_MARK(kAttentionDecode, kDependency);

  // Q as A fragments: row g is query head kvh * group + g (rows from `group` on are zero)
  unsigned qf[KS][4];
  {
    const __nv_bfloat16* q = qkv + (size_t)t * width + ((size_t)kvh * group + g) * HD;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      qf[ks][0] = g < group ? __ldcg(reinterpret_cast<const unsigned*>(q + ks * 16 + c2)) : 0u;
      qf[ks][2] = g < group ? __ldcg(reinterpret_cast<const unsigned*>(q + ks * 16 + 8 + c2)) : 0u;
      qf[ks][1] = qf[ks][3] = 0u;
    }
  }
  // the token's own key and value, from the step's activations: the dims this lane holds of Q
  // (asked for now, beside Q: one trip to L2 for all three)
  unsigned own_k[KS][2], own_v[2 * KS];
  if (own && warp == 0) {
    const __nv_bfloat16* ksrc = qkv + (size_t)t * width + (size_t)(n_heads + kvh) * HD;
    const __nv_bfloat16* vsrc = ksrc + (size_t)kv_heads * HD;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      own_k[ks][0] = __ldcg(reinterpret_cast<const unsigned*>(ksrc + ks * 16 + c2));
      own_k[ks][1] = __ldcg(reinterpret_cast<const unsigned*>(ksrc + ks * 16 + 8 + c2));
    }
#pragma unroll
    for (int i = 0; i < 2 * KS; ++i) own_v[i] = __ldcg(reinterpret_cast<const unsigned*>(vsrc + i * 8 + c2));
  }
  if (own) {
    // The token's own key and value go from the step's activations into the cache (nothing in this
    // launch reads the row: the page's box brings whatever it held, and the row is masked).
    const __nv_bfloat16* src = qkv + (size_t)t * width + (size_t)(n_heads + kvh) * HD;
    const int page = page_of(p / kPage);
    if (page >= 0) {
      const size_t dst = (((size_t)page * kv_heads + kvh) * kPage + (p % kPage)) * HD;
      constexpr int vecs = HD / 8;
      for (int i = threadIdx.x; i < 2 * vecs; i += kThreads) {
        const bool is_v = i >= vecs;
        const int j = (is_v ? i - vecs : i) * 8;
        const uint4 val = __ldcg(reinterpret_cast<const uint4*>(src + (is_v ? kv_heads * HD : 0) + j));
        *reinterpret_cast<uint4*>((is_v ? v_store : k_store) + dst + j) = val;
      }
    }
  }

  float o[2 * KS][4];
#pragma unroll
  for (int i = 0; i < 2 * KS; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;  // of row g, scores in base 2; l is this lane's share until the end

  for (int pg = first_pg + warp, it = 0; pg <= last_pg; pg += kWarps, ++it) {
    if (!tc::mbar_wait(bar, (unsigned)it & 1u)) g_gave_up = 1;  // the results of this launch are not valid
    if (page_of(pg) >= 0) {
      // S = Q K^T: 8 tiles of 8 keys
      float sc[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) sc[i][j] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          unsigned b[4];
          const int row = np * 16 + (lane & 7) + (lane >> 4) * 8;
          const int chunk = ks * 2 + ((lane >> 3) & 1);  // 16-byte chunk of the row's dims
          ldmatrix_x4(b, stage + (chunk >> 3) * kBox + swz(row, chunk & 7));
          mma_bf16(sc[2 * np], qf[ks], b[0], b[1]);
          mma_bf16(sc[2 * np + 1], qf[ks], b[2], b[3]);
        }
      }
      // scale, mask what lies outside [begin, end), the row's maximum
      const int key0 = pg * kPage;
      const bool edge = key0 < begin || key0 + kPage > end;
      float m_new = m_run;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int key = key0 + i * 8 + c2 + j;
          sc[i][j] = (!edge || (key >= begin && key < end)) ? sc[i][j] * scale_log2 : -INFINITY;
          m_new = fmaxf(m_new, sc[i][j]);
        }
      }
      m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, 1));
      m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, 2));
      const float base = m_new == -INFINITY ? 0.f : m_new;  // a row that has seen no key: nothing is NaN
      const float corr = weight(m_run, base);
      m_run = m_new;
      l_run *= corr;
#pragma unroll
      for (int i = 0; i < 2 * KS; ++i) {
        o[i][0] *= corr;
        o[i][1] *= corr;
      }
      unsigned pf[4][4];  // P as A fragments: 4 groups of 16 keys; rows 8 to 15 are not used
      float row_sum = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float e0 = exp2f(sc[i][0] - base), e1 = exp2f(sc[i][1] - base);
        row_sum += e0 + e1;
        pf[i >> 1][(i & 1) * 2] = pack_bf16(e0, e1);
        pf[i >> 1][(i & 1) * 2 + 1] = 0u;
      }
      l_run += row_sum;
      // O += P V
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
        for (int dn = 0; dn < KS; ++dn) {
          unsigned b[4];
          const int row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int chunk = dn * 2 + (lane >> 4);
          ldmatrix_x4_trans(b, stage + (kBoxes + (chunk >> 3)) * kBox + swz(row, chunk & 7));
          mma_bf16(o[2 * dn], pf[kk], b[0], b[1]);
          mma_bf16(o[2 * dn + 1], pf[kk], b[2], b[3]);
        }
      }
    }
    if (pg + kWarps <= last_pg) {  // the stage is read: this warp's next page can come
      __syncwarp();
      if (lane == 0) {
        tc::fence_async_smem();
        issue(pg + kWarps);
      }
    }
  }
  if (own && warp == 0) {
    float dot = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const float2 q0 = unpack_bf16(qf[ks][0]), q1 = unpack_bf16(qf[ks][2]);
      const float2 k0 = unpack_bf16(own_k[ks][0]), k1 = unpack_bf16(own_k[ks][1]);
      dot += (q0.x * k0.x + q0.y * k0.y) + (q1.x * k1.x + q1.y * k1.y);
    }
    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    dot += __shfl_xor_sync(0xffffffffu, dot, 2);
    const float sc = dot * scale_log2;
    const float m_new = fmaxf(m_run, sc);
    const float corr = weight(m_run, m_new), pj = exp2f(sc - m_new);
    m_run = m_new;
    l_run = l_run * corr + ((lane & 3) == 0 ? pj : 0.f);
#pragma unroll
    for (int i = 0; i < 2 * KS; ++i) {
      const float2 v = unpack_bf16(own_v[i]);
      o[i][0] = o[i][0] * corr + pj * v.x;
      o[i][1] = o[i][1] * corr + pj * v.y;
    }
  }
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  EMBER_MARK(kAttentionDecode, kPhaseA);  // keys folded

  // the warps' results, over the stages (every warp is done with them)
  float* s_m = reinterpret_cast<float*>(smem_raw);   // [kWarps][kMaxGroup]
  float* s_l = s_m + kWarps * kMaxGroup;             // [kWarps][kMaxGroup]
  float* s_acc = s_l + kWarps * kMaxGroup;           // [kWarps][kMaxGroup][HD]
  __syncthreads();
  if (g < group) {
    if ((lane & 3) == 0) {
      s_m[warp * kMaxGroup + g] = m_run;
      s_l[warp * kMaxGroup + g] = l_run;
    }
#pragma unroll
    for (int i = 0; i < 2 * KS; ++i) {
      s_acc[(warp * kMaxGroup + g) * HD + i * 8 + c2] = o[i][0];
      s_acc[(warp * kMaxGroup + g) * HD + i * 8 + c2 + 1] = o[i][1];
    }
  }
  __syncthreads();
  const int n_valid = last_chunk - first_chunk + 1;
  for (int i = threadIdx.x; i < group * HD; i += kThreads) {
    const int row = i / HD, d = i % HD;
    const int h = kvh * group + row;
    float M = s_m[row];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) M = fmaxf(M, s_m[w * kMaxGroup + row]);
    float L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {  // in warp order
      const float ww = weight(s_m[w * kMaxGroup + row], M);
      L += s_l[w * kMaxGroup + row] * ww;
      A += s_acc[(w * kMaxGroup + row) * HD + d] * ww;
    }
    const size_t item = ((size_t)t * n_heads + h) * n_chunks + c;
    if (n_valid == 1) {
      out[((size_t)t * n_heads + h) * HD + d] = __float2bfloat16_rn(A / L);
    } else if (CLUSTER) {  // one query head a block: row 0
      float* mine = c == last_chunk ? &s_part[c - first_chunk][0]
                                    : cg::this_cluster().map_shared_rank(&s_part[c - first_chunk][0], last_chunk);
      mine[d] = A;
      if (d == 0) {
        mine[HD] = M;
        mine[HD + 1] = L;
      }
    } else {
      part_acc[item * HD + d] = A;
      if (d == 0) {
        part_ml[item * 2] = M;
        part_ml[item * 2 + 1] = L;
      }
    }
  }
  if (CLUSTER) {
    cluster_arrive();
    if (n_valid == 1 || c != last_chunk) {
      EMBER_MARK(kAttentionDecode, kEnd);
      return;
    }
    cluster_wait();  // every chunk's result is in s_part
    for (int d = threadIdx.x; d < HD; d += kThreads) {
      float MM = -INFINITY, LL = 0.f, A = 0.f;
      for (int k = 0; k < n_valid; ++k) MM = fmaxf(MM, s_part[k][HD]);
      for (int k = 0; k < n_valid; ++k) {
        const float w = weight(s_part[k][HD], MM);
        LL += s_part[k][HD + 1] * w;
        A += s_part[k][d] * w;
      }
      out[((size_t)t * n_heads + kvh) * HD + d] = __float2bfloat16_rn(A / LL);
    }
    EMBER_MARK(kAttentionDecode, kMerged);
    return;
  }
  if (n_valid == 1) {
    EMBER_MARK(kAttentionDecode, kEnd);
    return;
  }
  EMBER_MARK(kAttentionDecode, kPhaseB);  // partial result on its way

  // the block that finishes this (token, key/value head) last merges its chunks
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* counter = &counters[t * n_heads + kvh * group];
    const int done = atomicAdd(counter, 1);
    s_last = done == n_valid - 1;
    if (s_last) *counter = 0;  // zero again for the next call
  }
  __syncthreads();
  EMBER_MARK(kAttentionDecode, kPhaseC);  // ticket taken
  if (!s_last) {
    EMBER_MARK(kAttentionDecode, kEnd);
    return;
  }
  __threadfence();
  for (int i = threadIdx.x; i < group * HD; i += kThreads) {
    const int row = i / HD, d = i % HD;
    const int h = kvh * group + row;
    const size_t item = ((size_t)t * n_heads + h) * n_chunks;
    float MM = -INFINITY, LL = 0.f, A = 0.f;
    if (n_valid <= kMergeAtOnce) {  // everything asked for at once: one trip to L2
      float2 ml[kMergeAtOnce];
      float a[kMergeAtOnce];
#pragma unroll
      for (int k = 0; k < kMergeAtOnce; ++k) {
        const int cc = min(first_chunk + k, last_chunk);
        ml[k] = __ldcg(reinterpret_cast<const float2*>(part_ml + (item + cc) * 2));
        a[k] = __ldcg(&part_acc[(item + cc) * HD + d]);
      }
#pragma unroll
      for (int k = 0; k < kMergeAtOnce; ++k)
        if (k < n_valid) MM = fmaxf(MM, ml[k].x);
#pragma unroll
      for (int k = 0; k < kMergeAtOnce; ++k) {
        if (k < n_valid) {
          const float w = weight(ml[k].x, MM);
          LL += ml[k].y * w;
          A += a[k] * w;
        }
      }
    } else {
      for (int cc = first_chunk; cc <= last_chunk; ++cc) MM = fmaxf(MM, __ldcg(&part_ml[(item + cc) * 2]));
      for (int cc = first_chunk; cc <= last_chunk; ++cc) {
        const float w = weight(__ldcg(&part_ml[(item + cc) * 2]), MM);
        LL += __ldcg(&part_ml[(item + cc) * 2 + 1]) * w;
        A += __ldcg(&part_acc[(item + cc) * HD + d]) * w;
      }
    }
    out[((size_t)t * n_heads + h) * HD + d] = __float2bfloat16_rn(A / LL);
  }
  EMBER_MARK(kAttentionDecode, kMerged);
}

struct MapKey {
  const void* ptr;
  long long rows;
  int cols;
  bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols; }
};
struct MapHash {
  size_t operator()(const MapKey& k) const {
    size_t h = 1469598103934665603ull;
    h = (h ^ reinterpret_cast<size_t>(k.ptr)) * 1099511628211ull;
    h = (h ^ (size_t)k.rows) * 1099511628211ull;
    return (h ^ (size_t)k.cols) * 1099511628211ull;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapHash> g_maps;  // a layer's cache comes back with every step

// [rows, hd] bfloat16 (rows = pages x key/value heads x 64), boxes of 64 rows x 64 dims
int cache_map(const void* ptr, long long rows, int hd, CUtensorMap* out) {
  const MapKey key{ptr, rows, hd};
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return 0;
  }
  CUtensorMap m;
  if (!tc::encode_bf16_sw128(&m, ptr, (size_t)rows, (size_t)hd, (size_t)hd * 2, kPage))
    return ember_fail("attention_decode_mma: the driver refused a tensor map for [%lld, %d]", rows, hd);
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps.emplace(key, m);
  *out = m;
  return 0;
}

template <int HD, int W>
int launch(const CUtensorMap& map_k, const CUtensorMap& map_v, const void* qkv, void* kc, void* vc, void* out,
           float* part_ml, float* part_acc, int* counters, const int* positions, const int* seq_slot, const int* pages,
           int max_blocks, int n_chunks, int T, int n_heads, int kv_heads, float scale, int window, int pages_per_chunk,
           int store_kv, const void* ahead_k, const void* ahead_v, cudaStream_t stream) {
  constexpr size_t smem = (size_t)W * 2 * (HD / 64) * kPage * 128 + 1024;
  static bool configured = false;  // per instantiation
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_mma_kernel<HD, false, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_decode_mma_kernel<HD, true, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ember_fail("attention_decode_mma: %s", cudaGetErrorString(e));
    configured = true;
  }
  // the option EMBER_OPT_DECODE_CLUSTER switched off merges through global scratch and a ticket (for measurements)
  const bool cluster_allowed = g_ember_options[EMBER_OPT_DECODE_CLUSTER] != 0;
  const bool cluster = cluster_allowed && n_heads == kv_heads && n_chunks >= 2 && n_chunks <= kMaxCluster;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_chunks, kv_heads, T);
  cfg.blockDim = dim3(W * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[0].val.programmaticStreamSerializationAllowed = pdl_allowed();
  attrs[1].id = cudaLaunchAttributeClusterDimension;
  attrs[1].val.clusterDim.x = n_chunks;
  attrs[1].val.clusterDim.y = 1;
  attrs[1].val.clusterDim.z = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = cluster ? 2 : 1;
  const __nv_bfloat16* q = (const __nv_bfloat16*)qkv;
  __nv_bfloat16* o = (__nv_bfloat16*)out;
  const float scale_log2 = scale * 1.4426950408889634f;
  __nv_bfloat16* ks = store_kv ? (__nv_bfloat16*)kc : (__nv_bfloat16*)nullptr;
  __nv_bfloat16* vs = store_kv ? (__nv_bfloat16*)vc : (__nv_bfloat16*)nullptr;
  const __nv_bfloat16* ak = (const __nv_bfloat16*)ahead_k;
  const __nv_bfloat16* av = (const __nv_bfloat16*)ahead_v;
  cudaError_t e =
      cluster ? cudaLaunchKernelEx(&cfg, attention_decode_mma_kernel<HD, true, W>, map_k, map_v, q, o, part_ml, part_acc, counters,
                                   positions, seq_slot, pages, max_blocks, n_heads, kv_heads, scale_log2, window,
                                   pages_per_chunk, n_chunks, ks, vs, ak, av)
              : cudaLaunchKernelEx(&cfg, attention_decode_mma_kernel<HD, false, W>, map_k, map_v, q, o, part_ml, part_acc, counters,
                                   positions, seq_slot, pages, max_blocks, n_heads, kv_heads, scale_log2, window,
                                   pages_per_chunk, n_chunks, ks, vs, ak, av);
  if (e != cudaSuccess) return ember_fail("attention_decode_mma: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace

// 0, or 1 if a warp of some launch since the last call gave up waiting for a page's keys and values
// (its results are not valid); the flag is cleared.  Synchronizes with the device.
EMBER_API int ember_attention_decode_mma_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gave_up, sizeof(int)) != cudaSuccess) return 0;
  if (v) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_gave_up, &zero, sizeof(int));
  }
  return v;
}

// The arguments of ember_attention_decode_ahead, and n_pages, the pages that kc and vc hold.  Returns 2
// (and launches nothing) for what this kernel has no instantiation for: a head size other than 64
// or 128, more than 8 query heads to a key/value head.
EMBER_API int ember_attention_decode_mma(const void* qkv, void* kc, void* vc, void* out, float* partials, int* counters,
                                         const int* positions, const int* token_seq, const int* seq_slot,
                                         const int* pages, int max_blocks, int n_blocks, int n_pages, int T, int n_heads,
                                         int kv_heads, int hd, float scale, int window, int pages_per_chunk, int store_kv,
                                         const void* ahead_k, const void* ahead_v, cudaStream_t stream) {
  (void)token_seq;
  EMBER_CHECK(T > 0 && n_heads > 0 && kv_heads > 0 && max_blocks > 0 && n_blocks > 0 && n_blocks <= max_blocks && n_pages > 0,
              "attention_decode_mma: bad sizes");
  EMBER_CHECK(n_heads % kv_heads == 0, "attention_decode_mma: %d heads are not a multiple of %d key/value heads", n_heads,
              kv_heads);
  EMBER_CHECK(window >= 0 && pages_per_chunk > 0, "attention_decode_mma: window %d, pages per chunk %d", window,
              pages_per_chunk);
  EMBER_CHECK(T <= 65535 && kv_heads <= 65535, "attention_decode_mma: %d tokens x %d heads exceed one launch", T, kv_heads);
  if ((hd != 64 && hd != 128) || n_heads / kv_heads > kMaxGroup) return 2;
  if (!tc::encoder()) return 2;
  const int n_chunks = (n_blocks + pages_per_chunk - 1) / pages_per_chunk;
  const size_t items = (size_t)T * n_heads;
  float* part_ml = partials;
  float* part_acc = part_ml + items * n_chunks * 2;
  CUtensorMap map_k, map_v;
  const long long rows = (long long)n_pages * kv_heads * kPage;
  if (cache_map(kc, rows, hd, &map_k) || cache_map(vc, rows, hd, &map_v)) return 1;
  // Chunks of three or four pages take four warps, a page each, so that all of a chunk's pages are on their
  // way from the block's first instruction (head size 64; three such blocks fit an SM).
  if (hd == 64 && pages_per_chunk >= 3 && (long long)n_chunks * kv_heads * T <= 3LL * sm_count())
    return launch<64, 4>(map_k, map_v, qkv, kc, vc, out, part_ml, part_acc, counters, positions, seq_slot, pages, max_blocks,
                         n_chunks, T, n_heads, kv_heads, scale, window, pages_per_chunk, store_kv, ahead_k, ahead_v, stream);
  if (hd == 64)
    return launch<64, 2>(map_k, map_v, qkv, kc, vc, out, part_ml, part_acc, counters, positions, seq_slot, pages, max_blocks,
                         n_chunks, T, n_heads, kv_heads, scale, window, pages_per_chunk, store_kv, ahead_k, ahead_v, stream);
  return launch<128, 2>(map_k, map_v, qkv, kc, vc, out, part_ml, part_acc, counters, positions, seq_slot, pages, max_blocks,
                        n_chunks, T, n_heads, kv_heads, scale, window, pages_per_chunk, store_kv, ahead_k, ahead_v, stream);
}

EMBER_TIMELINE_READER(attention_decode_mma)
