// Decode attention over the paged cache in bfloat16: one new token per sequence, the keys of a
// sequence split into chunks of pages that separate blocks work through, and the partial results
// merged.
//
// ember.cpp's decode attention is split-K too: a block per (head, chunk) scores its keys, takes
// the chunk's softmax and weighted value sum and writes (m, l, acc[head_dim]) to a scratch array;
// a second kernel merges the chunks in a fixed order,
// out = sum_c e^(m_c - M) acc_c / sum_c e^(m_c - M) l_c (decode_attn_tiled.cuh:58-185,
// cuda_kernels.cu:3117-3134).  This kernel is built for a batch of sequences of unequal length in
// pages and for streaming HBM: grid (chunk, head, token); 128 threads form 16 to 64 independent
// key streams (a key is read by hd/8 lanes, 16 bytes each, K and V in the same pass with an
// online softmax per stream), the streams are merged in shared memory, and the block that
// finishes a (token, head) last merges its chunks, so there is no second launch.  A chunk that
// lies past the token's position or before its window does nothing.
//
// Scratch (given by the caller, reused by every call): per (token, head, chunk) m, l and
// acc[head_dim] in float32, and one counter per (token, head) that is zero between calls.
// The grid covers the pages a sequence can hold at most, so a captured graph serves every length
// up to that.
#include "common.cuh"
#include "attention_common.cuh"

namespace {

constexpr int kThreads = 128;
constexpr int kUnroll = 4;          // keys a stream has in flight
constexpr int kMaxChunkPages = 64;  // page numbers of a chunk kept in shared memory
constexpr int kMergeAtOnce = 8;     // chunks whose partial results the merging block fetches in one batch
static_assert(kMaxChunkPages <= kThreads, "a thread fetches at most one page number of its chunk");

__device__ int g_gave_up = 0;  // set when a block's wait for its bulk copies ran out

// LPK: lanes per key; each lane owns 8 consecutive dims.  BULK: the chunk's keys and values come
// into shared memory by bulk copies, a page's rows for one head each (they are contiguous), two
// pages in flight; else by 16-byte loads into registers.  An SM has far more bytes of bulk copies
// in flight than of loads (a burst of loads of all resident blocks drained at about 30 KB a
// microsecond and SM, whether it came from DRAM or from L2), and the copies of a whole chunk are
// under way before the kernel in front has finished.
template <int LPK, bool BULK>
__global__ void __launch_bounds__(kThreads, BULK ? 6 : 8)
attention_decode_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ kc,
                        const __nv_bfloat16* __restrict__ vc, __nv_bfloat16* __restrict__ out,
                        float* __restrict__ part_ml, float* __restrict__ part_acc, int* __restrict__ counters,
                        const int* __restrict__ positions, const int* __restrict__ token_seq,
                        const int* __restrict__ seq_slot, const int* __restrict__ pages, int max_blocks, int n_heads,
                        int kv_heads, int hd, float scale, int window, int pages_per_chunk, int n_chunks,
                        __nv_bfloat16* __restrict__ k_store, __nv_bfloat16* __restrict__ v_store,
                        const __nv_bfloat16* __restrict__ ahead_k, const __nv_bfloat16* __restrict__ ahead_v) {
  constexpr int kGroups = 32 / LPK;           // key streams per warp
  constexpr int kStreams = 4 * kGroups;       // per block
  __shared__ float s_m[kStreams], s_l[kStreams];
  __shared__ float s_acc[kStreams][LPK * 8 + 1];
  __shared__ float s_w[kStreams];
  __shared__ int s_last;
  __shared__ int s_pages[kMaxChunkPages];
  extern __shared__ __align__(128) unsigned char s_stage[];  // BULK: [2 stages][K, V][kPage][hd]
  __shared__ unsigned long long s_bar[2];                    // BULK: a stage's copies have landed

  // Before waiting for the kernel in front (which makes this step's q, k and v), everything that
  // does not depend on it is fetched: the step's description, which the host wrote before the
  // step began, and the cached keys and values of earlier positions, which earlier steps wrote.
  pdl_trigger();
  // One token per sequence: token t is sequence t of the step (how a one-token-each step is laid
  // out), which spares a dependent load.
  const int c = blockIdx.x, h = blockIdx.y, t = blockIdx.z;
  const int s = t;
  __nv_bfloat16* o = out + ((size_t)t * n_heads + h) * hd;
  // The step's description is three loads that do not depend on one another (the sequence's slot,
  // the token's position, this chunk's page numbers): asked for together they are one trip to L2
  // in front of the keys' fetch, not three.  (A block that starts late, when the kernel in front
  // leaves an SM, has that chain on the step's critical path.)
  const int* my_pages = pages + (size_t)s * max_blocks;
  const bool cached_pages = pages_per_chunk <= kMaxChunkPages;  // at most one page number a thread
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
      for (int d = threadIdx.x; d < hd; d += kThreads) o[d] = __float2bfloat16_rn(0.f);
    return;
  }
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int chunk_keys = pages_per_chunk * kPage;
  const int first_chunk = lo / chunk_keys, last_chunk = p / chunk_keys;
  if (c < first_chunk || c > last_chunk) return;
  EMBER_MARK_START(kAttentionDecode);
  const bool own = k_store != nullptr && c == last_chunk;  // this block also takes the token's own key
  // cached keys of this chunk: [begin, end); the token's own position is not among them when this
  // launch stores it (it is taken from the step's activations instead)
  const int begin = max(lo, c * chunk_keys);
  const int end = min(k_store ? p : p + 1, (c + 1) * chunk_keys);
  const int kvh = h / (n_heads / kv_heads);
  const int width = (n_heads + 2 * kv_heads) * hd;
  if (cached_pages && (int)threadIdx.x < pages_per_chunk) s_pages[threadIdx.x] = my_page;
  if (BULK && threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"((unsigned)__cvta_generic_to_shared(&s_bar[0])));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"((unsigned)__cvta_generic_to_shared(&s_bar[1])));
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sid = warp * kGroups + lane / LPK, sub = lane % LPK;
  const bool dims = sub * 8 < hd;

  uint4 kraw[kUnroll], vraw[kUnroll];
  bool have[kUnroll];
  auto fetch = [&](int j0) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int j = j0 + u * kStreams + sid;
      int page = -1;
      if (j < end) page = cached_pages ? s_pages[j / kPage - c * pages_per_chunk] : my_pages[j / kPage];
      have[u] = page >= 0;
      kraw[u] = make_uint4(0, 0, 0, 0);
      vraw[u] = make_uint4(0, 0, 0, 0);
      if (dims && have[u]) {
        const size_t row = (((size_t)page * kv_heads + kvh) * kPage + (j % kPage)) * hd + sub * 8;
        kraw[u] = *reinterpret_cast<const uint4*>(kc + row);
        vraw[u] = *reinterpret_cast<const uint4*>(vc + row);
      }
    }
  };
  // A cache that this launch stores into holds, below p, only rows of earlier steps: they can be
  // fetched while the kernels in front finish.  A cache that another layer stored into earlier in
  // this same step (this launch only reads it) may not be touched before the wait: kernels that
  // were launched this way can be several deep in their waits.
  // BULK: pages of the chunk that hold keys of [begin, end), and the copy of one of them into a
  // stage (thread 0): rows r0 to r1 of the page, K and then V, counted on the stage's barrier.
  const int first_pg = begin / kPage, last_pg = end > begin ? (end - 1) / kPage : first_pg - 1;
  const unsigned half_stage = (unsigned)kPage * hd * 2;  // bytes of a page's keys for one head
  auto issue = [&](int pg, int st) {
    const int r0 = max(begin, pg * kPage) - pg * kPage, r1 = min(end, (pg + 1) * kPage) - pg * kPage;
    const int page = cached_pages ? s_pages[pg - c * pages_per_chunk] : my_pages[pg];
    const unsigned bytes = page >= 0 ? (unsigned)(r1 - r0) * hd * 2 : 0u;
    const unsigned bar = (unsigned)__cvta_generic_to_shared(&s_bar[st]);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(2u * bytes) : "memory");
    if (bytes) {
      const size_t row = (((size_t)page * kv_heads + kvh) * kPage + r0) * hd;
      const unsigned dst = (unsigned)__cvta_generic_to_shared(s_stage) + (unsigned)st * 2u * half_stage + (unsigned)r0 * hd * 2;
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
                   "l"(kc + row), "r"(bytes), "r"(bar)
                   : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst + half_stage),
                   "l"(vc + row), "r"(bytes), "r"(bar)
                   : "memory");
    }
  };
  if (!k_store) pdl_wait();
  if (BULK) {
    if (threadIdx.x == 0) {
      if (first_pg <= last_pg) issue(first_pg, 0);
      if (first_pg + 1 <= last_pg) issue(first_pg + 1, 1);
    }
  } else {
    fetch(begin);
  }
  if (ahead_k && h % (n_heads / kv_heads) == 0) {
    // The cache of the layer that attends next holds the same rows in the same pages.  Asking them
    // into L2 now, a layer early, turns that layer's trips to DRAM into trips to L2.  One bulk
    // prefetch per page and tensor: a page's rows for one head are contiguous.
    const int first_blk = c * pages_per_chunk;
    for (int i = threadIdx.x; i < 2 * pages_per_chunk; i += kThreads) {
      const int blk = first_blk + (i >> 1);
      const int r0 = max(begin, blk * kPage) - blk * kPage, r1 = min(end, (blk + 1) * kPage) - blk * kPage;
      if (r1 > r0 && blk < max_blocks) {
        const int page = my_pages[blk];
        if (page >= 0) {
          const __nv_bfloat16* at = ((i & 1) ? ahead_v : ahead_k) + (((size_t)page * kv_heads + kvh) * kPage + r0) * hd;
          const unsigned bytes = (unsigned)(r1 - r0) * hd * 2;
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(at), "r"(bytes) : "memory");
        }
      }
    }
  }
  if (k_store) pdl_wait();
  EMBER_MARK(kAttentionDecode, kDependency);

  float2 q[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) q[i] = make_float2(0.f, 0.f);
  if (dims) unpack8(__ldcg(reinterpret_cast<const uint4*>(qkv + (size_t)t * width + (size_t)h * hd + sub * 8)), q);
  uint4 own_k = make_uint4(0, 0, 0, 0), own_v = make_uint4(0, 0, 0, 0);
  if (own) {
    // The token's own key and value: from the step's activations into the cache (no separate
    // launch; blocks of other heads of the same group write the same bytes; nothing in this launch
    // reads the row), and into stream 0 of this block.
    const __nv_bfloat16* src = qkv + (size_t)t * width + (size_t)(n_heads + kvh) * hd;
    const int page = cached_pages ? s_pages[p / kPage - c * pages_per_chunk] : my_pages[p / kPage];
    if (page >= 0) {
      const size_t dst = (((size_t)page * kv_heads + kvh) * kPage + (p % kPage)) * hd;
      const int vecs = hd / 8;
      for (int i = threadIdx.x; i < 2 * vecs; i += kThreads) {
        const bool is_v = i >= vecs;
        const int j = (is_v ? i - vecs : i) * 8;
        const uint4 val = __ldcg(reinterpret_cast<const uint4*>(src + (is_v ? kv_heads * hd : 0) + j));
        *reinterpret_cast<uint4*>((is_v ? v_store : k_store) + dst + j) = val;
      }
    }
    if (sid == 0 && dims) {
      own_k = __ldcg(reinterpret_cast<const uint4*>(src + sub * 8));
      own_v = __ldcg(reinterpret_cast<const uint4*>(src + kv_heads * hd + sub * 8));
    }
  }

  float m = -INFINITY, l = 0.f;
  float2 acc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = make_float2(0.f, 0.f);

  // Every lane of a warp makes the same number of trips (the shuffles name all 32 lanes).  A trip
  // takes kUnroll keys per stream: their loads are issued together, then they are folded into the
  // stream's running softmax one after the other.
  if (BULK) {
    constexpr int kPerStream = kPage / kStreams;                // keys of a page that a stream takes
    constexpr int kTogether = kPerStream < 4 ? kPerStream : 4;  // ... folded together
    for (int pg = first_pg, it = 0; pg <= last_pg; ++pg, ++it) {
      const int st = it & 1;
      {  // the stage's copies have landed (a wait with a limit: a copy that never completes must not hang the GPU)
        const unsigned bar = (unsigned)__cvta_generic_to_shared(&s_bar[st]);
        const unsigned parity = (unsigned)(it >> 1) & 1u;
        unsigned done = 0;
        for (unsigned spin = 0; !done && spin < (1u << 24); ++spin)
          asm volatile(
              "{\n.reg .pred p;\n"
              "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
              "selp.u32 %0, 1, 0, p;\n}\n"
              : "=r"(done)
              : "r"(bar), "r"(parity)
              : "memory");
        if (!done) g_gave_up = 1;  // the results of this launch are not valid; the host asks with ember_attention_decode_status
      }
      const int page = cached_pages ? s_pages[pg - c * pages_per_chunk] : my_pages[pg];
      const unsigned char* ks = s_stage + (size_t)st * 2 * half_stage;
      const unsigned char* vs = ks + half_stage;
#pragma unroll
      for (int b = 0; b < kPerStream / kTogether; ++b) {
        uint4 kr[kTogether], vr[kTogether];
        bool hv[kTogether];
#pragma unroll
        for (int u = 0; u < kTogether; ++u) {
          const int r = sid + (b * kTogether + u) * kStreams;
          const int j = pg * kPage + r;
          hv[u] = page >= 0 && j >= begin && j < end;
          kr[u] = make_uint4(0, 0, 0, 0);
          vr[u] = make_uint4(0, 0, 0, 0);
          if (dims && hv[u]) {
            kr[u] = *reinterpret_cast<const uint4*>(ks + ((size_t)r * hd + sub * 8) * 2);
            vr[u] = *reinterpret_cast<const uint4*>(vs + ((size_t)r * hd + sub * 8) * 2);
          }
        }
        fold_keys<LPK, kTogether>(kr, vr, hv, q, scale, m, l, acc);
      }
      if (pg + 2 <= last_pg) {  // the stage is read: its next page can come
        __syncthreads();
        if (threadIdx.x == 0) issue(pg + 2, st);
      }
    }
  } else {
    for (int j0 = begin; j0 < end; j0 += kUnroll * kStreams) {
      if (j0 != begin) fetch(j0);
      fold_keys<LPK, kUnroll>(kraw, vraw, have, q, scale, m, l, acc);
    }
  }
  if (own && warp == 0) {  // all of warp 0: its shuffles are whole-warp
    const uint4 ok[1] = {own_k}, ov[1] = {own_v};
    const bool oh[1] = {sid == 0};
    fold_keys<LPK, 1>(ok, ov, oh, q, scale, m, l, acc);
  }

  EMBER_MARK(kAttentionDecode, kPhaseA);  // keys folded
  // merge the block's streams
  if (sub == 0) {
    s_m[sid] = m;
    s_l[sid] = l;
  }
  if (dims) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s_acc[sid][sub * 8 + 2 * i] = acc[i].x;
      s_acc[sid][sub * 8 + 2 * i + 1] = acc[i].y;
    }
  }
  __syncthreads();
  float M = -INFINITY;
#pragma unroll
  for (int i = 0; i < kStreams; ++i) M = fmaxf(M, s_m[i]);
  if (threadIdx.x < kStreams) s_w[threadIdx.x] = s_m[threadIdx.x] == -INFINITY ? 0.f : __expf(s_m[threadIdx.x] - M);
  __syncthreads();
  float L = 0.f;
#pragma unroll
  for (int i = 0; i < kStreams; ++i) L += s_l[i] * s_w[i];
  const int n_valid = last_chunk - first_chunk + 1;
  const size_t item = ((size_t)t * n_heads + h) * n_chunks;
  for (int d = threadIdx.x; d < hd; d += kThreads) {
    float A = 0.f;
#pragma unroll
    for (int i = 0; i < kStreams; ++i) A += s_acc[i][d] * s_w[i];
    if (n_valid == 1)
      o[d] = __float2bfloat16_rn(A / L);
    else
      part_acc[(item + c) * hd + d] = A;
  }
  if (n_valid == 1) {
    EMBER_MARK(kAttentionDecode, kEnd);
    return;
  }
  EMBER_MARK(kAttentionDecode, kPhaseB);  // streams merged, partial result on its way
  if (threadIdx.x == 0) {
    part_ml[(item + c) * 2] = M;
    part_ml[(item + c) * 2 + 1] = L;
  }

  // the block that finishes this (token, head) last merges its chunks
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(&counters[t * n_heads + h], 1);
    s_last = done == n_valid - 1;
    if (s_last) counters[t * n_heads + h] = 0;  // zero again for the next call
  }
  __syncthreads();
  EMBER_MARK(kAttentionDecode, kPhaseC);  // ticket taken
  if (!s_last) {
    EMBER_MARK(kAttentionDecode, kEnd);
    return;
  }
  __threadfence();
  if (n_valid <= kMergeAtOnce) {
    // Everything a thread needs of up to kMergeAtOnce chunks is asked for at once: one trip to L2
    // where the loops below make three.  Same sums in the same order.
    for (int d = threadIdx.x; d < hd; d += kThreads) {
      float2 ml[kMergeAtOnce];
      float a[kMergeAtOnce];
#pragma unroll
      for (int i = 0; i < kMergeAtOnce; ++i) {
        const int cc = min(first_chunk + i, last_chunk);
        ml[i] = __ldcg(reinterpret_cast<const float2*>(part_ml + (item + cc) * 2));
        a[i] = __ldcg(&part_acc[(item + cc) * hd + d]);
      }
      float MM = -INFINITY;
#pragma unroll
      for (int i = 0; i < kMergeAtOnce; ++i)
        if (i < n_valid) MM = fmaxf(MM, ml[i].x);
      float LL = 0.f, A = 0.f;
#pragma unroll
      for (int i = 0; i < kMergeAtOnce; ++i) {
        if (i < n_valid) {
          const float w = __expf(ml[i].x - MM);
          LL += ml[i].y * w;
          A += a[i] * w;
        }
      }
      o[d] = __float2bfloat16_rn(A / LL);
    }
    EMBER_MARK(kAttentionDecode, kMerged);
    return;
  }
  float MM = -INFINITY;
  for (int cc = first_chunk; cc <= last_chunk; ++cc) MM = fmaxf(MM, __ldcg(&part_ml[(item + cc) * 2]));
  float LL = 0.f;
  for (int cc = first_chunk; cc <= last_chunk; ++cc)
    LL += __ldcg(&part_ml[(item + cc) * 2 + 1]) * __expf(__ldcg(&part_ml[(item + cc) * 2]) - MM);
  for (int d = threadIdx.x; d < hd; d += kThreads) {
    float A = 0.f;
    for (int cc = first_chunk; cc <= last_chunk; ++cc)
      A += __ldcg(&part_acc[(item + cc) * hd + d]) * __expf(__ldcg(&part_ml[(item + cc) * 2]) - MM);
    o[d] = __float2bfloat16_rn(A / LL);
  }
  EMBER_MARK(kAttentionDecode, kMerged);
}

}  // namespace

// Floats of partial results a call needs: (m, l, acc[hd]) for every (token, head, chunk).
EMBER_API size_t ember_attention_decode_partials(int T, int n_heads, int hd, int n_blocks, int pages_per_chunk) {
  const size_t n_chunks = (size_t)((n_blocks + pages_per_chunk - 1) / pages_per_chunk);
  return (size_t)T * n_heads * n_chunks * (hd + 2);
}

// max_blocks: entries per sequence in `pages`.  n_blocks <= max_blocks: the pages that the
// longest sequence of this call can hold; the grid has a chunk for each pages_per_chunk of them.
// store_kv: write each token's own key and value (from qkv) into the cache before attending.
// partials: ember_attention_decode_partials(...) floats of scratch, contents irrelevant.
// counters: T * n_heads ints of scratch that are zero before the first call; every call leaves
// them zero.  Calls that share scratch must not overlap on the device.
// 0, or 1 if a block of some launch since the last call gave up waiting for its bulk copies (its
// results are not valid); the flag is cleared.  Synchronizes with the device.
EMBER_API int ember_attention_decode_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gave_up, sizeof(int)) != cudaSuccess) return 0;
  if (v) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_gave_up, &zero, sizeof(int));
  }
  return v;
}

// ahead_k, ahead_v: null, or the key and value pages of the layer that attends next (same shape, same
// page table): the rows this call reads are asked into L2 for that layer.
EMBER_API int ember_attention_decode_ahead(const void* qkv, const void* kc, const void* vc, void* out, float* partials,
                                           int* counters, const int* positions, const int* token_seq, const int* seq_slot,
                                           const int* pages, int max_blocks, int n_blocks, int T, int n_heads, int kv_heads,
                                           int hd, float scale, int window, int pages_per_chunk, int store_kv,
                                           const void* ahead_k, const void* ahead_v, cudaStream_t stream) {
  EMBER_CHECK(T > 0 && n_heads > 0 && kv_heads > 0 && max_blocks > 0 && n_blocks > 0 && n_blocks <= max_blocks,
              "attention_decode: bad sizes");
  EMBER_CHECK(n_heads % kv_heads == 0, "attention_decode: %d heads are not a multiple of %d key/value heads", n_heads,
              kv_heads);
  EMBER_CHECK(hd % 16 == 0 && hd >= 16 && hd <= 256, "attention_decode: head size %d is not a multiple of 16 in [16, 256]",
              hd);
  EMBER_CHECK(window >= 0 && pages_per_chunk > 0, "attention_decode: window %d, pages per chunk %d", window,
              pages_per_chunk);
  EMBER_CHECK(T <= 65535 && n_heads <= 65535, "attention_decode: %d tokens x %d heads exceed one launch", T, n_heads);
  const int n_chunks = (n_blocks + pages_per_chunk - 1) / pages_per_chunk;
  const size_t items = (size_t)T * n_heads;
  float* part_ml = partials;
  float* part_acc = part_ml + items * n_chunks * 2;
  dim3 grid(n_chunks, n_heads, T);
  cudaError_t e;
  // Bulk copies for head sizes up to 128 (two stages of a page's keys and values: 512 bytes per
  // value of the head size); the option EMBER_OPT_DECODE_BULK switched off takes the loads (for measurements).
  const bool bulk_allowed = g_ember_options[EMBER_OPT_DECODE_BULK] != 0;
  const bool bulk = bulk_allowed && hd <= 128;
  const size_t smem = bulk ? (size_t)4 * kPage * hd * 2 : 0;
#define EMBER_DECODE(LPK)                                                                                           \
  if (bulk) {                                                                                                       \
    static size_t configured = 0;                                                                                   \
    if (smem > 48 * 1024 && smem > configured) {                                                                    \
      e = cudaFuncSetAttribute(attention_decode_kernel<LPK, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                               (int)smem);                                                                          \
      if (e != cudaSuccess) return ember_fail("attention_decode: %s", cudaGetErrorString(e));                       \
      configured = smem;                                                                                            \
    }                                                                                                               \
    e = launch_pdl(attention_decode_kernel<LPK, true>, grid, dim3(kThreads), smem, stream, EMBER_DECODE_ARGS);      \
  } else {                                                                                                          \
    e = launch_pdl(attention_decode_kernel<LPK, false>, grid, dim3(kThreads), 0, stream, EMBER_DECODE_ARGS);        \
  }
#define EMBER_DECODE_ARGS                                                                                           \
  (const __nv_bfloat16*)qkv,                                                                                        \
                 (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, (__nv_bfloat16*)out, part_ml, part_acc, counters, \
                 positions, token_seq, seq_slot, pages, max_blocks, n_heads, kv_heads, hd, scale, window,           \
                 pages_per_chunk, n_chunks, store_kv ? (__nv_bfloat16*)kc : (__nv_bfloat16*)nullptr,                 \
                 store_kv ? (__nv_bfloat16*)vc : (__nv_bfloat16*)nullptr, (const __nv_bfloat16*)ahead_k,                \
                 (const __nv_bfloat16*)ahead_v
  if (hd <= 16) { EMBER_DECODE(2) }
  else if (hd <= 32) { EMBER_DECODE(4) }
  else if (hd <= 64) { EMBER_DECODE(8) }
  else if (hd <= 128) { EMBER_DECODE(16) }
  else e = launch_pdl(attention_decode_kernel<32, false>, grid, dim3(kThreads), 0, stream, EMBER_DECODE_ARGS);
#undef EMBER_DECODE
#undef EMBER_DECODE_ARGS
  if (e != cudaSuccess) return ember_fail("attention_decode: %s", cudaGetErrorString(e));
  return 0;
}

EMBER_API int ember_attention_decode(const void* qkv, const void* kc, const void* vc, void* out, float* partials,
                                     int* counters, const int* positions, const int* token_seq, const int* seq_slot,
                                     const int* pages, int max_blocks, int n_blocks, int T, int n_heads, int kv_heads,
                                     int hd, float scale, int window, int pages_per_chunk, int store_kv,
                                     cudaStream_t stream) {
  return ember_attention_decode_ahead(qkv, kc, vc, out, partials, counters, positions, token_seq, seq_slot, pages,
                                      max_blocks, n_blocks, T, n_heads, kv_heads, hd, scale, window, pages_per_chunk,
                                      store_kv, nullptr, nullptr, stream);
}

// ---------------------------------------------------------------------------- without allocation
// ember_attention_decode_static: the same decode attention for callers that must not allocate
// device memory.  It has no counterpart in ember.cpp; see ember_kernels.h for who needs it.
//
// The split kernel above needs scratch (partial results per (token, head, chunk), and a counter per
// (token, head)).  Here that scratch is two file-scope __device__ arrays of fixed size, which every
// GPU that loads this library holds from load until the process exits (4 MiB + 64 KiB).  In host
// code the arrays' names are only stand-ins, not device addresses, so their addresses are asked
// for once per device with cudaGetSymbolAddress, on that device, and kept.  That happens in the
// first call on a device, which should therefore come before any stream capture.
namespace {

constexpr size_t kStaticPartialFloats = (size_t)1 << 20;  // 4 MiB of partial results
constexpr int kStaticCounters = 1 << 14;                  // 16,384 (token, head) pairs

static __device__ __align__(256) float g_static_partials[kStaticPartialFloats];
static __device__ __align__(256) int g_static_counters[kStaticCounters];

constexpr int kMaxDevices = 64;
float* g_partials_on[kMaxDevices] = {};
int* g_counters_on[kMaxDevices] = {};

}  // namespace

EMBER_API int ember_attention_decode_static(const void* qkv, const void* kc, const void* vc, void* out,
                                            const int* positions, const int* token_seq, const int* seq_slot,
                                            const int* pages, int max_blocks, int n_blocks, int T, int n_heads,
                                            int kv_heads, int hd, float scale, int window, int pages_per_chunk,
                                            int store_kv, cudaStream_t stream) {
  EMBER_CHECK(T > 0 && n_heads > 0 && hd > 0 && n_blocks > 0 && pages_per_chunk > 0, "attention_decode_static: bad sizes");
  const size_t need = ember_attention_decode_partials(T, n_heads, hd, n_blocks, pages_per_chunk);
  EMBER_CHECK(need <= kStaticPartialFloats,
              "attention_decode_static: %d tokens x %d heads x %d chunks of head size %d need %zu floats of scratch, the "
              "built-in scratch holds %zu; use more pages per chunk or the entry point that takes scratch",
              T, n_heads, (n_blocks + pages_per_chunk - 1) / pages_per_chunk, hd, need, kStaticPartialFloats);
  EMBER_CHECK((long long)T * n_heads <= kStaticCounters,
              "attention_decode_static: %d tokens x %d heads exceed the built-in scratch's %d (token, head) pairs", T,
              n_heads, kStaticCounters);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return ember_fail("attention_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
  EMBER_CHECK(dev >= 0 && dev < kMaxDevices, "attention_decode_static: device %d", dev);
  if (!g_partials_on[dev]) {  // set-up, once per device, with that device current
    float* p = nullptr;
    int* c = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_static_partials);
    if (e != cudaSuccess) return ember_fail("attention_decode_static: address of the scratch: %s", cudaGetErrorString(e));
    e = cudaGetSymbolAddress((void**)&c, g_static_counters);
    if (e != cudaSuccess) return ember_fail("attention_decode_static: address of the counters: %s", cudaGetErrorString(e));
    g_counters_on[dev] = c;
    g_partials_on[dev] = p;
  }
  // The arrays keep what the last call left.  Partials are always written before they are read;
  // the counters must start at zero, so they are cleared here on the caller's stream.
  e = cudaMemsetAsync(g_counters_on[dev], 0, (size_t)T * n_heads * sizeof(int), stream);
  if (e != cudaSuccess) return ember_fail("attention_decode_static: clearing the counters: %s", cudaGetErrorString(e));
  return ember_attention_decode(qkv, kc, vc, out, g_partials_on[dev], g_counters_on[dev], positions, token_seq,
                                seq_slot, pages, max_blocks, n_blocks, T, n_heads, kv_heads, hd, scale, window,
                                pages_per_chunk, store_kv, stream);
}

EMBER_TIMELINE_READER(attention_decode)
