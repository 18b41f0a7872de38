// Prefill attention on the fifth-generation tensor cores (head size 64): the new tokens of each
// sequence against all keys up to their own positions, read from the paged cache, causal, with an
// optional window.  The same function as attention_prefill.cu (mma.sync), which stays as the
// kernel for other head sizes and as this one's twin in the tests.
//
// ember.cpp's prefill attention is a float32 flash kernel on the CUDA cores: 64 (token, head)
// rows against 32-key tiles, online softmax, 1/l at the end (cuda_kernels.cu:2276-2428).  Here a
// block takes 128 consecutive new tokens of one (sequence, head) and walks the cache's 64-key
// pages:
//
//   warp 0        TMA: the query tile once, then a key page and a value page per step into a ring
//                 of stages (`cp.async.bulk.tensor.2d`, 128-byte swizzle; a page of one head is
//                 64 rows of 128 bytes, exactly one box);
//   warp 1        `tcgen05.mma`: S = Q K^T (128 x 64, K-major operands) into one of two score
//                 buffers in tensor memory, a step ahead of the softmax, and, once the softmax
//                 warps have written P, O += P V (V read MN-major: the page as it lies in the
//                 cache) into the output accumulator, which stays in tensor memory;
//   warps 2 to 5  softmax, a query row a thread: `tcgen05.ld` of the row's 64 scores, mask by
//                 selection, maximum and sum in float32 (no shuffles: the row is in one thread),
//                 P in bfloat16 into shared memory in the swizzled layout the tensor core reads.
//                 The exponents are taken against a maximum that is moved (and O and l rescaled,
//                 `tcgen05.ld`/`st`) only when the true maximum has grown by more than 2^8 since:
//                 the sums stay consistent and O is rarely touched.  1/l at the end.
//
// Two blocks fit an SM, so one block's products run under the other's softmax.  Every wait on an
// mbarrier has a time limit (tc_common.cuh); a role whose wait runs out records a code and leaves,
// and the block frees its tensor memory and returns.
#include "tc_common.cuh"

namespace {

constexpr int HD = 64;         // head size: a row of Q, K or V is 128 bytes, one swizzle atom
constexpr int kQRows = 128;    // query rows a block
constexpr int kKeys = 64;      // keys a step: one page
constexpr int kStages = 3;     // key/value pages in flight
constexpr int kThreads = 192;  // loader warp, product warp, 4 softmax warps
constexpr int kTmemCols = 256;  // S (two buffers) at columns 0 and 64, O at column 128
constexpr int kQBytes = kQRows * HD * 2, kPageBytes = kKeys * HD * 2, kPBytes = kQRows * kKeys * 2;
constexpr int kSmem = 1024 + kQBytes + kStages * 2 * kPageBytes + 2 * kPBytes;
constexpr float kRescale = 8.0f;  // O and l are rescaled only when a row's maximum grows by more than 2^8

enum : int { ATT_LOADER = 11, ATT_PRODUCTS = 12, ATT_SOFTMAX = 13 };

struct AttArgs {
  __nv_bfloat16* out;
  const int* seq_slot;
  const int* seq_start;
  const int* seq_new;
  const int* cu_new;
  const int* pages;
  int max_blocks, n_heads, kv_heads, window, n_pages, n_seqs, n_tiles;
  float scale_log2;
  int* status;
};

__device__ __forceinline__ void tmem_st32(unsigned taddr, const unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::
          "r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
      "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
      "r"(r[31])
      : "memory");
}
__device__ __forceinline__ float ex2(float x) {  // 2^x, one instruction; results below 2^-126 are zero
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
// The largest of three, one instruction (sm_100).
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Two float32 operations an instruction (sm_100's packed forms; each half is the ordinary IEEE operation).
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n.reg .b64 ra, rb, rc, rd;\n"
      "mov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\nmov.b64 rc, {%6, %7};\n"
      "fma.rn.f32x2 rd, ra, rb, rc;\n"
      "mov.b64 {%0, %1}, rd;\n}\n"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("{\n.reg .b64 ra, rb, rd;\n"
      "mov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\n"
      "add.rn.f32x2 rd, ra, rb;\n"
      "mov.b64 {%0, %1}, rd;\n}\n"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

__global__ void __launch_bounds__(kThreads, 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const AttArgs p) {
  using namespace tc;
  extern __shared__ unsigned char smem_raw[];
  // barriers: q_full, kv_full[3], kv_empty[3], s_full[2], s_free[2], p_full[2], pv_done[2]
  __shared__ unsigned long long bars[15];
  __shared__ unsigned s_tmem;

  // Blocks are handed out in the order of their numbers.  The last tiles of a sequence have the
  // most keys before them, so the numbering goes by tile first, last tiles first, and inside a
  // tile over heads and sequences: the long blocks all start at once and the short ones fill in.
  const int per_tile = p.n_heads * p.n_seqs;
  const int tile = p.n_tiles - 1 - (int)blockIdx.x / per_tile;
  const int h = ((int)blockIdx.x % per_tile) % p.n_heads, s = ((int)blockIdx.x % per_tile) / p.n_heads;
  const int n_new = p.seq_new[s];
  if (tile * kQRows >= n_new) return;
  const int rows = min(kQRows, n_new - tile * kQRows);
  const int tok0 = p.cu_new[s] + tile * kQRows;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t out_width = (size_t)p.n_heads * HD;
  if (p.seq_slot[s] < 0) {  // padding: defined output, nothing read
    for (int i = threadIdx.x; i < rows * HD; i += kThreads)
      p.out[(size_t)(tok0 + i / HD) * out_width + (size_t)h * HD + i % HD] = __float2bfloat16_rn(0.f);
    return;
  }
  const int p0 = p.seq_start[s] + tile * kQRows;  // position of the tile's first row
  const int p_last = p0 + rows - 1;
  const int kb_first = p.window > 0 ? max(0, p0 - p.window + 1) / kKeys : 0;
  const int kb_last = p_last / kKeys;
  const int n_steps = kb_last - kb_first + 1;
  const int kvh = h / (p.n_heads / p.kv_heads);
  const int* my_pages = p.pages + (size_t)s * p.max_blocks;

  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const unsigned sQ = base, sKV = sQ + kQBytes, sP = sKV + kStages * 2 * kPageBytes;
  const unsigned bar0 = smem_u32(bars);
  const unsigned q_full = bar0, kv_full = bar0 + 8, kv_empty = bar0 + 32, s_full = bar0 + 56, s_free = bar0 + 72,
                 p_full = bar0 + 88, pv_done = bar0 + 104;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(kv_full + 8 * i, 1);
      mbar_init(kv_empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(s_full + 8 * i, 1);
      mbar_init(s_free + 8 * i, 4);
      mbar_init(p_full + 8 * i, 4);
      mbar_init(pv_done + 8 * i, 1);
    }
    mbar_init_fence();
    prefetch_map(&map_q);
    prefetch_map(&map_k);
    prefetch_map(&map_v);
  }
  if (warp == 1) tmem_alloc_1cta(smem_u32(&s_tmem), kTmemCols);
  fence_before();
  __syncthreads();
  fence_after();
  const unsigned tmem = s_tmem;

  if (warp == 0) {
    // ------------------------------------------------------------------ loader
    bool ok = true;
    if (lane == 0) {
      mbar_expect_tx(q_full, kQBytes);
      tma_load_2d(sQ, &map_q, h * HD, tok0, q_full);
    }
    int it = 0;
    for (; it < n_steps; ++it) {
      const int st = it % kStages;
      ok = mbar_wait(kv_empty + 8 * st, ((it / kStages) & 1) ^ 1);
      if (!ok) break;
      if (lane == 0) {
        int page = my_pages[kb_first + it];
        if (page < 0 || page >= p.n_pages) page = 0;  // a page the sequence does not hold: its keys are masked anyway
        const int row = (page * p.kv_heads + kvh) * kKeys;
        const unsigned dst = sKV + st * 2 * kPageBytes;
        mbar_expect_tx(kv_full + 8 * st, 2 * kPageBytes);
        tma_load_2d(dst, &map_k, 0, row, kv_full + 8 * st);
        tma_load_2d(dst + kPageBytes, &map_v, 0, row, kv_full + 8 * st);
      }
      __syncwarp();
    }
    if (!ok && lane == 0) atomicCAS(p.status, 0, ATT_LOADER);
    // copies land in this block's shared memory: the block may not end before them.  A stage is
    // handed back only after its copies landed and were used.
    for (int j = max(0, it - kStages); j < it; ++j)
      if (!mbar_wait(kv_empty + 8 * (j % kStages), (j / kStages) & 1)) break;
  } else if (warp == 1) {
    // ------------------------------------------------------------------ products
    // S of step j+1 is issued before P of step j is waited for: the scores of the next page are
    // ready when the softmax warps come for them.
    const unsigned idesc_s = instr_desc_bf16(kQRows, kKeys, false), idesc_o = instr_desc_bf16(kQRows, HD, true);
    const unsigned long long dq = smem_desc_sw128(sQ);
    bool ok = __all_sync(0xffffffffu, mbar_wait(q_full, 0));
    auto issue_s = [&](int it) -> bool {  // S[it & 1] = Q K_it^T
      const int st = it % kStages, b = it & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(kv_full + 8 * st, (it / kStages) & 1) && mbar_wait(s_free + 8 * b, ((it >> 1) & 1) ^ 1)))
        return false;
      fence_after();
      // every lane holds the same operands and one elected lane issues (tc_common.cuh)
      const unsigned long long dk = smem_desc_sw128(sKV + st * 2 * kPageBytes);
#pragma unroll
      for (int k = 0; k < HD / 16; ++k) umma_1cta_elect(tmem + 64 * b, dq + 2 * k, dk + 2 * k, idesc_s, k != 0);  // 32 bytes of a row a step
      umma_commit_1cta_elect(s_full + 8 * b);
      return true;
    };
    if (ok) ok = issue_s(0);
    for (int it = 0; it < n_steps && ok; ++it) {
      const int st = it % kStages, b = it & 1;
      if (it + 1 < n_steps) ok = issue_s(it + 1);
      if (!ok) break;
      ok = __all_sync(0xffffffffu, mbar_wait(p_full + 8 * b, (it >> 1) & 1));
      if (!ok) break;
      fence_after();
      const unsigned long long dp = smem_desc_sw128(sP + b * kPBytes);
      const unsigned long long dv = smem_desc_sw128(sKV + st * 2 * kPageBytes + kPageBytes);
#pragma unroll
      for (int k = 0; k < kKeys / 16; ++k)  // 16 keys a step: 32 bytes of a row of P, 16 rows (2,048 bytes) of V
        umma_1cta_elect(tmem + 128, dp + 2 * k, dv + 128 * k, idesc_o, (it | k) != 0);
      umma_commit_1cta_elect(pv_done + 8 * b);
      umma_commit_1cta_elect(kv_empty + 8 * st);
    }
    if (!ok && lane == 0) atomicCAS(p.status, 0, ATT_PRODUCTS);
  } else {
    // ------------------------------------------------------------------ softmax: thread = query row
    const int quarter = warp & 3;  // the 32 tensor-memory lanes this warp may read
    const int r = quarter * 32 + lane;
    const int pos = p0 + r;
    const unsigned taddr = tmem + ((unsigned)(quarter * 32) << 16);
    unsigned char* p_rows = smem_raw + (sP - smem_u32(smem_raw)) + r * 128;
    // m_used: the maximum the exponents are taken against.  It follows the true running maximum
    // only when that has grown by more than 2^kRescale since (then O and l are rescaled): all sums
    // stay consistent, and O, which lives in tensor memory, is touched rarely.
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int it = 0; it < n_steps; ++it) {
      const int b = it & 1;
      const int key0 = (kb_first + it) * kKeys;
      ok = mbar_wait(s_full + 8 * b, (it >> 1) & 1);
      if (!ok) break;
      fence_after();
      unsigned sc[2][32];
      tmem_ld32(taddr + 64 * b, sc[0]);
      tmem_ld32(taddr + 64 * b + 32, sc[1]);
      tmem_wait();
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free + 8 * b);
      // Most pages lie wholly before every row of the tile (and inside every row's window): only
      // the pages on the diagonal and at the window's edge are masked, by selection.
      const bool all_seen = key0 + kKeys - 1 <= p0 && (p.window <= 0 || key0 > p_last - p.window);
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains, not one of 64 links
      if (all_seen) {
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
          for (int c = 0; c < 32; c += 2)
            m4[(c >> 1) & 3] = max3(m4[(c >> 1) & 3], __uint_as_float(sc[half][c]), __uint_as_float(sc[half][c + 1]));
      } else {
        const int hi = pos - key0;                                            // keys with index <= hi
        const int lo = p.window > 0 ? pos - p.window + 1 - key0 : -(1 << 30);  // and >= lo
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int key = half * 32 + c;
            const float v = (key <= hi && key >= lo) ? __uint_as_float(sc[half][c]) : -INFINITY;
            sc[half][c] = __float_as_uint(v);
            m4[c & 3] = fmaxf(m4[c & 3], v);
          }
      }
      const float m_blk = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      const bool grow = m_blk > m_used && (m_used == -INFINITY || (m_blk - m_used) * p.scale_log2 > kRescale);
      float corr = 1.0f;
      if (grow) {
        corr = m_used == -INFINITY ? 0.f : ex2((m_used - m_blk) * p.scale_log2);
        m_used = m_blk;
        l_run *= corr;
      }
      // O holds something to rescale only after the first step, and only for rows that had a maximum
      const bool scale_o = grow && corr != 0.f && it > 0;
      if (__any_sync(0xffffffffu, scale_o)) {
        ok = mbar_wait(pv_done + 8 * (b ^ 1), ((it - 1) >> 1) & 1);  // the products of the step before are complete
        if (!ok) break;
        fence_after();
        const float f = scale_o ? corr : 1.0f;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          unsigned ov[32];
          tmem_ld32(taddr + 128 + 32 * half, ov);
          tmem_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * f);
          tmem_st32(taddr + 128 + 32 * half, ov);
        }
        tmem_wait_st();
        fence_before();
      }
      // a row that has seen no key yet keeps m = -inf; its exponent base is 0 so that nothing is NaN
      const float base_e = m_used == -INFINITY ? 0.f : m_used * p.scale_log2;
      // The buffer of P is free once the products of two steps ago have read it, and they have: the scores of
      // this step were issued after them, the tensor core finishes a block's products in the order they were
      // issued, and this step's scores were waited for above (their commit covers everything issued before).
      unsigned char* p_row = p_rows + b * kPBytes;
      float2 sum4[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
      const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), minus_base2 = make_float2(-base_e, -base_e);
      // (Half of the powers of two as a polynomial of degree 5 on the FMA pipe, so that the special-function
      // unit has 32 and not 64 a row: 25.7 against 25.2 microseconds a launch.  The unit is not what a step
      // waits for.)
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {  // 8 keys: one 16-byte chunk of the row of P
          unsigned w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 t = fma2(make_float2(__uint_as_float(sc[half][c8 * 8 + 2 * j]), __uint_as_float(sc[half][c8 * 8 + 2 * j + 1])),
                                  scale2, minus_base2);
            const float2 e = make_float2(ex2(t.x), ex2(t.y));
            sum4[j] = add2(sum4[j], e);
            const __nv_bfloat162 v2 = __floats2bfloat162_rn(e.x, e.y);
            w[j] = *reinterpret_cast<const unsigned*>(&v2);
          }
          const int chunk = half * 4 + c8;
          *reinterpret_cast<uint4*>(p_row + ((chunk ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      l_run += ((sum4[0].x + sum4[0].y) + (sum4[1].x + sum4[1].y)) + ((sum4[2].x + sum4[2].y) + (sum4[3].x + sum4[3].y));
      fence_async_smem();  // P is read by the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + 8 * b);
    }
    if (ok) ok = mbar_wait(pv_done + 8 * ((n_steps - 1) & 1), ((n_steps - 1) >> 1) & 1);
    if (!ok) {
      if (lane == 0) atomicCAS(p.status, 0, ATT_SOFTMAX);
    } else {
      fence_after();
      const float inv = 1.0f / l_run;
      __nv_bfloat16* dst = p.out + (size_t)(tok0 + r) * out_width + (size_t)h * HD;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        unsigned ov[32];
        tmem_ld32(taddr + 128 + 32 * half, ov);  // every lane of the warp takes part, whatever its row
        tmem_wait();
        if (r < rows) {
#pragma unroll
          for (int c8 = 0; c8 < 4; ++c8) {
            unsigned w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __nv_bfloat162 v2 = __floats2bfloat162_rn(__uint_as_float(ov[c8 * 8 + 2 * j]) * inv,
                                                              __uint_as_float(ov[c8 * 8 + 2 * j + 1]) * inv);
              w[j] = *reinterpret_cast<const unsigned*>(&v2);
            }
            *reinterpret_cast<uint4*>(dst + half * 32 + c8 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      fence_before();
    }
  }

  fence_before();
  __syncthreads();
  if (warp == 1) {
    fence_after();
    tmem_free_1cta(tmem, kTmemCols);
  }
}

}  // namespace

// Arguments as ember_attention_prefill, with the number of rows of qkv (`n_tokens`) and of pages in
// the cache (`n_pages`) that the tensor maps need.  Returns 0 on success, 1 on an error, 2 if the
// kernel does not take this head size or these pointers (the caller then takes the mma.sync kernel).
EMBER_API int ember_attention_prefill_tc(const void* qkv, const void* kc, const void* vc, void* out, const int* seq_slot,
                                         const int* seq_start, const int* seq_new, const int* cu_new, const int* pages,
                                         int max_blocks, int n_seqs, int max_new, int n_tokens, int n_pages, int n_heads,
                                         int kv_heads, int hd, float scale, int window, cudaStream_t stream) {
  if (hd != HD) return 2;
  EMBER_CHECK(n_seqs > 0 && max_new > 0 && n_tokens > 0 && n_pages > 0 && n_heads > 0 && kv_heads > 0 && max_blocks > 0,
              "attention_prefill_tc: bad sizes");
  EMBER_CHECK(n_heads % kv_heads == 0, "attention_prefill_tc: %d heads are not a multiple of %d key/value heads", n_heads,
              kv_heads);
  EMBER_CHECK(n_seqs <= 65535 && n_heads <= 65535, "attention_prefill_tc: %d sequences x %d heads exceed one launch", n_seqs,
              n_heads);
  EMBER_CHECK(window >= 0 && scale > 0.f, "attention_prefill_tc: window %d, scale %g", window, (double)scale);
  if (((uintptr_t)qkv | (uintptr_t)kc | (uintptr_t)vc | (uintptr_t)out) % 16) return 2;
  tc::Status& st = tc::status();
  if (!st.device || !tc::encoder()) return 2;
  const size_t width = (size_t)(n_heads + 2 * kv_heads) * HD;
  CUtensorMap map_q, map_k, map_v;
  if (!tc::encode_bf16_sw128(&map_q, qkv, (size_t)n_tokens, width, width * 2, kQRows) ||
      !tc::encode_bf16_sw128(&map_k, kc, (size_t)n_pages * kv_heads * kKeys, HD, HD * 2, kKeys) ||
      !tc::encode_bf16_sw128(&map_v, vc, (size_t)n_pages * kv_heads * kKeys, HD, HD * 2, kKeys))
    return ember_fail("attention_prefill_tc: the driver refused a tensor map");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return ember_fail("attention_prefill_tc: %s", cudaGetErrorString(e));
    configured = true;
  }
  AttArgs a;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.seq_slot = seq_slot, a.seq_start = seq_start, a.seq_new = seq_new, a.cu_new = cu_new, a.pages = pages;
  a.max_blocks = max_blocks, a.n_heads = n_heads, a.kv_heads = kv_heads, a.window = window, a.n_pages = n_pages;
  a.n_seqs = n_seqs, a.n_tiles = (max_new + kQRows - 1) / kQRows;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = st.device;
  const long long blocks = (long long)a.n_tiles * n_heads * n_seqs;
  EMBER_CHECK(blocks < (1ll << 31), "attention_prefill_tc: %lld blocks exceed one launch", blocks);
  dim3 grid((unsigned)blocks);
  attention_tc_kernel<<<grid, kThreads, kSmem, stream>>>(map_q, map_k, map_v, a);
  EMBER_LAUNCH_OK("attention_prefill_tc");
  return 0;
}
