// Prefill attention in bfloat16 on the tensor cores: the new tokens of each sequence against all
// keys up to their own positions, read from the paged cache, causal, with an optional window.
//
// ember.cpp's prefill attention is a float32 flash kernel on the CUDA cores: 64 (token, head)
// rows against 32-key tiles, online softmax, 1/l at the end (cuda_kernels.cu:2276-2428).  The same
// scheme here with bfloat16 operands on mma.sync m16n8k16 and float32 softmax and accumulators: a
// block takes 64 consecutive new tokens of one (sequence, head); each of its 4 warps owns 16 query
// rows; key blocks are the cache's 64-position pages, brought in with cp.async into a double
// buffer while the previous page is used.  The keys of a page beyond a query's position (or before
// its window) are masked by selection, never by arithmetic on what the page holds.
//
// Head sizes: multiples of 16 up to 128 (one instantiation each); larger heads take the plain
// kernel.
#include "common.cuh"

namespace {

constexpr int kThreads = 128;
constexpr int kRows = 64;  // query rows per block, and keys per page

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}

// A 64 x HD tile into shared memory rows of HD + 8 elements.  Rows at or past `valid_rows` are
// zero-filled.
template <int HD>
__device__ __forceinline__ void load_tile(__nv_bfloat16* dst, const __nv_bfloat16* src, size_t row_stride,
                                          int valid_rows) {
  constexpr int LD = HD + 8, CPR = HD / 8;
  for (int id = threadIdx.x; id < kRows * CPR; id += kThreads) {
    const int r = id / CPR, c = id % CPR;
    const bool ok = r < valid_rows;
    cp_async_16(dst + r * LD + c * 8, src + (ok ? (size_t)r * row_stride : 0) + c * 8, ok);
  }
}

template <int HD>
__global__ void __launch_bounds__(kThreads)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ kc,
                         const __nv_bfloat16* __restrict__ vc, __nv_bfloat16* __restrict__ out,
                         const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                         const int* __restrict__ seq_new, const int* __restrict__ cu_new,
                         const int* __restrict__ pages, int max_blocks, int n_heads, int kv_heads, float scale_log2,
                         int window) {
  constexpr int LD = HD + 8, KS = HD / 16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sK = sQ + kRows * LD;      // [2][64][LD]
  __nv_bfloat16* sV = sK + 2 * kRows * LD;  // [2][64][LD]

  // the last tiles of a sequence have the most keys before them: they are handed out first, so that the
  // launch does not end on a few long blocks
  const int tile = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, s = blockIdx.z;
  const int n_new = seq_new[s];
  if (tile * kRows >= n_new) return;
  const int rows = min(kRows, n_new - tile * kRows);
  const int tok0 = cu_new[s] + tile * kRows;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c2 = (lane & 3) * 2;
  const size_t out_width = (size_t)n_heads * HD;
  if (seq_slot[s] < 0) {  // padding: defined output, nothing read
    for (int i = threadIdx.x; i < rows * HD; i += kThreads)
      out[(size_t)(tok0 + i / HD) * out_width + (size_t)h * HD + i % HD] = __float2bfloat16_rn(0.f);
    return;
  }
  const int p0 = seq_start[s] + tile * kRows;  // position of the tile's first row
  const int p_last = p0 + rows - 1;
  const int kb_first = window > 0 ? max(0, p0 - window + 1) / kRows : 0;
  const int kb_last = p_last / kRows;
  const int kvh = h / (n_heads / kv_heads);
  const size_t qkv_width = (size_t)(n_heads + 2 * kv_heads) * HD;
  const int* my_pages = pages + (size_t)s * max_blocks;
  auto page_base = [&](int kb) { return ((size_t)max(my_pages[kb], 0) * kv_heads + kvh) * kRows * HD; };

  load_tile<HD>(sQ, qkv + (size_t)tok0 * qkv_width + (size_t)h * HD, qkv_width, rows);
  load_tile<HD>(sK, kc + page_base(kb_first), HD, kRows);
  load_tile<HD>(sV, vc + page_base(kb_first), HD, kRows);
  cp_async_commit();

  unsigned qf[KS][4];
  float o[2 * KS][4];
#pragma unroll
  for (int i = 0; i < 2 * KS; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int row_pos[2] = {p0 + warp * 16 + g, p0 + warp * 16 + g + 8};  // positions of this thread's two rows

  for (int kb = kb_first; kb <= kb_last; ++kb) {
    const int buf = (kb - kb_first) & 1;
    if (kb + 1 <= kb_last) {
      load_tile<HD>(sK + (buf ^ 1) * kRows * LD, kc + page_base(kb + 1), HD, kRows);
      load_tile<HD>(sV + (buf ^ 1) * kRows * LD, vc + page_base(kb + 1), HD, kRows);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (kb == kb_first) {
#pragma unroll
      for (int ks = 0; ks < KS; ++ks)
        ldmatrix_x4(qf[ks], sQ + (warp * 16 + (lane & 15)) * LD + ks * 16 + (lane >> 4) * 8);
    }
    const __nv_bfloat16* tK = sK + buf * kRows * LD;
    const __nv_bfloat16* tV = sV + buf * kRows * LD;

    // S = Q K^T for this warp's 16 rows and the page's 64 keys: 8 tiles of 8 keys
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
        ldmatrix_x4(b, tK + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(sc[2 * np], qf[ks], b[0], b[1]);
        mma_bf16(sc[2 * np + 1], qf[ks], b[2], b[3]);
      }
    }

    // mask by selection where the page crosses a query's position or its window's start
    const int key0 = kb * kRows;
    const bool need_mask = key0 + kRows - 1 > p0 + warp * 16 || (window > 0 && key0 < p_last - window + 1);
    if (need_mask) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int key = key0 + i * 8 + c2 + (j & 1);
          const int pos = row_pos[j >> 1];
          const bool seen = key <= pos && (window <= 0 || key > pos - window);
          if (!seen) sc[i][j] = -INFINITY;
        }
    }

    // online softmax in float32 (scores scaled into base 2)
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      m_new[0] = fmaxf(m_new[0], fmaxf(sc[i][0], sc[i][1]));
      m_new[1] = fmaxf(m_new[1], fmaxf(sc[i][2], sc[i][3]));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
      m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
    }
    float corr[2], base[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      // a row that has seen no key yet keeps m = -inf; its exponent base is 0 so that nothing is NaN
      base[r] = m_new[r] == -INFINITY ? 0.f : m_new[r] * scale_log2;
      corr[r] = m_run[r] == -INFINITY ? 0.f : exp2f(m_run[r] * scale_log2 - base[r]);
      m_run[r] = m_new[r];
      l_run[r] *= corr[r];
    }
#pragma unroll
    for (int i = 0; i < 2 * KS; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
    unsigned pf[4][4];  // P as A fragments: 4 groups of 16 keys
    float row_sum[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float e0 = exp2f(sc[i][0] * scale_log2 - base[0]), e1 = exp2f(sc[i][1] * scale_log2 - base[0]);
      const float e2 = exp2f(sc[i][2] * scale_log2 - base[1]), e3 = exp2f(sc[i][3] * scale_log2 - base[1]);
      row_sum[0] += e0 + e1;
      row_sum[1] += e2 + e3;
      pf[i >> 1][(i & 1) * 2] = pack_bf16(e0, e1);
      pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(e2, e3);
    }
    l_run[0] += row_sum[0];
    l_run[1] += row_sum[1];

    // O += P V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
      for (int dn = 0; dn < KS; ++dn) {
        unsigned b[4];
        ldmatrix_x4_trans(b, tV + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + dn * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * dn], pf[kk], b[0], b[1]);
        mma_bf16(o[2 * dn + 1], pf[kk], b[2], b[3]);
      }
    }
    __syncthreads();  // the other buffer is refilled at the top of the next trip
  }

  // 1 / l and the store; the sums of a row live in its four lanes
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + g + r * 8;
    if (row >= rows) continue;
    const float inv = 1.0f / l_run[r];
    __nv_bfloat16* dst = out + (size_t)(tok0 + row) * out_width + (size_t)h * HD;
#pragma unroll
    for (int i = 0; i < 2 * KS; ++i) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
      *reinterpret_cast<__nv_bfloat162*>(dst + i * 8 + c2) = v;
    }
  }
}

template <int HD>
int launch(const void* qkv, const void* kc, const void* vc, void* out, const int* seq_slot, const int* seq_start,
           const int* seq_new, const int* cu_new, const int* pages, int max_blocks, int n_seqs, int max_new,
           int n_heads, int kv_heads, float scale, int window, cudaStream_t stream) {
  const int smem = 5 * kRows * (HD + 8) * (int)sizeof(__nv_bfloat16);
  static bool configured = false;  // per instantiation
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return ember_fail("attention_prefill: %s", cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid((max_new + kRows - 1) / kRows, n_heads, n_seqs);
  attention_prefill_kernel<HD><<<grid, kThreads, smem, stream>>>(
      (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, (__nv_bfloat16*)out, seq_slot,
      seq_start, seq_new, cu_new, pages, max_blocks, n_heads, kv_heads, scale * 1.4426950408889634f, window);
  EMBER_LAUNCH_OK("attention_prefill");
  return 0;
}

}  // namespace

// Returns 0 on success, 1 on an error, 2 if this head size has no tensor-core instantiation (the
// caller then takes the plain kernel).
EMBER_API int ember_attention_prefill(const void* qkv, const void* kc, const void* vc, void* out, const int* seq_slot,
                                      const int* seq_start, const int* seq_new, const int* cu_new, const int* pages,
                                      int max_blocks, int n_seqs, int max_new, int n_heads, int kv_heads, int hd,
                                      float scale, int window, cudaStream_t stream) {
  EMBER_CHECK(n_seqs > 0 && max_new > 0 && n_heads > 0 && kv_heads > 0 && max_blocks > 0, "attention_prefill: bad sizes");
  EMBER_CHECK(n_heads % kv_heads == 0, "attention_prefill: %d heads are not a multiple of %d key/value heads", n_heads,
              kv_heads);
  EMBER_CHECK(hd % 16 == 0 && hd >= 16 && hd <= 256, "attention_prefill: head size %d is not a multiple of 16 in [16, 256]",
              hd);
  EMBER_CHECK(n_seqs <= 65535 && n_heads <= 65535, "attention_prefill: %d sequences x %d heads exceed one launch", n_seqs,
              n_heads);
  EMBER_CHECK(window >= 0, "attention_prefill: window %d", window);
  EMBER_CHECK(scale > 0.f, "attention_prefill: scale %g is not positive", (double)scale);
#define EMBER_PREFILL(HD)                                                                                           \
  case HD:                                                                                                          \
    return launch<HD>(qkv, kc, vc, out, seq_slot, seq_start, seq_new, cu_new, pages, max_blocks, n_seqs, max_new,   \
                      n_heads, kv_heads, scale, window, stream)
  switch (hd) {
    EMBER_PREFILL(16);
    EMBER_PREFILL(32);
    EMBER_PREFILL(48);
    EMBER_PREFILL(64);
    EMBER_PREFILL(80);
    EMBER_PREFILL(96);
    EMBER_PREFILL(112);
    EMBER_PREFILL(128);
    default:
      return 2;
  }
#undef EMBER_PREFILL
}
