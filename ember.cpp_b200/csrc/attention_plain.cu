// Writing keys and values into the paged cache, and the plain attention kernel over it.
//
// ember.cpp writes K[pos] = k, V[pos] = v per block (kv_write_kernel, graph_ir_cuda.cu:212-220)
// and then runs, per (query, head), scores = (q.k_j)*scale over the keys up to the query's own
// position, softmax, weighted sum of values (cpu_attention.cpp:92-211; baseline CUDA kernel
// cuda_kernels.cu:1728-1896).  The plain kernel here does the same for any mix of sequences,
// positions and lengths: one warp per (token, head), keys in groups of 32 counted from the first
// visible key, an online softmax whose order depends on the key positions alone.  A token's
// result therefore does not depend on the batch, the step's cut or the page numbers.  It is the
// kernel of the 32-bit path and the twin that the faster kernels are tested against.
//
// Cache layout: page p of a layer is [kv_heads][64][head_dim]; a sequence's position j lives in
// page pages[seq][j / 64] at row j % 64.
#include "common.cuh"

// One block per token; 16 bytes (4 float32 or 8 bfloat16 values, never across a head: VEC is taken
// only when a head's row is a multiple of 16 bytes) or one value per thread and trip, all of a
// thread's loads before its stores.
template <typename T, bool VEC>
__global__ void kv_store_kernel(const T* __restrict__ qkv, T* __restrict__ kc, T* __restrict__ vc,
                                const int* __restrict__ positions, const int* __restrict__ token_seq,
                                const int* __restrict__ seq_slot, const int* __restrict__ pages, int max_blocks,
                                int q_width, int kv_heads, int hd) {
  constexpr int kVec = VEC ? 16 / (int)sizeof(T) : 1;
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int s = token_seq[t];
  if (seq_slot[s] < 0) return;
  const int p = positions[t];
  const int page = pages[s * max_blocks + p / kPage];
  if (page < 0) return;
  const int kv_width = kv_heads * hd;
  const T* src = qkv + (size_t)t * (q_width + 2 * kv_width) + q_width;
  for (int i = threadIdx.x * kVec; i < kv_width; i += blockDim.x * kVec) {
    const int h = i / hd, d = i % hd;
    const size_t dst = (((size_t)page * kv_heads + h) * kPage + (p % kPage)) * hd + d;
    if constexpr (VEC) {
      const uint4 k = __ldcg(reinterpret_cast<const uint4*>(src + i));
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(src + kv_width + i));
      *reinterpret_cast<uint4*>(kc + dst) = k;
      *reinterpret_cast<uint4*>(vc + dst) = v;
    } else {
      const T k = __ldcg(src + i), v = __ldcg(src + kv_width + i);
      kc[dst] = k;
      vc[dst] = v;
    }
  }
}

EMBER_API int ember_kv_store(const void* qkv, void* kc, void* vc, const int* positions, const int* token_seq,
                             const int* seq_slot, const int* pages, int max_blocks, int T, int n_heads, int kv_heads,
                             int hd, int dtype, cudaStream_t stream) {
  EMBER_CHECK(T > 0 && n_heads > 0 && kv_heads > 0 && hd > 0 && max_blocks > 0, "kv_store: bad sizes");
  EMBER_CHECK(dtype == EMBER_F32 || dtype == EMBER_BF16, "kv_store: element type %d", dtype);
  const int qw = n_heads * hd;
  // 16-byte copies where every head's row, and so every row of the activations, is a multiple of 16 bytes
  const bool vec = hd * (dtype == EMBER_F32 ? 4 : 2) % 16 == 0;
  cudaError_t e;
#define EMBER_KV_STORE(T, VEC)                                                                                           \
  e = launch_pdl(kv_store_kernel<T, VEC>, dim3(T_tokens), dim3(128), 0, stream, (const T*)qkv, (T*)kc, (T*)vc, positions, \
                 token_seq, seq_slot, pages, max_blocks, qw, kv_heads, hd)
  const int T_tokens = T;
  if (dtype == EMBER_F32) {
    if (vec) EMBER_KV_STORE(float, true); else EMBER_KV_STORE(float, false);
  } else {
    if (vec) EMBER_KV_STORE(__nv_bfloat16, true); else EMBER_KV_STORE(__nv_bfloat16, false);
  }
#undef EMBER_KV_STORE
  if (e != cudaSuccess) return ember_fail("kv_store: %s", cudaGetErrorString(e));
  return 0;
}

// ---------------------------------------------------------------------------- tails of new pages
// Pages are not cleared when they pass from one sequence to the next, so a page that is new to a
// sequence holds what its last owner left there, NaN and Inf included.  The rows of such a page that
// the step does not write (those past the step's end) are zeroed here, in every tensor of the
// cache group, before the step runs: a kernel that loads whole pages and masks by selection still
// multiplies a probability of zero with those rows.  ember.cpp's kernel tests fill their caches
// with NaN to catch such reads (tools/window_attention_cuda_test.cu:57-86).
// grid (sequences, tensors); tails[i] = (page, first row) or (-1, 0).
template <typename U>  // the unit of a store: 16 bytes where rows are multiples of it, else 4 or 2
__global__ void clear_tails_kernel(void* const* __restrict__ tensors, const int* __restrict__ tails, int kv_heads,
                                   int row_bytes) {
  const int page = tails[2 * blockIdx.x], row0 = tails[2 * blockIdx.x + 1];
  if (page < 0 || row0 >= kPage) return;
  char* base = static_cast<char*>(tensors[blockIdx.y]);
  const int units = (kPage - row0) * row_bytes / (int)sizeof(U);
  U zero;
  memset(&zero, 0, sizeof(U));
  for (int h = 0; h < kv_heads; ++h) {
    U* dst = reinterpret_cast<U*>(base + (((size_t)page * kv_heads + h) * kPage + row0) * row_bytes);
    for (int i = threadIdx.x; i < units; i += blockDim.x) dst[i] = zero;
  }
}

EMBER_API int ember_clear_tails(void* const* tensors, int n_tensors, const int* tails, int n, int kv_heads, int hd,
                                int elem_bytes, cudaStream_t stream) {
  EMBER_CHECK(n_tensors > 0 && n > 0 && kv_heads > 0 && hd > 0, "clear_tails: bad sizes");
  EMBER_CHECK(elem_bytes == 2 || elem_bytes == 4, "clear_tails: elements of %d bytes", elem_bytes);
  EMBER_CHECK(n_tensors <= 65535, "clear_tails: %d tensors exceed one launch", n_tensors);
  const int row_bytes = hd * elem_bytes;
  const dim3 grid(n, n_tensors);
  if (row_bytes % 16 == 0)
    clear_tails_kernel<uint4><<<grid, 128, 0, stream>>>(tensors, tails, kv_heads, row_bytes);
  else if (row_bytes % 4 == 0)
    clear_tails_kernel<unsigned><<<grid, 128, 0, stream>>>(tensors, tails, kv_heads, row_bytes);
  else
    clear_tails_kernel<unsigned short><<<grid, 128, 0, stream>>>(tensors, tails, kv_heads, row_bytes);
  EMBER_LAUNCH_OK("clear_tails");
  return 0;
}

// ---------------------------------------------------------------------------- plain attention
constexpr int kMaxHeadDim = 256;

template <typename T>
__global__ void __launch_bounds__(128)
attention_plain_kernel(const T* __restrict__ qkv, const T* __restrict__ kc, const T* __restrict__ vc,
                       T* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ token_seq,
                       const int* __restrict__ seq_slot, const int* __restrict__ pages, int max_blocks, int T_tokens,
                       int n_heads, int kv_heads, int hd, float scale, int window) {
  __shared__ float q_s[4][kMaxHeadDim];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x * 4 + warp;
  if (item >= T_tokens * n_heads) return;  // whole warps leave together
  const int t = item / n_heads, h = item % n_heads;
  const int qkv_width = (n_heads + 2 * kv_heads) * hd;
  T* o = out + (size_t)t * n_heads * hd + (size_t)h * hd;
  const int s = token_seq[t];
  if (seq_slot[s] < 0) {
    for (int d = lane; d < hd; d += 32) o[d] = from_float<T>(0.f);
    return;
  }
  const int p = positions[t];
  const int g = h / (n_heads / kv_heads);
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int* my_pages = pages + (size_t)s * max_blocks;
  const T* q = qkv + (size_t)t * qkv_width + (size_t)h * hd;
  for (int d = lane; d < hd; d += 32) q_s[warp][d] = to_float(q[d]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[kMaxHeadDim / 32];
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = 0.f;

  for (int base = lo; base <= p; base += 32) {
    const int j = base + lane;
    const int page = j <= p ? my_pages[j / kPage] : -1;
    const bool valid = page >= 0;  // a page that is not held contributes nothing and is never read
    size_t row = 0;  // element offset of key/value row j of head g
    float sc = -INFINITY;
    if (valid) {
      row = (((size_t)page * kv_heads + g) * kPage + (j % kPage)) * hd;
      const T* k = kc + row;
      float dot = 0.f;
      for (int d = 0; d < hd; ++d) dot = fmaf(q_s[warp][d], to_float(k[d]), dot);
      sc = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(sc));
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float pj = valid ? expf(sc - m_new) : 0.f;
    l = l * corr + warp_sum(pj);
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] *= corr;
    const int n_valid = min(32, p - base + 1);
    for (int jj = 0; jj < n_valid; ++jj) {
      const float pv = __shfl_sync(0xffffffffu, pj, jj);
      const unsigned long long r = __shfl_sync(0xffffffffu, (unsigned long long)row, jj);
      const T* v = vc + r;
#pragma unroll
      for (int i = 0; i < kMaxHeadDim / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pv, to_float(v[d]), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = 1.0f / l;
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) o[d] = from_float<T>(acc[i] * inv);
  }
}

EMBER_API int ember_attention_plain(const void* qkv, const void* kc, const void* vc, void* out, const int* positions,
                                    const int* token_seq, const int* seq_slot, const int* pages, int max_blocks, int T,
                                    int n_heads, int kv_heads, int hd, float scale, int window, int dtype,
                                    cudaStream_t stream) {
  EMBER_CHECK(T > 0 && n_heads > 0 && kv_heads > 0 && max_blocks > 0, "attention: bad sizes");
  EMBER_CHECK(n_heads % kv_heads == 0, "attention: %d heads are not a multiple of %d key/value heads", n_heads,
              kv_heads);
  EMBER_CHECK(hd >= 1 && hd <= kMaxHeadDim, "attention: head size %d is not in [1, %d]", hd, kMaxHeadDim);
  EMBER_CHECK(window >= 0, "attention: window %d", window);
  const long long items = (long long)T * n_heads;
  const int grid = (int)((items + 3) / 4);
  if (dtype == EMBER_F32)
    attention_plain_kernel<float><<<grid, 128, 0, stream>>>((const float*)qkv, (const float*)kc, (const float*)vc,
                                                            (float*)out, positions, token_seq, seq_slot, pages,
                                                            max_blocks, T, n_heads, kv_heads, hd, scale, window);
  else if (dtype == EMBER_BF16)
    attention_plain_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
        (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, (__nv_bfloat16*)out, positions,
        token_seq, seq_slot, pages, max_blocks, T, n_heads, kv_heads, hd, scale, window);
  else
    return ember_fail("attention: element type %d", dtype);
  EMBER_LAUNCH_OK("attention_plain");
  return 0;
}
