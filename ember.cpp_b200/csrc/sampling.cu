// Sampling on the device: first-maximum argmax, or temperature with top-k and top-p.
//
// ember.cpp samples on the host from a row of logits (api.cpp:238-341): below temperature 0.05
// the first maximal index; else p = exp((l - max)/T), candidates ordered by (p, index)
// descending, the first top_k of them (<= 0 or >= vocab: all), of those the shortest prefix whose
// normalised sum reaches top_p, and a draw from what is left.  This kernel keeps that set exactly
// and draws from it by inverse CDF in index order with a counter-based uniform (ember.cpp uses
// std::mt19937, whose stream cannot be shared with other code; the distribution is the same).
//
// One block per row; nothing is sorted.  Each candidate has the 64-bit key (bits of p, index);
// the k-th largest key and the key at which the running mass reaches top_p are found by radix
// selection, 8 bits a pass, over counts and over masses held as integers (p * 2^40, so that sums
// do not depend on the order of addition).  Candidates are recomputed from the logits in each
// pass instead of being stored.
#include "common.cuh"

namespace {

constexpr int kThreads = 512;
constexpr double kMassScale = 1099511627776.0;  // 2^40

__device__ __forceinline__ unsigned long long splitmix_uniform24(unsigned long long seed, unsigned long long stream,
                                                                 unsigned long long counter) {
  unsigned long long z = seed * 0x9E3779B97F4A7C15ull + stream * 0xBF58476D1CE4E5B9ull +
                         counter * 0x94D049BB133111EBull + 0x2545F4914F6CDD1Dull;
  z ^= z >> 30;
  z *= 0xBF58476D1CE4E5B9ull;
  z ^= z >> 27;
  z *= 0x94D049BB133111EBull;
  z ^= z >> 31;
  return z >> 40;  // 24 bits
}

struct Cand {
  unsigned long long key;
  unsigned long long mass;
};

__device__ __forceinline__ Cand candidate(const float* row, int i, float mx, float inv_t) {
  const float l = row[i];
  float p = (l == l) ? expf((l - mx) * inv_t) : 0.f;  // a NaN logit gets no mass
  Cand c;
  c.key = ((unsigned long long)__float_as_uint(p) << 32) | (unsigned)i;
  c.mass = (unsigned long long)((double)p * kMassScale);
  return c;
}

__device__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  unsigned long long t = 0;
  for (int w = 0; w < kThreads / 32; ++w) t += scratch[w];
  return t;
}

// Radix selection over the keys, from the top byte down.  by_mass = false: the key of the
// `need`-th largest candidate.  by_mass = true: the key at which the running mass, taken in
// descending key order, first reaches `need`.
__device__ unsigned long long radix_select(const float* row, int V, float mx, float inv_t, bool by_mass,
                                           unsigned long long need, unsigned* cnt, unsigned long long* mass,
                                           unsigned long long* shared_prefix, unsigned long long* shared_need) {
  unsigned long long prefix = 0;
  for (int pass = 0; pass < 8; ++pass) {
    const int shift = 56 - 8 * pass;
    for (int b = threadIdx.x; b < 256; b += kThreads) {
      cnt[b] = 0;
      mass[b] = 0;
    }
    __syncthreads();
    const unsigned long long high_mask = pass == 0 ? 0ull : ~0ull << (shift + 8);
    for (int i = threadIdx.x; i < V; i += kThreads) {
      const Cand c = candidate(row, i, mx, inv_t);
      if ((c.key & high_mask) == prefix) {
        const int b = (int)((c.key >> shift) & 0xff);
        atomicAdd(&cnt[b], 1u);
        if (by_mass && c.mass) atomicAdd(&mass[b], c.mass);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long run = 0;
      int chosen = -1, lowest = -1;
      for (int b = 255; b >= 0; --b) {
        if (!cnt[b]) continue;
        lowest = b;
        const unsigned long long w = by_mass ? mass[b] : cnt[b];
        if (run + w >= need) {
          chosen = b;
          break;
        }
        run += w;
      }
      if (chosen < 0) {  // the remaining mass does not reach the target: keep everything
        chosen = lowest;
        run = 0;
        need = 0;
      } else {
        need -= run;
      }
      *shared_prefix = prefix | ((unsigned long long)chosen << shift);
      *shared_need = need;
    }
    __syncthreads();
    prefix = *shared_prefix;
    need = *shared_need;
    __syncthreads();
  }
  return prefix;
}

__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, int* __restrict__ out, int V, float temperature, int top_k,
              float top_p, unsigned long long seed, const int* __restrict__ streams,
              const int* __restrict__ counters) {
  __shared__ float s_val[kThreads / 32];
  __shared__ int s_idx[kThreads / 32];
  __shared__ unsigned long long s_u64[kThreads / 32];
  __shared__ unsigned s_cnt[256];
  __shared__ unsigned long long s_mass[256];
  __shared__ unsigned long long s_prefix, s_need;
  __shared__ unsigned long long s_seg[kThreads];
  __shared__ int s_result;

  const float* row = logits + (size_t)blockIdx.x * V;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  // first maximal index; NaN never wins
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += kThreads) {
    const float l = row[i];
    if (l > best || (l == best && i < best_i)) {
      best = l;
      best_i = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  if (lane == 0) {
    s_val[warp] = best;
    s_idx[warp] = best_i;
  }
  __syncthreads();
  best = s_val[0];
  best_i = s_idx[0];
  for (int w = 1; w < kThreads / 32; ++w)
    if (s_val[w] > best || (s_val[w] == best && s_idx[w] < best_i)) {
      best = s_val[w];
      best_i = s_idx[w];
    }
  if (best_i == 0x7fffffff) best_i = 0;  // a row of NaN or -inf
  if (temperature < 0.05f || best == -INFINITY) {
    if (threadIdx.x == 0) out[blockIdx.x] = best_i;
    return;
  }

  const float inv_t = 1.0f / temperature;
  if (top_k <= 0 || top_k > V) top_k = V;

  unsigned long long z = 0;
  for (int i = threadIdx.x; i < V; i += kThreads) z += candidate(row, i, best, inv_t).mass;
  z = block_sum_u64(z, s_u64);

  unsigned long long thr = 0;
  if (top_k < V) thr = radix_select(row, V, best, inv_t, false, (unsigned long long)top_k, s_cnt, s_mass, &s_prefix, &s_need);
  if (top_p < 1.0f) {
    const double target = ceil((double)fmaxf(top_p, 0.f) * (double)z);
    const unsigned long long thr_p =
        radix_select(row, V, best, inv_t, true, (unsigned long long)target, s_cnt, s_mass, &s_prefix, &s_need);
    if (thr_p > thr) thr = thr_p;
  }

  // inverse CDF in index order over the kept candidates: thread t owns a contiguous segment
  const int seg = (V + kThreads - 1) / kThreads;
  const int lo = threadIdx.x * seg, hi = min(V, lo + seg);
  unsigned long long mine = 0;
  for (int i = lo; i < hi; ++i) {
    const Cand c = candidate(row, i, best, inv_t);
    if (c.key >= thr) mine += c.mass;
  }
  s_seg[threadIdx.x] = mine;
  if (threadIdx.x == 0) s_result = best_i;  // if nothing is drawn (no mass at all), the maximum
  __syncthreads();
  unsigned long long before = 0, total = 0;
  for (int t = 0; t < kThreads; ++t) {
    if (t < (int)threadIdx.x) before += s_seg[t];
    total += s_seg[t];
  }
  const unsigned long long u24 = splitmix_uniform24(seed, (unsigned long long)streams[blockIdx.x],
                                                    (unsigned long long)counters[blockIdx.x]);
  // target = floor(total * u24 / 2^24), exact in 128 bits
  const unsigned long long target = (__umul64hi(total, u24) << 40) | ((total * u24) >> 24);
  if (total > 0 && before <= target && target < before + mine) {
    unsigned long long run = before;
    for (int i = lo; i < hi; ++i) {
      const Cand c = candidate(row, i, best, inv_t);
      if (c.key >= thr) {
        run += c.mass;
        if (run > target) {
          s_result = i;
          break;
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) out[blockIdx.x] = s_result;
}

}  // namespace

EMBER_API int ember_sample(const float* logits, int* out, int rows, int V, float temperature, int top_k, float top_p,
                           unsigned long long seed, const int* streams, const int* counters, cudaStream_t stream) {
  EMBER_CHECK(rows > 0 && V > 0, "sample: rows = %d, vocabulary = %d", rows, V);
  EMBER_CHECK(temperature >= 0.f, "sample: temperature %g is negative", (double)temperature);
  sample_kernel<<<rows, kThreads, 0, stream>>>(logits, out, V, temperature, top_k, top_p, seed, streams, counters);
  EMBER_LAUNCH_OK("sample");
  return 0;
}
