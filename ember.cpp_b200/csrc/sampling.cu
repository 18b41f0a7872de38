// Sampling on the device: first-maximum argmax, or temperature with top-k and top-p.
//
// ember.cpp samples on the host from a row of logits (api.cpp:238-341): below temperature 0.05
// the first maximal index; else p = exp((l - max)/T), candidates ordered by (p, index)
// descending, the first top_k of them (<= 0 or >= vocab: all), of those the shortest prefix whose
// normalised sum reaches top_p, and a draw from what is left.  This kernel keeps that set exactly
// and draws from it by inverse CDF in index order with a counter-based uniform (ember.cpp uses
// std::mt19937, whose stream cannot be shared with other code; the distribution is the same).
//
// The kernel's code runs once per row, straight through, and a step of a large model has pushed it out of every
// cache by then: what a row costs is, to a good part, fetching the code it runs.  So the ways that a row seldom
// takes (the radix selections) are functions of their own, out of line, and the usual way is short.
//
// One block per row; nothing is sorted.  Each candidate has the 64-bit key (bits of p, index);
// the k-th largest key and the key at which the running mass reaches top_p are found by radix
// selection over counts and over masses held as integers (p * 2^40, so that sums do not depend on
// the order of addition), 11 bits a pass, stopping as soon as the bucket holds one candidate.  The
// row's p values are kept in shared memory when the vocabulary fits (up to about 51,000 entries);
// otherwise they are recomputed from the logits in each pass.
//
// A small top_k (the usual case: 40 of 50,257) needs no selection over the whole row.  Each of the
// block's 512 threads knows the largest p among its own entries; the top_k-th largest of those 512
// values is a lower bound of the top_k-th largest p of the row (at least top_k entries reach it), so
// every candidate of the top_k lies at or above it, and with entries dealt to threads in turn only a
// few more do.  They are gathered into a short list and finished there; a row whose list would not
// fit (thousands of equal values at the edge) takes the radix selection instead.  The row itself comes
// into shared memory by 4-byte asynchronous copies, all in flight at once: one trip to L2, where the
// product that wrote the logits left them.
#include "common.cuh"

namespace {

constexpr int kThreads = 512;
constexpr int kBins = 2048;
constexpr double kMassScale = 1099511627776.0;  // 2^40
typedef unsigned long long u64;

__device__ __forceinline__ u64 splitmix_uniform24(u64 seed, u64 stream, u64 counter) {
  u64 z = seed * 0x9E3779B97F4A7C15ull + stream * 0xBF58476D1CE4E5B9ull + counter * 0x94D049BB133111EBull +
          0x2545F4914F6CDD1Dull;
  z ^= z >> 30;
  z *= 0xBF58476D1CE4E5B9ull;
  z ^= z >> 27;
  z *= 0x94D049BB133111EBull;
  z ^= z >> 31;
  return z >> 40;  // 24 bits
}

struct Row {
  const float* logits;  // global
  const float* cached;  // shared, or null
  float mx, inv_t;
  __device__ __forceinline__ float p(int i) const {
    if (cached) return cached[i];
    const float l = logits[i];
    return (l == l) ? expf((l - mx) * inv_t) : 0.f;  // a NaN logit gets no mass
  }
};

__device__ __forceinline__ u64 key_of(float p, int i) { return ((u64)__float_as_uint(p) << 32) | (unsigned)i; }
// floor(p * 2^40) for 0 <= p <= 1.  The product by a power of two is exact in float32 and the
// conversion truncates, so this is the integer the float64 form would give, without float64
// arithmetic (which this GPU has very little of).
__device__ __forceinline__ u64 mass_of(float p) { return __float2ull_rz(p * (float)kMassScale); }

// Sum over the block; every thread gets the total.  scratch: kThreads / 32 entries.
__device__ u64 block_sum(u64 v, u64* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  u64 t = 0;
  for (int w = 0; w < kThreads / 32; ++w) t += scratch[w];
  return t;
}

struct Pick {
  int bin;      // chosen bucket
  u64 before;   // weight of the buckets above it
  unsigned count;  // candidates in it
  bool none;       // no bucket reached the need: `bin` is the lowest non-empty one, everything is kept
};

// Walks the buckets from the highest down and finds the first non-empty one at which the running
// weight (counts, or masses) reaches `need`.  If none does, the lowest non-empty bucket with
// `before` = need (so that the caller's remaining need becomes 0: everything is kept).
__device__ __noinline__ Pick find_bucket(const unsigned* cnt, const u64* mass, bool by_mass, u64 need, u64* scratch, int* s_hit,
                            u64* s_before) {
  constexpr int kPer = kBins / kThreads;  // 4 buckets per thread, in descending order
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  u64 w[kPer], local = 0;
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int b = kBins - 1 - (threadIdx.x * kPer + j);
    w[j] = by_mass ? mass[b] : (u64)cnt[b];
    local += w[j];
  }
  // exclusive prefix of `local` over threads (thread 0 owns the highest buckets)
  u64 incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const u64 up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  if (threadIdx.x == 0) {
    *s_hit = 0x7fffffff;
    *s_before = 0;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = incl;
  __syncthreads();
  u64 base = 0;
  for (int i = 0; i < warp; ++i) base += scratch[i];
  u64 run = base + incl - local;
  int lowest = -1;
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int slot = threadIdx.x * kPer + j;
    const int b = kBins - 1 - slot;
    if (cnt[b]) {
      lowest = slot;
      if (run + w[j] >= need) atomicMin(s_hit, slot);
    }
    run += w[j];
  }
  __syncthreads();
  int hit = *s_hit;
  const bool none = hit == 0x7fffffff;
  __syncthreads();
  if (none) {  // nothing reaches the need: the lowest non-empty bucket
    if (threadIdx.x == 0) *s_hit = -1;
    __syncthreads();
    if (lowest >= 0) atomicMax(s_hit, lowest);
    __syncthreads();
    hit = *s_hit;
  }
  // the owner of the chosen bucket publishes the weight above it
  if (hit >= 0 && hit / kPer == (int)threadIdx.x) {
    u64 r = base + incl - local;
    for (int j = 0; j < hit % kPer; ++j) r += w[j];
    *s_before = none ? need : r;
  }
  __syncthreads();
  Pick pick;
  pick.bin = kBins - 1 - max(hit, 0);
  pick.before = *s_before;
  pick.count = cnt[pick.bin];
  pick.none = none;
  __syncthreads();
  return pick;
}

// Radix selection over the keys from the top bits down.  by_mass = false: the key of the
// `need`-th largest candidate.  by_mass = true: the key at which the running mass, in descending
// key order, first reaches `need`.  Returns a threshold: the candidates to keep are those with
// key >= threshold.
__device__ __noinline__ u64 radix_select(const Row& row, int V, bool by_mass, u64 need, unsigned* cnt, u64* mass, u64* scratch,
                            int* s_hit, u64* s_before) {
  const int shifts[6] = {53, 42, 32, 21, 10, 0};
  const int widths[6] = {11, 11, 10, 11, 11, 10};
  u64 prefix = 0;
  for (int pass = 0; pass < 6; ++pass) {
    const int shift = shifts[pass];
    if (pass >= 3 && ((u64)(V - 1) >> shift) == 0 && shift > 0) continue;  // no index has a bit here
    const u64 high_mask = pass == 0 ? 0ull : ~0ull << (shift + widths[pass]);
    const unsigned digit_mask = (1u << widths[pass]) - 1;
    for (int b = threadIdx.x; b < kBins; b += kThreads) {
      cnt[b] = 0;
      mass[b] = 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += kThreads) {
      const float p = row.p(i);
      const u64 key = key_of(p, i);
      if ((key & high_mask) == prefix) {
        const int b = (int)((key >> shift) & digit_mask);
        // lanes that hit the same bucket add once (a peaked row puts most candidates into one bucket)
        const unsigned peers = __match_any_sync(__activemask(), b);
        if ((threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&cnt[b], (unsigned)__popc(peers));
        if (by_mass) {
          const u64 m = mass_of(p);
          if (m) atomicAdd(&mass[b], m);
        }
      }
    }
    __syncthreads();
    const Pick pick = find_bucket(cnt, mass, by_mass, need, scratch, s_hit, s_before);
    prefix |= (u64)pick.bin << shift;
    if (pick.none) return prefix;  // the remaining weight does not reach the need: keep everything
    need -= pick.before;
    // one candidate left, or (by count) the whole bucket is wanted: every key in the bucket is kept
    if (pick.count == 1 || (!by_mass && (u64)pick.count == need)) return prefix;
  }
  return prefix;
}


constexpr int kSmallK = 512;   // top_k up to which the candidates are finished as a short list
constexpr int kListCap = 1024;  // entries of that list

// The end of both short ways: the candidates are in `list` (n <= kListCap keys, in any order; room for
// kListCap masses behind them).  Each one's rank and the mass above it by comparison with all others, the
// kept set (rank < top_k, and the mass above it short of the top_p target: the same set as the two radix
// selections give), and the draw in index order.
__device__ __noinline__ void finish_list(u64* list, int n, int top_k, bool use_p, u64 need_p, u64 u24, int fallback, int* out,
                            u64* scratch, int* s_hit) {
  u64* kept_mass = list + kListCap;
  constexpr int kPer = kListCap / kThreads;
  u64 my_key[kPer], my_mass[kPer];
#pragma unroll
  for (int t = 0; t < kPer; ++t) {
    const int e = threadIdx.x + t * kThreads;
    my_key[t] = 0;
    my_mass[t] = 0;
    if (e < n) {
      const u64 key = list[e];
      int rank = 0;
      u64 mass_above = 0;
      for (int j = 0; j < n; ++j) {
        const u64 other = list[j];
        if (other > key) {
          ++rank;
          mass_above += mass_of(__uint_as_float((unsigned)(other >> 32)));
        }
      }
      const bool keep = rank < top_k && (rank == 0 || !use_p || mass_above < need_p);
      my_key[t] = key;
      my_mass[t] = keep ? mass_of(__uint_as_float((unsigned)(key >> 32))) : 0;
    }
  }
  u64 total = 0;
#pragma unroll
  for (int t = 0; t < kPer; ++t) {
    const int e = threadIdx.x + t * kThreads;
    if (e < n) kept_mass[e] = my_mass[t];
    total += my_mass[t];
  }
  total = block_sum(total, scratch);  // its barriers also publish kept_mass
  if (threadIdx.x == 0) *s_hit = fallback;  // if nothing is drawn (no mass at all), the maximum
  __syncthreads();
  const u64 target = (__umul64hi(total, u24) << 40) | ((total * u24) >> 24);  // floor(total * u24 / 2^24)
#pragma unroll
  for (int t = 0; t < kPer; ++t) {
    const int e = threadIdx.x + t * kThreads;
    if (e < n && my_mass[t]) {
      const unsigned idx = (unsigned)my_key[t];
      u64 before = 0;
      for (int j = 0; j < n; ++j)
        if ((unsigned)list[j] < idx) before += kept_mass[j];
      if (before <= target && target < before + my_mass[t]) *s_hit = (int)idx;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) out[blockIdx.x] = *s_hit;
}

// The short way for a small top_k.  Radix passes by count run only until the candidates that can
// still be among the top_k (those above the chosen bucket, fewer than top_k, and the bucket itself)
// number at most kListCap; these are gathered into a list and finished there: each one's rank and
// the mass above it by comparison with all others, the kept set (rank < top_k, and the mass above
// it short of the top_p target: the same set as the two radix selections give), and the draw in
// index order.  Integer masses make every sum independent of the list's order.  Returns false
// (having written nothing) when the list would not fit, which takes a bucket of hundreds of
// candidates with the same leading digits on every level.
__device__ __noinline__ bool sample_small(const Row& row, int V, int top_k, bool use_p, u64 need_p, u64 u24, int fallback, int* out,
                             unsigned* cnt, u64* list, u64* scratch, int* s_hit, u64* s_before, int* s_n) {
  const int shifts[6] = {53, 42, 32, 21, 10, 0};
  const int widths[6] = {11, 11, 10, 11, 11, 10};
  u64 prefix = 0, need = (u64)top_k, above = 0;
  bool fits = false;
  for (int pass = 0; pass < 6 && !fits; ++pass) {
    const int shift = shifts[pass];
    if (pass >= 3 && ((u64)(V - 1) >> shift) == 0 && shift > 0) continue;
    const u64 high_mask = pass == 0 ? 0ull : ~0ull << (shift + widths[pass]);
    const unsigned digit_mask = (1u << widths[pass]) - 1;
    for (int b = threadIdx.x; b < kBins; b += kThreads) cnt[b] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += kThreads) {
      const u64 key = key_of(row.p(i), i);
      if ((key & high_mask) == prefix) {
        const int b = (int)((key >> shift) & digit_mask);
        const unsigned peers = __match_any_sync(__activemask(), b);
        if ((threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&cnt[b], (unsigned)__popc(peers));
      }
    }
    __syncthreads();
    const Pick pick = find_bucket(cnt, nullptr, false, need, scratch, s_hit, s_before);
    prefix |= (u64)pick.bin << shift;
    if (pick.none) return false;  // fewer candidates than top_k: not this function's case
    need -= pick.before;
    above += pick.before;
    fits = above + pick.count <= (u64)kListCap;
  }
  if (!fits) return false;
  if (threadIdx.x == 0) *s_n = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < V; i += kThreads) {
    const u64 key = key_of(row.p(i), i);
    if (key >= prefix) list[atomicAdd(s_n, 1)] = key;
  }
  __syncthreads();
  finish_list(list, *s_n, top_k, use_p, need_p, u24, fallback, out, scratch, s_hit);
  return true;
}

// The other way to the short list (see the head of the file): the threshold is the top_k-th largest of
// the threads' own maxima.  lmax: kThreads floats of scratch.  Returns false (nothing written) if more
// than kListCap entries reach the threshold.
__device__ __noinline__ bool sample_by_thread_maxima(const float* s_p, int V, float my_max, int top_k, bool use_p, u64 need_p, u64 u24,
                                        int fallback, int* out, float* lmax, u64* list, u64* scratch, int* s_hit, int* s_n) {
  // The top_k-th largest of the threads' maxima by radix selection over their bits, 8 bits a pass (p >= 0, so the
  // bits order as the values do; 0 stands for a thread without entries, below every p).
  __shared__ unsigned s_digit, s_left;
  unsigned* hist = reinterpret_cast<unsigned*>(lmax);  // 256 counters
  const unsigned key = my_max >= 0.f ? __float_as_uint(my_max) + 1u : 0u;
  unsigned prefix = 0, need = (unsigned)top_k;
  if (threadIdx.x == 0) *s_n = 0;
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (threadIdx.x < 256) hist[threadIdx.x] = 0;
    __syncthreads();
    if (shift == 24 || (key >> (shift + 8)) == (prefix >> (shift + 8))) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    __syncthreads();
    if (threadIdx.x < 32) {  // lane l owns the digits 255 - 8 l down to 248 - 8 l
      unsigned c[8], mine = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) mine += (c[j] = hist[255 - (threadIdx.x * 8 + j)]);
      unsigned incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned up = __shfl_up_sync(0xffffffffu, incl, o);
        if ((int)threadIdx.x >= o) incl += up;
      }
      unsigned before = incl - mine;  // keys in higher digits than this lane's
      if (before < need && need <= incl) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (before < need && need <= before + c[j]) {
            s_digit = 255u - (threadIdx.x * 8 + j);
            s_left = need - before;
          }
          before += c[j];
        }
      }
    }
    __syncthreads();
    prefix |= s_digit << shift;
    need = s_left;
  }
  const float thr = prefix ? __uint_as_float(prefix - 1u) : -1.f;  // (no entry at all in the top_k-th thread: everything)
  for (int i0 = threadIdx.x; i0 < V; i0 += 8 * kThreads) {  // eight reads in flight a thread (a write to the list
    float p[8];                                             // in between would hold the next read back)
#pragma unroll
    for (int j = 0; j < 8; ++j) p[j] = i0 + j * kThreads < V ? s_p[i0 + j * kThreads] : -2.f;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (p[j] >= thr) {
        const int at = atomicAdd(s_n, 1);
        if (at < kListCap) list[at] = key_of(p[j], i0 + j * kThreads);
      }
  }
  __syncthreads();
  const int n = *s_n;
  __syncthreads();
  if (n > kListCap) return false;
  finish_list(list, n, top_k, use_p, need_p, u24, fallback, out, scratch, s_hit);
  return true;
}

template <bool CACHED>
__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, int* __restrict__ out, int V, float temperature, int top_k,
              float top_p, u64 seed, const int* __restrict__ streams, const int* __restrict__ counters, u64 counter_base) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  u64* s_mass = reinterpret_cast<u64*>(smem_raw);                 // [kBins]; also the segment sums at the end
  unsigned* s_cnt = reinterpret_cast<unsigned*>(s_mass + kBins);  // [kBins]
  float* s_p = reinterpret_cast<float*>(s_cnt + kBins);           // [V] if CACHED
  __shared__ float s_val[kThreads / 32];
  __shared__ int s_idx[kThreads / 32];
  __shared__ u64 s_u64[kThreads / 32];
  __shared__ u64 s_before;
  __shared__ int s_hit, s_result, s_n;

  EMBER_MARK_START(kSample);
  const float* rowp = logits + (size_t)blockIdx.x * V;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  // The row comes into shared memory first when it fits, by asynchronous copies that are all in flight at once (no
  // registers wait for them): one trip to L2.  16 bytes a copy where the row allows: a row begins anywhere modulo 16
  // bytes (a vocabulary of 50,257), so its copy begins at the same offset in its buffer, and the few entries before
  // the first and after the last 16-byte boundary go singly.
  if (CACHED) {
    const int shift = (int)((reinterpret_cast<size_t>(rowp) >> 2) & 3);  // entries from a 16-byte boundary to the row
    s_p += shift;
    const int head = min(V, (4 - shift) & 3), body = (V - head) >> 2;
    for (int i = threadIdx.x; i < head; i += kThreads)
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(s_p + i)), "l"(rowp + i)
                   : "memory");
    for (int q = threadIdx.x; q < body; q += kThreads)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(s_p + head + 4 * q)),
                   "l"(rowp + head + 4 * q)
                   : "memory");
    for (int i = head + 4 * body + threadIdx.x; i < V; i += kThreads)
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(s_p + i)), "l"(rowp + i)
                   : "memory");
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
  }
  // first maximal index; NaN never wins
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  if (CACHED) {
    for (int i0 = threadIdx.x; i0 < V; i0 += 8 * kThreads) {  // eight reads in flight a thread
      float l[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) l[j] = i0 + j * kThreads < V ? s_p[i0 + j * kThreads] : -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (l[j] > best) {  // indices ascend, so the first maximum stays
          best = l[j];
          best_i = i0 + j * kThreads;
        }
    }
  } else {
    for (int i0 = threadIdx.x; i0 < V; i0 += 8 * kThreads) {  // eight loads in flight a thread
      float l[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) l[j] = i0 + j * kThreads < V ? __ldg(rowp + i0 + j * kThreads) : -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = i0 + j * kThreads;
        if (l[j] > best || (l[j] == best && i < best_i)) {  // indices ascend, so the first maximum stays
          best = l[j];
          best_i = i;
        }
      }
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

  Row row;
  row.logits = rowp;
  row.cached = nullptr;
  row.mx = best;
  row.inv_t = 1.0f / temperature;
  if (top_k <= 0 || top_k > V) top_k = V;

  u64 z = 0;
  float my_max = -1.f;  // the largest p among this thread's entries (CACHED)
  if (CACHED) {
#pragma unroll 4
    for (int i = threadIdx.x; i < V; i += kThreads) {
      const float l = s_p[i];
      const float p = (l == l) ? expf((l - row.mx) * row.inv_t) : 0.f;  // as Row::p
      s_p[i] = p;  // (an entry is read and written by this thread alone)
      my_max = fmaxf(my_max, p);
      z += mass_of(p);
    }
  } else {
    for (int i0 = threadIdx.x; i0 < V; i0 += 8 * kThreads) {
      float l[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) l[j] = i0 + j * kThreads < V ? __ldg(rowp + i0 + j * kThreads) : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = i0 + j * kThreads;
        if (i < V) z += mass_of((l[j] == l[j]) ? expf((l[j] - row.mx) * row.inv_t) : 0.f);  // as Row::p
      }
    }
  }
  z = block_sum(z, s_u64);  // its barriers also publish s_p
  if (CACHED) row.cached = s_p;

  if (top_k < V && top_k <= kSmallK) {
    const u64 u = splitmix_uniform24(seed, (u64)streams[blockIdx.x], (u64)counters[blockIdx.x] + counter_base);
    const u64 need_p = (u64)ceil((double)fmaxf(top_p, 0.f) * (double)z);
    if (CACHED && sample_by_thread_maxima(s_p, V, my_max, top_k, top_p < 1.0f, need_p, u, best_i, out,
                                          reinterpret_cast<float*>(s_cnt), s_mass, s_u64, &s_hit, &s_n))
      return;
    if (sample_small(row, V, top_k, top_p < 1.0f, need_p, u, best_i, out, s_cnt, s_mass, s_u64, &s_hit, &s_before, &s_n)) return;
  }

  u64 thr = 0;
  if (top_k < V) thr = radix_select(row, V, false, (u64)top_k, s_cnt, s_mass, s_u64, &s_hit, &s_before);
  if (top_p < 1.0f) {
    const double target = ceil((double)fmaxf(top_p, 0.f) * (double)z);
    const u64 thr_p = radix_select(row, V, true, (u64)target, s_cnt, s_mass, s_u64, &s_hit, &s_before);
    if (thr_p > thr) thr = thr_p;
  }

  // inverse CDF in index order over the kept candidates: thread t owns a contiguous segment
  u64* s_seg = s_mass;
  const int seg = (V + kThreads - 1) / kThreads;
  const int lo = threadIdx.x * seg, hi = min(V, lo + seg);
  u64 mine = 0;
  for (int i = lo; i < hi; ++i) {
    const float p = row.p(i);
    if (key_of(p, i) >= thr) mine += mass_of(p);
  }
  __syncthreads();
  s_seg[threadIdx.x] = mine;
  if (threadIdx.x == 0) s_result = best_i;  // if nothing is drawn (no mass at all), the maximum
  __syncthreads();
  u64 before = 0, total = 0;
  for (int t = 0; t < kThreads; ++t) {
    const u64 v = s_seg[t];
    if (t < (int)threadIdx.x) before += v;
    total += v;
  }
  const u64 u24 = splitmix_uniform24(seed, (u64)streams[blockIdx.x], (u64)counters[blockIdx.x] + counter_base);
  // target = floor(total * u24 / 2^24), exact in 128 bits
  const u64 target = (__umul64hi(total, u24) << 40) | ((total * u24) >> 24);
  if (total > 0 && before <= target && target < before + mine) {
    u64 run = before;
    for (int i = lo; i < hi; ++i) {
      const float p = row.p(i);
      if (key_of(p, i) >= thr) {
        run += mass_of(p);
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
                           unsigned long long seed, const int* streams, const int* counters,
                           unsigned long long counter_base, cudaStream_t stream) {
  EMBER_CHECK(rows > 0 && V > 0, "sample: rows = %d, vocabulary = %d", rows, V);
  EMBER_CHECK(temperature >= 0.f, "sample: temperature %g is negative", (double)temperature);
  const size_t bins = kBins * (sizeof(u64) + sizeof(unsigned));
  const size_t cached = bins + ((size_t)V + 4) * sizeof(float);  // (the row lies up to three entries into its buffer)
  static bool configured = false;
  const size_t limit = 226 * 1024;  // of the 227 KB a block may have; the kernel's static arrays take the rest
  if (cached <= limit) {
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(sample_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)limit);
      if (e != cudaSuccess) return ember_fail("sample: %s", cudaGetErrorString(e));
      configured = true;
    }
    sample_kernel<true><<<rows, kThreads, cached, stream>>>(logits, out, V, temperature, top_k, top_p, seed, streams,
                                                            counters, counter_base);
  } else {
    sample_kernel<false><<<rows, kThreads, bins, stream>>>(logits, out, V, temperature, top_k, top_p, seed, streams,
                                                           counters, counter_base);
  }
  EMBER_LAUNCH_OK("sample");
  return 0;
}

EMBER_TIMELINE_READER(sampling)
