// A whole decode step in one launch: a persistent kernel that runs a recorded program of the
// step's operations (embedding, layer norm, small-batch linear layers, decode attention) with a
// barrier across the grid where a launch boundary would be.
//
// ember.cpp captures its one-token step in a CUDA graph of about 17 kernel nodes a layer
// (graph_ir.cpp:4306-4373): the graph hides the host's launch cost, not the GPU's.  On this GPU a
// kernel node costs about 3.4 microseconds however small it is, while a layer of GPT-2 XL streams
// its 61 MB of weights in 9.4; a step launched kernel by kernel is bound by the boundaries between
// kernels.  Here the boundaries are grid barriers (about a microsecond), and the weights of the
// next linear layer are already on their way into shared memory while the grid waits at one.
//
// One block per SM, 16 warps.  The program is an array of EmberOp in device memory, written once
// when the step's shape is first seen; only the step's description (tokens, positions, pages)
// changes between launches.
//   linear     block b owns output features [N*b/G, N*(b+1)/G) in tiles of 16 rows; a tile is
//              brought in by cp.async in pieces of at most 1,664 values of K (double buffered,
//              the next piece always in flight, also across operations and barriers); the 16
//              warps take interleaved 32-wide slices on mma.sync with the operands swapped (as
//              linear_decode.cu), are summed in shared memory in warp order, then bias, GELU and
//              the float32 residual sum.
//   attention  a (token, head) pair per half block (8 warps), all its keys, online softmax per
//              stream, merged in shared memory; the token's own key and value are stored first.
//   layer norm a row per block.  embedding: a row per block.
// Activations written in one phase and read in the next go through L2 (ld.global.cg): L1 is not
// coherent between SMs.
//
// The grid barrier is the only place where a block waits for others.  The kernel is launched
// cooperatively, so all blocks are resident; every wait still has an iteration limit, after which
// the block raises the error flag and every block leaves at its next check.
#include <cooperative_groups.h>

#include "attention_common.cuh"
#include "common.cuh"

enum : int { EMBER_OP_EMBED = 0, EMBER_OP_LAYERNORM = 1, EMBER_OP_LINEAR = 2, EMBER_OP_ATTENTION = 3 };

struct alignas(16) EmberOp {
  int type, M, N, K;
  int act, out_f32, n_heads, kv_heads;
  int hd, window, store, max_blocks;
  int table_dtype, reserved;  // reserved: rows of the position table (embed), pages of the cache (attention)
  float eps, scale;
  const void* a;          // input rows (embed: token ids)
  const void* w;          // weight [N,K] / token table / norm gain
  const void* w2;         // position table / norm bias
  const float* bias;
  const float* residual;
  void* out;
  void* kc;
  void* vc;
  const int* positions;
  const int* seq_slot;
  const int* pages;
  const int* reserved_ptr;
};

namespace {

constexpr int kThreads = 512, kWarps = 16;
constexpr int kMaxPiece = 1664;                 // values of K in one staged piece of a tile
constexpr unsigned kSpinLimit = 1u << 22;       // polls of a barrier before a block gives up

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ uint4 ldcg16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

// how K is cut into pieces: the fewest pieces of at most kMaxPiece, each a multiple of 32
__host__ __device__ inline int piece_len(int K) {
  const int n = (K + kMaxPiece - 1) / kMaxPiece;
  return ((K + n - 1) / n + 31) / 32 * 32;
}
__host__ __device__ inline int piece_stride(int len) { return len + (((len / 32) & 1) ? 0 : 32); }

struct GridBarrier {
  unsigned count;
  unsigned generation;
};

// All blocks of the grid meet here.  Returns false if the wait ran out (the error flag is set).
__device__ bool grid_barrier(GridBarrier* bar, int* error) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    int ok = 1;
    __threadfence();
    const unsigned gen = *(volatile unsigned*)&bar->generation;
    if (atomicAdd(&bar->count, 1u) == gridDim.x - 1) {
      bar->count = 0;
      __threadfence();
      atomicAdd(&bar->generation, 1u);
    } else {
      unsigned spins = 0;
      while (*(volatile unsigned*)&bar->generation == gen) {
        if (*(volatile int*)error) {  // another block already gave up or found a bad index
          ok = 0;
          break;
        }
        if (++spins > kSpinLimit) {
          atomicCAS(error, 0, 1);
          ok = 0;
          break;
        }
        __nanosleep(32);
      }
    }
    __threadfence();
    if (*(volatile int*)error) ok = 0;
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

// ---------------------------------------------------------------------------- linear: the staged pieces
struct Cursor {  // a piece of a tile of a linear operation, in the order this block works through them
  int op, tile, piece;
};

struct LinearShape {
  int lo, hi, tiles, pieces, len;  // this block's rows [lo, hi), its 16-row tiles, pieces of K per tile, piece length
};

__device__ __forceinline__ LinearShape shape_of(const EmberOp& op) {
  LinearShape s;
  s.lo = (int)((long long)op.N * blockIdx.x / gridDim.x);
  s.hi = (int)((long long)op.N * (blockIdx.x + 1) / gridDim.x);
  s.tiles = (s.hi - s.lo + 15) / 16;
  s.len = piece_len(op.K);
  s.pieces = (op.K + s.len - 1) / s.len;
  return s;
}

// the first piece of the first linear operation at or after `from` in which this block has rows
__device__ Cursor first_piece(const EmberOp* ops, int n_ops, int from) {
  for (int i = from; i < n_ops; ++i)
    if (ops[i].type == EMBER_OP_LINEAR && shape_of(ops[i]).tiles > 0) return Cursor{i, 0, 0};
  return Cursor{n_ops, 0, 0};
}

__device__ Cursor next_piece(const EmberOp* ops, int n_ops, Cursor c) {
  const LinearShape s = shape_of(ops[c.op]);
  if (++c.piece < s.pieces) return c;
  c.piece = 0;
  if (++c.tile < s.tiles) return c;
  return first_piece(ops, n_ops, c.op + 1);
}

__device__ void stage_piece(const EmberOp& op, Cursor c, __nv_bfloat16* buf) {
  const LinearShape s = shape_of(op);
  const int ldw = piece_stride(s.len);
  const int k0 = c.piece * s.len;
  const int chunks = s.len / 8;
  const __nv_bfloat16* W = static_cast<const __nv_bfloat16*>(op.w);
  for (int i = threadIdx.x; i < 16 * chunks; i += kThreads) {
    const int r = i / chunks, ch = i % chunks;
    const int row = s.lo + c.tile * 16 + r, k = k0 + ch * 8;
    const bool ok = row < s.hi && k < op.K;
    cp_async_16(buf + r * ldw + ch * 8, W + (size_t)(ok ? row : s.lo) * op.K + (ok ? k : 0), ok);
  }
  asm volatile("cp.async.commit_group;\n" ::);
}

template <int MT>
__device__ void run_linear(const EmberOp* ops, int n_ops, int i, Cursor& staged, int& staged_buf, __nv_bfloat16* wbuf,
                           size_t buf_elems, float* red) {
  constexpr int kTile = 16 * 8 * MT;
  const EmberOp& op = ops[i];
  const LinearShape s = shape_of(op);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int ldw = piece_stride(s.len);
  const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(op.a);
  float acc[MT][4];
  for (int tile = 0; tile < s.tiles; ++tile) {
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[t][j] = 0.f;
    for (int piece = 0; piece < s.pieces; ++piece) {
      // `staged` is this piece (the block stages pieces in exactly the order it uses them)
      const int buf = staged_buf;
      const Cursor nxt = next_piece(ops, n_ops, staged);
      if (nxt.op < n_ops) {
        stage_piece(ops[nxt.op], nxt, wbuf + (size_t)(buf ^ 1) * buf_elems);
        asm volatile("cp.async.wait_group 1;\n" ::: "memory");
      } else {
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
      }
      staged = nxt;
      staged_buf = buf ^ 1;
      __syncthreads();
      const __nv_bfloat16* wt = wbuf + (size_t)buf * buf_elems;
      const int k0 = piece * s.len;
      const int slices = s.len / 32;
#pragma unroll 2
      for (int sl = warp; sl < slices; sl += kWarps) {
        const int kl = sl * 32 + c * 8, k = k0 + kl;
        const uint4 a_lo = *reinterpret_cast<const uint4*>(wt + g * ldw + kl);
        const uint4 a_hi = *reinterpret_cast<const uint4*>(wt + (g + 8) * ldw + kl);
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          const int m = t * 8 + g;
          const uint4 b = (k < op.K && m < op.M) ? ldcg16(x + (size_t)m * op.K + k) : make_uint4(0, 0, 0, 0);
          mma_bf16(acc[t], a_lo.x, a_hi.x, a_lo.y, a_hi.y, b.x, b.y);
          mma_bf16(acc[t], a_lo.z, a_hi.z, a_lo.w, a_hi.w, b.z, b.w);
        }
      }
      if (piece == s.pieces - 1) {
        // warps -> block in warp order, then the epilogue
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          float* mine = red + warp * kTile + t * 8;
          mine[g * (8 * MT) + c * 2] = acc[t][0];
          mine[g * (8 * MT) + c * 2 + 1] = acc[t][1];
          mine[(g + 8) * (8 * MT) + c * 2] = acc[t][2];
          mine[(g + 8) * (8 * MT) + c * 2 + 1] = acc[t][3];
        }
        __syncthreads();
        if (threadIdx.x < kTile) {
          const int r = threadIdx.x % 16, m = threadIdx.x / 16;
          const int n = s.lo + tile * 16 + r;
          if (m < op.M && n < s.hi) {
            float v = 0.f;
            for (int w = 0; w < kWarps; ++w) v += red[w * kTile + r * (8 * MT) + m];
            if (op.bias) v += op.bias[n];
            v = apply_act(v, op.act);
            const size_t at = (size_t)m * op.N + n;
            if (op.residual) v = __ldcg(op.residual + at) + v;
            if (op.out_f32)
              static_cast<float*>(op.out)[at] = v;
            else
              static_cast<__nv_bfloat16*>(op.out)[at] = __float2bfloat16_rn(v);
          }
        }
      }
      __syncthreads();  // the buffer and `red` are free again
    }
  }
}

// ---------------------------------------------------------------------------- rows
__device__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) t += scratch[w];
  return t;
}

__device__ void run_layernorm(const EmberOp& op, float* scratch) {
  const float* gamma = static_cast<const float*>(op.w);
  const float* beta = static_cast<const float*>(op.w2);
  const int K = op.K;
  for (int m = blockIdx.x; m < op.M; m += gridDim.x) {
    const float* r = static_cast<const float*>(op.a) + (size_t)m * K;
    float s = 0.f;
    for (int i = threadIdx.x; i < K; i += kThreads) s += __ldcg(r + i);
    const float mean = block_sum(s, scratch) / (float)K;
    float q = 0.f;
    for (int i = threadIdx.x; i < K; i += kThreads) {
      const float d = __ldcg(r + i) - mean;
      q += d * d;
    }
    const float inv = 1.0f / sqrtf(block_sum(q, scratch) / (float)K + op.eps);
    for (int i = threadIdx.x; i < K; i += kThreads) {
      const float v = (__ldcg(r + i) - mean) * inv * gamma[i] + beta[i];
      if (op.out_f32)
        static_cast<float*>(op.out)[(size_t)m * K + i] = v;
      else
        static_cast<__nv_bfloat16*>(op.out)[(size_t)m * K + i] = __float2bfloat16_rn(v);
    }
  }
}

// An index that came from the step's description and does not fit the table or cache it points
// into is recorded (error = 2) and its access skipped: nothing is read or written out of range.
__device__ __forceinline__ bool in_range(int v, int n, int* error) {
  if (v >= 0 && v < n) return true;
  atomicExch(error, 2);
  return false;
}

__device__ void run_embed(const EmberOp& op, int* error) {
  const int* tokens = static_cast<const int*>(op.a);
  const int d = op.K;
  for (int m = blockIdx.x; m < op.M; m += gridDim.x) {
    const int tok = tokens[m], pos = op.positions[m];
    if (!in_range(tok, op.N, error) || (op.w2 && !in_range(pos, op.reserved, error))) continue;
    float* o = static_cast<float*>(op.out) + (size_t)m * d;
    for (int i = threadIdx.x; i < d; i += kThreads) {
      float v;
      if (op.table_dtype == EMBER_BF16) {
        v = to_float(static_cast<const __nv_bfloat16*>(op.w)[(size_t)tok * d + i]);
        if (op.w2) v += to_float(static_cast<const __nv_bfloat16*>(op.w2)[(size_t)pos * d + i]);
      } else {
        v = static_cast<const float*>(op.w)[(size_t)tok * d + i];
        if (op.w2) v += static_cast<const float*>(op.w2)[(size_t)pos * d + i];
      }
      o[i] = v;
    }
  }
}

// ---------------------------------------------------------------------------- attention
__device__ __forceinline__ void half_sync(int half) { asm volatile("bar.sync %0, 256;\n" ::"r"(half + 1) : "memory"); }

// One (token, head) pair by the 8 warps of one half of the block; `scratch` is that half's.
template <int LPK>
__device__ void attend_item(const EmberOp& op, int t, int h, bool active, int half, float* scratch, int* error) {
  constexpr int kGroups = 32 / LPK, kStreams = 8 * kGroups, kRow = LPK * 8 + 1, kUnroll = 4;
  float* s_m = scratch;
  float* s_l = s_m + kStreams;
  float* s_w = s_l + kStreams;
  float* s_acc = s_w + kStreams;  // [kStreams][kRow]
  const int tid = threadIdx.x & 255, warp = tid >> 5, lane = tid & 31;
  const int sid = warp * kGroups + lane / LPK, sub = lane % LPK;
  const int hd = op.hd;
  const bool dims = sub * 8 < hd;
  float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  __nv_bfloat16* o = nullptr;
  bool padded = false;
  if (active) {
    o = static_cast<__nv_bfloat16*>(op.out) + ((size_t)t * op.n_heads + h) * hd;
    padded = op.seq_slot[t] < 0;
  }
  if (active && !padded) {
    int p = op.positions[t];
    if (!in_range(p, op.max_blocks * kPage, error)) p = 0;
    const int lo = op.window > 0 ? max(0, p - op.window + 1) : 0;
    const int end = op.store ? p : p + 1;  // the token's own key comes from the activations when it is stored here
    const int kvh = h / (op.n_heads / op.kv_heads);
    const int width = (op.n_heads + 2 * op.kv_heads) * hd;
    const int* my_pages = op.pages + (size_t)t * op.max_blocks;
    const __nv_bfloat16* qkv = static_cast<const __nv_bfloat16*>(op.a);
    const __nv_bfloat16* kc = static_cast<const __nv_bfloat16*>(op.kc);
    const __nv_bfloat16* vc = static_cast<const __nv_bfloat16*>(op.vc);
    float q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = 0.f;
    if (dims) unpack8(ldcg16(qkv + (size_t)t * width + (size_t)h * hd + sub * 8), q);
    const __nv_bfloat16* own = qkv + (size_t)t * width + (size_t)(op.n_heads + kvh) * hd;
    if (op.store) {
      const int page = my_pages[p / kPage];
      if (page >= 0 && in_range(page, op.reserved, error)) {
        const size_t dst = (((size_t)page * op.kv_heads + kvh) * kPage + (p % kPage)) * hd;
        const int vecs = hd / 8;
        for (int i = tid; i < 2 * vecs; i += 256) {
          const bool is_v = i >= vecs;
          const int j = (is_v ? i - vecs : i) * 8;
          const uint4 val = ldcg16(own + (is_v ? op.kv_heads * hd : 0) + j);
          *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(is_v ? op.vc : op.kc) + dst + j) = val;
        }
      }
    }
    for (int j0 = lo; j0 < end; j0 += kUnroll * kStreams) {
      uint4 kraw[kUnroll], vraw[kUnroll];
      bool have[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int j = j0 + u * kStreams + sid;
        const int page = j < end ? my_pages[j / kPage] : -1;
        have[u] = page >= 0 && in_range(page, op.reserved, error);
        kraw[u] = make_uint4(0, 0, 0, 0);
        vraw[u] = make_uint4(0, 0, 0, 0);
        if (dims && have[u]) {
          const size_t row = (((size_t)page * op.kv_heads + kvh) * kPage + (j % kPage)) * hd + sub * 8;
          // a cache that this step stored into elsewhere (another layer's) must be read past L1
          kraw[u] = op.store ? *reinterpret_cast<const uint4*>(kc + row) : ldcg16(kc + row);
          vraw[u] = op.store ? *reinterpret_cast<const uint4*>(vc + row) : ldcg16(vc + row);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) fold_key<LPK>(kraw[u], vraw[u], have[u], q, op.scale, m, l, acc);
    }
    if (op.store && warp == 0) {
      uint4 ok = make_uint4(0, 0, 0, 0), ov = make_uint4(0, 0, 0, 0);
      if (sid == 0 && dims) {
        ok = ldcg16(own + sub * 8);
        ov = ldcg16(own + op.kv_heads * hd + sub * 8);
      }
      fold_key<LPK>(ok, ov, sid == 0, q, op.scale, m, l, acc);
    }
  }
  // merge the half block's streams
  if (sub == 0) {
    s_m[sid] = m;
    s_l[sid] = l;
  }
  if (dims) {
#pragma unroll
    for (int i = 0; i < 8; ++i) s_acc[sid * kRow + sub * 8 + i] = acc[i];
  }
  half_sync(half);
  float M = -INFINITY;
  for (int i = 0; i < kStreams; ++i) M = fmaxf(M, s_m[i]);
  if (tid < kStreams) s_w[tid] = s_m[tid] == -INFINITY ? 0.f : __expf(s_m[tid] - M);
  half_sync(half);
  if (active) {
    float L = 0.f;
    for (int i = 0; i < kStreams; ++i) L += s_l[i] * s_w[i];
    for (int d = tid; d < hd; d += 256) {
      float A = 0.f;
      for (int i = 0; i < kStreams; ++i) A += s_acc[i * kRow + d] * s_w[i];
      o[d] = __float2bfloat16_rn(padded ? 0.f : A / L);
    }
  }
  half_sync(half);
}

__device__ void run_attention(const EmberOp& op, float* scratch_all, int scratch_floats, int* error) {
  const int half = threadIdx.x >> 8;
  float* scratch = scratch_all + half * scratch_floats;
  const int items = op.M * op.n_heads;
  const int slots = 2 * gridDim.x;
  for (int base = 0; base < items; base += slots) {  // every half block makes the same number of trips
    const int item = base + 2 * blockIdx.x + half;
    const bool active = item < items;
    const int t = active ? item / op.n_heads : 0, h = active ? item % op.n_heads : 0;
    if (op.hd <= 16) attend_item<2>(op, t, h, active, half, scratch, error);
    else if (op.hd <= 32) attend_item<4>(op, t, h, active, half, scratch, error);
    else if (op.hd <= 64) attend_item<8>(op, t, h, active, half, scratch, error);
    else if (op.hd <= 128) attend_item<16>(op, t, h, active, half, scratch, error);
    else attend_item<32>(op, t, h, active, half, scratch, error);
  }
}

constexpr int kAttnScratchFloats = 3 * 128 + 128 * 17 + 64;  // per half block; the largest of the five head-size cases

template <int MT>
__global__ void __launch_bounds__(kThreads, 1)
decode_program_kernel(const EmberOp* __restrict__ ops, int n_ops, GridBarrier* bar, int* error, int* trace) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const size_t buf_elems = (size_t)16 * piece_stride(kMaxPiece);
  __nv_bfloat16* wbuf = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [2][buf_elems]
  float* red = reinterpret_cast<float*>(wbuf + 2 * buf_elems);                       // [kWarps][16*8*MT]
  float* attn = red + kWarps * 16 * 8 * MT;                                          // [2][kAttnScratchFloats]
  float* rows = attn + 2 * kAttnScratchFloats;                                       // [kWarps]

  unsigned long long t_start = 0;
  Cursor staged = first_piece(ops, n_ops, 0);
  int staged_buf = 0;
  if (staged.op < n_ops) stage_piece(ops[staged.op], staged, wbuf);
  for (int i = 0; i < n_ops; ++i) {
    const EmberOp& op = ops[i];
    if (trace && threadIdx.x == 0) {  // a debugging aid: the operation each block has reached (host-visible memory)
      trace[blockIdx.x] = i + 1;
      if (blockIdx.x == 0 && i < 768) {  // and when block 0 began it, in nanoseconds since the kernel started
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (i == 0) t_start = now;
        trace[256 + i] = (int)(now - t_start);
      }
      __threadfence_system();
    }
    if (op.type == EMBER_OP_LINEAR) run_linear<MT>(ops, n_ops, i, staged, staged_buf, wbuf, buf_elems, red);
    else if (op.type == EMBER_OP_ATTENTION) run_attention(op, attn, kAttnScratchFloats, error);
    else if (op.type == EMBER_OP_LAYERNORM) run_layernorm(op, rows);
    else if (op.type == EMBER_OP_EMBED) run_embed(op, error);
    if (i + 1 < n_ops && !grid_barrier(bar, error)) break;
  }
  asm volatile("cp.async.wait_all;\n" ::: "memory");  // nothing of this block is in flight when it leaves
  if (trace && threadIdx.x == 0) {
    trace[blockIdx.x] = -1;  // left the kernel
    __threadfence_system();
  }
}

size_t program_smem(int mt) {
  return (size_t)2 * 16 * piece_stride(kMaxPiece) * sizeof(__nv_bfloat16) + (size_t)kWarps * 16 * 8 * mt * sizeof(float) +
         (size_t)2 * kAttnScratchFloats * sizeof(float) + kWarps * sizeof(float);
}

}  // namespace

EMBER_API int ember_decode_program_op_size() { return (int)sizeof(EmberOp); }

// Bytes of device memory for the barrier's state (zero before the first run; every run leaves it
// ready for the next).
EMBER_API int ember_decode_program_state_size() { return (int)sizeof(GridBarrier); }

// Runs a program of `n_ops` operations (device array) for up to 16 rows.  `state`: the barrier's
// state; `error`: one int on the device, zero before the run, non-zero afterwards if a block gave
// up waiting at a barrier (1) or an index of the step's description was out of range (2); the
// results are then not valid.
// `trace`: null, or 1,024 ints in memory the host can read (pinned and mapped): each block
// writes there the number of the operation it has reached (1-based; -1 once it has left), which
// is still readable after a fault; from entry 256 on, the time at which block 0 began each operation.
EMBER_API int ember_decode_program_run(const void* ops, int n_ops, int max_rows, void* state, int* error, int* trace,
                                       cudaStream_t stream) {
  EMBER_CHECK(n_ops > 0 && max_rows > 0 && max_rows <= 16, "decode_program: %d operations for %d rows", n_ops, max_rows);
  static int sms = 0;
  static bool configured[2] = {false, false};
  if (!sms) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return ember_fail("decode_program: %s", cudaGetErrorString(e));
  }
  const int mt = max_rows <= 8 ? 1 : 2;
  const size_t smem = program_smem(mt);
  const void* fn = mt == 1 ? (const void*)decode_program_kernel<1> : (const void*)decode_program_kernel<2>;
  if (!configured[mt - 1]) {
    cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ember_fail("decode_program: %s", cudaGetErrorString(e));
    int per_sm = 0;
    e = mt == 1 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_program_kernel<1>, kThreads, smem)
                : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_program_kernel<2>, kThreads, smem);
    if (e != cudaSuccess || per_sm < 1) return ember_fail("decode_program: the kernel does not fit an SM");
    configured[mt - 1] = true;
  }
  GridBarrier* bar = static_cast<GridBarrier*>(state);
  void* args[] = {(void*)&ops, (void*)&n_ops, (void*)&bar, (void*)&error, (void*)&trace};
  cudaError_t e = cudaLaunchCooperativeKernel(fn, dim3(sms), dim3(kThreads), args, smem, stream);
  if (e != cudaSuccess) return ember_fail("decode_program: %s", cudaGetErrorString(e));
  return 0;
}
