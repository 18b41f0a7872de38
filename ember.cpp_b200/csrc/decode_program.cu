// A whole decode step in one launch: a persistent kernel that runs a recorded program of the
// step's operations (embedding, layer norm, small-batch linear layers, decode attention) with a
// barrier across the grid where a launch boundary would be.
//
// ember.cpp captures its one-token step in a CUDA graph of about 17 kernel nodes a layer
// (graph_ir.cpp:4306-4373): the graph hides the host's launch cost, not the GPU's.  On this GPU a
// kernel node costs about 3.4 microseconds however small it is, while a layer of GPT-2 XL streams
// its 61 MB of weights in 9.4; a step launched kernel by kernel is bound by the boundaries between
// kernels.  Here the boundaries are grid barriers (one release-add and acquire-loads of a counter
// that is never reset), and the weights of the next linear layers are already on their way into
// shared memory while the grid waits at one.
//
// One block per SM, 16 warps.  The program is an array of EmberOp in device memory, written once
// when the step's shape is first seen; only the step's description (tokens, positions, pages)
// changes between launches.
//   linear     block b owns output features [N*b/G, N*(b+1)/G) in tiles of 16 rows; a tile is
//              brought in by bulk copies (a row of the tile each, counted on the slot's mbarrier) in
//              pieces of at most 800 values of K through a ring of seven slots (179 KB), six pieces
//              always in flight, also across operations and barriers:
//              the weights of the next linear layers stream in while the grid runs the attention
//              or waits.  The 16 warps take the 32-wide slices of K in turn on mma.sync with the
//              operands swapped (as linear_decode.cu); a warp's slices are the same in every tile,
//              so it keeps the activations it multiplies with in registers for the whole
//              operation (read once from L2; normed on the way when a layer norm precedes the
//              product: row statistics by two warps a row first).  Up to four tiles' sums stay in
//              registers, are summed in shared memory in warp order, then bias, GELU and the
//              float32 residual sum.  At most 8 rows, K up to 6,656 (2,048 with a norm).
//   attention  a (token, head) pair per half block (8 warps), all its keys, online softmax per
//              stream, merged in shared memory; the token's own key and value are stored first.
//   layer norm (one that no product follows) a row per block.  embedding: a row per block.
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
constexpr int kMaxPiece = 800;                  // values of K in one staged piece of a tile
constexpr int kSlots = 7;                       // pieces the ring holds
constexpr int kRows = 8;                        // rows (sequences) a program can have
constexpr int kGroup = 4;                       // tiles whose sums stay in registers before they are finished
constexpr int kNormK = 2048;                    // the widest row a fused layer norm takes
constexpr int kMaxJ = 13;                       // 32-wide slices of K a warp can own: K <= 13 * 16 * 32 = 6,656
constexpr unsigned kSpinLimit = 1u << 22;       // polls of a barrier before a block gives up

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ldcg16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

// how K is cut into pieces: the fewest pieces of at most kMaxPiece, each a multiple of 32
__host__ __device__ inline int piece_len(int K) {
  const int n = (K + kMaxPiece - 1) / kMaxPiece;
  return ((K + n - 1) / n + 31) / 32 * 32;
}
__host__ __device__ inline int piece_stride(int len) { return len + (((len / 32) & 1) ? 0 : 32); }

struct GridBarrier {
  unsigned long long count;  // arrivals, never reset: barrier number k of launch e is complete at (e * barriers + k) * blocks
  unsigned long long epoch;  // launches completed
};

// All blocks of the grid meet here.  `target`: the arrival count at which this barrier is complete.
// One release-add and acquire-loads until the count is there: each poll is one trip to L2.  Returns
// false if the wait ran out or another block reported an error (the error flag is set).
__device__ bool grid_barrier(GridBarrier* bar, unsigned long long target, int* error) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    int ok = 1;
    asm volatile("red.release.gpu.global.add.u64 [%0], 1;\n" ::"l"(&bar->count) : "memory");
    unsigned spins = 0;
    for (;;) {
      unsigned long long seen;
      asm volatile("ld.acquire.gpu.global.u64 %0, [%1];\n" : "=l"(seen) : "l"(&bar->count) : "memory");
      if (seen >= target) break;
      if ((++spins & 63u) == 0) {
        if (*(volatile int*)error) {  // another block already gave up or found a bad index
          ok = 0;
          break;
        }
        if (spins > kSpinLimit) {
          atomicCAS(error, 0, 1);
          ok = 0;
          break;
        }
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

// ---------------------------------------------------------------------------- linear: the staged pieces
struct LinearShape {
  int lo, hi, tiles, pieces, len;  // this block's rows [lo, hi), its 16-row tiles, pieces of K per tile, piece length
};

// (32-bit arithmetic: the launcher refuses programs whose N * blocks does not fit)
__device__ __forceinline__ LinearShape shape_of(const EmberOp& op) {
  LinearShape s;
  s.lo = (int)((unsigned)op.N * blockIdx.x / gridDim.x);
  s.hi = (int)((unsigned)op.N * (blockIdx.x + 1) / gridDim.x);
  s.tiles = (s.hi - s.lo + 15) / 16;
  s.len = piece_len(op.K);
  s.pieces = (op.K + s.len - 1) / s.len;
  return s;
}

struct Cursor {  // a piece of a tile of a linear operation, in the order this block works through them
  int op, tile, piece;
  LinearShape shape;  // of `op` for this block (worked out once per operation: it takes divisions)
};

// the first piece of the first linear operation at or after `from` in which this block has rows
__device__ Cursor first_piece(const EmberOp* ops, int n_ops, int from) {
  Cursor c;
  c.tile = c.piece = 0;
  for (c.op = from; c.op < n_ops; ++c.op)
    if (ops[c.op].type == EMBER_OP_LINEAR) {
      c.shape = shape_of(ops[c.op]);
      if (c.shape.tiles > 0) return c;
    }
  c.op = n_ops;
  c.shape = LinearShape{0, 0, 0, 0, 32};
  return c;
}

__device__ __forceinline__ Cursor next_piece(const EmberOp* ops, int n_ops, Cursor c) {
  if (++c.piece < c.shape.pieces) return c;
  c.piece = 0;
  if (++c.tile < c.shape.tiles) return c;
  return first_piece(ops, n_ops, c.op + 1);
}

// A slot of the ring: [16][ldw] weights, ldw = piece_stride(piece length).
constexpr int kSlotElems = 16 * kMaxPiece;

// Asks for the weights of piece `c`: a bulk copy for every row of the tile that the block owns, issued
// by the lanes of warp 0 and counted on the slot's mbarrier (no per-16-byte address arithmetic: the
// staging loop of 16-byte cp.async took more issue slots than the products).  Rows past the block's
// share are not fetched (their sums are dropped at the end); what a piece holds past K is zeroed
// by hand up to the next multiple of 32, so that the products meet no stale bits there.
__device__ void stage_piece(const EmberOp& op, const Cursor& c, __nv_bfloat16* slot, unsigned bar) {
  const LinearShape& s = c.shape;
  const int ldw = piece_stride(s.len);
  const int k0 = c.piece * s.len;
  const int valid = max(0, min(s.len, op.K - k0));            // values of K this piece really holds
  const int rows = max(0, min(16, s.hi - (s.lo + c.tile * 16)));
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    if (lane == 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"((unsigned)(rows * valid * 2))
                   : "memory");
    __syncwarp();
    if (lane < rows && valid > 0) {
      const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(op.w) + (size_t)(s.lo + c.tile * 16 + lane) * op.K + k0;
      const unsigned dst = (unsigned)__cvta_generic_to_shared(slot + lane * ldw);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
                   "l"(src), "r"((unsigned)(valid * 2)), "r"(bar)
                   : "memory");
    }
  }
  const int tail = min(s.len, (valid + 31) / 32 * 32) - valid;
  for (int i = threadIdx.x; i < 16 * tail; i += kThreads) slot[(i / tail) * ldw + valid + i % tail] = __float2bfloat16_rn(0.f);
}

// Waits until the copies into a slot have landed.  False (and the error flag set) when the wait ran out.
__device__ bool slot_wait(unsigned bar, unsigned parity, int* error) {
  for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
    unsigned done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  atomicCAS(error, 0, 3);
  return false;
}

// The ring of staged pieces, the same in every thread of the block.
struct Ring {
  Cursor tail;  // the oldest staged piece (the next to be used)
  Cursor head;  // the next piece to stage
  int count;    // staged and not yet used
  int tail_slot;
  unsigned parity;  // bit s: the phase of slot s's mbarrier that its next use waits for
  unsigned bars;    // shared-memory address of the slots' mbarriers
};

__device__ __forceinline__ bool fused_norm(const EmberOp& op) { return op.reserved != 0; }

// Stages the next piece if the ring has room.  Weights are constants of the model, so pieces of
// operations that have not begun may be staged at any time.
__device__ void stage_next(const EmberOp* ops, int n_ops, Ring& ring, __nv_bfloat16* wbuf) {
  if (ring.count >= kSlots || ring.head.op >= n_ops) return;
  __nv_bfloat16* slot = wbuf + (size_t)((ring.tail_slot + ring.count) % kSlots) * kSlotElems;
  stage_piece(ops[ring.head.op], ring.head, slot, ring.bars + 8 * ((ring.tail_slot + ring.count) % kSlots));
  if (ring.count == 0) ring.tail = ring.head;
  ring.head = next_piece(ops, n_ops, ring.head);
  ++ring.count;
}

// Mean and 1/sqrt(var + eps) of the operation's (at most kRows) float32 rows: two warps a row,
// the row in registers, mean, then the biased variance; the two warps' sums are added in warp
// order.  The rows were written by other SMs in the phase before: read from L2.
// stats: [2 * kRows]; part: [kWarps].
__device__ void row_stats(const EmberOp& op, float* stats, float* part) {
  constexpr int kVecs = kNormK / 4 / 64;  // float4 a lane
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = warp >> 1, l64 = (warp & 1) * 32 + lane;
  const int K = op.K, nv = K >> 2;
  const bool row_ok = m < op.M;
  const float4* r4 = reinterpret_cast<const float4*>(static_cast<const float*>(op.a) + (size_t)(row_ok ? m : 0) * K);
  float4 v[kVecs];
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < kVecs; ++j) {
    const int i = l64 + 64 * j;
    v[j] = (row_ok && i < nv) ? __ldcg(r4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
  }
  s = warp_sum(s);
  if (lane == 0) part[warp] = s;
  __syncthreads();
  const float mean = (part[warp & ~1] + part[warp | 1]) / (float)K;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < kVecs; ++j) {
    if (l64 + 64 * j < nv) {
      const float a0 = v[j].x - mean, a1 = v[j].y - mean, a2 = v[j].z - mean, a3 = v[j].w - mean;
      q += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
    }
  }
  q = warp_sum(q);
  __syncthreads();
  if (lane == 0) part[warp] = q;
  __syncthreads();
  if ((warp & 1) == 0 && lane == 0 && m < kRows) {
    stats[2 * m] = mean;
    stats[2 * m + 1] = 1.0f / sqrtf((part[warp] + part[warp + 1]) / (float)K + op.eps);
  }
  __syncthreads();
}

// The sums of up to kGroup tiles, warps -> block in warp order, then the epilogue.
__device__ void finish_tiles(const EmberOp& op, const LinearShape& s, int first_tile, int n_tiles, float (&acc)[kGroup][4],
                             float* red) {
  constexpr int kTile = 16 * 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
#pragma unroll
  for (int t = 0; t < kGroup; ++t) {
    if (t < n_tiles) {
      float* mine = red + (warp * kGroup + t) * kTile;
      mine[g * 8 + c * 2] = acc[t][0];
      mine[g * 8 + c * 2 + 1] = acc[t][1];
      mine[(g + 8) * 8 + c * 2] = acc[t][2];
      mine[(g + 8) * 8 + c * 2 + 1] = acc[t][3];
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[t][j] = 0.f;
  }
  __syncthreads();
  const int t = threadIdx.x / kTile, e = threadIdx.x % kTile;  // 512 threads: one output of one of four tiles each
  if (t < n_tiles) {
    const int r = e % 16, m = e / 16;
    const int n = s.lo + (first_tile + t) * 16 + r;
    if (m < op.M && n < s.hi) {
      float v = 0.f;
      for (int w = 0; w < kWarps; ++w) v += red[(w * kGroup + t) * kTile + r * 8 + m];
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
  __syncthreads();  // `red` is free again
}

// A warp owns the 32-wide slices of K whose number is its own modulo 16, in every tile: the
// activations it multiplies with never change during the operation, so it holds them in registers
// (8 values of row lane/4 a slice: the B fragments of two MMAs), read once from L2, normed on the
// way if the operation has a norm.
__device__ void run_linear(const EmberOp* ops, int n_ops, int i, Ring& ring, __nv_bfloat16* wbuf, float* red, float* part,
                           float* stats, int* error) {
  const EmberOp& op = ops[i];
  // this block's share: the ring's tail is this operation's first piece if the block has rows in it
  const LinearShape s = (ring.count > 0 && ring.tail.op == i) ? ring.tail.shape : shape_of(op);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int ldw = piece_stride(s.len);
  const int spp = s.len / 32;  // slices a piece
  const bool normed = fused_norm(op);
  if (normed) row_stats(op, stats, part);
  uint4 xr[kMaxJ];
#pragma unroll
  for (int j = 0; j < kMaxJ; ++j) {
    const int piece = (j * kWarps + warp) / spp;  // slice number -> where it lies in K as the pieces cut it
    const int k = piece * s.len + ((j * kWarps + warp) - piece * spp) * 32 + c * 8;
    xr[j] = make_uint4(0u, 0u, 0u, 0u);
    if (piece < s.pieces && k < op.K && g < op.M) {
      if (normed) {
        const float* r = static_cast<const float*>(op.a) + (size_t)g * op.K + k;
        const float4 v0 = __ldcg(reinterpret_cast<const float4*>(r)), v1 = __ldcg(reinterpret_cast<const float4*>(r) + 1);
        const float4* gm = reinterpret_cast<const float4*>(static_cast<const float*>(op.w2) + k);
        const float4* bt = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(op.reserved_ptr) + k);
        const float4 g0 = gm[0], g1 = gm[1], b0 = bt[0], b1 = bt[1];
        const float mean = stats[2 * g], inv = stats[2 * g + 1];
        const __nv_bfloat162 p0 = __floats2bfloat162_rn((v0.x - mean) * inv * g0.x + b0.x, (v0.y - mean) * inv * g0.y + b0.y);
        const __nv_bfloat162 p1 = __floats2bfloat162_rn((v0.z - mean) * inv * g0.z + b0.z, (v0.w - mean) * inv * g0.w + b0.w);
        const __nv_bfloat162 p2 = __floats2bfloat162_rn((v1.x - mean) * inv * g1.x + b1.x, (v1.y - mean) * inv * g1.y + b1.y);
        const __nv_bfloat162 p3 = __floats2bfloat162_rn((v1.z - mean) * inv * g1.z + b1.z, (v1.w - mean) * inv * g1.w + b1.w);
        xr[j].x = *reinterpret_cast<const unsigned*>(&p0);
        xr[j].y = *reinterpret_cast<const unsigned*>(&p1);
        xr[j].z = *reinterpret_cast<const unsigned*>(&p2);
        xr[j].w = *reinterpret_cast<const unsigned*>(&p3);
      } else {
        xr[j] = ldcg16(static_cast<const __nv_bfloat16*>(op.a) + (size_t)g * op.K + k);
      }
    }
  }
  float acc[kGroup][4];
#pragma unroll
  for (int t = 0; t < kGroup; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[t][j] = 0.f;
  for (int tile = 0; tile < s.tiles; ++tile) {
    const int tg = tile % kGroup;
    for (int piece = 0; piece < s.pieces; ++piece) {
      // the ring's tail is this piece: pieces are staged in exactly the order they are used
      if (ring.count == 0) stage_next(ops, n_ops, ring, wbuf);
      slot_wait(ring.bars + 8 * ring.tail_slot, (ring.parity >> ring.tail_slot) & 1u, error);
      ring.parity ^= 1u << ring.tail_slot;
      __syncthreads();  // all warps have left the slot used before this one (it may be refilled now)
      const __nv_bfloat16* wt = wbuf + (size_t)ring.tail_slot * kSlotElems;
      ring.tail = next_piece(ops, n_ops, ring.tail);
      ring.tail_slot = (ring.tail_slot + 1) % kSlots;
      --ring.count;
      // refill behind it (never the slot in use: at most kSlots - 1 are staged while one is used)
      while (ring.count < kSlots - 1 && ring.head.op < n_ops) stage_next(ops, n_ops, ring, wbuf);
      const int first = piece * spp;
#pragma unroll
      for (int j = 0; j < kMaxJ; ++j) {
        const int sl = j * kWarps + warp - first;  // this warp's j-th slice, counted inside this piece
        if (sl >= 0 && sl < spp) {
          const int kl = sl * 32 + c * 8;
          const uint4 a_lo = *reinterpret_cast<const uint4*>(wt + g * ldw + kl);
          const uint4 a_hi = *reinterpret_cast<const uint4*>(wt + (g + 8) * ldw + kl);
#pragma unroll
          for (int t = 0; t < kGroup; ++t) {
            if (t == tg) {
              mma_bf16(acc[t], a_lo.x, a_hi.x, a_lo.y, a_hi.y, xr[j].x, xr[j].y);
              mma_bf16(acc[t], a_lo.z, a_hi.z, a_lo.w, a_hi.w, xr[j].z, xr[j].w);
            }
          }
        }
      }
    }
    if (tg == kGroup - 1 || tile == s.tiles - 1) {
          finish_tiles(op, s, tile - tg, tg + 1, acc, red);
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

constexpr size_t kRingBytes = (size_t)kSlots * kSlotElems * sizeof(__nv_bfloat16);
constexpr size_t kRedFloats = (size_t)kWarps * kGroup * 16 * 8;  // also the attention's scratch
constexpr size_t kProgramSmem = kRingBytes + kRedFloats * sizeof(float) + 4 * kWarps * sizeof(float);
static_assert(kRedFloats >= 2 * (size_t)kAttnScratchFloats, "the attention's scratch shares the sums' buffer");
static_assert(kProgramSmem <= 227 * 1024, "shared memory of the persistent kernel");

__global__ void __launch_bounds__(kThreads, 1)
decode_program_kernel(const EmberOp* __restrict__ ops, int n_ops, GridBarrier* bar, int* error, int* trace) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* wbuf = reinterpret_cast<__nv_bfloat16*>(smem_raw);                      // the ring
  float* red = reinterpret_cast<float*>(smem_raw + kRingBytes);                           // [kWarps][kGroup][128]
  float* rows = red + kRedFloats;                                                         // [2 * kWarps]: sums of warps
  float* stats = rows + 2 * kWarps;                                                       // [2 * kRows]: mean, 1/sd

  unsigned long long t_start = 0;
  // arrivals before this launch: every block reads the epoch before its first arrival, and block 0
  // advances it only after its last barrier, which no block passes before all have arrived at the first
  const unsigned long long arrivals0 = *(volatile unsigned long long*)&bar->epoch * (unsigned long long)(n_ops - 1) * gridDim.x;
  __shared__ unsigned long long slot_bars[kSlots];
  if (threadIdx.x == 0) {
    for (int b = 0; b < kSlots; ++b)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"((unsigned)__cvta_generic_to_shared(&slot_bars[b])));
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  Ring ring;
  ring.parity = 0;
  ring.bars = (unsigned)__cvta_generic_to_shared(slot_bars);
  ring.head = first_piece(ops, n_ops, 0);
  ring.tail = ring.head;
  ring.count = 0;
  ring.tail_slot = 0;
  while (ring.count < kSlots && ring.head.op < n_ops) stage_next(ops, n_ops, ring, wbuf);
  for (int i = 0; i < n_ops; ++i) {
    const EmberOp& op = ops[i];
    if (trace && threadIdx.x == 0) {  // a debugging aid: the operation each block has reached
      trace[blockIdx.x] = i + 1;
      if (blockIdx.x == 0 && i < 768) {  // and when block 0 began it, in nanoseconds since the kernel started
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (i == 0) t_start = now;
        trace[256 + i] = (int)(now - t_start);
      }
    }
    if (op.type == EMBER_OP_LINEAR) {
      run_linear(ops, n_ops, i, ring, wbuf, red, rows, stats, error);
      while (ring.count < kSlots && ring.head.op < n_ops) stage_next(ops, n_ops, ring, wbuf);  // the next products' weights
    } else if (op.type == EMBER_OP_ATTENTION) {
      run_attention(op, red, kAttnScratchFloats, error);
    } else if (op.type == EMBER_OP_LAYERNORM) {
      run_layernorm(op, rows);
    } else if (op.type == EMBER_OP_EMBED) {
      run_embed(op, error);
    }
    if (i + 1 < n_ops && !grid_barrier(bar, arrivals0 + (unsigned long long)(i + 1) * gridDim.x, error)) break;
  }
  // nothing of this block is in flight when it leaves: pieces staged and never used (after an error) are waited for
  for (int j = 0; j < ring.count; ++j) {
    const int sl = (ring.tail_slot + j) % kSlots;
    slot_wait(ring.bars + 8 * sl, (ring.parity >> sl) & 1u, error);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) bar->epoch = bar->epoch + 1;
  if (trace && threadIdx.x == 0) trace[blockIdx.x] = -1;  // left the kernel
}

}  // namespace

EMBER_API int ember_decode_program_op_size() { return (int)sizeof(EmberOp); }

// Bytes of device memory for the barrier's state (zero before the first run; every run leaves it
// ready for the next).
EMBER_API int ember_decode_program_state_size() { return (int)sizeof(GridBarrier); }

// Runs a program of `n_ops` operations (device array) for up to 8 rows.  `state`: the barrier's
// state; `error`: one int on the device, zero before the run, non-zero afterwards if a block gave
// up waiting at a barrier (1) or an index of the step's description was out of range (2); the
// results are then not valid.
// `trace`: null, or 1,024 ints in memory the host can read (pinned and mapped): each block
// writes there the number of the operation it has reached (1-based; -1 once it has left), which
// is still readable after a fault; from entry 256 on, the time at which block 0 began each operation.
EMBER_API int ember_decode_program_run(const void* ops, int n_ops, int max_rows, void* state, int* error, int* trace,
                                       cudaStream_t stream) {
  EMBER_CHECK(n_ops > 0 && max_rows > 0 && max_rows <= kRows, "decode_program: %d operations for %d rows (at most 8)", n_ops,
              max_rows);
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return ember_fail("decode_program: %s", cudaGetErrorString(e));
  }
  const size_t smem = kProgramSmem;
  const void* fn = (const void*)decode_program_kernel;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ember_fail("decode_program: %s", cudaGetErrorString(e));
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_program_kernel, kThreads, smem);
    if (e != cudaSuccess || per_sm < 1) return ember_fail("decode_program: the kernel does not fit an SM");
    configured = true;
  }
  GridBarrier* bar = static_cast<GridBarrier*>(state);
  void* args[] = {(void*)&ops, (void*)&n_ops, (void*)&bar, (void*)&error, (void*)&trace};
  cudaError_t e = cudaLaunchCooperativeKernel(fn, dim3(sms), dim3(kThreads), args, smem, stream);
  if (e != cudaSuccess) return ember_fail("decode_program: %s", cudaGetErrorString(e));
  return 0;
}
