/* C declarations of entry points of libember_kernels.so that are meant to be called from outside
 * the Python package.  All of them take raw device pointers and a stream, return 0 on success and
 * leave a message for ember_last_error() otherwise. */
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* ember_last_error(void);

/* Decode attention over the paged cache (bfloat16, one new token per sequence) that allocates
 * nothing.  This entry point has no counterpart in ember.cpp.
 *
 * Who needs it: a host program that may not allocate device memory while it runs -- one that gave
 * the whole GPU to a memory pool of its own at start-up, one that runs under a fixed memory budget
 * that was checked once, or one that calls from a place where cudaMalloc is not allowed or too
 * costly because it synchronises the device (a latency-critical loop, a callback).  The library's
 * ordinary entry point, ember_attention_decode, takes its scratch from the caller; the Python
 * package gets that scratch from torch's allocator.  Here the scratch is built into the library:
 * two fixed __device__ arrays (4 MiB of partial results, 16,384 counters) that every GPU holds from
 * the moment it loads the library until the process ends.
 *
 * Limits: T * n_heads <= 16,384, and T * n_heads * ceil(n_blocks / pages_per_chunk) * (hd + 2)
 * <= 1,048,576 floats; larger calls are refused with a message (use more pages per chunk, or the
 * entry point that takes scratch).  It calls no cudaMalloc, cudaFree or allocating library
 * routine.  The first call on a device looks up the arrays' device addresses; make that call
 * before any stream capture.  All calls on a device share the arrays: two calls that overlap on
 * the GPU (different streams without an ordering between them) race and give wrong results.
 *
 * Arguments as ember_attention_decode without its two scratch pointers:
 *   qkv        bfloat16 [T, (n_heads + 2 kv_heads) * hd], the step's q | k | v
 *   kc, vc     the layer's key and value pages, bfloat16 [pages, kv_heads, 64, hd]
 *   out        bfloat16 [T, n_heads * hd]
 *   positions, token_seq [T]; seq_slot [sequences] (slot < 0: padding); pages [sequences, max_blocks]
 *   n_blocks   pages the longest sequence can hold in this call (<= max_blocks)
 *   store_kv   write each token's own key and value into the cache before attending */
int ember_attention_decode_static(const void* qkv, const void* kc, const void* vc, void* out, const int* positions,
                                  const int* token_seq, const int* seq_slot, const int* pages, int max_blocks,
                                  int n_blocks, int T, int n_heads, int kv_heads, int hd, float scale, int window,
                                  int pages_per_chunk, int store_kv, cudaStream_t stream);

/* Y[M,N] = A[M,K] . W[N,K]^T (+ bias) (activation) (+ residual): the tcgen05 product with its
 * epilogue.  A, W bfloat16 row-major and 16-byte aligned, K a multiple of 8; bias float32 [N] or
 * null; residual float32 [M,N] or null (out_dtype is then 0, float32, and out may be the residual's
 * buffer); act 0 none, 1 tanh GELU, 2 erf GELU; out_dtype 0 float32, 1 bfloat16; tile_n 0 (the
 * kernel chooses) or a multiple of 16 up to 256.  ember_tc_status() returns, after the stream was
 * synchronized, 0 or the code of a wait that ran out in a launch of a tcgen05 kernel since the last call. */
int ember_linear_tc(const void* A, const void* W, const float* bias, const float* residual, void* out, int M, int N, int K,
                    int act, int out_dtype, int tile_n, cudaStream_t stream);
int ember_tc_status(void);

#ifdef __cplusplus
}
#endif
