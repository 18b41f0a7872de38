// A measurement, not a part of any model: how many cycles one `tcgen05.mma` (kind::f16, bfloat16,
// cta_group::1) costs the thread that issues it, by instruction shape and by the way it is issued.
//
// What it found on a B200: an instruction of M = 128 costs its issuing thread 46 to 48 cycles up to
// N = 64, 64 cycles at N = 128 and 128 at N = 256, whichever way it is issued (from inside
// `if (threadIdx.x == 0)`, or by a whole converged warp whose lanes hold the same operands with
// `elect.sync` choosing the lane); from N = 128 on that is the arithmetic itself (8,100 flop a cycle),
// below it the pipe idles: a product of N = 64 runs at two thirds of the tensor peak at best, one of
// N = 16 at a fifth.  For M = 64 and N up to 64 the elected form is the faster one (24 to 33 cycles
// against 46).  Products that accumulate into one tensor-memory address cost no more than products into
// different ones.  `bench.py --umma-issue` prints the table.
#include "tc_common.cuh"

namespace {

using namespace tc;

__global__ void umma_issue_kernel(int m, int n, int iters, int elected, int commit_every, int wait_too, long long* out) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ unsigned long long bar, bar2, bar3;
  __shared__ unsigned s_tmem;
  const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    mbar_init(smem_u32(&bar2), 1);
    mbar_init(smem_u32(&bar3), 1);
    mbar_arrive(smem_u32(&bar3));  // its phase 0 is complete: a wait on it returns at once
    mbar_init_fence();
  }
  for (int i = threadIdx.x; i < 48 * 1024 / 4; i += blockDim.x)
    reinterpret_cast<unsigned*>(smem_raw + (base - smem_u32(smem_raw)))[i] = 0;  // operands: zeros
  if (warp == 0) tmem_alloc_1cta(smem_u32(&s_tmem), 256);
  fence_async_smem();
  fence_before();
  __syncthreads();
  fence_after();
  const unsigned tmem = s_tmem;
  const unsigned idesc = instr_desc_bf16(m, n, false);
  const unsigned long long da = smem_desc_sw128(base), db = smem_desc_sw128(base + 16384);
  bool ended = true;
  if (!elected) {
    if (threadIdx.x == 0) {
      const long long t0 = clock64();
      const int group = commit_every ? commit_every : iters;  // (nested loops: a remainder by a run-time number would cost more than the products)
      for (int i = 0; i < iters; i += group) {
        for (int j = 0; j < group; ++j) umma_1cta(tmem, da + 2 * (j & 3), db + 2 * (j & 3), idesc, 1);
        if (commit_every) umma_commit_1cta(smem_u32(&bar2));
      }
      const long long t1 = clock64();
      umma_commit_1cta(smem_u32(&bar));
      ended = mbar_wait(smem_u32(&bar), 0);
      out[0] = t1 - t0, out[1] = clock64() - t0, out[2] = ended;
    }
  } else if (warp == 0) {
    const long long t0 = clock64();
    const int group = commit_every ? commit_every : iters;
    for (int i = 0; i < iters; i += group) {
      if (wait_too) {  // what a kernel's loop does before the products of a stage: a wait that is already satisfied, and the fence
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar3), 0))) break;
        fence_after();
      }
      for (int j = 0; j < group; ++j) umma_1cta_elect(tmem, da + 2 * (j & 3), db + 2 * (j & 3), idesc, 1);
      if (commit_every) umma_commit_1cta_elect(smem_u32(&bar2));
    }
    const long long t1 = clock64();
    umma_commit_1cta_elect(smem_u32(&bar));
    ended = mbar_wait(smem_u32(&bar), 0);
    if (lane == 0) out[0] = t1 - t0, out[1] = clock64() - t0, out[2] = ended;
  }
  fence_before();
  __syncthreads();
  if (warp == 0) {
    fence_after();
    tmem_free_1cta(tmem, 256);
  }
}

}  // namespace

// One block issues `iters` products of M = m (64 or 128) by N = n (16 to 256, a multiple of 16) by K = 16
// on zeros and waits for them.  elected: 0 from a single thread's branch, 1 by a converged warp with
// elect.sync.  commit_every: 0, or a tcgen05.commit (to a barrier nobody waits on) after every so many products,
// as a kernel's loop hands its stages back; wait_too (elected form only): a satisfied mbarrier wait and a
// tcgen05.fence::after_thread_sync before each such group, as that loop has them.  out (device, 3 x int64): cycles to issue all, cycles until all are complete, 1 if the wait ended.
EMBER_API int ember_umma_issue_probe(int m, int n, int iters, int elected, int commit_every, int wait_too, long long* out,
                                     cudaStream_t stream) {
  EMBER_CHECK((m == 64 || m == 128) && n >= 16 && n <= 256 && n % 16 == 0, "umma_issue_probe: M = %d (64 or 128), N = %d (16 to 256 in 16s)",
              m, n);
  EMBER_CHECK(iters > 0 && iters <= 4096, "umma_issue_probe: %d products (1 to 4,096)", iters);
  static bool configured = false;
  if (!configured) {
    const cudaError_t e = cudaFuncSetAttribute(umma_issue_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (e != cudaSuccess) return ember_fail("umma_issue_probe: %s", cudaGetErrorString(e));
    configured = true;
  }
  EMBER_CHECK(commit_every >= 0, "umma_issue_probe: commit_every = %d", commit_every);
  umma_issue_kernel<<<1, 128, 100 * 1024, stream>>>(m, n, iters, elected, commit_every, wait_too, out);
  EMBER_LAUNCH_OK("umma_issue_probe");
  return 0;
}
