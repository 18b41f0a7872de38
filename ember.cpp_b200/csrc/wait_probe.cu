// A wait that nothing ends, with a short limit: the way the kernels' bounded waits give up, made to
// happen on purpose and harmlessly.
//
// Every wait on an mbarrier in the tcgen05 kernels (gemm_tc.cu, attention_tc.cu, linear_stream.cu)
// goes through tc::mbar_wait, which gives up after a time limit, after which the kernel records a
// code in the host-visible status word, lets its copies land, frees what it holds and returns; the
// host then finds the code (`ember_tc_status`) and refuses the launch's results.  In a correct
// program none of these waits ever runs out, so nothing exercises that path.  This entry point
// does: one block initialises an mbarrier that no copy and no thread will ever complete, waits on
// it through the same tc::mbar_wait with the limit the caller gives (a millisecond is plenty),
// records code 31 when the wait returns false, and ends.  Nothing faults, traps or hangs: the
// kernel runs for `limit_ns` and returns, and the context stays usable.
#include "tc_common.cuh"

namespace {

__global__ void wait_probe_kernel(unsigned long long limit_ns, int* status) {
  __shared__ unsigned long long bar;
  const unsigned addr = tc::smem_u32(&bar);
  if (threadIdx.x == 0) {
    tc::mbar_init(addr, 1);
    tc::mbar_init_fence();
  }
  __syncthreads();
  const bool ended = tc::mbar_wait(addr, 0, limit_ns);  // nobody arrives: this returns false after limit_ns
  if (!ended && threadIdx.x == 0) atomicCAS(status, 0, 31);
}

}  // namespace

// limit_ns: how long the wait may last, 1,000 to 100,000,000 (a test passes about a millisecond).
// After the stream has been synchronized `ember_tc_status()` returns 31 once.
EMBER_API int ember_wait_probe(unsigned long long limit_ns, cudaStream_t stream) {
  EMBER_CHECK(limit_ns >= 1000ull && limit_ns <= 100000000ull, "wait_probe: a limit of %llu ns is not between a microsecond and 0.1 s",
              limit_ns);
  if (!tc::status().device) return ember_fail("wait_probe: no host-visible status word");
  wait_probe_kernel<<<1, 32, 0, stream>>>(limit_ns, tc::status().device);
  EMBER_LAUNCH_OK("wait_probe");
  return 0;
}
