// Inline PTX of the fifth-generation tensor-core path that more than one kernel of this library
// uses: mbarriers with time-limited waits, TMA tile loads, tcgen05 descriptors, products, commits
// and tensor-memory loads, and the host's tensor-map encoder.
//
// Every wait on an mbarrier gives up after two seconds and returns false; the kernels that use it
// then record a status code in host-visible memory, wait (with the same limit) for what they
// still have in flight, free their tensor memory and return.
#pragma once

#include <cuda.h>

#include <unordered_map>

#include "common.cuh"

namespace tc {

constexpr unsigned long long kWaitNs = 2000000000ull;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Waits for the phase of the given parity to complete.  False when the time ran out.  The polling
// loop is one function for the whole kernel, not a copy at every wait: these kernels run their code
// once, straight through, and a kernel of 96 KB (what inlined, unrolled polling loops made of the
// weight-streaming product) waits on its instruction fetches.
static __device__ __noinline__ bool mbar_wait_poll(unsigned bar, unsigned parity, unsigned long long limit_ns) {
  unsigned long long t0, t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try(bar, parity)) return true;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (t - t0 > limit_ns) return false;
  }
}
// (the limit is a parameter so that a test can make a wait run out in a millisecond: wait_probe.cu)
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, unsigned long long limit_ns = kWaitNs) {
  if (mbar_try(bar, parity)) return true;
  return mbar_wait_poll(bar, parity, limit_ns);
}

// One box of a tensor map into this block's shared memory; completion counted on `bar`.  No
// multicast: every block fetches what it uses.
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(map) : "memory");
}

// Shared-memory matrix descriptor of a tile whose rows are 128 bytes, swizzled by 128 bytes, groups
// of eight rows 1,024 bytes apart: start address / 16; leading offset 1 (one swizzle atom wide: not
// used); stride offset 1,024 / 16; descriptor version 1; layout type 2 (128-byte swizzle).  The
// same bits describe a K-major tile (rows = M or N, 64 values of K a row) and an MN-major tile
// (rows = K, 64 values of M or N a row); which one it is stands in the instruction descriptor.
__device__ __forceinline__ unsigned long long smem_desc_sw128(unsigned addr) {
  return (unsigned long long)((addr & 0x3FFFF) >> 4) | (1ull << 16) | ((unsigned long long)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
// Instruction descriptor of kind::f16: float32 accumulator, bfloat16 A and B, A K-major, B K-major
// or (b_mn_major) MN-major, M = m, N = n.
__device__ __forceinline__ unsigned instr_desc_bf16(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((unsigned)(n >> 3) << 17) |
         ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_1cta(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc,
                                          unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same two instructions issued by a whole, converged warp whose lanes all hold the same
// operands: one elected lane issues.  Operands that are the same in every lane can live in the
// warp's uniform registers, which is where the instruction reads them.  Measured (`bench.py
// --umma-issue`, umma_probe.cu): for M = 128 both ways cost the same, 46 to 48 cycles an
// instruction up to N = 64, 64 at N = 128 and 128 at N = 256 (the arithmetic itself, so an
// instruction narrower than N = 128 leaves the pipe idle part of the time); for M = 64 and N up
// to 64 the elected form takes 24 to 33 cycles against 46.  The product loops use this form.
__device__ __forceinline__ void umma_1cta_elect(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc,
                                                unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p, e;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "elect.sync _|e, 0xffffffff;\n"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit_1cta_elect(unsigned bar) {
  asm volatile(
      "{\n.reg .pred e;\n"
      "elect.sync _|e, 0xffffffff;\n"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}\n" ::"r"(bar)
      : "memory");
}
// Arrives on the barrier once the products issued so far by this thread are complete.
__device__ __forceinline__ void umma_commit_1cta(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// Shared memory written by ordinary stores becomes visible to the tensor cores' and TMA's reads.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc_1cta(unsigned smem_dst, unsigned cols) {  // a whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_dst), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_free_1cta(unsigned taddr, unsigned cols) {  // the warp that allocated
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols) : "memory");
}
// 32 consecutive accumulator columns of this thread's lane (issue only; tmem_wait before use)
__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, "
      "[%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
        "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
        "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
// 16 consecutive accumulator columns of this thread's lane (issue only; tmem_wait before use)
__device__ __forceinline__ void tmem_ld16(unsigned taddr, unsigned (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// ------------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiled encoder() {
  static EncodeTiled fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    return (e == cudaSuccess && q == cudaDriverEntryPointSuccess) ? reinterpret_cast<EncodeTiled>(p) : nullptr;
  }();
  return fn;
}

// A [rows, cols] bfloat16 matrix whose rows are `row_bytes` apart, copied in boxes of box_rows x 64
// values with the 128-byte swizzle; what lies outside the matrix reads as zero.  Returns false if
// the driver refuses.
inline bool encode_bf16_sw128(CUtensorMap* out, const void* ptr, size_t rows, size_t cols, size_t row_bytes, int box_rows) {
  EncodeTiled enc = encoder();
  if (!enc) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A [rows, cols] float32 matrix whose rows are `row_bytes` apart, copied in boxes of box_rows x 128
// values as they lie (no swizzle: a row of the box is 512 consecutive bytes of shared memory); what
// lies outside the matrix reads as zero.
inline bool encode_f32_plain(CUtensorMap* out, const void* ptr, size_t rows, size_t cols, size_t row_bytes, int box_rows) {
  EncodeTiled enc = encoder();
  if (!enc) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A [rows, cols] bfloat16 row-major matrix (16-byte aligned, cols a multiple of 8), copied in boxes
// of box_rows x 64 values with the 128-byte swizzle; what lies outside the matrix reads as zero.
// Maps are kept by (address, shape, box).  0, or an error code after ember_fail.  (gemm_tc.cu)
int cached_map(const void* ptr, int rows, int cols, int box_rows, CUtensorMap* out);
// The same for a [rows, cols] float32 row-major matrix (cols a multiple of 4) in boxes of box_rows x 128 values, unswizzled.
int cached_map_f32(const void* ptr, int rows, int cols, int box_rows, CUtensorMap* out);

// One host-visible status word per process (pinned and mapped): kernels write a code there when a
// wait ran out; the host reads and clears it after it has synchronized.
struct Status {
  int* host = nullptr;
  int* device = nullptr;
};
inline Status& status() {
  static Status s = [] {
    Status t;
    if (cudaHostAlloc(reinterpret_cast<void**>(&t.host), sizeof(int), cudaHostAllocMapped) != cudaSuccess) return Status();
    *t.host = 0;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&t.device), t.host, 0) != cudaSuccess) return Status();
    return t;
  }();
  return s;
}

}  // namespace tc
