// Library matrix products of the bfloat16 path: Y[M,N] = A[M,K] . W[N,K]^T through cuBLASLt, with
// the bias, the tanh GELU and the float32 residual sum in the product's epilogue where the
// library has them.
//
// ember.cpp's engine uses a library for these too (cublasSgemm, cuda_kernels.cu:3617-3621; bias,
// GELU and the residual add as separate kernels after it, graph_ir_cuda.cu:67-76, 230-242).
// Operands are bfloat16, accumulation is float32; the output is bfloat16, or float32 when it is
// the residual stream or the logits.
//
// Row-major Y = A W^T is the column-major product Y^T[N,M] = op_T(W as K x N) . (A as K x M).
#include <cublasLt.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace {

struct PlanKey {
  int M, N, K, act, bias, residual, out_dtype;
  bool operator==(const PlanKey& o) const {
    return M == o.M && N == o.N && K == o.K && act == o.act && bias == o.bias && residual == o.residual &&
           out_dtype == o.out_dtype;
  }
};
struct PlanHash {
  size_t operator()(const PlanKey& k) const {
    size_t h = 1469598103934665603ull;
    const int v[7] = {k.M, k.N, k.K, k.act, k.bias, k.residual, k.out_dtype};
    for (int x : v) h = (h ^ (size_t)x) * 1099511628211ull;
    return h;
  }
};
struct Plan {
  cublasLtMatmulDesc_t op = nullptr;
  cublasLtMatrixLayout_t a = nullptr, b = nullptr, c = nullptr;
  cublasLtMatmulAlgo_t algo;
  bool bias_is_bf16 = false;
};

cublasLtHandle_t g_handle = nullptr;
std::mutex g_mutex;
std::unordered_map<PlanKey, Plan, PlanHash> g_plans;
// The algorithm that timing chose, kept per bucket of M (M rounded up to a multiple of 128): every new
// prompt-length mix is a new M, and timing eight candidates for each would put milliseconds into the
// request path; a bucket is timed once and its choice is checked (not timed) for the other M of the bucket.
std::unordered_map<PlanKey, cublasLtMatmulAlgo_t, PlanHash> g_tuned;
constexpr size_t kMaxPlans = 512;  // descriptors kept; beyond that all are dropped and made again as they come

void drop_plans() {
  for (auto& kv : g_plans) {
    cublasLtMatmulDescDestroy(kv.second.op);
    cublasLtMatrixLayoutDestroy(kv.second.a);
    cublasLtMatrixLayoutDestroy(kv.second.b);
    cublasLtMatrixLayoutDestroy(kv.second.c);
  }
  g_plans.clear();
}

const char* lt_status(cublasStatus_t s) {
  switch (s) {
    case CUBLAS_STATUS_NOT_INITIALIZED: return "not initialized";
    case CUBLAS_STATUS_ALLOC_FAILED: return "allocation failed";
    case CUBLAS_STATUS_INVALID_VALUE: return "invalid value";
    case CUBLAS_STATUS_ARCH_MISMATCH: return "architecture mismatch";
    case CUBLAS_STATUS_EXECUTION_FAILED: return "execution failed";
    case CUBLAS_STATUS_INTERNAL_ERROR: return "internal error";
    case CUBLAS_STATUS_NOT_SUPPORTED: return "not supported";
    default: return "error";
  }
}

#define LT_TRY(call)                                                         \
  do {                                                                       \
    cublasStatus_t s_ = (call);                                              \
    if (s_ != CUBLAS_STATUS_SUCCESS) return ember_fail("linear_bf16: %s: %s", #call, lt_status(s_)); \
  } while (0)

constexpr int kCandidates = 8;

// Builds the descriptors for one shape and asks the library for algorithms (its heuristic's
// order).  Returns 0 and fills `plan` with the first, or 2 when the library offers none for this
// combination; the others go to `more`.
int make_plan(const PlanKey& key, bool bias_bf16, size_t workspace_bytes, Plan* plan, cublasLtMatmulAlgo_t* more,
              int* n_more) {
  const cudaDataType_t out_type = key.out_dtype == EMBER_F32 ? CUDA_R_32F : CUDA_R_16BF;
  LT_TRY(cublasLtMatmulDescCreate(&plan->op, CUBLAS_COMPUTE_32F, CUDA_R_32F));
  const cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
  LT_TRY(cublasLtMatmulDescSetAttribute(plan->op, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta)));
  LT_TRY(cublasLtMatmulDescSetAttribute(plan->op, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb)));
  cublasLtEpilogue_t epi = CUBLASLT_EPILOGUE_DEFAULT;
  if (key.bias && key.act == EMBER_ACT_GELU_TANH) epi = CUBLASLT_EPILOGUE_GELU_BIAS;
  else if (key.act == EMBER_ACT_GELU_TANH) epi = CUBLASLT_EPILOGUE_GELU;
  else if (key.bias) epi = CUBLASLT_EPILOGUE_BIAS;
  LT_TRY(cublasLtMatmulDescSetAttribute(plan->op, CUBLASLT_MATMUL_DESC_EPILOGUE, &epi, sizeof(epi)));
  if (key.bias) {
    const cudaDataType_t bt = bias_bf16 ? CUDA_R_16BF : CUDA_R_32F;
    LT_TRY(cublasLtMatmulDescSetAttribute(plan->op, CUBLASLT_MATMUL_DESC_BIAS_DATA_TYPE, &bt, sizeof(bt)));
  }
  LT_TRY(cublasLtMatrixLayoutCreate(&plan->a, CUDA_R_16BF, key.K, key.N, key.K));  // W as K x N, ld K
  LT_TRY(cublasLtMatrixLayoutCreate(&plan->b, CUDA_R_16BF, key.K, key.M, key.K));  // A as K x M, ld K
  LT_TRY(cublasLtMatrixLayoutCreate(&plan->c, out_type, key.N, key.M, key.N));     // Y^T as N x M, ld N
  cublasLtMatmulPreference_t pref = nullptr;
  LT_TRY(cublasLtMatmulPreferenceCreate(&pref));
  LT_TRY(cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &workspace_bytes,
                                              sizeof(workspace_bytes)));
  cublasLtMatmulHeuristicResult_t result[kCandidates];
  int found = 0;
  cublasStatus_t s = cublasLtMatmulAlgoGetHeuristic(g_handle, plan->op, plan->a, plan->b, plan->c, plan->c, pref,
                                                    kCandidates, result, &found);
  cublasLtMatmulPreferenceDestroy(pref);
  if (s != CUBLAS_STATUS_SUCCESS || found == 0) {
    cublasLtMatmulDescDestroy(plan->op);
    cublasLtMatrixLayoutDestroy(plan->a);
    cublasLtMatrixLayoutDestroy(plan->b);
    cublasLtMatrixLayoutDestroy(plan->c);
    *plan = Plan();
    return 2;
  }
  plan->algo = result[0].algo;
  plan->bias_is_bf16 = bias_bf16;
  *n_more = 0;
  for (int i = 1; i < found; ++i)
    if (result[i].state == CUBLAS_STATUS_SUCCESS) more[(*n_more)++] = result[i].algo;
  return 0;
}

// Times the candidates on the call's own operands, writing to `scratch` (as large as the output),
// and keeps the fastest in `plan`.  The heuristic's first choice is not always the best for a
// given shape; this runs once per shape, synchronizes the stream, and is skipped without scratch.
void tune_plan(Plan* plan, const cublasLtMatmulAlgo_t* more, int n_more, const void* A, const void* W, const void* C,
               float beta, void* scratch, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  cudaEvent_t t0, t1;
  if (cudaEventCreate(&t0) != cudaSuccess) return;
  if (cudaEventCreate(&t1) != cudaSuccess) {
    cudaEventDestroy(t0);
    return;
  }
  const float one = 1.0f;
  float best_ms = 0.f;
  cublasLtMatmulAlgo_t best = plan->algo;
  for (int i = -1; i < n_more; ++i) {
    const cublasLtMatmulAlgo_t& algo = i < 0 ? plan->algo : more[i];
    bool ok = true;
    float ms = 0.f;
    for (int rep = 0; rep < 4 && ok; ++rep) {  // the first run is not timed
      if (rep == 1) cudaEventRecord(t0, stream);
      ok = cublasLtMatmul(g_handle, plan->op, &one, W, plan->a, A, plan->b, &beta, C ? C : scratch, plan->c, scratch,
                          plan->c, &algo, workspace, workspace_bytes, stream) == CUBLAS_STATUS_SUCCESS;
    }
    if (!ok || cudaEventRecord(t1, stream) != cudaSuccess || cudaEventSynchronize(t1) != cudaSuccess ||
        cudaEventElapsedTime(&ms, t0, t1) != cudaSuccess)
      continue;
    if (i < 0 || ms < best_ms) best_ms = ms, best = algo;
    if (i < 0) best_ms = ms;
  }
  plan->algo = best;
  cudaEventDestroy(t0);
  cudaEventDestroy(t1);
}

}  // namespace

// bias_f32 / bias_bf16: the same bias in both types (both null: no bias).  The float32 one is used
// where the library takes it with this output type, else the bfloat16 one.
// residual: float32 [M,N] added to the product (out is float32 then, and may be the same buffer).
// act: none or the tanh GELU (the erf form is not a library epilogue; the caller applies it).
// tune_scratch: null, or a buffer as large as the output: the first call for a shape whose bucket of
// M (multiples of 128) has not been timed yet then times the library's candidate algorithms there
// (synchronizing the stream) and keeps the fastest for the bucket.
EMBER_API int ember_linear_bf16(const void* A, const void* W, const float* bias_f32, const void* bias_bf16,
                                const float* residual, void* out, int M, int N, int K, int act, int out_dtype,
                                void* workspace, size_t workspace_bytes, void* tune_scratch, cudaStream_t stream) {
  EMBER_CHECK(M > 0 && N > 0 && K > 0, "linear_bf16: M = %d, N = %d, K = %d", M, N, K);
  EMBER_CHECK(act == EMBER_ACT_NONE || act == EMBER_ACT_GELU_TANH, "linear_bf16: activation %d is no library epilogue",
              act);
  EMBER_CHECK(out_dtype == EMBER_F32 || out_dtype == EMBER_BF16, "linear_bf16: output type %d", out_dtype);
  EMBER_CHECK(!residual || out_dtype == EMBER_F32, "linear_bf16: a residual sum needs a float32 output");
  EMBER_CHECK(K % 8 == 0, "linear_bf16: K = %d is not a multiple of 8 (16-byte rows)", K);
  EMBER_CHECK((bias_f32 == nullptr) == (bias_bf16 == nullptr), "linear_bf16: give the bias in both types or not at all");
  const PlanKey key{M, N, K, act, bias_f32 != nullptr, residual != nullptr, out_dtype};
  PlanKey bucket = key;
  bucket.M = (M + 127) / 128 * 128;
  // One lock from the look-up to the launch: a plan's descriptor is shared by all callers of its shape,
  // and the bias pointer is set on it for this call (the launch itself only queues work).
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_handle) LT_TRY(cublasLtCreate(&g_handle));
  auto it = g_plans.find(key);
  if (it == g_plans.end()) {
    if (g_plans.size() >= kMaxPlans) drop_plans();
    Plan fresh;
    cublasLtMatmulAlgo_t more[kCandidates];
    int n_more = 0;
    int rc = make_plan(key, /*bias_bf16=*/false, workspace_bytes, &fresh, more, &n_more);
    if (rc == 2 && key.bias) rc = make_plan(key, /*bias_bf16=*/true, workspace_bytes, &fresh, more, &n_more);
    if (rc == 2) return ember_fail("linear_bf16: the library has no algorithm for M=%d N=%d K=%d", M, N, K);
    if (rc != 0) return rc;
    if (tune_scratch) {
      auto tuned = g_tuned.find(bucket);
      cublasLtMatmulHeuristicResult_t check;
      if (tuned != g_tuned.end()) {  // this bucket was timed before: its choice, if the library takes it for this M too
        if (cublasLtMatmulAlgoCheck(g_handle, fresh.op, fresh.a, fresh.b, fresh.c, fresh.c, &tuned->second, &check) ==
                CUBLAS_STATUS_SUCCESS &&
            check.state == CUBLAS_STATUS_SUCCESS && check.workspaceSize <= workspace_bytes)
          fresh.algo = tuned->second;
      } else if (n_more > 0) {
        if (key.bias) {
          const void* bias = fresh.bias_is_bf16 ? bias_bf16 : (const void*)bias_f32;
          LT_TRY(cublasLtMatmulDescSetAttribute(fresh.op, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &bias, sizeof(bias)));
        }
        tune_plan(&fresh, more, n_more, A, W, residual, residual ? 1.0f : 0.0f, tune_scratch, workspace, workspace_bytes,
                  stream);
        g_tuned.emplace(bucket, fresh.algo);
      }
    }
    it = g_plans.emplace(key, fresh).first;
  }
  const Plan& plan = it->second;
  if (key.bias) {
    const void* bias = plan.bias_is_bf16 ? bias_bf16 : (const void*)bias_f32;
    LT_TRY(cublasLtMatmulDescSetAttribute(plan.op, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &bias, sizeof(bias)));
  }
  const float one = 1.0f, zero = 0.0f;
  const void* C = residual ? (const void*)residual : (const void*)out;
  LT_TRY(cublasLtMatmul(g_handle, plan.op, &one, W, plan.a, A, plan.b, residual ? &one : &zero, C, plan.c, out, plan.c,
                        &plan.algo, workspace, workspace_bytes, stream));
  return 0;
}
