// bf16 matrix products through cuBLASLt, where libmir's engine also calls a library
// (CublasLtBf16Plan / DenseMatmulPlan of the external mircuda crate,
// cuda/src/backend/linear/autotune/candidate.rs:3-6,18-22).
//
//   out[M, N] = beta * out + x[M, K] . w[N, K]^T (+ bias[N])
// x and w are bf16 row-major; out is bf16 or float row-major; accumulation is 32-bit.
// In cuBLAS's column-major terms that is C[N, M] = op_T(w as K x N) . (x as K x M).
// Plans (descriptor, layouts, heuristic algorithm) are cached per shape.
#include <cublasLt.h>
#include <map>
#include <mutex>
#include <tuple>
#include "common.cuh"

namespace {

struct Plan {
  cublasLtMatmulDesc_t op = nullptr;
  cublasLtMatrixLayout_t w = nullptr, x = nullptr, c = nullptr;
  cublasLtMatmulAlgo_t algo;
};

using Key = std::tuple<int, int, int, int, int, int, int, int, size_t>;

cublasLtHandle_t g_handle = nullptr;
std::mutex g_mutex;
std::map<Key, Plan> g_plans;

#define LT_CHECK(call)                                                     \
  do {                                                                     \
    const cublasStatus_t status_ = (call);                                 \
    if (status_ != CUBLAS_STATUS_SUCCESS) {                                \
      mir_set_error("cuBLASLt: %s failed with status %d", #call, (int)status_); \
      return MIR_LIBRARY_ERROR;                                            \
    }                                                                      \
  } while (0)

int make_plan(const Key& key, Plan& plan) {
  const int m = std::get<0>(key), n = std::get<1>(key), k = std::get<2>(key);
  const int ldx = std::get<3>(key), ldw = std::get<4>(key), ldo = std::get<5>(key);
  const int out_f32 = std::get<6>(key), has_bias = std::get<7>(key);
  const size_t workspace = std::get<8>(key);
  LT_CHECK(cublasLtMatmulDescCreate(&plan.op, CUBLAS_COMPUTE_32F, CUDA_R_32F));
  const cublasOperation_t trans = CUBLAS_OP_T, none = CUBLAS_OP_N;
  LT_CHECK(cublasLtMatmulDescSetAttribute(plan.op, CUBLASLT_MATMUL_DESC_TRANSA, &trans, sizeof(trans)));
  LT_CHECK(cublasLtMatmulDescSetAttribute(plan.op, CUBLASLT_MATMUL_DESC_TRANSB, &none, sizeof(none)));
  const cudaDataType_t out_type = out_f32 ? CUDA_R_32F : CUDA_R_16BF;
  if (has_bias) {
    const cublasLtEpilogue_t epilogue = CUBLASLT_EPILOGUE_BIAS;
    LT_CHECK(cublasLtMatmulDescSetAttribute(plan.op, CUBLASLT_MATMUL_DESC_EPILOGUE, &epilogue, sizeof(epilogue)));
    LT_CHECK(cublasLtMatmulDescSetAttribute(plan.op, CUBLASLT_MATMUL_DESC_BIAS_DATA_TYPE, &out_type, sizeof(out_type)));
  }
  LT_CHECK(cublasLtMatrixLayoutCreate(&plan.w, CUDA_R_16BF, k, n, ldw));
  LT_CHECK(cublasLtMatrixLayoutCreate(&plan.x, CUDA_R_16BF, k, m, ldx));
  LT_CHECK(cublasLtMatrixLayoutCreate(&plan.c, out_type, n, m, ldo));
  cublasLtMatmulPreference_t preference = nullptr;
  LT_CHECK(cublasLtMatmulPreferenceCreate(&preference));
  LT_CHECK(cublasLtMatmulPreferenceSetAttribute(preference, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &workspace,
                                                sizeof(workspace)));
  cublasLtMatmulHeuristicResult_t result;
  int found = 0;
  const cublasStatus_t status = cublasLtMatmulAlgoGetHeuristic(g_handle, plan.op, plan.w, plan.x, plan.c, plan.c,
                                                               preference, 1, &result, &found);
  cublasLtMatmulPreferenceDestroy(preference);
  if (status != CUBLAS_STATUS_SUCCESS || found == 0) {
    mir_set_error("cuBLASLt has no algorithm for m %d n %d k %d (status %d)", m, n, k, (int)status);
    return MIR_LIBRARY_ERROR;
  }
  plan.algo = result.algo;
  return MIR_OK;
}

}  // namespace

// bias has the dtype of out.  workspace may be null when workspace_bytes is 0.
MIR_EXPORT int mir_gemm_bf16_lt(const void* x, int ldx, const void* w, int ldw, const void* bias, void* out, int ldo,
                                int out_f32, int m, int n, int k, float beta, void* workspace,
                                size_t workspace_bytes, cudaStream_t stream) {
  if (m == 0 || n == 0) return MIR_OK;
  if (m < 0 || n < 0 || k <= 0 || ldx < k || ldw < k || ldo < n) {
    mir_set_error("gemm_bf16: bad sizes m %d n %d k %d ldx %d ldw %d ldo %d", m, n, k, ldx, ldw, ldo);
    return MIR_BAD_ARGUMENT;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_handle) LT_CHECK(cublasLtCreate(&g_handle));
  const Key key(m, n, k, ldx, ldw, ldo, out_f32, bias != nullptr, workspace_bytes);
  auto it = g_plans.find(key);
  if (it == g_plans.end()) {
    Plan plan;
    const int status = make_plan(key, plan);
    if (status != MIR_OK) return status;
    it = g_plans.emplace(key, plan).first;
  }
  Plan& plan = it->second;
  if (bias) LT_CHECK(cublasLtMatmulDescSetAttribute(plan.op, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &bias, sizeof(bias)));
  const float alpha = 1.0f;
  LT_CHECK(cublasLtMatmul(g_handle, plan.op, &alpha, w, plan.w, x, plan.x, &beta, out, plan.c, out, plan.c, &plan.algo,
                          workspace, workspace_bytes, stream));
  mir_count_launch("gemm_bf16_lt");
  return MIR_OK;
}
