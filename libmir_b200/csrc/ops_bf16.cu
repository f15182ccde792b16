// Which kernel runs a bfloat16 matrix product, decided in one place for every caller (the Python launchers and the
// layer executor):
//
//   up to few_rows_max rows (decode steps, short portions)   the tcgen05 weight-streaming kernel (gemm_tc_stream.cu),
//                                                            which also takes over the RMSNorms around it
//   gate-up with SiLU, from tensor_core_min_rows rows        the tcgen05 many-rows kernel (gemm_tc.cu)
//   everything else                                          cuBLASLt (gemm_lt.cu), where libmir also calls a library
//                                                            (cuda/src/backend/linear/mod.rs:141-194)
//
// The thresholds are options with the measurements that chose them; mir_set_option changes them for A/B runs.
#include <cstring>
#include "common.cuh"
#define MIR_WITH_BF16
#include "launchers.h"

namespace {

// Up to how many rows a product runs the weight-streaming kernel rather than the library.  The kernel takes up to
// 128; measured alone at 64 rows it loses to cuBLASLt (12.2 / 8.5, 17.0 / 15.2, 14.9 / 8.2 us), and at 17 to 32
// rows it is about as fast, but there it also takes over the two RMSNorms of a layer and the SwiGLU, which the
// library path runs as kernels of their own: decode steps at Qwen3-4B sizes, library / streaming: batch 17 3.76 /
// 3.56 ms, batch 24 4.11 / 3.91 ms, batch 32 4.50 / 4.31 ms; batch 64 6.27 / 6.65 ms.
int g_few_rows_max = 32;
// Up to how many rows the streaming kernel writes and reads what a folded norm needs (kNormStatStride).
int g_folded_norm_max_rows = 32;
// From how many rows the tcgen05 kernel computes the gated feed-forward product.  Measured at K 2,560, I 9,728:
// 2,048 rows 153 us against 175 us for the library product and the SiLU-multiply kernel, 512 rows 55 against 59,
// 128 rows 26 against 37, 32 rows 25 against 26.
int g_tensor_core_min_rows = 128;
// The streaming epilogues in use (bit 0 store, 1 accumulate, 2 float32, 3 SwiGLU); the rest go to the library.
int g_few_rows_modes = 0xF;

enum Mode : int { STORE = 0, ACCUM = 1, F32 = 2, SWIGLU = 3 };

struct Option { const char* name; int* value; };
Option g_options[] = {{"few_rows_max", &g_few_rows_max}, {"folded_norm_max_rows", &g_folded_norm_max_rows},
                      {"tensor_core_min_rows", &g_tensor_core_min_rows}, {"few_rows_modes", &g_few_rows_modes}};

bool few_rows_ok(const void* x, int ldx, int m, int k) {
  return m > 0 && m <= g_few_rows_max && m <= 128 && k % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 15) == 0;
}

}  // namespace

MIR_EXPORT int mir_set_option(const char* name, int value) {
  for (const Option& option : g_options)
    if (strcmp(option.name, name) == 0) { *option.value = value; return MIR_OK; }
  mir_set_error("unknown option %s", name);
  return MIR_BAD_ARGUMENT;
}

MIR_EXPORT int mir_get_option(const char* name) {
  for (const Option& option : g_options)
    if (strcmp(option.name, name) == 0) return *option.value;
  return -1;
}

// out = (out if accumulate) + x . w^T (+ bias); x [m, k] and w [n, k] bfloat16, out bfloat16 or float32 (only float32
// accumulates), bias of out's dtype.  sumsq / sumsq_tiles / eps: x is a folded norm's weighted rows, each token's
// results are scaled (store epilogue of the streaming kernel only; MIR_CANNOT_FOLD if this product cannot).
// sumsq_out / next_weight / weighted_out: an accumulating few-rows product also leaves what the norm that follows
// needs; *wrote_stats says whether it did.
MIR_EXPORT int mir_linear_bf16(const void* x, int ldx, const void* w, const void* bias, void* out, int ldo, int out_f32,
                               int accumulate, int m, int n, int k, const float* sumsq, int sumsq_tiles, float eps,
                               float* sumsq_out, const float* next_weight, void* weighted_out, int ld_weighted,
                               void* workspace, size_t workspace_bytes, cudaStream_t stream, int* wrote_stats) {
  if (wrote_stats) *wrote_stats = 0;
  if (accumulate && !out_f32) {
    mir_set_error("linear: only a float32 output accumulates");
    return MIR_BAD_ARGUMENT;
  }
  const int mode = out_f32 ? (accumulate ? ACCUM : F32) : STORE;
  const bool few = few_rows_ok(x, ldx, m, k) && ((g_few_rows_modes >> mode) & 1);
  if (sumsq != nullptr && !(few && mode == STORE && m <= g_folded_norm_max_rows)) return MIR_CANNOT_FOLD;
  if (few) {
    const bool stats = mode == ACCUM && sumsq_out != nullptr && next_weight != nullptr && weighted_out != nullptr &&
                       m <= g_folded_norm_max_rows;
    const int status = mir_gemm_tc_stream_bf16(mode, x, ldx, w, bias, out, ldo, m, n, k, 0, sumsq, sumsq_tiles, eps,
                                               stats ? sumsq_out : nullptr, stats ? next_weight : nullptr,
                                               stats ? weighted_out : nullptr, stats ? ld_weighted : 0, stream);
    if (status == MIR_OK && wrote_stats) *wrote_stats = stats ? 1 : 0;
    return status;
  }
  return mir_gemm_bf16_lt(x, ldx, w, k, bias, out, ldo, out_f32, m, n, k, accumulate ? 1.0f : 0.0f, workspace,
                          workspace_bytes, stream);
}

// out[m, inter] = silu(x w_gate^T) * (x w_up^T) with w_gate_up = [w_gate; w_up] of shape [2 inter, k]; out is
// contiguous bfloat16.  sumsq...: x is a folded norm's weighted rows (MIR_CANNOT_FOLD if the rows are too many).
// gate_up_scratch [m, 2 inter] bfloat16 is used by the library path only (33 to tensor_core_min_rows - 1 rows).
MIR_EXPORT int mir_gate_up_silu_bf16(const void* x, int ldx, const void* w_gate_up, void* out, int m, int inter, int k,
                                     const float* sumsq, int sumsq_tiles, float eps, void* gate_up_scratch,
                                     void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  const bool few = few_rows_ok(x, ldx, m, k) && ((g_few_rows_modes >> SWIGLU) & 1);
  if (sumsq != nullptr && !(few && m <= g_folded_norm_max_rows)) return MIR_CANNOT_FOLD;
  if (few)
    return mir_gemm_tc_stream_bf16(SWIGLU, x, ldx, w_gate_up, nullptr, out, inter, m, inter, k, inter, sumsq, sumsq_tiles,
                                   eps, nullptr, nullptr, nullptr, 0, stream);
  if (m >= g_tensor_core_min_rows && k % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 15) == 0)
    return mir_gemm_tc_bf16(SWIGLU, x, ldx, w_gate_up, nullptr, out, inter, m, inter, k, inter, stream);
  if (gate_up_scratch == nullptr) {
    mir_set_error("gate_up_silu: %d rows run the library product, which needs scratch for [rows, 2 x %d]", m, inter);
    return MIR_BAD_ARGUMENT;
  }
  int status = mir_gemm_bf16_lt(x, ldx, w_gate_up, k, nullptr, gate_up_scratch, 2 * inter, 0, m, 2 * inter, k, 0.0f,
                                workspace, workspace_bytes, stream);
  if (status != MIR_OK) return status;
  return mir_silu_mul(1, gate_up_scratch, out, m, inter, stream);
}
