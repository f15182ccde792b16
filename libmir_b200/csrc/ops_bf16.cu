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
#include <algorithm>
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
// Whether single decoded tokens run the tcgen05 attention kernel where it takes the sizes (else the mma.sync kernel).
int g_decode_tensor_cores = 1;
// Keys one CTA of the mma.sync decode kernel takes (a multiple of 64, at most 512).  Measured (attention and merge,
// us, 256 against 512 keys): batch 1 at 2,120 keys 7.8 / 15.9, at 32,768 keys 37 / 45; batch 8 at 2,120 keys 20.0 /
// 20.7, at 8,192 keys 54 / 84; batch 32 at 2,120 keys 56 / 66; batch 64 102 / 106.
int g_decode_partition_keys = 256;
// Keys one CTA of the tcgen05 decode kernel takes: 0 lets mir_decode_partition_keys choose, else this many.
int g_decode_tc_partition_keys = 0;

enum Mode : int { STORE = 0, ACCUM = 1, F32 = 2, SWIGLU = 3 };

struct Option { const char* name; int* value; };
Option g_options[] = {{"few_rows_max", &g_few_rows_max}, {"folded_norm_max_rows", &g_folded_norm_max_rows},
                      {"tensor_core_min_rows", &g_tensor_core_min_rows}, {"few_rows_modes", &g_few_rows_modes},
                      {"decode_tensor_cores", &g_decode_tensor_cores}, {"decode_partition_keys", &g_decode_partition_keys},
                      {"decode_tc_partition_keys", &g_decode_tc_partition_keys}};

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

// How many keys one CTA of split decode attention takes for `rows` single tokens whose longest context (or the
// width of the block tables of a captured step) is `longest` keys; the number of partitions is ceil(longest / that).
// The tcgen05 kernel keeps three CTAs on an SM, and a CTA costs about 5 us to start and end and 2.5 us per tile of
// 128 keys, so the choice is the partition with the fewest waves x (5 + 2.5 tiles): measured (attention and merge,
// us, partitions of 128 / 256 / 512 / 1,024 keys) batch 1 at 2,112 keys 7.8 / 9.2 / 12.6 / 19.2; batch 8: 23.1 / 20.0 /
// 19.1 / 23.3; batch 32: 73.5 / 56.3 / 52.5 / 55.6; batch 64: 142 / 106 / 96.1 / 95.9; batch 8 at 8,192 keys 76.3 / 54.0 /
// 51.2 / 54.7; batch 1 at 32,768 keys 49.2 / 33.8 / 31.2 / 28.1; batch 8 at 32,768 keys 262 / 197 / 174 / 169.
MIR_EXPORT int mir_decode_partition_keys(int rows, int heads, int kv_heads, int head_dim, int page_size, int longest) {
  if (!g_decode_tensor_cores || !mir_decode_attention_tc_takes(head_dim, page_size, 128)) return g_decode_partition_keys;
  if (g_decode_tc_partition_keys > 0) return g_decode_tc_partition_keys;
  const long long group = kv_heads > 0 ? (heads + kv_heads - 1) / kv_heads : 1;
  const long long units = (long long)std::max(rows, 1) * std::max(kv_heads, 1) * ((group + 15) / 16);
  const long long resident = 3ll * mir_sm_count();
  int best = 128;
  double best_cost = 0.0;
  for (int partition = 128; partition <= 1024; partition *= 2) {
    const long long full = std::max(longest, 1) / partition, rest = std::max(longest, 1) % partition;
    // CTAs that take a whole partition; the one with the rest of the keys is short and fills a gap
    const long long ctas = units * (full + (rest * 2 > partition ? 1 : 0));
    const long long waves = std::max(1ll, (ctas + resident - 1) / resident);
    const double cost = (double)waves * (5.0 + 2.5 * std::min(partition, std::max(longest, 1) + 127) / 128.0);
    if (partition == 128 || cost < best_cost) { best = partition; best_cost = cost; }
  }
  return best;
}

// Attention of single decoded tokens over the pages: the tcgen05 kernel where it takes the sizes, else the mma.sync
// kernel.  Arguments as mir_decode_attention_bf16, and how many token rows the cache tensors have.
MIR_EXPORT int mir_decode_attention_paged_bf16(const void* q, long long q_stride, void* out, const void* k_pages,
                                               const void* v_pages, long long cache_rows, const int* block_table,
                                               int table_width, const int* positions, int rows, int page_size,
                                               int heads, int kv_heads, int head_dim, float scale, int window,
                                               int partition, int num_partitions, float* scratch,
                                               long long scratch_floats, cudaStream_t stream) {
  if (g_decode_tensor_cores && cache_rows > 0 && mir_decode_attention_tc_takes(head_dim, page_size, partition))
    return mir_decode_attention_tc_bf16(q, q_stride, out, k_pages, v_pages, cache_rows, block_table, table_width,
                                        positions, rows, page_size, heads, kv_heads, head_dim, scale, window, partition,
                                        num_partitions, scratch, scratch_floats, stream);
  return mir_decode_attention_bf16(q, q_stride, out, k_pages, v_pages, block_table, table_width, positions, rows,
                                   page_size, heads, kv_heads, head_dim, scale, window, partition, num_partitions,
                                   scratch, scratch_floats, stream);
}

// What a caller has to provide for the attention of `rows` single tokens whose longest context (or block-table width)
// is `longest` keys: keys per partition, partitions, floats of scratch, as mir_decode_attention_paged_bf16 will use them.
MIR_EXPORT int mir_decode_attention_plan(int rows, int heads, int kv_heads, int head_dim, int page_size, int longest,
                                         int* partition, int* partitions, long long* scratch_floats) {
  const int keys = mir_decode_partition_keys(rows, heads, kv_heads, head_dim, page_size, longest);
  const int count = std::max(1, (std::max(longest, 1) + keys - 1) / keys);
  *partition = keys;
  *partitions = count;
  *scratch_floats = mir_decode_attention_scratch_floats(rows, heads, head_dim, count);
  return MIR_OK;
}

// The output head: float32 logits out[m, n] = x . w^T.  Up to few_rows_max rows run the weight-streaming kernel, which
// then also leaves each row's candidates for its largest logit (see mir_gemm_tc_stream_head_bf16) if best_value is
// given: *wrote_best says whether it did (a library product leaves none).
MIR_EXPORT int mir_head_logits_bf16(const void* x, int ldx, const void* w, void* out, int ldo, int m, int n, int k,
                                    float* best_value, int* best_index, int best_stride, void* workspace,
                                    size_t workspace_bytes, cudaStream_t stream, int* wrote_best) {
  if (wrote_best) *wrote_best = 0;
  if (best_value != nullptr && best_index != nullptr && few_rows_ok(x, ldx, m, k) && (g_few_rows_modes & (1 << F32)) &&
      best_stride >= mir_gemm_tc_stream_head_candidates(n) && ldo >= n) {
    const int status = mir_gemm_tc_stream_head_bf16(x, ldx, w, out, ldo, m, n, k, best_value, best_index, best_stride,
                                                    stream);
    if (status == MIR_OK && wrote_best) *wrote_best = 1;
    return status;
  }
  return mir_linear_bf16(x, ldx, w, nullptr, out, ldo, 1, 0, m, n, k, nullptr, 0, 0.0f, nullptr, nullptr, nullptr, 0,
                         workspace, workspace_bytes, stream, nullptr);
}
