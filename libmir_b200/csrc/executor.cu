// The layer executor: one call from the host runs a run of consecutive decoder layers of the built-in kind
// (RMSNorm -> softmax attention over the paged cache with rotary positions -> residual -> RMSNorm -> SwiGLU ->
// residual) for the packed rows of a step, issuing every launch from native code.
//
// The parts of such a layer can also be run one by one from Python (libmir_b200/parts), which is how parts of other
// kinds run and how each part is tested alone; this file is the same sequence of launches without a Python
// interpreter between them: about a dozen launches per layer at a few microseconds each instead of a dozen
// microseconds each, which is what bounds every step that is not a replay of a captured graph.  libmir's host side
// is native as well (cuda/src/backend/dense/feed_forward.rs:81-150, cuda/src/backend/model/session/prefill/packed.rs:23-89).
//
// What it decides itself, like the Python parts do:
//   * an RMSNorm between two few-rows products is folded into them (the product before it leaves sums of squares
//     and weighted rows, the product after it scales its results) when the step has few enough rows;
//   * attention: bfloat16 with head_dim 64 or 128 runs the single-token rows (packed first) on the split decode
//     kernel and the portions on the tcgen05 or mma.sync kernel; everything else runs the reference kernel.
// Compiled into both libraries: without MIR_WITH_BF16 it runs the float32 engine only.
#include <algorithm>
#include "common.cuh"
#include "launchers.h"

extern "C" {

struct MirNormDesc {
  const float* weight;           // null: the layer has no such norm (the residual would have to be cast: not handled here)
  float eps;
  int size;
};

struct MirLayerDesc {
  MirNormDesc mixer_norm;
  // attention
  const void* w_qkv;             // [(heads + 2 kv_heads) head_dim, hidden]
  const void* b_qkv;             // engine dtype, or null
  const void* w_o;               // [hidden, heads head_dim]
  const void* b_o;               // engine dtype, or null
  const float* q_norm;           // [head_dim] or null
  const float* k_norm;
  const float* inv_freq;         // [rotary_dim / 2] or null
  int heads, kv_heads, head_dim, rotary_dim, window, group, writes_cache, page_size;
  float scale, qk_eps;
  void* k_pages;
  void* v_pages;
  long long cache_rows;
  // feed-forward (w_gate_up null: the layer has none)
  MirNormDesc ff_norm;
  const void* w_gate_up;         // [2 inter, hidden]
  const void* w_down;            // [hidden, inter]
  int inter;
  int pad;
};

struct MirGroupDesc {
  const int* block_table;        // [rows, table_width]
  const int* slot_mapping;       // [tokens]
  int table_width;
  int pad;
};

struct MirStepDesc {
  int bf16;                      // engine dtype: 1 bfloat16, 0 float32
  int tokens, rows, singles, single_context, max_context, decode_only, hidden;
  const int* positions;
  const int* row_of_token;
  const int* query_starts;
  const int* context_lens;
  const MirGroupDesc* groups;
  int n_groups;
  int fuse_norm;                 // fold RMSNorms into the few-rows products around them where possible
  float* residual;               // [tokens, hidden], 32-bit
  // scratch, sized by the host for the largest layer of the run
  void* normed;                  // [tokens, hidden] engine dtype
  void* qkv;                     // [tokens, max (heads + 2 kv_heads) head_dim]
  void* mixed;                   // [tokens, max heads head_dim]
  void* hidden_act;              // [tokens, max inter]
  void* gate_up;                 // [tokens, 2 max inter] or null (then rows that need it are refused)
  float* sumsq[2];               // [ceil(hidden / 16), 32] each
  void* weighted[2];             // [tokens, hidden] bfloat16 each
  float* attention_scratch;
  long long attention_scratch_floats;
  void* workspace;               // for the library products
  size_t workspace_bytes;
  int prefill_tensor_cores;      // 0 never the tcgen05 prompt kernel
  int prefill_tensor_core_min_portion;
  const float* norm_after;       // weight of the norm that the block after this run starts with, or null
  cudaStream_t stream;
};

}  // extern "C"

namespace {

#define MIR_TRY(call)                    \
  do {                                   \
    const int status_ = (call);          \
    if (status_ != MIR_OK) return status_; \
  } while (0)

struct Run {
  const MirStepDesc& step;
  const float* stats_for = nullptr;   // the norm weight that sumsq[current] / weighted[current] were prepared for
  int current = 0;

  explicit Run(const MirStepDesc& s) : step(s) {}

  bool may_fold() const {
#ifdef MIR_WITH_BF16
    return step.fuse_norm && step.bf16 && step.tokens <= std::min(mir_get_option("folded_norm_max_rows"),
                                                                  mir_get_option("few_rows_max"));
#else
    return false;
#endif
  }

  // out = x . w^T (+ bias) in the engine dtype; x is the norm `norm` of the residual, folded if its statistics are
  // at hand and the product can take them, else computed by the norm kernel first.
  int project_normed(const MirNormDesc& norm, const void* w, const void* bias, void* out, int n) {
    const int m = step.tokens, k = step.hidden;
#ifdef MIR_WITH_BF16
    if (step.bf16 && stats_for != nullptr && stats_for == norm.weight) {
      const int status = mir_linear_bf16(step.weighted[current], k, w, bias, out, n, 0, 0, m, n, k, step.sumsq[current],
                                         (k + 15) / 16, norm.eps, nullptr, nullptr, nullptr, 0, step.workspace,
                                         step.workspace_bytes, step.stream, nullptr);
      if (status != MIR_CANNOT_FOLD) return status;
    }
#endif
    MIR_TRY(mir_rms_norm(step.bf16, step.residual, norm.weight, step.normed, nullptr, m, k, norm.eps, step.stream));
#ifdef MIR_WITH_BF16
    if (step.bf16)
      return mir_linear_bf16(step.normed, k, w, bias, out, n, 0, 0, m, n, k, nullptr, 0, 0.0f, nullptr, nullptr, nullptr,
                             0, step.workspace, step.workspace_bytes, step.stream, nullptr);
#endif
    return mir_gemm_f32((const float*)step.normed, k, (const float*)w, k, (const float*)bias, (float*)out, n, m, n, k,
                        0.0f, step.stream);
  }

  // residual += x . w^T (+ bias); prepares the norm `upcoming` (may be null) for folding if the product can.
  int accumulate(const void* x, int k, const void* w, const void* bias, const MirNormDesc* upcoming) {
    const int m = step.tokens, n = step.hidden;
    stats_for = nullptr;
#ifdef MIR_WITH_BF16
    if (step.bf16) {
      if (bias != nullptr) MIR_TRY(mir_add_bias(1, step.residual, bias, m, n, step.stream));   // a bfloat16 bias
      const bool prepare = may_fold() && upcoming != nullptr && upcoming->weight != nullptr && upcoming->size == n;
      const int next = current ^ 1;
      int wrote = 0;
      MIR_TRY(mir_linear_bf16(x, k, w, nullptr, step.residual, n, 1, 1, m, n, k, nullptr, 0, 0.0f,
                              prepare ? step.sumsq[next] : nullptr, prepare ? upcoming->weight : nullptr,
                              prepare ? step.weighted[next] : nullptr, n, step.workspace, step.workspace_bytes,
                              step.stream, &wrote));
      if (wrote) {
        current = next;
        stats_for = upcoming->weight;
      }
      return MIR_OK;
    }
#endif
    return mir_gemm_f32((const float*)x, k, (const float*)w, k, (const float*)bias, step.residual, n, m, n, k, 1.0f,
                        step.stream);
  }

  int attend(const MirLayerDesc& layer) {
    const MirGroupDesc& group = step.groups[layer.group];
    const int width = (layer.heads + 2 * layer.kv_heads) * layer.head_dim;
#ifdef MIR_WITH_BF16
    if (step.bf16 && (layer.head_dim == 64 || layer.head_dim == 128)) {
      // the single-token rows come first in the batch: they run as decoded tokens (keys split over CTAs, the heads
      // of a KV group in one CTA), the prompt portions after them as tiles of queries
      const int singles = step.decode_only ? step.rows : step.singles;
      if (singles > 0) {
        const int longest = step.decode_only ? step.max_context : step.single_context;
        const int partition = mir_decode_partition_keys(singles, layer.heads, layer.kv_heads, layer.head_dim,
                                                        layer.page_size, longest);
        const int count = std::max(1, (longest + partition - 1) / partition);
        MIR_TRY(mir_decode_attention_paged_bf16(step.qkv, width, step.mixed, layer.k_pages, layer.v_pages,
                                                layer.cache_rows, group.block_table, group.table_width, step.positions,
                                                singles, layer.page_size, layer.heads, layer.kv_heads, layer.head_dim,
                                                layer.scale, layer.window, partition, count, step.attention_scratch,
                                                step.attention_scratch_floats, step.stream));
      }
      if (singles < step.rows) {
        const int rows = step.rows - singles, portion_tokens = step.tokens - singles;
        const int* table = group.block_table + (size_t)singles * group.table_width;
        const bool tensor_cores = step.prefill_tensor_cores && layer.scale > 0.0f &&
                                  portion_tokens >= step.prefill_tensor_core_min_portion * rows &&
                                  mir_prefill_attention_tc_takes(layer.head_dim, layer.page_size);
        if (tensor_cores)
          return mir_prefill_attention_tc_bf16(step.qkv, width, step.mixed, layer.k_pages, layer.v_pages, layer.cache_rows,
                                               table, group.table_width, step.query_starts + singles,
                                               step.context_lens + singles, rows, step.tokens, layer.page_size,
                                               layer.heads, layer.kv_heads, layer.head_dim, layer.scale, layer.window,
                                               step.stream);
        return mir_prefill_attention_bf16(step.qkv, width, step.mixed, layer.k_pages, layer.v_pages, table,
                                          group.table_width, step.query_starts + singles, step.context_lens + singles,
                                          rows, step.tokens, layer.page_size, layer.heads, layer.kv_heads, layer.head_dim,
                                          layer.scale, layer.window, step.stream);
      }
      return MIR_OK;
    }
#endif
    return mir_paged_attention_generic(step.bf16, step.qkv, width, step.mixed, layer.k_pages, layer.v_pages,
                                       group.block_table, group.table_width, step.row_of_token, step.positions,
                                       step.tokens, layer.page_size, layer.heads, layer.kv_heads, layer.head_dim,
                                       layer.scale, layer.window, step.stream);
  }

  int feed_forward(const MirLayerDesc& layer, const MirNormDesc* upcoming) {
    const int m = step.tokens, k = step.hidden, inter = layer.inter;
#ifdef MIR_WITH_BF16
    if (step.bf16) {
      int status = MIR_CANNOT_FOLD;
      if (stats_for != nullptr && stats_for == layer.ff_norm.weight)
        status = mir_gate_up_silu_bf16(step.weighted[current], k, layer.w_gate_up, step.hidden_act, m, inter, k,
                                       step.sumsq[current], (k + 15) / 16, layer.ff_norm.eps, step.gate_up,
                                       step.workspace, step.workspace_bytes, step.stream);
      if (status == MIR_CANNOT_FOLD) {
        MIR_TRY(mir_rms_norm(1, step.residual, layer.ff_norm.weight, step.normed, nullptr, m, k, layer.ff_norm.eps,
                             step.stream));
        status = mir_gate_up_silu_bf16(step.normed, k, layer.w_gate_up, step.hidden_act, m, inter, k, nullptr, 0, 0.0f,
                                       step.gate_up, step.workspace, step.workspace_bytes, step.stream);
      }
      MIR_TRY(status);
      return accumulate(step.hidden_act, inter, layer.w_down, nullptr, upcoming);
    }
#endif
    if (step.gate_up == nullptr) {
      mir_set_error("executor: the float32 feed-forward needs scratch for [rows, 2 x intermediate]");
      return MIR_BAD_ARGUMENT;
    }
    MIR_TRY(mir_rms_norm(0, step.residual, layer.ff_norm.weight, step.normed, nullptr, m, k, layer.ff_norm.eps, step.stream));
    MIR_TRY(mir_gemm_f32((const float*)step.normed, k, (const float*)layer.w_gate_up, k, nullptr, (float*)step.gate_up,
                         2 * inter, m, 2 * inter, k, 0.0f, step.stream));
    MIR_TRY(mir_silu_mul(0, step.gate_up, step.hidden_act, m, inter, step.stream));
    return accumulate(step.hidden_act, inter, layer.w_down, nullptr, upcoming);
  }
};

}  // namespace

// Size of the descriptors, so that the host can check that its mirror of them matches this build.
MIR_EXPORT int mir_executor_layout(int* layer_bytes, int* step_bytes, int* group_bytes) {
  *layer_bytes = (int)sizeof(MirLayerDesc);
  *step_bytes = (int)sizeof(MirStepDesc);
  *group_bytes = (int)sizeof(MirGroupDesc);
  return MIR_OK;
}

// Runs layers[0 .. count) on the step's packed rows: every layer adds its two branches into step->residual.
// stats_in: the weight of the norm for which sumsq[0] / weighted[0] already hold statistics of the residual (null:
// none).  *stats_out receives the weight of the norm that the last product prepared into sumsq[*stats_index] /
// weighted[*stats_index] (null: none), so that a caller that runs more layers afterwards can go on folding.
MIR_EXPORT int mir_run_layers(const MirLayerDesc* layers, int count, const MirStepDesc* step, const float* stats_in,
                              const float** stats_out, int* stats_index) {
  if (step == nullptr || layers == nullptr || count < 0 || step->tokens < 0 || step->hidden <= 0) {
    mir_set_error("executor: bad arguments");
    return MIR_BAD_ARGUMENT;
  }
#ifndef MIR_WITH_BF16
  if (step->bf16) {
    mir_set_error("executor: this library runs the float32 engine only");
    return MIR_BAD_ARGUMENT;
  }
#endif
  if (step->tokens == 0) return MIR_OK;
  Run run(*step);
  run.stats_for = stats_in;
  for (int index = 0; index < count; ++index) {
    const MirLayerDesc& layer = layers[index];
    if (layer.mixer_norm.weight == nullptr || layer.group < 0 || layer.group >= step->n_groups ||
        (layer.w_gate_up != nullptr && layer.ff_norm.weight == nullptr)) {
      mir_set_error("executor: layer %d is not of the kind this executor runs", index);
      return MIR_BAD_ARGUMENT;
    }
    const MirGroupDesc& group = step->groups[layer.group];
    const int width = (layer.heads + 2 * layer.kv_heads) * layer.head_dim;
    // the norm that follows each branch: the feed-forward's, then the next layer's first (or the caller's)
    MirNormDesc after_layer = {step->norm_after, 0.0f, step->hidden};
    const MirNormDesc* next_first = index + 1 < count ? &layers[index + 1].mixer_norm : &after_layer;
    const bool has_ff = layer.w_gate_up != nullptr;
    MIR_TRY(run.project_normed(layer.mixer_norm, layer.w_qkv, layer.b_qkv, step->qkv, width));
    MIR_TRY(mir_qk_rope_store(step->bf16, step->qkv, step->positions, group.slot_mapping, layer.inv_freq, layer.q_norm,
                              layer.k_norm, layer.k_pages, layer.v_pages, step->tokens, layer.heads, layer.kv_heads,
                              layer.head_dim, layer.rotary_dim, layer.qk_eps, layer.writes_cache ? 1 : 0, step->stream));
    MIR_TRY(run.attend(layer));
    MIR_TRY(run.accumulate(step->mixed, layer.heads * layer.head_dim, layer.w_o, layer.b_o,
                           has_ff ? &layer.ff_norm : next_first));
    if (has_ff) MIR_TRY(run.feed_forward(layer, next_first));
  }
  if (stats_out) *stats_out = run.stats_for;
  if (stats_index) *stats_index = run.current;
  return MIR_OK;
}
