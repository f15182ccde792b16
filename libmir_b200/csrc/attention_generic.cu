// Paged grouped-query softmax attention, one code path for portions of prompts and for decoded
// tokens, any head size that is a multiple of 8 up to 256, any number of heads and groups,
// optional sliding window, float or bf16 storage.  One warp per (token, query head).
//
// This is the reference kernel of the engine: the 32-bit path always runs it, and the bf16 path
// runs it for the sizes its faster kernels refuse.  The order in which a query's keys are reduced
// depends only on the query's own position and window (32 keys at a time from the first visible
// key), never on how the step was cut or what else is in the batch, so a position's output is
// bit-identical under every work split.
//
// Replaces libmir's paged_attention_bf16.cu:14-93, paged_attention_batch_bf16.cu:14-102 and
// paged_prefill_attention_batch_bf16.cu:14-124: score = (q . k) * scale, running maximum and
// denominator, all in 32-bit; key j is visible to the query at position p iff j <= p and
// (window == 0 or j > p - window).
#include <cfloat>
#include "common.cuh"

using namespace mir;

constexpr int kMaxHeadDim = 256;
constexpr int kWarpsPerBlock = 4;

template <typename T>
__global__ void paged_attention_generic_kernel(
    const T* __restrict__ q, size_t q_token_stride, T* __restrict__ out, const T* __restrict__ k_pages,
    const T* __restrict__ v_pages, const int* __restrict__ block_table, int table_width,
    const int* __restrict__ row_of_token, const int* __restrict__ positions, int page_size, int heads, int kv_heads,
    int head_dim, float scale, int window) {
  __shared__ float q_shared[kWarpsPerBlock][kMaxHeadDim];
  const int lane = threadIdx.x;
  const int warp = threadIdx.y;
  const int head = blockIdx.y * kWarpsPerBlock + warp;
  const int token = blockIdx.x;
  if (head >= heads) return;
  const int row = row_of_token[token];
  const int position = positions[token];
  const int kv_head = head / (heads / kv_heads);
  const int* table = block_table + (size_t)row * table_width;
  const int first_key = (window > 0 && position + 1 > window) ? position + 1 - window : 0;

  const T* q_row = q + (size_t)token * q_token_stride + (size_t)head * head_dim;
  for (int d = lane; d < head_dim; d += 32) q_shared[warp][d] = to_float(q_row[d]);
  __syncwarp();

  float acc[kMaxHeadDim / 32];
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = 0.0f;
  float running_max = -FLT_MAX;
  float denominator = 0.0f;

  for (int base = first_key; base <= position; base += 32) {
    const int key = base + lane;
    const bool valid = key <= position;
    float score = -FLT_MAX;
    size_t key_offset = 0;
    if (valid) {
      const int page = table[key / page_size];
      key_offset = (((size_t)page * page_size + key % page_size) * kv_heads + kv_head) * head_dim;
      const T* k_row = k_pages + key_offset;
      float dot = 0.0f;
      for (int d = 0; d < head_dim; d += 8) {
        float k8[8];
        load8(k_row + d, k8);
#pragma unroll
        for (int i = 0; i < 8; ++i) dot = fmaf(q_shared[warp][d + i], k8[i], dot);
      }
      score = dot * scale;
    }
    const float next_max = fmaxf(running_max, warp_max(score));
    const float correction = expf(running_max - next_max);
    const float weight = valid ? expf(score - next_max) : 0.0f;
    denominator = denominator * correction + warp_sum(weight);
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] *= correction;
    const int keys_here = min(32, position - base + 1);
    for (int j = 0; j < keys_here; ++j) {
      const float w = __shfl_sync(0xffffffffu, weight, j);
      const size_t offset = __shfl_sync(0xffffffffu, key_offset, j);
      const T* v_row = v_pages + offset;
#pragma unroll
      for (int i = 0; i < kMaxHeadDim / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) acc[i] = fmaf(w, to_float(v_row[d]), acc[i]);
      }
    }
    running_max = next_max;
  }

  T* out_row = out + ((size_t)token * heads + head) * head_dim;
  const float inverse = denominator > 0.0f ? 1.0f / denominator : 0.0f;   // a padded row has no keys
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < head_dim) out_row[d] = from_float<T>(acc[i] * inverse);
  }
}

// q: first query element of token 0; q_token_stride in elements (the packed QKV row width).
MIR_EXPORT int mir_paged_attention_generic(int bf16, const void* q, long long q_token_stride, void* out,
                                           const void* k_pages, const void* v_pages, const int* block_table,
                                           int table_width, const int* row_of_token, const int* positions, int tokens,
                                           int page_size, int heads, int kv_heads, int head_dim, float scale,
                                           int window, cudaStream_t stream) {
  if (tokens == 0) return MIR_OK;
  if (tokens < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || page_size <= 0 || table_width <= 0 ||
      window < 0) {
    mir_set_error("paged_attention: bad sizes (tokens %d, heads %d, kv heads %d, page %d, table width %d)", tokens,
                  heads, kv_heads, page_size, table_width);
    return MIR_BAD_ARGUMENT;
  }
  if (head_dim <= 0 || head_dim > kMaxHeadDim || head_dim % 8) {
    mir_set_error("paged_attention: head_dim %d is not a multiple of 8 in [8, %d]", head_dim, kMaxHeadDim);
    return MIR_BAD_ARGUMENT;
  }
  const dim3 grid(tokens, (heads + kWarpsPerBlock - 1) / kWarpsPerBlock);
  const dim3 block(32, kWarpsPerBlock);
  if (bf16)
    paged_attention_generic_kernel<<<grid, block, 0, stream>>>(
        (const __nv_bfloat16*)q, (size_t)q_token_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_pages,
        (const __nv_bfloat16*)v_pages, block_table, table_width, row_of_token, positions, page_size, heads, kv_heads,
        head_dim, scale, window);
  else
    paged_attention_generic_kernel<<<grid, block, 0, stream>>>(
        (const float*)q, (size_t)q_token_stride, (float*)out, (const float*)k_pages, (const float*)v_pages,
        block_table, table_width, row_of_token, positions, page_size, heads, kv_heads, head_dim, scale, window);
  return mir_check_launch("paged_attention_generic");
}
