// Per-head q/k RMSNorm, rotary position encoding and the write of K and V into cache pages, in one
// kernel over the packed [T, (Hq + 2 Hkv) D] output of the QKV projection.
//
// Replaces libmir's qkv_postprocess_bf16.cu:71-183 and kv_cache_bf16.cu:74-97 (two launches and a
// round trip of k and v through memory).  Differences on purpose: the normalised value is not
// rounded to bf16 before the rotation, and the angle table is passed in (so that llama3 scaling,
// which libmir's CUDA loader ignores, is the same code path as the plain table).
//
// q is rotated in place; k (rotated) and v go straight to
//   pages[(slot_mapping[t]) * Hkv + h][:]  with slot = page * page_size + position % page_size,
// and a negative slot means "do not write" (a padded row of a captured decode batch).
#include "common.cuh"

using namespace mir;

template <typename T>
__global__ void qk_rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ slot_mapping, const float* __restrict__ inv_freq,
                                     const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                                     T* __restrict__ k_pages, T* __restrict__ v_pages, int heads, int kv_heads,
                                     int head_dim, int rotary_dim, float eps, int write_kv) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int token = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int warps = gridDim.y * (blockDim.x >> 5);
  const int units = heads + 2 * kv_heads;
  const size_t row_width = (size_t)units * head_dim;
  T* row = qkv + (size_t)token * row_width;
  const float position = (float)positions[token];
  const int slot = slot_mapping ? slot_mapping[token] : -1;
  const int half = rotary_dim / 2;

  for (int unit = warp; unit < units; unit += warps) {
    T* src = row + (size_t)unit * head_dim;
    if (unit >= heads + kv_heads) {                 // a value head: copy to its page
      if (!write_kv || slot < 0) continue;
      T* dst = v_pages + ((size_t)slot * kv_heads + (unit - heads - kv_heads)) * head_dim;
      for (int d = lane; d < head_dim; d += 32) dst[d] = src[d];
      continue;
    }
    const bool is_query = unit < heads;
    if (!is_query && (!write_kv || slot < 0)) continue;
    const float* norm = is_query ? q_norm : k_norm;
    float inverse = 1.0f;
    if (norm) {
      float sum = 0.0f;
      for (int d = lane; d < head_dim; d += 32) {
        const float v = to_float(src[d]);
        sum = fmaf(v, v, sum);
      }
      sum = warp_sum(sum);
      inverse = rsqrtf(sum / (float)head_dim + eps);
    }
    T* dst = is_query ? src : k_pages + ((size_t)slot * kv_heads + (unit - heads)) * head_dim;
    for (int pair = lane; pair < half; pair += 32) {
      float first = to_float(src[pair]);
      float second = to_float(src[pair + half]);
      if (norm) {
        first = first * inverse * norm[pair];
        second = second * inverse * norm[pair + half];
      }
      float sine, cosine;
      sincosf(position * inv_freq[pair], &sine, &cosine);
      dst[pair] = from_float<T>(first * cosine - second * sine);
      dst[pair + half] = from_float<T>(first * sine + second * cosine);
    }
    for (int d = rotary_dim + lane; d < head_dim; d += 32) {
      float v = to_float(src[d]);
      if (norm) v = v * inverse * norm[d];
      dst[d] = from_float<T>(v);
    }
  }
}

MIR_EXPORT int mir_qk_rope_store(int bf16, void* qkv, const int* positions, const int* slot_mapping,
                                 const float* inv_freq, const float* q_norm, const float* k_norm, void* k_pages,
                                 void* v_pages, int tokens, int heads, int kv_heads, int head_dim, int rotary_dim,
                                 float eps, int write_kv, cudaStream_t stream) {
  if (tokens == 0) return MIR_OK;
  if (tokens < 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0 || rotary_dim < 0 || rotary_dim > head_dim ||
      (rotary_dim & 1)) {
    mir_set_error("qk_rope_store: bad sizes (heads %d, kv heads %d, head_dim %d, rotary_dim %d)", heads, kv_heads,
                  head_dim, rotary_dim);
    return MIR_BAD_ARGUMENT;
  }
  // one warp per head (query, key or value) of a token: 4 warps per CTA, enough CTAs per token to cover them
  const int units = heads + 2 * kv_heads;
  const int threads = 128;
  const dim3 grid(tokens, (units + 3) / 4);
  if (bf16)
    return mir_launch("qk_rope_store", qk_rope_store_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, 0,
                      (__nv_bfloat16*)qkv, positions, slot_mapping, inv_freq, q_norm, k_norm, (__nv_bfloat16*)k_pages,
                      (__nv_bfloat16*)v_pages, heads, kv_heads, head_dim, rotary_dim, eps, write_kv);
  return mir_launch("qk_rope_store", qk_rope_store_kernel<float>, grid, dim3(threads), 0, stream, 0, (float*)qkv,
                    positions, slot_mapping, inv_freq, q_norm, k_norm, (float*)k_pages, (float*)v_pages, heads,
                    kv_heads, head_dim, rotary_dim, eps, write_kv);
}
