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
// write_kv: 0 only the queries are treated (a reader of another entry's cache), 1 keys and values go to their
// pages, 2 keys are normed and rotated in place like the queries and nothing goes to the pages (a position
// encoding of another kind works on them next; a second call with 1 and neither norm nor rotation then stores).
#include "common.cuh"
#include "trace.cuh"

using namespace mir;

// Two consecutive elements as floats, and back.
__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ void store2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store2(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// One CTA per (token, slice of the token's heads): the token's cosines and sines are computed once into shared
// memory, then each warp takes heads (query, key or value) of the slice.  PAIRED: head_dim is even and
// rotary_dim a multiple of 4, so every lane works on two neighbouring elements (4- or 8-byte accesses).
template <typename T, bool PAIRED>
__global__ void qk_rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ slot_mapping, const float* __restrict__ inv_freq,
                                     const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                                     T* __restrict__ k_pages, T* __restrict__ v_pages, int heads, int kv_heads,
                                     int head_dim, int rotary_dim, float eps, int write_kv, int units_per_cta) {
  extern __shared__ float angles[];                 // [half] cosines then [half] sines of this token
  grid_launch_dependents();
  grid_dependency_wait();
  const int token = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int units = heads + 2 * kv_heads;
  const size_t row_width = (size_t)units * head_dim;
  T* row = qkv + (size_t)token * row_width;
  const float position = (float)positions[token];
  const int slot = slot_mapping ? slot_mapping[token] : -1;
  const int half = rotary_dim / 2;
  for (int pair = threadIdx.x; pair < half; pair += blockDim.x)
    sincosf(position * inv_freq[pair], &angles[half + pair], &angles[pair]);
  __syncthreads();
  const int unit_begin = blockIdx.y * units_per_cta, unit_end = min(units, unit_begin + units_per_cta);

  for (int unit = unit_begin + warp; unit < unit_end; unit += warps) {
    T* src = row + (size_t)unit * head_dim;
    if (unit >= heads + kv_heads) {                 // a value head: copy to its page
      if (write_kv != 1 || slot < 0) continue;
      T* dst = v_pages + ((size_t)slot * kv_heads + (unit - heads - kv_heads)) * head_dim;
      if ((head_dim * sizeof(T)) % 16 == 0 && ((uintptr_t)src & 15) == 0 && ((uintptr_t)dst & 15) == 0) {
        const int chunks = head_dim * (int)sizeof(T) / 16;
        for (int c = lane; c < chunks; c += 32) reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
      } else {
        for (int d = lane; d < head_dim; d += 32) dst[d] = src[d];
      }
      continue;
    }
    const bool is_query = unit < heads;
    const bool key_in_place = write_kv == 2;        // normed and rotated keys stay in the packed row
    if (!is_query && !key_in_place && (!write_kv || slot < 0)) continue;
    const float* norm = is_query ? q_norm : k_norm;
    float inverse = 1.0f;
    if (norm) {
      float sum = 0.0f;
      if (PAIRED) {
        for (int d = 2 * lane; d < head_dim; d += 64) {
          const float2 v = load2(src + d);
          sum = fmaf(v.x, v.x, fmaf(v.y, v.y, sum));
        }
      } else {
        for (int d = lane; d < head_dim; d += 32) {
          const float v = to_float(src[d]);
          sum = fmaf(v, v, sum);
        }
      }
      sum = warp_sum(sum);
      inverse = rsqrtf(sum / (float)head_dim + eps);
    }
    T* dst = (is_query || key_in_place) ? src : k_pages + ((size_t)slot * kv_heads + (unit - heads)) * head_dim;
    if (PAIRED) {
      for (int pair = 2 * lane; pair < half; pair += 64) {
        float2 first = load2(src + pair), second = load2(src + pair + half);
        if (norm) {
          first.x *= inverse * norm[pair]; first.y *= inverse * norm[pair + 1];
          second.x *= inverse * norm[pair + half]; second.y *= inverse * norm[pair + half + 1];
        }
        const float c0 = angles[pair], c1 = angles[pair + 1], s0 = angles[half + pair], s1 = angles[half + pair + 1];
        store2(dst + pair, first.x * c0 - second.x * s0, first.y * c1 - second.y * s1);
        store2(dst + pair + half, first.x * s0 + second.x * c0, first.y * s1 + second.y * c1);
      }
      for (int d = rotary_dim + 2 * lane; d < head_dim; d += 64) {
        float2 v = load2(src + d);
        if (norm) { v.x *= inverse * norm[d]; v.y *= inverse * norm[d + 1]; }
        store2(dst + d, v.x, v.y);
      }
    } else {
      for (int pair = lane; pair < half; pair += 32) {
        float first = to_float(src[pair]);
        float second = to_float(src[pair + half]);
        if (norm) {
          first = first * inverse * norm[pair];
          second = second * inverse * norm[pair + half];
        }
        const float cosine = angles[pair], sine = angles[half + pair];
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
}

// time stamps (trace.cuh) of the first and the last CTA of the kernel below: 0 start, 1 the projection is over,
// 2 end; tag 100 / 101
MIR_TRACE_DEFINE(rope)

// bf16, the whole head rotated (rotary_dim == head_dim), half a head a multiple of 8 elements: L = half / 8 lanes
// take one head, each with two 16-byte pieces (elements 8 l .. 8 l + 7 and their partners half a head further),
// so a warp works on 32 / L heads at once and every access is 16 bytes wide.
template <int L>
__global__ void qk_rope_store_wide_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                                          const int* __restrict__ slot_mapping, const float* __restrict__ inv_freq,
                                          const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                                          __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                                          int heads, int kv_heads, float eps, int write_kv, int units_per_cta) {
  constexpr int HALF = 8 * L, DIM = 2 * HALF, GROUPS = 32 / L;
  __shared__ float angles[DIM];                      // [HALF] cosines then [HALF] sines of this token
  grid_launch_dependents();
  MIR_TRACE_BEGIN(rope, (blockIdx.x == 0 && blockIdx.y == 0) || (blockIdx.x == gridDim.x - 1 && blockIdx.y == gridDim.y - 1),
                  100 + (blockIdx.x == 0 && blockIdx.y == 0 ? 0 : 1))
  if (threadIdx.x == 0) MIR_TRACE_POINT(rope, 0);
  const int token = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int group = lane / L, l = lane % L;
  const int units = heads + 2 * kv_heads;
  __nv_bfloat16* row = qkv + (size_t)token * units * DIM;
  const float position = (float)positions[token];
  const int slot = slot_mapping ? slot_mapping[token] : -1;
  // positions and slots are older than the kernel before this one (the projection): the angles are computed
  // while it may still be running, then this kernel waits for its rows
  for (int pair = threadIdx.x; pair < HALF; pair += blockDim.x)
    sincosf(position * inv_freq[pair], &angles[HALF + pair], &angles[pair]);
  grid_dependency_wait();
  __syncthreads();
  if (threadIdx.x == 0) MIR_TRACE_POINT(rope, 1);
  const int unit_begin = blockIdx.y * units_per_cta, unit_end = min(units, unit_begin + units_per_cta);
  for (int base = unit_begin + warp * GROUPS; base < unit_end; base += warps * GROUPS) {
    const int unit = base + group;
    const bool active = unit < unit_end;
    const bool is_query = unit < heads, is_value = unit >= heads + kv_heads;
    const __nv_bfloat16* src = row + (size_t)unit * DIM;
    uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
    if (active) {
      a = *reinterpret_cast<const uint4*>(src + 8 * l);
      b = *reinterpret_cast<const uint4*>(src + HALF + 8 * l);
    }
    const bool in_place = is_query || (write_kv == 2 && !is_value);
    const bool writes = active && (in_place || (write_kv == 1 && slot >= 0));
    __nv_bfloat16* dst = nullptr;
    if (writes)
      dst = in_place ? row + (size_t)unit * DIM
                     : (is_value ? v_pages + ((size_t)slot * kv_heads + (unit - heads - kv_heads)) * DIM
                                 : k_pages + ((size_t)slot * kv_heads + (unit - heads)) * DIM);
    float fa[8], fb[8];
    {
      const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(ha[i]), y = __bfloat1622float2(hb[i]);
        fa[2 * i] = x.x; fa[2 * i + 1] = x.y; fb[2 * i] = y.x; fb[2 * i + 1] = y.y;
      }
    }
    const float* norm = (!active || is_value) ? nullptr : (is_query ? q_norm : k_norm);
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) sum = fmaf(fa[i], fa[i], fmaf(fb[i], fb[i], sum));
#pragma unroll
    for (int o = L / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);   // every lane takes part
    if (norm) {
      const float inverse = rsqrtf(sum / (float)DIM + eps);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        fa[i] *= inverse * norm[8 * l + i];
        fb[i] *= inverse * norm[HALF + 8 * l + i];
      }
    }
    if (!writes) continue;
    if (!is_value) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float cosine = angles[8 * l + i], sine = angles[HALF + 8 * l + i];
        const float first = fa[i], second = fb[i];
        fa[i] = first * cosine - second * sine;
        fb[i] = first * sine + second * cosine;
      }
      __nv_bfloat162* ha = reinterpret_cast<__nv_bfloat162*>(&a);
      __nv_bfloat162* hb = reinterpret_cast<__nv_bfloat162*>(&b);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        ha[i] = __floats2bfloat162_rn(fa[2 * i], fa[2 * i + 1]);
        hb[i] = __floats2bfloat162_rn(fb[2 * i], fb[2 * i + 1]);
      }
    }
    *reinterpret_cast<uint4*>(dst + 8 * l) = a;                // a value head is copied as it is
    *reinterpret_cast<uint4*>(dst + HALF + 8 * l) = b;
  }
  if (threadIdx.x == 0) MIR_TRACE_POINT(rope, 2);
}

template <int L>
int launch_rope_wide(__nv_bfloat16* qkv, const int* positions, const int* slot_mapping, const float* inv_freq,
                     const float* q_norm, const float* k_norm, __nv_bfloat16* k_pages, __nv_bfloat16* v_pages, int tokens,
                     int heads, int kv_heads, float eps, int write_kv, cudaStream_t stream) {
  const int units = heads + 2 * kv_heads;
  const bool many = tokens >= 256;                     // one CTA of 8 warps per token, else CTAs of 4 warps
  const int threads = many ? 256 : 128;
  const int units_per_cta = many ? units : 4 * (32 / L);
  const dim3 grid(tokens, (units + units_per_cta - 1) / units_per_cta);
  return mir_launch_with(mir_pdl_for_streaming(), "qk_rope_store", qk_rope_store_wide_kernel<L>, grid, dim3(threads), 0, stream, 0, qkv, positions,
                    slot_mapping, inv_freq, q_norm, k_norm, k_pages, v_pages, heads, kv_heads, eps, write_kv, units_per_cta);
}

template <typename T>
int launch_rope(T* qkv, const int* positions, const int* slot_mapping, const float* inv_freq, const float* q_norm,
                const float* k_norm, T* k_pages, T* v_pages, int tokens, int heads, int kv_heads, int head_dim,
                int rotary_dim, float eps, int write_kv, cudaStream_t stream) {
  // few tokens: 4 warps per CTA and enough CTAs per token to give every head a warp; many tokens: one CTA of 8
  // warps per token, so that the token's angles are computed once
  const int units = heads + 2 * kv_heads;
  const bool many = tokens >= 256;
  const int threads = many ? 256 : 128;
  const int units_per_cta = many ? units : 4;
  const dim3 grid(tokens, (units + units_per_cta - 1) / units_per_cta);
  const size_t smem = (size_t)rotary_dim * sizeof(float);
  const bool paired = (head_dim % 2 == 0) && (rotary_dim % 4 == 0) && ((uintptr_t)qkv % (2 * sizeof(T)) == 0) &&
                      ((uintptr_t)k_pages % (2 * sizeof(T)) == 0);
  if (paired)
    return mir_launch("qk_rope_store", qk_rope_store_kernel<T, true>, grid, dim3(threads), smem, stream, 0, qkv, positions,
                      slot_mapping, inv_freq, q_norm, k_norm, k_pages, v_pages, heads, kv_heads, head_dim, rotary_dim,
                      eps, write_kv, units_per_cta);
  return mir_launch("qk_rope_store", qk_rope_store_kernel<T, false>, grid, dim3(threads), smem, stream, 0, qkv, positions,
                    slot_mapping, inv_freq, q_norm, k_norm, k_pages, v_pages, heads, kv_heads, head_dim, rotary_dim, eps,
                    write_kv, units_per_cta);
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
  if (rotary_dim > 8192) { mir_set_error("qk_rope_store: rotary_dim %d is too large", rotary_dim); return MIR_BAD_ARGUMENT; }
  if (bf16 && rotary_dim == head_dim && head_dim % 16 == 0 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)k_pages & 15) == 0 &&
      ((uintptr_t)v_pages & 15) == 0) {
    __nv_bfloat16* q = (__nv_bfloat16*)qkv;
    __nv_bfloat16* kp = (__nv_bfloat16*)k_pages;
    __nv_bfloat16* vp = (__nv_bfloat16*)v_pages;
    switch (head_dim / 16) {                             // lanes per head
      case 1: return launch_rope_wide<1>(q, positions, slot_mapping, inv_freq, q_norm, k_norm, kp, vp, tokens, heads, kv_heads, eps, write_kv, stream);
      case 2: return launch_rope_wide<2>(q, positions, slot_mapping, inv_freq, q_norm, k_norm, kp, vp, tokens, heads, kv_heads, eps, write_kv, stream);
      case 4: return launch_rope_wide<4>(q, positions, slot_mapping, inv_freq, q_norm, k_norm, kp, vp, tokens, heads, kv_heads, eps, write_kv, stream);
      case 8: return launch_rope_wide<8>(q, positions, slot_mapping, inv_freq, q_norm, k_norm, kp, vp, tokens, heads, kv_heads, eps, write_kv, stream);
      case 16: return launch_rope_wide<16>(q, positions, slot_mapping, inv_freq, q_norm, k_norm, kp, vp, tokens, heads, kv_heads, eps, write_kv, stream);
      default: break;                                    // other head sizes: the kernel below
    }
  }
  if (bf16)
    return launch_rope((__nv_bfloat16*)qkv, positions, slot_mapping, inv_freq, q_norm, k_norm, (__nv_bfloat16*)k_pages,
                       (__nv_bfloat16*)v_pages, tokens, heads, kv_heads, head_dim, rotary_dim, eps, write_kv, stream);
  return launch_rope((float*)qkv, positions, slot_mapping, inv_freq, q_norm, k_norm, (float*)k_pages, (float*)v_pages,
                     tokens, heads, kv_heads, head_dim, rotary_dim, eps, write_kv, stream);
}
