// Embedding gather, RMSNorm, SiLU-gate and bias kernels.  The residual stream is 32-bit in both
// engine dtypes; T is the storage type of weights and activations (float or bf16).
//
// What each replaces in libmir: embedding_bf16.cu:3-19, rms_norm_bf16.cu:3-36,
// elementwise_bf16.cu:42-70 (packed gate|up), select_row_bf16.cu (row gather, folded into the norm).
#include <cuda_fp16.h>
#include "common.cuh"

using namespace mir;

// out[r, :] = float(table[ids[r], :]) * scale.  An id outside [0, vocab) gives a row of zeros;
// the host rejects such ids before the launch.
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                             int hidden, int vocab, float scale) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int row = blockIdx.x;
  const int id = ids[row];
  const bool ok = id >= 0 && id < vocab;
  const T* src = table + (size_t)(ok ? id : 0) * hidden;
  float* dst = out + (size_t)row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = ok ? to_float(src[c]) * scale : 0.0f;
}

// y[r, :] = x[src(r), :] * rsqrt(mean(x^2) + eps) * w, src(r) = rows ? rows[r] : r.
// Sum of squares and scaling in 32-bit with a fixed reduction tree.
template <typename Tout>
__global__ void rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                                Tout* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[32];
  grid_launch_dependents();
  grid_dependency_wait();

  const int row = blockIdx.x;
  const float* src = x + (size_t)(rows ? rows[row] : row) * hidden;
  float sum = 0.0f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = src[c];
    sum = fmaf(v, v, sum);
  }
  sum = block_sum(sum, scratch);
  const float inverse = rsqrtf(sum / (float)hidden + eps);
  Tout* dst = out + (size_t)row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = from_float<Tout>(src[c] * inverse * weight[c]);
}

// The same with 16-byte loads (hidden a multiple of 4); the second pass finds the row in L1.
template <typename Tout>
__global__ void rms_norm_vec4_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                                     Tout* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[32];
  grid_launch_dependents();
  grid_dependency_wait();
  const int row = blockIdx.x;
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[row] : row) * hidden);
  const float4* w4 = reinterpret_cast<const float4*>(weight);
  const int quads = hidden >> 2;
  float sum = 0.0f;
  for (int c = threadIdx.x; c < quads; c += blockDim.x) {
    const float4 v = src[c];
    sum = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, sum))));
  }
  sum = block_sum(sum, scratch);
  const float inverse = rsqrtf(sum / (float)hidden + eps);
  Tout* dst = out + (size_t)row * hidden;
  for (int c = threadIdx.x; c < quads; c += blockDim.x) {
    const float4 v = src[c];
    const float4 w = __ldg(w4 + c);
    const float a = v.x * inverse * w.x, b = v.y * inverse * w.y, d = v.z * inverse * w.z, e = v.w * inverse * w.w;
    if (sizeof(Tout) == 4) {
      reinterpret_cast<float4*>(dst)[c] = make_float4(a, b, d, e);
    } else {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(d, e);
      uint2 packed;
      packed.x = *reinterpret_cast<const uint32_t*>(&lo);
      packed.y = *reinterpret_cast<const uint32_t*>(&hi);
      reinterpret_cast<uint2*>(dst)[c] = packed;
    }
  }
}

// out[r, c] = silu(gu[r, c]) * gu[r, inter + c]; gu rows are [gate | up].
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total) {
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const size_t row = index / inter;
  const int col = (int)(index - row * inter);
  const float g = to_float(gu[row * 2 * inter + col]);
  const float u = to_float(gu[row * 2 * inter + inter + col]);
  out[index] = from_float<T>(g / (1.0f + expf(-g)) * u);
}

// The same, 8 columns per thread with 16-byte loads and stores (inter a multiple of 8, bf16).
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                       int inter, size_t total8) {
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total8) return;
  const int per_row = inter / 8;
  const size_t row = index / per_row;
  const int col = (int)(index - row * per_row) * 8;
  float g[8], u[8];
  load8(gu + row * 2 * inter + col, g);
  load8(gu + row * 2 * inter + inter + col, u);
  uint4 packed;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    h[i] = __floats2bfloat162_rn(g[2 * i] / (1.0f + expf(-g[2 * i])) * u[2 * i],
                                 g[2 * i + 1] / (1.0f + expf(-g[2 * i + 1])) * u[2 * i + 1]);
  *reinterpret_cast<uint4*>(out + row * inter + col) = packed;
}

// x[r, c] += bias[c]  (32-bit residual; used when a projection that accumulates into the residual has a bias).
template <typename T>
__global__ void add_bias_kernel(float* __restrict__ x, const T* __restrict__ bias, int cols, size_t total) {
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  x[index] += to_float(bias[index % cols]);
}

// dst[i] = T(src[i]) for the load-time casts (dense_cast.cu:4-18) and for copying logits rows.
template <typename Tin, typename Tout>
__global__ void cast_kernel(const Tin* __restrict__ src, Tout* __restrict__ dst, size_t total) {
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index < total) dst[index] = from_float<Tout>(to_float(src[index]));
}

#define LAUNCH_1D(kernel, total, ...)                                                      \
  do {                                                                                     \
    const size_t n_ = (total);                                                             \
    if (n_ == 0) return MIR_OK;                                                            \
    kernel<<<(unsigned)((n_ + 255) / 256), 256, 0, stream>>>(__VA_ARGS__);                 \
  } while (0)

MIR_EXPORT int mir_embed(int bf16, const void* table, const int* ids, float* out, int rows, int hidden, int vocab,
                         float scale, cudaStream_t stream) {
  if (rows == 0) return MIR_OK;
  if (rows < 0 || hidden <= 0 || vocab <= 0) { mir_set_error("embed: bad sizes"); return MIR_BAD_ARGUMENT; }
  if (bf16)
    return mir_launch("embed", embed_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, 0,
                      (const __nv_bfloat16*)table, ids, out, hidden, vocab, scale);
  return mir_launch("embed", embed_kernel<float>, dim3(rows), dim3(256), 0, stream, 0, (const float*)table, ids, out,
                    hidden, vocab, scale);
}

MIR_EXPORT int mir_rms_norm(int bf16, const float* x, const float* weight, void* out, const int* rows, int n_rows,
                            int hidden, float eps, cudaStream_t stream) {
  if (n_rows == 0) return MIR_OK;
  if (n_rows < 0 || hidden <= 0) { mir_set_error("rms_norm: bad sizes"); return MIR_BAD_ARGUMENT; }
  if ((hidden & 3) == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)weight & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const int vec_threads = hidden >= 1024 ? 256 : 128;
    if (bf16)
      return mir_launch("rms_norm", rms_norm_vec4_kernel<__nv_bfloat16>, dim3(n_rows), dim3(vec_threads), 0, stream, 0,
                        x, weight, (__nv_bfloat16*)out, rows, hidden, eps);
    return mir_launch("rms_norm", rms_norm_vec4_kernel<float>, dim3(n_rows), dim3(vec_threads), 0, stream, 0, x, weight,
                      (float*)out, rows, hidden, eps);
  }
  const int threads = hidden >= 2048 ? 512 : 256;
  if (bf16)
    return mir_launch("rms_norm", rms_norm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, 0, x, weight,
                      (__nv_bfloat16*)out, rows, hidden, eps);
  return mir_launch("rms_norm", rms_norm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, 0, x, weight,
                    (float*)out, rows, hidden, eps);
}

MIR_EXPORT int mir_silu_mul(int bf16, const void* gu, void* out, int rows, int inter, cudaStream_t stream) {
  if (rows < 0 || inter <= 0) { mir_set_error("silu_mul: bad sizes"); return MIR_BAD_ARGUMENT; }
  const size_t total = (size_t)rows * inter;
  if (bf16 && inter % 8 == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0)
    LAUNCH_1D(silu_mul_bf16x8_kernel, total / 8, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, total / 8);
  else if (bf16) LAUNCH_1D(silu_mul_kernel, total, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, total);
  else LAUNCH_1D(silu_mul_kernel, total, (const float*)gu, (float*)out, inter, total);
  return mir_check_launch("silu_mul");
}

MIR_EXPORT int mir_add_bias(int bf16, float* x, const void* bias, int rows, int cols, cudaStream_t stream) {
  if (rows < 0 || cols <= 0) { mir_set_error("add_bias: bad sizes"); return MIR_BAD_ARGUMENT; }
  const size_t total = (size_t)rows * cols;
  if (bf16) LAUNCH_1D(add_bias_kernel, total, x, (const __nv_bfloat16*)bias, cols, total);
  else LAUNCH_1D(add_bias_kernel, total, x, (const float*)bias, cols, total);
  return mir_check_launch("add_bias");
}

// kind: 0 f32->bf16, 1 bf16->f32, 2 f16->bf16, 3 f16->f32 (what a checkpoint may store, to what the engine keeps).
MIR_EXPORT int mir_cast(int kind, const void* src, void* dst, size_t total, cudaStream_t stream) {
  if (kind == 0) LAUNCH_1D(cast_kernel, total, (const float*)src, (__nv_bfloat16*)dst, total);
  else if (kind == 1) LAUNCH_1D(cast_kernel, total, (const __nv_bfloat16*)src, (float*)dst, total);
  else if (kind == 2) LAUNCH_1D(cast_kernel, total, (const __half*)src, (__nv_bfloat16*)dst, total);
  else if (kind == 3) LAUNCH_1D(cast_kernel, total, (const __half*)src, (float*)dst, total);
  else { mir_set_error("cast: unknown kind %d", kind); return MIR_BAD_ARGUMENT; }
  return mir_check_launch("cast");
}

// Random weights on the device: element i of a tensor is a normal deviate (Box-Muller on two uniforms from the
// SplitMix64 of seed + 2 i and seed + 2 i + 1) times `deviation`: the same for a seed whatever the launch shape.
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, size_t total, unsigned long long seed, float deviation) {
  const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const unsigned long long a = splitmix64(seed + 2ull * index), b = splitmix64(seed + 2ull * index + 1ull);
  const float u = ((float)(a >> 40) + 0.5f) * (1.0f / 16777216.0f);      // (0, 1)
  const float v = (float)(b >> 40) * (1.0f / 16777216.0f);               // [0, 1)
  out[index] = from_float<T>(deviation * sqrtf(-2.0f * logf(u)) * cospif(2.0f * v));
}

MIR_EXPORT int mir_random_normal(int bf16, void* out, size_t total, unsigned long long seed, float deviation,
                                 cudaStream_t stream) {
  if (bf16) LAUNCH_1D(random_normal_kernel, total, (__nv_bfloat16*)out, total, seed, deviation);
  else LAUNCH_1D(random_normal_kernel, total, (float*)out, total, seed, deviation);
  return mir_check_launch("random_normal");
}

// ---- decode batches that run as a captured graph -------------------------------------------------
// Before the layers: where each row's new key/value goes, from its position and block table.  A row
// with a negative position is padding (the batch is smaller than the captured size): no cache write.
__global__ void decode_prepare_kernel(const int* __restrict__ positions, const int* __restrict__ block_table,
                                      int table_width, int page_size, int* __restrict__ slot_mapping,
                                      int* __restrict__ context_lens, int rows) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  const int position = positions[row];
  int slot = -1;
  if (position >= 0) {
    const int block = position / page_size;
    const int page = block < table_width ? block_table[(size_t)row * table_width + block] : -1;
    if (page >= 0) slot = page * page_size + position % page_size;
  }
  slot_mapping[row] = slot;
  context_lens[row] = position >= 0 ? position + 1 : 0;
}

// After sampling: the sampled token is the next step's input, positions move on by one, and the token is
// appended to a log so that several steps can run without the host reading each one.
__global__ void decode_advance_kernel(const int* __restrict__ sampled, int* __restrict__ tokens,
                                      int* __restrict__ positions, int* __restrict__ token_log, int log_steps,
                                      int* __restrict__ step_counter, int rows) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int step = *step_counter;
  __syncthreads();
  for (int row = threadIdx.x; row < rows; row += blockDim.x) {
    const int token = sampled[row];
    tokens[row] = token;
    if (positions[row] >= 0) positions[row] += 1;
    if (step < log_steps) token_log[(size_t)step * rows + row] = token;
  }
  if (threadIdx.x == 0) *step_counter = step + 1;
}

MIR_EXPORT int mir_decode_prepare(const int* positions, const int* block_table, int table_width, int page_size,
                                  int* slot_mapping, int* context_lens, int rows, cudaStream_t stream) {
  if (rows <= 0) return MIR_OK;
  return mir_launch("decode_prepare", decode_prepare_kernel, dim3((rows + 127) / 128), dim3(128), 0, stream, 0,
                    positions, block_table, table_width, page_size, slot_mapping, context_lens, rows);
}

MIR_EXPORT int mir_decode_advance(const int* sampled, int* tokens, int* positions, int* token_log, int log_steps,
                                  int* step_counter, int rows, cudaStream_t stream) {
  if (rows <= 0) return MIR_OK;
  return mir_launch("decode_advance", decode_advance_kernel, dim3(1), dim3(256), 0, stream, 0, sampled, tokens,
                    positions, token_log, log_steps, step_counter, rows);
}
