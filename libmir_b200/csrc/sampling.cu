// Sampling on the device over 32-bit logits [rows, vocab]: one block per row, per-row options.
//
//   greedy      temperature <= FLT_EPSILON or top_k == 1: highest logit, lowest id on ties
//               (libmir cuda/kernels/sampling_bf16.cu:18-27)
//   full        top_k == 0 and top_p >= 1: weights exp((l - max) / T) in 64-bit, the first token in
//               VOCABULARY order whose cumulative weight reaches draw * total
//               (runtime/src/sampling/mod.rs:82-116)
//   ranked      otherwise: candidates ordered by (score descending, id ascending), top-p truncation
//               (first rank whose cumulative share reaches top_p), then top-k, then the first token in
//               RANK order whose cumulative weight reaches draw * kept total
//               (runtime/src/sampling/mod.rs:72-80,118-135, candidate.rs:69-107)
// The uniform draw in [0, 1) comes from the host's SplitMix64, one per row and step, as in libmir
// (src/generation/sampling.rs:36-41).  Non-finite logits are not candidates.
//
// The ranked mode sorts 64-bit keys (orderable(score) << 32 | ~id) with a bitonic network in a
// scratch buffer of rows * pow2ceil(vocab) keys that the caller provides.
#include <cfloat>
#include <cooperative_groups.h>
#include "common.cuh"

namespace cg = cooperative_groups;
using namespace mir;

constexpr int kThreads = 1024;
constexpr int kSlices = 8;     // CTAs of a cluster that share the scan for a row's highest logit

struct SampleOptions {   // one per row; mirrored by a numpy structured dtype on the host
  double draw;
  float temperature;
  float top_p;
  int top_k;
  int pad;
};

__device__ __forceinline__ bool is_greedy(const SampleOptions& o) {
  return o.temperature <= FLT_EPSILON || o.top_k == 1;
}
__device__ __forceinline__ bool is_full(const SampleOptions& o) { return o.top_k == 0 && o.top_p >= 1.0f; }

// (value, index) maximum with ties to the lower index; the whole block gets the result.
__device__ void block_argmax(float& value, int& index, float* s_value, int* s_index) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, value, o);
    const int other_index = __shfl_xor_sync(0xffffffffu, index, o);
    if (other > value || (other == value && other_index < index)) { value = other; index = other_index; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { s_value[warp] = value; s_index[warp] = index; }
  __syncthreads();
  value = s_value[lane];
  index = s_index[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, value, o);
    const int other_index = __shfl_xor_sync(0xffffffffu, index, o);
    if (other > value || (other == value && other_index < index)) { value = other; index = other_index; }
  }
}

__device__ double block_sum_f64(double v, double* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  double total = scratch[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
  return total;
}

// First index i in [0, n) (n split into kThreads contiguous chunks) whose inclusive cumulative weight
// reaches `target`; `weight(i)` must be callable by any thread.  Returns through *found (shared).
// chunk_sums: kThreads doubles of shared memory.  Falls back to `fallback` when rounding leaves none.
template <typename W>
__device__ int first_reaching(W weight, int n, double target, double* chunk_sums, int* found, int fallback) {
  const int chunk = (n + kThreads - 1) / kThreads;
  const int begin = min(n, (int)threadIdx.x * chunk), end = min(n, begin + chunk);
  double mine = 0.0;
  for (int i = begin; i < end; ++i) mine += weight(i);
  __syncthreads();
  chunk_sums[threadIdx.x] = mine;
  if (threadIdx.x == 0) *found = -1;
  __syncthreads();
  if (threadIdx.x == 0) {   // exclusive prefix, in order
    double running = 0.0;
    for (int t = 0; t < kThreads; ++t) {
      const double s = chunk_sums[t];
      chunk_sums[t] = running;
      running += s;
    }
  }
  __syncthreads();
  const double before = chunk_sums[threadIdx.x];
  if (end > begin && before < target && before + mine >= target) {
    double remaining = target - before;
    int hit = end - 1;
    for (int i = begin; i < end; ++i) {
      remaining -= weight(i);
      if (remaining <= 0.0) { hit = i; break; }
    }
    *found = hit;
  }
  __syncthreads();
  int result = *found;
  if (result < 0) result = target <= 0.0 ? 0 : fallback;
  __syncthreads();
  return result;
}

__device__ __forceinline__ unsigned orderable(float v) {
  const unsigned bits = __float_as_uint(v);
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}
__device__ __forceinline__ float from_orderable(unsigned key) {
  return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

__global__ void __launch_bounds__(kThreads) sample_kernel(const float* __restrict__ logits, size_t ld, int vocab,
                                                           const SampleOptions* __restrict__ options,
                                                           unsigned long long* __restrict__ sort_keys, int padded,
                                                           int* __restrict__ tokens) {
  __shared__ float s_value[32];
  __shared__ int s_index[32];
  __shared__ double s_sum[32];
  __shared__ double chunk_sums[kThreads];
  __shared__ int found;
  grid_launch_dependents();
  grid_dependency_wait();
  // A cluster of kSlices CTAs per row: each finds the highest logit of its slice of the vocabulary, the first CTA
  // takes the best of them out of distributed shared memory (ties to the lowest id, as one scan would) and goes
  // on alone if the row is not greedy.
  __shared__ float slice_value;
  __shared__ int slice_index;
  cg::cluster_group cluster = cg::this_cluster();
  const int row = blockIdx.x, slice = blockIdx.y;
  const SampleOptions opt = options[row];
  const float* l = logits + (size_t)row * ld;

  const int per_slice = (vocab + kSlices - 1) / kSlices;
  const int slice_begin = slice * per_slice, slice_end = min(vocab, slice_begin + per_slice);
  float best = -FLT_MAX;
  int best_index = 0x7fffffff;
  for (int i = slice_begin + threadIdx.x; i < slice_end; i += kThreads) {
    const float v = l[i];
    if (isfinite(v) && (v > best || (v == best && i < best_index))) { best = v; best_index = i; }
  }
  block_argmax(best, best_index, s_value, s_index);
  if (threadIdx.x == 0) { slice_value = best; slice_index = best_index; }
  cluster.sync();
  if (slice == 0) {
    for (int other = 1; other < kSlices; ++other) {
      const float v = *cluster.map_shared_rank(&slice_value, other);
      const int i = *cluster.map_shared_rank(&slice_index, other);
      if (v > best || (v == best && i < best_index)) { best = v; best_index = i; }
    }
  }
  cluster.sync();                                   // the other CTAs keep their shared memory until it was read
  if (slice != 0) return;
  if (best_index == 0x7fffffff) best_index = 0;   // no finite logit: the host reports it
  if (is_greedy(opt)) {
    if (threadIdx.x == 0) tokens[row] = best_index;
    return;
  }
  const double temperature = (double)opt.temperature;

  if (is_full(opt)) {
    auto weight = [&](int i) -> double {
      const float v = l[i];
      return isfinite(v) ? exp((double)(v - best) / temperature) : 0.0;
    };
    double mine = 0.0;
    for (int i = threadIdx.x; i < vocab; i += kThreads) mine += weight(i);
    const double total = block_sum_f64(mine, s_sum);
    const int token = first_reaching(weight, vocab, opt.draw * total, chunk_sums, &found, best_index);
    if (threadIdx.x == 0) tokens[row] = token;
    return;
  }

  // ranked: sort keys descending (score, then lower id first)
  if (sort_keys == nullptr) {
    if (threadIdx.x == 0) tokens[row] = -1;   // the launcher refuses this before the launch
    return;
  }
  unsigned long long* keys = sort_keys + (size_t)row * padded;
  for (int i = threadIdx.x; i < padded; i += kThreads) {
    unsigned long long key = 0ull;
    if (i < vocab && isfinite(l[i])) key = ((unsigned long long)orderable(l[i]) << 32) | (unsigned)(~(unsigned)i);
    keys[i] = key;
  }
  __syncthreads();
  for (int size = 2; size <= padded; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < padded / 2; t += kThreads) {
        const int low = 2 * t - (t & (stride - 1));
        const int high = low + stride;
        const bool descending = (low & size) == 0;
        const unsigned long long a = keys[low], b = keys[high];
        if ((a < b) == descending) { keys[low] = b; keys[high] = a; }
      }
      __syncthreads();
    }
  }
  auto ranked_weight = [&](int i) -> double {
    const unsigned long long key = keys[i];
    if (key == 0ull) return 0.0;
    return exp((double)(from_orderable((unsigned)(key >> 32)) - best) / temperature);
  };
  double mine = 0.0;
  for (int i = threadIdx.x; i < vocab; i += kThreads) mine += ranked_weight(i);
  const double total = block_sum_f64(mine, s_sum);
  int keep = vocab;
  if (opt.top_p < 1.0f)
    keep = first_reaching(ranked_weight, vocab, (double)opt.top_p * total, chunk_sums, &found, vocab - 1) + 1;
  if (opt.top_k > 0) keep = min(keep, opt.top_k);
  mine = 0.0;
  for (int i = threadIdx.x; i < keep; i += kThreads) mine += ranked_weight(i);
  const double kept_total = block_sum_f64(mine, s_sum);
  const int rank = first_reaching(ranked_weight, keep, opt.draw * kept_total, chunk_sums, &found, keep - 1);
  if (threadIdx.x == 0) tokens[row] = (int)(~(unsigned)(keys[rank] & 0xffffffffull));
}

// Repetition penalty on the logits in place: a positive score is divided by the penalty, a negative one
// multiplied (runtime/src/sampling/candidate.rs:92-107).  `ids` holds each row's DISTINCT history tokens.
__global__ void penalty_kernel(float* __restrict__ logits, size_t ld, int vocab, const int* __restrict__ ids,
                               const int* __restrict__ id_rows, const float* __restrict__ penalties, int count) {
  const int index = blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= count) return;
  const int row = id_rows[index], id = ids[index];
  const float penalty = penalties[row];
  if (penalty <= 1.0f || id < 0 || id >= vocab) return;
  float* slot = logits + (size_t)row * ld + id;
  const float v = *slot;
  *slot = signbit(v) ? v * penalty : v / penalty;
}

MIR_EXPORT int mir_sample(const float* logits, long long ld, int rows, int vocab, const void* options,
                          void* sort_keys, long long sort_keys_capacity, int needs_ranked, int* tokens,
                          cudaStream_t stream) {
  if (rows == 0) return MIR_OK;
  if (rows < 0 || vocab <= 0 || ld < vocab) { mir_set_error("sample: bad sizes"); return MIR_BAD_ARGUMENT; }
  int padded = 1;
  while (padded < vocab) padded <<= 1;
  if (needs_ranked && (sort_keys == nullptr || sort_keys_capacity < (long long)rows * padded)) {
    mir_set_error("sample: top-k / top-p sampling needs a scratch of %lld keys, got %lld", (long long)rows * padded,
                  sort_keys_capacity);
    return MIR_BAD_ARGUMENT;
  }
  return mir_launch("sample", sample_kernel, dim3(rows, kSlices), dim3(kThreads), 0, stream, kSlices, logits, (size_t)ld, vocab,
                    (const SampleOptions*)options, needs_ranked ? (unsigned long long*)sort_keys : nullptr, padded,
                    tokens);
}

MIR_EXPORT int mir_repetition_penalty(float* logits, long long ld, int vocab, const int* ids, const int* id_rows,
                                      const float* penalties, int count, cudaStream_t stream) {
  if (count == 0) return MIR_OK;
  penalty_kernel<<<(count + 255) / 256, 256, 0, stream>>>(logits, (size_t)ld, vocab, ids, id_rows, penalties, count);
  return mir_check_launch("repetition_penalty");
}
