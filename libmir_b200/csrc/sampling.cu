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
// Keys are 64 bits, orderable(score) << 32 | ~id, so that one comparison orders by score and then by lower id
// (libmir's tie rule).  The ranked mode first looks at the 1,024 best tokens, found by counting (libmir looks at
// chunks of candidates and merges them, cuda/kernels/sampling_bf16.cu:30-133, with top_k capped at 64); only a
// draw that they cannot decide sorts the whole vocabulary, in a scratch buffer of rows * pow2ceil(vocab) keys
// that the caller provides.
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

// Inclusive sum over the block of one double per thread (thread order); every thread gets its own inclusive value,
// *total (shared) the sum of all.  scratch: 32 doubles.
__device__ double block_scan_f64(double v, double* scratch, double* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const double other = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += other;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    double w = scratch[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const double other = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += other;
    }
    scratch[lane] = w;
    if (lane == 31) *total = w;
  }
  __syncthreads();
  return v + (warp > 0 ? scratch[warp - 1] : 0.0);
}

// Where, in rank order (score descending, then id ascending), the cumulative weight first reaches a target: the
// orderable score at which it happens, the weight and the number of tokens that score higher, and how many tokens
// share that score.  Found without sorting: three passes over the orderable scores (11 + 11 + 10 bits), each adding
// the weights and the counts of the tokens that match the bits found so far into the bins of the next bits (the
// lanes of a warp that hit the same bin add once, 64-bit sums), summed over the cluster by slice 0, which scans the
// bins from the top.  If rounding lets no bin reach the target, the lowest score is the answer.
struct Crossing {
  unsigned key;          // orderable score of the rank at which the target is reached
  unsigned above_count;  // tokens that score higher
  unsigned ties;         // tokens with exactly this score
  unsigned pad;
  double above_weight;   // weight of the tokens that score higher
};

constexpr int kSearchBins = 2048;

template <typename Weight>
__device__ Crossing find_crossing(cg::cluster_group& cluster, const float* __restrict__ l, int slice, int slice_begin,
                                  int slice_end, Weight weight, double target, unsigned char* overlay, double* s_sum,
                                  Crossing* shared_result) {
  int* counts = reinterpret_cast<int*>(overlay);                                  // kSearchBins
  double* weights = reinterpret_cast<double*>(overlay + kSearchBins * sizeof(int));  // kSearchBins
  unsigned prefix = 0u, above_count = 0u, ties = 0u;
  double above_weight = 0.0;
  const int lane = threadIdx.x & 31;
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = pass == 0 ? 21 : (pass == 1 ? 10 : 0);
    const int bins = pass == 2 ? 1024 : kSearchBins;
    const unsigned fixed_mask = pass == 0 ? 0u : (pass == 1 ? 0xffe00000u : 0xfffffc00u);
    for (int i = threadIdx.x; i < kSearchBins; i += kThreads) { counts[i] = 0; weights[i] = 0.0; }
    __syncthreads();
    for (int i0 = slice_begin; i0 < slice_end; i0 += kThreads) {
      const int i = i0 + (int)threadIdx.x;
      bool match = false;
      unsigned bin = 0u;
      double w = 0.0;
      if (i < slice_end) {
        const float v = l[i];
        if (isfinite(v)) {
          const unsigned key = orderable(v);
          if ((key & fixed_mask) == prefix) { match = true; bin = (key >> shift) & (unsigned)(bins - 1); w = weight(i); }
        }
      }
      unsigned todo = __ballot_sync(0xffffffffu, match);
      while (todo != 0u) {                                     // one round per distinct bin among the warp's lanes
        const int leader = __ffs(todo) - 1;
        const unsigned leader_bin = __shfl_sync(0xffffffffu, bin, leader);
        const unsigned group = __ballot_sync(0xffffffffu, match && bin == leader_bin) & todo;
        double sum = (group >> lane) & 1u ? w : 0.0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == leader) {
          atomicAdd(&counts[leader_bin], __popc(group));
          atomicAdd(&weights[leader_bin], sum);
        }
        todo &= ~group;
      }
    }
    cluster.sync();
    if (slice == 0) {
      for (int i = threadIdx.x; i < bins; i += kThreads) {
        int count = counts[i];
        double sum = weights[i];
        for (int other = 1; other < kSlices; ++other) {
          count += cluster.map_shared_rank(counts, other)[i];
          sum += cluster.map_shared_rank(weights, other)[i];
        }
        counts[i] = count;
        weights[i] = sum;
      }
      __syncthreads();
      // from the top bin down, two bins per thread
      constexpr int per_thread = kSearchBins / kThreads;
      int my_counts[per_thread];
      double my_weights[per_thread];
      int count_sum = 0;
      double weight_sum = 0.0;
#pragma unroll
      for (int j = 0; j < per_thread; ++j) {
        const int b = bins - 1 - ((int)threadIdx.x * per_thread + j);
        my_counts[j] = b >= 0 ? counts[b] : 0;
        my_weights[j] = b >= 0 ? weights[b] : 0.0;
        count_sum += my_counts[j];
        weight_sum += my_weights[j];
      }
      __shared__ double scan_total;
      __shared__ int lowest_bin;
      const double weight_upto = block_scan_f64(weight_sum, s_sum, &scan_total);
      const double count_upto = block_scan_f64((double)count_sum, s_sum, &scan_total);   // counts: exact in a double
      if (threadIdx.x == 0) { lowest_bin = bins; shared_result->pad = 0u; }
      __syncthreads();
      for (int j = 0; j < per_thread; ++j) {                     // the lowest bin that holds a token: the answer if none reaches
        const int b = bins - 1 - ((int)threadIdx.x * per_thread + j);
        if (b >= 0 && my_counts[j] > 0) atomicMin(&lowest_bin, b);
      }
      __syncthreads();
      double running_weight = above_weight + (weight_upto - weight_sum);
      unsigned running_count = above_count + (unsigned)(count_upto - (double)count_sum);
      const bool reaches = running_weight < target && running_weight + weight_sum >= target;
      if (reaches) {
        // the first of this thread's bins with which the running weight reaches the target (rounding may let the sum
        // of the bins reach it and no single step: then the last bin that holds a token)
        int chosen = -1, last_held = -1;
        double weight_before = running_weight;
        unsigned count_before = running_count;
        for (int j = 0; j < per_thread && chosen < 0; ++j) {
          if (my_counts[j] > 0) last_held = j;
          if (my_counts[j] > 0 && running_weight + my_weights[j] >= target) {
            chosen = j;
            break;
          }
          running_weight += my_weights[j];
          running_count += (unsigned)my_counts[j];
        }
        if (chosen < 0 && last_held >= 0) {
          chosen = last_held;
          running_weight = weight_before;
          running_count = count_before;
          for (int j = 0; j < chosen; ++j) { running_weight += my_weights[j]; running_count += (unsigned)my_counts[j]; }
        }
        if (chosen >= 0) {
          const int b = bins - 1 - ((int)threadIdx.x * per_thread + chosen);
          shared_result->key = prefix | ((unsigned)b << shift);
          shared_result->above_count = running_count;
          shared_result->above_weight = running_weight;
          shared_result->ties = (unsigned)my_counts[chosen];
          shared_result->pad = 1u;
        }
      }
      __syncthreads();
      if (shared_result->pad == 0u && threadIdx.x == 0) {        // nothing reached the target (or it is not positive)
        const int b = target <= 0.0 ? -1 : lowest_bin;
        int top = bins - 1;
        while (top > 0 && counts[top] == 0) --top;                // target <= 0: the highest bin that holds a token
        const int chosen = (b < 0 || b >= bins) ? top : b;
        unsigned count_above = above_count;
        double weight_above = above_weight;
        for (int other = bins - 1; other > chosen; --other) { count_above += (unsigned)counts[other]; weight_above += weights[other]; }
        shared_result->key = prefix | ((unsigned)chosen << shift);
        shared_result->above_count = count_above;
        shared_result->above_weight = weight_above;
        shared_result->ties = (unsigned)counts[chosen];
      }
      __syncthreads();
    }
    cluster.sync();
    const Crossing* result = cluster.map_shared_rank(shared_result, 0);
    prefix = result->key;
    above_count = result->above_count;
    above_weight = result->above_weight;
    ties = result->ties;
    cluster.sync();                                               // read by everyone before the next pass rewrites it
  }
  Crossing out;
  out.key = prefix;
  out.above_count = above_count;
  out.above_weight = above_weight;
  out.ties = ties;
  out.pad = 0u;
  return out;
}

// How many of `ties` tokens of weight `each`, added one after the other to `above`, it takes to reach `target`
// (at least 1, at most `ties`).
__device__ unsigned ties_needed(double above, double each, unsigned ties, double target) {
  if (ties <= 1u || !(each > 0.0)) return max(1u, min(ties, 1u));
  double guess = ceil((target - above) / each);
  if (!(guess >= 1.0)) guess = 1.0;
  if (guess > (double)ties) guess = (double)ties;
  unsigned count = (unsigned)guess;
  while (count > 1u && above + (double)(count - 1u) * each >= target) --count;
  while (count < ties && above + (double)count * each < target) ++count;
  return count;
}

constexpr int kCandidates = 1024;       // ranked sampling looks at this many best tokens first ...
constexpr int kCandidateRoom = 2048;    // ... and takes up to this many when scores tie at the threshold
constexpr int kBins = 4096;

// One cluster of kSlices CTAs per row; slice s owns the ids [s, s + 1) * ceil(vocab / kSlices).
//
//   every mode  each slice finds its highest logit; slice 0 takes the best of them (ties to the lowest id, as one
//               scan would).
//   full        each thread sums the 64-bit weights of a contiguous chunk of its slice; prefix sums over threads and
//               slices locate the chunk in which the cumulative weight (vocabulary order) reaches draw * total, and
//               that thread walks its chunk.
//   ranked      the kCandidates best tokens are found without sorting the vocabulary: three counting passes over
//               the orderable scores (12 + 12 + 8 bits, histograms added up over the cluster) give the score that
//               the kCandidates-th best token has; everything at or above it goes to slice 0, which sorts it
//               (bitonic, shared memory) and takes prefix sums in rank order.  That decides the draw whenever the
//               nucleus (top_p of the total weight of ALL tokens) or top_k ends inside the candidates.  When it
//               does not (a flat distribution with top_p alone, or thousands of tied scores), slice 0 sorts the
//               whole vocabulary in the caller's scratch as before: slow and exact.
__global__ void __launch_bounds__(kThreads) sample_kernel(const float* __restrict__ logits, size_t ld, int vocab,
                                                           const SampleOptions* __restrict__ options,
                                                           unsigned long long* __restrict__ sort_keys, int padded,
                                                           int* __restrict__ tokens,
                                                           const float* __restrict__ candidate_value,
                                                           const int* __restrict__ candidate_index, int given) {
  __shared__ float s_value[32];
  __shared__ int s_index[32];
  __shared__ double s_sum[32];
  __shared__ double chunk_sums[kThreads];
  __shared__ int found;
  __shared__ __align__(16) unsigned char overlay[kCandidateRoom * (sizeof(unsigned long long) + sizeof(double))];
  __shared__ float slice_value;                    // this slice's best, then (slice 0) the row's best
  __shared__ int slice_index;
  __shared__ double slice_total;                   // sum of this slice's weights
  __shared__ unsigned select_prefix, select_above; // slice 0: the threshold found so far; tokens strictly above it
  __shared__ int candidate_count;                  // slice 0: candidates gathered
  __shared__ int search_mode;                      // slice 0: 0 the candidates decided, 1 the nucleus must be searched
  __shared__ Crossing crossing;                    // slice 0: result of a pass of find_crossing
  grid_launch_dependents();
  grid_dependency_wait();
  cg::cluster_group cluster = cg::this_cluster();
  const int row = blockIdx.x, slice = blockIdx.y;
  const SampleOptions opt = options[row];
  const float* l = logits + (size_t)row * ld;

  const int per_slice = (vocab + kSlices - 1) / kSlices;
  const int slice_begin = min(vocab, slice * per_slice), slice_end = min(vocab, slice_begin + per_slice);
  float best = -FLT_MAX;
  int best_index = 0x7fffffff;
  if (candidate_value != nullptr) {
    // the kernel that wrote the logits left the largest finite one of every 32 columns (and its column, ties to the
    // lower one; -FLT_MAX and 0x7fffffff where there is none): the row's largest is among these
    const int per = (given + kSlices - 1) / kSlices;
    const int begin = min(given, slice * per), end = min(given, begin + per);
    for (int c = begin + threadIdx.x; c < end; c += kThreads) {
      const float v = candidate_value[(size_t)row * given + c];
      const int i = candidate_index[(size_t)row * given + c];
      if (i < vocab && (v > best || (v == best && i < best_index))) { best = v; best_index = i; }
    }
  } else {
    for (int i = slice_begin + threadIdx.x; i < slice_end; i += kThreads) {
      const float v = l[i];
      if (isfinite(v) && (v > best || (v == best && i < best_index))) { best = v; best_index = i; }
    }
  }
  block_argmax(best, best_index, s_value, s_index);
  if (threadIdx.x == 0) { slice_value = best; slice_index = best_index; }
  cluster.sync();
  if (slice == 0 && threadIdx.x == 0) {
    for (int other = 1; other < kSlices; ++other) {
      const float v = *cluster.map_shared_rank(&slice_value, other);
      const int i = *cluster.map_shared_rank(&slice_index, other);
      if (v > best || (v == best && i < best_index)) { best = v; best_index = i; }
    }
    if (best_index == 0x7fffffff) best_index = 0;   // no finite logit: the host reports it
  }
  cluster.sync();                                   // slice 0 has read the slices' results ...
  if (slice == 0 && threadIdx.x == 0) { slice_value = best; slice_index = best_index; }
  cluster.sync();                                   // ... and published the row's
  best = *cluster.map_shared_rank(&slice_value, 0);
  best_index = *cluster.map_shared_rank(&slice_index, 0);
  if (is_greedy(opt)) {
    if (slice == 0 && threadIdx.x == 0) tokens[row] = best_index;
    cluster.sync();                                 // nobody leaves while its shared memory may still be read
    return;
  }
  const double temperature = (double)opt.temperature;
  auto weight = [&](int i) -> double {
    const float v = l[i];
    return isfinite(v) ? exp((double)(v - best) / temperature) : 0.0;
  };

  // every mode below needs the total weight: per thread a contiguous chunk of the slice, in vocabulary order
  const int slice_len = slice_end - slice_begin;
  const int chunk = (slice_len + kThreads - 1) / kThreads;
  const int begin = min(slice_end, slice_begin + (int)threadIdx.x * chunk), end = min(slice_end, begin + chunk);
  double mine = 0.0;
  for (int i = begin; i < end; ++i) mine += weight(i);
  const double inclusive = block_scan_f64(mine, s_sum, &slice_total);
  cluster.sync();
  double total = 0.0, before_slice = 0.0;
  for (int other = 0; other < kSlices; ++other) {
    const double t = *cluster.map_shared_rank(&slice_total, other);
    if (other < slice) before_slice += t;
    total += t;
  }

  if (is_full(opt)) {
    const double target = opt.draw * total;
    if (slice == 0 && threadIdx.x == 0) tokens[row] = target <= 0.0 ? 0 : best_index;   // unless a chunk is found
    cluster.sync();
    const double before = before_slice + inclusive - mine;
    if (target > 0.0 && end > begin && before < target && before + mine >= target) {
      double remaining = target - before;
      int hit = end - 1;
      for (int i = begin; i < end; ++i) {
        remaining -= weight(i);
        if (remaining <= 0.0) { hit = i; break; }
      }
      tokens[row] = hit;
    }
    cluster.sync();
    return;
  }

  // ---- ranked: the score of the kCandidates-th best token, by counting
  int* histogram = reinterpret_cast<int*>(overlay);                 // kBins counters (16 KB of the overlay)
  unsigned prefix = 0u;                                             // the threshold's leading bits found so far
  unsigned above = 0u;                                              // tokens whose score is above every threshold bucket
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = pass == 0 ? 20 : (pass == 1 ? 8 : 0);
    const int bins = pass == 2 ? 256 : kBins;
    const unsigned fixed_mask = pass == 0 ? 0u : (pass == 1 ? 0xfff00000u : 0xffffff00u);
    for (int i = threadIdx.x; i < kBins; i += kThreads) histogram[i] = 0;
    __syncthreads();
    for (int i = slice_begin + threadIdx.x; i < slice_end; i += kThreads) {
      const float v = l[i];
      if (!isfinite(v)) continue;
      const unsigned key = orderable(v);
      if ((key & fixed_mask) != prefix) continue;
      // scores crowd into a few bins: the lanes of a warp that hit the same bin count once, through their first lane
      const unsigned bin = (key >> shift) & (unsigned)(bins - 1);
      const unsigned same = __match_any_sync(__activemask(), bin);
      if ((int)(__ffs(same) - 1) == (int)(threadIdx.x & 31)) atomicAdd(&histogram[bin], __popc(same));
    }
    cluster.sync();
    if (slice == 0) {
      // add the slices' histograms up, then find from the top the bin in which the count reaches kCandidates
      for (int i = threadIdx.x; i < bins; i += kThreads) {
        int sum = 0;
        for (int other = 0; other < kSlices; ++other) sum += cluster.map_shared_rank(histogram, other)[i];
        reinterpret_cast<int*>(overlay + kBins * sizeof(int))[i] = sum;          // the cluster's histogram
      }
      __syncthreads();
      {
        // from the top bin down: thread t takes the bins [hi - 4 t - 3, hi - 4 t], a block-wide running sum finds the
        // bin in which the count of tokens at or above it first reaches kCandidates
        const int* all = reinterpret_cast<const int*>(overlay + kBins * sizeof(int));
        const int per_thread = kBins / kThreads;                     // 4
        int mine[kBins / kThreads];
        int sum = 0;
#pragma unroll
        for (int j = 0; j < per_thread; ++j) {
          const int bin = bins - 1 - ((int)threadIdx.x * per_thread + j);
          mine[j] = bin >= 0 ? all[bin] : 0;
          sum += mine[j];
        }
        __shared__ double all_bins;
        const double upto = block_scan_f64((double)sum, s_sum, &all_bins);      // counts: exact in a double
        unsigned running = above + (unsigned)(upto - (double)sum);              // tokens above this thread's bins
        if (threadIdx.x == 0) { select_above = above + (unsigned)all_bins - (unsigned)all[0]; select_prefix = prefix; }
        __syncthreads();
        if (running < (unsigned)kCandidates && running + (unsigned)sum >= (unsigned)kCandidates) {
#pragma unroll
          for (int j = 0; j < per_thread; ++j) {
            const int bin = bins - 1 - ((int)threadIdx.x * per_thread + j);
            if (bin < 0) break;
            if (running + (unsigned)mine[j] >= (unsigned)kCandidates) {
              select_above = running;                                 // strictly above bin `bin`
              select_prefix = prefix | ((unsigned)bin << shift);
              break;
            }
            running += (unsigned)mine[j];
          }
        }
        __syncthreads();
      }
    }
    cluster.sync();                                                  // (slice 0 has read everyone's histogram)
    prefix = *cluster.map_shared_rank(&select_prefix, 0);
    above = *cluster.map_shared_rank(&select_above, 0);
  }
  // `prefix` is now the orderable score of the threshold: fewer than kCandidates tokens score above it.  Everything
  // at or above it goes to slice 0 (if it has room: ties at the threshold may be many).
  unsigned long long* candidates = reinterpret_cast<unsigned long long*>(overlay);
  double* cumulative = reinterpret_cast<double*>(overlay + kCandidateRoom * sizeof(unsigned long long));
  // each slice collects its own candidates first (behind the places slice 0 sorts in: the upper half of the overlay),
  // then reserves a range in slice 0's list with one remote addition and copies them there
  unsigned long long* local = reinterpret_cast<unsigned long long*>(cumulative);
  __shared__ int local_count, remote_base;
  if (threadIdx.x == 0) { candidate_count = 0; local_count = 0; }
  for (int i = threadIdx.x; i < kCandidateRoom; i += kThreads) candidates[i] = 0ull;
  __syncthreads();
  for (int i0 = slice_begin; i0 < slice_end; i0 += kThreads) {
    const int i = i0 + (int)threadIdx.x;
    unsigned key = 0u;
    bool take = false;
    if (i < slice_end) {
      const float v = l[i];
      if (isfinite(v)) { key = orderable(v); take = key >= prefix; }
    }
    const unsigned takers = __ballot_sync(0xffffffffu, take);
    if (takers == 0u) continue;
    const int lane = threadIdx.x & 31;
    int base = 0;
    if (lane == 0) base = atomicAdd(&local_count, __popc(takers));
    base = __shfl_sync(0xffffffffu, base, 0);
    const int at = base + __popc(takers & ((1u << lane) - 1u));
    if (take && at < kCandidateRoom) local[at] = ((unsigned long long)key << 32) | (unsigned)(~(unsigned)i);
  }
  cluster.sync();                                                    // slice 0's list is cleared, every local list is complete
  if (threadIdx.x == 0) remote_base = atomicAdd(cluster.map_shared_rank(&candidate_count, 0), local_count);
  __syncthreads();
  {
    unsigned long long* remote = cluster.map_shared_rank(candidates, 0);
    const int count = min(local_count, kCandidateRoom);
    for (int i = threadIdx.x; i < count; i += kThreads)
      if (remote_base + i < kCandidateRoom) remote[remote_base + i] = local[i];
  }
  cluster.sync();
  const int gathered = slice == 0 ? candidate_count : 0;
  int token = -1;
  if (slice == 0 && gathered <= kCandidateRoom) {
    // sort the candidates descending (score, then lower id first); empty places hold 0 and sink to the end
    for (int size = 2; size <= kCandidateRoom; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        const int t = threadIdx.x;                                   // kCandidateRoom / 2 pairs, one per thread
        const int low = 2 * t - (t & (stride - 1)), high = low + stride;
        const bool descending = (low & size) == 0;
        const unsigned long long a = candidates[low], b = candidates[high];
        if ((a < b) == descending) { candidates[low] = b; candidates[high] = a; }
        __syncthreads();
      }
    }
    // prefix sums of the weights in rank order: two ranks per thread
    double pair[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const unsigned long long key = candidates[2 * threadIdx.x + j];
      pair[j] = key == 0ull ? 0.0 : exp((double)(from_orderable((unsigned)(key >> 32)) - best) / temperature);
    }
    __shared__ double candidates_total;
    const double upto = block_scan_f64(pair[0] + pair[1], s_sum, &candidates_total);
    cumulative[2 * threadIdx.x] = upto - pair[1];
    cumulative[2 * threadIdx.x + 1] = upto;
    __syncthreads();
    // the first rank whose cumulative weight reaches `target`, among the first `count` ranks; -1 if none does
    auto first_rank_reaching = [&](double target, int count) -> int {
      if (threadIdx.x == 0) found = -1;
      __syncthreads();
      for (int j = 0; j < 2; ++j) {
        const int rank = 2 * threadIdx.x + j;
        if (rank < count && cumulative[rank] >= target && (rank == 0 || cumulative[rank - 1] < target)) found = rank;
      }
      __syncthreads();
      const int result = found;
      __syncthreads();
      return result;
    };
    // Do the candidates decide the draw?  `everything`: no bin ever reached kCandidates, the threshold is the lowest
    // score there is and the candidates are all the row's finite tokens.
    const bool everything = prefix == 0u;
    int keep_p = gathered;                                           // ranks the nucleus keeps, if it ends in here
    bool beyond = !everything;                                       // ... or it ends beyond the candidates
    if (opt.top_p < 1.0f) {
      const double target = (double)opt.top_p * total;
      const int rank = target <= 0.0 ? 0 : first_rank_reaching(target, gathered);
      if (rank >= 0) { keep_p = rank + 1; beyond = false; }
    }
    int keep = -1;
    if (!beyond) keep = opt.top_k > 0 ? min(keep_p, opt.top_k) : keep_p;
    else if (opt.top_k > 0 && opt.top_k <= gathered) keep = opt.top_k;
    if (gathered == 0) {
      token = best_index;                                            // no finite logit
    } else if (keep > 0) {
      const double kept_total = cumulative[keep - 1];
      const double target = opt.draw * kept_total;
      int rank = target <= 0.0 ? 0 : first_rank_reaching(target, keep);
      if (rank < 0) rank = keep - 1;
      token = (int)(~(unsigned)(candidates[rank] & 0xffffffffull));
    }
  }
  // The candidates decided (slice 0 knows), or the nucleus ends beyond them and is searched for by the whole cluster;
  // what then still cannot be decided (a top_k wider than the candidates that cuts the nucleus) is left to the sort.
  if (slice == 0 && threadIdx.x == 0) {
    search_mode = token >= 0 ? 0 : (opt.top_p < 1.0f ? 1 : 2);
    if (token >= 0) tokens[row] = token;
  }
  cluster.sync();
  const int mode = *cluster.map_shared_rank(&search_mode, 0);
  cluster.sync();                                                    // (read by everyone before slice 0 goes on)
  if (mode == 0) return;
  if (mode == 1) {
    const Crossing edge = find_crossing(cluster, l, slice, slice_begin, slice_end, weight, (double)opt.top_p * total,
                                        overlay, s_sum, &crossing);
    const double edge_weight = exp((double)(from_orderable(edge.key) - best) / temperature);
    const unsigned edge_ties = ties_needed(edge.above_weight, edge_weight, edge.ties, (double)opt.top_p * total);
    const unsigned keep_p = edge.above_count + edge_ties;            // ranks the nucleus keeps
    if (opt.top_k <= 0 || (unsigned)opt.top_k >= keep_p) {
      const double kept_total = edge.above_weight + (double)edge_ties * edge_weight;
      const double target = opt.draw * kept_total;
      if (target <= 0.0) {
        if (slice == 0 && threadIdx.x == 0) tokens[row] = best_index;   // rank 0: the best score, the lowest id
        return;
      }
      const Crossing hit = find_crossing(cluster, l, slice, slice_begin, slice_end, weight, target, overlay, s_sum,
                                         &crossing);
      const double hit_weight = exp((double)(from_orderable(hit.key) - best) / temperature);
      const unsigned nth = ties_needed(hit.above_weight, hit_weight, hit.ties, target);   // 1-based, in id order
      // the nth token (ascending id) whose score is exactly hit.key: per thread a contiguous chunk of the slice
      int held = 0;
      for (int i = begin; i < end; ++i) {
        const float v = l[i];
        held += (isfinite(v) && orderable(v) == hit.key) ? 1 : 0;
      }
      const double held_upto = block_scan_f64((double)held, s_sum, &slice_total);    // counts: exact in a double
      cluster.sync();
      double held_before = held_upto - (double)held;
      for (int other = 0; other < slice; ++other) held_before += *cluster.map_shared_rank(&slice_total, other);
      if ((double)nth > held_before && (double)nth <= held_before + (double)held) {
        unsigned remaining = nth - (unsigned)held_before;
        for (int i = begin; i < end; ++i) {
          const float v = l[i];
          if (isfinite(v) && orderable(v) == hit.key && --remaining == 0u) { tokens[row] = i; break; }
        }
      }
      cluster.sync();                                                // nobody leaves while its totals may still be read
      return;
    }
  }
  if (slice != 0) return;

  // ---- the whole vocabulary, sorted in the caller's scratch
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
  int keep = vocab;
  if (opt.top_p < 1.0f)
    keep = first_reaching(ranked_weight, vocab, (double)opt.top_p * total, chunk_sums, &found, vocab - 1) + 1;
  if (opt.top_k > 0) keep = min(keep, opt.top_k);
  double kept = 0.0;
  for (int i = threadIdx.x; i < keep; i += kThreads) kept += ranked_weight(i);
  const double kept_total = block_sum_f64(kept, s_sum);
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

// best_value / best_index [rows][best_count] (or null): per row, candidates among which its largest finite logit is,
// as the output head's kernel leaves them (every finite logit is <= the candidate of its group of columns).
MIR_EXPORT int mir_sample(const float* logits, long long ld, int rows, int vocab, const void* options,
                          void* sort_keys, long long sort_keys_capacity, int needs_ranked, int* tokens,
                          const float* best_value, const int* best_index, int best_count, cudaStream_t stream) {
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
                    tokens, best_count > 0 && best_index != nullptr ? best_value : (const float*)nullptr, best_index,
                    best_count);
}

MIR_EXPORT int mir_repetition_penalty(float* logits, long long ld, int vocab, const int* ids, const int* id_rows,
                                      const float* penalties, int count, cudaStream_t stream) {
  if (count == 0) return MIR_OK;
  penalty_kernel<<<(count + 255) / 256, 256, 0, stream>>>(logits, (size_t)ld, vocab, ids, id_rows, penalties, count);
  return mir_check_launch("repetition_penalty");
}
