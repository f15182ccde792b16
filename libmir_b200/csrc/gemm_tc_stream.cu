// bf16 matrix products for FEW rows (1 to 128 tokens: decode steps and short portions) on tcgen05, built to
// stream the weights at memory speed:
//
//   out[M, N] = epilogue(x[M, K] . w[N, K]^T)
//
// The roles of the operands are swapped against the many-rows kernel: a tile of 128 weight rows is the A operand
// (M = 128 of the instruction), the tokens are the B operand (N = tokens rounded up to 16), so the tensor cores
// are fed whole 16 KB boxes of weights and a few hundred bytes of activations per step, and the accumulator
// D[128 features, tokens] in tensor memory is the transposed output tile.
//
//   producer   one thread: per 64-wide step of K one TMA box of weights (128 rows x 64; with the SwiGLU epilogue 64
//              gate rows and the 64 up rows that belong to them) and one of activations into a ring of stages.
//   issuer     one warp that stays converged, the products predicated on its elected lane, the ring's stage counted
//              (tcgen05.cuh says why): four tcgen05.mma (128 x tokens x 16) per stage, tcgen05.commit frees the stage.
//   epilogue   four warps: read the accumulator (lane = feature), transpose it through shared memory.
//
// K is cut over a cluster of 1, 2, 4 or 8 CTAs so that up to 444 CTAs run whatever the shape (three fit on an SM;
// what counts is that together they keep enough bytes in flight, not how they spread over the SMs).  Each
// CTA of the cluster then finishes a share of the tokens: it adds the partial tiles over distributed shared
// memory in rank order and applies the epilogue: store bf16 / accumulate into the 32-bit residual / 32-bit store / SwiGLU, bias, and the two halves
// of a folded RMSNorm (scale each token's results by rsqrt(mean of squares + eps) of its input; leave the sums
// of squares and the weighted bf16 copy of the rows it updates).  Waits on mbarriers are bounded in time.
// libmir takes these products from a library (cuda/src/backend/linear/mod.rs:141-194).
#include <algorithm>
#include <cfloat>
#include <cooperative_groups.h>
#include "tcgen05.cuh"
#include "trace.cuh"

namespace cg = cooperative_groups;
using namespace mir;
using namespace mir::tc;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kStepK = 64;
constexpr int kWeightBytes = 128 * 128;     // a stage's weights: 128 rows of 128 bytes
constexpr int kMaxStages = 8;
constexpr int kThreads = 6 * 32;            // producer warp, issuer warp, four epilogue warps
constexpr int kRingBytes = 72 * 1024;       // per CTA, so that three CTAs fit on an SM
int g_ring_bytes = kRingBytes;               // for measurements
enum Epilogue : int { STORE = 0, ACCUM = 1, F32 = 2, SWIGLU = 3 };

__device__ int g_tc_stream_error = 0;
// time stamps (trace.cuh) of the first and the last CTA of a launch: 0 start, 1 the ring's first weights are asked
// for, 2 the kernel before is over, 3 the activations are asked for, 4 the first stage has landed, 5 the last one,
// 6 the products are over, 7 after the first cluster barrier, 8 results written, 9 after the second barrier;
// tag = 2 x epilogue + (0 first CTA, 1 last)
MIR_TRACE_DEFINE(stream)

struct StreamNorm {
  const float* sumsq;        // consumer: [sumsq_tiles][kNormStatStride] partial sums of squares of x's rows before weighting
  int sumsq_tiles;
  float eps;
  float* sumsq_out;          // producer (ACCUM): [ceil(n / 16)][kNormStatStride] partial sums of squares of the rows it updates
  const float* next_weight;  // producer: [n] weight of the norm that follows, or null
  bf16* weighted_out;        // producer: [m, ld_weighted] bf16(new residual * next_weight)
  int ld_weighted;
  float* best_value;         // float32 epilogue (the output head): [m][best_stride] the largest finite result of every
  int* best_index;           //   32 columns (entry 4 x tile + warp) and its column, ties to the lower column; or null
  int best_stride;
};

// (Shared memory lets three CTAs share an SM; the registers are capped as if six did: 56 instead of up to 95 per
// thread, no spills, and the captured decode step at Qwen3-4B sizes takes 2.621 instead of 2.638 ms at batch 8,
// 2.226 instead of 2.241 ms at batch 1.)
template <int MODE>
__global__ void __launch_bounds__(kThreads, 6)
tc_stream_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                 const void* __restrict__ bias, void* __restrict__ out, int ldo, int m, int n, int k, int up_offset,
                 int tokens, int tile_rows, int stages, int stage_stride, uint32_t tmem_columns, StreamNorm norm) {
  grid_launch_dependents();
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long barriers[2 * kMaxStages + 1];
  __shared__ uint32_t tmem_base_slot;
  __shared__ float scale[kNormStatStride];
  cg::cluster_group cluster = cg::this_cluster();
  const int splits = gridDim.y, split = blockIdx.y;           // the cluster spans gridDim.y
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // tile_rows output features per CTA (128, 64 or 32; with the SwiGLU epilogue 64 gate and 64 up rows).  The A
  // operand always spans 128 rows of shared memory: rows beyond the tile hold whatever was there, and the
  // accumulator rows they produce are never read.
  const int n0 = blockIdx.x * tile_rows;
  const uint32_t weight_bytes = (MODE == SWIGLU ? 128u : (uint32_t)tile_rows) * 128u;
  const int total_steps = (k + kStepK - 1) / kStepK;
  const int per_split = (total_steps + splits - 1) / splits;
  const int step_begin = split * per_split;
  const int my_steps = max(0, min(total_steps, step_begin + per_split) - step_begin);
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t full0 = smem_u32(&barriers[0]), empty0 = smem_u32(&barriers[kMaxStages]);
  const uint32_t done = smem_u32(&barriers[2 * kMaxStages]);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      barrier_init(full0 + 8 * s, 1);
      barrier_init(empty0 + 8 * s, 1);
    }
    barrier_init(done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(tmem_columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tensor_fence_before_sync();
  __syncthreads();
  tensor_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  MIR_TRACE_BEGIN(stream, (blockIdx.x == 0 && blockIdx.y == 0) || (blockIdx.x == gridDim.x - 1 && blockIdx.y == gridDim.y - 1),
                  2 * MODE + (blockIdx.x == 0 && blockIdx.y == 0 ? 0 : 1))
  if (threadIdx.x == 0) MIR_TRACE_POINT(stream, 0);

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      const uint32_t stage_bytes = weight_bytes + (uint32_t)tokens * 128u;
      auto load_weights = [&](int i, uint32_t barrier, uint32_t dst) {
        const int k0 = (step_begin + i) * kStepK;
        barrier_expect_bytes(barrier, stage_bytes);
        tma_load_2d(dst, &w_map, barrier, k0, n0);
        if (MODE == SWIGLU) tma_load_2d(dst + kWeightBytes / 2, &w_map, barrier, k0, up_offset + n0);
      };
      // The weights belong to no kernel: the whole ring is filled with them before this kernel waits for the one
      // before it, whose results are only the activations.  Launched with programmatic stream serialization, the
      // CTA becomes resident while that kernel still runs (if its CTAs leave the shared memory), and its first
      // products can start the moment the activations exist.
      const int ahead = min(stages, my_steps);
      for (int i = 0; i < ahead; ++i)
        load_weights(i, full0 + 8 * i, smem_base + (uint32_t)i * (uint32_t)stage_stride);
      MIR_TRACE_POINT(stream, 1);
      grid_dependency_wait();
      MIR_TRACE_POINT(stream, 2);
      for (int i = 0; i < ahead; ++i)
        tma_load_2d(smem_base + (uint32_t)i * (uint32_t)stage_stride + weight_bytes, &x_map, full0 + 8 * i,
                    (step_begin + i) * kStepK, 0);
      MIR_TRACE_POINT(stream, 3);
      // (the stage and its parity are counted, not divided: `ahead` stages are filled, so step `ahead` takes stage
      // ahead % stages = 0 when the ring was filled, in its second turn)
      int stage = ahead == stages ? 0 : ahead;
      uint32_t parity = ahead == stages ? 1u : 0u;
      for (int i = ahead; i < my_steps; ++i) {
        if (!wait_barrier(empty0 + 8 * stage, parity ^ 1u)) { g_tc_stream_error = 1; break; }
        const uint32_t barrier = full0 + 8 * stage;
        const uint32_t dst = smem_base + (uint32_t)stage * (uint32_t)stage_stride;
        load_weights(i, barrier, dst);
        tma_load_2d(dst + weight_bytes, &x_map, barrier, (step_begin + i) * kStepK, 0);
        if (++stage == stages) { stage = 0; parity ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ issuer: the whole warp stays converged, the
    // products are predicated on the elected lane and take their descriptors as 32-bit halves (tcgen05.cuh); the
    // stage and its parity are counted, not divided
    {
      const uint32_t idesc = instruction_descriptor(128, tokens);
      const uint32_t elected = elect_one();
      const uint32_t a_low0 = operand_low(smem_base), b_low0 = operand_low(smem_base + weight_bytes);
      const uint32_t stage_step = (uint32_t)stage_stride >> 4;
      bool alive = true;
      uint32_t stage = 0, parity = 0;
      for (int i = 0; i < my_steps; ++i) {
        if (alive && !wait_barrier(full0 + 8 * stage, parity)) { g_tc_stream_error = 2; alive = false; }
        if (elected && i == 0) MIR_TRACE_POINT(stream, 4);
        if (elected && i == my_steps - 1) MIR_TRACE_POINT(stream, 5);
        tensor_fence_after_sync();
        const uint32_t a_low = a_low0 + stage * stage_step, b_low = b_low0 + stage * stage_step;
        mma_bf16_ss_halves(tmem_base, a_low, b_low, idesc, i > 0 ? 1u : 0u, elected);
#pragma unroll
        for (int kk = 1; kk < kStepK / 16; ++kk)
          mma_bf16_ss_halves<true>(tmem_base, a_low + 2u * kk, b_low + 2u * kk, idesc, elected);
        mma_commit_elected(empty0 + 8 * stage, elected);
        if (++stage == (uint32_t)stages) { stage = 0; parity ^= 1u; }
      }
      mma_commit_elected(done, elected);
    }
  }
  // ---------------------------------------------------------------------- the tile, transposed, into shared memory
  // (the ring is free once `done` has completed: every box has landed and every product has read it)
  float* tile = reinterpret_cast<float*>(smem);               // [tokens][128]
  constexpr int BATCH = 4;                                    // tokens whose loads are in flight together
  float old_first[BATCH] = {0.0f, 0.0f, 0.0f, 0.0f};          // ACCUM: the residual under this thread's first tokens
  float extra = 0.0f, next_weight = 0.0f;                     // this thread's column of the bias and of the next norm's weight
  if (warp >= 2) {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                      // feature row of the tile = accumulator lane
    const int tid = threadIdx.x - 64;                         // 0..127
    // While the products run: what the epilogue needs from earlier kernels.  Per token 1, or the folded norm's
    // rsqrt(mean of squares + eps) (8 threads per token add the tiles' sums); and the old residual values.
    grid_dependency_wait();
    if (tid < kNormStatStride) scale[tid] = 1.0f;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (norm.sumsq != nullptr) {
      const int token = tid >> 2, part = tid & 3;              // 4 threads per token, 32 tokens
      float sum = 0.0f;
      if (token < m)
        for (int t = part; t < norm.sumsq_tiles; t += 4) sum += norm.sumsq[t * kNormStatStride + token];
#pragma unroll
      for (int o = 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (part == 0) scale[token] = rsqrtf(sum / (float)k + norm.eps);
    }
    if (MODE != SWIGLU && tid < tile_rows && n0 + tid < n) {
      if (bias != nullptr)
        extra = MODE == STORE ? __bfloat162float(reinterpret_cast<const bf16*>(bias)[n0 + tid])
                              : reinterpret_cast<const float*>(bias)[n0 + tid];
      if (MODE == ACCUM && norm.weighted_out != nullptr) next_weight = norm.next_weight[n0 + tid];
    }
    if (MODE == ACCUM && tid < tile_rows && n0 + tid < n) {
#pragma unroll
      for (int j = 0; j < BATCH; ++j) {
        const int token = split + j * splits;
        if (token < m) old_first[j] = reinterpret_cast<const float*>(out)[(size_t)token * ldo + n0 + tid];
      }
    }
    const bool alive = wait_barrier(done, 0);
    if (tid == 0) MIR_TRACE_POINT(stream, 6);
    if (!alive) g_tc_stream_error = 3;
    tensor_fence_after_sync();
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
    for (int c0 = 0; c0 < tokens; c0 += 16) {
      float v[16];
      tmem_load_16(lane_base + c0, v);
#pragma unroll
      for (int i = 0; i < 16; ++i) tile[(size_t)(c0 + i) * 128 + row] = (alive && my_steps > 0) ? v[i] : 0.0f;
    }
    tensor_fence_before_sync();
  }
  cluster.sync();                                             // every CTA's partial tile is in its shared memory
  if (threadIdx.x == 64) MIR_TRACE_POINT(stream, 7);
  if (warp == 1) {                                            // (the accumulator has been read out)
    tensor_fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_columns) : "memory");
  }
  // The peers keep their shared memory until it was read: every thread arrives at a second cluster barrier as soon
  // as its last remote values are in registers, before it writes its results, and waits for it at the very end.
  // The arrival orders nothing in memory (what it guards are loads that have returned), so it is a relaxed one: a
  // releasing arrival cost 0.06 ms of a 2.56 ms decode step.
  bool arrived = false;
  // Every CTA of the cluster finishes a share of the tokens (token = split, split + splits, ...): it adds the
  // cluster's partial tiles over distributed shared memory in rank order and applies the epilogue.
  if (warp >= 2) {
    const int tid = threadIdx.x - 64;                         // 0..127
    const float* peers[8];
#pragma unroll
    for (int rank = 0; rank < 8; ++rank) peers[rank] = cluster.map_shared_rank(tile, rank < splits ? rank : 0);
    auto cluster_sum = [&](int token, int row) {
      float parts[8];
#pragma unroll
      for (int rank = 0; rank < 8; ++rank) parts[rank] = rank < splits ? peers[rank][(size_t)token * 128 + row] : 0.0f;
      float total = parts[0];
#pragma unroll
      for (int rank = 1; rank < 8; ++rank) total += parts[rank];
      return total;
    };
    // four tokens at a time, so that their loads (partial tiles, the old residual) are in flight together
    if (MODE == SWIGLU) {
      // 64 features per tile: the two halves of the threads take alternate tokens of this CTA's share
      const int feature = tid & 63, column = n0 + feature;
      const int stride = 2 * splits;
      for (int token0 = split + splits * (tid >> 6); token0 < m; token0 += BATCH * stride) {
        float gate[BATCH], up[BATCH];
#pragma unroll
        for (int j = 0; j < BATCH; ++j) {
          const int token = token0 + j * stride;
          gate[j] = token < m ? cluster_sum(token, feature) : 0.0f;
          up[j] = token < m ? cluster_sum(token, 64 + feature) : 0.0f;
        }
        if (token0 + BATCH * stride >= m) {                   // this thread's last reads of its peers' tiles are over
          asm volatile("" ::"f"(gate[0]), "f"(gate[1]), "f"(gate[2]), "f"(gate[3]), "f"(up[0]), "f"(up[1]), "f"(up[2]), "f"(up[3]) : "memory");
          asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory");
          arrived = true;
        }
#pragma unroll
        for (int j = 0; j < BATCH; ++j) {
          const int token = token0 + j * stride;
          if (token < m && column < n) {
            const float s = token < kNormStatStride ? scale[token] : 1.0f;
            const float g = gate[j] * s;
            reinterpret_cast<bf16*>(out)[(size_t)token * ldo + column] = __float2bfloat16_rn(g / (1.0f + __expf(-g)) * (up[j] * s));
          }
        }
      }
    } else {
      const int column = n0 + tid;
      const bool in_range = tid < tile_rows && column < n;
      for (int token0 = split; token0 < m; token0 += BATCH * splits) {
        float value[BATCH], old[BATCH];
#pragma unroll
        for (int j = 0; j < BATCH; ++j) {
          const int token = token0 + j * splits;
          value[j] = (token < m && in_range) ? cluster_sum(token, tid) : 0.0f;
          old[j] = token0 == split ? old_first[j]
                   : ((MODE == ACCUM && token < m && in_range) ? reinterpret_cast<const float*>(out)[(size_t)token * ldo + column] : 0.0f);
        }
        if (token0 + BATCH * splits >= m) {                   // this thread's last reads of its peers' tiles are over
          asm volatile("" ::"f"(value[0]), "f"(value[1]), "f"(value[2]), "f"(value[3]) : "memory");
          asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory");
          arrived = true;
        }
#pragma unroll
        for (int j = 0; j < BATCH; ++j) {
          const int token = token0 + j * splits;
          if (token >= m) break;                              // the same for every thread
          const float result = value[j] * (token < kNormStatStride ? scale[token] : 1.0f) + extra + old[j];
          if (in_range) {
            if (MODE == STORE) {
              reinterpret_cast<bf16*>(out)[(size_t)token * ldo + column] = __float2bfloat16_rn(result);
            } else {
              reinterpret_cast<float*>(out)[(size_t)token * ldo + column] = result;
              if (MODE == ACCUM && norm.weighted_out != nullptr)
                norm.weighted_out[(size_t)token * norm.ld_weighted + column] = __float2bfloat16_rn(result * next_weight);
            }
          }
          if (MODE == F32 && norm.best_value != nullptr) {
            // The head's logits: what a sampler asks first is each row's largest one.  Every warp leaves the best of
            // its 32 columns, so that the sampling kernel looks at V / 32 candidates instead of V logits.
            const bool counts = in_range && isfinite(result);
            float best = counts ? result : -FLT_MAX;
            int best_column = counts ? column : 0x7fffffff;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
              const float other = __shfl_xor_sync(0xffffffffu, best, o);
              const int other_column = __shfl_xor_sync(0xffffffffu, best_column, o);
              if (other > best || (other == best && other_column < best_column)) { best = other; best_column = other_column; }
            }
            if ((tid & 31) == 0) {
              const size_t at = (size_t)token * norm.best_stride + blockIdx.x * 4 + (tid >> 5);
              norm.best_value[at] = best;
              norm.best_index[at] = best_column;
            }
          }
          if (MODE == ACCUM && norm.sumsq_out != nullptr && token < kNormStatStride) {
            // sum of squares of 16 neighbouring new residual values of this token (16 consecutive lanes)
            float square = in_range ? result * result : 0.0f;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) square += __shfl_xor_sync(0xffffffffu, square, o);
            if ((tid & 15) == 0 && in_range) norm.sumsq_out[(size_t)(column >> 4) * kNormStatStride + token] = square;
          }
        }
      }
    }
  }
  if (threadIdx.x == 64) MIR_TRACE_POINT(stream, 8);
  if (!arrived) asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
  if (threadIdx.x == 64) MIR_TRACE_POINT(stream, 9);
}

int g_forced_splits = 0;                                      // for measurements: 0 = choose

int g_forced_rows = 0;

// Tile height and how many CTAs share K.  Measured on B200 (8 rows, inside a CUDA graph, us): whole 128-row tiles
// beat 64- and 32-row tiles at every shape (QKV 9.0 / 15.5 / 18.1, output projection 7.7 / 10.5 / 11.5), and K is
// best cut as far as one wave of CTAs allows (three fit on an SM): output projection 7.7 with 8 CTAs per tile,
// 10.4 with 4, 16.8 with 2.
void choose_shape(int n, int total_steps, bool swiglu, int* tile_rows, int* splits) {
  const int rows = swiglu ? 64 : 128;
  const int tiles = (n + rows - 1) / rows;
  int s = 1;
  while (s < 8 && tiles * s * 2 <= 3 * 148 && total_steps / (s * 2) >= 4) s *= 2;
  *tile_rows = rows;
  *splits = s;
}

template <int MODE>
int launch(const void* x, int ldx, const void* w, const void* bias, void* out, int ldo, int m, int n, int k,
           int up_offset, const StreamNorm& norm, cudaStream_t stream) {
  const int tokens = (m + 15) / 16 * 16;
  const int total_steps = (k + kStepK - 1) / kStepK;
  int tile_rows, splits;
  choose_shape(n, total_steps, MODE == SWIGLU, &tile_rows, &splits);
  if (g_forced_splits > 0) splits = g_forced_splits;
  if (g_forced_rows > 0 && MODE != SWIGLU) tile_rows = g_forced_rows;
  CUtensorMap w_map, x_map;
  int status = tensor_map_for(w, MODE == SWIGLU ? up_offset + n : n, k, k, tile_rows, &w_map);
  if (status != MIR_OK) return status;
  status = tensor_map_for(x, m, k, ldx, tokens, &x_map);
  if (status != MIR_OK) return status;
  const int weight_bytes = (MODE == SWIGLU ? 128 : tile_rows) * 128;
  const int stage_stride = (weight_bytes + tokens * 128 + 1023) / 1024 * 1024;
  const int tile_bytes = tokens * 128 * 4;                    // the transposed tile reuses the ring
  int stages = std::max(2, std::min(kMaxStages, g_ring_bytes / stage_stride));
  while (stages * stage_stride < tile_bytes) ++stages;
  // the A operand of the last stage reads 128 rows whatever the tile's height: room for that behind the ring
  const size_t smem = (size_t)stages * stage_stride + std::max(0, kWeightBytes - stage_stride) + 1024;
  static bool configured = false;
  if (!configured) {
    const cudaError_t err = cudaFuncSetAttribute(tc_stream_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 208 * 1024);
    if (err != cudaSuccess) {
      mir_set_error("tc_stream: cannot reserve shared memory: %s", cudaGetErrorString(err));
      return MIR_CUDA_ERROR;
    }
    configured = true;
  }
  const int tiles = (n + tile_rows - 1) / tile_rows;
  uint32_t tmem_columns = 32;
  while ((int)tmem_columns < tokens) tmem_columns *= 2;
  return mir_launch_with(mir_pdl_for_streaming(), "tc_stream", tc_stream_kernel<MODE>, dim3(tiles, splits), dim3(kThreads), smem, stream, splits, w_map,
                    x_map, bias, out, ldo, m, n, k, up_offset, tokens, tile_rows, stages, stage_stride, tmem_columns, norm);
}

}  // namespace

MIR_EXPORT int mir_gemm_tc_stream_error() {
  int flag = 0;
  if (cudaMemcpyFromSymbol(&flag, g_tc_stream_error, sizeof(int)) != cudaSuccess) return -1;
  return flag;
}

MIR_EXPORT int mir_gemm_tc_stream_max_rows() { return 128; }

// For measurements: 1, 2, 4 or 8 CTAs per cluster, the ring's size in KB, the tile's height (0: the launcher chooses).
MIR_EXPORT int mir_gemm_tc_stream_set_splits(int splits, int ring_kb, int tile_rows) {
  if ((splits != 0 && splits != 1 && splits != 2 && splits != 4 && splits != 8) || ring_kb < 32 || ring_kb > 200 ||
      (tile_rows != 0 && tile_rows != 32 && tile_rows != 64 && tile_rows != 128)) {
    mir_set_error("tc_stream: splits must be 0, 1, 2, 4 or 8, the ring 32..200 KB, the tile 0, 32, 64 or 128 rows");
    return MIR_BAD_ARGUMENT;
  }
  g_forced_splits = splits;
  g_forced_rows = tile_rows;
  g_ring_bytes = ring_kb * 1024;
  return MIR_OK;
}

// mode: 0 store bf16 (+ bf16 bias), 1 accumulate into float (+ float bias), 2 float (+ float bias), 3 SwiGLU (w =
// [gate rows; up rows], up rows start at up_offset, n = output columns).  sumsq / sumsq_tiles / eps: x is a folded
// norm's weighted rows and every token's results are scaled by rsqrt(sum of its partial sums / k + eps) (store and
// SwiGLU).  sumsq_out / next_weight / weighted_out: the accumulate epilogue also leaves the partial sums of squares
// of the rows it updates and those rows times next_weight as bf16.  1 <= m <= 128, k and ldx multiples of 8, x and
// w 16-byte aligned.  The sums of squares and the weighted rows are defined for up to kNormStatStride (32) tokens.
MIR_EXPORT int mir_gemm_tc_stream_bf16(int mode, const void* x, int ldx, const void* w, const void* bias, void* out,
                                       int ldo, int m, int n, int k, int up_offset, const float* sumsq,
                                       int sumsq_tiles, float eps, float* sumsq_out, const float* next_weight,
                                       void* weighted_out, int ld_weighted, cudaStream_t stream) {
  if (m == 0 || n == 0) return MIR_OK;
  if (m < 0 || m > 128 || n < 0 || k <= 0 || (k % 8) || ldo < n || ((uintptr_t)w & 15) || (ldx % 8) || ldx < k ||
      ((uintptr_t)x & 15) || x == nullptr) {
    mir_set_error("tc_stream: needs 1..128 rows, k and the row stride multiples of 8 and 16-byte aligned operands "
                  "(m %d n %d k %d ldx %d ldo %d)", m, n, k, ldx, ldo);
    return MIR_BAD_ARGUMENT;
  }
  if ((sumsq_out != nullptr || weighted_out != nullptr) && (mode != ACCUM || m > kNormStatStride)) {
    mir_set_error("tc_stream: sums of squares and weighted rows are written by the accumulate epilogue for up to %d rows",
                  kNormStatStride);
    return MIR_BAD_ARGUMENT;
  }
  if (sumsq != nullptr && (sumsq_tiles <= 0 || m > kNormStatStride || (mode != STORE && mode != SWIGLU))) {
    mir_set_error("tc_stream: a folded norm needs its partial sums, up to %d rows, and the store or SwiGLU epilogue",
                  kNormStatStride);
    return MIR_BAD_ARGUMENT;
  }
  if (weighted_out != nullptr && (next_weight == nullptr || sumsq_out == nullptr || ld_weighted < n)) {
    mir_set_error("tc_stream: weighted rows need the next norm's weight, a row stride >= n, and sums of squares");
    return MIR_BAD_ARGUMENT;
  }
  StreamNorm norm;
  norm.sumsq = sumsq;
  norm.sumsq_tiles = sumsq_tiles;
  norm.eps = eps;
  norm.sumsq_out = sumsq_out;
  norm.next_weight = next_weight;
  norm.weighted_out = (bf16*)weighted_out;
  norm.ld_weighted = ld_weighted;
  norm.best_value = nullptr;
  norm.best_index = nullptr;
  norm.best_stride = 0;
  switch (mode) {
    case STORE: return launch<STORE>(x, ldx, w, bias, out, ldo, m, n, k, 0, norm, stream);
    case ACCUM: return launch<ACCUM>(x, ldx, w, bias, out, ldo, m, n, k, 0, norm, stream);
    case F32: return launch<F32>(x, ldx, w, bias, out, ldo, m, n, k, 0, norm, stream);
    case SWIGLU:
      if (bias) { mir_set_error("tc_stream: the SwiGLU epilogue takes no bias"); return MIR_BAD_ARGUMENT; }
      return launch<SWIGLU>(x, ldx, w, nullptr, out, ldo, m, n, k, up_offset, norm, stream);
  }
  mir_set_error("tc_stream: unknown mode %d", mode);
  return MIR_BAD_ARGUMENT;
}

// Entries per row that mir_gemm_tc_stream_head_bf16 leaves for n output columns: four per tile of 128 columns.
MIR_EXPORT int mir_gemm_tc_stream_head_candidates(int n) { return n <= 0 ? 0 : (n + 127) / 128 * 4; }

// The output head: the float32 epilogue (out[m, n] = x . w^T), which also leaves, per row, the largest finite logit of every 32 columns and its column (ties to the lower column) in
// best_value / best_index [m][best_stride], best_stride >= mir_gemm_tc_stream_head_candidates(n): the sampling kernel
// finds a row's largest logit among these instead of among all n.
MIR_EXPORT int mir_gemm_tc_stream_head_bf16(const void* x, int ldx, const void* w, void* out, int ldo, int m, int n, int k,
                                            float* best_value, int* best_index, int best_stride, cudaStream_t stream) {
  if (m == 0 || n == 0) return MIR_OK;
  if (m < 0 || m > 128 || n < 0 || k <= 0 || (k % 8) || ldo < n || ((uintptr_t)w & 15) || (ldx % 8) || ldx < k ||
      ((uintptr_t)x & 15) || x == nullptr || best_value == nullptr || best_index == nullptr ||
      best_stride < mir_gemm_tc_stream_head_candidates(n) || g_forced_rows != 0) {
    mir_set_error("tc_stream: the head needs 1..128 rows, k and the row stride multiples of 8, 16-byte aligned operands "
                  "and room for %d candidates per row (m %d n %d k %d ldx %d ldo %d stride %d)",
                  mir_gemm_tc_stream_head_candidates(n), m, n, k, ldx, ldo, best_stride);
    return MIR_BAD_ARGUMENT;
  }
  StreamNorm norm;
  norm.sumsq = nullptr;
  norm.sumsq_tiles = 0;
  norm.eps = 0.0f;
  norm.sumsq_out = nullptr;
  norm.next_weight = nullptr;
  norm.weighted_out = nullptr;
  norm.ld_weighted = 0;
  norm.best_value = best_value;
  norm.best_index = best_index;
  norm.best_stride = best_stride;
  return launch<F32>(x, ldx, w, nullptr, out, ldo, m, n, k, 0, norm, stream);
}
