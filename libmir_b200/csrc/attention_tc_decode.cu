// Attention of single decoded tokens over the paged cache on the 5th-generation tensor cores (tcgen05), head_dim
// 128, bf16, split over the keys:
//
//   out[h] = softmax_j(scale q_h . k_j) v_j     over the keys j <= position (and inside the window, if any)
//
// A CTA takes one request, one KV head (all query heads of its group, up to 16) and one partition of the keys, and
// walks over the partition in tiles of 128 keys.  The products are transposed so that the 128 keys (then the 128
// elements of the head) are the M side of the tensor cores and the handful of query heads the N side (16):
//
//   S^T = K Q^T     A = the key tile as the cache stores it (rows of keys, K-major), B = the group's queries,
//                   accumulator [128 keys, 16 heads] in tensor memory;
//   P^T = exp2(scale S^T - m)   one key per softmax thread (tcgen05.ld of its lane), the maximum over the 128 keys by
//                   warp reductions and one exchange through shared memory, written as bf16 into shared memory in
//                   the layout of a B operand;
//   O^T += V^T P^T  A = the value tile as the cache stores it (MN-major: nothing is transposed), accumulator
//                   [128 elements, 16 heads] in tensor memory for the whole partition.
//
// Keys and values arrive as one TMA box per page and 64-wide half of the head (cp.async.bulk.tensor.2d through a
// tensor map over the cache, 128-byte swizzle), issued by one warp; a page the block table does not have (-1:
// released by a window) or that lies beyond the context is fetched from outside the tensor (a negative row), where
// TMA writes zeros: no address is ever formed from such an entry, and nothing stale stays in shared memory.  One
// thread issues the products.  A CTA holds one key tile and one value tile (64 KB), three CTAs share an SM: while
// one waits for its tiles the others compute.  The partitions' results (unnormalised O, maximum, denominator) go to
// the caller's scratch in the layout of the mma.sync kernel and are merged by the same merge kernel.
// Masked keys get probability 0 by selection, never by arithmetic on what the cache holds there.
// Every mbarrier wait is bounded in time; a role whose wait runs out raises g_tc_decode_error and stops waiting,
// the CTA still frees its tensor memory and returns.
// libmir splits decode attention over the keys on CUDA cores and wmma
// (cuda/kernels/paged_attention_batch_split_bf16.cu); the formula as the Metal engine states it is
// metal/src/engine/dense/swiglu/attention.rs:93-107.
#include <algorithm>
#include "tcgen05.cuh"
#include "launchers.h"
#include "trace.cuh"

using namespace mir;
using namespace mir::tc;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kKeys = 128;                  // keys per tile
constexpr int kDim = 128;                   // head_dim
constexpr int kHeads = 16;                  // query heads one CTA serves (the N side of both products)
constexpr int kHalf = 128 * 128;            // bytes of a 128-row x 64-element half tile
constexpr int kTile = 2 * kHalf;            // 32 KB
constexpr int kSmallHalf = kHeads * 128;    // bytes of a 16-row x 64-element half of Q or P^T
constexpr int kOffK = 0, kOffV = kTile, kOffQ = 2 * kTile, kOffP = 2 * kTile + 2 * kSmallHalf;
constexpr int kSmemBytes = 2 * kTile + 4 * kSmallHalf + 1024;
constexpr int kSoftmaxThreads = 128;
constexpr int kThreads = kSoftmaxThreads + 64;   // four softmax warps, the loader, the issuer
constexpr uint32_t kTmemColumns = 32;       // S^T at 0, O^T at 16
constexpr float kRescaleThreshold = 8.0f;   // log2 of how far a tile's maximum may exceed the running one

enum { K_FULL = 0, K_FREE, V_FULL, V_FREE, S_FULL, P_READY, Q_READY, O_DONE, BARRIERS };

__device__ int g_tc_decode_error = 0;
// time stamps (trace.cuh) of the grid's first CTA and of the last row's last live partition: 0 start, 1 set up,
// 2 loader: first loads may go, 3 softmax: the kernel before is over, 4 issuer: the queries are in shared memory,
// 5 first scores issued, 6 first scores there, 7 first P written, 8 last scores there, 9 last P written, 10 last
// product over, 11 results written, 12 end; value = tiles of the CTA; tag 200 first CTA, 201 the other
MIR_TRACE_DEFINE(decode)

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// N consecutive accumulator columns of this thread's lane.
template <int N> __device__ __forceinline__ void tmem_load(uint32_t address, float (&v)[N]);
template <> __device__ __forceinline__ void tmem_load<4>(uint32_t address, float (&v)[4]) {
  uint32_t r[4];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(address)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(r[i]);
}
template <> __device__ __forceinline__ void tmem_load<8>(uint32_t address, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(address)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
template <> __device__ __forceinline__ void tmem_load<16>(uint32_t address, float (&v)[16]) { tmem_load_16(address, v); }

template <int N> __device__ __forceinline__ void tmem_store(uint32_t address, const float (&v)[N]);
template <> __device__ __forceinline__ void tmem_store<4>(uint32_t address, const float (&v)[4]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(address),
               "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
               "r"(__float_as_uint(v[3]))
               : "memory");
}
template <> __device__ __forceinline__ void tmem_store<8>(uint32_t address, const float (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(address),
               "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
               "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
               "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7]))
               : "memory");
}
template <> __device__ __forceinline__ void tmem_store<16>(uint32_t address, const float (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(address),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
      "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
      "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
      "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
      "r"(__float_as_uint(v[15]))
      : "memory");
}

// Byte offset of element (row, column) of a [16 rows, 128 columns] bf16 operand stored K-major as two halves of 64
// columns, each row 128 bytes, with the 128-byte swizzle (16-byte chunk index xor row mod 8).
__device__ __forceinline__ uint32_t small_operand_offset(int row, int column) {
  const int half = column >> 6, within = column & 63;
  return (uint32_t)(half * kSmallHalf + row * 128 + ((((within >> 3) ^ (row & 7))) << 4) + (within & 7) * 2);
}

// G: how many columns of the accumulators the softmax threads touch (the group's heads rounded up to 4, 8 or 16).
template <int G>
__global__ void __launch_bounds__(kThreads)
tc_decode_attention_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                           const __grid_constant__ CUtensorMap k_tile_map,
                           const __grid_constant__ CUtensorMap v_tile_map,
                           const bf16* __restrict__ q, size_t q_stride, const int* __restrict__ block_table,
                           int table_width, const int* __restrict__ positions, int page_size, int heads, int kv_heads,
                           float scale_log2, int window, int partition, int num_partitions, int part_slow,
                           float* __restrict__ partial_o, float* __restrict__ partial_ml, bf16* __restrict__ out) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long barriers[BARRIERS];
  __shared__ uint32_t tmem_base_slot;
  __shared__ float exchange[2][4][G];                          // [tile parity][warp][head]: the warps' maxima
  __shared__ float sums[4][G];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int part = part_slow ? blockIdx.z : blockIdx.x, row = part_slow ? blockIdx.x : blockIdx.z;
  const int group = heads / kv_heads;
  const int group_tiles = (group + kHeads - 1) / kHeads;
  const int kv_head = blockIdx.y / group_tiles;
  const int head0 = kv_head * group + (blockIdx.y % group_tiles) * kHeads;
  const int valid_heads = min(kHeads, kv_head * group + group - head0);
  grid_launch_dependents();
  // Launched with programmatic stream serialization, this kernel may start while the kernel before it (which
  // writes the newest key and value and rotates q) still runs.  Positions and block tables are older than that
  // kernel, and so is every key but the newest.
  const int position = positions[row];
  const int context = position + 1;
  const int first_key = (window > 0 && context > window) ? context - window : 0;
  const int part_end = min(context, (part + 1) * partition);
  const int begin = max(part * partition, first_key / kKeys * kKeys);
  if (position < 0 || begin >= part_end || *reinterpret_cast<volatile int*>(&g_tc_decode_error) != 0) {
    grid_dependency_wait();                                   // (a padding row, or a partition the merge skips too)
    return;
  }
  const int tiles = (part_end - begin + kKeys - 1) / kKeys;

  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar0 = smem_u32(&barriers[0]);
  auto bar = [&](int index) { return bar0 + 8u * (uint32_t)index; };
  if (threadIdx.x == kSoftmaxThreads) {
    for (int i = 0; i < BARRIERS; ++i)
      barrier_init(bar(i), (i == P_READY || i == Q_READY) ? (uint32_t)kSoftmaxThreads : 1u);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(kTmemColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tensor_fence_before_sync();
  __syncthreads();
  tensor_fence_after_sync();
  const uint32_t tmem_s = tmem_base_slot, tmem_o = tmem_base_slot + 16u;
  MIR_TRACE_BEGIN(decode, (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ||
                              (part_end == context && blockIdx.y == gridDim.y - 1 &&
                               row == (int)(part_slow ? gridDim.x : gridDim.z) - 1),
                  200 + (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 ? 0 : 1))
  if (threadIdx.x == 0) {
    MIR_TRACE_VALUE(decode, tiles);
    MIR_TRACE_POINT(decode, 0);
    MIR_TRACE_POINT(decode, 1);
  }

  if (warp == 4) {
    // ------------------------------------------------------------------ loader
    // lane l loads half (l & 1) of page slot (l >> 1): at most 16 pages of 8 keys, so one round of 32 lanes
    const int* table = block_table + (size_t)row * table_width;
    const int pages_per_tile = kKeys / page_size;
    const int slot = lane >> 1, half = lane & 1;
    const bool loads = lane < 2 * pages_per_tile;
    // the newest key is the kernel's before this one; every other key is older
    if (part_end > position) grid_dependency_wait();
    if (lane == 0) MIR_TRACE_POINT(decode, 2);
    auto row_of = [&](int t) {
      const int key = begin + t * kKeys + slot * page_size;
      int page = -1;
      // (a position beyond what the table holds reads no entry: its keys count as released)
      if (loads && t < tiles && key < part_end && key + page_size > first_key && key / page_size < table_width)
        page = table[key / page_size];
      return page >= 0 ? page * page_size : -page_size;       // a negative row lies outside the tensor: zeros
    };
    int cache_row = row_of(0);
    bool alive = true;
    for (int t = 0; t < tiles && alive; ++t) {
      const uint32_t parity = (uint32_t)t & 1u;
      const int next_row = row_of(t + 1);                     // on its way while this tile's slots are awaited
      // A copy instruction costs the warp about 75 cycles for every lane that takes part: 2,400 cycles for the keys
      // and values of a tile of 16-key pages.  Where the tile's pages lie one behind the other in the pool (a prompt's
      // pages do while the pool is not fragmented), two lanes fetch each of them as two boxes of 128 keys.
      const int first_row = __shfl_sync(0xffffffffu, cache_row, 0);
      const bool in_a_row = first_row >= 0 && __all_sync(0xffffffffu, !loads || cache_row == first_row + slot * page_size);
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t full = bar(which ? V_FULL : K_FULL), free_bar = bar(which ? V_FREE : K_FREE);
        int ok = 1;
        if (lane == 0) ok = wait_barrier(free_bar, parity ^ 1u) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) { if (lane == 0) g_tc_decode_error = 1; alive = false; break; }
        if (lane == 0) barrier_expect_bytes(full, (uint32_t)kTile);
        __syncwarp();
        if (in_a_row) {
          if (lane < 2)
            tma_load_2d(smem_base + (which ? kOffV : kOffK) + (uint32_t)lane * kHalf, which ? &v_tile_map : &k_tile_map,
                        full, kv_head * kDim + lane * 64, first_row);
        } else if (loads) {
          tma_load_2d(smem_base + (which ? kOffV : kOffK) + (uint32_t)half * kHalf + (uint32_t)(slot * page_size) * 128u,
                      which ? &v_map : &k_map, full, kv_head * kDim + half * 64, cache_row);
        }
      }
      cache_row = next_row;
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ issuer: the whole warp stays converged, the
    // products are predicated on the elected lane and take their descriptors as 32-bit halves (tcgen05.cuh: a product
    // of 16 columns is over in a few cycles, and a lone thread in a divergent branch needs longer than that to issue
    // the next one)
    {
      constexpr uint32_t idesc_scores = instruction_descriptor(kKeys, kHeads, false);
      constexpr uint32_t idesc_values = instruction_descriptor(kDim, kHeads, false) | (1u << 15);   // A MN-major
      const uint32_t elected = elect_one();
      const uint32_t k_low = operand_low(smem_base + kOffK), q_low = operand_low(smem_base + kOffQ);
      const uint32_t v_low = operand_low_mn_major(smem_base + kOffV, kHalf), p_low = operand_low(smem_base + kOffP);
      bool alive = true;
      auto check = [&](int index, uint32_t parity) {
        if (alive && !wait_barrier(bar(index), parity)) { g_tc_decode_error = 2; alive = false; }
      };
      auto issue_scores = [&](int t) {
        check(K_FULL, (uint32_t)t & 1u);
        tensor_fence_after_sync();
        mma_bf16_ss_halves<false>(tmem_s, k_low, q_low, idesc_scores, elected);
#pragma unroll
        for (int kk = 1; kk < kDim / 16; ++kk)
          mma_bf16_ss_halves<true>(tmem_s, k_low + (uint32_t)(kk >> 2) * (uint32_t)(kHalf >> 4) + (uint32_t)(kk & 3) * 2u,
                                   q_low + (uint32_t)(kk >> 2) * (uint32_t)(kSmallHalf >> 4) + (uint32_t)(kk & 3) * 2u,
                                   idesc_scores, elected);
        mma_commit_elected(bar(S_FULL), elected);
        mma_commit_elected(bar(K_FREE), elected);
      };
      check(Q_READY, 0u);
      if (elected) MIR_TRACE_POINT(decode, 4);
      issue_scores(0);
      if (elected) MIR_TRACE_POINT(decode, 5);
      for (int t = 0; t < tiles; ++t) {
        const uint32_t parity = (uint32_t)t & 1u;
        check(V_FULL, parity);
        check(P_READY, parity);
        tensor_fence_after_sync();
        mma_bf16_ss_halves(tmem_o, v_low, p_low, idesc_values, t > 0 ? 1u : 0u, elected);
#pragma unroll
        for (int kk = 1; kk < kKeys / 16; ++kk)
          mma_bf16_ss_halves<true>(tmem_o, v_low + (uint32_t)kk * (2048u >> 4),
                                   p_low + (uint32_t)(kk >> 2) * (uint32_t)(kSmallHalf >> 4) + (uint32_t)(kk & 3) * 2u,
                                   idesc_values, elected);
        mma_commit_elected(bar(V_FREE), elected);
        // the next scores are issued behind this product, so that their barrier also says that O^T may be rescaled
        if (t + 1 < tiles) issue_scores(t + 1);
        else mma_commit_elected(bar(O_DONE), elected);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax: thread = key of the tile, then element
    const int r = warp * 32 + lane;
    const uint32_t lane_bits = (uint32_t)(warp * 32) << 16;
    bool alive = true;
    grid_dependency_wait();                                   // q comes from the kernel before
    if (r == 0) MIR_TRACE_POINT(decode, 3);
    {
      // the group's queries as a B operand: 16 rows (heads beyond the group are zero) x 128 elements
      unsigned char* q_smem = smem + kOffQ;
      for (int chunk = r; chunk < kHeads * (kDim / 8); chunk += kSoftmaxThreads) {
        const int h = chunk / (kDim / 8), c = chunk % (kDim / 8);
        uint4 value = make_uint4(0u, 0u, 0u, 0u);
        if (h < valid_heads)
          value = *reinterpret_cast<const uint4*>(q + (size_t)row * q_stride + (size_t)(head0 + h) * kDim + c * 8);
        *reinterpret_cast<uint4*>(q_smem + small_operand_offset(h, c * 8)) = value;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      barrier_arrive(bar(Q_READY));
    }
    float reference[G], denominator[G];
#pragma unroll
    for (int g = 0; g < G; ++g) { reference[g] = -INFINITY; denominator[g] = 0.0f; }
    unsigned char* p_smem = smem + kOffP;
    for (int t = 0; t < tiles; ++t) {
      const uint32_t parity = (uint32_t)t & 1u;
      const int key = begin + t * kKeys + r;
      const bool visible = key >= first_key && key <= position;
      if (alive && !wait_barrier(bar(S_FULL), parity)) { g_tc_decode_error = 3; alive = false; }
      if (r == 0 && t == 0) MIR_TRACE_POINT(decode, 6);
      if (r == 0 && t == tiles - 1) MIR_TRACE_POINT(decode, 8);
      tensor_fence_after_sync();
      float s[G];
      tmem_load<G>(tmem_s + lane_bits, s);
      float* mine = &exchange[t & 1][warp][0];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        s[g] = visible ? s[g] * scale_log2 : -INFINITY;
        const float top = warp_max(s[g]);
        if (lane == g) mine[g] = top;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
      float factor[G];
      bool grow = false;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float top = fmaxf(fmaxf(exchange[t & 1][0][g], exchange[t & 1][1][g]),
                                fmaxf(exchange[t & 1][2][g], exchange[t & 1][3][g]));
        const bool rises = top > reference[g] + kRescaleThreshold;
        factor[g] = rises ? fast_exp2(reference[g] - top) : 1.0f;   // 0 when nothing was seen before
        reference[g] = rises ? top : reference[g];
        grow = grow || rises;
      }
      // The product with the last tile's P is over (these scores were issued behind it), so O^T may be rescaled:
      // this thread's lane is an element of the head, its columns are the heads.
      if (t > 0 && grow) {
        float o[G];
        tmem_load<G>(tmem_o + lane_bits, o);
#pragma unroll
        for (int g = 0; g < G; ++g) o[g] *= factor[g];
        tmem_store<G>(tmem_o + lane_bits, o);
        tmem_store_wait();
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float p = visible ? fast_exp2(s[g] - reference[g]) : 0.0f;
        denominator[g] = denominator[g] * factor[g] + p;
        *reinterpret_cast<bf16*>(p_smem + small_operand_offset(g, r)) = __float2bfloat16_rn(p);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tensor_fence_before_sync();
      barrier_arrive(bar(P_READY));
      if (r == 0 && t == 0) MIR_TRACE_POINT(decode, 7);
      if (r == 0 && t == tiles - 1) MIR_TRACE_POINT(decode, 9);
    }
    // the denominators: every thread holds its keys' share
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float total = warp_sum(denominator[g]);
      if (lane == g) sums[warp][g] = total;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
    if (alive && !wait_barrier(bar(O_DONE), 0u)) { g_tc_decode_error = 3; alive = false; }
    if (r == 0) MIR_TRACE_POINT(decode, 10);
    tensor_fence_after_sync();
    float o[G];
    tmem_load<G>(tmem_o + lane_bits, o);
    if (alive) {
#pragma unroll
      for (int g = 0; g < G; ++g) {
        if (g >= valid_heads) break;
        const float denom = (sums[0][g] + sums[1][g]) + (sums[2][g] + sums[3][g]);
        const size_t head = (size_t)row * heads + head0 + g;
        if (num_partitions == 1) {
          out[head * kDim + r] = __float2bfloat16_rn(denom > 0.0f ? o[g] / denom : 0.0f);
        } else {
          partial_o[(head * num_partitions + part) * kDim + r] = denom > 0.0f ? o[g] : 0.0f;
          if (r == 0) {
            partial_ml[(head * num_partitions + part) * 2] = reference[g];
            partial_ml[(head * num_partitions + part) * 2 + 1] = denom;
          }
        }
      }
    }
    if (r == 0) MIR_TRACE_POINT(decode, 11);
    tensor_fence_before_sync();
  }
  __syncthreads();
  if (warp == 5) {
    tensor_fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_s), "r"(kTmemColumns) : "memory");
  }
  if (threadIdx.x == 0) MIR_TRACE_POINT(decode, 12);
}

template <int G>
int launch(const CUtensorMap& k_map, const CUtensorMap& v_map, const CUtensorMap& k_tile_map,
           const CUtensorMap& v_tile_map, const bf16* q, size_t q_stride, const int* block_table,
           int table_width, const int* positions, int rows, int page_size, int heads, int kv_heads, float scale,
           int window, int partition, int num_partitions, float* partial_o, float* partial_ml, bf16* out,
           cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    const cudaError_t err = cudaFuncSetAttribute(tc_decode_attention_kernel<G>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (err != cudaSuccess) {
      mir_set_error("decode_attention_tc: cannot reserve %d bytes of shared memory: %s", kSmemBytes,
                    cudaGetErrorString(err));
      return MIR_CUDA_ERROR;
    }
    configured = true;
  }
  const int group = heads / kv_heads;
  const int units = kv_heads * ((group + kHeads - 1) / kHeads);
  // the partition is the fast index (a request's CTAs start together), except for a handful of rows, where
  // partitions beyond the contexts (dead CTAs of a captured batch) are dispatched last
  const dim3 grid = rows <= 4 ? dim3(rows, units, num_partitions) : dim3(num_partitions, units, rows);
  return mir_launch_with(mir_pdl_for_streaming(), "decode_attention_tc", tc_decode_attention_kernel<G>, grid,
                         dim3(kThreads), (size_t)kSmemBytes, stream, 0, k_map, v_map, k_tile_map, v_tile_map, q, q_stride,
                         block_table,
                         table_width, positions, page_size, heads, kv_heads, scale * 1.4426950408889634f, window,
                         partition, num_partitions, rows <= 4 ? 1 : 0, partial_o, partial_ml, out);
}

}  // namespace

// 0 if no bounded wait of the tcgen05 decode attention ever ran out; else which role gave up last (1 loader,
// 2 issuer, 3 softmax).  Synchronises the device.
MIR_EXPORT int mir_decode_attention_tc_error() {
  int flag = 0;
  if (cudaMemcpyFromSymbol(&flag, g_tc_decode_error, sizeof(int)) != cudaSuccess) return -1;
  return flag;
}

// Whether the tcgen05 kernel takes these sizes: head_dim 128, pages of 8 to 128 keys that divide 128, partitions
// that are multiples of 128 keys.
MIR_EXPORT int mir_decode_attention_tc_takes(int head_dim, int page_size, int partition) {
  return head_dim == kDim && page_size >= 8 && page_size <= kKeys && kKeys % page_size == 0 &&
         page_size % 8 == 0 && partition > 0 && partition % kKeys == 0;
}

// One token per row, as mir_decode_attention_bf16; k_pages and v_pages are [cache_rows, kv_heads, 128].
MIR_EXPORT int mir_decode_attention_tc_bf16(const void* q, long long q_stride, void* out, const void* k_pages,
                                            const void* v_pages, long long cache_rows, const int* block_table,
                                            int table_width, const int* positions, int rows, int page_size, int heads,
                                            int kv_heads, int head_dim, float scale, int window, int partition,
                                            int num_partitions, float* scratch, long long scratch_floats,
                                            cudaStream_t stream) {
  if (rows == 0) return MIR_OK;
  if (!mir_decode_attention_tc_takes(head_dim, page_size, partition) || heads <= 0 || kv_heads <= 0 ||
      heads % kv_heads || table_width <= 0 || window < 0 || rows < 0 || rows > 65535 || num_partitions <= 0 ||
      num_partitions > 65535 || (q_stride % 8) || q_stride < (long long)heads * kDim || ((uintptr_t)q & 15) ||
      ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) || cache_rows <= 0 || cache_rows > 0x7fffffffll ||
      (long long)partition * num_partitions > 0x7fffffffll) {
    mir_set_error("decode_attention_tc: takes head_dim 128, pages of 8..128 keys that divide 128, partitions that are "
                  "multiples of 128 and 16-byte aligned tensors (head_dim %d, page %d, partition %d, "
                  "heads %d, kv heads %d, rows %d, partitions %d)",
                  head_dim, page_size, partition, heads, kv_heads, rows, num_partitions);
    return MIR_BAD_ARGUMENT;
  }
  const long long need = mir_decode_attention_scratch_floats(rows, heads, head_dim, num_partitions);
  if (need < 0 || (need > 0 && (scratch == nullptr || scratch_floats < need))) {
    mir_set_error("decode_attention_tc: scratch of %lld floats is needed, got %lld", need, scratch_floats);
    return MIR_BAD_ARGUMENT;
  }
  CUtensorMap k_map, v_map, k_tile_map, v_tile_map;
  int status = tensor_map_for(k_pages, (int)cache_rows, kv_heads * kDim, kv_heads * kDim, page_size, &k_map);
  if (status != MIR_OK) return status;
  status = tensor_map_for(v_pages, (int)cache_rows, kv_heads * kDim, kv_heads * kDim, page_size, &v_map);
  if (status != MIR_OK) return status;
  status = tensor_map_for(k_pages, (int)cache_rows, kv_heads * kDim, kv_heads * kDim, kKeys, &k_tile_map);
  if (status != MIR_OK) return status;
  status = tensor_map_for(v_pages, (int)cache_rows, kv_heads * kDim, kv_heads * kDim, kKeys, &v_tile_map);
  if (status != MIR_OK) return status;
  const int group = heads / kv_heads;
  const int columns = std::min(group, kHeads);
  float* partial_o = scratch;
  float* partial_ml = scratch ? scratch + (size_t)rows * heads * num_partitions * head_dim : nullptr;
#define MIR_SPLIT(G)                                                                                                 \
  launch<G>(k_map, v_map, k_tile_map, v_tile_map, (const bf16*)q, (size_t)q_stride, block_table, table_width, positions, rows, page_size, heads, \
            kv_heads, scale, window, partition, num_partitions, partial_o, partial_ml, (bf16*)out, stream)
  status = columns <= 4 ? MIR_SPLIT(4) : (columns <= 8 ? MIR_SPLIT(8) : MIR_SPLIT(16));
#undef MIR_SPLIT
  if (status != MIR_OK || num_partitions == 1) return status;
  return mir_decode_merge_bf16(partial_o, partial_ml, positions, rows, heads, head_dim, window, partition,
                               num_partitions, out, stream);
}
