// Tensor-core paged attention for bf16 (head_dim 64 or 128), two kernels:
//
//   decode   one token per request.  Split over the keys (flash-decoding): a CTA takes one
//            (request, kv head, partition of the keys) and serves the whole group of query heads that
//            share the kv head, so keys and values are read from HBM once per group, not once per head.
//            Each of its 4 warps streams its own 16-key tiles through a cp.async double buffer; partial
//            results (unnormalised output, running maximum, denominator) are merged by a second kernel.
//            Replaces libmir's paged_attention_batch_split_bf16.cu:24-424 (SIMT / wmma 16x16x16).
//   prefill  portions of prompts (and any mixed batch).  FlashAttention-2 style: a CTA takes 64
//            consecutive tokens of one request's portion and one query head; keys/values of the
//            request's history AND of the portion itself come from the cache pages (the portion's were
//            written by the kernel that ran before).  Replaces the per-token kernel
//            paged_prefill_attention_batch_bf16.cu:14-124 and the opaque FmhaBf16Plan.
//
// Both use mma.sync.m16n8k16 (bf16 in, 32-bit accumulate) with ldmatrix from padded shared-memory rows
// (row stride head_dim + 8 elements: an odd number of 16-byte chunks, so ldmatrix is conflict-free).
// Scores, maxima, exponentials and sums are 32-bit.  Keys outside [first visible, position] are masked
// before the maximum is taken; a tile's tail beyond the context is zero-filled, never read.
#include <algorithm>
#include <cfloat>
#include "common.cuh"
#include "trace.cuh"

using namespace mir;
typedef __nv_bfloat16 bf16;

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;   // 0 bytes read: the 16 bytes of shared memory are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// 2^x for x <= 0 (or -inf): the hardware approximation (2 ulp), far below what rounding the weights to bf16 loses.
__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// Copy ROWS consecutive keys and their values (one kv head, head_dim bf16 each) from the pages into padded
// shared-memory rows with THREADS threads.  Row i holds key `first_key + i`; rows whose key is >= limit
// are zero-filled, and so are rows whose page the block table marks as released (a negative entry: a sliding
// window has passed the page; such keys are masked by the caller, and no address is formed from the entry).
// One instruction of a warp copies whole rows: head_dim / 8 consecutive lanes take the
// consecutive 16-byte pieces of a row, so every 32-byte sector that is requested is used in full (a lane
// that walked along its own row would ask for each sector twice, once per half).  The rows of one
// instruction are GROUP consecutive keys; when the page size is a multiple of GROUP they lie in one page
// and the block table is read once for all of them (the same address for every lane).
template <int D, int ROWS, int THREADS>
__device__ __forceinline__ void load_tile(bf16* k_dst, bf16* v_dst, const bf16* __restrict__ k_pages,
                                          const bf16* __restrict__ v_pages, const int* __restrict__ table,
                                          int page_size, int kv_heads, int kv_head, int first_key, int limit,
                                          int thread) {
  constexpr int STRIDE = D + 8;
  constexpr int CHUNKS = D / 8;                    // 16-byte pieces per row
  constexpr int GROUP = THREADS / CHUNKS;          // rows per instruction
  static_assert(ROWS % GROUP == 0, "tile rows must be a multiple of the rows one instruction copies");
  const int sub = thread / CHUNKS, piece = thread % CHUNKS;
  if (page_size % ROWS == 0 && first_key % ROWS == 0) {
    // the whole tile lies in one page: one table read, then constant strides
    const int block = first_key / page_size;
    const int entry = first_key < limit ? table[block] : -1;
    const int page = entry < 0 ? 0 : entry;
    const size_t row_stride = (size_t)kv_heads * D;
    const size_t base = ((size_t)page * page_size + (first_key - block * page_size)) * row_stride + (size_t)kv_head * D +
                        piece * 8;
#pragma unroll
    for (int i = 0; i < ROWS / GROUP; ++i) {
      const int r = i * GROUP + sub;
      const bool valid = entry >= 0 && first_key + r < limit;
      const size_t offset = valid ? base + r * row_stride : 0;
      cp_async16(smem_u32(k_dst + r * STRIDE + piece * 8), k_pages + offset, valid);
      cp_async16(smem_u32(v_dst + r * STRIDE + piece * 8), v_pages + offset, valid);
    }
    return;
  }
  const bool one_page = page_size % GROUP == 0 && first_key % GROUP == 0;
#pragma unroll
  for (int i = 0; i < ROWS / GROUP; ++i) {
    const int r = i * GROUP + sub;
    const int key = first_key + r;
    bool valid = key < limit;
    size_t offset = 0;
    if (valid) {
      const int lookup_key = one_page ? first_key + i * GROUP : key;
      const int block = lookup_key / page_size;
      const int page = table[block];
      valid = page >= 0;
      if (valid) offset = (((size_t)page * page_size + (key - block * page_size)) * kv_heads + kv_head) * D + piece * 8;
    }
    cp_async16(smem_u32(k_dst + r * STRIDE + piece * 8), k_pages + offset, valid);
    cp_async16(smem_u32(v_dst + r * STRIDE + piece * 8), v_pages + offset, valid);
  }
}

// S[16 x NT*8 keys] += Q[16 x D] . K^T for NT n-tiles of 8 keys (NT even).
template <int D, int NT>
__device__ __forceinline__ void scores(float (&s)[NT][4], const uint32_t (&qa)[D / 16][4], const bf16* k_tile,
                                       int lane) {
  constexpr int STRIDE = D + 8;
  const int mat = lane >> 3, rowin = lane & 7;
  const bf16* base = k_tile + ((mat >> 1) * 8 + rowin) * STRIDE + (mat & 1) * 8;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
    for (int pair = 0; pair < NT / 2; ++pair) {
      uint32_t b[4];
      ldmatrix_x4(b, smem_u32(base + pair * 16 * STRIDE + ks * 16));
      mma_bf16(s[2 * pair], qa[ks], b[0], b[1]);
      mma_bf16(s[2 * pair + 1], qa[ks], b[2], b[3]);
    }
  }
}

// O[16 x D] += P[16 x NT*8 keys] . V.
template <int D, int NT>
__device__ __forceinline__ void values(float (&o)[D / 8][4], const uint32_t (&pa)[NT / 2][4], const bf16* v_tile,
                                       int lane) {
  constexpr int STRIDE = D + 8;
  const int mat = lane >> 3, rowin = lane & 7;
  const bf16* base = v_tile + ((mat & 1) * 8 + rowin) * STRIDE + (mat >> 1) * 8;
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
#pragma unroll
    for (int np = 0; np < D / 16; ++np) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, smem_u32(base + kk * 16 * STRIDE + np * 16));
      mma_bf16(o[2 * np], pa[kk], b[0], b[1]);
      mma_bf16(o[2 * np + 1], pa[kk], b[2], b[3]);
    }
  }
}

// Online-softmax update of one 16-row block with the scores of NT*8 keys (already scaled to log2 units and
// masked with -inf).  m/l are per thread for its two rows (lane/4 and lane/4 + 8); l is a per-thread partial
// sum that the caller reduces over the quad at the end.
template <int D, int NT>
__device__ __forceinline__ void softmax(float (&s)[NT][4], float (&m)[2], float (&l)[2], float (&o)[D / 8][4],
                                        uint32_t (&pa)[NT / 2][4]) {
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
    mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
  }
  mx0 = quad_max(mx0);
  mx1 = quad_max(mx1);
  const float new0 = fmaxf(m[0], mx0), new1 = fmaxf(m[1], mx1);
  const float ref0 = new0 == -INFINITY ? 0.0f : new0, ref1 = new1 == -INFINITY ? 0.0f : new1;
  const float corr0 = exp2f(m[0] - ref0), corr1 = exp2f(m[1] - ref1);
  m[0] = new0;
  m[1] = new1;
  float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    s[nt][0] = exp2f(s[nt][0] - ref0);
    s[nt][1] = exp2f(s[nt][1] - ref0);
    s[nt][2] = exp2f(s[nt][2] - ref1);
    s[nt][3] = exp2f(s[nt][3] - ref1);
    sum0 += s[nt][0] + s[nt][1];
    sum1 += s[nt][2] + s[nt][3];
  }
  l[0] = l[0] * corr0 + sum0;
  l[1] = l[1] * corr1 + sum1;
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    o[nt][0] *= corr0;
    o[nt][1] *= corr0;
    o[nt][2] *= corr1;
    o[nt][3] *= corr1;
  }
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
    pa[kk][0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    pa[kk][1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    pa[kk][2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    pa[kk][3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
  }
}

// ------------------------------------------------------------------------------------------------ decode
constexpr int kDecodeWarps = 4;
constexpr int kDecodeTile = 16;
// tiles of 16 keys in flight per warp: 2 where the CTAs are many (three CTAs fit on an SM), 3 where they are few and
// a CTA's chain of dependent copies sets the kernel's time (batch 8, 2,120 keys: 20.0 against 21.7 us; batch 64:
// 118 against 105 us)
constexpr int kDecodeHeads = 8;                 // query heads one CTA serves (rows 8..15 of the tile are padding)
constexpr int kDecodeMaxPartition = 512;
constexpr int kDecodeMaxTiles = kDecodeMaxPartition / (kDecodeWarps * kDecodeTile);   // tiles per warp

// One CTA: one request, one kv head (up to 8 of its query heads), one partition of the keys.
// Per 16-key tile a warp computes S = Q K^T (heads on the M side, 8 real rows), the softmax update of its
// 8 heads, and O^T += V^T P^T (head_dim on the M side, heads on the N side: the padding rows cost nothing
// here, and P^T in the layout the product wants is exactly the layout S came out in).
template <int D, int kDecodeStages>
__global__ void __launch_bounds__(kDecodeWarps * 32)
decode_attention_kernel(const bf16* __restrict__ q, size_t q_stride, const bf16* __restrict__ k_pages,
                        const bf16* __restrict__ v_pages, const int* __restrict__ block_table, int table_width,
                        const int* __restrict__ positions, int page_size, int heads, int kv_heads, float scale_log2,
                        int window, int partition, int num_partitions, int part_slow, float* __restrict__ partial_o,
                        float* __restrict__ partial_ml, bf16* __restrict__ out) {
  constexpr int STRIDE = D + 8;
  constexpr int TILE_ELEMS = kDecodeTile * STRIDE;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad = lane & 3, group_row = lane >> 2;
  // The partition is the fast index of the grid (a request's CTAs start together), except for a handful of rows,
  // where it is the slow one, so that partitions beyond the contexts (dead CTAs of a captured batch, whose table is
  // wider than any context) are dispatched last: batch 1 at 2,112 keys 8.4 against 9.4 us, batch 8 19.8 against 19.4.
  const int part = part_slow ? blockIdx.z : blockIdx.x, row = part_slow ? blockIdx.x : blockIdx.z;
  const int group = heads / kv_heads;
  const int group_tiles = (group + kDecodeHeads - 1) / kDecodeHeads;
  const int kv_head = blockIdx.y / group_tiles;
  const int head0 = kv_head * group + (blockIdx.y % group_tiles) * kDecodeHeads;
  const int valid_rows = min(kDecodeHeads, kv_head * group + group - head0);
  grid_launch_dependents();
  // Launched with programmatic stream serialization, this kernel may start while the kernel before it (which
  // writes the newest key and value and rotates q) still runs.  Positions and block tables are older than that
  // kernel, and so is every key but the newest: the first copies of old keys start before the wait.
  const int position = positions[row];
  if (position < 0) return;                                   // padding row of a captured batch
  const int context = position + 1;
  const int first_key = (window > 0 && context > window) ? context - window : 0;
  const int part_begin = part * partition;
  const int part_end = min(context, part_begin + partition);
  const int begin = max(part_begin, first_key / kDecodeTile * kDecodeTile);
  if (begin >= part_end) return;                              // the merge skips this partition the same way

  // this warp's buffers: [stage][K | V][16 rows][STRIDE]
  bf16* stage_base = reinterpret_cast<bf16*>(smem_raw) + (size_t)warp * kDecodeStages * 2 * TILE_ELEMS;
  const int* table = block_table + (size_t)row * table_width;
  const int stride_keys = kDecodeWarps * kDecodeTile;
  const int my_begin = begin + warp * kDecodeTile;
  const int my_tiles = my_begin < part_end ? (part_end - my_begin + stride_keys - 1) / stride_keys : 0;

  // the first copies are on their way before anything else is done; if one of them covers the newest key, the
  // kernel that writes it has to be over first
  const bool early = my_begin + (kDecodeStages - 2) * stride_keys + kDecodeTile <= position;
  if (!early) grid_dependency_wait();
#pragma unroll
  for (int j = 0; j < kDecodeStages - 1; ++j) {
    if (j < my_tiles) {
      bf16* dst = stage_base + j * 2 * TILE_ELEMS;
      load_tile<D, kDecodeTile, 32>(dst, dst + TILE_ELEMS, k_pages, v_pages, table, page_size, kv_heads, kv_head,
                                    my_begin + j * stride_keys, part_end, lane);
    }
    cp_async_commit();
  }

  if (early) grid_dependency_wait();                          // q (and the newest key) come from the kernel before
  // Q fragments: rows 0..7 are the heads of the group, rows 8..15 are zero
  uint32_t qa[D / 16][4];
  {
    const int c = quad * 2;
    const bf16* q_row = q + (size_t)row * q_stride + (size_t)(head0 + group_row) * D;
    const bool real = group_row < valid_rows;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qa[ks][0] = real ? *reinterpret_cast<const uint32_t*>(q_row + ks * 16 + c) : 0u;
      qa[ks][1] = 0u;
      qa[ks][2] = real ? *reinterpret_cast<const uint32_t*>(q_row + ks * 16 + 8 + c) : 0u;
      qa[ks][3] = 0u;
    }
  }

  float ot[D / 16][4];                                         // O^T: [d = mt*16 + lane/4 (+8)][head = quad*2 (+1)]
#pragma unroll
  for (int mt = 0; mt < D / 16; ++mt) ot[mt][0] = ot[mt][1] = ot[mt][2] = ot[mt][3] = 0.0f;
  float m = -INFINITY, l = 0.0f;                               // of head lane/4 (l: this lane's share)

#pragma unroll
  for (int j = 0; j < kDecodeMaxTiles; ++j) {
    if (j >= my_tiles) break;
    constexpr int kAhead = kDecodeStages - 1;
    if (j + kAhead < my_tiles) {
      bf16* dst = stage_base + ((j + kAhead) % kDecodeStages) * 2 * TILE_ELEMS;
      load_tile<D, kDecodeTile, 32>(dst, dst + TILE_ELEMS, k_pages, v_pages, table, page_size, kv_heads, kv_head,
                                    my_begin + (j + kAhead) * stride_keys, part_end, lane);
    }
    cp_async_commit();
    cp_async_wait<kDecodeStages - 1>();
    __syncwarp();
    const int tile = my_begin + j * stride_keys;
    const bf16* k_tile = stage_base + (j % kDecodeStages) * 2 * TILE_ELEMS;
    const bf16* v_tile = k_tile + TILE_ELEMS;
    float s[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
    scores<D, 2>(s, qa, k_tile, lane);
    float v00 = s[0][0] * scale_log2, v01 = s[0][1] * scale_log2, v10 = s[1][0] * scale_log2, v11 = s[1][1] * scale_log2;
    if (tile + kDecodeTile > context || tile < first_key) {     // only the edge tiles need a mask
      const int key = tile + quad * 2;
      if (key < first_key || key > position) v00 = -INFINITY;
      if (key + 1 < first_key || key + 1 > position) v01 = -INFINITY;
      if (key + 8 < first_key || key + 8 > position) v10 = -INFINITY;
      if (key + 9 < first_key || key + 9 > position) v11 = -INFINITY;
    }
    const float tile_max = quad_max(fmaxf(fmaxf(v00, v01), fmaxf(v10, v11)));
    const float next = fmaxf(m, tile_max);
    const float ref = next == -INFINITY ? 0.0f : next;
    const float corr = exp2_fast(m - ref);
    m = next;
    v00 = exp2_fast(v00 - ref);
    v01 = exp2_fast(v01 - ref);
    v10 = exp2_fast(v10 - ref);
    v11 = exp2_fast(v11 - ref);
    l = l * corr + (v00 + v01 + v10 + v11);
    if (__any_sync(0xffffffffu, corr != 1.0f)) {                // the maximum moved for some head: rescale O^T
      const float corr_a = __shfl_sync(0xffffffffu, corr, quad * 8);        // head quad*2   lives in lanes 8*quad..
      const float corr_b = __shfl_sync(0xffffffffu, corr, quad * 8 + 4);    // head quad*2+1
#pragma unroll
      for (int mt = 0; mt < D / 16; ++mt) {
        ot[mt][0] *= corr_a;
        ot[mt][1] *= corr_b;
        ot[mt][2] *= corr_a;
        ot[mt][3] *= corr_b;
      }
    }
    const uint32_t pb0 = pack_bf16(v00, v01), pb1 = pack_bf16(v10, v11);   // P^T: keys 0..7 and 8..15 of the tile
    {
      const int mat = lane >> 3, rowin = lane & 7;
      const bf16* base = v_tile + ((mat >> 1) * 8 + rowin) * STRIDE + (mat & 1) * 8;
#pragma unroll
      for (int mt = 0; mt < D / 16; ++mt) {
        uint32_t a[4];
        ldmatrix_x4_trans(a, smem_u32(base + mt * 16));
        mma_bf16(ot[mt], a, pb0, pb1);
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();
  l = quad_sum(l);
  __syncthreads();                                            // every warp is done with its pipeline buffers

  // combine the 4 warps through shared memory
  float* o_sm = reinterpret_cast<float*>(smem_raw);           // [warps][8 heads][D]
  float* m_sm = o_sm + kDecodeWarps * kDecodeHeads * D;       // [warps][8]
  float* l_sm = m_sm + kDecodeWarps * kDecodeHeads;
  {
    float* mine = o_sm + (size_t)warp * kDecodeHeads * D;
    const int head_a = quad * 2, head_b = head_a + 1;
#pragma unroll
    for (int mt = 0; mt < D / 16; ++mt) {
      const int d = mt * 16 + group_row;
      mine[head_a * D + d] = ot[mt][0];
      mine[head_b * D + d] = ot[mt][1];
      mine[head_a * D + d + 8] = ot[mt][2];
      mine[head_b * D + d + 8] = ot[mt][3];
    }
    if (quad == 0) {
      m_sm[warp * kDecodeHeads + group_row] = m;
      l_sm[warp * kDecodeHeads + group_row] = l;
    }
  }
  __syncthreads();
  for (int index = threadIdx.x; index < valid_rows * D; index += kDecodeWarps * 32) {
    const int r = index / D, d = index % D;
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) top = fmaxf(top, m_sm[w * kDecodeHeads + r]);
    float acc = 0.0f, denom = 0.0f;
    if (top != -INFINITY) {
#pragma unroll
      for (int w = 0; w < kDecodeWarps; ++w) {
        const float weight = exp2f(m_sm[w * kDecodeHeads + r] - top);
        acc += o_sm[((size_t)w * kDecodeHeads + r) * D + d] * weight;
        denom += l_sm[w * kDecodeHeads + r] * weight;
      }
    }
    const size_t head = (size_t)row * heads + head0 + r;
    if (num_partitions == 1) {
      out[head * D + d] = __float2bfloat16_rn(denom > 0.0f ? acc / denom : 0.0f);
    } else {
      partial_o[(head * num_partitions + part) * D + d] = acc;
      if (d == 0) {
        partial_ml[(head * num_partitions + part) * 2] = top;
        partial_ml[(head * num_partitions + part) * 2 + 1] = denom;
      }
    }
  }
}

// One CTA of four warps per (request, head).  The partitions are shared out over the warps (each lane four
// consecutive elements of the head, 16-byte loads, four partitions in flight), so a long context's hundred
// partitions cost a few rounds of loads, not a hundred; the warps' sums meet in shared memory.
// time stamps (trace.cuh) of the merge's first and last CTA: 0 start, 1 the attention kernel is over, 2 end; tag 300 / 301
MIR_TRACE_DEFINE(merge)
constexpr int kMergeWarps = 4;
template <int D>
__global__ void __launch_bounds__(kMergeWarps * 32)
decode_merge_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                    const int* __restrict__ positions, int heads, int window, int partition, int num_partitions,
                    bf16* __restrict__ out) {
  constexpr int LANES = D / 4;                                 // lanes of a warp that hold elements
  __shared__ float warp_top[kMergeWarps];
  __shared__ float sums[kMergeWarps][D + 1];                   // [warp][elements, then the denominator]
  const int head = blockIdx.x, row = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  grid_launch_dependents();
  MIR_TRACE_BEGIN(merge, (blockIdx.x == 0 && blockIdx.y == 0) || (blockIdx.x == gridDim.x - 1 && blockIdx.y == gridDim.y - 1),
                  300 + (blockIdx.x == 0 && blockIdx.y == 0 ? 0 : 1))
  if (threadIdx.x == 0) MIR_TRACE_POINT(merge, 0);
  grid_dependency_wait();
  if (threadIdx.x == 0) MIR_TRACE_POINT(merge, 1);
  const int position = positions[row];
  const size_t index = (size_t)row * heads + head;
  if (position < 0) {
    for (int d = threadIdx.x; d < D; d += blockDim.x) out[index * D + d] = __float2bfloat16_rn(0.0f);
    return;
  }
  const int context = position + 1;
  const int first_key = (window > 0 && context > window) ? context - window : 0;
  const int first_part = (first_key / kDecodeTile * kDecodeTile) / partition;
  const int last_part = min(position / partition, num_partitions - 1);   // (a caller with too few partitions reads nothing beyond them)
  const float* ml = partial_ml + index * num_partitions * 2;
  const float* o = partial_o + index * num_partitions * D;
  // the largest maximum over all partitions
  float top = -INFINITY;
  for (int p = first_part + (int)threadIdx.x; p <= last_part; p += kMergeWarps * 32) top = fmaxf(top, ml[2 * p]);
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, offset));
  if (lane == 0) warp_top[warp] = top;
  __syncthreads();
  top = fmaxf(fmaxf(warp_top[0], warp_top[1]), fmaxf(warp_top[2], warp_top[3]));
  // this warp's partitions
  float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  float denom = 0.0f;
  constexpr int kAhead = 4;
  for (int p0 = first_part + warp; p0 <= last_part; p0 += kMergeWarps * kAhead) {
    float4 piece[kAhead];
    float weight[kAhead], part_denom[kAhead];
#pragma unroll
    for (int i = 0; i < kAhead; ++i) {
      const int p = p0 + i * kMergeWarps;
      const bool live = p <= last_part;
      piece[i] = (live && lane < LANES) ? *reinterpret_cast<const float4*>(o + (size_t)p * D + 4 * lane)
                                        : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      weight[i] = live ? ml[2 * p] : -INFINITY;
      part_denom[i] = live ? ml[2 * p + 1] : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < kAhead; ++i) {
      const float w = weight[i] > -INFINITY ? exp2f(weight[i] - top) : 0.0f;   // (a partition that saw no key)
      acc.x += piece[i].x * w; acc.y += piece[i].y * w; acc.z += piece[i].z * w; acc.w += piece[i].w * w;
      denom += part_denom[i] * w;
    }
  }
  if (lane < LANES) {
    sums[warp][4 * lane] = acc.x; sums[warp][4 * lane + 1] = acc.y;
    sums[warp][4 * lane + 2] = acc.z; sums[warp][4 * lane + 3] = acc.w;
  }
  if (lane == 0) sums[warp][D] = denom;
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float total = (sums[0][d] + sums[1][d]) + (sums[2][d] + sums[3][d]);
    const float all = (sums[0][D] + sums[1][D]) + (sums[2][D] + sums[3][D]);
    out[index * D + d] = __float2bfloat16_rn(all > 0.0f ? total / all : 0.0f);
  }
  if (threadIdx.x == 0) MIR_TRACE_POINT(merge, 2);
}

// The same for up to kMergeFew partitions: one warp per (request, head), every lane D / 32 consecutive elements of
// the head and all partitions' loads in flight at once; no shared memory, no barrier.  (64 requests of five
// partitions: 3 us where the kernel above takes 7.)
constexpr int kMergeFew = 8;
template <int D>
__global__ void __launch_bounds__(kMergeWarps * 32)
decode_merge_few_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                        const int* __restrict__ positions, int heads, int window, int partition, int num_partitions,
                        bf16* __restrict__ out) {
  constexpr int PER = D / 32;                                  // elements per lane: 4 or 2
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x * kMergeWarps + warp, row = blockIdx.y;
  grid_launch_dependents();
  MIR_TRACE_BEGIN(merge, (blockIdx.x == 0 && blockIdx.y == 0) || (blockIdx.x == gridDim.x - 1 && blockIdx.y == gridDim.y - 1),
                  300 + (blockIdx.x == 0 && blockIdx.y == 0 ? 0 : 1))
  if (threadIdx.x == 0) MIR_TRACE_POINT(merge, 0);
  grid_dependency_wait();
  if (threadIdx.x == 0) MIR_TRACE_POINT(merge, 1);
  if (head >= heads) return;
  const int position = positions[row];
  const size_t index = (size_t)row * heads + head;
  bf16* dst = out + index * D + PER * lane;
  if (position < 0) {
#pragma unroll
    for (int i = 0; i < PER; ++i) dst[i] = __float2bfloat16_rn(0.0f);
    return;
  }
  const int context = position + 1;
  const int first_key = (window > 0 && context > window) ? context - window : 0;
  const int first_part = (first_key / kDecodeTile * kDecodeTile) / partition;
  const int last_part = min(position / partition, num_partitions - 1);
  const float* ml = partial_ml + index * num_partitions * 2;
  const float* o = partial_o + index * num_partitions * D + PER * lane;
  float piece[kMergeFew][PER], reference[kMergeFew], denominators[kMergeFew];
#pragma unroll
  for (int i = 0; i < kMergeFew; ++i) {
    const int p = first_part + i;
    const bool live = p <= last_part;
    reference[i] = live ? ml[2 * p] : -INFINITY;
    denominators[i] = live ? ml[2 * p + 1] : 0.0f;
#pragma unroll
    for (int j = 0; j < PER; ++j) piece[i][j] = 0.0f;
    if (live) {
      if (PER == 4) {
        const float4 v = *reinterpret_cast<const float4*>(o + (size_t)p * D);
        piece[i][0] = v.x; piece[i][1] = v.y; piece[i][2] = v.z; piece[i][PER - 1] = v.w;
      } else {
        const float2 v = *reinterpret_cast<const float2*>(o + (size_t)p * D);
        piece[i][0] = v.x; piece[i][1] = v.y;
      }
    }
  }
  float top = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMergeFew; ++i) top = fmaxf(top, reference[i]);
  float acc[PER], denom = 0.0f;
#pragma unroll
  for (int j = 0; j < PER; ++j) acc[j] = 0.0f;
#pragma unroll
  for (int i = 0; i < kMergeFew; ++i) {
    const float w = reference[i] > -INFINITY ? exp2f(reference[i] - top) : 0.0f;   // (a partition that saw no key)
#pragma unroll
    for (int j = 0; j < PER; ++j) acc[j] += piece[i][j] * w;
    denom += denominators[i] * w;
  }
#pragma unroll
  for (int j = 0; j < PER; j += 2)
    *reinterpret_cast<__nv_bfloat162*>(dst + j) =
        __floats2bfloat162_rn(denom > 0.0f ? acc[j] / denom : 0.0f, denom > 0.0f ? acc[j + 1] / denom : 0.0f);
  if (threadIdx.x == 0) MIR_TRACE_POINT(merge, 2);
}

// ------------------------------------------------------------------------------------------------ prefill
constexpr int kPrefillWarps = 4;
constexpr int kQueryTile = kPrefillWarps * 16;     // 64 tokens per CTA
constexpr int kKeyTile = 64;

template <int D>
__global__ void __launch_bounds__(kPrefillWarps * 32, 3)
prefill_attention_kernel(const bf16* __restrict__ q, size_t q_stride, bf16* __restrict__ out,
                         const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                         const int* __restrict__ block_table, int table_width, const int* __restrict__ query_starts,
                         const int* __restrict__ context_lens, int num_rows, int page_size, int heads, int kv_heads,
                         float scale_log2, int window) {
  constexpr int STRIDE = D + 8;
  constexpr int TILE_ELEMS = kKeyTile * STRIDE;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* buffers = reinterpret_cast<bf16*>(smem_raw);          // [stage][K | V][64][STRIDE]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x;                                // the fast index: all heads of the longest tile start first
  const int kv_head = head / (heads / kv_heads);

  grid_launch_dependents();
  grid_dependency_wait();
  // which request row and which 64-token tile of its portion this CTA has
  int row = -1, local_tile = 0;
  {
    int remaining = gridDim.y - 1 - blockIdx.y;              // late tiles see the most keys: start them first
    for (int r = 0; r < num_rows; ++r) {
      const int tiles = (query_starts[r + 1] - query_starts[r] + kQueryTile - 1) / kQueryTile;
      if (remaining < tiles) { row = r; local_tile = remaining; break; }
      remaining -= tiles;
    }
  }
  if (row < 0) return;
  const int q_begin = query_starts[row];
  const int count = query_starts[row + 1] - q_begin;
  const int start_position = context_lens[row] - count;
  const int local0 = local_tile * kQueryTile;
  const int tile_rows = min(kQueryTile, count - local0);
  const int first_position = start_position + local0;
  const int last_position = first_position + tile_rows - 1;
  const int* table = block_table + (size_t)row * table_width;

  // this warp's 16 query rows
  const int r0 = lane >> 2, r1 = r0 + 8, c = (lane & 3) * 2;
  const int local_r0 = warp * 16 + r0, local_r1 = warp * 16 + r1;
  const bool valid0 = local_r0 < tile_rows, valid1 = local_r1 < tile_rows;
  const int pos0 = min(first_position + local_r0, last_position), pos1 = min(first_position + local_r1, last_position);
  uint32_t qa[D / 16][4];
  {
    const bf16* q_row0 = q + (size_t)(q_begin + local0 + local_r0) * q_stride + (size_t)head * D;
    const bf16* q_row1 = q + (size_t)(q_begin + local0 + local_r1) * q_stride + (size_t)head * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qa[ks][0] = valid0 ? *reinterpret_cast<const uint32_t*>(q_row0 + ks * 16 + c) : 0u;
      qa[ks][1] = valid1 ? *reinterpret_cast<const uint32_t*>(q_row1 + ks * 16 + c) : 0u;
      qa[ks][2] = valid0 ? *reinterpret_cast<const uint32_t*>(q_row0 + ks * 16 + 8 + c) : 0u;
      qa[ks][3] = valid1 ? *reinterpret_cast<const uint32_t*>(q_row1 + ks * 16 + 8 + c) : 0u;
    }
  }
  float o[D / 8][4];
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

  const int first_key = (window > 0 && first_position + 1 > window) ? first_position + 1 - window : 0;
  const int key_begin = first_key / kKeyTile * kKeyTile;
  const int key_end = last_position + 1;                       // exclusive
  const int warp_last = min(first_position + warp * 16 + 15, last_position);
  const int warp_first = min(first_position + warp * 16, last_position);
  const int warp_first_key = (window > 0 && warp_first + 1 > window) ? warp_first + 1 - window : 0;

  load_tile<D, kKeyTile, kPrefillWarps * 32>(buffers, buffers + TILE_ELEMS, k_pages, v_pages, table, page_size, kv_heads, kv_head,
                         key_begin, key_end, threadIdx.x);
  cp_async_commit();
  int stage = 0;
  for (int key0 = key_begin; key0 < key_end; key0 += kKeyTile, stage ^= 1) {
    const int next = key0 + kKeyTile;
    if (next < key_end) {
      bf16* dst = buffers + (stage ^ 1) * 2 * TILE_ELEMS;
      load_tile<D, kKeyTile, kPrefillWarps * 32>(dst, dst + TILE_ELEMS, k_pages, v_pages, table, page_size, kv_heads, kv_head, next,
                             key_end, threadIdx.x);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const bf16* k_tile = buffers + stage * 2 * TILE_ELEMS;
    const bf16* v_tile = k_tile + TILE_ELEMS;
    // this warp needs the tile only if some key of it is visible to some of its rows
    if (key0 <= warp_last && key0 + kKeyTile > warp_first_key) {
      const bool needs_mask = key0 + kKeyTile - 1 > warp_first || (window > 0 && key0 < warp_last + 1 - window + 15);
      constexpr int NT = kKeyTile / 8;
      float s[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
      scores<D, NT>(s, qa, k_tile, lane);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          bool visible = true;
          if (needs_mask) {
            const int key = key0 + nt * 8 + c + (e & 1);
            const int pos = (e < 2) ? pos0 : pos1;
            visible = key <= pos && (window <= 0 || key > pos - window);
          }
          s[nt][e] = visible ? s[nt][e] * scale_log2 : -INFINITY;
        }
      uint32_t pa[NT / 2][4];
      softmax<D, NT>(s, m, l, o, pa);
      values<D, NT>(o, pa, v_tile, lane);
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  l[0] = quad_sum(l[0]);
  l[1] = quad_sum(l[1]);
  const float inv0 = l[0] > 0.0f ? 1.0f / l[0] : 0.0f, inv1 = l[1] > 0.0f ? 1.0f / l[1] : 0.0f;
  bf16* out0 = out + ((size_t)(q_begin + local0 + local_r0) * heads + head) * D;
  bf16* out1 = out + ((size_t)(q_begin + local0 + local_r1) * heads + head) * D;
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    if (valid0) *reinterpret_cast<uint32_t*>(out0 + nt * 8 + c) = pack_bf16(o[nt][0] * inv0, o[nt][1] * inv0);
    if (valid1) *reinterpret_cast<uint32_t*>(out1 + nt * 8 + c) = pack_bf16(o[nt][2] * inv1, o[nt][3] * inv1);
  }
}

// Opt in to more than 48 KB of dynamic shared memory.  `done` is the caller's flag for this one kernel.
template <typename Kernel>
int set_smem(Kernel kernel, size_t bytes, const char* what, bool& done) {
  if (bytes <= 48 * 1024 || done) return MIR_OK;
  const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (err != cudaSuccess) {
    mir_set_error("%s: cannot reserve %zu bytes of shared memory: %s", what, bytes, cudaGetErrorString(err));
    return MIR_CUDA_ERROR;
  }
  done = true;
  return MIR_OK;
}

// The merge kernel for this many partitions.  (A window can only lower the number of partitions a row has.)
template <int D>
int launch_merge(const float* partial_o, const float* partial_ml, const int* positions, int rows, int heads, int window,
                 int partition, int num_partitions, bf16* out, cudaStream_t stream) {
  if (num_partitions <= kMergeFew)
    return mir_launch("decode_merge", decode_merge_few_kernel<D>, dim3((heads + kMergeWarps - 1) / kMergeWarps, rows),
                      dim3(kMergeWarps * 32), 0, stream, 0, partial_o, partial_ml, positions, heads, window, partition,
                      num_partitions, out);
  return mir_launch("decode_merge", decode_merge_kernel<D>, dim3(heads, rows), dim3(kMergeWarps * 32), 0, stream, 0,
                    partial_o, partial_ml, positions, heads, window, partition, num_partitions, out);
}

template <int D, int STAGES>
int launch_decode_staged(const bf16* q, size_t q_stride, bf16* out, const bf16* k_pages, const bf16* v_pages,
                         const int* block_table, int table_width, const int* positions, int rows, int page_size,
                         int heads, int kv_heads, float scale, int window, int partition, int num_partitions,
                         float* partial_o, float* partial_ml, cudaStream_t stream) {
  const size_t pipeline = (size_t)kDecodeWarps * STAGES * 2 * kDecodeTile * (D + 8) * sizeof(bf16);
  const size_t combine = (size_t)kDecodeWarps * kDecodeHeads * (D + 2) * sizeof(float);
  const size_t smem = pipeline > combine ? pipeline : combine;
  static bool smem_set = false;                               // per head size and depth: this function is a template
  int status = set_smem(decode_attention_kernel<D, STAGES>, smem, "decode_attention", smem_set);
  if (status != MIR_OK) return status;
  const int group = heads / kv_heads;
  const int units = kv_heads * ((group + kDecodeHeads - 1) / kDecodeHeads);
  const dim3 grid = rows <= 4 ? dim3(rows, units, num_partitions) : dim3(num_partitions, units, rows);
  status = mir_launch_with(mir_pdl_for_streaming(), "decode_attention", decode_attention_kernel<D, STAGES>, grid,
                           dim3(kDecodeWarps * 32), smem, stream, 0, q, q_stride, k_pages, v_pages, block_table,
                           table_width, positions, page_size, heads, kv_heads, scale * 1.4426950408889634f, window,
                           partition, num_partitions, rows <= 4 ? 1 : 0, partial_o, partial_ml, out);
  if (status != MIR_OK || num_partitions == 1) return status;
  return launch_merge<D>(partial_o, partial_ml, positions, rows, heads, window, partition, num_partitions, out, stream);
}

long long g_deep_ring_ctas = 1536;                              // up to this many CTAs run three tiles in flight per warp
template <int D>
int launch_decode(const bf16* q, size_t q_stride, bf16* out, const bf16* k_pages, const bf16* v_pages,
                  const int* block_table, int table_width, const int* positions, int rows, int page_size, int heads,
                  int kv_heads, float scale, int window, int partition, int num_partitions, float* partial_o,
                  float* partial_ml, cudaStream_t stream) {
  const int group = heads / kv_heads;
  const long long ctas = (long long)num_partitions * kv_heads * ((group + kDecodeHeads - 1) / kDecodeHeads) * rows;
  if (ctas <= g_deep_ring_ctas)
    return launch_decode_staged<D, 3>(q, q_stride, out, k_pages, v_pages, block_table, table_width, positions, rows,
                                      page_size, heads, kv_heads, scale, window, partition, num_partitions, partial_o,
                                      partial_ml, stream);
  return launch_decode_staged<D, 2>(q, q_stride, out, k_pages, v_pages, block_table, table_width, positions, rows,
                                    page_size, heads, kv_heads, scale, window, partition, num_partitions, partial_o,
                                    partial_ml, stream);
}

template <int D>
int launch_prefill(const bf16* q, size_t q_stride, bf16* out, const bf16* k_pages, const bf16* v_pages,
                   const int* block_table, int table_width, const int* query_starts, const int* context_lens,
                   int num_rows, int tokens, int page_size, int heads, int kv_heads, float scale, int window,
                   cudaStream_t stream) {
  const size_t smem = (size_t)2 * 2 * kKeyTile * (D + 8) * sizeof(bf16);
  static bool smem_set = false;
  int status = set_smem(prefill_attention_kernel<D>, smem, "prefill_attention", smem_set);
  if (status != MIR_OK) return status;
  const int tiles = (tokens + kQueryTile - 1) / kQueryTile + num_rows;   // an upper bound; spare CTAs return
  if (tiles > 65535) {
    mir_set_error("prefill_attention: %d tokens in %d rows are more than one launch takes", tokens, num_rows);
    return MIR_BAD_ARGUMENT;
  }
  return mir_launch("prefill_attention", prefill_attention_kernel<D>, dim3(heads, tiles), dim3(kPrefillWarps * 32),
                    smem, stream, 0, q, q_stride, out, k_pages, v_pages, block_table, table_width, query_starts,
                    context_lens, num_rows, page_size, heads, kv_heads, scale * 1.4426950408889634f, window);
}

bool bad_common(const char* what, int heads, int kv_heads, int head_dim, int page_size, int table_width, int window) {
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || page_size <= 0 || table_width <= 0 || window < 0) {
    mir_set_error("%s: bad sizes (heads %d, kv heads %d, page %d, table width %d)", what, heads, kv_heads, page_size,
                  table_width);
    return true;
  }
  if (head_dim != 64 && head_dim != 128) {
    mir_set_error("%s: head_dim %d is not one of 64, 128 (the reference kernel takes the other sizes)", what, head_dim);
    return true;
  }
  return false;
}

}  // namespace

// For measurements: up to how many CTAs split decode attention keeps three (instead of two) tiles in flight per warp.
MIR_EXPORT void mir_decode_attention_set_deep_ring_ctas(long long ctas) { g_deep_ring_ctas = ctas; }


// How many floats of scratch decode attention needs: partial outputs and (maximum, denominator) pairs.
// Arguments that cannot be meant (negative, or so large that the product would leave 63 bits) give -1.
MIR_EXPORT long long mir_decode_attention_scratch_floats(int rows, int heads, int head_dim, int num_partitions) {
  if (rows < 0 || heads < 0 || head_dim < 0 || num_partitions < 0) return -1;
  if (num_partitions <= 1) return 0;
  const unsigned __int128 floats = (unsigned __int128)rows * (unsigned)heads * (unsigned)num_partitions * (unsigned)(head_dim + 2);
  return floats > (unsigned __int128)(1ll << 62) ? -1 : (long long)floats;
}

// The merge of the partitions' results alone (the tcgen05 decode kernel leaves them in the same layout): scratch as
// mir_decode_attention_bf16 lays it out, partial outputs then (maximum, denominator) pairs.
MIR_EXPORT int mir_decode_merge_bf16(const float* partial_o, const float* partial_ml, const int* positions, int rows,
                                     int heads, int head_dim, int window, int partition, int num_partitions, void* out,
                                     cudaStream_t stream) {
  if (rows <= 0 || rows > 65535 || heads <= 0 || partition <= 0 || num_partitions <= 0 || window < 0 ||
      (head_dim != 64 && head_dim != 128) || partial_o == nullptr || partial_ml == nullptr) {
    mir_set_error("decode_merge: bad sizes (rows %d, heads %d, head_dim %d, partition %d, partitions %d)", rows, heads,
                  head_dim, partition, num_partitions);
    return MIR_BAD_ARGUMENT;
  }
  if (head_dim == 64)
    return launch_merge<64>(partial_o, partial_ml, positions, rows, heads, window, partition, num_partitions, (bf16*)out,
                            stream);
  return launch_merge<128>(partial_o, partial_ml, positions, rows, heads, window, partition, num_partitions, (bf16*)out,
                           stream);
}

// One token per row.  `partition` (a multiple of 64) is how many keys one CTA takes; num_partitions must be
// >= ceil(longest context / partition).  scratch holds mir_decode_attention_scratch_floats floats.
MIR_EXPORT int mir_decode_attention_bf16(const void* q, long long q_stride, void* out, const void* k_pages,
                                         const void* v_pages, const int* block_table, int table_width,
                                         const int* positions, int rows, int page_size, int heads, int kv_heads,
                                         int head_dim, float scale, int window, int partition, int num_partitions,
                                         float* scratch, long long scratch_floats, cudaStream_t stream) {
  if (rows == 0) return MIR_OK;
  if (bad_common("decode_attention", heads, kv_heads, head_dim, page_size, table_width, window)) return MIR_BAD_ARGUMENT;
  if (rows < 0 || rows > 65535 || partition <= 0 || partition % 64 || partition > kDecodeMaxPartition ||
      num_partitions <= 0 || num_partitions > 65535) {
    mir_set_error("decode_attention: bad rows %d, partition %d or partition count %d", rows, partition, num_partitions);
    return MIR_BAD_ARGUMENT;
  }
  const long long need = mir_decode_attention_scratch_floats(rows, heads, head_dim, num_partitions);
  if (need < 0 || (need > 0 && (scratch == nullptr || scratch_floats < need))) {
    mir_set_error("decode_attention: scratch of %lld floats is needed, got %lld", need, scratch_floats);
    return MIR_BAD_ARGUMENT;
  }
  float* partial_o = scratch;
  float* partial_ml = scratch ? scratch + (size_t)rows * heads * num_partitions * head_dim : nullptr;
  if (head_dim == 64)
    return launch_decode<64>((const bf16*)q, (size_t)q_stride, (bf16*)out, (const bf16*)k_pages, (const bf16*)v_pages,
                             block_table, table_width, positions, rows, page_size, heads, kv_heads, scale, window,
                             partition, num_partitions, partial_o, partial_ml, stream);
  return launch_decode<128>((const bf16*)q, (size_t)q_stride, (bf16*)out, (const bf16*)k_pages, (const bf16*)v_pages,
                            block_table, table_width, positions, rows, page_size, heads, kv_heads, scale, window,
                            partition, num_partitions, partial_o, partial_ml, stream);
}

// Any mix of portions: row r has tokens query_starts[r] .. query_starts[r+1]-1 of the packed batch, and its
// request holds context_lens[r] tokens after this step (so the portion starts at context_lens[r] - count).
MIR_EXPORT int mir_prefill_attention_bf16(const void* q, long long q_stride, void* out, const void* k_pages,
                                          const void* v_pages, const int* block_table, int table_width,
                                          const int* query_starts, const int* context_lens, int num_rows, int tokens,
                                          int page_size, int heads, int kv_heads, int head_dim, float scale,
                                          int window, cudaStream_t stream) {
  if (tokens == 0 || num_rows == 0) return MIR_OK;
  if (bad_common("prefill_attention", heads, kv_heads, head_dim, page_size, table_width, window)) return MIR_BAD_ARGUMENT;
  if (tokens < 0 || num_rows < 0) {
    mir_set_error("prefill_attention: bad tokens %d, rows %d or heads %d", tokens, num_rows, heads);
    return MIR_BAD_ARGUMENT;
  }
  if (head_dim == 64)
    return launch_prefill<64>((const bf16*)q, (size_t)q_stride, (bf16*)out, (const bf16*)k_pages, (const bf16*)v_pages,
                              block_table, table_width, query_starts, context_lens, num_rows, tokens, page_size, heads,
                              kv_heads, scale, window, stream);
  return launch_prefill<128>((const bf16*)q, (size_t)q_stride, (bf16*)out, (const bf16*)k_pages, (const bf16*)v_pages,
                             block_table, table_width, query_starts, context_lens, num_rows, tokens, page_size, heads,
                             kv_heads, scale, window, stream);
}

// ------------------------------------------------------------------------------------------------
// The variant for callers that cannot allocate (declared and explained in no_alloc.h): the partial
// results live in an array that is part of this library's device image.
#include <mutex>
#include "no_alloc.h"

static __device__ __align__(256) float g_static_decode_scratch[MIR_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_static_scratch_address[kMaxDevices] = {};      // device address of the array, per device, once known
std::mutex g_static_scratch_mutex;

// In host code the array's name only stands for the symbol; the address a kernel can use has to be asked
// for, with the device that will run the kernel current.  Done once per device.
int static_scratch_for_current_device(float** address) {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess || device < 0 || device >= kMaxDevices) {
    mir_set_error("decode_attention_static: cannot identify the current device: %s", cudaGetErrorString(err));
    return MIR_CUDA_ERROR;
  }
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_address[device] == nullptr) {
    void* found = nullptr;
    err = cudaGetSymbolAddress(&found, g_static_decode_scratch);
    if (err != cudaSuccess || found == nullptr) {
      mir_set_error("decode_attention_static: cudaGetSymbolAddress failed on device %d: %s", device,
                    cudaGetErrorString(err));
      return MIR_CUDA_ERROR;
    }
    g_static_scratch_address[device] = static_cast<float*>(found);
  }
  *address = g_static_scratch_address[device];
  return MIR_OK;
}
}  // namespace

MIR_EXPORT int mir_decode_attention_bf16_static(const void* q, long long q_stride, void* out, const void* k_pages,
                                                const void* v_pages, const int* block_table, int table_width,
                                                const int* positions, int rows, int page_size, int heads,
                                                int kv_heads, int head_dim, float scale, int window, int partition,
                                                int num_partitions, cudaStream_t stream) {
  if (rows == 0) return MIR_OK;
  // the same checks as the ordinary entry point, before any size is computed from the arguments
  if (bad_common("decode_attention_static", heads, kv_heads, head_dim, page_size, table_width, window)) return MIR_BAD_ARGUMENT;
  if (rows < 0 || rows > 65535 || partition <= 0 || partition % 64 || partition > kDecodeMaxPartition ||
      num_partitions <= 0) {
    mir_set_error("decode_attention_static: bad rows %d, partition %d or partition count %d", rows, partition,
                  num_partitions);
    return MIR_BAD_ARGUMENT;
  }
  const long long need = mir_decode_attention_scratch_floats(rows, heads, head_dim, num_partitions);
  if (need < 0 || need > (long long)MIR_STATIC_SCRATCH_FLOATS) {
    mir_set_error("decode_attention_static: this call needs %lld floats of scratch (rows %d x heads %d x partitions "
                  "%d x (head_dim %d + 2)), the built-in array holds %u; use fewer rows or partitions per call, or "
                  "mir_decode_attention_bf16 with scratch of your own",
                  need, rows, heads, num_partitions, head_dim, (unsigned)MIR_STATIC_SCRATCH_FLOATS);
    return MIR_BAD_ARGUMENT;
  }
  float* scratch = nullptr;
  if (need > 0) {
    const int status = static_scratch_for_current_device(&scratch);
    if (status != MIR_OK) return status;
  }
  return mir_decode_attention_bf16(q, q_stride, out, k_pages, v_pages, block_table, table_width, positions, rows,
                                   page_size, heads, kv_heads, head_dim, scale, window, partition, num_partitions,
                                   scratch, need, stream);
}
