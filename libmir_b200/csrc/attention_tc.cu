// Causal attention of prompt portions over the paged cache on the 5th-generation tensor cores (tcgen05),
// head_dim 128, bf16:
//
//   out[i] = softmax_j(scale q_i . k_j) v_j     over the keys j <= position(i) (and inside the window, if any)
//
// A work item is 128 consecutive query tokens of one request and one head; a CTA (one per SM) walks over the
// request's keys in tiles of 128 for one item after the other (the heaviest items first, dealt out to the CTAs back
// and forth so that every CTA gets about the same number of key tiles), and every ring and barrier runs on across
// the items: the loaders fetch the next item's queries and first keys while the softmax threads still merge and
// write the last item's result, which took half of a CTA's life when every item had a CTA of its own.
// Per tile:  S = Q K^T  (tcgen05.mma, 128 x 128 x 128, accumulator in tensor memory),  P = exp2(scale S - m) by the
// softmax threads (one query row per thread, read with tcgen05.ld and written back with tcgen05.st as packed bf16
// pairs over the scores they came from: the A operand of the next product stays in tensor memory and never
// touches shared memory),  O += P V  (tcgen05.mma with A in tensor memory, accumulator stays in tensor memory for
// the whole row of tiles).  Roles:
//
//   loaders   two warps for keys (the CTA's even and odd tiles; the first also fetches Q, once per item), one for
//             values, into a ring of three key tiles and one of two value tiles (cp.async.bulk.tensor.2d through
//             tensor maps over the cache, 128-byte swizzle).  A copy instruction costs a warp about 75 cycles for every
//             lane that takes part, so where a tile's pages lie one behind the other in the pool (while the pool is
//             not fragmented they do) two lanes fetch the tile as two boxes of 128 keys; else one lane per page and
//             64-wide half of the head (16 lanes for pages of 16 keys: 1,200 cycles, which then set the kernel's
//             pace).  Pages the block table does not have (-1) are skipped.  The rest of a tile's work is a handful of
//             instructions (what does not change with the tile is worked out per item, stages are counted, the block
//             table is read two tiles ahead).  Registers are handed out to four warps at a time: the twentieth warp
//             costs the others nothing.
//   issuer    one warp that stays converged; the products are predicated on its elected lane and take their
//             descriptors as 32-bit halves (tcgen05.cuh says why: a lone thread in a divergent branch fed the tensor
//             cores a 64-cycle product only every 80 to 95 cycles beside the softmax warps).  Three score
//             accumulators and one for the output: S(t+3) = Q K(t+3)^T takes the accumulator that holds P(t), so it
//             is issued right behind O += P(t) V(t) (the tensor cores run products in the order of issue), and the
//             scores of a stream's next tile are there before its softmax of this one is over.
//   softmax   two streams of eight warps take the key tiles in turn (stream s the tiles t = s, s + 2, ...), so that
//             while one computes exponentials the other reads scores, finds its maximum and writes P.  A row has one
//             running reference (its maximum, raised only when a tile's maximum exceeds it by more than 2^8), which
//             the streams hand to each other through shared memory tile by tile (REF_READY; the value is known right
//             after a tile's maximum, long before its exponentials are done), one output accumulator, and a partial
//             denominator per stream, which are added when the row of tiles is over.  The stream that raises the
//             reference rescales O (tcgen05.ld / tcgen05.st) once the product of the tile before has ended (PV_DONE);
//             the product with its own P is not issued before it arrives, so nothing else touches O meanwhile.
//             Within a stream, query row r = accumulator lane r belongs to two threads, which take 64 columns each
//             (of the scores; 32 of P) and share the row's maximum through shared memory.
//             (kShared = false is the form this one replaced, kept for measurements: every stream with a reference,
//             a denominator and an output accumulator of its own over its tiles, two score accumulators, the two
//             results merged at the end.  There a stream's next scores can only be issued behind its product with V,
//             because P lies over the scores and tensor memory has no room for a third accumulator beside two
//             outputs: softmax, product and next scores of a stream form a chain of 1,800 + 1,040 cycles.)
//
// V is read as an MN-major operand (rows of keys, 64 head elements per 128-byte row) exactly as the cache stores
// it; nothing is transposed.  A hidden key's score is set to -inf by selection (in tiles that hide any), never by
// arithmetic on what the cache holds there, so its probability is exactly 0; the V ring starts zeroed, so a skipped
// page cannot inject a NaN (0 x NaN) into O.
// Every wait is bounded in time; a role whose wait runs out raises g_tc_attention_error and stops waiting, the
// CTA still frees its tensor memory and returns.
// libmir computes prompt attention with a library plan (FmhaBf16Plan of its external mircuda crate,
// cuda/src/backend/attention/prefill/varlen.rs:1-23) or, over pages, with one thread block per token
// (cuda/kernels/paged_prefill_attention_batch_bf16.cu:30-35,52-123); the formula as the Metal engine states it is
// metal/src/engine/dense/swiglu/attention.rs:93-107.
#include <algorithm>
#include "tcgen05.cuh"
#include "trace.cuh"

using namespace mir;
using namespace mir::tc;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kRows = 128;                  // query tokens per work item
constexpr int kKeys = 128;                  // keys per tile
constexpr int kDim = 128;                   // head_dim
constexpr int kHalf = 128 * 128;            // bytes of a 128-row x 64-element half tile
constexpr int kTile = 2 * kHalf;            // 32 KB
constexpr int kKeyStages = 3;              // the key ring: a tile is asked for when the product with the one three back is over
constexpr int kOffQ = 0, kOffK = kTile, kOffV = (1 + kKeyStages) * kTile;
constexpr int kSmemBytes = (3 + kKeyStages) * kTile + 1024;
constexpr int kParts = 2;                   // softmax threads per query row and stream (each takes 64 columns)
constexpr int kCols = kKeys / kParts;       // columns of a tile that one softmax thread handles
constexpr int kStreamThreads = kRows * kParts;
// key loader (even tiles), issuer, eight softmax warps per stream, value loader, key loader (odd tiles): registers are
// handed out to four warps at a time, so the twentieth warp costs the others nothing
__host__ __device__ constexpr int threads_for(int streams) { return (4 + 8 * streams) * 32; }
constexpr int kFirstSoftmaxWarp = 2;
constexpr uint32_t kTmemColumns = 512;      // S0 at 0, S1 at 128, O of stream 0 at 256, of stream 1 at 384
constexpr float kRescaleThreshold = 8.0f;   // log2 of how far a tile's maximum may exceed the running one

// barrier indices
enum { Q_FULL = 0, K_FULL = 1, K_FREE = K_FULL + kKeyStages, V_FULL = K_FREE + kKeyStages, V_FREE = V_FULL + 2,
       S_FULL = V_FREE + 2, P_READY = S_FULL + 3, ITEM_DONE = P_READY + 3, Q_FREE, O_FREE, REF_READY, PV_DONE = REF_READY + 2,
       BARRIERS = PV_DONE + 2 };
// Tiles are counted over all items of a CTA (g): stage g & 1 of the value ring (and of REF_READY, PV_DONE), phase
// parity (g >> 1) & 1; the key ring and the score accumulators: g % 3 and (g / 3) & 1, kept as running counters where
// a role sees every tile (with kShared = false the score accumulators go by g & 1).  P_READY has one barrier per
// score accumulator: the two streams work on neighbouring tiles at the same time, and the arrivals of one must not
// count for the other's tile.  Items are counted too (n): Q_FULL, Q_FREE,
// ITEM_DONE and O_FREE complete once per item.
__device__ int g_tc_attention_error = 0;
int g_streams = 2;
int g_shared = 1;                           // the streams share a row's reference and one output accumulator
int g_ctas = 0;                             // for measurements: 0 = one CTA per SM

#ifdef MIR_TRACE
// Cycle stamps (clock64 of the SM) of the first CTA's key tiles, one row of 16 per tile counted over its items:
// 0 keys requested, 1 values requested, 2 scores issued, 3 issuer starts waiting for P, 4 issuer has P (product with
// V issued next), 5 softmax starts waiting for the scores, 6 has them, 7 has read them, 8 knows the row's maximum,
// 9 has the exponentials, 10 has written P and arrived (the softmax stamps: first warp of each stream); issuer again:
// 11 starts waiting for the keys, 12 has them, 13 starts waiting for the values (3: has them), 14 product with V issued;
// key loader: 15 keys' copies issued.  Rows 200 + n hold the end of the CTA's n-th item as its first softmax warp
// sees it: 0 its tiles are done, 1 the streams have exchanged maxima and denominators, 2 the item's last product is
// over, 3 the accumulators are read, 4 the rows are stored; 5 (row of the next item) the next item is known.
constexpr int kTraceTiles = 256;
__device__ long long g_prompt_tiles[kTraceTiles * 16];
#define ATT_STAMP(tile, index)                                                                  \
  do {                                                                                          \
    if (blockIdx.x == 0 && (tile) >= 0 && (tile) < kTraceTiles) g_prompt_tiles[(tile) * 16 + (index)] = clock64(); \
  } while (0)
#else
#define ATT_STAMP(tile, index) do { } while (0)
#endif

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 32 consecutive accumulator columns of this thread's lane, without waiting for them (tmem_load_wait()).
__device__ __forceinline__ void tmem_load_32_nowait(uint32_t address, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(address)
      : "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// One tile of the softmax for this thread's part (kCols columns starting at `first`) of its row: the scores are
// read once (all loads in flight, one wait), then the visible maximum (columns low..high of the tile; all if
// !MASKED: the hidden ones are set to -inf first), which the kParts threads of a row exchange through `shared_max` (one float per part, kRows apart)
// and the named barrier `team` of the stream's warps that hold the row's quarter of lanes; then the decision whether
// the running maximum rises, and p = exp2(scale s - reference) packed to bf16.  Returns the sum of this thread's p.
// With a reference that the streams share (SHARED): the row's reference after the tile before comes from the other
// stream (`from`: its barrier and where it left the value; none for an item's first tile), this tile's is left for the
// next (`to`); `reference` is then the one this thread's partial denominator is scaled to, `factor` what the output
// accumulator has to be multiplied by (if `grow`), `own_factor` what the denominator has to be.
struct Handoff {
  bool has_from;
  uint32_t from_barrier, from_parity;
  const float* from;
  uint32_t to_barrier;
  float* to;
};
template <bool MASKED, bool SHARED>
__device__ __forceinline__ float softmax_tile(uint32_t scores, int first, int low, int high, float scale_log2,
                                              float& reference, float& factor, bool& grow,
                                              uint32_t (&packed)[kCols / 2], float* shared_max, int part, int team,
                                              int stamp_tile, const Handoff& handoff, float& own_factor, bool& alive) {
  float v[kCols];
#pragma unroll
  for (int c0 = 0; c0 < kCols; c0 += 32) tmem_load_32_nowait(scores + first + c0, v + c0);
  tmem_load_wait();
#pragma unroll
  for (int c = 0; c < kCols; ++c) asm volatile("" : "+f"(v[c])::"memory");   // no use of v moves above the wait
  ATT_STAMP(stamp_tile, 7);
  if (MASKED) {
    // a hidden key's score becomes -inf by selection (whatever the cache held there, a NaN too), once; from here on
    // the tile is handled like any other: -inf never wins the maximum and its exponential is exactly 0
    const int lo = low - first, hi = high - first;
#pragma unroll
    for (int c = 0; c < kCols; ++c) v[c] = (c >= lo && c <= hi) ? v[c] : -INFINITY;
  }
  float best[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};        // four chains instead of one
#pragma unroll
  for (int c = 0; c < kCols; ++c) best[c & 3] = fmaxf(best[c & 3], v[c]);
  float maximum = fmaxf(fmaxf(best[0], best[1]), fmaxf(best[2], best[3]));
  shared_max[part * kRows] = maximum;
  asm volatile("bar.sync %0, %1;" ::"r"(team), "n"(32 * kParts) : "memory");
#pragma unroll
  for (int other = 0; other < kParts; ++other) maximum = fmaxf(maximum, shared_max[other * kRows]);
  ATT_STAMP(stamp_tile, 8);
  maximum *= scale_log2;                                               // scale > 0
  if (SHARED) {
    float before = -INFINITY;
    if (handoff.has_from) {
      if (alive && !wait_barrier(handoff.from_barrier, handoff.from_parity)) { g_tc_attention_error = 3; alive = false; }
      before = *handoff.from;
    }
    const float now = maximum > before + kRescaleThreshold ? maximum : before;
    if (part == 0) *handoff.to = now;
    barrier_arrive(handoff.to_barrier);
    grow = now != before;
    factor = grow ? fast_exp2(before - now) : 1.0f;                    // 0 when nothing was seen before
    own_factor = reference == now ? 1.0f : fast_exp2(reference - now); // (-inf - -inf is no number: the first branch)
    reference = now;
  } else {
    grow = maximum > reference + kRescaleThreshold;
    factor = grow ? fast_exp2(reference - maximum) : 1.0f;             // 0 when nothing was seen before
    reference = grow ? maximum : reference;
    own_factor = factor;
  }
  // (a row that has seen no key yet, in this tile either, has reference -inf: -inf - -inf would not be a number)
  const float shift = (MASKED && reference == -INFINITY) ? 0.0f : -reference;
  float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
  for (int c = 0; c < kCols; c += 2) {
    const float p0 = fast_exp2(fmaf(v[c], scale_log2, shift));
    const float p1 = fast_exp2(fmaf(v[c + 1], scale_log2, shift));
    sums[(c >> 1) & 3] += p0 + p1;
    const __nv_bfloat162 pair2 = __floats2bfloat162_rn(p0, p1);
    packed[c >> 1] = *reinterpret_cast<const uint32_t*>(&pair2);
  }
  return (sums[0] + sums[1]) + (sums[2] + sums[3]);
}

// What one work item is: which queries, which keys.
struct Work {
  bool valid;
  int head, kv_head, q_row0, tile_rows, first_position, last_position, first_key, key_begin, key_end, tiles;
  const int* table;
};

// Item `index` of the launch: head = index % heads (the fast index, so that the heads of a group, which read the
// same keys, run at the same time), and the batch's `query_tiles` query tiles from the last one of the last row
// backwards (late tiles see the most keys: they come first).
__device__ __forceinline__ Work work_item(int index, int items, int query_tiles, int heads, int kv_heads, int num_rows,
                                          const int* __restrict__ query_starts, const int* __restrict__ context_lens,
                                          const int* __restrict__ block_table, int table_width, int window) {
  Work w;
  w.valid = false;
  if (index < 0 || index >= items) return w;
  w.head = index % heads;
  w.kv_head = w.head / (heads / kv_heads);
  int remaining = query_tiles - 1 - index / heads;
  int row = -1, local_tile = 0;
  for (int r = 0; r < num_rows; ++r) {
    const int tiles = (query_starts[r + 1] - query_starts[r] + kRows - 1) / kRows;
    if (remaining < tiles) { row = r; local_tile = remaining; break; }
    remaining -= tiles;
  }
  if (row < 0) return w;
  const int q_begin = query_starts[row];
  const int count = query_starts[row + 1] - q_begin;
  const int start_position = context_lens[row] - count;
  const int local0 = local_tile * kRows;
  w.q_row0 = q_begin + local0;
  w.tile_rows = min(kRows, count - local0);
  w.first_position = start_position + local0;
  w.last_position = w.first_position + w.tile_rows - 1;
  w.table = block_table + (size_t)row * table_width;
  w.first_key = (window > 0 && w.first_position + 1 > window) ? w.first_position + 1 - window : 0;
  w.key_begin = w.first_key / kKeys * kKeys;
  w.key_end = w.last_position + 1;                            // exclusive
  w.tiles = (w.key_end - w.key_begin + kKeys - 1) / kKeys;
  w.valid = true;
  return w;
}

// The k-th item of CTA `cta` of `ctas`: round k deals the items k * ctas .. (k + 1) * ctas - 1 out forwards if k is
// even and backwards if it is odd, so that the CTA that got the heaviest item of one round gets the lightest of the
// next.  -1 when the rounds are over.
__device__ __forceinline__ int item_of(int k, int cta, int ctas, int items) {
  if ((long long)k * ctas >= items) return -1;
  return k * ctas + ((k & 1) ? ctas - 1 - cta : cta);
}

template <int kStreams, bool kShared>
__global__ void __launch_bounds__(threads_for(kStreams), 1)
tc_prefill_attention_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                            const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap k_tile_map,
                            const __grid_constant__ CUtensorMap v_tile_map, bf16* __restrict__ out,
                            const int* __restrict__ block_table, int table_width, const int* __restrict__ query_starts,
                            const int* __restrict__ context_lens, int num_rows, int page_size, int heads, int kv_heads,
                            float scale_log2, int window, int tile_slots) {
  constexpr int kThreads = threads_for(kStreams);
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long barriers[BARRIERS];
  __shared__ uint32_t tmem_base_slot;
  __shared__ float exchange[kStreams][2][kParts][kRows];     // [stream][its tile parity][part][row]: a row's maxima
  __shared__ float denominators[2][kStreams][kParts][kRows]; // [item parity]...: a slow thread may still read the last item's
  __shared__ float references[2][kStreams][kRows];
  __shared__ float handed[2][kRows];                          // kShared: a row's reference after the CTA's tile g, by g & 1
  __shared__ int query_tiles_slot;
  if (*reinterpret_cast<volatile int*>(&g_tc_attention_error) != 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, ctas = gridDim.x;

  grid_launch_dependents();
  grid_dependency_wait();
  if (threadIdx.x == 0) {
    // how many query tiles the batch really has (the launch was sized for at most tile_slots)
    int total = 0;
    for (int r = 0; r < num_rows; ++r) total += (query_starts[r + 1] - query_starts[r] + kRows - 1) / kRows;
    query_tiles_slot = min(total, tile_slots);
  }
  __syncthreads();
  const int query_tiles = query_tiles_slot;
  const int items = heads * query_tiles;
  auto work = [&](int k) {
    return work_item(item_of(k, cta, ctas, items), items, query_tiles, heads, kv_heads, num_rows, query_starts,
                     context_lens, block_table, table_width, window);
  };
  auto more = [&](int k) { return (long long)k * ctas < items; };

  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar0 = smem_u32(&barriers[0]);
  auto bar = [&](int index) { return bar0 + 8u * (uint32_t)index; };
  if (threadIdx.x == 0) {
    for (int i = 0; i < BARRIERS; ++i) {
      const bool many = (i >= P_READY && i < P_READY + 3) || i == REF_READY || i == REF_READY + 1;   // a stream's threads arrive
      const bool all = i == O_FREE;                                        // every softmax thread of every stream
      barrier_init(bar(i), all ? (uint32_t)(kStreamThreads * kStreams) : (many ? (uint32_t)kStreamThreads : 1u));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // the V ring starts as zeros (see the note on skipped pages above)
  for (int i = threadIdx.x; i < 2 * kTile / 16; i += kThreads)
    *reinterpret_cast<uint4*>(smem + kOffV + (size_t)i * 16) = make_uint4(0u, 0u, 0u, 0u);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(kTmemColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tensor_fence_before_sync();
  __syncthreads();
  tensor_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  // split keys: S0 at 0, S1 at 128, O of stream 0 at 256, of stream 1 at 384; shared reference: S0, S1, S2, O at 384
  const uint32_t tmem_o = tmem_base + (kShared ? 384u : 256u);

  constexpr int kValueLoader = kFirstSoftmaxWarp + 8 * kStreams;   // the warp behind the softmax warps
  if (warp == 0 || warp >= kValueLoader) {
    // ------------------------------------------------------------------ loaders: warp 0 keys (and Q), the last warp
    // values (apart, so that the keys of a later tile do not queue behind values whose stage is still being read).
    // These warps share their schedulers with four softmax warps each and every instruction of theirs takes long, so
    // a tile costs them as few as can be: everything that does not change with the tile is worked out before the
    // loop, the stage and its parity are counted, not divided, and the block table is read two tiles ahead.
    const int which = warp == kValueLoader ? 1 : 0;           // keys or values
    // the keys have two loaders, which take the CTA's even and odd tiles (one loader's loop set the kernel's pace)
    const int turns = which ? 1 : 2, turn = warp == 0 ? 0 : 1;
    const int page_shift = 31 - __clz(page_size);             // pages are powers of two (they divide 128)
    const int pages_per_tile = kKeys >> page_shift;
    const uint32_t box_bytes = (uint32_t)page_size * 128u;
    // lane l loads half (l & 1) of page slot (l >> 1): at most 16 pages of 8 keys, so one round of 32 lanes
    const int slot = lane >> 1, half = lane & 1;
    const bool loads = lane < 2 * pages_per_tile;
    const uint32_t lane_dst = smem_base + (which ? kOffV : kOffK) + (uint32_t)half * kHalf +
                              (uint32_t)(slot * page_size) * 128u;
    const CUtensorMap* map = which ? &v_map : &k_map;
    const CUtensorMap* tile_map = which ? &v_tile_map : &k_tile_map;     // boxes of 128 keys
    const uint32_t tile_dst = smem_base + (which ? kOffV : kOffK);
    const int stages = which ? 2 : kKeyStages;
    const uint32_t full0 = bar(which ? V_FULL : K_FULL), free0 = bar(which ? V_FREE : K_FREE);
    int stage = 0;                                            // of the CTA's tile g = g0 + t: g % stages,
    uint32_t parity = 0;                                      // (g / stages) & 1
    int g0 = 0, n = 0;
    bool alive = true;
    for (int k = 0; more(k) && alive; ++k) {
      const Work w = work(k);
      if (!w.valid) continue;
      if (warp == 0) {
        // the queries, once the products with the last item's are over
        if (n > 0 && !wait_barrier(bar(Q_FREE), (uint32_t)(n - 1) & 1u)) { g_tc_attention_error = 1; break; }
        if (lane == 0) {
          barrier_expect_bytes(bar(Q_FULL), kTile);
          tma_load_2d(smem_base + kOffQ, &q_map, bar(Q_FULL), w.head * kDim, w.q_row0);
          tma_load_2d(smem_base + kOffQ + kHalf, &q_map, bar(Q_FULL), w.head * kDim + 64, w.q_row0);
        }
      }
      const int x = w.kv_head * kDim + half * 64;
      const int lane_key = w.key_begin + slot * page_size;    // the first key of this lane's page in tile 0
      const int* entry = w.table + (lane_key >> page_shift);  // its block table entry; pages_per_tile further per tile
      const int tiles = w.tiles, key_end = w.key_end, first_visible = w.first_key - page_size;
      auto page_of = [&](int t) {
        const int key = lane_key + t * kKeys;
        return (loads && t < tiles && key < key_end && key > first_visible) ? entry[t * pages_per_tile] : -1;
      };
      // this loader's tiles of the item: every one, or those whose number in the CTA is even (odd)
      const int first_tile = turns == 1 ? 0 : ((g0 & 1) == turn ? 0 : 1);
      if (turns == 2 && first_tile == 1) {                     // (the ring's other loader has tile 0)
        if (++stage == stages) { stage = 0; parity ^= 1u; }
      }
      int page_next = page_of(first_tile), page_after = page_of(first_tile + turns);
      for (int t = first_tile; t < tiles; t += turns) {
        const int page = page_next;
        page_next = page_after;
        page_after = page_of(t + 2 * turns);                  // on its way while these tiles' stages are awaited
        const uint32_t full = full0 + 8u * (uint32_t)stage;
        if (!wait_barrier(free0 + 8u * (uint32_t)stage, parity ^ 1u)) { g_tc_attention_error = 1; alive = false; break; }
        if (lane == 0) ATT_STAMP(g0 + t, which);
        // A copy instruction costs the warp about 75 cycles for every lane that takes part (16 lanes: 1,200 cycles a
        // tile, which set the kernel's pace).  Where the tile's pages lie one behind the other in the pool, as they do
        // while the pool is not fragmented, two lanes fetch the whole tile, one box of 128 keys for each half.
        const int first_page = __shfl_sync(0xffffffffu, page, 0);
        const bool in_a_row = first_page >= 0 && __all_sync(0xffffffffu, !loads || page == first_page + slot);
        if (in_a_row) {
          if (lane == 0) barrier_expect_bytes(full, kTile);
          __syncwarp();
          if (lane < 2)
            tma_load_2d(tile_dst + (uint32_t)lane * kHalf + (uint32_t)stage * kTile, tile_map, full,
                        w.kv_head * kDim + lane * 64, first_page << page_shift);
        } else {
          const unsigned valid = __ballot_sync(0xffffffffu, page >= 0);
          if (lane == 0) barrier_expect_bytes(full, (uint32_t)__popc(valid) * box_bytes);
          __syncwarp();
          if (page >= 0) tma_load_2d(lane_dst + (uint32_t)stage * kTile, map, full, x, page << page_shift);
        }
        if (lane == 0 && which == 0) ATT_STAMP(g0 + t, 15);
        if (++stage == stages) { stage = 0; parity ^= 1u; }
        if (turns == 2 && t + 1 < tiles) {                     // the other loader's tile
          if (++stage == stages) { stage = 0; parity ^= 1u; }
        }
      }
      g0 += tiles;
      ++n;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ issuer: the whole warp stays converged, the
    // products are predicated on the elected lane (see tcgen05.cuh on issuing from a whole warp)
    constexpr uint32_t idesc_qk = instruction_descriptor(kRows, kKeys, false);
    constexpr uint32_t idesc_pv = instruction_descriptor(kRows, kDim, true);
    const uint32_t elected = elect_one();
    const uint32_t q_low = operand_low(smem_base + kOffQ), k_low = operand_low(smem_base + kOffK);
    const uint32_t v_low = operand_low_mn_major(smem_base + kOffV, kHalf);
    bool alive = true;
    int g0 = 0, n = 0;
    uint32_t key_stage = 0, key_parity = 0;                   // of the next tile of scores: g % kKeyStages, (g / kKeyStages) & 1
    uint32_t p_stage = 0, p_parity = 0;                       // kShared: of the next product with V: g % 3, (g / 3) & 1
    static_assert(!kShared || kKeyStages == 3, "the score accumulators go round with the key ring");
    for (int k = 0; more(k); ++k) {
      const Work w = work(k);
      if (!w.valid) continue;
      const int tiles = __shfl_sync(0xffffffffu, w.tiles, 0);             // (tells the compiler it is warp-uniform)
      if (alive && !wait_barrier(bar(Q_FULL), (uint32_t)n & 1u)) { g_tc_attention_error = 2; alive = false; }
      auto issue_scores = [&](int t) {
        const int g = g0 + t;
        const uint32_t stage = (uint32_t)g & 1u;
        if (elected) ATT_STAMP(g, 11);
        if (alive && !wait_barrier(bar(K_FULL + key_stage), key_parity)) { g_tc_attention_error = 2; alive = false; }
        if (elected) ATT_STAMP(g, 12);
        tensor_fence_after_sync();
        // (with the shared reference the scores have three buffers and go round with the key ring)
        const uint32_t score_stage = kShared ? key_stage : stage;
        const uint32_t b_low = k_low + key_stage * (uint32_t)(kTile >> 4), d = tmem_base + score_stage * 128u;
        mma_bf16_ss_halves<false>(d, q_low, b_low, idesc_qk, elected);
#pragma unroll
        for (int kk = 1; kk < kDim / 16; ++kk) {
          constexpr uint32_t kHalfStep = (uint32_t)(kHalf >> 4);
          const uint32_t offset = (uint32_t)(kk >> 2) * kHalfStep + (uint32_t)(kk & 3) * 2u;
          mma_bf16_ss_halves<true>(d, q_low + offset, b_low + offset, idesc_qk, elected);
        }
        mma_commit_elected(bar(S_FULL + score_stage), elected);
        mma_commit_elected(bar(K_FREE + key_stage), elected);
        if (elected) ATT_STAMP(g, 2);
        if (t == tiles - 1) mma_commit_elected(bar(Q_FREE), elected);   // the item's last product with its queries
        if (++key_stage == (uint32_t)kKeyStages) { key_stage = 0; key_parity ^= 1u; }   // (scores are issued in order)
      };
      // P(t) is written over S(t) in tensor memory, so S(t + 2), which takes the same accumulator, is issued
      // behind the product with P(t): the tensor cores run products in the order of issue, and while they work
      // on one stream's tile the other stream's softmax threads work on theirs
      // With the shared reference there are three score accumulators and one for the output: S(t + 3) takes the one
      // that holds P(t), and a stream's next scores are there before its softmax of this tile is over.
      constexpr int kAhead = kShared ? 3 : 2;
      issue_scores(0);
      if (tiles > 1) issue_scores(1);
      if (kShared && tiles > 2) issue_scores(2);
      for (int t = 0; t < tiles; ++t) {
        const int g = g0 + t;
        const uint32_t stage = (uint32_t)g & 1u;
        const uint32_t parity = (uint32_t)(g >> 1) & 1u;
        if (elected) ATT_STAMP(g, 13);
        if (alive && !wait_barrier(bar(V_FULL + stage), parity)) { g_tc_attention_error = 2; alive = false; }
        if (elected) ATT_STAMP(g, 3);
        const uint32_t p_slot = kShared ? p_stage : stage, p_turn = kShared ? p_parity : parity;
        if (alive && !wait_barrier(bar(P_READY + p_slot), p_turn)) { g_tc_attention_error = 2; alive = false; }
        if (elected) ATT_STAMP(g, 4);
        // the output accumulators are the last item's until every softmax thread has read them out
        if (t == 0 && n > 0 && alive && !wait_barrier(bar(O_FREE), (uint32_t)(n - 1) & 1u)) {
          g_tc_attention_error = 2;
          alive = false;
        }
        tensor_fence_after_sync();
        const uint32_t p = tmem_base + p_slot * 128u;
        const uint32_t b_low = v_low + stage * (uint32_t)(kTile >> 4);
        const uint32_t o = kShared ? tmem_o : tmem_o + (uint32_t)(t % kStreams) * 128u;
        // P: 16 keys are 8 columns of packed pairs further on; V: 16 rows of keys (2 KB) further down
        mma_bf16_ts_halves(o, p, b_low, idesc_pv, t >= (kShared ? 1 : kStreams) ? 1u : 0u, elected);
#pragma unroll
        for (int kk = 1; kk < kKeys / 16; ++kk)
          mma_bf16_ts_halves(o, p + (uint32_t)kk * 8u, b_low + (uint32_t)kk * (2048u >> 4), idesc_pv, 1u, elected);
        mma_commit_elected(bar(V_FREE + stage), elected);
        if (kShared) {
          mma_commit_elected(bar(PV_DONE + stage), elected);  // (a stream that raises the reference waits for it)
          if (++p_stage == 3u) { p_stage = 0; p_parity ^= 1u; }
        }
        if (elected) ATT_STAMP(g, 14);
        if (t == tiles - 1) mma_commit_elected(bar(ITEM_DONE), elected);
        if (t + kAhead < tiles) issue_scores(t + kAhead);
      }
      g0 += tiles;
      ++n;
    }
  } else {
    // ------------------------------------------------------------------ softmax: kStreams streams of eight warps
    const int stream = (warp - kFirstSoftmaxWarp) >> 3;       // takes the tiles t = stream, stream + kStreams, ...
    const int quarter = warp & 3;                             // the accumulator lanes this warp may touch
    const int part = ((warp - kFirstSoftmaxWarp) >> 2) & 1;   // which kCols columns of the row it takes
    const int r = quarter * 32 + lane;
    const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
    const int first = part * kCols;
    const uint32_t my_o = tmem_o + (kShared ? 0u : (uint32_t)stream * 128u) + lane_bits;
    bool alive = true;
    // (a thread whose wait ran out keeps walking the tiles without waiting, so that the row's named barrier
    // still sees all of its threads)
    int g0 = 0, n = 0;
    for (int k = 0; more(k); ++k) {
      const Work w = work(k);
      if (!w.valid) continue;
      ATT_STAMP(((lane == 0 && quarter == 0 && part == 0 && stream == 0) ? 200 + n : -1), 5);
      const bool valid_row = r < w.tile_rows;
      const int position = w.first_position + min(r, w.tile_rows - 1);
      float reference = -INFINITY, denominator = 0.0f;        // running maximum (scaled, log2 domain), partial sum
      for (int t = stream; t < w.tiles; t += kStreams) {
        const int g = g0 + t;
        const int stage = kShared ? g % 3 : g & 1;            // the score accumulator of the tile
        const uint32_t parity = (uint32_t)(kShared ? g / 3 : g >> 1) & 1u;
        const int key0 = w.key_begin + t * kKeys;
        const int stamp_tile = (lane == 0 && quarter == 0 && part == 0) ? g : -1;
        ATT_STAMP(stamp_tile, 5);
        if (alive && !wait_barrier(bar(S_FULL + stage), parity)) { g_tc_attention_error = 3; alive = false; }
        ATT_STAMP(stamp_tile, 6);
        tensor_fence_after_sync();
        const uint32_t scores = tmem_base + (uint32_t)stage * 128u + lane_bits;
        // keys of this tile that row r may see: columns [low, high]; most tiles are visible to every row
        const int high = position - key0;                     // last visible column, may be >= 128 or < 0
        const int low = window > 0 ? position - window + 1 - key0 : -1;
        const bool every = key0 + kKeys - 1 <= w.first_position && (window == 0 || w.last_position - window + 1 <= key0);
        uint32_t packed[kCols / 2];
        bool grow;
        float factor;
        float* shared_max = &exchange[stream][(t / kStreams) & 1][0][r];
        const int team = 1 + stream * 4 + quarter;
        Handoff handoff;
        handoff.has_from = kShared && t > 0;                  // the row's reference after the CTA's tile g - 1
        handoff.from_barrier = bar(REF_READY + ((g - 1) & 1));
        handoff.from_parity = (uint32_t)((g - 1) >> 1) & 1u;
        handoff.from = &handed[(g - 1) & 1][r];
        handoff.to_barrier = bar(REF_READY + (g & 1));
        handoff.to = &handed[g & 1][r];
        float own_factor;
        const float sum = every ? softmax_tile<false, kShared>(scores, first, low, high, scale_log2, reference, factor, grow,
                                                               packed, shared_max, part, team, stamp_tile, handoff,
                                                               own_factor, alive)
                                : softmax_tile<true, kShared>(scores, first, low, high, scale_log2, reference, factor, grow,
                                                              packed, shared_max, part, team, stamp_tile, handoff,
                                                              own_factor, alive);
        ATT_STAMP(stamp_tile, 9);
        denominator = denominator * own_factor + sum;
        // Split keys: this stream's previous product (tile t - kStreams) is over: S(t) was issued behind it, and the
        // scores' barrier completes only when everything issued before it has.  So its O may be rescaled now.
        // Shared reference: the one accumulator holds the products up to tile t - 1, whose end is waited for (the
        // product with this tile's P is not issued before this stream arrives, so nothing else touches O meanwhile).
        const bool rescale = (kShared ? t > 0 : t >= kStreams) && __any_sync(0xffffffffu, grow);
        if (kShared && rescale) {
          if (alive && !wait_barrier(bar(PV_DONE + ((g - 1) & 1)), (uint32_t)((g - 1) >> 1) & 1u)) {
            g_tc_attention_error = 3;
            alive = false;
          }
          tensor_fence_after_sync();
        }
        if (rescale) {
#pragma unroll 1
          for (int c0 = 0; c0 < kDim / kParts; c0 += 32) {
            float o[32];
            tmem_load_32(my_o + first + c0, o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= factor;
            tmem_store_32(my_o + first + c0, o);
          }
        }
        // P as the A operand of the product with V, in tensor memory over the scores it came from: this row's lane,
        // two keys per 32-bit column, this thread's kCols keys from column first / 2 on (its partner has read its
        // half of the scores: the two met at the row's barrier inside softmax_tile)
        tmem_store_32_bits(scores + (uint32_t)(first / 2), packed);
        tmem_store_wait();
        tensor_fence_before_sync();
        barrier_arrive(bar(P_READY + stage));
        ATT_STAMP(stamp_tile, 10);
      }
      // every softmax thread learns every stream's maximum and denominator (the sum of its two threads' parts)
      [[maybe_unused]] const int stamp_item = (lane == 0 && quarter == 0 && part == 0 && stream == 0) ? 200 + n : -1;
      ATT_STAMP(stamp_item, 0);
      const int slot = n & 1;
      denominators[slot][stream][part][r] = denominator;
      if (part == 0) references[slot][stream][r] = reference;
      asm volatile("bar.sync %0, %1;" ::"r"(9), "n"(kStreamThreads * kStreams) : "memory");
      ATT_STAMP(stamp_item, 1);
      float top = -INFINITY;
#pragma unroll
      for (int other = 0; other < kStreams; ++other) top = fmaxf(top, references[slot][other][r]);
      float weight[kStreams], total = 0.0f;
#pragma unroll
      for (int other = 0; other < kStreams; ++other) {
        const float theirs = references[slot][other][r];      // -inf: that stream saw no key of this row
        weight[other] = theirs > -INFINITY ? fast_exp2(theirs - top) : 0.0f;
        total += (denominators[slot][other][0][r] + denominators[slot][other][1][r]) * weight[other];
      }
      // the item's last product is over
      if (alive && !wait_barrier(bar(ITEM_DONE), (uint32_t)n & 1u)) {
        g_tc_attention_error = 3;
        alive = false;
      }
      tensor_fence_after_sync();
      ATT_STAMP(stamp_item, 2);
      {
        // this thread's columns of the output: the row's 128 are shared out over all its softmax threads
        constexpr int kOut = kDim / (kParts * kStreams);
        const int column = (stream * kParts + part) * kOut;
        const float inverse = total > 0.0f ? 1.0f / total : 0.0f;
        bf16* dst = out + ((size_t)(w.q_row0 + r) * heads + w.head) * kDim + column;
#pragma unroll 1
        for (int c0 = 0; c0 < kOut; c0 += 32) {
          float o[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0.0f;
#pragma unroll
          for (int other = 0; other < (kShared ? 1 : kStreams); ++other) {
            if (kShared) {
              // one accumulator, scaled to the last tile's reference, which is the largest
              float theirs[32];
              tmem_load_32(tmem_o + lane_bits + column + c0, theirs);
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = inverse > 0.0f ? theirs[i] * inverse : 0.0f;
            } else if (other < w.tiles) {                     // a stream without a tile never wrote its O
              float theirs[32];
              tmem_load_32(tmem_o + (uint32_t)other * 128u + lane_bits + column + c0, theirs);
              const float share = weight[other] * inverse;
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] += share > 0.0f ? theirs[i] * share : 0.0f;
            }
          }
          if (c0 + 32 >= kOut) {
            // the accumulators are read out: the next item's products may overwrite them
            tensor_fence_before_sync();
            barrier_arrive(bar(O_FREE));
            ATT_STAMP(stamp_item, 3);
          }
          if (valid_row && alive) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 packed_out;
              __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed_out);
#pragma unroll
              for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(o[i + 2 * j], o[i + 2 * j + 1]);
              *reinterpret_cast<uint4*>(dst + c0 + i) = packed_out;
            }
          }
        }
      }
      ATT_STAMP(stamp_item, 4);
      g0 += w.tiles;
      ++n;
    }
    tensor_fence_before_sync();
  }
  __syncthreads();
  if (warp == 1) {
    tensor_fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns) : "memory");
  }
}


}  // namespace

#ifdef MIR_TRACE
// The first CTA's tile stamps of the last launch (cycles), [kTraceTiles][16]; returns the number of rows.
MIR_EXPORT int mir_trace_read_prompt_tiles(long long* host, int capacity) {
  const int rows = capacity < kTraceTiles ? capacity : kTraceTiles;
  if (cudaDeviceSynchronize() != cudaSuccess ||
      cudaMemcpyFromSymbol(host, g_prompt_tiles, sizeof(long long) * 16 * rows) != cudaSuccess)
    return -1;
  return rows;
}
#endif

// 0 if no bounded wait of the tcgen05 attention ever ran out; else which role gave up last (1 loader, 2 issuer,
// 3 softmax).  Synchronises the device.
MIR_EXPORT int mir_prefill_attention_tc_error() {
  int flag = 0;
  if (cudaMemcpyFromSymbol(&flag, g_tc_attention_error, sizeof(int)) != cudaSuccess) return -1;
  return flag;
}

// Whether the tcgen05 kernel takes these sizes (head_dim 128, pages of 8 to 128 keys that divide 128).
MIR_EXPORT int mir_prefill_attention_tc_takes(int head_dim, int page_size) {
  return head_dim == kDim && page_size >= 8 && page_size <= kKeys && kKeys % page_size == 0 && page_size % 8 == 0;
}

// Any mix of portions: row r has tokens query_starts[r] .. query_starts[r+1]-1 of the packed batch, and its
// context_lens[r] cached tokens include them.  q is the packed [tokens, q_stride] buffer whose first
// heads * 128 columns are the rotated queries; out is [tokens, heads * 128]; k_pages and v_pages are
// [cache_rows, kv_heads, 128].
MIR_EXPORT int mir_prefill_attention_tc_bf16(const void* q, long long q_stride, void* out, const void* k_pages,
                                             const void* v_pages, long long cache_rows, const int* block_table,
                                             int table_width, const int* query_starts, const int* context_lens,
                                             int num_rows, int tokens, int page_size, int heads, int kv_heads,
                                             int head_dim, float scale, int window, cudaStream_t stream) {
  if (num_rows == 0 || tokens == 0) return MIR_OK;
  if (!mir_prefill_attention_tc_takes(head_dim, page_size) || heads <= 0 || kv_heads <= 0 || heads % kv_heads ||
      table_width <= 0 || window < 0 || num_rows < 0 || tokens < 0 || scale <= 0.0f ||
      (q_stride % 8) || q_stride < (long long)heads * kDim || ((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) ||
      ((uintptr_t)v_pages & 15) || ((uintptr_t)out & 15) || cache_rows <= 0 || cache_rows > 0x7fffffffll ||
      q_stride > 0x7fffffffll) {
    mir_set_error("prefill_attention_tc: takes head_dim 128, pages of 8..128 keys that divide 128, a positive scale "
                  "and 16-byte aligned tensors (head_dim %d, page %d, heads %d, kv heads %d)", head_dim, page_size,
                  heads, kv_heads);
    return MIR_BAD_ARGUMENT;
  }
  CUtensorMap q_map, k_map, v_map, k_tile_map, v_tile_map;
  int status = tensor_map_for(q, tokens, (int)q_stride, (int)q_stride, kRows, &q_map);
  if (status != MIR_OK) return status;
  status = tensor_map_for(k_pages, (int)cache_rows, kv_heads * kDim, kv_heads * kDim, page_size, &k_map);
  if (status != MIR_OK) return status;
  status = tensor_map_for(v_pages, (int)cache_rows, kv_heads * kDim, kv_heads * kDim, page_size, &v_map);
  if (status != MIR_OK) return status;
  status = tensor_map_for(k_pages, (int)cache_rows, kv_heads * kDim, kv_heads * kDim, kKeys, &k_tile_map);
  if (status != MIR_OK) return status;
  status = tensor_map_for(v_pages, (int)cache_rows, kv_heads * kDim, kv_heads * kDim, kKeys, &v_tile_map);
  if (status != MIR_OK) return status;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(tc_prefill_attention_kernel<2, false>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(tc_prefill_attention_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kSmemBytes);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(tc_prefill_attention_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kSmemBytes);
    if (err != cudaSuccess) {
      mir_set_error("prefill_attention_tc: cannot reserve %d bytes of shared memory: %s", kSmemBytes,
                    cudaGetErrorString(err));
      return MIR_CUDA_ERROR;
    }
    configured = true;
  }
  const int tile_slots = (tokens + kRows - 1) / kRows + num_rows;   // an upper bound; spare items are skipped
  const long long items = (long long)tile_slots * heads;
  if (items > 0x7fffffffll) {
    mir_set_error("prefill_attention_tc: %d tokens in %d rows are more than one launch takes", tokens, num_rows);
    return MIR_BAD_ARGUMENT;
  }
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    cudaGetDevice(&device);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 148;
  }
  const int ctas = (int)std::min<long long>(items, g_ctas > 0 ? g_ctas : sms);
  if (g_streams == 2 && g_shared)
    return mir_launch("prefill_attention_tc", tc_prefill_attention_kernel<2, true>, dim3(ctas), dim3(threads_for(2)),
                      (size_t)kSmemBytes, stream, 0, q_map, k_map, v_map, k_tile_map, v_tile_map, (bf16*)out, block_table, table_width,
                      query_starts, context_lens, num_rows, page_size, heads, kv_heads,
                      scale * 1.4426950408889634f, window, tile_slots);
  if (g_streams == 2)
    return mir_launch("prefill_attention_tc", tc_prefill_attention_kernel<2, false>, dim3(ctas), dim3(threads_for(2)),
                      (size_t)kSmemBytes, stream, 0, q_map, k_map, v_map, k_tile_map, v_tile_map, (bf16*)out, block_table, table_width,
                      query_starts, context_lens, num_rows, page_size, heads, kv_heads,
                      scale * 1.4426950408889634f, window, tile_slots);
  return mir_launch("prefill_attention_tc", tc_prefill_attention_kernel<1, false>, dim3(ctas), dim3(threads_for(1)),
                    (size_t)kSmemBytes, stream, 0, q_map, k_map, v_map, k_tile_map, v_tile_map, (bf16*)out, block_table, table_width,
                    query_starts, context_lens, num_rows, page_size, heads, kv_heads,
                    scale * 1.4426950408889634f, window, tile_slots);
}

// For measurements: 2 (the default) splits a row's key tiles over two softmax streams, 1 runs one stream.
MIR_EXPORT int mir_prefill_attention_tc_set_streams(int streams) {
  if (streams != 1 && streams != 2) return MIR_BAD_ARGUMENT;
  g_streams = streams;
  return MIR_OK;
}

// For measurements: 1 (the default) the two streams share a row's running reference, three score accumulators and
// one output accumulator; 0 each stream keeps a softmax of its own over its tiles and the two are merged.
MIR_EXPORT int mir_prefill_attention_tc_set_shared(int shared) {
  if (shared != 0 && shared != 1) return MIR_BAD_ARGUMENT;
  g_shared = shared;
  return MIR_OK;
}

// For measurements: at most this many CTAs (0: one per SM).  As many CTAs as there are items gives every item a CTA
// of its own.
MIR_EXPORT int mir_prefill_attention_tc_set_ctas(int ctas) {
  if (ctas < 0) return MIR_BAD_ARGUMENT;
  g_ctas = ctas;
  return MIR_OK;
}
