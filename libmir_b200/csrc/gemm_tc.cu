// bf16 matrix products for many rows on the 5th-generation tensor cores (tcgen05), written by hand:
//
//   out[M, N] = epilogue(x[M, K] . w[N, K]^T)          x, w row-major bf16 ("K-major" for both operands)
//
// One CTA per SM walks over tiles of the output: 128 tokens x `width` accumulator columns (for the SwiGLU
// epilogue width / 2 gate features and the width / 2 up features that belong to them); width is 256 unless
// the product has fewer columns.  Three roles:
//
//   producer   one thread.  Per 64-wide step of K it asks the TMA unit for the x box (128 rows x 64) and the
//              w box(es) with cp.async.bulk.tensor.2d into a ring of shared-memory stages laid out with the
//              128-byte swizzle that tcgen05.mma reads.  Out-of-range rows and k arrive as zeros, so M, N and K
//              need not be multiples of the tile.  An mbarrier per stage counts the bytes in.
//   issuer     one warp that stays converged, the products predicated on its elected lane (tcgen05.cuh says why).
//              When a stage is full it issues four tcgen05.mma (128 x width x 16 each, operands
//              straight from shared memory through matrix descriptors, accumulator in tensor memory) and then
//              tcgen05.commit, which arrives on the stage's "empty" barrier once the tensor cores have read the
//              stage, so the producer can refill it.  After a tile's last step a commit arrives on the
//              accumulator's "full" barrier.  Two accumulators alternate: the products of the next tile run
//              while the epilogue reads the last one.
//   epilogue   eight warps; warp i may read accumulator lanes 32 (i mod 4) .. + 31 (one token row per thread),
//              and the two warps of a quarter take alternate chunks of 32 columns.  They
//              wait for "full", read the accumulator with tcgen05.ld (32 columns at a time), hand the
//              accumulator back ("free" barrier) as soon as its last columns are in registers, apply the
//              epilogue and write the row to global memory.
//
// Epilogues:  STORE  out bf16 = acc (+ bias)
//             ACCUM  out float += acc (+ bias)            the residual stream
//             F32    out float = acc (+ bias)
//             SWIGLU out bf16 = silu(acc_gate) * acc_up   w holds [gate rows; up rows]; the [M, 2 I] intermediate
//                                                         of the two-kernel formulation is never written
// Tensor memory: all 512 columns (two accumulators of 128 lanes x 256 columns), allocated by one warp and freed
// by the same warp; the shared-memory ring leaves room for one CTA per SM only.
// Every wait is bounded in time; a role whose wait runs out raises g_tc_gemm_error and stops waiting, the CTA
// still frees its tensor memory and returns.
// libmir takes these products from a library (DenseMatmulPlan / CublasLtBf16Plan of the mircuda crate,
// cuda/src/backend/linear/mod.rs:141-194) and applies the gate in a second kernel
// (cuda/kernels/elementwise_bf16.cu:42-70).
#include <algorithm>
#include "tcgen05.cuh"

using namespace mir;
using namespace mir::tc;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kTileM = 128;                 // tokens per CTA
constexpr int kStepK = 64;                  // k per stage: 128 bytes, one swizzle row
constexpr int kStages = 4;                  // shared-memory ring
constexpr int kStageStride = (kTileM + 256) * 128;   // 48 KB: 128 token rows and up to 256 weight rows of 128 bytes
constexpr int kEpilogueWarps = 8;          // two per quarter of the accumulator lanes; they share its columns
constexpr int kThreads = (2 + kEpilogueWarps) * 32;  // producer warp, issuer warp, epilogue warps
constexpr uint32_t kTmemColumns = 512;      // two accumulators of up to 256 columns
enum Epilogue : int { STORE = 0, ACCUM = 1, F32 = 2, SWIGLU = 3 };

__device__ int g_tc_gemm_error = 0;

// One CTA per SM walks over output tiles (token tile fastest, so CTAs that run together share weight rows in
// L2).  A tile is 128 tokens x `width` accumulator columns (width a multiple of 16, at most 256; with the SwiGLU
// epilogue width / 2 gate columns followed by width / 2 up columns).  Two accumulators of 256 columns alternate,
// so the epilogue of one tile overlaps the products of the next.
template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
               const void* __restrict__ bias, void* __restrict__ out, int ldo, int m, int n, int k, int up_offset,
               int width, int token_tiles, int tiles) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long barriers[2 * kStages + 4];   // full, empty, accumulator full[2], free[2]
  __shared__ uint32_t tmem_base_slot;
  if (*reinterpret_cast<volatile int*>(&g_tc_gemm_error) != 0) return;   // an earlier wait ran out: do not queue up more
  // the swizzle pattern repeats every 1024 bytes; the stages start on such a boundary
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t full0 = smem_u32(&barriers[0]), empty0 = smem_u32(&barriers[kStages]);
  const uint32_t acc_full0 = smem_u32(&barriers[2 * kStages]), acc_free0 = smem_u32(&barriers[2 * kStages + 2]);
  const int steps = (k + kStepK - 1) / kStepK;
  const int out_width = MODE == SWIGLU ? width / 2 : width;  // output columns of a tile
  const uint32_t stage_bytes = (uint32_t)(kTileM + width) * 128u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(full0 + 8 * s) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(empty0 + 8 * s) : "memory");
    }
    for (int b = 0; b < 2; ++b) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(acc_full0 + 8 * b) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(acc_free0 + 8 * b), "r"(kEpilogueWarps) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {                                          // this warp owns the tensor memory: all 512 columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(kTmemColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
  grid_launch_dependents();
  grid_dependency_wait();                                   // x (and out for ACCUM) come from earlier kernels

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      const uint64_t xm = reinterpret_cast<uint64_t>(&x_map), wm = reinterpret_cast<uint64_t>(&w_map);
      uint32_t count = 0;                                    // stages filled so far, over all tiles
      bool alive = true;
      for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
        const int m0 = (tile % token_tiles) * kTileM, n0 = (tile / token_tiles) * out_width;
        for (int step = 0; step < steps; ++step, ++count) {
          const uint32_t stage = count % kStages, parity = (count / kStages) & 1u;
          if (!wait_barrier(empty0 + 8 * stage, parity ^ 1u)) { g_tc_gemm_error = 1; alive = false; break; }
          const uint32_t barrier = full0 + 8 * stage;
          const uint32_t dst = smem_u32(smem + (size_t)stage * kStageStride);
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(barrier), "r"(stage_bytes) : "memory");
          asm volatile(
              "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
                  "r"(dst), "l"(xm), "r"(barrier), "r"(step * kStepK), "r"(m0)
              : "memory");
          // the weight map's box has out_width rows: one box, or a gate box and an up box behind it
          asm volatile(
              "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
                  "r"(dst + kTileM * 128), "l"(wm), "r"(barrier), "r"(step * kStepK), "r"(n0)
              : "memory");
          if (MODE == SWIGLU)
            asm volatile(
                "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
                    "r"(dst + (kTileM + out_width) * 128), "l"(wm), "r"(barrier), "r"(step * kStepK), "r"(up_offset + n0)
                : "memory");
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ issuer: the whole warp stays converged, the
    // products are predicated on the elected lane (see tcgen05.cuh on issuing from a whole warp)
    {
      const uint32_t idesc = instruction_descriptor(kTileM, width);
      const uint32_t elected = elect_one();
      const uint32_t a_low0 = operand_low(smem_u32(smem)), b_low0 = operand_low(smem_u32(smem) + kTileM * 128);
      uint32_t stage = 0, parity = 0, local = 0;             // of the stages consumed so far; tiles of this CTA
      bool alive = true;
      for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
        const uint32_t buffer = local & 1u, use = (local >> 1) & 1u;
        // the epilogue must have read this accumulator's previous tile
        if (alive && !wait_barrier(acc_free0 + 8 * buffer, use ^ 1u)) { g_tc_gemm_error = 2; alive = false; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t accumulator = tmem_base + buffer * 256u;
        for (int step = 0; step < steps; ++step) {
          if (alive && !wait_barrier(full0 + 8 * stage, parity)) { g_tc_gemm_error = 2; alive = false; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_low = a_low0 + stage * (uint32_t)(kStageStride >> 4);
          const uint32_t b_low = b_low0 + stage * (uint32_t)(kStageStride >> 4);
          // 16 k = 32 bytes further along the swizzled rows: the start address moves by 32 bytes
          mma_bf16_ss_halves(accumulator, a_low, b_low, idesc, step > 0 ? 1u : 0u, elected);
#pragma unroll
          for (int kk = 1; kk < kStepK / 16; ++kk)
            mma_bf16_ss_halves<true>(accumulator, a_low + 2u * kk, b_low + 2u * kk, idesc, elected);
          mma_commit_elected(empty0 + 8 * stage, elected);   // the stage is free once these have read it
          if (++stage == (uint32_t)kStages) { stage = 0; parity ^= 1u; }
        }
        mma_commit_elected(acc_full0 + 8 * buffer, elected); // this tile's accumulator is complete
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: one token row per thread
    const int quarter = warp & 3;                            // the accumulator lanes this warp may read
    const int half = (warp - 2) >> 2;                        // which of every two 32-column chunks it takes
    uint32_t local = 0;
    bool alive = true;
    for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x, ++local) {
      const uint32_t buffer = local & 1u, use = (local >> 1) & 1u;
      const int m0 = (tile % token_tiles) * kTileM, n0 = (tile / token_tiles) * out_width;
      const int row = m0 + quarter * 32 + lane;
      if (!wait_barrier(acc_full0 + 8 * buffer, use)) { g_tc_gemm_error = 3; alive = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_base = tmem_base + buffer * 256u + ((uint32_t)(quarter * 32) << 16);
      bool released = false;
      auto release = [&]() {                                 // this warp has read all it needs of the accumulator
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_free0 + 8 * buffer) : "memory");
        released = true;
      };
#pragma unroll 1
      for (int c0 = half * 32; c0 < out_width; c0 += 64) {
        float v[32];
        tmem_load_32(lane_base + c0, v);
        if (MODE == SWIGLU) {
          float u[32];
          tmem_load_32(lane_base + out_width + c0, u);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __fdividef(v[i], 1.0f + __expf(-v[i])) * u[i];
        }
        if (c0 + 64 >= out_width) release();                 // the last columns are in registers
        const int limit = min(n, n0 + out_width);            // columns of this tile that exist
        if (row < m) {
          if (MODE == STORE || MODE == SWIGLU) {
            bf16* dst = reinterpret_cast<bf16*>(out) + (size_t)row * ldo + n0 + c0;
            if (n0 + c0 + 32 <= limit && (ldo % 8) == 0) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                float b8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                if (MODE == STORE && bias) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) b8[j] = __bfloat162float(reinterpret_cast<const bf16*>(bias)[n0 + c0 + i + j]);
                }
                uint4 packed;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[i + 2 * j] + b8[2 * j], v[i + 2 * j + 1] + b8[2 * j + 1]);
                *reinterpret_cast<uint4*>(dst + i) = packed;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                if (n0 + c0 + i < limit) {
                  float value = v[i];
                  if (MODE == STORE && bias) value += __bfloat162float(reinterpret_cast<const bf16*>(bias)[n0 + c0 + i]);
                  dst[i] = __float2bfloat16_rn(value);
                }
              }
            }
          } else {
            float* dst = reinterpret_cast<float*>(out) + (size_t)row * ldo + n0 + c0;
            if (n0 + c0 + 32 <= limit && (ldo % 4) == 0 && bias == nullptr) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                float4 value = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                if (MODE == ACCUM) {
                  const float4 old = *reinterpret_cast<const float4*>(dst + i);
                  value.x += old.x; value.y += old.y; value.z += old.z; value.w += old.w;
                }
                *reinterpret_cast<float4*>(dst + i) = value;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                if (n0 + c0 + i < limit) {
                  float value = v[i];
                  if (bias) value += reinterpret_cast<const float*>(bias)[n0 + c0 + i];
                  dst[i] = MODE == ACCUM ? dst[i] + value : value;
                }
              }
            }
          }
        }
      }
      if (!released) release();                              // a tile too narrow to give this warp any columns
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ host
int g_forced_width = 0;                                      // for measurements: 0 = choose

int sm_count() {
  static int count = 0;
  if (count == 0) {
    int device = 0;
    cudaGetDevice(&device);
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) count = 148;
  }
  return count;
}

// Accumulator columns of a tile.  Measured on B200 (2,048 tokens, K 2,560 to 9,728): a step of K takes about
// 0.4 us whether the tile is 192, 224 or 256 columns wide (the ring of four stages is bound by the latency of
// its refills, not by the products), so the widest tile is the fastest even where a narrower one would fill the
// last round of tiles better.  `columns` is the number of accumulator columns over all tiles (2 n with the
// SwiGLU epilogue), `step` what the width must be a multiple of.
int choose_width(long long columns, int step) {
  if (g_forced_width >= step && g_forced_width <= 256 && g_forced_width % step == 0) return g_forced_width;
  const long long rounded = (columns + step - 1) / step * step;
  return (int)std::min<long long>(256, rounded);
}

template <int MODE>
int launch(const void* x, int ldx, const void* w, const void* bias, void* out, int ldo, int m, int n, int k,
           int up_offset, cudaStream_t stream) {
  const int token_tiles = (m + kTileM - 1) / kTileM;
  const int width = MODE == SWIGLU ? choose_width(2ll * n, 32) : choose_width(n, 16);
  const int out_width = MODE == SWIGLU ? width / 2 : width;
  CUtensorMap x_map, w_map;
  int status = tensor_map_for(x, m, k, ldx, kTileM, &x_map);
  if (status != MIR_OK) return status;
  status = tensor_map_for(w, MODE == SWIGLU ? up_offset + n : n, k, k, out_width, &w_map);
  if (status != MIR_OK) return status;
  const size_t smem = (size_t)kStages * kStageStride + 1024;
  static bool configured = false;
  if (!configured) {
    const cudaError_t err = cudaFuncSetAttribute(tc_gemm_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) {
      mir_set_error("tc_gemm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
      return MIR_CUDA_ERROR;
    }
    configured = true;
  }
  const long long tiles = (long long)((n + out_width - 1) / out_width) * token_tiles;
  if (tiles > 0x7fffffffll) { mir_set_error("tc_gemm: too many tiles"); return MIR_BAD_ARGUMENT; }
  const dim3 grid((unsigned)std::min<long long>(tiles, sm_count()));
  return mir_launch("tc_gemm", tc_gemm_kernel<MODE>, grid, dim3(kThreads), smem, stream, 0, x_map, w_map, bias, out, ldo,
                    m, n, k, up_offset, width, token_tiles, (int)tiles);
}

}  // namespace

// 0 if no bounded wait of the tcgen05 product ever ran out; else which role gave up last (1 producer, 2 issuer,
// 3 epilogue).  Synchronises the device.
MIR_EXPORT int mir_gemm_tc_error() {
  int flag = 0;
  if (cudaMemcpyFromSymbol(&flag, g_tc_gemm_error, sizeof(int)) != cudaSuccess) return -1;
  return flag;
}

// For measurements: fix the accumulator width of a tile (a multiple of 32, 32..256), or 0 to let the launcher
// choose.
MIR_EXPORT int mir_gemm_tc_set_width(int width) {
  if (width != 0 && (width < 32 || width > 256 || width % 32)) {
    mir_set_error("tc_gemm: the width must be 0 or a multiple of 32 up to 256");
    return MIR_BAD_ARGUMENT;
  }
  g_forced_width = width;
  return MIR_OK;
}

// mode: 0 store bf16, 1 accumulate into float, 2 float, 3 SwiGLU (w = [gate; up],
// up rows start at up_offset, n = number of output columns).  k and ldx must be multiples of 8, x and w 16-byte
// aligned; m, n, k need not be multiples of the tile sizes.
MIR_EXPORT int mir_gemm_tc_bf16(int mode, const void* x, int ldx, const void* w, const void* bias, void* out, int ldo,
                                int m, int n, int k, int up_offset, cudaStream_t stream) {
  if (m == 0 || n == 0) return MIR_OK;
  if (m < 0 || n < 0 || k <= 0 || (k % 8) || (ldx % 8) || ldx < k || ldo < n || ((uintptr_t)x & 15) ||
      ((uintptr_t)w & 15) || m > 65535 * kTileM) {
    mir_set_error("tc_gemm: k and the row stride must be multiples of 8 and the operands 16-byte aligned "
                  "(m %d n %d k %d ldx %d ldo %d)", m, n, k, ldx, ldo);
    return MIR_BAD_ARGUMENT;
  }
  switch (mode) {
    case STORE: return launch<STORE>(x, ldx, w, bias, out, ldo, m, n, k, 0, stream);
    case ACCUM: return launch<ACCUM>(x, ldx, w, bias, out, ldo, m, n, k, 0, stream);
    case F32: return launch<F32>(x, ldx, w, bias, out, ldo, m, n, k, 0, stream);
    case SWIGLU:
      if (bias) { mir_set_error("tc_gemm: the SwiGLU epilogue takes no bias"); return MIR_BAD_ARGUMENT; }
      return launch<SWIGLU>(x, ldx, w, nullptr, out, ldo, m, n, k, up_offset, stream);
  }
  mir_set_error("tc_gemm: unknown mode %d", mode);
  return MIR_BAD_ARGUMENT;
}
