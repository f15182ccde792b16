// bf16 matrix products for many rows with PAIRS of SMs on one tile (tcgen05 cta_group::2):
//
//   out[M, N] = epilogue(x[M, K] . w[N, K]^T)
//
// Two CTAs of a cluster share a tile of 256 tokens x 256 accumulator columns.  Each loads its own 128 token rows
// (A operand) and its own 128 of the 256 weight rows (half of the B operand) per 64-wide step of K: 32 KB per
// stage and CTA instead of 48 KB for a 128 x 256 tile of its own, so the ring holds six stages, and one
// tcgen05.mma.cta_group::2 (256 x 256 x 16, issued by the even CTA's issuer thread) does the work of two.  The
// accumulator rows of each CTA's tokens land in that CTA's tensor memory; each CTA runs its own epilogue.
//   - TMA loads of both CTAs signal the even CTA's "full" barrier (cp.async.bulk.tensor with .cta_group::2);
//   - tcgen05.commit.cta_group::2 with a multicast mask frees the stage in both CTAs and announces the
//     accumulator to both epilogues;
//   - the odd CTA's epilogue warps arrive on the even CTA's "accumulator free" barrier across the cluster.
// Epilogues as in the one-CTA kernel (store / accumulate / 32-bit / SwiGLU: the even CTA then holds the gate rows
// of the tile, the odd CTA the up rows).  Waits on mbarriers are bounded in time; the cluster's own barrier at
// the start and the end is reached by every thread unconditionally.
#include <algorithm>
#include <cooperative_groups.h>
#include "tcgen05.cuh"

namespace cg = cooperative_groups;
using namespace mir;
using namespace mir::tc;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kTileM = 128;                 // tokens per CTA (256 per pair)
constexpr int kStepK = 64;
constexpr int kStages = 6;
constexpr int kStageStride = 2 * 128 * 128; // 32 KB: 128 token rows and 128 weight rows of 128 bytes
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = (2 + kEpilogueWarps) * 32;
constexpr uint32_t kTmemColumns = 512;      // two accumulators of 256 columns
enum Epilogue : int { STORE = 0, ACCUM = 1, F32 = 2, SWIGLU = 3 };

__device__ int g_tc_pair_error = 0;

__device__ __forceinline__ void mma_pair_bf16_ss(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in BOTH CTAs once every product issued so far is done.
__device__ __forceinline__ void mma_pair_commit(uint32_t barrier) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(barrier),
               "h"((unsigned short)3)
               : "memory");
}
// One box into this CTA's shared memory; the bytes count on the EVEN CTA's barrier at offset `barrier`.
__device__ __forceinline__ void tma_pair_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t barrier, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
          "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(barrier & 0xFEFFFFFFu), "r"(x), "r"(y)
      : "memory");
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
tc_gemm_pair_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
                    const void* __restrict__ bias, void* __restrict__ out, int ldo, int m, int n, int k, int up_offset,
                    int token_tiles, int tiles) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long barriers[2 * kStages + 4];   // full, empty, accumulator full[2], free[2]
  __shared__ uint32_t tmem_base_slot;
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t rank = cluster.block_rank();                // 0: issues the products; 1: its peer
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t full0 = smem_u32(&barriers[0]), empty0 = smem_u32(&barriers[kStages]);
  const uint32_t acc_full0 = smem_u32(&barriers[2 * kStages]), acc_free0 = smem_u32(&barriers[2 * kStages + 2]);
  const int steps = (k + kStepK - 1) / kStepK;
  constexpr int out_width = MODE == SWIGLU ? 128 : 256;      // output columns of a tile
  const int pairs = gridDim.x / 2, pair = blockIdx.x / 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      barrier_init(full0 + 8 * s, 1);
      barrier_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      barrier_init(acc_full0 + 8 * b, 1);
      barrier_init(acc_free0 + 8 * b, 2 * kEpilogueWarps);   // the epilogue warps of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {                                           // the same warp in both CTAs
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(kTmemColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tensor_fence_before_sync();
  cluster.sync();                                            // both CTAs' barriers and tensor memory exist
  tensor_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  grid_launch_dependents();
  grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (in both CTAs)
    if (lane == 0) {
      uint32_t count = 0;
      bool alive = true;
      for (int tile = pair; tile < tiles && alive; tile += pairs) {
        const int m0 = (tile % token_tiles) * 256 + (int)rank * kTileM;
        const int n0 = (tile / token_tiles) * out_width;
        // this CTA's 128 of the tile's 256 weight rows: features n0 + 128 rank.., or gate rows (0) / up rows (1)
        const int w_row = MODE == SWIGLU ? (rank == 0 ? n0 : up_offset + n0) : n0 + (int)rank * 128;
        for (int step = 0; step < steps; ++step, ++count) {
          const uint32_t stage = count % kStages, parity = (count / kStages) & 1u;
          if (!wait_barrier(empty0 + 8 * stage, parity ^ 1u)) { g_tc_pair_error = 1; alive = false; break; }
          const uint32_t barrier = full0 + 8 * stage;
          const uint32_t dst = smem_u32(smem + (size_t)stage * kStageStride);
          if (rank == 0) barrier_expect_bytes(barrier, 2u * kStageStride);     // the bytes of both CTAs
          tma_pair_load_2d(dst, &x_map, barrier, step * kStepK, m0);
          tma_pair_load_2d(dst + kTileM * 128, &w_map, barrier, step * kStepK, w_row);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ issuer (the even CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = instruction_descriptor(256, 256);
      uint32_t count = 0, local = 0;
      bool alive = true;
      for (int tile = pair; tile < tiles; tile += pairs, ++local) {
        const uint32_t buffer = local & 1u, use = (local >> 1) & 1u;
        if (alive && !wait_barrier(acc_free0 + 8 * buffer, use ^ 1u)) { g_tc_pair_error = 2; alive = false; }
        tensor_fence_after_sync();
        const uint32_t accumulator = tmem_base + buffer * 256u;
        for (int step = 0; step < steps; ++step, ++count) {
          const uint32_t stage = count % kStages, parity = (count / kStages) & 1u;
          if (alive && !wait_barrier(full0 + 8 * stage, parity)) { g_tc_pair_error = 2; alive = false; }
          tensor_fence_after_sync();
          const uint32_t a_base = smem_u32(smem + (size_t)stage * kStageStride);
          const uint32_t b_base = a_base + kTileM * 128;
#pragma unroll
          for (int kk = 0; kk < kStepK / 16; ++kk)
            mma_pair_bf16_ss(accumulator, operand_descriptor(a_base + kk * 32), operand_descriptor(b_base + kk * 32), idesc,
                             (step > 0 || kk > 0) ? 1u : 0u);
          mma_pair_commit(empty0 + 8 * stage);               // frees the stage in both CTAs
        }
        mma_pair_commit(acc_full0 + 8 * buffer);             // both epilogues may read their rows
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (in both CTAs): one token row per thread
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    uint32_t local = 0;
    bool alive = true;
    // the even CTA's "accumulator free" barriers, as seen from this CTA
    uint32_t free_remote[2];
#pragma unroll
    for (int b = 0; b < 2; ++b)
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(free_remote[b]) : "r"(acc_free0 + 8 * b), "r"(0u));
    for (int tile = pair; tile < tiles && alive; tile += pairs, ++local) {
      const uint32_t buffer = local & 1u, use = (local >> 1) & 1u;
      const int m0 = (tile % token_tiles) * 256 + (int)rank * kTileM;
      const int n0 = (tile / token_tiles) * out_width;
      const int row = m0 + quarter * 32 + lane;
      if (!wait_barrier(acc_full0 + 8 * buffer, use)) { g_tc_pair_error = 3; alive = false; break; }
      tensor_fence_after_sync();
      const uint32_t lane_base = tmem_base + buffer * 256u + ((uint32_t)(quarter * 32) << 16);
      bool released = false;
      auto release = [&]() {                                 // this warp has read all it needs of the accumulator
        tensor_fence_before_sync();
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(free_remote[buffer]) : "memory");
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
      if (!released) release();
    }
    tensor_fence_before_sync();
  }
  cluster.sync();                                            // no CTA leaves while its peer may still signal it
  if (warp == 1) {
    tensor_fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns) : "memory");
  }
}

int pair_sm_count() {
  static int count = 0;
  if (count == 0) {
    int device = 0;
    cudaGetDevice(&device);
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) count = 148;
  }
  return count;
}

template <int MODE>
int launch_pair(const void* x, int ldx, const void* w, const void* bias, void* out, int ldo, int m, int n, int k,
                int up_offset, cudaStream_t stream) {
  constexpr int out_width = MODE == SWIGLU ? 128 : 256;
  const int token_tiles = (m + 255) / 256;
  CUtensorMap x_map, w_map;
  int status = tensor_map_for(x, m, k, ldx, kTileM, &x_map);
  if (status != MIR_OK) return status;
  status = tensor_map_for(w, MODE == SWIGLU ? up_offset + n : n, k, k, 128, &w_map);
  if (status != MIR_OK) return status;
  const size_t smem = (size_t)kStages * kStageStride + 1024;
  static bool configured = false;
  if (!configured) {
    const cudaError_t err = cudaFuncSetAttribute(tc_gemm_pair_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) {
      mir_set_error("tc_gemm_pair: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
      return MIR_CUDA_ERROR;
    }
    configured = true;
  }
  const long long tiles = (long long)((n + out_width - 1) / out_width) * token_tiles;
  if (tiles > 0x7fffffffll) { mir_set_error("tc_gemm_pair: too many tiles"); return MIR_BAD_ARGUMENT; }
  const int pairs = (int)std::min<long long>(tiles, pair_sm_count() / 2);
  return mir_launch_cluster(false, "tc_gemm_pair", tc_gemm_pair_kernel<MODE>, dim3(2 * pairs), dim3(kThreads), smem, stream,
                            dim3(2, 1, 1), x_map, w_map, bias, out, ldo, m, n, k, up_offset, token_tiles, (int)tiles);
}

}  // namespace

MIR_EXPORT int mir_gemm_tc_pair_error() {
  int flag = 0;
  if (cudaMemcpyFromSymbol(&flag, g_tc_pair_error, sizeof(int)) != cudaSuccess) return -1;
  return flag;
}

// Modes, operands and limits as mir_gemm_tc_bf16.
MIR_EXPORT int mir_gemm_tc_pair_bf16(int mode, const void* x, int ldx, const void* w, const void* bias, void* out,
                                     int ldo, int m, int n, int k, int up_offset, cudaStream_t stream) {
  if (m == 0 || n == 0) return MIR_OK;
  if (m < 0 || n < 0 || k <= 0 || (k % 8) || (ldx % 8) || ldx < k || ldo < n || ((uintptr_t)x & 15) ||
      ((uintptr_t)w & 15) || m > 65535 * 256) {
    mir_set_error("tc_gemm_pair: k and the row stride must be multiples of 8 and the operands 16-byte aligned "
                  "(m %d n %d k %d ldx %d ldo %d)", m, n, k, ldx, ldo);
    return MIR_BAD_ARGUMENT;
  }
  switch (mode) {
    case STORE: return launch_pair<STORE>(x, ldx, w, bias, out, ldo, m, n, k, 0, stream);
    case ACCUM: return launch_pair<ACCUM>(x, ldx, w, bias, out, ldo, m, n, k, 0, stream);
    case F32: return launch_pair<F32>(x, ldx, w, bias, out, ldo, m, n, k, 0, stream);
    case SWIGLU:
      if (bias) { mir_set_error("tc_gemm_pair: the SwiGLU epilogue takes no bias"); return MIR_BAD_ARGUMENT; }
      return launch_pair<SWIGLU>(x, ldx, w, nullptr, out, ldo, m, n, k, up_offset, stream);
  }
  mir_set_error("tc_gemm_pair: unknown mode %d", mode);
  return MIR_BAD_ARGUMENT;
}
