// bf16 matrix products for many rows on the 5th-generation tensor cores (tcgen05), written by hand:
//
//   out[M, N] = epilogue(x[M, K] . w[N, K]^T)          x, w row-major bf16 ("K-major" for both operands)
//
// One CTA computes a 128-token x 128-feature tile of the output (for the SwiGLU epilogue: 128 gate features
// and the 128 up features that belong to them, 256 accumulator columns).  Three roles, one warp or more each:
//
//   producer   one thread.  Per 64-wide step of K it asks the TMA unit for the x box (128 rows x 64) and the
//              w box(es) (128 rows x 64) with cp.async.bulk.tensor.2d into a ring of shared-memory stages laid
//              out with the 128-byte swizzle that tcgen05.mma reads.  Out-of-range rows and k arrive as zeros,
//              so M, N and K need not be multiples of the tile.  An mbarrier per stage counts the bytes in.
//   issuer     one thread.  When a stage is full it issues four tcgen05.mma (128 x N x 16 each, operands
//              straight from shared memory through matrix descriptors, accumulator in tensor memory) and then
//              tcgen05.commit, which arrives on the stage's "empty" barrier once the tensor cores have read the
//              stage, so the producer can refill it.  After the last step a commit arrives on the "done" barrier.
//   epilogue   four warps; warp i owns accumulator lanes 32 i .. 32 i + 31 (one token row per thread).  They
//              wait for "done", read the accumulator with tcgen05.ld (32 columns at a time), apply the epilogue
//              and write the row to global memory.
//
// Epilogues:  STORE  out bf16 = acc (+ bias)
//             ACCUM  out float += acc (+ bias)            the residual stream
//             F32    out float = acc (+ bias)
//             SWIGLU out bf16 = silu(acc_gate) * acc_up   w holds [gate rows; up rows]; the [M, 2 I] intermediate
//                                                         of the two-kernel formulation is never written
// Tensor memory: 128 lanes x 128 (or 256) 32-bit columns, allocated by one warp and freed by the same warp.
// Every wait is bounded in time; a role whose wait runs out raises g_tc_gemm_error and stops waiting, the CTA
// still frees its tensor memory and returns.
// libmir takes these products from a library (DenseMatmulPlan / CublasLtBf16Plan of the mircuda crate,
// cuda/src/backend/linear/mod.rs:141-194) and applies the gate in a second kernel
// (cuda/kernels/elementwise_bf16.cu:42-70).
#include <cuda.h>
#include <map>
#include <mutex>
#include <tuple>
#include "common.cuh"

using namespace mir;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kTileM = 128;                 // tokens per CTA
constexpr int kTileN = 128;                 // features per accumulator half
constexpr int kStepK = 64;                  // k per stage: 128 bytes, one swizzle row
constexpr int kBoxBytes = 128 * kStepK * 2; // 16 KB: a 128-row x 64-k box
constexpr int kThreads = 6 * 32;            // producer warp, issuer warp, four epilogue warps
enum Epilogue : int { STORE = 0, ACCUM = 1, F32 = 2, SWIGLU = 3 };

__device__ int g_tc_gemm_error = 0;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

constexpr unsigned long long kWaitNanoseconds = 500ull * 1000ull * 1000ull;

__device__ __forceinline__ unsigned long long global_nanoseconds() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Wait for the phase with the given parity; false if the time limit ran out.
__device__ __forceinline__ bool wait_barrier(uint32_t barrier, uint32_t parity) {
  unsigned long long start = 0;
  for (unsigned poll = 1;; ++poll) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred P1;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, P1;\n\t}"
        : "=r"(done)
        : "r"(barrier), "r"(parity)
        : "memory");
    if (done) return true;
    if ((poll & 63u) == 0u) {
      const unsigned long long now = global_nanoseconds();
      if (start == 0) start = now;
      else if (now - start > kWaitNanoseconds) return false;
    }
  }
}

// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes with the 128-byte
// swizzle (8 rows x 128 B = one 1024-byte atom): start address, stride between 8-row groups 1024 B,
// descriptor version 1 (Blackwell), layout type 2 (SWIZZLE_128B).  All byte quantities are in 16-byte units.
__device__ __forceinline__ uint64_t operand_descriptor(uint32_t smem_address) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_address >> 4) & 0x3FFF);          // bits [0, 14)  start address
  desc |= (uint64_t)1 << 16;                                 // bits [16, 30) leading byte offset (unused here)
  desc |= (uint64_t)(1024 >> 4) << 32;                       // bits [32, 46) stride byte offset
  desc |= (uint64_t)1 << 46;                                 // bits [46, 48) version
  desc |= (uint64_t)2 << 61;                                 // bits [61, 64) SWIZZLE_128B
  return desc;
}

// Instruction descriptor: D float32, A and B bf16, both K-major, M x N.
__host__ __device__ constexpr uint32_t instruction_descriptor(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void mma_bf16_ss(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t barrier) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(barrier) : "memory");
}

// 32 consecutive accumulator columns of this thread's lane.
__device__ __forceinline__ void tmem_load_32(uint32_t address, float (&v)[32]) {
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
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// STAGES stages of [x box | w box (| second w box)]; dynamic shared memory starts on a 1024-byte boundary.
template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
               const void* __restrict__ bias, void* __restrict__ out, int ldo, int m, int n, int k, int up_offset,
               int stages) {
  constexpr int HALVES = MODE == SWIGLU ? 2 : 1;            // accumulator halves of 128 columns
  constexpr int STAGE_BYTES = (1 + HALVES) * kBoxBytes;
  constexpr uint32_t TMEM_COLUMNS = HALVES * kTileN;
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long barriers[2 * 8 + 1];   // full[8], empty[8], done
  __shared__ uint32_t tmem_base_slot;
  if (*reinterpret_cast<volatile int*>(&g_tc_gemm_error) != 0) return;   // an earlier wait ran out: do not queue up more
  // the swizzle pattern repeats every 1024 bytes; the stages start on such a boundary
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * kTileM, n0 = blockIdx.x * kTileN;
  const uint32_t full0 = smem_u32(&barriers[0]), empty0 = smem_u32(&barriers[8]), done = smem_u32(&barriers[16]);
  const int steps = (k + kStepK - 1) / kStepK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(full0 + 8 * s) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(empty0 + 8 * s) : "memory");
    }
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(done) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {                                          // this warp owns the tensor memory allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(TMEM_COLUMNS)
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
      for (int step = 0; step < steps; ++step) {
        const int stage = step % stages;
        const uint32_t parity = (uint32_t)(step / stages) & 1u;
        if (!wait_barrier(empty0 + 8 * stage, parity ^ 1u)) { g_tc_gemm_error = 1; break; }
        const uint32_t barrier = full0 + 8 * stage;
        const uint32_t dst = smem_u32(smem + (size_t)stage * STAGE_BYTES);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(barrier), "r"((uint32_t)STAGE_BYTES) : "memory");
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
                "r"(dst), "l"(xm), "r"(barrier), "r"(step * kStepK), "r"(m0)
            : "memory");
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
                "r"(dst + kBoxBytes), "l"(wm), "r"(barrier), "r"(step * kStepK), "r"(n0)
            : "memory");
        if (MODE == SWIGLU)
          asm volatile(
              "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
                  "r"(dst + 2 * kBoxBytes), "l"(wm), "r"(barrier), "r"(step * kStepK), "r"(up_offset + n0)
              : "memory");
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ issuer
    if (lane == 0) {
      constexpr uint32_t idesc = instruction_descriptor(kTileM, HALVES * kTileN);
      bool alive = true;
      for (int step = 0; step < steps; ++step) {
        const int stage = step % stages;
        const uint32_t parity = (uint32_t)(step / stages) & 1u;
        if (alive && !wait_barrier(full0 + 8 * stage, parity)) { g_tc_gemm_error = 2; alive = false; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_base = smem_u32(smem + (size_t)stage * STAGE_BYTES);
        const uint32_t b_base = a_base + kBoxBytes;          // gate rows then, for SwiGLU, up rows: 256 rows of B
#pragma unroll
        for (int kk = 0; kk < kStepK / 16; ++kk) {
          // 16 k = 32 bytes further along the swizzled rows: the start address moves by 32 bytes
          const uint64_t a_desc = operand_descriptor(a_base + kk * 32);
          const uint64_t b_desc = operand_descriptor(b_base + kk * 32);
          mma_bf16_ss(tmem_base, a_desc, b_desc, idesc, (step > 0 || kk > 0) ? 1u : 0u);
        }
        mma_commit(empty0 + 8 * stage);                      // the stage is free once these have read it
      }
      mma_commit(done);                                      // the accumulator is complete
    }
  } else {
    // ------------------------------------------------------------------ epilogue: one token row per thread
    const int quarter = warp & 3;                            // the accumulator lanes this warp may read
    const int row = m0 + quarter * 32 + lane;
    const bool alive = wait_barrier(done, 0);
    if (!alive) g_tc_gemm_error = 3;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    if (alive) {
#pragma unroll 1
      for (int c0 = 0; c0 < kTileN; c0 += 32) {
        float v[32];
        tmem_load_32(lane_base + c0, v);
        if (MODE == SWIGLU) {
          float u[32];
          tmem_load_32(lane_base + kTileN + c0, u);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = v[i] / (1.0f + __expf(-v[i])) * u[i];
        }
        if (row < m) {
          if (MODE == STORE || MODE == SWIGLU) {
            bf16* dst = reinterpret_cast<bf16*>(out) + (size_t)row * ldo + n0 + c0;
            if (n0 + c0 + 32 <= n && (ldo % 8) == 0) {
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
              for (int i = 0; i < 32; ++i) {
                if (n0 + c0 + i >= n) break;
                float value = v[i];
                if (MODE == STORE && bias) value += __bfloat162float(reinterpret_cast<const bf16*>(bias)[n0 + c0 + i]);
                dst[i] = __float2bfloat16_rn(value);
              }
            }
          } else {
            float* dst = reinterpret_cast<float*>(out) + (size_t)row * ldo + n0 + c0;
            if (n0 + c0 + 32 <= n && (ldo % 4) == 0 && bias == nullptr) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                float4 value = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                if (MODE == ACCUM) {
                  const float4 old = *reinterpret_cast<const float4*>(dst + i);
                  value.x += old.x; value.y += old.y; value.z += old.z; value.w += old.w;
                }
                *reinterpret_cast<float4*>(dst + i) = value;
              }
            } else
            for (int i = 0; i < 32; ++i) {
              if (n0 + c0 + i >= n) break;
              float value = v[i];
              if (bias) value += reinterpret_cast<const float*>(bias)[n0 + c0 + i];
              dst[i] = MODE == ACCUM ? dst[i] + value : value;
            }
          }
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLUMNS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::mutex g_mutex;
int g_stages_swiglu = 4, g_stages_other = 6;
EncodeTiled g_encode = nullptr;
std::map<std::tuple<const void*, int, int, int>, CUtensorMap> g_maps;

// Tensor map of a row-major bf16 matrix [rows, k] with row stride ld: boxes of 128 rows x 64 k, 128-byte
// swizzle, out-of-range elements read as zero.
int tensor_map_for(const void* base, int rows, int k, int ld, CUtensorMap* map) {
  std::lock_guard<std::mutex> lock(g_mutex);
  const auto key = std::make_tuple(base, rows, k, ld);
  auto found = g_maps.find(key);
  if (found != g_maps.end()) {
    *map = found->second;
    return MIR_OK;
  }
  if (g_encode == nullptr) {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess || entry == nullptr) {
      mir_set_error("tc_gemm: the driver has no cuTensorMapEncodeTiled");
      return MIR_LIBRARY_ERROR;
    }
    g_encode = reinterpret_cast<EncodeTiled>(entry);
  }
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kStepK, 128u};
  const cuuint32_t element_strides[2] = {1, 1};
  CUtensorMap made;
  const CUresult status = g_encode(&made, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                                   box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (status != CUDA_SUCCESS) {
    mir_set_error("tc_gemm: cuTensorMapEncodeTiled refused a %d x %d matrix with row stride %d (status %d)", rows, k,
                  ld, (int)status);
    return MIR_LIBRARY_ERROR;
  }
  if (g_maps.size() > 4096) g_maps.clear();                  // activation buffers come and go
  g_maps.emplace(key, made);
  *map = made;
  return MIR_OK;
}

template <int MODE>
int launch(const void* x, int ldx, const void* w, const void* bias, void* out, int ldo, int m, int n, int k,
           int up_offset, cudaStream_t stream) {
  constexpr int HALVES = MODE == SWIGLU ? 2 : 1;
  constexpr int STAGE_BYTES = (1 + HALVES) * kBoxBytes;
  CUtensorMap x_map, w_map;
  int status = tensor_map_for(x, m, k, ldx, &x_map);
  if (status != MIR_OK) return status;
  status = tensor_map_for(w, MODE == SWIGLU ? up_offset + n : n, k, k, &w_map);
  if (status != MIR_OK) return status;
  const int stages = MODE == SWIGLU ? g_stages_swiglu : g_stages_other;
  const size_t smem = (size_t)stages * STAGE_BYTES + 1024;
  static bool configured = false;
  if (!configured) {
    const cudaError_t err = cudaFuncSetAttribute(tc_gemm_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (MODE == SWIGLU ? 4 : 6) * STAGE_BYTES + 1024);
    if (err != cudaSuccess) {
      mir_set_error("tc_gemm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
      return MIR_CUDA_ERROR;
    }
    configured = true;
  }
  const dim3 grid((n + kTileN - 1) / kTileN, (m + kTileM - 1) / kTileM);
  return mir_launch("tc_gemm", tc_gemm_kernel<MODE>, grid, dim3(kThreads), smem, stream, 0, x_map, w_map, bias, out, ldo,
                    m, n, k, up_offset, stages);
}

}  // namespace

// 0 if no bounded wait of the tcgen05 product ever ran out; else which role gave up last (1 producer, 2 issuer,
// 3 epilogue).  Synchronises the device.
MIR_EXPORT int mir_gemm_tc_error() {
  int flag = 0;
  if (cudaMemcpyFromSymbol(&flag, g_tc_gemm_error, sizeof(int)) != cudaSuccess) return -1;
  return flag;
}

// Stages of the shared-memory ring (1..4 with the SwiGLU epilogue, 1..6 otherwise).  Fewer stages let two CTAs
// share an SM, so that one's epilogue overlaps the other's products.
MIR_EXPORT int mir_gemm_tc_set_stages(int swiglu, int other) {
  if (swiglu < 1 || swiglu > 4 || other < 1 || other > 6) {
    mir_set_error("tc_gemm: stages out of range");
    return MIR_BAD_ARGUMENT;
  }
  g_stages_swiglu = swiglu;
  g_stages_other = other;
  return MIR_OK;
}

// mode as in mir_gemm_skinny_bf16: 0 store bf16, 1 accumulate into float, 2 float, 3 SwiGLU (w = [gate; up],
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
