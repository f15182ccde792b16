// tcgen05 / TMA / mbarrier building blocks shared by the kernels that run on the 5th-generation tensor cores:
// bounded mbarrier waits, shared-memory matrix descriptors for the 128-byte swizzle, instruction descriptors,
// tcgen05.mma / commit / ld / st wrappers, and a cache of TMA tensor maps (host side).
#pragma once
#include <cuda.h>
#include <map>
#include <mutex>
#include <tuple>
#include "common.cuh"

namespace mir {
namespace tc {

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

// The same for an MN-major operand (rows of the K dimension, each 128 bytes = 64 consecutive elements of the M
// or N dimension, 128-byte swizzle): 8 rows of K are 1024 bytes apart (stride byte offset), the next 64
// elements of M or N start `block_bytes` further (leading byte offset).
__device__ __forceinline__ uint64_t operand_descriptor_mn_major(uint32_t smem_address, uint32_t block_bytes) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_address >> 4) & 0x3FFF);
  desc |= (uint64_t)((block_bytes >> 4) & 0x3FFF) << 16;
  desc |= (uint64_t)(1024 >> 4) << 32;
  desc |= (uint64_t)1 << 46;
  desc |= (uint64_t)2 << 61;
  return desc;
}

// Instruction descriptor: D float32, A and B bf16, A K-major, B K-major or MN-major, M x N.
__host__ __device__ constexpr uint32_t instruction_descriptor(int m, int n, bool b_mn_major = false) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
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

// The same with the A operand in tensor memory: 128 lanes are its rows, every 32-bit column holds two consecutive
// 16-bit elements of K (a K of 16 is 8 columns from `tmem_a` on).
__device__ __forceinline__ void mma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

// Issuing from a whole warp.  A thread that issues products shares its scheduler with the CTA's other warps, and
// every instruction it needs between two products is one it has to win an issue slot for; when the others are busy
// (a softmax, an epilogue) a lone thread in a divergent branch, whose descriptors the compiler has to build in
// ordinary registers and move to uniform ones, fed the tensor cores a product of 64 cycles only every 80 to 170.
// So the issuing warp stays converged: all its lanes run the loop, the products are predicated on `elected`
// (elect_one(), taken once), and the descriptors are passed in two 32-bit halves: the upper half is the same for
// every operand with the 128-byte swizzle (stride byte offset 1024, version 1), the lower half holds the address in
// 16-byte units (and the leading byte offset of an MN-major operand), so the operand 16 bytes * n further on is
// `low + n`.  Measured beside 16 warps that saturate the schedulers: 71 cycles a product against 177.
constexpr uint32_t kOperandHigh = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t operand_low(uint32_t smem_address) {
  return ((smem_address >> 4) & 0x3FFFu) | (1u << 16);
}
__device__ __forceinline__ uint32_t operand_low_mn_major(uint32_t smem_address, uint32_t block_bytes) {
  return ((smem_address >> 4) & 0x3FFFu) | (((block_bytes >> 4) & 0x3FFFu) << 16);
}
// 1 in one lane of the (converged) warp, 0 in the others.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t elected;
  asm volatile("{\n\t.reg .pred q;\n\telect.sync _|q, 0xffffffff;\n\tselp.b32 %0, 1, 0, q;\n\t}" : "=r"(elected));
  return elected;
}
template <bool kAccumulate>
__device__ __forceinline__ void mma_bf16_ss_halves(uint32_t tmem_d, uint32_t a_low, uint32_t b_low, uint32_t idesc,
                                                   uint32_t elected) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 q, %7, 0;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, {%6, %6, %6, %6}, p;\n\t}"
      :
      : "r"(tmem_d), "r"(a_low), "r"(b_low), "r"(idesc), "n"(kAccumulate ? 1 : 0), "r"(kOperandHigh), "r"(0u),
        "r"(elected)
      : "memory");
}
// The same with the accumulate flag in a register.
__device__ __forceinline__ void mma_bf16_ss_halves(uint32_t tmem_d, uint32_t a_low, uint32_t b_low, uint32_t idesc,
                                                   uint32_t accumulate, uint32_t elected) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 q, %7, 0;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, {%6, %6, %6, %6}, p;\n\t}"
      :
      : "r"(tmem_d), "r"(a_low), "r"(b_low), "r"(idesc), "r"(accumulate), "r"(kOperandHigh), "r"(0u), "r"(elected)
      : "memory");
}
__device__ __forceinline__ void mma_bf16_ts_halves(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_low, uint32_t idesc,
                                                   uint32_t accumulate, uint32_t elected) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 db;\n\t"
      "setp.ne.b32 q, %7, 0;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, {%6, %6, %6, %6}, p;\n\t}"
      :
      : "r"(tmem_d), "r"(tmem_a), "r"(b_low), "r"(idesc), "r"(accumulate), "r"(kOperandHigh), "r"(0u), "r"(elected)
      : "memory");
}
// mma_commit by the elected lane of a converged warp.
__device__ __forceinline__ void mma_commit_elected(uint32_t barrier, uint32_t elected) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(barrier), "r"(elected)
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

// 16 consecutive accumulator columns of this thread's lane.
__device__ __forceinline__ void tmem_load_16(uint32_t address, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(address)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Write 32 consecutive accumulator columns of this thread's lane; tmem_store_wait() before anyone reads them.
__device__ __forceinline__ void tmem_store_32(uint32_t address, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(address), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
        "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])),
        "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])),
        "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])),
        "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
// Write 32 consecutive 32-bit columns of this thread's lane (raw bits); tmem_store_wait() before anyone reads them.
__device__ __forceinline__ void tmem_store_32_bits(uint32_t address, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(address), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void barrier_init(uint32_t barrier, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(barrier), "r"(count) : "memory");
}
__device__ __forceinline__ void barrier_arrive(uint32_t barrier) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(barrier) : "memory");
}
__device__ __forceinline__ void barrier_expect_bytes(uint32_t barrier, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(barrier), "r"(bytes) : "memory");
}
// One box of a 2-d tensor map into shared memory; the bytes count on `barrier`.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t barrier, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(barrier), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tensor_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tensor_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ------------------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Tensor map of a row-major bf16 matrix [rows, k] with row stride ld: boxes of box_rows rows x 64 k, 128-byte
// swizzle, out-of-range elements read as zero.
inline int tensor_map_for(const void* base, int rows, int k, int ld, int box_rows, CUtensorMap* map) {
  static std::mutex g_mutex;
  static EncodeTiled g_encode = nullptr;
  static std::map<std::tuple<const void*, int, int, int, int>, CUtensorMap> g_maps;
  std::lock_guard<std::mutex> lock(g_mutex);
  const auto key = std::make_tuple(base, rows, k, ld, box_rows);
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
      mir_set_error("tensor map: the driver has no cuTensorMapEncodeTiled");
      return MIR_LIBRARY_ERROR;
    }
    g_encode = reinterpret_cast<EncodeTiled>(entry);
  }
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  const cuuint32_t element_strides[2] = {1, 1};
  CUtensorMap made;
  const CUresult status = g_encode(&made, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                                   box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (status != CUDA_SUCCESS) {
    mir_set_error("tensor map: cuTensorMapEncodeTiled refused a %d x %d matrix with row stride %d (status %d)", rows, k,
                  ld, (int)status);
    return MIR_LIBRARY_ERROR;
  }
  if (g_maps.size() > 4096) g_maps.clear();                  // activation buffers come and go
  g_maps.emplace(key, made);
  *map = made;
  return MIR_OK;
}


}  // namespace tc
}  // namespace mir
