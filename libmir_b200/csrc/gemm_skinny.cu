// Matrix products with few rows (1 to 16 tokens) in bf16: the decode step's projections.
//
//   out[M, N] = epilogue(x[M, K] . w[N, K]^T)
// With so few tokens the product is a stream of the weights: the work is to read w once at the speed of
// HBM.  A CTA owns 16 rows of w (32 for the SwiGLU epilogue) over a slice of K.  One warp asks the copy
// engine for each row's slice with a single bulk copy (cp.async.bulk, completion counted by an mbarrier),
// so the CTA's whole share of the weights is in flight after a few dozen instructions and no thread
// spends registers or address arithmetic on it.  When the bytes have landed the 8 warps take every 8th
// block of 32 k: 16 rows of w are the M side of mma.m16n8k16, 8 tokens the N side.  The partial sums of
// the warps are added in shared memory in warp order; K is cut over the CTAs of a thread-block cluster
// (so that matrices with few rows still fill the GPU, and so that a slice fits in shared memory), whose
// leader adds its peers' sums, in rank order, straight out of their shared memory.  The result is
// deterministic and needs neither atomics nor scratch in global memory.
//
// No data is rearranged for the fragments: inside one mma the order of k does not matter as long as
// both operands use the same order, so a lane takes 8 consecutive k of a row of w (16 bytes of shared
// memory) and the same 8 consecutive k of its token of x, and feeds them as (k, k+1 | k+4, k+5) and
// (k+2, k+3 | k+6, k+7) of two mma steps.  Rows in shared memory are padded so that the 16-byte reads of
// a warp fall on different banks.
//
// Epilogues (fused so that no extra kernel or round trip of the result is needed):
//   STORE   out bf16 = acc (+ bias)                       QKV projection
//   ACCUM   out float += acc (+ bias)                     output and down projections into the residual
//   F32     out float = acc (+ bias)                      output head (32-bit logits)
//   SWIGLU  out bf16 = silu(acc_gate) * acc_up            w holds [gate rows; up rows]: one launch, and
//                                                         the gate|up intermediate is never written
// Waits on the mbarrier are bounded: a CTA that gives up raises a flag that mir_stream_gemm_error()
// reads, and carries on (its output is then wrong, but nothing hangs).
// libmir plans a GEMV only for one token (DenseVectorPlan, cuda/src/backend/linear/autotune/
// candidate.rs:92-98) and otherwise a library GEMM followed by separate add / gate kernels
// (cuda/kernels/elementwise_bf16.cu:3-11,42-70).
#include <cooperative_groups.h>
#include "common.cuh"

namespace cg = cooperative_groups;

using namespace mir;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kWarps = 8;
enum Epilogue : int { STORE = 0, ACCUM = 1, F32 = 2, SWIGLU = 3 };

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_cached(const bf16* p, bool valid) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (valid) v = __ldg(reinterpret_cast<const uint4*>(p));
  return v;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ int g_stream_gemm_error = 0;                    // set when a bounded wait gave up

constexpr unsigned long long kWaitNanoseconds = 200ull * 1000ull * 1000ull;   // a copy of a few KB takes microseconds

__device__ __forceinline__ unsigned long long global_nanoseconds() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Wait for the phase with the given parity; false if the time limit ran out.  test_wait never blocks.
__device__ __forceinline__ bool wait_barrier(uint32_t barrier, uint32_t parity) {
  const unsigned long long start = global_nanoseconds();
  for (;;) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred P1;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, P1;\n\t}"
        : "=r"(done)
        : "r"(barrier), "r"(parity)
        : "memory");
    if (done) return true;
    if (global_nanoseconds() - start > kWaitNanoseconds) return false;
    __nanosleep(64);
  }
}

// RS row sets of 16 rows of w per CTA (for SWIGLU: RS/2 gate sets then RS/2 up sets), NT tiles of 8 tokens.
// Dynamic shared memory: [barrier, 128 bytes][RS*16 rows of w, row_bytes each][warps][PARTIAL][PARTIAL].
template <int RS, int NT, int MODE>
__global__ void __launch_bounds__(kWarps * 32)
skinny_gemm_kernel(const bf16* __restrict__ x, int ldx, const bf16* __restrict__ w, const void* __restrict__ bias,
                   void* __restrict__ out, int ldo, int m, int n, int k, int up_offset, int k_per_split,
                   int row_bytes) {
  constexpr int SETS = MODE == SWIGLU ? RS / 2 : RS;       // row sets that become distinct output columns
  constexpr int ROWS = RS * 16;
  constexpr int TOKENS = NT * 8;
  constexpr int PARTIAL = RS * 16 * TOKENS;                // floats of one CTA's partial result
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t barrier = smem_u32(smem);
  unsigned char* w_rows = smem + 128;
  float* reduce = reinterpret_cast<float*>(w_rows + (size_t)ROWS * row_bytes);
  float* cta_sum = reduce + kWarps * PARTIAL;
  cg::cluster_group cluster = cg::this_cluster();
  const int splits = gridDim.y, split = blockIdx.y;        // the cluster spans gridDim.y: K is cut into `splits`
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad = lane & 3, group = lane >> 2;
  const int n0 = blockIdx.x * 16 * SETS;
  const int k0 = split * k_per_split;
  const int k_len = max(0, min(k - k0, k_per_split));      // this CTA's slice of K (a multiple of 8)
  const uint32_t slice_bytes = (uint32_t)k_len * 2u;

  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(barrier) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0) {
    // which global row each shared-memory row holds; rows past the end of w are left out and read as zero
    int valid_rows = 0;
    for (int r = lane; r < ROWS; r += 32) {
      const int rs = r / 16;
      const int set = MODE == SWIGLU ? rs % SETS : rs;
      if (n0 + set * 16 + (r % 16) < n) ++valid_rows;
    }
    valid_rows = __reduce_add_sync(0xffffffffu, valid_rows);
    if (lane == 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(barrier),
                   "r"(slice_bytes * (uint32_t)valid_rows)
                   : "memory");
    __syncwarp();
    if (slice_bytes > 0) {
      for (int r = lane; r < ROWS; r += 32) {
        const int rs = r / 16;
        const int set = MODE == SWIGLU ? rs % SETS : rs;
        const int base = (MODE == SWIGLU && rs >= SETS) ? up_offset : 0;
        const int row = n0 + set * 16 + (r % 16);
        if (row >= n) continue;
        const bf16* src = w + (size_t)(base + row) * k + k0;
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         smem_u32(w_rows + (size_t)r * row_bytes)),
                     "l"(src), "r"(slice_bytes), "r"(barrier)
                     : "memory");
      }
    }
  }

  // The weights do not depend on the kernel before this one: their copies are under way.  Everything from
  // here on reads activations or writes results, so it waits for that kernel to be complete.
  grid_launch_dependents();
  grid_dependency_wait();

  const bf16* x_row[NT];
  bool ok_x[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int token = nt * 8 + group;
    ok_x[nt] = token < m;
    x_row[nt] = x + (size_t)token * ldx + k0 + quad * 8;
  }
  bool ok_lo[RS], ok_hi[RS];
#pragma unroll
  for (int rs = 0; rs < RS; ++rs) {
    const int set = MODE == SWIGLU ? rs % SETS : rs;
    ok_lo[rs] = n0 + set * 16 + group < n;
    ok_hi[rs] = n0 + set * 16 + group + 8 < n;
  }
  float acc[RS][NT][4];
#pragma unroll
  for (int rs = 0; rs < RS; ++rs)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[rs][nt][0] = acc[rs][nt][1] = acc[rs][nt][2] = acc[rs][nt][3] = 0.0f;

  if (!wait_barrier(barrier, 0)) {
    g_stream_gemm_error = 1;
    wait_barrier(barrier, 0);                              // once more, so that no copy lands after the CTA left
  }

  const int blocks = (k_len + 31) / 32;
  constexpr int U = 4;
  for (int block0 = warp; block0 < blocks; block0 += kWarps * U) {
    uint4 b[U][NT];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int offset = (block0 + u * kWarps) * 32;
      const bool in_k = offset + quad * 8 + 8 <= k_len;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) b[u][nt] = load_cached(x_row[nt] + offset, in_k && ok_x[nt]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int offset = (block0 + u * kWarps) * 32;
      if (offset >= k_len) continue;                       // the same for the whole warp: mma.sync needs all lanes
      const bool in_k = offset + quad * 8 + 8 <= k_len;    // a lane past the end of the slice feeds zeros
#pragma unroll
      for (int rs = 0; rs < RS; ++rs) {
        const unsigned char* lo = w_rows + (size_t)(rs * 16 + group) * row_bytes + (size_t)offset * 2 + quad * 16;
        uint4 a_lo = make_uint4(0u, 0u, 0u, 0u), a_hi = make_uint4(0u, 0u, 0u, 0u);
        if (in_k && ok_lo[rs]) a_lo = *reinterpret_cast<const uint4*>(lo);
        if (in_k && ok_hi[rs]) a_hi = *reinterpret_cast<const uint4*>(lo + (size_t)8 * row_bytes);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          mma_bf16(acc[rs][nt], a_lo.x, a_hi.x, a_lo.z, a_hi.z, b[u][nt].x, b[u][nt].z);
          mma_bf16(acc[rs][nt], a_lo.y, a_hi.y, a_lo.w, a_hi.w, b[u][nt].y, b[u][nt].w);
        }
      }
    }
  }

  // partial sums of the 8 warps -> shared memory -> one sum per CTA
  float* mine = reduce + (size_t)warp * PARTIAL;
#pragma unroll
  for (int rs = 0; rs < RS; ++rs)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int token = nt * 8 + quad * 2;
      float* base = mine + (size_t)rs * 16 * TOKENS;
      base[group * TOKENS + token] = acc[rs][nt][0];
      base[group * TOKENS + token + 1] = acc[rs][nt][1];
      base[(group + 8) * TOKENS + token] = acc[rs][nt][2];
      base[(group + 8) * TOKENS + token + 1] = acc[rs][nt][3];
    }
  __syncthreads();
  for (int index = threadIdx.x; index < PARTIAL; index += kWarps * 32) {
    float total = 0.0f;
#pragma unroll
    for (int wp = 0; wp < kWarps; ++wp) total += reduce[(size_t)wp * PARTIAL + index];
    cta_sum[index] = total;
  }
  cluster.sync();                                          // every CTA's sum is in its shared memory
  if (split == 0) {
    // outputs of the cluster: SETS * 16 columns x m tokens; consecutive threads take consecutive columns
    const int columns = SETS * 16;
    for (int index = threadIdx.x; index < columns * m; index += kWarps * 32) {
      const int token = index / columns, local = index % columns;
      const int column = n0 + local;
      if (column >= n) continue;
      const int set = local / 16, row = local % 16;
      const int at = (set * 16 + row) * TOKENS + token;
      float value = 0.0f, other = 0.0f;
      for (int rank = 0; rank < splits; ++rank) {
        const float* peer = cluster.map_shared_rank(cta_sum, rank);
        value += peer[at];
        if (MODE == SWIGLU) other += peer[at + SETS * 16 * TOKENS];
      }
      if (MODE == SWIGLU) {
        reinterpret_cast<bf16*>(out)[(size_t)token * ldo + column] =
            __float2bfloat16_rn(value / (1.0f + expf(-value)) * other);
      } else if (MODE == STORE) {
        if (bias) value += __bfloat162float(reinterpret_cast<const bf16*>(bias)[column]);
        reinterpret_cast<bf16*>(out)[(size_t)token * ldo + column] = __float2bfloat16_rn(value);
      } else {
        if (bias) value += reinterpret_cast<const float*>(bias)[column];
        float* dst = reinterpret_cast<float*>(out) + (size_t)token * ldo + column;
        *dst = MODE == ACCUM ? *dst + value : value;
      }
    }
  }
  cluster.sync();                                          // peers keep their shared memory until it was read
}

constexpr int kTargetCtas = 4 * 148;
constexpr int kSliceBudget = 80 * 1024;                    // bytes of weights one CTA holds (two CTAs fit an SM)

template <int RS, int NT, int MODE>
int launch(const bf16* x, int ldx, const bf16* w, const void* bias, void* out, int ldo, int m, int n, int k,
           int up_offset, cudaStream_t stream) {
  constexpr int SETS = MODE == SWIGLU ? RS / 2 : RS;
  constexpr int ROWS = RS * 16;
  const int tiles = (n + 16 * SETS - 1) / (16 * SETS);
  // cut K: first until a slice fits in shared memory, then further while the GPU is not full
  int splits = 1;
  auto per_split = [&](int s) { return ((k + s - 1) / s + 31) / 32 * 32; };
  while (splits < 8 && (size_t)ROWS * per_split(splits) * 2 > (size_t)kSliceBudget) splits *= 2;
  if ((size_t)ROWS * per_split(splits) * 2 > (size_t)200 * 1024) {
    mir_set_error("skinny_gemm: k %d is too long for this kernel (a slice of %d rows must fit in shared memory)", k,
                  ROWS);
    return MIR_BAD_ARGUMENT;
  }
  while (splits < 8 && tiles * splits < kTargetCtas && per_split(splits * 2) >= 512) splits *= 2;
  const int k_per_split = per_split(splits);
  int row_bytes = k_per_split * 2;
  if ((row_bytes / 16) % 2 == 0) row_bytes += 16;          // an odd number of 16-byte units: no bank conflicts
  const size_t smem = 128 + (size_t)ROWS * row_bytes + (size_t)(kWarps + 1) * RS * 16 * NT * 8 * sizeof(float);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    const cudaError_t err = cudaFuncSetAttribute(skinny_gemm_kernel<RS, NT, MODE>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) {
      mir_set_error("skinny_gemm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
      return MIR_CUDA_ERROR;
    }
    configured = smem;
  }
  return mir_launch("skinny_gemm", skinny_gemm_kernel<RS, NT, MODE>, dim3(tiles, splits, 1), dim3(kWarps * 32), smem,
                    stream, splits, x, ldx, w, bias, out, ldo, m, n, k, up_offset, k_per_split, row_bytes);
}

template <int MODE>
int dispatch(const bf16* x, int ldx, const bf16* w, const void* bias, void* out, int ldo, int m, int n, int k,
             int up_offset, cudaStream_t stream) {
  if (MODE == SWIGLU) {                          // two row sets (gate, up) per output set
    if (m <= 8) return launch<2, 1, MODE>(x, ldx, w, bias, out, ldo, m, n, k, up_offset, stream);
    return launch<2, 2, MODE>(x, ldx, w, bias, out, ldo, m, n, k, up_offset, stream);
  }
  if (m <= 8) return launch<1, 1, MODE>(x, ldx, w, bias, out, ldo, m, n, k, up_offset, stream);
  return launch<1, 2, MODE>(x, ldx, w, bias, out, ldo, m, n, k, up_offset, stream);
}

}  // namespace

MIR_EXPORT int mir_skinny_gemm_max_rows() { return 16; }

// 1 if a CTA of the few-rows product ever gave up waiting for its weights (then its output was wrong), else 0.
// Synchronises the device.
MIR_EXPORT int mir_stream_gemm_error() {
  int flag = 0;
  if (cudaMemcpyFromSymbol(&flag, g_stream_gemm_error, sizeof(int)) != cudaSuccess) return -1;
  return flag;
}

// mode: 0 out bf16 = x w^T (+bias bf16); 1 out float += x w^T (+bias float); 2 out float = x w^T (+bias float);
// 3 out bf16 [m, n] = silu(x w[0:n]^T) * (x w[up_offset : up_offset + n]^T).
// Needs m <= 16, k a multiple of 8, ldx a multiple of 8, and x and w on 16-byte boundaries.
MIR_EXPORT int mir_gemm_skinny_bf16(int mode, const void* x, int ldx, const void* w, const void* bias, void* out,
                                    int ldo, int m, int n, int k, int up_offset, cudaStream_t stream) {
  if (m == 0 || n == 0) return MIR_OK;
  if (m < 0 || m > 16 || n < 0 || k <= 0 || (k % 8) || (ldx % 8) || ldx < k || ldo < n ||
      ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) {
    mir_set_error("skinny_gemm: needs 1..16 rows, k and the row stride multiples of 8 and 16-byte aligned operands "
                  "(m %d n %d k %d ldx %d ldo %d)", m, n, k, ldx, ldo);
    return MIR_BAD_ARGUMENT;
  }
  const bf16* xx = (const bf16*)x;
  const bf16* ww = (const bf16*)w;
  switch (mode) {
    case STORE: return dispatch<STORE>(xx, ldx, ww, bias, out, ldo, m, n, k, 0, stream);
    case ACCUM: return dispatch<ACCUM>(xx, ldx, ww, bias, out, ldo, m, n, k, 0, stream);
    case F32: return dispatch<F32>(xx, ldx, ww, bias, out, ldo, m, n, k, 0, stream);
    case SWIGLU:
      if (bias) { mir_set_error("skinny_gemm: the SwiGLU epilogue takes no bias"); return MIR_BAD_ARGUMENT; }
      return dispatch<SWIGLU>(xx, ldx, ww, nullptr, out, ldo, m, n, k, up_offset, stream);
  }
  mir_set_error("skinny_gemm: unknown mode %d", mode);
  return MIR_BAD_ARGUMENT;
}
