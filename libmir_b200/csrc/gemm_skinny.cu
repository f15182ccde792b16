// Matrix products with few rows (1 to 16 tokens) in bf16: the decode step's projections.
//
//   out[M, N] = epilogue(x[M, K] . w[N, K]^T)
// With so few tokens the product is a stream of the weights: the work is to read w once at the speed of
// HBM.  The roles are swapped for the tensor cores: 16 rows of w are the M side of mma.m16n8k16 and 8
// tokens are the N side.  A CTA owns a strip of rows of w; its 8 warps split K between them (every warp
// takes every 8th block of 32 k), each lane reading 16 bytes of a row at a time, and the 8 partial
// sums are added in shared memory in warp order.  When a matrix has too few rows to fill the GPU that
// way, K is also split over the CTAs of a thread-block cluster, whose leader adds the partial sums of
// its peers, in rank order, straight out of their shared memory (distributed shared memory).  The
// result is deterministic and needs neither atomics nor scratch in global memory.
//
// No data is rearranged for the fragments: inside one mma the order of k does not matter as long as
// both operands use the same order, so a lane keeps the 8 consecutive k it loaded from a row of w and
// the same 8 consecutive k of its token of x, and feeds them as (k, k+1 | k+4, k+5) and
// (k+2, k+3 | k+6, k+7) of two mma steps.
//
// Epilogues (fused so that no extra kernel or round trip of the result is needed):
//   STORE   out bf16 = acc (+ bias)                       QKV projection, output head in bf16
//   ACCUM   out float += acc (+ bias)                     output and down projections into the residual
//   F32     out float = acc (+ bias)                      output head (32-bit logits)
//   SWIGLU  out bf16 = silu(acc_gate) * acc_up            w holds [gate rows; up rows]: one launch, and
//                                                         the gate|up intermediate is never written
// Two more fusions remove the RMSNorm kernel between products.  The ACCUM epilogue can also write, per token,
// the sum of squares of the 16 residual values it has just produced (`sumsq_out[tile][token]`); a later STORE
// or SWIGLU product can take the 32-bit residual itself as its input together with those partial sums: it
// adds them up in tile order, forms rsqrt(mean + eps), and normalises and rounds the values it reads on the
// fly, exactly as the norm kernel would have (NormFusion below).
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

__device__ __forceinline__ uint4 load_stream(const bf16* p, bool valid) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (valid) v = __ldcs(reinterpret_cast<const uint4*>(p));      // read once: do not keep in L1
  return v;
}
__device__ __forceinline__ uint4 load_cached(const bf16* p, bool valid) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (valid) v = __ldg(reinterpret_cast<const uint4*>(p));
  return v;
}

// Optional fusion of an RMSNorm into the products around it, without work in the inner loop:
//   - an accumulating product (it updates the residual r) also writes, per 16-column tile and token, the sum of
//     squares of the new values (`sumsq_out`), and the new values times the NEXT norm's weight, rounded to bf16
//     (`weighted_out` = bf16(r * g));
//   - the product after that norm takes `weighted_out` as its x and multiplies each token's results by
//     rsqrt(sum of squares / k + eps) (`sumsq`): W (r g s) = s W (r g), since s is one number per token.
// Each value is rounded to bf16 once, as when the norm runs as a kernel of its own.
struct NormFusion {
  const float* sumsq;        // consumer: [sumsq_tiles][kNormStatStride] partial sums of squares of x's rows before weighting
  int sumsq_tiles;
  float eps;
  float* sumsq_out;          // producer (ACCUM): [tiles][kNormStatStride] partial sums of squares of the rows it updates
  const float* next_weight;  // producer: [n] weight of the norm that follows, or null
  bf16* weighted_out;        // producer: [m, ld_weighted] bf16(new residual * next_weight)
  int ld_weighted;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// RS row sets of 16 rows of w per warp (for SWIGLU: RS/2 gate sets then RS/2 up sets), NT tiles of 8 tokens,
// U blocks of 32 k loaded before their products are issued.
template <int RS, int NT, int U, int MODE>
__global__ void __launch_bounds__(kWarps * 32)
skinny_gemm_kernel(const bf16* __restrict__ x, int ldx, const bf16* __restrict__ w, const void* __restrict__ bias,
                   void* __restrict__ out, int ldo, int m, int n, int k, int up_offset, NormFusion norm) {
  constexpr int SETS = MODE == SWIGLU ? RS / 2 : RS;       // row sets that become distinct output columns
  constexpr int TOKENS = NT * 8;
  constexpr int PARTIAL = RS * 16 * TOKENS;                // floats of one CTA's partial result
  extern __shared__ float shared[];                        // [warps][PARTIAL] then [PARTIAL] (the CTA's sum)
  float* cta_sum = shared + kWarps * PARTIAL;
  __shared__ float inverse_rms[16];
  cg::cluster_group cluster = cg::this_cluster();
  const int splits = gridDim.y, split = blockIdx.y;        // the cluster spans gridDim.y: K is cut into `splits`
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad = lane & 3, group = lane >> 2;
  const int n0 = blockIdx.x * 16 * SETS;
  grid_launch_dependents();

  const bf16* w_lo[RS];
  const bf16* w_hi[RS];
  bool ok_lo[RS], ok_hi[RS];
#pragma unroll
  for (int rs = 0; rs < RS; ++rs) {
    const int set = MODE == SWIGLU ? rs % SETS : rs;
    const int base = (MODE == SWIGLU && rs >= SETS) ? up_offset : 0;
    const int row = n0 + set * 16 + group;
    ok_lo[rs] = row < n;
    ok_hi[rs] = row + 8 < n;
    w_lo[rs] = w + (size_t)(base + row) * k + quad * 8;
    w_hi[rs] = w + (size_t)(base + row + 8) * k + quad * 8;
  }
  const bf16* x_row[NT];
  bool ok_x[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int token = nt * 8 + group;
    ok_x[nt] = token < m;
    x_row[nt] = x + (size_t)token * ldx + quad * 8;
  }

  float acc[RS][NT][4];
#pragma unroll
  for (int rs = 0; rs < RS; ++rs)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[rs][nt][0] = acc[rs][nt][1] = acc[rs][nt][2] = acc[rs][nt][3] = 0.0f;

  grid_dependency_wait();                                  // x and out belong to the kernels before this one
  const int blocks = (k + 31) / 32;
  const int per_split = (blocks + splits - 1) / splits;
  const int block_begin = split * per_split, block_end = min(blocks, block_begin + per_split);
  for (int block0 = block_begin + warp; block0 < block_end; block0 += kWarps * U) {
    uint4 a_lo[U][RS], a_hi[U][RS], b[U][NT];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int block = block0 + u * kWarps;
      const int offset = block * 32;
      const bool in_k = block < block_end && offset + quad * 8 + 8 <= k;
#pragma unroll
      for (int rs = 0; rs < RS; ++rs) {
        a_lo[u][rs] = load_stream(w_lo[rs] + offset, in_k && ok_lo[rs]);
        a_hi[u][rs] = load_stream(w_hi[rs] + offset, in_k && ok_hi[rs]);
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) b[u][nt] = load_cached(x_row[nt] + offset, in_k && ok_x[nt]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int rs = 0; rs < RS; ++rs)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          mma_bf16(acc[rs][nt], a_lo[u][rs].x, a_hi[u][rs].x, a_lo[u][rs].z, a_hi[u][rs].z, b[u][nt].x, b[u][nt].z);
          mma_bf16(acc[rs][nt], a_lo[u][rs].y, a_hi[u][rs].y, a_lo[u][rs].w, a_hi[u][rs].w, b[u][nt].y, b[u][nt].w);
        }
  }

  // one scale per token: 1, or the folded norm's rsqrt(mean of squares + eps); read after the syncs below
  if (threadIdx.x < 16) inverse_rms[threadIdx.x] = 1.0f;
  if (norm.sumsq != nullptr) {
    // 16 threads per token add the tiles' partial sums in a fixed order
    __syncthreads();
    const int token = threadIdx.x >> 4, part = threadIdx.x & 15;
    float sum = 0.0f;
    if (token < m)
      for (int tile = part; tile < norm.sumsq_tiles; tile += 16) sum += norm.sumsq[tile * kNormStatStride + token];
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (part == 0 && token < 16) inverse_rms[token] = rsqrtf(sum / (float)k + norm.eps);
  }
  // partial sums of the 8 warps -> shared memory -> one sum per CTA
  float* mine = shared + (size_t)warp * PARTIAL;
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
    for (int wp = 0; wp < kWarps; ++wp) total += shared[(size_t)wp * PARTIAL + index];
    cta_sum[index] = total;
  }
  cluster.sync();                                          // every CTA's sum is in its shared memory
  if (split == 0) {
    // outputs of the cluster: SETS * 16 columns x m tokens; consecutive threads take consecutive columns
    const int columns = SETS * 16;
    const int passes = (columns * TOKENS + kWarps * 32 - 1) / (kWarps * 32);
    for (int pass = 0; pass < passes; ++pass) {
      const int index = pass * kWarps * 32 + threadIdx.x;
      const int token = index / columns, local = index % columns;
      const int column = n0 + local;
      const bool active = token < m && column < n;
      float value = 0.0f, other = 0.0f;
      if (active) {
        const int set = local / 16, row = local % 16;
        const int at = (set * 16 + row) * TOKENS + token;
        for (int rank = 0; rank < splits; ++rank) {
          const float* peer = cluster.map_shared_rank(cta_sum, rank);
          value += peer[at];
          if (MODE == SWIGLU) other += peer[at + SETS * 16 * TOKENS];
        }
        const float scale = inverse_rms[token];              // 1 unless a norm is folded into this product
        value *= scale;
        other *= scale;
        if (MODE == SWIGLU) {
          reinterpret_cast<bf16*>(out)[(size_t)token * ldo + column] =
              __float2bfloat16_rn(value / (1.0f + expf(-value)) * other);
        } else if (MODE == STORE) {
          if (bias) value += __bfloat162float(reinterpret_cast<const bf16*>(bias)[column]);
          reinterpret_cast<bf16*>(out)[(size_t)token * ldo + column] = __float2bfloat16_rn(value);
        } else {
          if (bias) value += reinterpret_cast<const float*>(bias)[column];
          float* dst = reinterpret_cast<float*>(out) + (size_t)token * ldo + column;
          value = MODE == ACCUM ? *dst + value : value;
          *dst = value;
          if (MODE == ACCUM && norm.weighted_out != nullptr)
            norm.weighted_out[(size_t)token * norm.ld_weighted + column] =
                __float2bfloat16_rn(value * norm.next_weight[column]);
        }
      }
      if (MODE == ACCUM && norm.sumsq_out != nullptr) {
        // sum of squares of this tile's 16 new residual values of each token (16 consecutive lanes per token)
        float square = active ? value * value : 0.0f;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) square += __shfl_xor_sync(0xffffffffu, square, o);
        if (local == 0 && token < m) norm.sumsq_out[(size_t)blockIdx.x * kNormStatStride + token] = square;
      }
    }
  }
  cluster.sync();                                          // peers keep their shared memory until it was read
}

constexpr int kTargetCtas = 4 * 148;

template <int RS, int NT, int U, int MODE>
int launch(const bf16* x, int ldx, const bf16* w, const void* bias, void* out, int ldo, int m, int n, int k,
           int up_offset, const NormFusion& norm, cudaStream_t stream) {
  constexpr int SETS = MODE == SWIGLU ? RS / 2 : RS;
  const size_t smem = (size_t)(kWarps + 1) * RS * 16 * NT * 8 * sizeof(float);
  const int tiles = (n + 16 * SETS - 1) / (16 * SETS);
  const int blocks = (k + 31) / 32;
  int splits = 1;                                          // cut K over a cluster until the GPU is full
  while (splits < 8 && tiles * splits < kTargetCtas && blocks / (splits * 2 * kWarps) >= 2) splits *= 2;
  return mir_launch("skinny_gemm", skinny_gemm_kernel<RS, NT, U, MODE>, dim3(tiles, splits, 1), dim3(kWarps * 32), smem,
                    stream, splits, x, ldx, w, bias, out, ldo, m, n, k, up_offset, norm);
}

template <int MODE>
int dispatch(const bf16* x, int ldx, const bf16* w, const void* bias, void* out, int ldo, int m, int n, int k,
             int up_offset, const NormFusion& norm, cudaStream_t stream) {
  if (MODE == SWIGLU) {                          // two row sets (gate, up) per output set
    if (m <= 8) return launch<2, 1, 4, MODE>(x, ldx, w, bias, out, ldo, m, n, k, up_offset, norm, stream);
    return launch<2, 2, 4, MODE>(x, ldx, w, bias, out, ldo, m, n, k, up_offset, norm, stream);
  }
  if (m <= 8) return launch<1, 1, 8, MODE>(x, ldx, w, bias, out, ldo, m, n, k, up_offset, norm, stream);
  return launch<1, 2, 8, MODE>(x, ldx, w, bias, out, ldo, m, n, k, up_offset, norm, stream);
}

}  // namespace

MIR_EXPORT int mir_skinny_gemm_max_rows() { return 16; }

// mode: 0 out bf16 = x w^T (+bias bf16); 1 out float += x w^T (+bias float); 2 out float = x w^T (+bias float);
// 3 out bf16 [m, n] = silu(x w[0:n]^T) * (x w[up_offset : up_offset + n]^T).
// Needs m <= 16, k a multiple of 8, ldx a multiple of 8, and x and w on 16-byte boundaries.
// Norm fusion (all optional, see NormFusion): with `sumsq` [sumsq_tiles][kNormStatStride] each token's results are
// multiplied by rsqrt(sum / k + eps) (modes 0 and 3); with `sumsq_out` (mode 1 only) the product also writes the
// partial sums of squares of the rows it updates, [ceil(n / 16)][16] floats, and with `weighted_out` and
// `next_weight` the new rows times that weight as bf16.
MIR_EXPORT int mir_gemm_skinny_bf16(int mode, const void* x, int ldx, const void* w, const void* bias, void* out,
                                    int ldo, int m, int n, int k, int up_offset, const float* sumsq, int sumsq_tiles,
                                    float eps, float* sumsq_out, const float* next_weight, void* weighted_out,
                                    int ld_weighted, cudaStream_t stream) {
  if (m == 0 || n == 0) return MIR_OK;
  if (m < 0 || m > 16 || n < 0 || k <= 0 || (k % 8) || ldo < n || ((uintptr_t)w & 15) || (ldx % 8) || ldx < k ||
      ((uintptr_t)x & 15) || x == nullptr) {
    mir_set_error("skinny_gemm: needs 1..16 rows, k and the row stride multiples of 8 and 16-byte aligned operands "
                  "(m %d n %d k %d ldx %d ldo %d)", m, n, k, ldx, ldo);
    return MIR_BAD_ARGUMENT;
  }
  if ((sumsq_out != nullptr || weighted_out != nullptr) && mode != ACCUM) {
    mir_set_error("skinny_gemm: sums of squares and weighted rows are written by the accumulate epilogue only");
    return MIR_BAD_ARGUMENT;
  }
  if (sumsq != nullptr && (sumsq_tiles <= 0 || (mode != STORE && mode != SWIGLU))) {
    mir_set_error("skinny_gemm: a folded norm needs its partial sums, and the store or SwiGLU epilogue");
    return MIR_BAD_ARGUMENT;
  }
  if (weighted_out != nullptr && (next_weight == nullptr || sumsq_out == nullptr || ld_weighted < n)) {
    mir_set_error("skinny_gemm: weighted rows need the next norm's weight, a row stride >= n, and sums of squares");
    return MIR_BAD_ARGUMENT;
  }
  NormFusion norm;
  norm.sumsq = sumsq;
  norm.sumsq_tiles = sumsq_tiles;
  norm.eps = eps;
  norm.sumsq_out = sumsq_out;
  norm.next_weight = next_weight;
  norm.weighted_out = (bf16*)weighted_out;
  norm.ld_weighted = ld_weighted;
  const bf16* xx = (const bf16*)x;
  const bf16* ww = (const bf16*)w;
  switch (mode) {
    case STORE: return dispatch<STORE>(xx, ldx, ww, bias, out, ldo, m, n, k, 0, norm, stream);
    case ACCUM: return dispatch<ACCUM>(xx, ldx, ww, bias, out, ldo, m, n, k, 0, norm, stream);
    case F32: return dispatch<F32>(xx, ldx, ww, bias, out, ldo, m, n, k, 0, norm, stream);
    case SWIGLU:
      if (bias) { mir_set_error("skinny_gemm: the SwiGLU epilogue takes no bias"); return MIR_BAD_ARGUMENT; }
      return dispatch<SWIGLU>(xx, ldx, ww, nullptr, out, ldo, m, n, k, up_offset, norm, stream);
  }
  mir_set_error("skinny_gemm: unknown mode %d", mode);
  return MIR_BAD_ARGUMENT;
}
