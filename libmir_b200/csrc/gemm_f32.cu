// C[M, N] = beta * C + A[M, K] . W[N, K]^T (+ bias[N]) in true 32-bit: plain FMA on CUDA cores, no
// tensor cores and no TF32.  This is the matrix product of the float32 engine.
//
// Each output element is one chain of fmaf over k = 0 .. K-1 in ascending order, so its value does
// not depend on M, on the tile it falls in or on what else is in the batch.  libmir has no 32-bit
// model path on CUDA (its ProjectionFormat has no F32 member, cuda/src/backend/linear/mod.rs:80-88);
// this kernel exists to show faults that bf16 rounding hides.
#include "common.cuh"

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ a, int lda,
                                                        const float* __restrict__ w, int ldw,
                                                        const float* __restrict__ bias, float* __restrict__ c, int ldc,
                                                        int m, int n, int k, float beta) {
  __shared__ float a_tile[BK][BM + 1];
  __shared__ float w_tile[BK][BN + 1];
  const int tid = threadIdx.x;
  const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
  const int ty = tid / (BN / TN), tx = tid % (BN / TN);
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < k; k0 += BK) {
    // 64 x 16 elements of each operand, 256 threads: 4 elements each; consecutive threads read consecutive k.
#pragma unroll
    for (int i = 0; i < (BM * BK) / 256; ++i) {
      const int index = tid + i * 256;
      const int r = index / BK, kk = index % BK;
      const int gr = row0 + r, gk = k0 + kk;
      a_tile[kk][r] = (gr < m && gk < k) ? a[(size_t)gr * lda + gk] : 0.0f;
      const int gc = col0 + r;
      w_tile[kk][r] = (gc < n && gk < k) ? w[(size_t)gc * ldw + gk] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[TM], wv[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) av[i] = a_tile[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) wv[j] = w_tile[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gr = row0 + ty * TM + i;
    if (gr >= m) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gc = col0 + tx * TN + j;
      if (gc >= n) continue;
      float value = acc[i][j];
      if (bias) value += bias[gc];
      float* dst = c + (size_t)gr * ldc + gc;
      *dst = beta != 0.0f ? fmaf(beta, *dst, value) : value;
    }
  }
}

MIR_EXPORT int mir_gemm_f32(const float* a, int lda, const float* w, int ldw, const float* bias, float* c, int ldc,
                            int m, int n, int k, float beta, cudaStream_t stream) {
  if (m == 0 || n == 0) return MIR_OK;
  if (m < 0 || n < 0 || k <= 0 || lda < k || ldw < k || ldc < n) {
    mir_set_error("gemm_f32: bad sizes m %d n %d k %d lda %d ldw %d ldc %d", m, n, k, lda, ldw, ldc);
    return MIR_BAD_ARGUMENT;
  }
  const dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
  if (grid.y > 65535) {
    mir_set_error("gemm_f32: %d rows exceed the grid limit", m);
    return MIR_BAD_ARGUMENT;
  }
  gemm_f32_kernel<<<grid, 256, 0, stream>>>(a, lda, w, ldw, bias, c, ldc, m, n, k, beta);
  return mir_check_launch("gemm_f32");
}
