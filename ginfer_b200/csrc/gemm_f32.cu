// C[M, N] = A[M, K] * W[N, K]^T (+ bias[N]) in true fp32: FMA on the CUDA cores, no tensor-core
// mode of reduced precision.  This is the matrix product of the 32-bit path.  The reference has no
// fp32 product at all (ginfer/core/op/kernels/cuda/gemm_kernel/gemm_kernel.cu:166 registers f16 and
// bf16 only).  Every output element sums over k in ascending order whatever M is, so a row's result
// does not depend on what else is in the batch.
#include "common.cuh"

namespace gf {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W,
                const float* __restrict__ bias, float* __restrict__ C, int M, int N, int K,
                int lda, int ldc) {
  __shared__ float As[BK][BM + 1];
  __shared__ float Ws[BK][BN + 1];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid % 16, ty = tid / 16;          // 16 x 16 threads, each TM x TN outputs
  float acc[TM][TN] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 k = 1024 elements per operand, 4 per thread; k runs fastest within a row
    for (int e = tid; e < BM * BK; e += 256) {
      const int r = e / BK, kk = e % BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
      As[kk][r] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
      Ws[kk][r] = (gn < N && gk < K) ? W[(size_t)gn * K + gk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j] + (bias ? bias[gn] : 0.f);
    }
  }
}

}  // namespace gf

using namespace gf;

GF_DEFINE_PDL_SWITCH

GF_EXPORT int gf_gemm_f32(const float* A, int lda, const float* W, const float* bias, float* C,
                          int ldc, int M, int N, int K, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  gemm_f32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(A, W, bias, C, M, N, K, lda, ldc);
  return launch_status();
}
