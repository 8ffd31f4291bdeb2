// True float32 matrix product for the 32-bit path: C[M, N] = A[M, K] * W[N, K]^T with
// both operands stored K-major, as activations and `[out, in]` weights are.  Plain FFMA
// on the CUDA cores: no tensor cores and no reduced-precision mode, so a fault that
// bfloat16 rounding would hide shows up.  Each output element is one thread's sum over
// k in ascending order, whatever M is, so a row's result does not depend on the batch.
#include "common.cuh"

namespace ms {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C, int M, int N, int K,
                int lda, int ldw, int ldc) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int load_row = tid / 4, load_k = (tid % 4) * 4;
  float acc[TM][TN] = {};

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + load_k + i;
      const int am = m0 + load_row, wn = n0 + load_row;
      As[load_k + i][load_row] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.f;
      Ws[load_k + i][load_row] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
  }
}

}  // namespace ms

using namespace ms;

MS_EXPORT int ms_gemm_f32(const float* A, const float* W, float* C, int M, int N, int K, int lda, int ldw, int ldc,
                          cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  MS_REQUIRE(K > 0, "gemm_f32: inner size must be positive, got %d", K);
  MS_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm_f32: a row stride is smaller than its row (lda %d ldw %d ldc %d)",
             lda, ldw, ldc);
  const int grid_m = (M + BM - 1) / BM, grid_n = (N + BN - 1) / BN;
  MS_REQUIRE(grid_m <= 65535, "gemm_f32: %d rows in one launch is too many", M);
  dim3 grid(grid_n, grid_m);
  ms::launch(gemm_f32_kernel, grid, 256, 0, stream, A, W, C, M, N, K, lda, ldw, ldc);
  MS_CHECK_LAUNCH("gemm_f32");
  return 0;
}
