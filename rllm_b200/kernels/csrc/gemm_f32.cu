// C[M, N] = A[M, K] . W[N, K]^T in true float32: FFMA on CUDA cores, no tensor
// cores and no reduced-precision matrix mode.  This is every projection of the
// 32-bit path (the reference calls a library matmul there,
// crates/rllm-model/src/layers.rs:162-175).
//
// Each output element is one thread's sequential sum over k = 0 .. K-1, so a
// row's result does not depend on M: the same token gives the same bits alone,
// in a portion of a prompt or in a mixed batch.
#include "common.cuh"

#define GF_BM 64
#define GF_BN 64
#define GF_BK 16

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw,
                float* __restrict__ C, int ldc, int M, int N, int K) {
  __shared__ float As[GF_BK][GF_BM + 4];
  __shared__ float Ws[GF_BK][GF_BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * GF_BM, n0 = blockIdx.x * GF_BN;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // each thread loads 4 elements of A and 4 of W per k-tile: row = tid / 4, k = (tid % 4) * 4 ..
  const int lr = tid / 4, lk = (tid % 4) * 4;
  for (int k0 = 0; k0 < K; k0 += GF_BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + lk + u;
      const int am = m0 + lr, wn = n0 + lr;
      As[lk + u][lr] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.f;
      Ws[lk + u][lr] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GF_BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[k][tn + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + tm + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tn + j;
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
  }
}

RLLM_EXPORT int rllm_gemm_f32(const float* A, int lda, const float* W, int ldw, float* C, int ldc,
                              int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || lda < K || ldw < K || ldc < N) return RLLM_E_BADARG;
  dim3 grid((N + GF_BN - 1) / GF_BN, (M + GF_BM - 1) / GF_BM);
  if (grid.y > 65535) return RLLM_E_UNSUPPORTED;
  gemm_f32_kernel<<<grid, 256, 0, stream>>>(A, lda, W, ldw, C, ldc, M, N, K);
  RLLM_LAUNCH_CHECK();
  return 0;
}
