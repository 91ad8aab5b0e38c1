// C[M,N] = A[M,K] . W[N,K]^T in true 32-bit: FFMA on the CUDA cores, no tensor-core
// mode of reduced precision anywhere.  The reference runs its 32-bit path through a
// library product with TF32 switched off (engine/engine.py:190-192); this kernel makes
// the precision a property of the code instead of a global flag.  Each output sums its
// K products in ascending k whatever M is, so a row's result does not depend on which
// other rows share the launch.
#include "common.cuh"

namespace ek {

template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
sgemm_nt_kernel(float* __restrict__ C, const float* __restrict__ A, const float* __restrict__ W,
                int M, int N, int K, int lda, int ldw, int ldc) {
  constexpr int THREADS = (BM / TM) * (BN / TN);
  constexpr int PAD = 4;
  __shared__ __align__(16) float As[BK][BM + PAD];
  __shared__ __align__(16) float Ws[BK][BN + PAD];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int idx = tid; idx < BM * BK; idx += THREADS) {
      const int row = idx / BK, kk = idx % BK;
      const int gm = m0 + row, gk = k0 + kk;
      As[kk][row] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
    }
    for (int idx = tid; idx < BN * BK; idx += THREADS) {
      const int row = idx / BK, kk = idx % BK;
      const int gn = n0 + row, gk = k0 + kk;
      Ws[kk][row] = (gn < N && gk < K) ? W[(size_t)gn * ldw + gk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
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
      if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j];
    }
  }
}

}  // namespace ek

EK_EXPORT int ek_gemm_nt_f32(float* C, const float* A, const float* W, int M, int N, int K, int lda,
                             int ldw, int ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || lda < K || ldw < K || ldc < N) return EK_ERR_ARG;
  if (M <= 16) {
    constexpr int BM = 16, BN = 128, BK = 16, TM = 2, TN = 4;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return EK_ERR_ARG;
    ek::sgemm_nt_kernel<BM, BN, BK, TM, TN><<<grid, (BM / TM) * (BN / TN), 0, stream>>>(
        C, A, W, M, N, K, lda, ldw, ldc);
  } else {
    constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return EK_ERR_ARG;
    ek::sgemm_nt_kernel<BM, BN, BK, TM, TN><<<grid, (BM / TM) * (BN / TN), 0, stream>>>(
        C, A, W, M, N, K, lda, ldw, ldc);
  }
  EK_RETURN_LAUNCH_STATUS();
}
