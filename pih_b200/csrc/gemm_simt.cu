// C[M,N] = A[M,K] . W[N,K]^T on CUDA cores with 32-bit FMA accumulation.
//
// This is the matrix product of the true 32-bit path (no tensor cores, no
// TF32, no split tricks) and the plain twin of the tensor-core products.  It
// also takes bf16 inputs and writes bf16 or fp32.  Every output element is
// accumulated by one thread in ascending k — sixteen products into a partial
// sum, the partial sums into the total, which keeps the rounding error of a
// long sum (k of a thousand and more) near that of a short one — so a row's
// result does not depend on how many other rows the call holds: cutting a
// prompt into portions or batching it with other requests cannot change a bit.
//
// The reference runs all products through a library
// (src/backend/cuda/gemm_plan.cpp:83-199: row-major A[m,k], W[n,k] with
// CUBLAS_OP_T, 32-bit compute); it has no kernel of its own for them.
#include "common.cuh"

namespace pih {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TC>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TA* __restrict__ W, TC* __restrict__ C, int M, int N,
                 int K, long long lda, long long ldw, long long ldc) {
  wait_for_prior_kernels();
  launch_dependents();                                   // (the next kernel's blocks may become resident and wait)
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN);        // 0..15 -> columns
  const int ty = tid / (BN / TN);        // 0..15 -> rows
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64x16 elements per operand, 256 threads -> 4 each
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      const int r = e / BK, c = e % BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? to_float<TA>(A[static_cast<long long>(gm) * lda + gk]) : 0.0f;
      Ws[c][r] = (gn < N && gk < K) ? to_float<TA>(W[static_cast<long long>(gn) * ldw + gk]) : 0.0f;
    }
    __syncthreads();
    float part[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) part[i][j] = 0.0f;
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
        for (int j = 0; j < TN; ++j) part[i][j] = fmaf(a[i], w[j], part[i][j]);
    }
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] += part[i][j];
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn < N) C[static_cast<long long>(gm) * ldc + gn] = from_float<TC>(acc[i][j]);
    }
  }
}

}  // namespace pih

using namespace pih;

extern "C" int pih_gemm_simt(int in_dtype, int out_dtype, const void* A, const void* W, void* C, int M,
                             int N, int K, long long lda, long long ldw, long long ldc, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return PIH_ERR_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return PIH_ERR_UNSUPPORTED;
  if (in_dtype == PIH_F32 && out_dtype == PIH_F32)
    launch_kernel(gemm_simt_kernel<float, float>, dim3(grid), dim3(256), 0, s, static_cast<const float*>(A),
                                                        static_cast<const float*>(W),
                                                        static_cast<float*>(C), M, N, K, lda, ldw, ldc);
  else if (in_dtype == PIH_BF16 && out_dtype == PIH_BF16)
    launch_kernel(gemm_simt_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(grid), dim3(256), 0, s, 
        static_cast<const __nv_bfloat16*>(A), static_cast<const __nv_bfloat16*>(W),
        static_cast<__nv_bfloat16*>(C), M, N, K, lda, ldw, ldc);
  else if (in_dtype == PIH_BF16 && out_dtype == PIH_F32)
    launch_kernel(gemm_simt_kernel<__nv_bfloat16, float>, dim3(grid), dim3(256), 0, s, 
        static_cast<const __nv_bfloat16*>(A), static_cast<const __nv_bfloat16*>(W),
        static_cast<float*>(C), M, N, K, lda, ldw, ldc);
  else
    return PIH_ERR_BAD_ARGUMENT;
  PIH_LAUNCH_CHECK();
  return 0;
}
