// Plain tiled matrix product on the CUDA cores with 32-bit accumulation:
//   C[m][n] (=|+=) sum_k A[m][k] * W[n][k]        A: [M][K], W: [N][K] (row-major, "out x in")
// It is the matrix product of the true 32-bit path and the reference beside the tensor-core
// kernels.  Every output element is one thread's sum over k in ascending order, so a row's
// result does not depend on which other rows are in the batch.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TW, typename TC, bool ACCUMULATE>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                        TC* __restrict__ C, int M, int N, int K,
                                                        int lda, int ldw, int ldc) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // each thread loads 4 elements of each tile per k-step: row = tid / 4, k = (tid % 4) * 4 ..
  const int lrow = tid / 4, lk = (tid % 4) * 4;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      const int m = m0 + lrow, n = n0 + lrow;
      As[lk + i][lrow] = (m < M && k < K) ? to_f32(A[(size_t)m * lda + k]) : 0.f;
      Ws[lk + i][lrow] = (n < N && k < K) ? to_f32(W[(size_t)n * ldw + k]) : 0.f;
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
      if (n >= N) continue;
      TC* c = C + (size_t)m * ldc + n;
      if (ACCUMULATE)
        *c = from_f32<TC>(to_f32(*c) + acc[i][j]);
      else
        *c = from_f32<TC>(acc[i][j]);
    }
  }
}

template <typename TA, typename TW, typename TC>
int launch(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw, int ldc,
           int accumulate, cudaStream_t s) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (accumulate)
    gemm_simt_kernel<TA, TW, TC, true><<<grid, 256, 0, s>>>((const TA*)A, (const TW*)W, (TC*)C, M, N, K, lda, ldw, ldc);
  else
    gemm_simt_kernel<TA, TW, TC, false><<<grid, 256, 0, s>>>((const TA*)A, (const TW*)W, (TC*)C, M, N, K, lda, ldw, ldc);
  return launch_status();
}
}  // namespace

// dtypes: a, w in {f32, bf16}; c in {f32, bf16}.  accumulate: C += A W^T (C must be f32).
LLM_EXPORT int llm_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, void* C,
                             int c_dtype, int M, int N, int K, int lda, int ldw, int ldc,
                             int accumulate, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return LLM_ERR_ARGUMENT;
  if (accumulate && c_dtype != LLM_F32) return LLM_ERR_UNSUPPORTED;
#define GO(TA, TW, TC) return launch<TA, TW, TC>(A, W, C, M, N, K, lda, ldw, ldc, accumulate, stream)
  if (a_dtype == LLM_F32 && w_dtype == LLM_F32 && c_dtype == LLM_F32) GO(float, float, float);
  if (a_dtype == LLM_BF16 && w_dtype == LLM_BF16 && c_dtype == LLM_F32) GO(bf16, bf16, float);
  if (a_dtype == LLM_BF16 && w_dtype == LLM_BF16 && c_dtype == LLM_BF16) GO(bf16, bf16, bf16);
  if (a_dtype == LLM_BF16 && w_dtype == LLM_F32 && c_dtype == LLM_F32) GO(bf16, float, float);
  if (a_dtype == LLM_BF16 && w_dtype == LLM_F32 && c_dtype == LLM_BF16) GO(bf16, float, bf16);
  if (a_dtype == LLM_F32 && w_dtype == LLM_BF16 && c_dtype == LLM_F32) GO(float, bf16, float);
#undef GO
  return LLM_ERR_UNSUPPORTED;
}
