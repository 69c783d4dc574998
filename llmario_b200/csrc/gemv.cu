// Weight-streaming matrix product for a handful of rows (decode): bfloat16 weights and
// activations, 32-bit accumulation.
//   C[m][n] (=|+=) sum_k A[m][k] * W[n][k],   1 <= M <= 8
// Each warp owns four weight rows and all M activation rows; lanes stride over k in 16-byte
// pieces, so every weight byte is read once, coalesced, with several loads in flight per lane.
// A second entry fuses the gated activation: rows n and ff + n of the stacked gate/up matrix are
// reduced by the same warp and silu(gate) * up is written.
// The order of each sum depends on K only, not on M or on which rows share the launch.
#include "common.cuh"

namespace {
constexpr int ROWS = 4;      // weight rows per warp
constexpr int WARPS = 8;
constexpr int MAXM = 8;

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// mode 0: store to C (TC), 1: C(f32) += , 2: gated (rows r and r + half), store TC
template <int M, typename TC, int MODE>
__global__ void __launch_bounds__(WARPS * 32) gemv_kernel(const bf16* __restrict__ A,
                                                          const bf16* __restrict__ W,
                                                          TC* __restrict__ C, int N, int K, int lda,
                                                          int ldw, int ldc, int half) {
  pdl_trigger();
  pdl_wait();
  const int warp = blockIdx.x * WARPS + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  // gated: this warp owns ROWS/2 outputs: gate rows n0.., up rows half + n0..
  const int outs = MODE == 2 ? ROWS / 2 : ROWS;
  const int n0 = warp * outs;
  const int limit = MODE == 2 ? half : N;
  if (n0 >= limit) return;
  const bf16* wrow[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    int n = MODE == 2 ? (r < outs ? n0 + r : half + n0 + (r - outs)) : n0 + r;
    if ((MODE == 2 ? (n0 + (r % outs)) : n) >= limit) n = n0;  // out of range: recompute row n0
    wrow[r] = W + (size_t)n * ldw;
  }
  float acc[ROWS][M];
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = 0.f;

  for (int k = lane * 8; k < K; k += 32 * 8) {
    uint4 wv[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) wv[r] = __ldg(reinterpret_cast<const uint4*>(wrow[r] + k));
    float wf[ROWS][8];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) unpack8(wv[r], wf[r]);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const uint4 av = *reinterpret_cast<const uint4*>(A + (size_t)m * lda + k);
      float af[8];
      unpack8(av, af);
#pragma unroll
      for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[r][m] = fmaf(wf[r][j], af[j], acc[r][m]);
    }
  }
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = warp_sum(acc[r][m]);
  if (lane == 0) {
    if (MODE == 2) {
#pragma unroll
      for (int r = 0; r < outs; ++r) {
        if (n0 + r >= half) continue;
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float g = acc[r][m], u = acc[r + outs][m];
          C[(size_t)m * ldc + n0 + r] = from_f32<TC>(g / (1.0f + expf(-g)) * u);
        }
      }
    } else {
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        if (n0 + r >= N) continue;
#pragma unroll
        for (int m = 0; m < M; ++m) {
          TC* c = C + (size_t)m * ldc + n0 + r;
          if (MODE == 1) *c = from_f32<TC>(to_f32(*c) + acc[r][m]);
          else *c = from_f32<TC>(acc[r][m]);
        }
      }
    }
  }
}

template <int M, typename TC, int MODE>
void launch_m(const bf16* A, const bf16* W, TC* C, int N, int K, int lda, int ldw, int ldc, int half,
              cudaStream_t s) {
  const int outs = MODE == 2 ? ROWS / 2 : ROWS;
  const int limit = MODE == 2 ? half : N;
  const int warps = (limit + outs - 1) / outs;
  const int blocks = (warps + WARPS - 1) / WARPS;
  (void)launch_pdl(gemv_kernel<M, TC, MODE>, blocks, WARPS * 32, 0, s, A, W, C, N, K, lda, ldw, ldc, half);
}

template <typename TC, int MODE>
int launch(const bf16* A, const bf16* W, TC* C, int M, int N, int K, int lda, int ldw, int ldc,
           int half, cudaStream_t s) {
  switch (M) {
    case 1: launch_m<1, TC, MODE>(A, W, C, N, K, lda, ldw, ldc, half, s); break;
    case 2: launch_m<2, TC, MODE>(A, W, C, N, K, lda, ldw, ldc, half, s); break;
    case 3: launch_m<3, TC, MODE>(A, W, C, N, K, lda, ldw, ldc, half, s); break;
    case 4: launch_m<4, TC, MODE>(A, W, C, N, K, lda, ldw, ldc, half, s); break;
    case 5: launch_m<5, TC, MODE>(A, W, C, N, K, lda, ldw, ldc, half, s); break;
    case 6: launch_m<6, TC, MODE>(A, W, C, N, K, lda, ldw, ldc, half, s); break;
    case 7: launch_m<7, TC, MODE>(A, W, C, N, K, lda, ldw, ldc, half, s); break;
    case 8: launch_m<8, TC, MODE>(A, W, C, N, K, lda, ldw, ldc, half, s); break;
    default: return LLM_ERR_UNSUPPORTED;
  }
  return launch_status();
}
}  // namespace

// A, W bfloat16; K a multiple of 8 with 16-byte aligned rows; 1 <= M <= 8.
// mode 0: C = A W^T (c_dtype f32 or bf16); mode 1: C += A W^T (f32);
// mode 2: W is [2*half][K] (gate rows then up rows), C[m][n] = silu(gate) * up, n < half.
LLM_EXPORT int llm_gemv_bf16(const void* A, const void* W, void* C, int c_dtype, int M, int N,
                             int K, int lda, int ldw, int ldc, int mode, int half,
                             cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > MAXM || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0) return LLM_ERR_UNSUPPORTED;
  if (((uintptr_t)A | (uintptr_t)W) & 15) return LLM_ERR_UNSUPPORTED;
  const bf16* a = (const bf16*)A;
  const bf16* w = (const bf16*)W;
  if (mode == 1) {
    if (c_dtype != LLM_F32) return LLM_ERR_UNSUPPORTED;
    return launch<float, 1>(a, w, (float*)C, M, N, K, lda, ldw, ldc, half, stream);
  }
  if (mode == 0) {
    if (c_dtype == LLM_F32) return launch<float, 0>(a, w, (float*)C, M, N, K, lda, ldw, ldc, half, stream);
    if (c_dtype == LLM_BF16) return launch<bf16, 0>(a, w, (bf16*)C, M, N, K, lda, ldw, ldc, half, stream);
    return LLM_ERR_UNSUPPORTED;
  }
  if (mode == 2) {
    if (N != 2 * half) return LLM_ERR_ARGUMENT;
    if (c_dtype == LLM_F32) return launch<float, 2>(a, w, (float*)C, M, N, K, lda, ldw, ldc, half, stream);
    if (c_dtype == LLM_BF16) return launch<bf16, 2>(a, w, (bf16*)C, M, N, K, lda, ldw, ldc, half, stream);
    return LLM_ERR_UNSUPPORTED;
  }
  return LLM_ERR_ARGUMENT;
}
