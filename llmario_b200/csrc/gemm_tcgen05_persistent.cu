// Persistent form of the tcgen05 matrix product for many rows (prompt portions):
//     C[t][n] (=|+=) sum_k X[t][k] * W[n][k],   tiles of 128 weight rows x 256 tokens.
// One CTA per SM walks over output tiles (tile = blockIdx.x, + gridDim.x, ...; tiles that share a
// weight tile are neighbours, so they run at the same time on different SMs and meet in L2).
//
//   warp 0     TMA producer: runs ahead across tile boundaries through a ring of shared-memory
//              stages (W tile 16 KB + X tile 32 KB each)
//   warp 1     issues tcgen05.mma 128 x 256 x 16 into one of two TMEM accumulators (2 x 256 columns)
//   warps 2-5  epilogue of the other accumulator while the next tile is being multiplied: TMEM ->
//              registers -> shared memory in chunks of 32 tokens -> TMA store (or TMA add-reduction
//              into the float32 residual stream), two chunk buffers in flight
//
// The same epilogues as the one-tile kernel: store, residual add, gated silu(g) * u.  The output
// must be reachable by TMA (16-byte aligned rows); the caller falls back to the one-tile kernel
// otherwise.  Every mbarrier wait is bounded.
#include "tcgen05.cuh"

namespace {

constexpr int BN = 256;          // tokens per tile
constexpr int CH = 32;           // tokens per epilogue chunk

template <int STAGES, int FEAT, typename TC>
struct alignas(1024) PersistentStorage {
  uint8_t a[STAGES][TILE_M * TILE_K * 2];
  uint8_t b[STAGES][BN * TILE_K * 2];
  alignas(128) TC out[2][CH * FEAT];
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int dead;
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <int STAGES, int EPI, typename TC>
__global__ void __launch_bounds__(192, 1) gemm_persistent_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
    const __grid_constant__ CUtensorMap map_c, int T, int N, int K, int half, int interleaved, int m_tiles,
    int n_tiles, int* __restrict__ status) {
  constexpr int FEAT = EPI == EPI_GATED ? 64 : TILE_M;
  extern __shared__ uint8_t raw[];
  auto& sm = *reinterpret_cast<PersistentStorage<STAGES, FEAT, TC>*>(
      (reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = (K + TILE_K - 1) / TILE_K;
  const int tiles = m_tiles * n_tiles;
  constexpr uint32_t STAGE_BYTES = TILE_M * TILE_K * 2 + BN * TILE_K * 2;
  constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)(TILE_M >> 4) << 24);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.acc_full[b], 1);
      mbar_init(&sm.acc_empty[b], 4);      // one arrival per epilogue warp
    }
    sm.dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------------ producer
    auto load_w = [&](int s, int n0, int k) {
      mbar_expect_tx(&sm.full[s], STAGE_BYTES);
      if (EPI == EPI_GATED && interleaved) {
        tma_load_2d(sm.a[s], &map_w, k, 2 * n0, &sm.full[s]);     // 16 gate rows, 16 up rows, ... as stored
      } else if (EPI == EPI_GATED) {
#pragma unroll
        for (int b = 0; b < 8; ++b)
          tma_load_2d(sm.a[s] + b * 16 * TILE_K * 2, &map_w, k, ((b & 1) ? half : 0) + n0 + (b >> 1) * 16,
                      &sm.full[s]);
      } else {
        tma_load_2d(sm.a[s], &map_w, k, n0, &sm.full[s]);
      }
    };
    long long it = 0;       // k-blocks issued so far, over all tiles of this CTA
    bool ok = true;
    bool first = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
      const int n0 = (tile / n_tiles) * FEAT, t0 = (tile % n_tiles) * BN;
      int kb = 0;
      if (first) {
        // weights do not depend on earlier kernels: fetch a ring of them before waiting
        const int head = min(nkb, STAGES);
        for (int i = 0; i < head; ++i) load_w(i, n0, i * TILE_K);
        pdl_wait();
        for (int i = 0; i < head; ++i) tma_load_2d(sm.b[i], &map_x, i * TILE_K, t0, &sm.full[i]);
        it = head;
        kb = head;
        first = false;
      }
      for (; kb < nkb; ++kb, ++it) {
        const int s = (int)(it % STAGES);
        ok = mbar_wait(&sm.empty[s], (uint32_t)((it / STAGES) & 1) ^ 1);
        if (!ok) { atomicExch(status, 1); sm.dead = 1; break; }
        load_w(s, n0, kb * TILE_K);
        tma_load_2d(sm.b[s], &map_x, kb * TILE_K, t0, &sm.full[s]);
      }
    }
    if (!ok) {      // let what is in flight land before the shared memory is given up
      for (long long i = max(0LL, it - STAGES); i < it; ++i)
        mbar_wait(&sm.full[i % STAGES], (uint32_t)((i / STAGES) & 1));
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------------ MMA issuer
    long long it = 0;
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      ok = mbar_wait(&sm.acc_empty[buf], (uint32_t)((local >> 1) & 1) ^ 1);
      if (!ok) { atomicExch(status, 2); sm.dead = 1; break; }
      tc_fence_after();
      const uint32_t acc = tmem + (uint32_t)buf * BN;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = (int)(it % STAGES);
        ok = mbar_wait(&sm.full[s], (uint32_t)((it / STAGES) & 1));
        if (!ok) { atomicExch(status, 2); sm.dead = 1; break; }
        tc_fence_after();
        const uint64_t da = smem_desc(smem_u32(sm.a[s]));
        const uint64_t db = smem_desc(smem_u32(sm.b[s]));
#pragma unroll
        for (int k = 0; k < TILE_K / UMMA_K; ++k)
          tc_mma(acc, da + (uint64_t)(k * UMMA_K * 2 >> 4), db + (uint64_t)(k * UMMA_K * 2 >> 4), idesc,
                 (kb > 0 || k > 0) ? 1u : 0u);
        tc_commit(&sm.empty[s]);
      }
      if (ok) tc_commit(&sm.acc_full[buf]);
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const bool issuer = warp == 2 && lane == 0;
    pdl_wait();
    int local = 0;
    int chunk_no = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
      const int n0 = (tile / n_tiles) * FEAT, t0 = (tile % n_tiles) * BN;
      const int buf = local & 1;
      bool ok = mbar_wait(&sm.acc_full[buf], (uint32_t)((local >> 1) & 1));
      if (!ok) { if (lane == 0) atomicExch(status, 3); sm.dead = 1; }
      // the four warps decide together whether to go on
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (sm.dead) break;
      tc_fence_after();
      const uint32_t acc = tmem + (uint32_t)buf * BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN; c += CH, ++chunk_no) {
        TC* stage_out = sm.out[chunk_no & 1];
        // the store that last used this buffer (two chunks ago) must have read it
        if (issuer) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (int h = 0; h < CH / 16; ++h) {
          uint32_t v[16];
          tmem_ld16(acc + (uint32_t)(c + h * 16), v);
          tmem_ld_wait();
          if (EPI == EPI_GATED) {
            const int f = q * 16 + (lane & 15);
            const int col0 = h * 16 + (lane < 16 ? 0 : 8);
            float r[8];
            gated_columns<TC>(v, lane, r);
#pragma unroll
            for (int i = 0; i < 8; ++i) stage_out[(col0 + i) * FEAT + f] = from_f32<TC>(r[i]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              stage_out[(h * 16 + j) * FEAT + row] = from_f32<TC>(__uint_as_float(v[j]));
          }
        }
        if (c + CH >= BN) {           // this accumulator has been read completely
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.acc_empty[buf]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (issuer) {
          const uint32_t src = smem_u32(stage_out);
          if (EPI == EPI_ACCUM)
            asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
                         ::"l"(&map_c), "r"(src), "r"(n0), "r"(t0 + c) : "memory");
          else
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                         ::"l"(&map_c), "r"(src), "r"(n0), "r"(t0 + c) : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
    }
    if (issuer) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

template <int STAGES, int EPI, typename TC>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mc, int T, int N, int K, int half,
           int interleaved, int sm_count, int* status, cudaStream_t stream) {
  constexpr int FEAT = EPI == EPI_GATED ? 64 : TILE_M;
  auto kernel = gemm_persistent_kernel<STAGES, EPI, TC>;
  constexpr int smem = (int)sizeof(PersistentStorage<STAGES, FEAT, TC>) + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int limit = EPI == EPI_GATED ? half : N;
  const int m_tiles = (limit + FEAT - 1) / FEAT, n_tiles = (T + BN - 1) / BN;
  const int grid = m_tiles * n_tiles < sm_count ? m_tiles * n_tiles : sm_count;
  return launch_pdl(kernel, grid, 192, smem, stream, mw, mx, mc, T, N, K, half, interleaved, m_tiles, n_tiles,
                    status);
}
}  // namespace

// The persistent kernel for bfloat16 X [T][K], W [N][K]; modes as llm_gemm_tcgen05 (no K split).
// Returns LLM_ERR_UNSUPPORTED when the output cannot be written by TMA.
int llm_gemm_tcgen05_persistent(const void* X, const void* W, void* C, int c_dtype, int T, int N, int K,
                                int lda, int ldw, int ldc, int mode, int half, int* status,
                                cudaStream_t stream) {
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  const int esize = c_dtype == LLM_F32 ? 4 : 2;
  if (((uintptr_t)C & 15) || ((size_t)ldc * esize) % 16) return LLM_ERR_UNSUPPORTED;
  CUtensorMap mw, mx, mc;
  if (!llm_tensor_map(W, N, K, ldw, mode == 2 ? 16 : TILE_M, TILE_K, 0, &mw)) return LLM_ERR_UNSUPPORTED;
  if (!llm_tensor_map(X, T, K, lda, BN, TILE_K, 0, &mx)) return LLM_ERR_UNSUPPORTED;
  const int out_cols = mode >= 2 ? half : N;
  if (!llm_tensor_map(C, T, out_cols, ldc, CH, mode >= 2 ? 64 : TILE_M, c_dtype == LLM_F32 ? 2 : 1, &mc))
    return LLM_ERR_UNSUPPORTED;
  if (mode == 0) {
    if (c_dtype == LLM_F32) return launch<4, EPI_STORE, float>(mw, mx, mc, T, N, K, half, mode == 3, sm_count, status, stream);
    if (c_dtype == LLM_BF16) return launch<4, EPI_STORE, bf16>(mw, mx, mc, T, N, K, half, mode == 3, sm_count, status, stream);
  } else if (mode == 1) {
    if (c_dtype == LLM_F32) return launch<4, EPI_ACCUM, float>(mw, mx, mc, T, N, K, half, mode == 3, sm_count, status, stream);
  } else if (mode == 2 || mode == 3) {
    if (c_dtype == LLM_BF16) return launch<4, EPI_GATED, bf16>(mw, mx, mc, T, N, K, half, mode == 3, sm_count, status, stream);
    if (c_dtype == LLM_F32) return launch<4, EPI_GATED, float>(mw, mx, mc, T, N, K, half, mode == 3, sm_count, status, stream);
  }
  return LLM_ERR_UNSUPPORTED;
}
