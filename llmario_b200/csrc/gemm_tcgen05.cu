// Matrix product on the 5th-generation tensor cores (tcgen05) for bfloat16 operands:
//     C[t][n] (=|+=) sum_k X[t][k] * W[n][k]          X: [T][K] activations, W: [N][K] weights
// computed transposed, D = W X^T: a CTA owns 128 weight rows (the UMMA "M" side, one TMEM lane per
// output feature) and a tile of BN tokens (the UMMA "N" side, one TMEM column per token).  Because
// the weights sit on the 128-wide side, the same kernel serves a prompt portion of thousands of
// tokens and a decode step of a few: BN goes from 16 to 256 and the weight tile is streamed once.
//
//   warp 0   producer: TMA loads of the W tile (128 x 64) and the X tile (BN x 64), both K-major
//            with the 128-byte swizzle, into a ring of STAGES shared-memory stages (mbarriers)
//   warp 1   allocates TMEM; one lane issues tcgen05.mma (128 x BN x 16 per instruction, four per
//            stage) and frees stages with tcgen05.commit
//   warps 2-5  epilogue: tcgen05.ld of the 32 TMEM lanes of their quarter, then coalesced stores
//
// Epilogues: store bfloat16 / float32, add into a float32 residual stream, or the gated
// activation silu(g) * u with 64 gate rows and their 64 up rows interleaved in one 128-row tile.
// The finished tile is laid out in shared memory and leaves through one TMA store, or one TMA
// add-reduction for the residual add and for the partial sums of a split K range (gridDim.z > 1);
// an output whose rows are not 16-byte multiples is written with plain stores and atomics.
//
// Every wait on an mbarrier is bounded; when a bound runs out the kernel records where in
// *status, drains the loads it still has in flight, frees its TMEM and returns.
#include <cuda.h>

#include <cstring>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

#include "tcgen05.cuh"

int llm_zero_f32(float* p, int rows, int cols, int ld, cudaStream_t stream);   // elementwise.cu
int llm_gemm_tcgen05_pair(const void* X, const void* W, void* C, int c_dtype, int T, int N, int K, int lda,
                          int ldw, int ldc, int mode, int half, int* status, cudaStream_t stream);
int llm_gemm_tcgen05_persistent(const void* X, const void* W, void* C, int c_dtype, int T, int N, int K,
                                int lda, int ldw, int ldc, int mode, int half, int* status,
                                cudaStream_t stream);                        // gemm_tcgen05_persistent.cu

namespace {


template <int BN, int STAGES>
struct alignas(1024) SharedStorage {
  uint8_t a[STAGES][TILE_M * TILE_K * 2];
  uint8_t b[STAGES][BN * TILE_K * 2 < 1024 ? 1024 : BN * TILE_K * 2];
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full;
  uint32_t tmem_base;
};

// grid: (feature tiles, token tiles, K splits).  Features per tile: 128, or 64 when gated.
template <int BN, int STAGES, int EPI, typename TC>
__global__ void __launch_bounds__(192) gemm_tcgen05_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
    const __grid_constant__ CUtensorMap map_c, int tma_out, TC* __restrict__ C, int ldc, int T, int N,
    int K, int half, int interleaved, int* __restrict__ status) {
  extern __shared__ uint8_t raw[];
  auto& sm = *reinterpret_cast<SharedStorage<BN, STAGES>*>(
      (reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int feat_per_tile = EPI == EPI_GATED ? 64 : TILE_M;
  const int n0 = blockIdx.x * feat_per_tile;
  const int t0 = blockIdx.y * BN;
  const int kblocks = (K + TILE_K - 1) / TILE_K;
  const int per_split = (kblocks + gridDim.z - 1) / gridDim.z;
  const int kb_begin = blockIdx.z * per_split;
  const int kb_end = min(kblocks, kb_begin + per_split);
  const int nkb = kb_end - kb_begin;
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  constexpr uint32_t STAGE_BYTES = TILE_M * TILE_K * 2 + BN * TILE_K * 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    mbar_init(&sm.acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  if (nkb > 0) {
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------------- producer
      // The weights do not depend on any earlier kernel: the first ring of weight tiles is
      // requested at once, the activation tiles only after the earlier kernels are done.
      auto load_w = [&](int i) {
        const int s = i % STAGES;
        mbar_expect_tx(&sm.full[s], STAGE_BYTES);
        const int k = (kb_begin + i) * TILE_K;
        if (EPI == EPI_GATED && interleaved) {
          // the matrix is stored with 16 gate rows, their 16 up rows, the next 16 gate rows, ...
          tma_load_2d(sm.a[s], &map_w, k, 2 * n0, &sm.full[s]);
        } else if (EPI == EPI_GATED) {
          // 16 gate rows, their 16 up rows, the next 16 gate rows, ...: every 32-lane quarter of
          // the accumulator then holds gate and up of the same 16 features
#pragma unroll
          for (int b = 0; b < 8; ++b)
            tma_load_2d(sm.a[s] + b * 16 * TILE_K * 2, &map_w, k, ((b & 1) ? half : 0) + n0 + (b >> 1) * 16,
                        &sm.full[s]);
        } else {
          tma_load_2d(sm.a[s], &map_w, k, n0, &sm.full[s]);
        }
      };
      auto load_x = [&](int i) {
        const int s = i % STAGES;
        tma_load_2d(sm.b[s], &map_x, (kb_begin + i) * TILE_K, t0, &sm.full[s]);
      };
      const int head = min(nkb, STAGES);
      for (int i = 0; i < head; ++i) load_w(i);
      pdl_wait();
      for (int i = 0; i < head; ++i) load_x(i);
      int issued = head;
      bool ok = true;
      for (int i = head; i < nkb; ++i) {
        const int s = i % STAGES;
        ok = mbar_wait(&sm.empty[s], ((i / STAGES) & 1) ^ 1);
        if (!ok) { atomicExch(status, 1); break; }
        load_w(i);
        load_x(i);
        issued = i + 1;
      }
      if (!ok) {
        // drain: the loads already issued must land before this CTA's shared memory is given up
        for (int i = max(0, issued - STAGES); i < issued; ++i)
          mbar_wait(&sm.full[i % STAGES], (i / STAGES) & 1);
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc = instr_desc<BN>();
      bool ok = true;
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES;
        ok = mbar_wait(&sm.full[s], (i / STAGES) & 1);
        if (!ok) { atomicExch(status, 2); break; }
        tc_fence_after();
        const uint64_t da = smem_desc(smem_u32(sm.a[s]));
        const uint64_t db = smem_desc(smem_u32(sm.b[s]));
#pragma unroll
        for (int k = 0; k < TILE_K / UMMA_K; ++k)
          tc_mma(tmem, da + (uint64_t)(k * UMMA_K * 2 >> 4), db + (uint64_t)(k * UMMA_K * 2 >> 4), idesc,
                 (i > 0 || k > 0) ? 1u : 0u);
        tc_commit(&sm.empty[s]);   // frees the stage when these MMAs have read it
      }
      tc_commit(&sm.acc_full);     // arrives when every MMA above has completed
    } else if (warp >= 2) {
      // ---------------------------------------------------------------- epilogue
      const int q = warp & 3;                 // TMEM lane quarter this warp may read
      const int row = q * 32 + lane;          // row of the 128-row tile
      pdl_wait();   // the output may still be read or written by earlier kernels
      const bool ok = mbar_wait(&sm.acc_full, 0);
      if (!ok && lane == 0) atomicExch(status, 3);
      tc_fence_after();
      if (ok) {
        const bool split = gridDim.z > 1;
        // With a tensor map for the output the tile is laid out in shared memory as
        // [token][feature] (the pipeline stages are free by now) and written by one TMA store,
        // or added by one TMA reduction (residual add, partial sums of a K split).
        constexpr int FEAT = EPI == EPI_GATED ? 64 : TILE_M;
        TC* stage_out = reinterpret_cast<TC*>(&sm.a[0][0]);
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          uint32_t v[16];
          tmem_ld16(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)c, v);
          tmem_ld_wait();
          if (EPI == EPI_GATED) {
            // lanes 0..15 hold gate of feature q*16 + lane, lanes 16..31 the matching up values
            // (both halves of the warp compute: eight columns each, see gated_columns)
            const int f = q * 16 + (lane & 15);
            const int n = n0 + f;
            const int col0 = c + (lane < 16 ? 0 : 8);
            float r[8];
            gated_columns<TC>(v, lane, r);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int t = t0 + col0 + i;
              const TC a = from_f32<TC>(r[i]);
              if (tma_out) stage_out[(col0 + i) * FEAT + f] = a;
              else if (t < T && n < half) C[(size_t)t * ldc + n] = a;
            }
          } else {
            const int n = n0 + row;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = t0 + c + j;
              const float a = __uint_as_float(v[j]);
              if (tma_out) {
                stage_out[(c + j) * FEAT + row] = from_f32<TC>(a);
              } else if (t < T && n < N) {
                TC* dst = C + (size_t)t * ldc + n;
                if (EPI == EPI_ACCUM || split) {
                  if (split) atomicAdd(reinterpret_cast<float*>(dst), a);
                  else *dst = from_f32<TC>(to_f32(*dst) + a);
                } else {
                  *dst = from_f32<TC>(a);
                }
              }
            }
          }
        }
        if (tma_out) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (warp == 2 && lane == 0) {
            const uint32_t src = smem_u32(stage_out);
            if (EPI == EPI_ACCUM || split)
              asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(&map_c), "r"(src), "r"(n0), "r"(t0) : "memory");
            else
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(&map_c), "r"(src), "r"(n0), "r"(t0) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// host side: tensor maps (made once per matrix and cached) and launch
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encoder() {
  static EncodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(p);
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  long long rows, cols, ld;
  int box_rows, box_cols, kind;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows &&
           box_cols == o.box_cols && kind == o.kind;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    h ^= std::hash<long long>()(k.rows * 1315423911LL + k.cols * 2654435761LL + k.ld * 97 + k.box_rows * 31 +
                                k.box_cols * 7 + k.kind) +
         0x9e3779b97f4a7c15ULL + (h << 6) + (h >> 2);
    return h;
  }
};

// A [rows][cols] matrix with row stride ld (elements), tiled in boxes of box_rows x box_cols.
// kind 0: bf16 operand, 128-byte swizzle; kind 1: bf16 output, no swizzle; kind 2: f32 output.
}  // namespace

bool llm_tensor_map(const void* ptr, long long rows, long long cols, long long ld, int box_rows, int box_cols,
                    int kind, CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{ptr, rows, cols, ld, box_rows, box_cols, kind};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  EncodeTiled enc = encoder();
  if (!enc) return false;
  const int esize = kind == 2 ? 4 : 2;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * esize};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUtensorMap m;
  CUresult r = enc(&m, kind == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                   const_cast<void*>(ptr), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   kind == 0 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}

// A bfloat16 tensor of `rank` dimensions (innermost first: extents `dims`, strides in bytes of
// dimensions 1 .. rank-1 in `strides`), tiled in boxes of `box` elements with the 128-byte
// swizzle.  Cached like the matrices above.
bool llm_tensor_map_tiled(const void* ptr, int rank, const long long* dims, const long long* strides,
                          const int* box, CUtensorMap* out) {
  struct Key {
    const void* ptr;
    int rank;
    long long dims[5], strides[4];
    int box[5];
    bool operator==(const Key& o) const { return memcmp(this, &o, sizeof(Key)) == 0; }
  };
  struct KeyHash {
    size_t operator()(const Key& k) const {
      size_t h = 1469598103934665603ULL;
      const unsigned char* b = reinterpret_cast<const unsigned char*>(&k);
      for (size_t i = 0; i < sizeof(Key); ++i) h = (h ^ b[i]) * 1099511628211ULL;
      return h;
    }
  };
  static std::unordered_map<Key, CUtensorMap, KeyHash> cache;
  static std::mutex mu;
  if (rank < 2 || rank > 5) return false;
  Key key;
  memset(&key, 0, sizeof(key));
  key.ptr = ptr;
  key.rank = rank;
  for (int i = 0; i < rank; ++i) key.dims[i] = dims[i], key.box[i] = box[i];
  for (int i = 0; i + 1 < rank; ++i) key.strides[i] = strides[i];
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  EncodeTiled enc = encoder();
  if (!enc) return false;
  cuuint64_t gd[5], gs[4];
  cuuint32_t bx[5], el[5];
  for (int i = 0; i < rank; ++i) gd[i] = (cuuint64_t)dims[i], bx[i] = (cuuint32_t)box[i], el[i] = 1;
  for (int i = 0; i + 1 < rank; ++i) gs[i] = (cuuint64_t)strides[i];
  CUtensorMap m;
  CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), gd, gs, bx, el,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}

namespace {

template <int BN, int STAGES, int EPI, typename TC>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, TC* C, int ldc, int T, int N, int K, int half,
           int splits, int interleaved, int* status, cudaStream_t stream) {
  // the output goes through TMA when its rows are 16-byte multiples on a 16-byte aligned base
  CUtensorMap mc = mw;
  int tma_out = 0;
  const int out_cols = EPI == EPI_GATED ? half : N;
  if (((uintptr_t)C & 15) == 0 && ((size_t)ldc * sizeof(TC)) % 16 == 0 &&
      llm_tensor_map(C, T, out_cols, ldc, BN, EPI == EPI_GATED ? 64 : TILE_M, sizeof(TC) == 4 ? 2 : 1, &mc))
    tma_out = 1;
  auto kernel = gemm_tcgen05_kernel<BN, STAGES, EPI, TC>;
  constexpr int smem = (int)sizeof(SharedStorage<BN, STAGES>) + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int feat = EPI == EPI_GATED ? 64 : TILE_M;
  const int limit = EPI == EPI_GATED ? half : N;
  dim3 grid((limit + feat - 1) / feat, (T + BN - 1) / BN, splits);
  return launch_pdl(kernel, grid, 192, smem, stream, mw, mx, mc, tma_out, C, ldc, T, N, K, half, interleaved,
                    status);
}

template <int EPI, typename TC>
int dispatch(int bn, const CUtensorMap& mw, const CUtensorMap& mx, TC* C, int ldc, int T, int N, int K,
             int half, int splits, int interleaved, int* status, cudaStream_t stream) {
  switch (bn) {
    case 16: return launch<16, 6, EPI, TC>(mw, mx, C, ldc, T, N, K, half, splits, interleaved, status, stream);
    case 32: return launch<32, 5, EPI, TC>(mw, mx, C, ldc, T, N, K, half, splits, interleaved, status, stream);
    case 64: return launch<64, 4, EPI, TC>(mw, mx, C, ldc, T, N, K, half, splits, interleaved, status, stream);
    case 128: return launch<128, 3, EPI, TC>(mw, mx, C, ldc, T, N, K, half, splits, interleaved, status, stream);
  }
  return LLM_ERR_UNSUPPORTED;
}
}  // namespace

// X [T][K] and W [N][K] bfloat16 with 16-byte aligned rows (K, lda, ldw multiples of 8).
//   mode 0: C = X W^T (c_dtype bf16 or f32; with splits > 1: f32, zeroed here first)
//   mode 1: C += X W^T (f32)
//   mode 2: W = [gate; up] with `half` rows each, C[t][n] = silu(gate) * up, n < half
//   mode 3: the same with W stored interleaved: 16 gate rows, their 16 up rows, 16 gate rows, ...
// bn: token tile, one of 16, 32, 64, 128, or 256 for the persistent kernel.  out_is_zero: with
// mode 0 and splits > 1 the caller guarantees that C holds zeros (it is not cleared here).  status: device int, set non-zero when a wait
// inside the kernel gave up.
LLM_EXPORT int llm_gemm_tcgen05(const void* X, const void* W, void* C, int c_dtype, int T, int N, int K,
                                int lda, int ldw, int ldc, int mode, int half, int bn, int splits,
                                int out_is_zero, int* status, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || lda % 8 || ldw % 8) return LLM_ERR_UNSUPPORTED;
  if (((uintptr_t)X | (uintptr_t)W) & 15) return LLM_ERR_UNSUPPORTED;
  if (splits < 1) return LLM_ERR_ARGUMENT;
  if (bn == 256) {
    // many rows: the persistent kernels (tiles of 256 tokens, epilogue overlapped with the next
    // tile), on CTA pairs where that form exists; if the output cannot be written by TMA, the
    // one-tile kernel with 128 tokens
    // (the pair kernel cuts K itself where its adding epilogue allows, so it also takes the
    // products for which the caller asked for a split)
    if (splits == 1 || mode == 1) {
      int r = llm_gemm_tcgen05_pair(X, W, C, c_dtype, T, N, K, lda, ldw, ldc, mode, half, status, stream);
      if (r != LLM_ERR_UNSUPPORTED) return r;
    }
    if (splits == 1) {
      int r = llm_gemm_tcgen05_persistent(X, W, C, c_dtype, T, N, K, lda, ldw, ldc, mode, half, status, stream);
      if (r != LLM_ERR_UNSUPPORTED) return r;
    }
    bn = 128;
  }
  const int kblocks = (K + TILE_K - 1) / TILE_K;
  if (splits > kblocks) splits = kblocks;
  // no split may be empty
  while (splits > 1 && (splits - 1) * ((kblocks + splits - 1) / splits) >= kblocks) --splits;
  CUtensorMap mw, mx;
  if (!llm_tensor_map(W, N, K, ldw, mode == 2 ? 16 : TILE_M, TILE_K, 0, &mw)) return LLM_ERR_UNSUPPORTED;
  if (!llm_tensor_map(X, T, K, lda, bn, TILE_K, 0, &mx)) return LLM_ERR_UNSUPPORTED;
  if (mode == 0) {
    if (c_dtype == LLM_F32 && splits > 1 && !(out_is_zero)) {   // partial sums are added into zeros
      const int z = llm_zero_f32((float*)C, T, N, ldc, stream);
      if (z != 0) return z;
    }
    if (c_dtype == LLM_F32)
      return dispatch<EPI_STORE, float>(bn, mw, mx, (float*)C, ldc, T, N, K, half, splits, 0, status, stream);
    if (c_dtype == LLM_BF16 && splits == 1)
      return dispatch<EPI_STORE, bf16>(bn, mw, mx, (bf16*)C, ldc, T, N, K, half, 1, mode == 3, status, stream);
    return LLM_ERR_UNSUPPORTED;
  }
  if (mode == 1) {
    if (c_dtype != LLM_F32) return LLM_ERR_UNSUPPORTED;
    return dispatch<EPI_ACCUM, float>(bn, mw, mx, (float*)C, ldc, T, N, K, half, splits, 0, status, stream);
  }
  if (mode == 2 || mode == 3) {
    if (N != 2 * half || (mode == 3 && half % 16)) return LLM_ERR_ARGUMENT;
    if (c_dtype == LLM_BF16)
      return dispatch<EPI_GATED, bf16>(bn, mw, mx, (bf16*)C, ldc, T, N, K, half, 1, mode == 3, status, stream);
    if (c_dtype == LLM_F32)
      return dispatch<EPI_GATED, float>(bn, mw, mx, (float*)C, ldc, T, N, K, half, 1, mode == 3, status, stream);
    return LLM_ERR_UNSUPPORTED;
  }
  return LLM_ERR_ARGUMENT;
}
