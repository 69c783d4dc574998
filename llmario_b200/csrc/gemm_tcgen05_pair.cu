// The persistent tcgen05 matrix product on CTA pairs (tcgen05 cta_group::2) for many rows:
//     C[t][n] (=|+=) sum_k X[t][k] * W[n][k],   tiles of 256 weight rows x 256 tokens per pair.
// Two CTAs on neighbouring SMs (a cluster of two) share one tile.  Each loads HALF of both
// operands into its own shared memory (its 128 weight rows, its 128 tokens: 32 KB per stage instead
// of the 48 KB a lone CTA needs for half the tile), the leader CTA issues one
// tcgen05.mma.cta_group::2 of 256 x 256 x 16 that reads both halves from both CTAs, and each CTA
// ends up with the accumulator of its own 128 weight rows x 256 tokens in its own tensor memory.
// A third less shared-memory fill per flop is what the lone-CTA kernel lacked: its tensor pipe
// waited for operands.
//
//   warp 0     TMA producer of this CTA's halves, running ahead across tiles through a ring of stages
//              (both CTAs' loads count their bytes on the LEADER's barrier of the stage)
//   warp 1     leader CTA only: waits until a stage is full in both CTAs, issues the MMAs, and commits
//              them to the stage's "empty" barrier in both CTAs (tcgen05.commit ... multicast::cluster)
//   warps 2-5  epilogue of one of two accumulators (2 x 256 TMEM columns) while the next tile is
//              multiplied: TMEM -> registers -> shared memory in chunks of 32 tokens -> TMA store or
//              TMA add-reduction; the leader learns from both CTAs when an accumulator is drained
//
// Epilogues: store, residual add, gated silu(g) * u with gate and up rows interleaved in blocks of
// 16.  The output must be reachable by TMA.  Every wait is bounded: a CTA that gives up sets
// *status and walks to the final cluster barrier, where its peer (whose own waits run out in
// turn) meets it before tensor memory is freed.  No load is multicast.
#include "tcgen05.cuh"

extern int g_llm_pair_ksplits;

namespace {

constexpr int BN = 256;          // tokens per pair tile
constexpr int HALF_N = 128;      // tokens this CTA loads
constexpr int CH = 32;           // tokens per epilogue chunk

template <int STAGES, int FEAT, typename TC>
struct alignas(1024) PairStorage {
  uint8_t a[STAGES][TILE_M * TILE_K * 2];      // this CTA's 128 weight rows
  uint8_t b[STAGES][HALF_N * TILE_K * 2];      // this CTA's 128 tokens
  alignas(128) TC out[2][CH * FEAT];
  uint64_t full[STAGES];        // leader's: the bytes of both CTAs' halves are counted here
  uint64_t empty[STAGES];       // both: the MMAs that read this stage are done
  uint64_t acc_full[2];         // both: the tile's MMAs are done
  uint64_t acc_empty[2];        // leader: both CTAs have drained the accumulator
  uint32_t tmem_base;
  int dead;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void pair_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_local(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// arrive on the barrier at the same shared-memory offset in CTA `cta` of the pair
__device__ __forceinline__ void mbar_arrive_in(uint64_t* bar, uint32_t cta) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(bar)), "r"(cta));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
// bounded wait on a barrier that the other CTA (or an MMA commit from it) arrives on
__device__ __forceinline__ bool mbar_wait_pair(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  long long start = 0;
  for (uint32_t i = 0;; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (i == 0) start = clock64();
    else if (clock64() - start > WAIT_CYCLES) return false;
  }
}
// the shared::cluster address of `p` as CTA `cta` of the pair holds it
__device__ __forceinline__ uint32_t in_cta(const void* p, uint32_t cta) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(p)), "r"(cta));
  return remote;
}
// TMA tile load into this CTA's shared memory whose bytes are counted on a barrier that may be the
// other CTA's (`bar_cluster`: a shared::cluster address)
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster)
      : "memory");
}
__device__ __forceinline__ void pair_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// when the MMAs issued so far are done, arrive on the barrier at this offset in both CTAs
__device__ __forceinline__ void pair_commit(uint64_t* bar) {
  const uint16_t both = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(both)
      : "memory");
}

template <int STAGES, int EPI, typename TC>
__global__ void __launch_bounds__(192, 1) gemm_pair_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
    const __grid_constant__ CUtensorMap map_c, int T, int N, int K, int half, int m_tiles, int n_tiles,
    int ksplits, int* __restrict__ status) {
  constexpr int FEAT = EPI == EPI_GATED ? 64 : TILE_M;     // output features of this CTA per tile
  extern __shared__ uint8_t raw[];
  auto& sm = *reinterpret_cast<PairStorage<STAGES, FEAT, TC>*>(
      (reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int nkb = (K + TILE_K - 1) / TILE_K;
  const int tiles = m_tiles * n_tiles;
  // A work item is a tile and one of `ksplits` ranges of K (more than one only with the adding
  // epilogue, whose partial sums meet in memory): item w is tile w % tiles, range w / tiles.
  const int works = tiles * ksplits;
  constexpr uint32_t STAGE_BYTES = TILE_M * TILE_K * 2 + HALF_N * TILE_K * 2;
  // float32 accumulator, bf16 A and B, both K-major, N = 256, M = 256 over the pair
  constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)((2 * TILE_M) >> 4) << 24);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.full[s], 1);          // the leader's producer, expecting the bytes of both CTAs
      mbar_init(&sm.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.acc_full[b], 1);
      mbar_init(&sm.acc_empty[b], 8);     // four epilogue warps in each CTA
    }
    sm.dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  pair_sync();               // both CTAs' barriers exist before either signals the other
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------------ producer (both CTAs)
    // Both CTAs' loads count their bytes on the LEADER's barrier of the stage; only the leader's
    // producer arrives there, expecting the bytes of both (the other CTA's bytes may be counted
    // before that arrival: the count is signed).
    uint32_t full_addr[STAGES];
    for (int s = 0; s < STAGES; ++s) full_addr[s] = in_cta(&sm.full[s], 0);
    auto load_w = [&](int s, int row0, int k) {
      if (leader) mbar_expect_tx(&sm.full[s], 2 * STAGE_BYTES);
      tma_load_2d_pair(sm.a[s], &map_w, k, row0, full_addr[s]);
    };
    long long it = 0;
    bool ok = true;
    bool first = true;
    for (int work = pair; work < works && ok; work += n_pairs) {
      const int tile = work % tiles, ks = work / tiles;
      const int kb0 = (int)((long long)ks * nkb / ksplits), kb1 = (int)((long long)(ks + 1) * nkb / ksplits);
      const int f0 = (tile / n_tiles) * (2 * FEAT) + (int)rank * FEAT;      // first output feature
      const int row0 = EPI == EPI_GATED ? 2 * f0 : f0;                      // first weight row
      const int t0 = (tile % n_tiles) * BN + (int)rank * HALF_N;
      int kb = kb0;
      if (first) {
        // weights do not depend on earlier kernels: fetch a ring of them before waiting
        const int head = min(kb1 - kb0, STAGES);
        for (int i = 0; i < head; ++i) load_w(i, row0, (kb0 + i) * TILE_K);
        pdl_wait();
        for (int i = 0; i < head; ++i) tma_load_2d_pair(sm.b[i], &map_x, (kb0 + i) * TILE_K, t0, full_addr[i]);
        it = head;
        kb = kb0 + head;
        first = false;
      }
      for (; kb < kb1; ++kb, ++it) {
        const int s = (int)(it % STAGES);
        ok = mbar_wait_pair(&sm.empty[s], (uint32_t)((it / STAGES) & 1) ^ 1);
        if (!ok) { atomicExch(status, 1); sm.dead = 1; break; }
        load_w(s, row0, kb * TILE_K);
        tma_load_2d_pair(sm.b[s], &map_x, kb * TILE_K, t0, full_addr[s]);
      }
    }
    // A producer gives up only after a wait of about two seconds, far longer than any load it
    // still has in flight needs to land; the final barrier of the pair comes after that.
  } else if (warp == 1 && lane == 0 && leader) {
    // ------------------------------------------------------------------ leader: MMA issuer
    long long it = 0;
    int local = 0;
    bool ok = true;
    for (int work = pair; work < works && ok; work += n_pairs, ++local) {
      const int ks = work / tiles;
      const int kb0 = (int)((long long)ks * nkb / ksplits), kb1 = (int)((long long)(ks + 1) * nkb / ksplits);
      const int buf = local & 1;
      ok = mbar_wait_pair(&sm.acc_empty[buf], (uint32_t)((local >> 1) & 1) ^ 1);
      if (!ok) { atomicExch(status, 2); sm.dead = 1; break; }
      tc_fence_after();
      const uint32_t acc = tmem + (uint32_t)buf * BN;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = (int)(it % STAGES);
        ok = mbar_wait_pair(&sm.full[s], (uint32_t)((it / STAGES) & 1));
        if (!ok) { atomicExch(status, 2); sm.dead = 1; break; }
        tc_fence_after();
        const uint64_t da = smem_desc(smem_u32(sm.a[s]));
        const uint64_t db = smem_desc(smem_u32(sm.b[s]));
#pragma unroll
        for (int k = 0; k < TILE_K / UMMA_K; ++k)
          pair_mma(acc, da + (uint64_t)(k * UMMA_K * 2 >> 4), db + (uint64_t)(k * UMMA_K * 2 >> 4), idesc,
                   (kb > kb0 || k > 0) ? 1u : 0u);
        pair_commit(&sm.empty[s]);
      }
      if (ok) pair_commit(&sm.acc_full[buf]);
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const bool issuer = warp == 2 && lane == 0;
    pdl_wait();
    int local = 0;
    int chunk_no = 0;
    for (int work = pair; work < works; work += n_pairs, ++local) {
      const int tile = work % tiles;
      const int n0 = (tile / n_tiles) * (2 * FEAT) + (int)rank * FEAT, t0 = (tile % n_tiles) * BN;
      const int buf = local & 1;
      bool ok = mbar_wait_pair(&sm.acc_full[buf], (uint32_t)((local >> 1) & 1));
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
          if (lane == 0) {
            if (leader) mbar_arrive_local(&sm.acc_empty[buf]);
            else mbar_arrive_in(&sm.acc_empty[buf], 0);
          }
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
  // Neither CTA may go while the other can still read its shared memory, signal its barriers or
  // write its tensor memory.
  tc_fence_before();
  __syncwarp();
  pair_sync();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

template <int STAGES, int EPI, typename TC>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mc, int T, int N, int K, int half,
           int sm_count, int* status, cudaStream_t stream) {
  constexpr int FEAT = EPI == EPI_GATED ? 64 : TILE_M;
  auto kernel = gemm_pair_kernel<STAGES, EPI, TC>;
  constexpr int smem = (int)sizeof(PairStorage<STAGES, FEAT, TC>) + 1024;
  static_assert(smem <= 227 * 1024, "the stages and output chunks fit one SM");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int limit = EPI == EPI_GATED ? half : N;
  const int m_tiles = (limit + 2 * FEAT - 1) / (2 * FEAT), n_tiles = (T + BN - 1) / BN;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // as many pairs as the device holds at once (an SM without a free neighbour stays empty)
  static int resident_pairs = 0;
  if (!resident_pairs) {
    cfg.gridDim = dim3(sm_count & ~1);
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      return LLM_ERR_UNSUPPORTED;
    }
    resident_pairs = n < sm_count / 2 ? n : sm_count / 2;
  }
  // The adding epilogue lets K be cut.  With few tiles to a pair the last round of tiles leaves
  // most pairs idle (160 tiles on 74 pairs: three rounds for the work of 2.2), and with fewer
  // tiles than pairs some never work.  A work item costs its 64-wide blocks of K plus about six
  // blocks' worth of start and epilogue (fitted to measured times of seven shapes); K is cut into
  // the number of ranges, each of at least eight blocks, for which the rounds cost least.
  int ksplits = 1;
  if (EPI == EPI_ACCUM) {
    const int tiles = m_tiles * n_tiles, nkb = (K + TILE_K - 1) / TILE_K;
    double best = 0;
    for (int s = 1; s <= 8 && nkb / s >= 8; ++s) {
      const int rounds = (tiles * s + resident_pairs - 1) / resident_pairs;
      const double cost = rounds * ((double)nkb / s + 6.0);
      if (s == 1 || cost < best * 0.99) best = cost, ksplits = s;
    }
    if (g_llm_pair_ksplits > 0 && nkb / g_llm_pair_ksplits >= 1) ksplits = g_llm_pair_ksplits;
  }
  const int works = m_tiles * n_tiles * ksplits;
  const int pairs = works < resident_pairs ? works : resident_pairs;
  cfg.gridDim = dim3(2 * pairs);
  // directly behind the rotation kernel the pair kernel starts only when that kernel is done
  cfg.numAttrs = (g_llm_pdl && !g_llm_after_rotation) ? 2 : 1;
  g_llm_after_rotation = 0;
  return (int)cudaLaunchKernelEx(&cfg, kernel, mw, mx, mc, T, N, K, half, m_tiles, n_tiles, ksplits, status);
}
}  // namespace

// The pair kernel for bfloat16 X [T][K], W [N][K]; modes 0, 1 and 3 of llm_gemm_tcgen05 (no K
// split; the gated form only with interleaved rows).  Returns LLM_ERR_UNSUPPORTED when the output
// cannot be written by TMA or the mode is not one of these: the caller then uses the one-CTA kernel.
int g_llm_pair = 1;   // 0: the dispatcher keeps to the one-CTA kernels (for comparisons)
int g_llm_pair_ksplits = 0;   // > 0: this many ranges of K in the adding epilogue (for measurements)
LLM_EXPORT void llm_set_pair_ksplits(int n) { g_llm_pair_ksplits = n; }
LLM_EXPORT void llm_set_pair(int on) { g_llm_pair = on ? 1 : 0; }

int llm_gemm_tcgen05_pair(const void* X, const void* W, void* C, int c_dtype, int T, int N, int K, int lda,
                          int ldw, int ldc, int mode, int half, int* status, cudaStream_t stream) {
  if (!g_llm_pair) return LLM_ERR_UNSUPPORTED;
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  if (mode != 0 && mode != 1 && mode != 3) return LLM_ERR_UNSUPPORTED;
  const int esize = c_dtype == LLM_F32 ? 4 : 2;
  if (((uintptr_t)C & 15) || ((size_t)ldc * esize) % 16) return LLM_ERR_UNSUPPORTED;
  CUtensorMap mw, mx, mc;
  if (!llm_tensor_map(W, N, K, ldw, TILE_M, TILE_K, 0, &mw)) return LLM_ERR_UNSUPPORTED;
  if (!llm_tensor_map(X, T, K, lda, HALF_N, TILE_K, 0, &mx)) return LLM_ERR_UNSUPPORTED;
  const int out_cols = mode == 3 ? half : N;
  if (!llm_tensor_map(C, T, out_cols, ldc, CH, mode == 3 ? 64 : TILE_M, c_dtype == LLM_F32 ? 2 : 1, &mc))
    return LLM_ERR_UNSUPPORTED;
  if (mode == 0) {
    if (c_dtype == LLM_F32) return launch<5, EPI_STORE, float>(mw, mx, mc, T, N, K, half, sm_count, status, stream);
    if (c_dtype == LLM_BF16) return launch<6, EPI_STORE, bf16>(mw, mx, mc, T, N, K, half, sm_count, status, stream);
  } else if (mode == 1) {
    if (c_dtype == LLM_F32) return launch<5, EPI_ACCUM, float>(mw, mx, mc, T, N, K, half, sm_count, status, stream);
  } else {
    if (N != 2 * half || half % 16) return LLM_ERR_ARGUMENT;
    if (c_dtype == LLM_BF16) return launch<6, EPI_GATED, bf16>(mw, mx, mc, T, N, K, half, sm_count, status, stream);
    if (c_dtype == LLM_F32) return launch<6, EPI_GATED, float>(mw, mx, mc, T, N, K, half, sm_count, status, stream);
  }
  return LLM_ERR_UNSUPPORTED;
}
