// Paged causal attention for prompt portions on tcgen05 with TWO query tiles per CTA (bfloat16).
//
// The one-tile kernel (attention_tcgen05.cu) is bound by its softmax: one thread per row works
// through a key tile in about 2,300 cycles while the tensor core needs about 1,000 for the two
// products of that tile.  Here a CTA takes an item of up to 2 x 128 / G consecutive tokens of one
// request and one KV head, as two query tiles A and B of 128 rows ((token, head of the group)
// pairs) with a softmax warpgroup each.  Every K and V tile is loaded once and used by both; while
// one warpgroup is busy with the scores of its tile, the tensor core works for the other:
//
//   warp 0     TMA: both Q tiles once, then K tiles and V tiles through two rings of two stages
//              (boxes of 64 columns x up to 128 positions: pages of 32 positions or more)
//   warp 1     one lane issues, tile after tile:  O_A += P_A V(j-1);  S_A = Q_A K(j)^T;
//              O_B += P_B V(j-1);  S_B = Q_B K(j)^T   (P is read from tensor memory, V is an
//              N-major operand); a stream's scores, its P and its next scores follow one another in
//              the same TMEM columns, so the order of issue is all the ordering they need
//   warps 2-5  softmax of tile A, warps 6-9 of tile B, one thread per row as in the one-tile kernel:
//              the row's 128 scores in registers, maximum, exponentials and sum in 32-bit, P back as
//              bfloat16 over the scores, the output rescaled only when the row's maximum has grown by
//              more than 2^8; at the end O / l is written
//
// TMEM (all 512 columns): scores A, scores B, output A, output B, 128 columns each.  Every
// mbarrier wait is bounded.  Head sizes 64 and 128; G must divide 128.
#include "attention_tc_common.cuh"

namespace {

constexpr int ROWS = 128;          // rows of a query tile (TMEM lanes)
constexpr int KT = 128;            // keys per tile
constexpr int STAGES = 2;

template <int HD>
struct alignas(1024) Attn2Storage {
  uint8_t q[2][ROWS * HD * 2];                 // per query tile: [HD/64 halves][128 rows][128 bytes]
  uint8_t k[STAGES][KT * HD * 2];              // [HD/64 halves][128 keys][128 bytes]
  uint8_t v[STAGES][KT * HD * 2];
  uint64_t q_full;
  uint64_t k_full[STAGES], k_empty[STAGES];
  uint64_t v_full[STAGES], v_empty[STAGES];
  uint64_t s_full[2];                          // per query tile
  uint64_t p_full[2];
  uint64_t o_done[2];
  uint32_t tmem_base;
  int dead;
};

template <int HD>
__global__ void __launch_bounds__(320, 1) attention_tcgen05_x2_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
    long long rows_per_page, int v_row_off, bf16* __restrict__ out, const int* __restrict__ block_table,
    int table_stride, const int* __restrict__ items, int Hq, int Hkv, int page_size, float scale_log2,
    int window, int* __restrict__ status) {
  constexpr int HALVES = HD / 64;
  constexpr uint32_t S_COLS = KT;
  constexpr uint32_t O_COL = 2 * S_COLS;       // first column of output A; output B follows
  constexpr uint32_t O_COLS = 128;
  constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(KT >> 3) << 17) |
                               ((uint32_t)(ROWS >> 4) << 24);
  constexpr uint32_t IDESC_O = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) |
                               ((uint32_t)(ROWS >> 4) << 24);
  extern __shared__ uint8_t raw[];
  auto& sm = *reinterpret_cast<Attn2Storage<HD>*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the last items of a prompt have the most keys to walk: they are started first
  const Item it = reinterpret_cast<const Item*>(items)[gridDim.x - 1 - blockIdx.x];
  const int kvh = blockIdx.y;
  const int G = Hq / Hkv;
  const int cap = ROWS / G;                                  // tokens of one query tile
  const int tok_a = it.tokens < cap ? it.tokens : cap;       // tokens of tile A
  const int tok_b = it.tokens - tok_a;                       // tokens of tile B (0: there is none)
  const int hi_a = it.pos_start + tok_a - 1, hi_b = it.pos_start + it.tokens - 1;
  const int lo = (window > 0 && it.pos_start + 1 > window) ? it.pos_start + 1 - window : 0;
  const int tile_first = lo / KT;
  const int nt_a = hi_a / KT - tile_first + 1;               // key tiles of A
  const int nt_b = tok_b > 0 ? hi_b / KT - tile_first + 1 : 0;
  const int ntiles = nt_a > nt_b ? nt_a : nt_b;

  if (threadIdx.x == 0) {
    mbar_init(&sm.q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.k_full[s], 1);
      mbar_init(&sm.k_empty[s], 1);
      mbar_init(&sm.v_full[s], 1);
      mbar_init(&sm.v_empty[s], 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(&sm.s_full[x], 1);
      mbar_init(&sm.p_full[x], 4);           // one arrival per softmax warp of the tile
      mbar_init(&sm.o_done[x], 1);
    }
    sm.dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (warp >= 2) {
    // TMA brings whole pages; a page without a key of the item is not fetched and leaves what the
    // stage held.  Such values meet zero weights and must be finite: start from zeros.
    uint4* v4 = reinterpret_cast<uint4*>(sm.v);
    for (int i = threadIdx.x - 64; i < STAGES * KT * HD * 2 / 16; i += 256) v4[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  // only now may the next kernel of the stream be scheduled: every CTA of this one that is
  // running holds its tensor memory, so a successor that also allocates some cannot starve it
  pdl_trigger();

  if (warp == 0) {
    if (lane == 0) {
      // ---------------------------------------------------------------- loads
      pdl_wait();
      mbar_expect_tx(&sm.q_full, (tok_b > 0 ? 2 : 1) * ROWS * HD * 2);
#pragma unroll
      for (int h = 0; h < HALVES; ++h) {
        tma_load_3d(sm.q[0] + h * ROWS * 128, &map_q, h * 64, kvh * G, it.row_start, &sm.q_full);
        if (tok_b > 0)
          tma_load_3d(sm.q[1] + h * ROWS * 128, &map_q, h * 64, kvh * G, it.row_start + cap, &sm.q_full);
      }
      const int R = page_size < KT ? page_size : KT;
      const int* table = block_table + (size_t)it.slot * table_stride;
      bool ok = true;
      // K of tile j, then V of tile j: each through its own ring (a K stage is free again after
      // the scores of both query tiles, a V stage after both second products)
      auto load = [&](uint8_t* dst, uint64_t* full, int j, int row_off) {
        const int base = (tile_first + j) * KT;
        uint32_t bytes = 0;
        for (int p = base; p < base + KT; p += R)
          if (p <= hi_b || p <= hi_a) {
            if (p + R - 1 >= lo) bytes += (uint32_t)R * HD * 2;
          }
        mbar_expect_tx(full, bytes);
        for (int p = base; p < base + KT; p += R) {
          if ((p > hi_b && p > hi_a) || p + R - 1 < lo) continue;   // no key of the item here
          const long long row = (long long)table[p / page_size] * rows_per_page + (long long)kvh * page_size +
                                p % page_size + row_off;
#pragma unroll
          for (int h = 0; h < HALVES; ++h)
            tma_load_2d(dst + h * KT * 128 + (p - base) * 128, &map_kv, h * 64, (int)row, full);
        }
      };
      for (int j = 0; j < ntiles && ok; ++j) {
        const int s = j % STAGES;
        const uint32_t ph = (uint32_t)((j / STAGES) & 1);
        ok = mbar_wait(&sm.k_empty[s], ph ^ 1);
        if (!ok) { atomicExch(status, 5); sm.dead = 1; break; }
        load(sm.k[s], &sm.k_full[s], j, 0);
        ok = mbar_wait(&sm.v_empty[s], ph ^ 1);
        if (!ok) { atomicExch(status, 5); sm.dead = 1; break; }
        load(sm.v[s], &sm.v_full[s], j, v_row_off);
      }
      // (a give-up comes after a wait of about two seconds: nothing is in flight any more)
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      bool ok = mbar_wait(&sm.q_full, 0);
      if (!ok) { atomicExch(status, 6); sm.dead = 1; }
      const int nt[2] = {nt_a, nt_b};
      for (int j = 0; j <= ntiles && ok; ++j) {
        const int s = j % STAGES;
        bool k_ready = false;
        for (int x = 0; x < 2 && ok; ++x) {
          // ---- O_x += P_x V(j-1)
          if (j >= 1 && j - 1 < nt[x]) {
            const int i = j - 1, sv = i % STAGES;
            if (x == 0 || i >= nt[0]) {       // first user of V(i) in this round
              ok = mbar_wait(&sm.v_full[sv], (uint32_t)((i / STAGES) & 1));
              if (!ok) { atomicExch(status, 6); sm.dead = 1; break; }
            }
            ok = mbar_wait(&sm.p_full[x], (uint32_t)(i & 1));
            if (!ok) { atomicExch(status, 6); sm.dead = 1; break; }
            tc_fence_after();
            const uint32_t p_addr = tmem + (uint32_t)x * S_COLS;     // P over the first KT/2 columns
#pragma unroll
            for (int ks = 0; ks < KT / UMMA_K; ++ks)
              tc_mma_ts(tmem + O_COL + (uint32_t)x * O_COLS, p_addr + (uint32_t)ks * (UMMA_K / 2),
                        smem_desc_mn(smem_u32(sm.v[sv]) + (uint32_t)ks * UMMA_K * 128, KT * 128), IDESC_O,
                        (i > 0 || ks > 0) ? 1u : 0u);
            tc_commit(&sm.o_done[x]);
            // the last of the two tiles to use V(i) gives the stage back
            const bool last_user = x == 1 || i >= nt[1];
            if (last_user) tc_commit(&sm.v_empty[sv]);
          }
          // ---- S_x = Q_x K(j)^T
          if (j < nt[x]) {
            if (!k_ready) {
              ok = mbar_wait(&sm.k_full[s], (uint32_t)((j / STAGES) & 1));
              if (!ok) { atomicExch(status, 6); sm.dead = 1; break; }
              tc_fence_after();
              k_ready = true;
            }
            const uint32_t acc = tmem + (uint32_t)x * S_COLS;
#pragma unroll
            for (int ks = 0; ks < HD / UMMA_K; ++ks) {
              const uint32_t off = (uint32_t)(ks / 4) * (ROWS * 128) + (uint32_t)(ks % 4) * 32;
              const uint32_t offk = (uint32_t)(ks / 4) * (KT * 128) + (uint32_t)(ks % 4) * 32;
              tc_mma(acc, smem_desc(smem_u32(sm.q[x]) + off), smem_desc(smem_u32(sm.k[s]) + offk), IDESC_S,
                     ks > 0 ? 1u : 0u);
            }
            tc_commit(&sm.s_full[x]);
            const bool last_user = x == 1 || j >= nt[1];
            if (last_user) tc_commit(&sm.k_empty[s]);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax, one row per thread
    const int x = warp >= 6 ? 1 : 0;                 // which query tile
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    const int tok = row / G, head = kvh * G + row % G;
    const int first_tok = x * cap;                    // first token of this tile inside the item
    const int tokens_x = x ? tok_b : tok_a;
    const int nt_x = x ? nt_b : nt_a;
    const bool rvalid = tok < tokens_x;
    const int rpos = it.pos_start + first_tok + tok;
    const int rlo = (window > 0 && rpos + 1 > window) ? rpos + 1 - window : 0;
    const int pos0 = it.pos_start + first_tok;        // first position of the tile
    const uint32_t s_addr = tmem + lane_base + (uint32_t)x * S_COLS;
    const uint32_t o_addr = tmem + lane_base + O_COL + (uint32_t)x * O_COLS;
    const uint32_t bar_id = 1 + x;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    pdl_wait();
    for (int j = 0; j < nt_x; ++j) {
      ok = mbar_wait(&sm.s_full[x], (uint32_t)(j & 1));
      if (!ok) { if (lane == 0) atomicExch(status, 7); sm.dead = 1; }
      asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
      if (sm.dead) { ok = false; break; }
      tc_fence_after();
      const int base = (tile_first + j) * KT;
      const int c_hi = rvalid ? min(KT - 1, rpos - base) : -1;
      const int c_lo = max(0, rlo - base);
      // a tile that every row of the query tile sees completely needs no per-key tests
      const bool interior = tokens_x * G >= ROWS && base + KT - 1 <= pos0 &&
                            (window <= 0 || base >= pos0 + tokens_x - window);
      uint32_t v[KT];
#pragma unroll
      for (int c = 0; c < KT; c += 32) tmem_ld32(s_addr + c, v + c);
      tmem_ld_wait();
      if (!interior) {
#pragma unroll
        for (int i = 0; i < KT; ++i)
          if (i < c_lo || i > c_hi) v[i] = 0xff800000u;      // -inf: the key is not visible
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < KT; i += 4) {
        mx[0] = fmaxf(mx[0], __uint_as_float(v[i]));
        mx[1] = fmaxf(mx[1], __uint_as_float(v[i + 1]));
        mx[2] = fmaxf(mx[2], __uint_as_float(v[i + 2]));
        mx[3] = fmaxf(mx[3], __uint_as_float(v[i + 3]));
      }
      float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      m_tile *= scale_log2;
      // the scale in use is replaced only when the maximum has grown by more than 2^8
      const bool grow = m_tile > m_used + 8.0f;
      float factor = 1.f;
      if (grow) {
        factor = m_used == -INFINITY ? 0.f : ex2(m_used - m_tile);
        m_used = m_tile;
        l *= factor;
      }
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // rare once the maximum has settled: the rows of this warp in O are rescaled, for which
        // the product P V of the tile before must be complete
        bool done = mbar_wait(&sm.o_done[x], (uint32_t)((j - 1) & 1));
        if (!done) { if (lane == 0) atomicExch(status, 7); sm.dead = 1; }
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
          uint32_t w[32];
          tmem_ld32(o_addr + c, w);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(__uint_as_float(w[i]) * factor);
          tmem_st32(o_addr + c, w);
        }
        tmem_st_wait();
      }
      const float muse = m_used == -INFINITY ? 0.f : m_used;
#pragma unroll
      for (int i = 0; i < KT; ++i)
        v[i] = __float_as_uint(ex2(fmaf(__uint_as_float(v[i]), scale_log2, -muse)));
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < KT; i += 4) {
        sum[0] += __uint_as_float(v[i]);
        sum[1] += __uint_as_float(v[i + 1]);
        sum[2] += __uint_as_float(v[i + 2]);
        sum[3] += __uint_as_float(v[i + 3]);
      }
      l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
#pragma unroll
      for (int c = 0; c < KT; c += 32) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          pk[i >> 1] = pack2(__uint_as_float(v[c + i]), __uint_as_float(v[c + i + 1]));
        tmem_st16(s_addr + (c >> 1), pk);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.p_full[x]);
    }
    if (ok && nt_x > 0) {
      // ---- the last product, then O / l
      bool done = mbar_wait(&sm.o_done[x], (uint32_t)((nt_x - 1) & 1));
      if (!done) { if (lane == 0) atomicExch(status, 7); }
      done = __all_sync(0xffffffffu, done);
      if (done) {
        tc_fence_after();
        const float inv = 1.0f / l;
        bf16* dst = out + ((size_t)(it.row_start + first_tok + tok) * Hq + head) * HD;
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
          uint32_t w[32];
          tmem_ld32(o_addr + c, w);
          tmem_ld_wait();
          if (rvalid) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 u;
              u.x = pack2(__uint_as_float(w[i]) * inv, __uint_as_float(w[i + 1]) * inv);
              u.y = pack2(__uint_as_float(w[i + 2]) * inv, __uint_as_float(w[i + 3]) * inv);
              u.z = pack2(__uint_as_float(w[i + 4]) * inv, __uint_as_float(w[i + 5]) * inv);
              u.w = pack2(__uint_as_float(w[i + 6]) * inv, __uint_as_float(w[i + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c + i) = u;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mkv, long long rows_per_page, int v_row_off, bf16* out,
           const int* table, int table_stride, const int* items, int n_items, int Hq, int Hkv, int page_size,
           float scale, int window, int* status, cudaStream_t s) {
  auto kernel = attention_tcgen05_x2_kernel<HD>;
  constexpr int smem = (int)sizeof(Attn2Storage<HD>) + 1024;
  static_assert(smem <= 227 * 1024, "two query tiles and two stages of keys and values fit one SM");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(n_items, Hkv);
  return launch_pdl(kernel, grid, 320, smem, s, mq, mkv, rows_per_page, v_row_off, out, table, table_stride, items,
                    Hq, Hkv, page_size, scale * 1.4426950408889634f, window, status);
}
}  // namespace

// As llm_attention_tcgen05 with items of up to 2 * 128 / (Hq / Hkv) tokens: two query tiles per
// CTA.  K and V come by TMA only: the pages must hold a power of two of at least 32 positions,
// else LLM_ERR_UNSUPPORTED (the one-tile kernel takes every page size).
LLM_EXPORT int llm_attention_tcgen05_x2(const void* q, void* out, int rows, const void* k_cache,
                                        const void* v_cache, long long page_stride, long long n_pages,
                                        const int* block_table, int table_stride, const int* items,
                                        int n_items, int Hq, int Hkv, int hd, int page_size, float scale,
                                        int window, int* status, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv) return LLM_ERR_ARGUMENT;
  const int G = Hq / Hkv;
  if ((hd != 64 && hd != 128) || ROWS % G) return LLM_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) return LLM_ERR_UNSUPPORTED;
  const long long v_off = (const bf16*)v_cache - (const bf16*)k_cache;
  if (n_pages <= 0 || page_size < 32 || (page_size & (page_size - 1)) || page_stride % hd || v_off <= 0 ||
      v_off % hd || n_pages * (page_stride / hd) >= (1LL << 31))
    return LLM_ERR_UNSUPPORTED;
  CUtensorMap mq, mkv;
  if (!llm_q_tensor_map(q, rows, Hq, hd, G, &mq)) return LLM_ERR_UNSUPPORTED;
  const long long rows_per_page = page_stride / hd;
  if (!llm_tensor_map(k_cache, n_pages * rows_per_page, hd, hd, page_size < KT ? page_size : KT, 64, 0, &mkv))
    return LLM_ERR_UNSUPPORTED;
  if (hd == 128)
    return launch<128>(mq, mkv, rows_per_page, (int)(v_off / hd), (bf16*)out, block_table, table_stride, items,
                       n_items, Hq, Hkv, page_size, scale, window, status, stream);
  return launch<64>(mq, mkv, rows_per_page, (int)(v_off / hd), (bf16*)out, block_table, table_stride, items,
                    n_items, Hq, Hkv, page_size, scale, window, status, stream);
}
