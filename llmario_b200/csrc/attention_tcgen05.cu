// Paged causal attention for prompt portions on the 5th-generation tensor cores (bfloat16).
//
// A CTA takes one work item (up to 128 / G consecutive tokens of one request, G = query heads per
// KV head) and one KV head.  Its 128 rows are (token, head of the group) pairs, one TMEM lane
// each.  Keys are walked in tiles of 128 aligned to absolute positions:
//
//   warp 0     TMA: the Q tile once (a 3-D box over [token][head][dim])
//   warps 6-9  K and V tiles of the pages named by the block table, as 16-byte cp.async copies
//              into the 128-byte-swizzled layout the tensor core reads, a ring of three stages.
//              With pages of 32 positions or more warp 0 fetches them by TMA instead (boxes of
//              64 columns x up to 128 positions, 4 to 16 KB); for smaller pages the TMA unit,
//              which spends ~140 cycles per box whatever its size, is slower than the copies.
//   warp 1     one lane issues  S = Q K^T  (A and B from shared memory, K-major) into one of two
//              TMEM score buffers, and  O += P V  (A = P from TMEM, B = V from shared memory,
//              N-major); the order is S0, S1, PV0, S2, PV1, ... so the products of one tile
//              overlap the softmax of the other
//   warps 2-5  softmax, one thread per row: the row's 128 scores come into registers with one
//              tcgen05.ld round trip (maximum, exponentials and sum in 32-bit), P goes back as bfloat16 over
//              the score buffer with tcgen05.st; the output accumulator is rescaled only when a
//              row's maximum has grown by more than 2^8 since the scale in use (the exact
//              normalisation happens once at the end); finally O / l is written
//
// TMEM: scores 2 x 128 columns, output head_dim columns.  Every mbarrier wait is bounded.
// Head sizes 64 and 128; G must divide 128; any page size.
#include "attention_tc_common.cuh"

namespace {

constexpr int ROWS = 128;          // rows of a CTA (TMEM lanes)
constexpr int KT = 128;            // keys per tile
constexpr int KV_STAGES = 3;

template <int HD>
struct alignas(1024) AttnStorage {
  uint8_t q[ROWS * HD * 2];                    // [HD/64 halves][128 rows][128 bytes]
  uint8_t k[KV_STAGES][KT * HD * 2];           // [HD/64 halves][128 keys][128 bytes]
  uint8_t v[KV_STAGES][KT * HD * 2];
  uint64_t q_full;
  uint64_t kv_full[KV_STAGES];
  uint64_t kv_empty[KV_STAGES];
  uint64_t s_full[2];
  uint64_t p_full[2];
  uint64_t o_done;
  uint64_t q_empty;                            // persistent form: the last scores of a work item are done
  uint64_t o_free;                             // persistent form: the softmax warps have read the output
  uint32_t tmem_base;
  int dead;                                    // a bounded wait gave up somewhere in the CTA
  int stop[2];                                 // the copy of `dead` that the softmax warps act on, per tile parity
  float xmax[2][ROWS];                         // two threads per row: the maxima of their halves of a tile
};

// SPLIT: two threads per row, each with 64 of a tile's 128 score columns (warps 2-5 the first
// half, warps 6-9 the second); used when warps 6-9 have no copying to do (K/V by TMA).
template <int HD, bool SPLIT>
__global__ void __launch_bounds__(320, 1) attention_tcgen05_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, int tma_kv,
    long long rows_per_page, int v_row_off, const bf16* __restrict__ k_cache,
    const bf16* __restrict__ v_cache, long long page_stride, bf16* __restrict__ out, const int* __restrict__ block_table, int table_stride,
    const int* __restrict__ items, int Hq, int Hkv, int page_size, float scale_log2, int window,
    int* __restrict__ status) {
  constexpr int HALVES = HD / 64;
  constexpr uint32_t S_COLS = KT;              // fp32 scores of a tile
  constexpr uint32_t O_COL = 2 * S_COLS;       // first column of the output accumulator
  // S = Q K^T: M 128, N 128, A and B K-major;  O += P V: M 128, N HD, B N-major
  constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(KT >> 3) << 17) |
                               ((uint32_t)(ROWS >> 4) << 24);
  constexpr uint32_t IDESC_O = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) |
                               ((uint32_t)(ROWS >> 4) << 24);
  extern __shared__ uint8_t raw[];
  auto& sm = *reinterpret_cast<AttnStorage<HD>*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the last items of a prompt have the most keys to walk: they are started first
  const Item it = reinterpret_cast<const Item*>(items)[gridDim.x - 1 - blockIdx.x];
  const int kvh = blockIdx.y;
  const int G = Hq / Hkv;
  const int hi = it.pos_start + it.tokens - 1;
  const int lo = (window > 0 && it.pos_start + 1 > window) ? it.pos_start + 1 - window : 0;
  const int tile_first = lo / KT;
  const int ntiles = hi / KT - tile_first + 1;

  if (threadIdx.x == 0) {
    mbar_init(&sm.q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&sm.kv_full[s], tma_kv ? 1 : 128);   // the TMA thread, or one arrival per producer thread
      mbar_init(&sm.kv_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.s_full[b], 1);
      mbar_init(&sm.p_full[b], SPLIT ? 8 : 4);   // one arrival per softmax warp
    }
    mbar_init(&sm.o_done, 1);
    sm.dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tma_kv && warp >= 6) {
    // TMA brings whole pages; a page without a key of the item is not fetched and leaves what
    // the stage held.  Such values meet zero weights and must be finite: start from zeros.
    uint4* v4 = reinterpret_cast<uint4*>(sm.v);
    for (int i = threadIdx.x - 192; i < KV_STAGES * KT * HD * 2 / 16; i += 128) v4[i] = make_uint4(0, 0, 0, 0);
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
    // ------------------------------------------------------------------ the Q tile
    if (lane == 0) {
      pdl_wait();
      mbar_expect_tx(&sm.q_full, ROWS * HD * 2);
#pragma unroll
      for (int h = 0; h < HALVES; ++h)
        tma_load_3d(sm.q + h * ROWS * 128, &map_q, h * 64, kvh * G, it.row_start, &sm.q_full);
      if (tma_kv) {
        // K and V tiles by TMA: one box of 64 columns x R positions per page (or per tile when
        // a page holds more than a tile), half and operand
        const int R = page_size < KT ? page_size : KT;
        const int* table = block_table + (size_t)it.slot * table_stride;
        bool ok = true;
        int issued = 0;
        for (int j = 0; j < ntiles && ok; ++j) {
          const int s = j % KV_STAGES;
          ok = mbar_wait(&sm.kv_empty[s], (uint32_t)((j / KV_STAGES) & 1) ^ 1);
          if (!ok) { atomicExch(status, 5); sm.dead = 1; break; }
          const int base = (tile_first + j) * KT;
          uint32_t bytes = 0;
          for (int p = base; p < base + KT; p += R)
            if (p <= hi && p + R - 1 >= lo) bytes += (uint32_t)R * HD * 2 * 2;
          mbar_expect_tx(&sm.kv_full[s], bytes);
          for (int p = base; p < base + KT; p += R) {
            if (p > hi || p + R - 1 < lo) continue;      // no key of the item here: the page may be gone
            const long long row = (long long)table[p / page_size] * rows_per_page + (long long)kvh * page_size +
                                  p % page_size;
            const int dst = (p - base) * 128;
#pragma unroll
            for (int h = 0; h < HALVES; ++h) {
              tma_load_2d(sm.k[s] + h * KT * 128 + dst, &map_kv, h * 64, (int)row, &sm.kv_full[s]);
              tma_load_2d(sm.v[s] + h * KT * 128 + dst, &map_kv, h * 64, (int)(row + v_row_off), &sm.kv_full[s]);
            }
          }
          issued = j + 1;
        }
        if (!ok)      // let what is in flight land before the shared memory is given up
          for (int j = max(0, issued - KV_STAGES); j < issued; ++j)
            mbar_wait(&sm.kv_full[j % KV_STAGES], (uint32_t)((j / KV_STAGES) & 1));
      }
    }
  } else if (warp >= 6 && !SPLIT) {
    // ------------------------------------------------------------------ K and V tiles
    // Thread p of the 128 copies the 16-byte piece (p % CPR) of rows (p / CPR), + 128 / CPR, ...
    // of every tile: its column and its row inside a group of eight never change, so the
    // swizzled destination advances by a constant.  Rows without a key are zero-filled.
    constexpr int CPR = HD / 8;                 // 16-byte pieces per row
    constexpr int RPP = 128 / CPR;              // rows per pass of the 128 threads
    const int p = threadIdx.x - 192;
    const int c = p % CPR, r0 = p / CPR;
    const uint32_t dst0 = (uint32_t)(c >> 3) * (KT * 128) + (uint32_t)r0 * 128 + (uint32_t)(((c & 7) ^ (r0 & 7)) << 4);
    const int* table = block_table + (size_t)it.slot * table_stride;
    pdl_wait();
    bool ok = true;
    for (int j = 0; j < ntiles; ++j) {
      const int s = j % KV_STAGES;
      ok = mbar_wait(&sm.kv_empty[s], (uint32_t)((j / KV_STAGES) & 1) ^ 1);
      if (!ok) { if (p == 0) atomicExch(status, 5); sm.dead = 1; break; }
      const int base = (tile_first + j) * KT;
      const uint32_t kdst = smem_u32(sm.k[s]) + dst0, vdst = smem_u32(sm.v[s]) + dst0;
      auto copy_row = [&](int r, long long off, bool live) {
        const int bytes = live ? 16 : 0;
        const uint32_t d = (uint32_t)(r - r0) * 128;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(kdst + d), "l"(k_cache + off), "r"(bytes)
                     : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(vdst + d), "l"(v_cache + off), "r"(bytes)
                     : "memory");
      };
      if (page_size >= 16 && (page_size & (page_size - 1)) == 0) {
        // pages of a power of two of at least 16 positions: the block-table entries of the
        // tile (at most eight) are fetched together, then every copy is one address addition
        const int rows_here = page_size >= KT ? KT : page_size;      // rows of the tile in one page
        const int ppt = KT / rows_here;
        const int p_first = base / page_size, inp0 = base % page_size;
        long long pb[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const int pos0 = base + g * rows_here;
          const bool live_page = g < ppt && pos0 <= hi && pos0 + rows_here - 1 >= lo;
          pb[g] = live_page ? (long long)table[p_first + g] * page_stride : -1;
        }
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          if (g >= ppt) break;
          for (int rr = r0; rr < rows_here; rr += RPP) {
            const int r = g * rows_here + rr, pos = base + r;
            const bool live = pb[g] >= 0 && pos >= lo && pos <= hi;
            copy_row(r, live ? pb[g] + ((long long)kvh * page_size + inp0 + rr) * HD + c * 8 : 0, live);
          }
        }
      } else {
        for (int r = r0; r < KT; r += RPP) {      // RPP is a multiple of 8 or divides it: r & 7 == r0 & 7
          const int pos = base + r;
          const bool live = pos >= lo && pos <= hi;
          long long off = 0;
          if (live)
            off = (long long)table[pos / page_size] * page_stride +
                  ((long long)kvh * page_size + pos % page_size) * HD + c * 8;
          copy_row(r, off, live);
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      if (j > 0) {      // the tile before this one has landed: hand it to the tensor core
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(&sm.kv_full[(j - 1) % KV_STAGES]);
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (ok && ntiles > 0) mbar_arrive(&sm.kv_full[(ntiles - 1) % KV_STAGES]);
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------------ MMA issuer
    bool ok = mbar_wait(&sm.q_full, 0);
    if (!ok) { atomicExch(status, 6); sm.dead = 1; }
    for (int j = 0; j <= ntiles && ok; ++j) {
      if (j < ntiles) {
        const int s = j % KV_STAGES, b = j & 1;
        ok = mbar_wait(&sm.kv_full[s], (uint32_t)((j / KV_STAGES) & 1));
        if (!ok) { atomicExch(status, 6); sm.dead = 1; break; }
        tc_fence_after();
        const uint32_t acc = tmem + (uint32_t)b * S_COLS;
#pragma unroll
        for (int ks = 0; ks < HD / UMMA_K; ++ks) {
          const uint32_t off = (uint32_t)(ks / 4) * (ROWS * 128) + (uint32_t)(ks % 4) * 32;
          const uint32_t offk = (uint32_t)(ks / 4) * (KT * 128) + (uint32_t)(ks % 4) * 32;
          tc_mma(acc, smem_desc(smem_u32(sm.q) + off), smem_desc(smem_u32(sm.k[s]) + offk), IDESC_S,
                 ks > 0 ? 1u : 0u);
        }
        tc_commit(&sm.s_full[b]);
      }
      if (j >= 1) {
        const int i = j - 1, s = i % KV_STAGES, b = i & 1;
        ok = mbar_wait(&sm.p_full[b], (uint32_t)((i >> 1) & 1));
        if (!ok) { atomicExch(status, 6); sm.dead = 1; break; }
        tc_fence_after();
        const uint32_t p_addr = tmem + (uint32_t)b * S_COLS;     // P over the first KT/2 columns
#pragma unroll
        for (int ks = 0; ks < KT / UMMA_K; ++ks)
          tc_mma_ts(tmem + O_COL, p_addr + (uint32_t)ks * (UMMA_K / 2),
                    smem_desc_mn(smem_u32(sm.v[s]) + (uint32_t)ks * UMMA_K * 128, KT * 128), IDESC_O,
                    (i > 0 || ks > 0) ? 1u : 0u);
        tc_commit(&sm.kv_empty[s]);
        tc_commit(&sm.o_done);
      }
    }
  } else if (warp >= 2 && (warp < 6 || SPLIT)) {
    // ------------------------------------------------------------------ softmax
    // One thread per row, or (SPLIT) two: the thread of warps 2-5 takes the first 64 score columns
    // of a tile and the first half of the output columns, its partner in warps 6-9 (same TMEM
    // lane) the second; they exchange the maxima of their halves through shared memory once per
    // tile, decide alike, and add their sums at the end.
    constexpr int COLS = SPLIT ? KT / 2 : KT;           // score columns of this thread
    constexpr int OC = SPLIT ? HD / 2 : HD;             // output columns of this thread
    const int half = SPLIT && warp >= 6 ? 1 : 0;
    const int c0 = half * COLS, oc0 = half * OC;
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    const int tok = row / G, head = kvh * G + row % G;
    const bool rvalid = tok < it.tokens;
    const int rpos = it.pos_start + tok;
    const int rlo = (window > 0 && rpos + 1 > window) ? rpos + 1 - window : 0;
    const uint32_t pair_bar = 2 + q4;                    // named barrier of the two warps of a quarter
    const uint32_t x_addr = tmem + lane_base + O_COL + HD;   // spare columns: the sums of the two halves of a row meet here
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    pdl_wait();
    for (int j = 0; j < ntiles; ++j) {
      const int b = j & 1;
      ok = mbar_wait(&sm.s_full[b], (uint32_t)((j >> 1) & 1));
      if (!ok) { if (lane == 0) atomicExch(status, 7); sm.dead = 1; }
      // All softmax warps go on or all stop: one thread copies the flag before the barrier and
      // all read the copy behind it (a warp that read the flag itself could see another value
      // than its neighbour and leave it alone at the next barrier).  A wait that gives up after
      // the copy was made stops the CTA one tile later.
      if (threadIdx.x == 64) *(volatile int*)&sm.stop[b] = *(volatile int*)&sm.dead;
      if (SPLIT) asm volatile("bar.sync 1, 256;" ::: "memory");
      else asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*(volatile int*)&sm.stop[b]) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem + lane_base + (uint32_t)b * S_COLS;
      const int base = (tile_first + j) * KT;
      // keys of this tile the row sees: columns c_lo .. c_hi
      const int c_hi = rvalid ? min(KT - 1, rpos - base) : -1;
      const int c_lo = max(0, rlo - base);
      // a tile that every row of the CTA sees completely needs no per-key tests
      const bool interior = it.tokens * G >= ROWS && base + KT - 1 <= it.pos_start &&
                            (window <= 0 || base >= hi + 1 - window);
      // ---- this thread's scores into registers (one round trip to tensor memory)
      uint32_t v[COLS];
#pragma unroll
      for (int c = 0; c < COLS; c += 32) tmem_ld32(s_addr + c0 + c, v + c);
      tmem_ld_wait();
      if (!interior) {
#pragma unroll
        for (int i = 0; i < COLS; ++i)
          if (c0 + i < c_lo || c0 + i > c_hi) v[i] = 0xff800000u;      // -inf: the key is not visible
      }
      // four independent chains, so that a comparison does not wait for the one before it
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < COLS; i += 4) {
        mx[0] = fmaxf(mx[0], __uint_as_float(v[i]));
        mx[1] = fmaxf(mx[1], __uint_as_float(v[i + 1]));
        mx[2] = fmaxf(mx[2], __uint_as_float(v[i + 2]));
        mx[3] = fmaxf(mx[3], __uint_as_float(v[i + 3]));
      }
      float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      if (SPLIT) {
        // The two threads of a row pass the maxima of their halves through shared memory.  (A
        // thread writes its word again in the next tile, behind that tile's barrier of all
        // softmax warps, which its partner reaches only after this read.)
        sm.xmax[half][row] = m_tile;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        m_tile = fmaxf(m_tile, sm.xmax[half ^ 1][row]);
      }
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
        // Rare once the maximum has settled: the rows of this warp in O are rescaled (with two
        // threads per row each its half of the columns; both see the same maxima and decide
        // alike).  Only then must the product P V of the tile before be complete (it writes O);
        // otherwise the exponentials below run while it is still going.  (That product cannot
        // be more than one phase behind: it needs this warp's P of the tile before.)
        bool done = mbar_wait(&sm.o_done, (uint32_t)((j - 1) & 1));
        if (!done) { if (lane == 0) atomicExch(status, 7); sm.dead = 1; }
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < OC; c += 32) {
          uint32_t w[32];
          tmem_ld32(tmem + lane_base + O_COL + oc0 + c, w);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(__uint_as_float(w[i]) * factor);
          tmem_st32(tmem + lane_base + O_COL + oc0 + c, w);
        }
        tmem_st_wait();
      }
      // ---- exponentials, sum, P as bfloat16 over the scores (masked scores are -inf: weight 0)
      const float muse = m_used == -INFINITY ? 0.f : m_used;
      // all exponentials first (independent of one another), then the sums, then the packing
#pragma unroll
      for (int i = 0; i < COLS; ++i)
        v[i] = __float_as_uint(ex2(fmaf(__uint_as_float(v[i]), scale_log2, -muse)));
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < COLS; i += 4) {
        sum[0] += __uint_as_float(v[i]);
        sum[1] += __uint_as_float(v[i + 1]);
        sum[2] += __uint_as_float(v[i + 2]);
        sum[3] += __uint_as_float(v[i + 3]);
      }
      l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
#pragma unroll
      for (int c = 0; c < COLS; c += 32) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          pk[i >> 1] = pack2(__uint_as_float(v[c + i]), __uint_as_float(v[c + i + 1]));
        tmem_st16(s_addr + ((c0 + c) >> 1), pk);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.p_full[b]);
    }
    if (ok) {
      // ---- the last product, then O / l
      bool done = mbar_wait(&sm.o_done, (uint32_t)((ntiles - 1) & 1));
      if (!done) { if (lane == 0) atomicExch(status, 7); }
      done = __all_sync(0xffffffffu, done);
      if (SPLIT) {      // the row's sum is the sum of the two halves' sums
        tmem_st1(x_addr + (uint32_t)(4 + half), __float_as_uint(l));
        tmem_st_wait();
        tc_fence_before();
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        tc_fence_after();
        const uint32_t other = tmem_ld1(x_addr + (uint32_t)(4 + (half ^ 1)));
        tmem_ld_wait();
        l += __uint_as_float(other);
      }
      if (done) {
        tc_fence_after();
        const float inv = 1.0f / l;
        bf16* dst = out + ((size_t)(it.row_start + tok) * Hq + head) * HD + oc0;
#pragma unroll 1
        for (int c = 0; c < OC; c += 32) {
          uint32_t w[32];
          tmem_ld32(tmem + lane_base + O_COL + oc0 + c, w);
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

// ------------------------------------------------------------------------------------------------
// The persistent form (keys and values by TMA, two softmax threads per row).  A prompt of a few
// thousand tokens is thousands of (item, KV head) pairs; as CTAs of 230 KB they run one to an SM,
// one after the other, and each pays its start (barriers, tensor-memory allocation, the first
// loads) and its end (the write of the output, the exit) with nothing beside it: about 5 us per
// CTA.  Here one CTA per SM walks its share of the pairs.  The rings of key / value tiles and of
// score buffers run on across pairs, so the loads and the first score products of the next pair
// go on while the softmax warps write the output of the one before; the Q tile is fetched as
// soon as the last scores that read the old one are done.  Pairs are dealt in rounds over the
// CTAs, every other round backwards, which evens out the slope of a causal prompt (the first CTA
// would otherwise get the heaviest pair of every round).
template <int HD>
struct Work {
  Item it;
  int kvh, hi, lo, tile_first, ntiles;
};

template <int HD>
__device__ __forceinline__ bool work_at(int round, const int* __restrict__ items, int n_items, int Hkv, int window,
                                        Work<HD>& w) {
  const int grid = (int)gridDim.x, cta = (int)blockIdx.x;
  const int idx = round * grid + ((round & 1) ? grid - 1 - cta : cta);
  if (idx >= n_items * Hkv) return false;
  // the last items of a prompt have the most keys to walk: they come first
  w.it = reinterpret_cast<const Item*>(items)[n_items - 1 - idx / Hkv];
  w.kvh = idx % Hkv;
  w.hi = w.it.pos_start + w.it.tokens - 1;
  w.lo = (window > 0 && w.it.pos_start + 1 > window) ? w.it.pos_start + 1 - window : 0;
  w.tile_first = w.lo / KT;
  w.ntiles = w.hi / KT - w.tile_first + 1;
  return true;
}

template <int HD>
__global__ void __launch_bounds__(320, 1) attention_tcgen05_persistent_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
    long long rows_per_page, int v_row_off, bf16* __restrict__ out, const int* __restrict__ block_table,
    int table_stride, const int* __restrict__ items, int n_items, int Hq, int Hkv, int page_size,
    float scale_log2, int window, int* __restrict__ status) {
  constexpr int HALVES = HD / 64;
  constexpr uint32_t S_COLS = KT;
  constexpr uint32_t O_COL = 2 * S_COLS;
  constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(KT >> 3) << 17) |
                               ((uint32_t)(ROWS >> 4) << 24);
  constexpr uint32_t IDESC_O = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) |
                               ((uint32_t)(ROWS >> 4) << 24);
  extern __shared__ uint8_t raw[];
  auto& sm = *reinterpret_cast<AttnStorage<HD>*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = Hq / Hkv;
  const int rounds = (n_items * Hkv + (int)gridDim.x - 1) / (int)gridDim.x;

  if (threadIdx.x == 0) {
    mbar_init(&sm.q_full, 1);
    mbar_init(&sm.q_empty, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&sm.kv_full[s], 1);
      mbar_init(&sm.kv_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.s_full[b], 1);
      mbar_init(&sm.p_full[b], 8);             // one arrival per softmax warp
    }
    mbar_init(&sm.o_done, 1);
    mbar_init(&sm.o_free, 8);
    sm.dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (warp >= 6) {
    // a page without a key of the item is not fetched and leaves what the stage held; such
    // values meet zero weights and must be finite: start from zeros
    uint4* v4 = reinterpret_cast<uint4*>(sm.v);
    for (int i = threadIdx.x - 192; i < KV_STAGES * KT * HD * 2 / 16; i += 128) v4[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  pdl_trigger();          // after the allocation, as in the kernel above


  if (warp == 0) {
    // ------------------------------------------------------------------ loads
    if (lane == 0) {
      pdl_wait();
      const int R = page_size < KT ? page_size : KT;
      bool ok = true;
      uint32_t T = 0;           // key tiles asked for so far, over all work items
      uint32_t st = 0, ph = 0;  // the ring stage of tile T and the parity of its use
      int W = 0;                // work items started
      for (int r = 0; r < rounds && ok; ++r) {
        Work<HD> w;
        if (!work_at<HD>(r, items, n_items, Hkv, window, w)) continue;
        // the Q tile may be replaced once the last scores of the item before are done
        if (W > 0) ok = mbar_wait(&sm.q_empty, (uint32_t)((W - 1) & 1));
        if (!ok) { atomicExch(status, 5); sm.dead = 1; break; }
        mbar_expect_tx(&sm.q_full, ROWS * HD * 2);
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
          tma_load_3d(sm.q + h * ROWS * 128, &map_q, h * 64, w.kvh * G, w.it.row_start, &sm.q_full);
        ++W;
        const int* table = block_table + (size_t)w.it.slot * table_stride;
        for (int j = 0; j < w.ntiles; ++j) {
          const int s = (int)st;
          ok = mbar_wait(&sm.kv_empty[s], ph ^ 1);
          if (!ok) { atomicExch(status, 5); sm.dead = 1; break; }
          const int base = (w.tile_first + j) * KT;
          uint32_t bytes = 0;
          for (int p = base; p < base + KT; p += R)
            if (p <= w.hi && p + R - 1 >= w.lo) bytes += (uint32_t)R * HD * 2 * 2;
          mbar_expect_tx(&sm.kv_full[s], bytes);
          for (int p = base; p < base + KT; p += R) {
            if (p > w.hi || p + R - 1 < w.lo) continue;      // no key of the item here: the page may be gone
            const long long row = (long long)table[p / page_size] * rows_per_page +
                                  (long long)w.kvh * page_size + p % page_size;
            const int dst = (p - base) * 128;
#pragma unroll
            for (int h = 0; h < HALVES; ++h) {
              tma_load_2d(sm.k[s] + h * KT * 128 + dst, &map_kv, h * 64, (int)row, &sm.kv_full[s]);
              tma_load_2d(sm.v[s] + h * KT * 128 + dst, &map_kv, h * 64, (int)(row + v_row_off), &sm.kv_full[s]);
            }
          }
          ++T;
          if (++st == KV_STAGES) st = 0, ph ^= 1;
        }
      }
      if (!ok) {      // let what is in flight land before the shared memory is given up
        for (uint32_t t = T > KV_STAGES ? T - KV_STAGES : 0; t < T; ++t)
          mbar_wait(&sm.kv_full[t % KV_STAGES], (t / KV_STAGES) & 1);
        if (W > 0) mbar_wait(&sm.q_full, (uint32_t)((W - 1) & 1));
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------------ MMA issuer
    bool ok = true;
    uint32_t T = 0, TP = 0;   // score products and P V products issued so far, over all work items
    uint32_t st = 0, ph = 0, stp = 0;      // ring stage and parity of tile T; ring stage of tile TP
    int W = 0;
    for (int r = 0; r < rounds && ok; ++r) {
      Work<HD> w;
      if (!work_at<HD>(r, items, n_items, Hkv, window, w)) continue;
      ok = mbar_wait(&sm.q_full, (uint32_t)(W & 1));
      if (!ok) { atomicExch(status, 6); sm.dead = 1; break; }
      for (int j = 0; j <= w.ntiles && ok; ++j) {
        if (j < w.ntiles) {
          const int s = (int)st, b = (int)(T & 1);
          ok = mbar_wait(&sm.kv_full[s], ph);
          if (!ok) { atomicExch(status, 6); sm.dead = 1; break; }
          tc_fence_after();
          // (score buffer b last held P of tile T - 2, whose P V was issued before this product)
          const uint32_t acc = tmem + (uint32_t)b * S_COLS;
#pragma unroll
          for (int ks = 0; ks < HD / UMMA_K; ++ks) {
            const uint32_t off = (uint32_t)(ks / 4) * (ROWS * 128) + (uint32_t)(ks % 4) * 32;
            tc_mma(acc, smem_desc(smem_u32(sm.q) + off), smem_desc(smem_u32(sm.k[s]) + off), IDESC_S,
                   ks > 0 ? 1u : 0u);
          }
          tc_commit(&sm.s_full[b]);
          if (j == w.ntiles - 1) tc_commit(&sm.q_empty);
          ++T;
          if (++st == KV_STAGES) st = 0, ph ^= 1;
        }
        if (j >= 1) {
          const int s = (int)stp, b = (int)(TP & 1);
          ok = mbar_wait(&sm.p_full[b], (TP >> 1) & 1);
          // the first P V of an item starts the output anew: the output of the item before must
          // have been read
          if (ok && j == 1 && W > 0) ok = mbar_wait(&sm.o_free, (uint32_t)((W - 1) & 1));
          if (!ok) { atomicExch(status, 6); sm.dead = 1; break; }
          tc_fence_after();
          const uint32_t p_addr = tmem + (uint32_t)b * S_COLS;     // P over the first KT/2 columns
#pragma unroll
          for (int ks = 0; ks < KT / UMMA_K; ++ks)
            tc_mma_ts(tmem + O_COL, p_addr + (uint32_t)ks * (UMMA_K / 2),
                      smem_desc_mn(smem_u32(sm.v[s]) + (uint32_t)ks * UMMA_K * 128, KT * 128), IDESC_O,
                      (j > 1 || ks > 0) ? 1u : 0u);
          tc_commit(&sm.kv_empty[s]);
          tc_commit(&sm.o_done);
          ++TP;
          if (++stp == KV_STAGES) stp = 0;
        }
      }
      ++W;
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------------ softmax
    // Two threads per row, as in the kernel above; the counters of tiles run on across items.
    constexpr int COLS = KT / 2;
    constexpr int OC = HD / 2;
    const int half = warp >= 6 ? 1 : 0;
    const int c0 = half * COLS, oc0 = half * OC;
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    const uint32_t x_addr = tmem + lane_base + O_COL + HD;   // spare columns: the sums of the two halves of a row meet here
    auto pair_sync = [&]() {      // the two warps of a quarter (immediate ids: six barriers in all)
      if (q4 == 0) asm volatile("bar.sync 2, 64;" ::: "memory");
      else if (q4 == 1) asm volatile("bar.sync 3, 64;" ::: "memory");
      else if (q4 == 2) asm volatile("bar.sync 4, 64;" ::: "memory");
      else asm volatile("bar.sync 5, 64;" ::: "memory");
    };
    bool ok = true;
    uint32_t T = 0;
    pdl_wait();
    for (int r = 0; r < rounds && ok; ++r) {
      Work<HD> w;
      if (!work_at<HD>(r, items, n_items, Hkv, window, w)) continue;
      const int tok = row / G, head = w.kvh * G + row % G;
      const bool rvalid = tok < w.it.tokens;
      const int rpos = w.it.pos_start + tok;
      const int rlo = (window > 0 && rpos + 1 > window) ? rpos + 1 - window : 0;
      float m_used = -INFINITY, l = 0.f;
      for (int j = 0; j < w.ntiles; ++j, ++T) {
        const int b = (int)(T & 1);
        ok = mbar_wait(&sm.s_full[b], (T >> 1) & 1);
        if (!ok) { if (lane == 0) atomicExch(status, 7); sm.dead = 1; }
        // all eight warps go on or all stop (see the kernel above)
        if (threadIdx.x == 64) *(volatile int*)&sm.stop[b] = *(volatile int*)&sm.dead;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (*(volatile int*)&sm.stop[b]) { ok = false; break; }
        tc_fence_after();
        const uint32_t s_addr = tmem + lane_base + (uint32_t)b * S_COLS;
        const int base = (w.tile_first + j) * KT;
        const int c_hi = rvalid ? min(KT - 1, rpos - base) : -1;
        const int c_lo = max(0, rlo - base);
        const bool interior = w.it.tokens * G >= ROWS && base + KT - 1 <= w.it.pos_start &&
                              (window <= 0 || base >= w.hi + 1 - window);
        uint32_t v[COLS];
#pragma unroll
        for (int c = 0; c < COLS; c += 32) tmem_ld32(s_addr + c0 + c, v + c);
        tmem_ld_wait();
        if (!interior) {
#pragma unroll
          for (int i = 0; i < COLS; ++i)
            if (c0 + i < c_lo || c0 + i > c_hi) v[i] = 0xff800000u;      // -inf: the key is not visible
        }
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < COLS; i += 4) {
          mx[0] = fmaxf(mx[0], __uint_as_float(v[i]));
          mx[1] = fmaxf(mx[1], __uint_as_float(v[i + 1]));
          mx[2] = fmaxf(mx[2], __uint_as_float(v[i + 2]));
          mx[3] = fmaxf(mx[3], __uint_as_float(v[i + 3]));
        }
        float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        sm.xmax[half][row] = m_tile;             // the partner's half of the row: through shared memory
        pair_sync();
        m_tile = fmaxf(m_tile, sm.xmax[half ^ 1][row]) * scale_log2;
        const bool grow = m_tile > m_used + 8.0f;
        float factor = 1.f;
        if (grow) {
          factor = m_used == -INFINITY ? 0.f : ex2(m_used - m_tile);
          m_used = m_tile;
          l *= factor;
        }
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          // the product P V of the tile before writes O: it must be complete
          bool done = mbar_wait(&sm.o_done, (T - 1) & 1);
          if (!done) { if (lane == 0) atomicExch(status, 7); sm.dead = 1; }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < OC; c += 32) {
            uint32_t u[32];
            tmem_ld32(tmem + lane_base + O_COL + oc0 + c, u);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) u[i] = __float_as_uint(__uint_as_float(u[i]) * factor);
            tmem_st32(tmem + lane_base + O_COL + oc0 + c, u);
          }
          tmem_st_wait();
        }
        const float muse = m_used == -INFINITY ? 0.f : m_used;
#pragma unroll
        for (int i = 0; i < COLS; ++i)
          v[i] = __float_as_uint(ex2(fmaf(__uint_as_float(v[i]), scale_log2, -muse)));
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < COLS; i += 4) {
          sum[0] += __uint_as_float(v[i]);
          sum[1] += __uint_as_float(v[i + 1]);
          sum[2] += __uint_as_float(v[i + 2]);
          sum[3] += __uint_as_float(v[i + 3]);
        }
        l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
#pragma unroll
        for (int c = 0; c < COLS; c += 32) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            pk[i >> 1] = pack2(__uint_as_float(v[c + i]), __uint_as_float(v[c + i + 1]));
          tmem_st16(s_addr + ((c0 + c) >> 1), pk);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.p_full[b]);
      }
      if (!ok) break;
      // ---- the item's last product, then O / l
      bool done = mbar_wait(&sm.o_done, (T - 1) & 1);
      if (!done) { if (lane == 0) atomicExch(status, 7); sm.dead = 1; }
      done = __all_sync(0xffffffffu, done);
      tmem_st1(x_addr + (uint32_t)(4 + half), __float_as_uint(l));
      tmem_st_wait();
      tc_fence_before();
      pair_sync();
      tc_fence_after();
      const uint32_t other = tmem_ld1(x_addr + (uint32_t)(4 + (half ^ 1)));
      tmem_ld_wait();
      l += __uint_as_float(other);
      const float inv = 1.0f / l;
      bf16* dst = out + ((size_t)(w.it.row_start + tok) * Hq + head) * HD + oc0;
      // the whole half row into registers, so that the next item's first P V need not wait for
      // the stores
      uint32_t u[OC];
#pragma unroll
      for (int c = 0; c < OC; c += 32) tmem_ld32(tmem + lane_base + O_COL + oc0 + c, u + c);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.o_free);
      if (rvalid && done) {
#pragma unroll
        for (int i = 0; i < OC; i += 8) {
          uint4 pk4;
          pk4.x = pack2(__uint_as_float(u[i]) * inv, __uint_as_float(u[i + 1]) * inv);
          pk4.y = pack2(__uint_as_float(u[i + 2]) * inv, __uint_as_float(u[i + 3]) * inv);
          pk4.z = pack2(__uint_as_float(u[i + 4]) * inv, __uint_as_float(u[i + 5]) * inv);
          pk4.w = pack2(__uint_as_float(u[i + 6]) * inv, __uint_as_float(u[i + 7]) * inv);
          *reinterpret_cast<uint4*>(dst + i) = pk4;
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

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

bool llm_q_tensor_map(const void* q, int rows, int Hq, int hd, int G, CUtensorMap* out) {
  static EncodeTiled enc = nullptr;
  if (!enc) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult r;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &r) != cudaSuccess ||
        r != cudaDriverEntryPointSuccess)
      return false;
    enc = reinterpret_cast<EncodeTiled>(p);
  }
  cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)Hq, (cuuint64_t)rows};
  cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)Hq * hd * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(ROWS / G)};
  cuuint32_t elem[3] = {1, 1, 1};
  return enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

namespace {
template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mkv, int tma_kv, long long rows_per_page, int v_row_off,
           const bf16* kc, const bf16* vc, long long page_stride, bf16* out,
           const int* table, int table_stride, const int* items, int n_items, int Hq, int Hkv, int page_size,
           float scale, int window, int persistent, int* status, cudaStream_t s) {
  constexpr int smem = (int)sizeof(AttnStorage<HD>) + 1024;
  static_assert(smem <= 227 * 1024, "the Q tile and three stages of K and V fit one SM");
  if (tma_kv && persistent) {
    // more (item, KV head) pairs than SMs: one CTA per SM walks its share of them
    static int sms = 0;
    if (!sms) {
      int dev = 0;
      if (cudaGetDevice(&dev) != cudaSuccess ||
          cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return LLM_ERR_UNSUPPORTED;
    }
    if ((long long)n_items * Hkv > sms) {
      auto pk = attention_tcgen05_persistent_kernel<HD>;
      static bool pconf = false;
      if (!pconf) {
        cudaError_t e = cudaFuncSetAttribute(pk, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        pconf = true;
      }
      return launch_pdl(pk, dim3(sms), 320, smem, s, mq, mkv, rows_per_page, v_row_off, out, table, table_stride,
                        items, n_items, Hq, Hkv, page_size, scale * 1.4426950408889634f, window, status);
    }
  }
  // keys and values by TMA leave warps 6-9 free: they take half of every row's softmax
  auto kernel = tma_kv ? attention_tcgen05_kernel<HD, true> : attention_tcgen05_kernel<HD, false>;
  static bool configured[2] = {false, false};
  if (!configured[tma_kv ? 1 : 0]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured[tma_kv ? 1 : 0] = true;
  }
  dim3 grid(n_items, Hkv);
  return launch_pdl(kernel, grid, 320, smem, s, mq, mkv, tma_kv, rows_per_page, v_row_off, kc, vc, page_stride, out,
                    table, table_stride, items, Hq, Hkv, page_size, scale * 1.4426950408889634f, window, status);
}
}  // namespace

// q, out: [rows][Hq * hd] bfloat16; k_cache / v_cache: this layer call's K and V planes of page 0 in a
// cache [page][...][kv head][position][head dim] with `page_stride` elements from page to page;
// items: n_items x (first row, tokens <= 128 / (Hq / Hkv), request slot, first position).
// n_pages: pages of the cache; when positive and the pages hold a power of two of at least 32
// positions, K and V are fetched by TMA, else (or with n_pages 0) by cp.async copies.
// persistent: non-zero lets the kernel run, when K and V come by TMA and there are more (item, KV
// head) pairs than SMs, as one CTA per SM that walks its share of the pairs; that pays while the
// items are short (it saves about 3 us per pair) and costs a few percent when they are long.
LLM_EXPORT int llm_attention_tcgen05(const void* q, void* out, int rows, const void* k_cache,
                                     const void* v_cache, long long page_stride, long long n_pages,
                                     const int* block_table,
                                     int table_stride, const int* items, int n_items, int Hq, int Hkv,
                                     int hd, int page_size, float scale, int window, int persistent,
                                     int* status, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv) return LLM_ERR_ARGUMENT;
  const int G = Hq / Hkv;
  if ((hd != 64 && hd != 128) || ROWS % G) return LLM_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) return LLM_ERR_UNSUPPORTED;
  if ((page_stride * 2) % 16) return LLM_ERR_UNSUPPORTED;
  CUtensorMap mq;
  if (!llm_q_tensor_map(q, rows, Hq, hd, G, &mq)) return LLM_ERR_UNSUPPORTED;
  // The cache seen from this layer call's K plane as rows of hd elements: page p, KV head h,
  // position i is row p * rows_per_page + h * page_size + i; the V plane lies v_row_off rows on.
  CUtensorMap mkv = mq;
  int tma_kv = 0, v_row_off = 0;
  long long rows_per_page = 0;
  const long long v_off = (const bf16*)v_cache - (const bf16*)k_cache;
  if (n_pages > 0 && page_size >= 32 && (page_size & (page_size - 1)) == 0 && page_stride % hd == 0 &&
      v_off > 0 && v_off % hd == 0 && n_pages * (page_stride / hd) < (1LL << 31)) {
    rows_per_page = page_stride / hd;
    v_row_off = (int)(v_off / hd);
    tma_kv = llm_tensor_map(k_cache, n_pages * rows_per_page, hd, hd, page_size < KT ? page_size : KT, 64, 0, &mkv)
                 ? 1 : 0;
  }
  if (hd == 128)
    return launch<128>(mq, mkv, tma_kv, rows_per_page, v_row_off, (const bf16*)k_cache, (const bf16*)v_cache,
                       page_stride, (bf16*)out, block_table, table_stride, items, n_items, Hq, Hkv, page_size, scale,
                       window, persistent, status, stream);
  return launch<64>(mq, mkv, tma_kv, rows_per_page, v_row_off, (const bf16*)k_cache, (const bf16*)v_cache,
                    page_stride, (bf16*)out, block_table, table_stride, items, n_items, Hq, Hkv, page_size, scale,
                    window, persistent, status, stream);
}
