// Decode attention with the cache streamed by the TMA unit.
//
// The arithmetic is that of attention_decode.cu (keys on the M side of mma.sync m16n8k16, at most
// eight (token, head) pairs per item, 32-bit running maximum and sum per pair, optional split of
// the key range).  What differs is how K and V reach shared memory.  The cache of a group of
// layers is one tensor [page][cache slot][K|V][kv head][position][head dim].  One tensor map of
// five dimensions describes it (64 columns of a row, the 64-column halves of a row, the
// positions of a page, the KV heads, the K and V planes of all pages and cache slots), and ONE
// tile load brings the keys and the values of a page and KV head: up to 64 positions, 8 KB for a
// page of 16 at head size 128.  The TMA unit spends about the same time on a load whatever its
// size, so few large loads are what lets a warp stream at the memory's speed.  The bytes are
// counted on an mbarrier per stage of a ring of three tiles of 32 keys (four such CTAs to an SM
// at head size 128: the same bytes in flight as three CTAs with two tiles of 64 keys, but a
// fourth warp to work on them, which streams a tenth to a sixth faster); the warp spends its
// instructions on the products and not on addresses.  Head sizes 64 and 128; other sizes use attention_decode.cu.
#include "attention_common.cuh"
#include "tcgen05.cuh"

namespace {
constexpr int DECODE_KT = 32, DECODE_STAGES = 3;   // keys of a tile, tiles in flight per warp

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}

// Byte offset, inside a stage, of 16-byte chunk c (0 .. HD/8-1) of key row r (0 .. KT-1) of the
// K (kv = 0) or V (kv = 1) tile.  A stage holds KT >> lgR loads of R = 1 << lgR positions, each
// laid out as the TMA unit writes its box: [K|V][position][HD * 2 bytes], with the 128-byte
// swizzle (the chunk index is xor-ed with bits 7..9 of the address; stages are 1024-byte aligned).
template <int HD> __device__ __forceinline__ int tile_off(int kv, int r, int c, int lgR) {
  const int lin = ((((r >> lgR) * 2 + kv) << lgR) + (r & ((1 << lgR) - 1))) * (HD * 2) + (c >> 3) * 128;
  return lin + (((c & 7) ^ ((lin >> 7) & 7)) << 4);
}

// What the fused form needs beside the attention's own arguments: it starts from the output of
// the q/k/v product and does the per-head norm, the rotation and the cache write of the new
// token itself, so that a decode step has no kernel between that product and attention.
struct Fused {
  float* proj;              // [rows][proj_stride] 32-bit: Hq heads of q, then Hkv of k and Hkv of v
  int proj_stride;
  const float* q_norm_w;    // [HD] each; null: heads are not normed
  const float* k_norm_w;
  const float2* cos_sin;    // [rows][HD/2] (cos, sin) of the row's position, scale factor included
  bf16* k_cache;            // planes of this call's cache slot; null: the cache belongs to
  bf16* v_cache;            // another call, there is no k or v in proj
  long long page_stride;
  float eps;
  int clear;                // clear what was read of proj (q only when keys are not split: with
};                          // split keys several CTAs read it and the merge clears it)

template <int HD, int KT, int STAGES, bool FUSED>
__global__ void __launch_bounds__(32, 4) flash_decode_tma_kernel(
    const __grid_constant__ CUtensorMap map_kv, const bf16* __restrict__ q, bf16* __restrict__ out,
    float* __restrict__ part_o, float* __restrict__ part_ml, const int* __restrict__ block_table,
    int table_stride, const int* __restrict__ items, const int* __restrict__ row_slot,
    const int* __restrict__ row_pos, int Hq, int Hkv, int page_size, int n_slots, int slot,
    float scale_log2, int window, int splits, int* __restrict__ status, const Fused fu) {
  constexpr int KS = HD / 16, MT = KT / 16, DM = HD / 16;
  constexpr int TILE_BYTES = KT * HD * 2;            // one K or V tile
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* kv_tiles = smem;                          // [STAGES][2 * TILE_BYTES]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * 2 * TILE_BYTES);
  pdl_trigger();

  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  if (lane == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();

  // Before the wait on the kernels ahead in the stream, only what none of them writes is read:
  // the work items, rows and block tables (complete before the step's first layer starts: the
  // embedding kernel waits before it lets its dependents start) and the keys and values of
  // positions below the item's first one, which earlier steps wrote.
  const Item it = items ? reinterpret_cast<const Item*>(items)[blockIdx.x]
                        : Item{(int)blockIdx.x, 1, row_slot[blockIdx.x], row_pos[blockIdx.x]};
  const int kvh = blockIdx.y, z = blockIdx.z;
  const int G = Hq / Hkv;
  const int pairs = it.tokens * G;                 // <= 8
  const int hi = it.pos_start + it.tokens - 1;
  const int lo = (window > 0 && it.pos_start + 1 > window) ? it.pos_start + 1 - window : 0;
  const int tile_first = lo / KT, tile_last = hi / KT;
  const int ntiles = tile_last - tile_first + 1;
  const int per = (ntiles + splits - 1) / splits;
  const int tb0 = tile_first + z * per;
  const int tb1 = min(tile_last + 1, tb0 + per);
  const int* table = block_table + (size_t)it.slot * table_stride;

  // The pages of a tile are asked for R = min(page_size, KT) positions at a time, K and V of
  // them in one box.  The warp keeps 32 entries of the block table in its lanes (one load for
  // every 32 pages walked), so that no tile waits on a load of a page number.
  const int R = page_size < KT ? page_size : KT;
  const int lgR = 31 - __clz(R);
  const int lgP = 31 - __clz(page_size);            // pages hold a power of two of positions here
  const int last_page = hi >> lgP;
  int held_from = (tb0 * KT) >> lgP;
  int held = held_from + lane <= last_page ? table[held_from + lane] : 0;
  auto load_tile = [&](int tb, int stage) {         // the whole warp calls it; lane 0 issues
    const int base = tb * KT;
    uint32_t bytes = 0;
    for (int p = base; p < base + KT; p += R)
      if (p <= hi && p + R - 1 >= lo) bytes += (uint32_t)R * HD * 2 * 2;
    if (lane == 0) mbar_expect_tx(&full[stage], bytes);
    for (int p = base; p < base + KT; p += R) {
      if (p > hi || p + R - 1 < lo) continue;       // no key of the item here: the page may be gone
      const int pi = p >> lgP;
      if (pi < held_from || pi >= held_from + 32) {
        held_from = pi;
        held = pi + lane <= last_page ? table[pi + lane] : 0;
      }
      const int plane = (__shfl_sync(0xffffffffu, held, pi - held_from) * n_slots + slot) * 2;
      if (lane == 0)
        tma_load_5d(kv_tiles + stage * 2 * TILE_BYTES + ((p - base) >> lgR) * (2 * R * HD * 2), &map_kv, 0, 0,
                    p & (page_size - 1), kvh, plane, &full[stage]);
    }
  };
  int early = 0;          // tiles asked for before the wait: those wholly below the new positions
  for (; early < STAGES && tb0 + early < tb1 && (tb0 + early + 1) * KT <= it.pos_start; ++early)
    load_tile(tb0 + early, early);
  pdl_wait();
  for (int i = early; i < STAGES && tb0 + i < tb1; ++i) load_tile(tb0 + i, i);

  int cpos[2], clo[2];
  bool cvalid[2];
  size_t crow[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int n = 2 * t + j;
    cvalid[j] = n < pairs;
    const int tok = cvalid[j] ? n / G : 0, head = kvh * G + (cvalid[j] ? n % G : 0);
    cpos[j] = it.pos_start + tok;
    clo[j] = (window > 0 && cpos[j] + 1 > window) ? cpos[j] + 1 - window : 0;
    crow[j] = (size_t)(it.row_start + tok) * Hq + head;
  }
  uint32_t qf[KS][2];
  if constexpr (!FUSED) {
    const bool valid = g < pairs;
    const int tok = valid ? g / G : 0, head = kvh * G + (valid ? g % G : 0);
    const bf16* src = q + ((size_t)(it.row_start + tok) * Hq + head) * HD + 2 * t;
#pragma unroll
    for (int k = 0; k < KS; ++k) {
      qf[k][0] = valid ? *reinterpret_cast<const uint32_t*>(src + k * 16) : 0u;
      qf[k][1] = valid ? *reinterpret_cast<const uint32_t*>(src + k * 16 + 8) : 0u;
    }
  }
  // The fused form (items of one token): the lane's 2 * KS pairs of query values are made here
  // from the projection, in the layout of the fragments: norm over the head (the four lanes of
  // a pair hold it), rotation of (c, c + HD/2), which lie in the same lane, rounding once.
  uint32_t k_new[2] = {0u, 0u}, v_new[2] = {0u, 0u};    // this lane's part of the new key and value
  bool writer = false;
  if constexpr (FUSED) {
    constexpr int NP = HD / 64;              // new key and value: lane l has elements NP*l .. and those + HD/2
    const bool valid = g < G;
    float* row = fu.proj + (size_t)it.row_start * fu.proj_stride;
    float* src = row + (kvh * G + (valid ? g : 0)) * HD + 2 * t;
    float* ks = row + (Hq + kvh) * HD;
    float* vs = row + (Hq + Hkv + kvh) * HD;
    const float2* cs_row = fu.cos_sin + (size_t)it.row_start * (HD / 2);
    // The CTA whose keys end with the new position makes the new key and value, writes them to
    // the cache and keeps them: its last tile comes from memory without them.
    writer = fu.k_cache != nullptr && tb0 <= tile_last && tb1 == tile_last + 1;
    // every load first, so that they are in flight together; then the clearing stores; then the sums
    float2 x[KS][2], w[KS][2];
    float4 cs[KS / 2][2];
    float a[NP], b[NP], va[NP], vb[NP], wa[NP], wb[NP];
    float2 kcs[NP];
#pragma unroll
    for (int k = 0; k < KS; ++k)
#pragma unroll
      for (int j = 0; j < 2; ++j)
        x[k][j] = valid ? *reinterpret_cast<const float2*>(src + 16 * k + 8 * j) : make_float2(0.f, 0.f);
    if (writer) {
#pragma unroll
      for (int e = 0; e < NP; ++e) {
        a[e] = ks[NP * lane + e], b[e] = ks[HD / 2 + NP * lane + e];
        va[e] = vs[NP * lane + e], vb[e] = vs[HD / 2 + NP * lane + e];
        kcs[e] = cs_row[NP * lane + e];
        wa[e] = fu.k_norm_w ? fu.k_norm_w[NP * lane + e] : 1.f;
        wb[e] = fu.k_norm_w ? fu.k_norm_w[HD / 2 + NP * lane + e] : 1.f;
      }
    }
#pragma unroll
    for (int k = 0; k < KS; ++k)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        if (fu.q_norm_w) w[k][j] = *reinterpret_cast<const float2*>(fu.q_norm_w + 16 * k + 8 * j + 2 * t);
        if (k < KS / 2) cs[k][j] = *reinterpret_cast<const float4*>(cs_row + 16 * k + 8 * j + 2 * t);   // (cos, sin) x 2
      }
    if (fu.clear) {
      if (splits == 1 && valid) {
#pragma unroll
        for (int k = 0; k < KS; ++k)
#pragma unroll
          for (int j = 0; j < 2; ++j) *reinterpret_cast<float2*>(src + 16 * k + 8 * j) = make_float2(0.f, 0.f);
      }
      if (writer) {
#pragma unroll
        for (int e = 0; e < NP; ++e) {
          ks[NP * lane + e] = 0.f, ks[HD / 2 + NP * lane + e] = 0.f;
          vs[NP * lane + e] = 0.f, vs[HD / 2 + NP * lane + e] = 0.f;
        }
      }
    }
    if (fu.q_norm_w) {
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < KS; ++k)
#pragma unroll
        for (int j = 0; j < 2; ++j) ss += x[k][j].x * x[k][j].x + x[k][j].y * x[k][j].y;
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      const float sc = 1.0f / sqrtf(ss / (float)HD + fu.eps);
#pragma unroll
      for (int k = 0; k < KS; ++k)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          x[k][j].x = x[k][j].x * sc * w[k][j].x;
          x[k][j].y = x[k][j].y * sc * w[k][j].y;
        }
    }
#pragma unroll
    for (int k = 0; k < KS / 2; ++k)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float4 c = cs[k][j];
        const float2 lo2 = x[k][j], hi2 = x[k + KS / 2][j];
        qf[k][j] = pack_bf16(lo2.x * c.x - hi2.x * c.y, lo2.y * c.z - hi2.y * c.w);
        qf[k + KS / 2][j] = pack_bf16(lo2.x * c.y + hi2.x * c.x, lo2.y * c.w + hi2.y * c.z);
      }
    if (writer) {
      if (fu.k_norm_w) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < NP; ++e) ss += a[e] * a[e];
#pragma unroll
        for (int e = 0; e < NP; ++e) ss += b[e] * b[e];
        ss = warp_sum(ss);
        const float sc = 1.0f / sqrtf(ss / (float)HD + fu.eps);
#pragma unroll
        for (int e = 0; e < NP; ++e) {
          a[e] = a[e] * sc * wa[e];
          b[e] = b[e] * sc * wb[e];
        }
      }
      float ra[2] = {0.f, 0.f}, rb[2] = {0.f, 0.f};
#pragma unroll
      for (int e = 0; e < NP; ++e) {
        ra[e] = a[e] * kcs[e].x - b[e] * kcs[e].y;
        rb[e] = a[e] * kcs[e].y + b[e] * kcs[e].x;
      }
      k_new[0] = pack_bf16(ra[0], ra[1]), k_new[1] = pack_bf16(rb[0], rb[1]);
      v_new[0] = pack_bf16(va[0], NP > 1 ? va[NP - 1] : 0.f);
      v_new[1] = pack_bf16(vb[0], NP > 1 ? vb[NP - 1] : 0.f);
      const size_t at = (size_t)table[hi / page_size] * fu.page_stride +
                        (size_t)(kvh * page_size + hi % page_size) * HD;
      if (NP == 2) {
        *reinterpret_cast<uint32_t*>(fu.k_cache + at + 2 * lane) = k_new[0];
        *reinterpret_cast<uint32_t*>(fu.k_cache + at + HD / 2 + 2 * lane) = k_new[1];
        *reinterpret_cast<uint32_t*>(fu.v_cache + at + 2 * lane) = v_new[0];
        *reinterpret_cast<uint32_t*>(fu.v_cache + at + HD / 2 + 2 * lane) = v_new[1];
      } else {
        reinterpret_cast<uint16_t*>(fu.k_cache + at)[lane] = (uint16_t)k_new[0];
        reinterpret_cast<uint16_t*>(fu.k_cache + at)[HD / 2 + lane] = (uint16_t)k_new[1];
        reinterpret_cast<uint16_t*>(fu.v_cache + at)[lane] = (uint16_t)v_new[0];
        reinterpret_cast<uint16_t*>(fu.v_cache + at)[HD / 2 + lane] = (uint16_t)v_new[1];
      }
    }
  }
  float o[DM][4];
#pragma unroll
  for (int d = 0; d < DM; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  bool alive = true;
  for (int tb = tb0; tb < tb1; ++tb) {
    const int n_it = tb - tb0;
    const int stage = n_it % STAGES;
    alive = mbar_wait(&full[stage], (uint32_t)(n_it / STAGES) & 1);
    alive = __all_sync(0xffffffffu, alive);
    if (!alive) {
      if (lane == 0) atomicExch(status, 4);
      break;
    }
    uint8_t* tile = kv_tiles + stage * 2 * TILE_BYTES;
    // A page without a key of the item is not fetched (only the first tile under a window and
    // the last tile have such pages).  Its values meet zero weights and must be finite, and
    // shared memory starts with whatever it held: clear them.  (Its keys may be anything: their
    // scores are replaced by -inf.)
    {
      const int base = tb * KT;
      for (int p = base; p < base + KT; p += R)
        if (p > hi || p + R - 1 < lo) {
          uint4* vz = reinterpret_cast<uint4*>(tile + ((p - base) >> lgR) * (2 * R * HD * 2) + R * HD * 2);
          for (int i = lane; i < R * HD * 2 / 16; i += 32) vz[i] = make_uint4(0, 0, 0, 0);
        }
      if (FUSED && writer && tb == tile_last) {      // the new key and value, over what memory held there
        constexpr int NP = HD / 64;
        const int r = hi - base, c0 = NP * lane, c1 = HD / 2 + NP * lane;
        uint8_t* k0 = tile + tile_off<HD>(0, r, c0 >> 3, lgR) + (c0 & 7) * 2;
        uint8_t* k1 = tile + tile_off<HD>(0, r, c1 >> 3, lgR) + (c1 & 7) * 2;
        uint8_t* v0 = tile + tile_off<HD>(1, r, c0 >> 3, lgR) + (c0 & 7) * 2;
        uint8_t* v1 = tile + tile_off<HD>(1, r, c1 >> 3, lgR) + (c1 & 7) * 2;
        if (NP == 2) {
          *reinterpret_cast<uint32_t*>(k0) = k_new[0], *reinterpret_cast<uint32_t*>(k1) = k_new[1];
          *reinterpret_cast<uint32_t*>(v0) = v_new[0], *reinterpret_cast<uint32_t*>(v1) = v_new[1];
        } else {
          *reinterpret_cast<uint16_t*>(k0) = (uint16_t)k_new[0], *reinterpret_cast<uint16_t*>(k1) = (uint16_t)k_new[1];
          *reinterpret_cast<uint16_t*>(v0) = (uint16_t)v_new[0], *reinterpret_cast<uint16_t*>(v1) = (uint16_t)v_new[1];
        }
      }
      __syncwarp();
    }

    // ---- S^T = K Q^T
    float s[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) s[mt][0] = s[mt][1] = s[mt][2] = s[mt][3] = 0.f;
#pragma unroll
    for (int k = 0; k < KS; ++k) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t a[4];
        const int mi = lane >> 3;
        ldmatrix_x4(a, tile + tile_off<HD>(0, mt * 16 + (mi & 1) * 8 + (lane & 7), 2 * k + (mi >> 1), lgR));
        mma_bf16(s[mt], a, qf[k][0], qf[k][1]);
      }
    }
    // ---- mask, running maximum per pair, exponentials
    const int base = tb * KT;
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = e & 1;
        const int p = base + mt * 16 + g + 8 * (e >> 1);
        const bool vis = cvalid[j] && p <= cpos[j] && p >= clo[j];
        s[mt][e] = vis ? s[mt][e] * scale_log2 : -INFINITY;
        tmax[j] = fmaxf(tmax[j], s[mt][e]);
      }
    float corr[2], muse[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      tmax[j] = fmaxf(tmax[j], __shfl_xor_sync(0xffffffffu, tmax[j], 4));
      tmax[j] = fmaxf(tmax[j], __shfl_xor_sync(0xffffffffu, tmax[j], 8));
      tmax[j] = fmaxf(tmax[j], __shfl_xor_sync(0xffffffffu, tmax[j], 16));
      const float mnew = fmaxf(m[j], tmax[j]);
      muse[j] = mnew == -INFINITY ? 0.f : mnew;
      corr[j] = fast_exp2(m[j] - muse[j]);
      m[j] = mnew;
      l[j] *= corr[j];
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pexp = fast_exp2(s[mt][e] - muse[e & 1]);
        s[mt][e] = pexp;
        l[e & 1] += pexp;
      }
    if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
      for (int d = 0; d < DM; ++d) {
        o[d][0] *= corr[0]; o[d][1] *= corr[1];
        o[d][2] *= corr[0]; o[d][3] *= corr[1];
      }
    }
    // ---- O^T += V^T P^T
#pragma unroll
    for (int kk = 0; kk < MT; ++kk) {
      const uint32_t b0 = movmatrix_trans(pack_bf16(s[kk][0], s[kk][1]));
      const uint32_t b1 = movmatrix_trans(pack_bf16(s[kk][2], s[kk][3]));
#pragma unroll
      for (int d = 0; d < DM; ++d) {
        uint32_t a[4];
        const int mi = lane >> 3;
        ldmatrix_x4_trans(a, tile + tile_off<HD>(1, kk * 16 + (mi >> 1) * 8 + (lane & 7), 2 * d + (mi & 1), lgR));
        mma_bf16(o[d], a, b0, b1);
      }
    }
    __syncwarp();                  // every lane has read this stage
    if (tb + STAGES < tb1) {
      if (lane == 0) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      load_tile(tb + STAGES, stage);
    }
  }
  if (!alive) {   // let the loads that are still in flight land before the shared memory goes
    for (int i = 0; i < STAGES; ++i) mbar_wait(&full[i], 0), mbar_wait(&full[i], 1);
    return;
  }

#pragma unroll
  for (int j = 0; j < 2; ++j) {
    l[j] += __shfl_xor_sync(0xffffffffu, l[j], 4);
    l[j] += __shfl_xor_sync(0xffffffffu, l[j], 8);
    l[j] += __shfl_xor_sync(0xffffffffu, l[j], 16);
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    if (!cvalid[j]) continue;
    if (splits == 1) {
      const float inv = 1.0f / l[j];
      bf16* dst = out + crow[j] * HD;
#pragma unroll
      for (int d = 0; d < DM; ++d) {
        dst[d * 16 + g] = __float2bfloat16_rn(o[d][j] * inv);
        dst[d * 16 + g + 8] = __float2bfloat16_rn(o[d][2 + j] * inv);
      }
    } else {
      float* dst = part_o + (crow[j] * splits + z) * HD;
#pragma unroll
      for (int d = 0; d < DM; ++d) {
        dst[d * 16 + g] = o[d][j];
        dst[d * 16 + g + 8] = o[d][2 + j];
      }
      if (g == 0) {
        part_ml[(crow[j] * splits + z) * 2] = m[j];
        part_ml[(crow[j] * splits + z) * 2 + 1] = l[j];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// The persistent form, for steps of single new tokens whose (request, KV head) units would make
// several waves of CTAs.  As many one-warp CTAs as the GPU holds at once share the tiles of ALL
// units evenly: the tiles are numbered unit by unit (request-major, then KV head), CTA w takes
// tiles [w Q, (w + 1) Q), and so walks the end of one unit, whole units, and the start of another.
// No wave is left half empty, and the ring of tiles runs on from one unit to the next.  Each
// piece of a unit that a CTA computes goes to part_o / part_ml as part z = w - (first tile of the
// unit) / Q; the CTA that computes a unit's last tile marks the parts after its own as empty
// (maximum -inf), and llm_attention_merge reads `parts` of them per (row, head).  Q is chosen on
// the device (every CTA computes the same numbers from the rows' positions): the tiles per CTA,
// but never so few that a unit would need more than `parts` pieces.
// ---------------------------------------------------------------------------------------------
constexpr int PERSIST_MAX_ROWS = 256;

struct Cursor {       // a tile of the CTA's run and the unit it belongs to
  int r, kvh;         // request row and KV head
  int rel, t;         // tile of the unit counted from its first, tiles of the unit
  int first;          // the unit's first tile (lo / KT)
  int lo, hi, slot;   // lowest and highest position the row reads, its request slot
};

template <int HD, int KT, int STAGES>
__global__ void __launch_bounds__(32, 4) flash_decode_persistent_kernel(
    const __grid_constant__ CUtensorMap map_kv, const bf16* __restrict__ q, float* __restrict__ part_o,
    float* __restrict__ part_ml, const int* __restrict__ block_table, int table_stride,
    const int* __restrict__ row_slot, const int* __restrict__ row_pos, int rows, int Hq, int Hkv, int page_size,
    int n_slots, int slot, float scale_log2, int window, int parts, int* __restrict__ status) {
  constexpr int KS = HD / 16, MT = KT / 16, DM = HD / 16;
  constexpr int TILE_BYTES = KT * HD * 2;
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* kv_tiles = smem;                          // [STAGES][2 * TILE_BYTES]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * 2 * TILE_BYTES);
  int* s_pref = reinterpret_cast<int*>(full + STAGES);          // [rows + 1] tiles of the rows before
  int* s_pos = s_pref + PERSIST_MAX_ROWS + 1;
  int* s_slot = s_pos + PERSIST_MAX_ROWS;
  pdl_trigger();

  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  if (lane == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");

  // ---- every CTA: the tiles of every row (positions and slots are complete before the step's
  // first layer starts, so they are read before the wait), their running sum, the longest unit
  const int G = Hq / Hkv;
  constexpr int PER_LANE = PERSIST_MAX_ROWS / 32;
  int mine[PER_LANE], sum = 0, longest = 0;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int r = lane * PER_LANE + i;
    int tiles = 0;
    if (r < rows) {
      const int pos = row_pos[r];
      const int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
      tiles = pos / KT - lo / KT + 1;
      s_pos[r] = pos;
      s_slot[r] = row_slot[r];
    }
    mine[i] = tiles;
    sum += tiles;
    longest = max(longest, tiles);
  }
  int before = sum;                                   // inclusive scan over the lanes
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, before, o);
    if (lane >= o) before += v;
  }
  const int total_rows = __shfl_sync(0xffffffffu, before, 31);
  before -= sum;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int r = lane * PER_LANE + i;
    if (r <= rows) s_pref[r] = before;
    before += mine[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, o));
  __syncwarp();
  const long long T = (long long)total_rows * Hkv;    // tiles of all units
  long long Q = (T + gridDim.x - 1) / gridDim.x;
  const int least = (longest + parts - 2) / (parts - 1);        // a unit makes at most `parts` pieces
  if (Q < least) Q = least;
  const long long g0 = (long long)blockIdx.x * Q;
  const long long g1 = min(T, g0 + Q);
  if (g0 >= g1) return;

  const int R = page_size < KT ? page_size : KT;
  const int lgR = 31 - __clz(R);
  const int lgP = 31 - __clz(page_size);

  auto row_info = [&](int r, Cursor& c) {
    c.r = r;
    c.hi = s_pos[r];
    c.lo = (window > 0 && c.hi + 1 > window) ? c.hi + 1 - window : 0;
    c.first = c.lo / KT;
    c.t = c.hi / KT - c.first + 1;
    c.slot = s_slot[r];
  };
  auto locate = [&](long long gi, Cursor& c) {        // the tile numbered gi
    int a = 0, b = rows - 1;
    while (a < b) {
      const int mid = (a + b + 1) >> 1;
      if ((long long)s_pref[mid] * Hkv <= gi) a = mid; else b = mid - 1;
    }
    row_info(a, c);
    const int rem = (int)(gi - (long long)s_pref[a] * Hkv);
    c.kvh = rem / c.t;
    c.rel = rem % c.t;
  };
  auto advance = [&](Cursor& c) {
    if (++c.rel < c.t) return;
    c.rel = 0;
    if (++c.kvh < Hkv) return;
    c.kvh = 0;
    if (c.r + 1 < rows) row_info(c.r + 1, c);
  };

  // The producer keeps 32 entries of the current row's block table in the warp's lanes.
  int held_row = -1, held_from = 0, held = 0;
  auto load_tile = [&](const Cursor& c, int stage) {  // the whole warp calls it; lane 0 issues
    const int base = (c.first + c.rel) * KT;
    const int* table = block_table + (size_t)c.slot * table_stride;
    const int last_page = c.hi >> lgP;
    uint32_t bytes = 0;
    for (int p = base; p < base + KT; p += R)
      if (p <= c.hi && p + R - 1 >= c.lo) bytes += (uint32_t)R * HD * 2 * 2;
    if (lane == 0) mbar_expect_tx(&full[stage], bytes);
    for (int p = base; p < base + KT; p += R) {
      if (p > c.hi || p + R - 1 < c.lo) continue;
      const int pi = p >> lgP;
      if (held_row != c.r || pi < held_from || pi >= held_from + 32) {
        held_row = c.r;
        held_from = pi;
        held = pi + lane <= last_page ? table[pi + lane] : 0;
      }
      const int plane = (__shfl_sync(0xffffffffu, held, pi - held_from) * n_slots + slot) * 2;
      if (lane == 0)
        tma_load_5d(kv_tiles + stage * 2 * TILE_BYTES + ((p - base) >> lgR) * (2 * R * HD * 2), &map_kv, 0, 0,
                    p & (page_size - 1), c.kvh, plane, &full[stage]);
    }
  };

  Cursor prod, cons;
  locate(g0, prod);
  cons = prod;
  long long issued = g0;
  // tiles wholly below the row's new position hold nothing the kernel ahead writes
  while (issued < g1 && issued - g0 < STAGES && (prod.first + prod.rel + 1) * KT <= prod.hi) {
    load_tile(prod, (int)(issued - g0) % STAGES);
    advance(prod);
    ++issued;
  }
  pdl_wait();
  while (issued < g1 && issued - g0 < STAGES) {
    load_tile(prod, (int)(issued - g0) % STAGES);
    advance(prod);
    ++issued;
  }

  uint32_t qf[KS][2];
  float o[DM][4];
  float m[2], l[2];
  bool cvalid[2];
  size_t crow[2];
  bool fresh = true;
  bool alive = true;
  int n_it = 0;
  for (long long gi = g0; gi < g1; ++gi, ++n_it) {
    if (fresh) {                                   // a piece begins: this unit's queries, empty sums
      fresh = false;
      const bool valid = g < G;
      const bf16* src = q + ((size_t)cons.r * Hq + cons.kvh * G + (valid ? g : 0)) * HD + 2 * t;
#pragma unroll
      for (int k = 0; k < KS; ++k) {
        qf[k][0] = valid ? *reinterpret_cast<const uint32_t*>(src + k * 16) : 0u;
        qf[k][1] = valid ? *reinterpret_cast<const uint32_t*>(src + k * 16 + 8) : 0u;
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int n = 2 * t + j;
        cvalid[j] = n < G;
        crow[j] = (size_t)cons.r * Hq + cons.kvh * G + (cvalid[j] ? n : 0);
        m[j] = -INFINITY;
        l[j] = 0.f;
      }
#pragma unroll
      for (int d = 0; d < DM; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    }
    const int stage = n_it % STAGES;
    alive = mbar_wait(&full[stage], (uint32_t)(n_it / STAGES) & 1);
    alive = __all_sync(0xffffffffu, alive);
    if (!alive) {
      if (lane == 0) atomicExch(status, 5);
      break;
    }
    uint8_t* tile = kv_tiles + stage * 2 * TILE_BYTES;
    const int base = (cons.first + cons.rel) * KT;
    {
      // a page without a key of the row was not fetched: its values meet zero weights and must
      // be finite (its keys may be anything: their scores are replaced by -inf)
      for (int p = base; p < base + KT; p += R)
        if (p > cons.hi || p + R - 1 < cons.lo) {
          uint4* vz = reinterpret_cast<uint4*>(tile + ((p - base) >> lgR) * (2 * R * HD * 2) + R * HD * 2);
          for (int i = lane; i < R * HD * 2 / 16; i += 32) vz[i] = make_uint4(0, 0, 0, 0);
        }
      __syncwarp();
    }
    // ---- S^T = K Q^T
    float s[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) s[mt][0] = s[mt][1] = s[mt][2] = s[mt][3] = 0.f;
#pragma unroll
    for (int k = 0; k < KS; ++k) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t a[4];
        const int mi = lane >> 3;
        ldmatrix_x4(a, tile + tile_off<HD>(0, mt * 16 + (mi & 1) * 8 + (lane & 7), 2 * k + (mi >> 1), lgR));
        mma_bf16(s[mt], a, qf[k][0], qf[k][1]);
      }
    }
    // ---- mask, running maximum per pair, exponentials
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = e & 1;
        const int p = base + mt * 16 + g + 8 * (e >> 1);
        const bool vis = cvalid[j] && p <= cons.hi && p >= cons.lo;
        s[mt][e] = vis ? s[mt][e] * scale_log2 : -INFINITY;
        tmax[j] = fmaxf(tmax[j], s[mt][e]);
      }
    float corr[2], muse[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      tmax[j] = fmaxf(tmax[j], __shfl_xor_sync(0xffffffffu, tmax[j], 4));
      tmax[j] = fmaxf(tmax[j], __shfl_xor_sync(0xffffffffu, tmax[j], 8));
      tmax[j] = fmaxf(tmax[j], __shfl_xor_sync(0xffffffffu, tmax[j], 16));
      const float mnew = fmaxf(m[j], tmax[j]);
      muse[j] = mnew == -INFINITY ? 0.f : mnew;
      corr[j] = fast_exp2(m[j] - muse[j]);
      m[j] = mnew;
      l[j] *= corr[j];
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pexp = fast_exp2(s[mt][e] - muse[e & 1]);
        s[mt][e] = pexp;
        l[e & 1] += pexp;
      }
    if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
      for (int d = 0; d < DM; ++d) {
        o[d][0] *= corr[0]; o[d][1] *= corr[1];
        o[d][2] *= corr[0]; o[d][3] *= corr[1];
      }
    }
    // ---- O^T += V^T P^T
#pragma unroll
    for (int kk = 0; kk < MT; ++kk) {
      const uint32_t b0 = movmatrix_trans(pack_bf16(s[kk][0], s[kk][1]));
      const uint32_t b1 = movmatrix_trans(pack_bf16(s[kk][2], s[kk][3]));
#pragma unroll
      for (int d = 0; d < DM; ++d) {
        uint32_t a[4];
        const int mi = lane >> 3;
        ldmatrix_x4_trans(a, tile + tile_off<HD>(1, kk * 16 + (mi >> 1) * 8 + (lane & 7), 2 * d + (mi & 1), lgR));
        mma_bf16(o[d], a, b0, b1);
      }
    }
    __syncwarp();                  // every lane has read this stage
    if (issued < g1) {
      if (lane == 0) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      load_tile(prod, stage);
      advance(prod);
      ++issued;
    }
    // ---- the piece ends with the unit or with this CTA's run: its sums go out as one part
    const bool unit_end = cons.rel == cons.t - 1;
    if (unit_end || gi == g1 - 1) {
      const long long unit_first = (long long)s_pref[cons.r] * Hkv + (long long)cons.kvh * cons.t;
      const int z = (int)((long long)blockIdx.x - unit_first / Q);
      float lsum[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        lsum[j] = l[j];
        lsum[j] += __shfl_xor_sync(0xffffffffu, lsum[j], 4);
        lsum[j] += __shfl_xor_sync(0xffffffffu, lsum[j], 8);
        lsum[j] += __shfl_xor_sync(0xffffffffu, lsum[j], 16);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        if (!cvalid[j]) continue;
        float* dst = part_o + (crow[j] * parts + z) * HD;
#pragma unroll
        for (int d = 0; d < DM; ++d) {
          dst[d * 16 + g] = o[d][j];
          dst[d * 16 + g + 8] = o[d][2 + j];
        }
        if (g == 0) {
          part_ml[(crow[j] * parts + z) * 2] = m[j];
          part_ml[(crow[j] * parts + z) * 2 + 1] = lsum[j];
          if (unit_end)                            // no CTA computes a part after this one
            for (int zz = z + 1; zz < parts; ++zz) part_ml[(crow[j] * parts + zz) * 2] = -INFINITY;
        }
      }
      fresh = true;
    }
    advance(cons);
  }
  if (!alive)     // let the loads that are still in flight land before the shared memory goes
    for (int i = 0; i < STAGES; ++i) mbar_wait(&full[i], 0), mbar_wait(&full[i], 1);
}

template <int HD>
int launch_persistent(const CUtensorMap& map, const bf16* q, float* part_o, float* part_ml, const int* table,
                      int table_stride, const int* row_slot, const int* row_pos, int rows, int Hq, int Hkv,
                      int page_size, int n_slots, int slot, float scale, int window, int parts, int ctas,
                      int* status, cudaStream_t s) {
  constexpr int KT = DECODE_KT, STAGES = DECODE_STAGES;
  auto kernel = flash_decode_persistent_kernel<HD, KT, STAGES>;
  constexpr int smem = 2 * STAGES * KT * HD * 2 + STAGES * 8 + (3 * PERSIST_MAX_ROWS + 1) * 4 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return launch_pdl(kernel, dim3(ctas), 32, smem, s, map, q, part_o, part_ml, table, table_stride, row_slot,
                    row_pos, rows, Hq, Hkv, page_size, n_slots, slot, scale * 1.4426950408889634f, window, parts,
                    status);
}

template <int HD, bool FUSED>
int launch(const CUtensorMap& map, const bf16* q, bf16* out, float* part_o, float* part_ml, const int* table,
           int table_stride, const int* items, const int* row_slot, const int* row_pos, int n_items, int Hq,
           int Hkv, int page_size, int n_slots, int slot, float scale, int window, int splits, int* status,
           const Fused& fu, cudaStream_t s) {
  constexpr int KT = DECODE_KT, STAGES = DECODE_STAGES;
  auto kernel = flash_decode_tma_kernel<HD, KT, STAGES, FUSED>;
  constexpr int smem = 2 * STAGES * KT * HD * 2 + STAGES * 8 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(n_items, Hkv, splits);
  return launch_pdl(kernel, grid, 32, smem, s, map, q, out, part_o, part_ml, table, table_stride, items,
                    row_slot, row_pos, Hq, Hkv, page_size, n_slots, slot, scale * 1.4426950408889634f, window,
                    splits, status, fu);
}

int check_and_map(const void* storage, long long n_pages, int n_slots, int slot, int Hq, int Hkv, int hd,
                  int page_size, int splits, const float* part_o, const float* part_ml, CUtensorMap* map) {
  if (Hkv <= 0 || Hq % Hkv || splits < 1) return LLM_ERR_ARGUMENT;
  if (splits > 1 && (!part_o || !part_ml)) return LLM_ERR_ARGUMENT;
  if (hd != 64 && hd != 128) return LLM_ERR_UNSUPPORTED;
  if (!(DECODE_KT % page_size == 0 || page_size % DECODE_KT == 0)) return LLM_ERR_UNSUPPORTED;
  if (page_size & (page_size - 1)) return LLM_ERR_UNSUPPORTED;
  const long long planes = n_pages * n_slots * 2;
  if (planes >= (1LL << 31) || slot < 0 || slot >= n_slots) return LLM_ERR_UNSUPPORTED;
  // innermost first: 64 columns, the halves of a row, the positions of a page, the KV heads, the
  // K and V planes of every (page, cache slot)
  const int R = page_size < DECODE_KT ? page_size : DECODE_KT;
  const long long dims[5] = {64, hd / 64, page_size, Hkv, planes};
  const long long strides[4] = {128, (long long)hd * 2, (long long)page_size * hd * 2,
                                (long long)Hkv * page_size * hd * 2};
  const int box[5] = {64, hd / 64, R, 1, 2};
  return llm_tensor_map_tiled(storage, 5, dims, strides, box, map) ? 0 : LLM_ERR_UNSUPPORTED;
}
}  // namespace

// storage: the group's whole cache [n_pages][n_slots][2][Hkv][page_size][hd] bfloat16, contiguous;
// slot: the cache slot of this layer call.  page_size: a power of two.
// Other arguments as llm_attention_decode.
LLM_EXPORT int llm_attention_decode_tma(const void* q, void* out, float* part_o, float* part_ml,
                                        const void* storage, long long n_pages, int n_slots, int slot,
                                        const int* block_table, int table_stride, const int* items,
                                        const int* row_slot, const int* row_pos, int n_items, int Hq,
                                        int Hkv, int hd, int page_size, float scale, int window,
                                        int splits, int* status, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  CUtensorMap map;
  if (int e = check_and_map(storage, n_pages, n_slots, slot, Hq, Hkv, hd, page_size, splits, part_o, part_ml, &map))
    return e;
  const Fused none = {};
#define GO(HD)                                                                                          \
  return launch<HD, false>(map, (const bf16*)q, (bf16*)out, part_o, part_ml, block_table, table_stride,  \
                           items, row_slot, row_pos, n_items, Hq, Hkv, page_size, (int)n_slots, slot, scale, \
                           window, splits, status, none, stream)
  if (hd == 128) GO(128);
  GO(64);
#undef GO
}

// The persistent form for steps of single new tokens (see flash_decode_persistent_kernel): rows
// one-token items described by row_slot / row_pos, at most 256 of them and at most eight query
// heads per KV head.  It always writes `parts` parts per (row, head) into part_o / part_ml
// ([rows * Hq * parts][hd] and [...][2] floats; 2 <= parts <= 32), of which some are marked empty,
// and is followed by llm_attention_merge with splits = parts.  ctas: how many one-warp CTAs to
// launch (what the GPU holds at once: three per SM).
LLM_EXPORT int llm_attention_decode_persistent(const void* q, float* part_o, float* part_ml,
                                               const void* storage, long long n_pages, int n_slots,
                                               int slot, const int* block_table, int table_stride,
                                               const int* row_slot, const int* row_pos, int rows, int Hq,
                                               int Hkv, int hd, int page_size, float scale, int window,
                                               int parts, int ctas, int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!row_slot || !row_pos || parts < 2 || parts > 32 || ctas <= 0 || window < 0) return LLM_ERR_ARGUMENT;
  if (rows > PERSIST_MAX_ROWS || (Hkv > 0 && Hq / Hkv > 8)) return LLM_ERR_UNSUPPORTED;
  CUtensorMap map;
  if (int e = check_and_map(storage, n_pages, n_slots, slot, Hq, Hkv, hd, page_size, parts, part_o, part_ml, &map))
    return e;
#define GO(HD)                                                                                              \
  return launch_persistent<HD>(map, (const bf16*)q, part_o, part_ml, block_table, table_stride, row_slot,    \
                               row_pos, rows, Hq, Hkv, page_size, (int)n_slots, slot, scale, window, parts,   \
                               ctas, status, stream)
  if (hd == 128) GO(128);
  GO(64);
#undef GO
}

// The decode step's form: every row is one new token of its own request (row_slot, row_pos).
// proj [rows][proj_stride] is the 32-bit output of the q/k/v product (Hq heads of q, then, with
// k_cache given, Hkv heads of k and Hkv of v).  The kernel norms each head of q and k
// (q_norm_w / k_norm_w, 32-bit [hd], both or neither), rotates them whole by cos_sin
// [rows][hd/2] (cos, sin), writes the new key and value into k_cache / v_cache (the planes of
// this call's cache slot, pages page_stride elements apart) and attends.  With clear it zeroes
// what it consumed of proj, except the queries when splits > 1: several CTAs read those, and
// llm_attention_merge_clear zeroes them after all have.  The arithmetic of norm and rotation is
// that of llm_qk_norm_rope_store.
LLM_EXPORT int llm_attention_decode_fused(float* proj, int proj_stride, void* out, float* part_o,
                                          float* part_ml, const void* storage, long long n_pages,
                                          int n_slots, int slot, void* k_cache, void* v_cache,
                                          long long page_stride, const int* block_table,
                                          int table_stride, const int* row_slot, const int* row_pos,
                                          int rows, const float* q_norm_w, const float* k_norm_w,
                                          const float* cos_sin, float eps, int clear, int Hq, int Hkv,
                                          int hd, int page_size, float scale, int window, int splits,
                                          int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!proj || !cos_sin || !row_slot || !row_pos || (q_norm_w == nullptr) != (k_norm_w == nullptr) ||
      (k_cache == nullptr) != (v_cache == nullptr))
    return LLM_ERR_ARGUMENT;
  if (Hkv > 0 && Hq / Hkv > 8) return LLM_ERR_UNSUPPORTED;      // one token's heads are the eight columns
  if (proj_stride & 1) return LLM_ERR_UNSUPPORTED;               // 8-byte loads
  CUtensorMap map;
  if (int e = check_and_map(storage, n_pages, n_slots, slot, Hq, Hkv, hd, page_size, splits, part_o, part_ml, &map))
    return e;
  const Fused fu = {proj, proj_stride, q_norm_w, k_norm_w, reinterpret_cast<const float2*>(cos_sin),
                    (bf16*)k_cache, (bf16*)v_cache, page_stride, eps, clear};
#define GO(HD)                                                                                          \
  return launch<HD, true>(map, nullptr, (bf16*)out, part_o, part_ml, block_table, table_stride, nullptr,  \
                          row_slot, row_pos, rows, Hq, Hkv, page_size, (int)n_slots, slot, scale, window,   \
                          splits, status, fu, stream)
  if (hd == 128) GO(128);
  GO(64);
#undef GO
}
