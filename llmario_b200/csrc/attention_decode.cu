// Paged attention for decode rows (bfloat16): keys on the M side of the tensor-core tile.
//
// A work item has at most eight (token, query head) pairs: one decode token of a group of up to
// eight heads, or two tokens of a group of four.  The pairs are the eight columns of
// mma.sync m16n8k16:
//     S^T [keys x pairs] = K [keys x hd] . Q^T [hd x pairs]          (K is the A operand)
//     O^T [hd x pairs]  += V^T [hd x keys] . P^T [keys x pairs]      (V^T is the A operand)
// so no tensor-core row is spent on padding (the row-major form of attention_flash.cu uses 16
// query rows per warp, of which a decode step fills four) and the accumulators take a quarter of
// the registers.  P^T reaches the B-operand layout by one movmatrix transpose per eight keys.
// The running maximum and sum are kept per pair in 32-bit; keys are walked in tiles of 32
// aligned to absolute positions and can be split across blockIdx.z with the partial results
// merged by llm_attention_merge.
//
// One warp per CTA; K and V tiles arrive by cp.async, page by page, through a ring of stages
// (more than two did not pay: fewer CTAs fit an SM).
#include "attention_common.cuh"

namespace {

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}

template <int HD, int KT, int STAGES>
__global__ void __launch_bounds__(32, 6) flash_decode_kernel(
    const bf16* __restrict__ q, bf16* __restrict__ out, float* __restrict__ part_o,
    float* __restrict__ part_ml, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
    long long page_stride, const int* __restrict__ block_table, int table_stride,
    const int* __restrict__ items, const int* __restrict__ row_slot, const int* __restrict__ row_pos,
    int Hq, int Hkv, int page_size, float scale_log2, int window, int splits) {
  constexpr int CPR = HD / 8;            // 16-byte chunks per key row
  constexpr int KS = HD / 16;            // k-steps of K Q^T
  constexpr int MT = KT / 16;            // key m-tiles of S^T
  constexpr int DM = HD / 16;            // dim m-tiles of O^T
  extern __shared__ __align__(128) uint8_t smem_raw[];
  pdl_trigger();
  pdl_wait();
  bf16* ks = reinterpret_cast<bf16*>(smem_raw);               // [STAGES][KT][HD]
  bf16* vs = ks + STAGES * KT * HD;                            // [STAGES][KT][HD]

  const Item it = items ? reinterpret_cast<const Item*>(items)[blockIdx.x]
                        : Item{(int)blockIdx.x, 1, row_slot[blockIdx.x], row_pos[blockIdx.x]};
  const int kvh = blockIdx.y, z = blockIdx.z;
  const int G = Hq / Hkv;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int pairs = it.tokens * G;                 // <= 8
  const int hi = it.pos_start + it.tokens - 1;
  const int lo = (window > 0 && it.pos_start + 1 > window) ? it.pos_start + 1 - window : 0;
  const int tile_first = lo / KT, tile_last = hi / KT;
  const int ntiles = tile_last - tile_first + 1;
  const int per = (ntiles + splits - 1) / splits;
  const int tb0 = tile_first + z * per;
  const int tb1 = min(tile_last + 1, tb0 + per);
  const int* table = block_table + (size_t)it.slot * table_stride;

  // the two columns (pairs) of the accumulators this thread holds: 2t and 2t + 1
  int cpos[2], clo[2];
  bool cvalid[2];
  size_t crow[2];       // (row * Hq + head) of the pair
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int n = 2 * t + j;
    cvalid[j] = n < pairs;
    const int tok = cvalid[j] ? n / G : 0, head = kvh * G + (cvalid[j] ? n % G : 0);
    cpos[j] = it.pos_start + tok;
    clo[j] = (window > 0 && cpos[j] + 1 > window) ? cpos[j] + 1 - window : 0;
    crow[j] = (size_t)(it.row_start + tok) * Hq + head;
  }
  // Q^T as the B operand: this thread supplies pair n = g
  uint32_t qf[KS][2];
  {
    const bool valid = g < pairs;
    const int tok = valid ? g / G : 0, head = kvh * G + (valid ? g % G : 0);
    const bf16* src = q + ((size_t)(it.row_start + tok) * Hq + head) * HD + 2 * t;
#pragma unroll
    for (int k = 0; k < KS; ++k) {
      qf[k][0] = valid ? *reinterpret_cast<const uint32_t*>(src + k * 16) : 0u;
      qf[k][1] = valid ? *reinterpret_cast<const uint32_t*>(src + k * 16 + 8) : 0u;
    }
  }

  float o[DM][4];
#pragma unroll
  for (int d = 0; d < DM; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  auto load_tile = [&](int tb, int stage) {
    bf16* kd = ks + stage * KT * HD;
    bf16* vd = vs + stage * KT * HD;
    const int base = tb * KT;
    const int first = max(lo, base), last = min(hi, base + KT - 1);
    if (first > base || last < base + KT - 1) {     // rows without a key: finite values
      for (int id = lane; id < KT * CPR; id += 32) {
        const int j = id / CPR, c = id % CPR;
        if (base + j < first || base + j > last) {
          const int dst = j * HD + swizzle<CPR>(j, c) * 8;
          *reinterpret_cast<uint4*>(kd + dst) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(vd + dst) = make_uint4(0, 0, 0, 0);
        }
      }
    }
    for (int p0 = first; p0 <= last;) {
      const int pg = p0 / page_size;
      const int in_page = p0 - pg * page_size;
      const int run = min(page_size - in_page, last - p0 + 1);
      const long long off = (long long)table[pg] * page_stride + ((long long)kvh * page_size + in_page) * HD;
      const bf16* ksrc = k_cache + off;
      const bf16* vsrc = v_cache + off;
      const int j0 = p0 - base;
      for (int id = lane; id < run * CPR; id += 32) {
        const int j = id / CPR, c = id % CPR;
        const int src = j * HD + c * 8;
        const int dst = (j0 + j) * HD + swizzle<CPR>(j0 + j, c) * 8;
        cp_async16(kd + dst, ksrc + src, true);
        cp_async16(vd + dst, vsrc + src, true);
      }
      p0 += run;
    }
  };

  // STAGES - 1 tiles are requested ahead of the one being multiplied
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {
    if (tb0 + i < tb1) load_tile(tb0 + i, i);
    cp_async_commit();
  }
  for (int tb = tb0; tb < tb1; ++tb) {
    const int stage = (tb - tb0) % STAGES;
    if (tb + STAGES - 1 < tb1) load_tile(tb + STAGES - 1, (tb - tb0 + STAGES - 1) % STAGES);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncwarp();
    const bf16* kt = ks + stage * KT * HD;
    const bf16* vt = vs + stage * KT * HD;

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
        const int row = mt * 16 + (mi & 1) * 8 + (lane & 7), chunk = 2 * k + (mi >> 1);
        ldmatrix_x4(a, kt + row * HD + swizzle<CPR>(row, chunk) * 8);
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
      // P^T of these 16 keys into the B-operand layout: (keys 2t, 2t+1 ; pair g)
      const uint32_t b0 = movmatrix_trans(pack_bf16(s[kk][0], s[kk][1]));
      const uint32_t b1 = movmatrix_trans(pack_bf16(s[kk][2], s[kk][3]));
#pragma unroll
      for (int d = 0; d < DM; ++d) {
        uint32_t a[4];
        const int mi = lane >> 3;
        const int row = kk * 16 + (mi >> 1) * 8 + (lane & 7), chunk = 2 * d + (mi & 1);
        ldmatrix_x4_trans(a, vt + row * HD + swizzle<CPR>(row, chunk) * 8);
        mma_bf16(o[d], a, b0, b1);
      }
    }
    __syncwarp();
  }
  cp_async_wait<0>();

  // ---- finish: the sums of a pair are spread over the eight lanes with the same t
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

template <int HD>
int launch(const bf16* q, bf16* out, float* part_o, float* part_ml, const bf16* kc, const bf16* vc,
           long long page_stride, const int* table, int table_stride, const int* items,
           const int* row_slot, const int* row_pos, int n_items, int Hq, int Hkv, int page_size,
           float scale, int window, int splits, cudaStream_t s) {
  constexpr int KT = 32, STAGES = 2;
  auto kernel = flash_decode_kernel<HD, KT, STAGES>;
  constexpr int smem = 2 * STAGES * KT * HD * 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(n_items, Hkv, splits);
  return launch_pdl(kernel, grid, 32, smem, s, q, out, part_o, part_ml, kc, vc, page_stride, table,
                    table_stride, items, row_slot, row_pos, Hq, Hkv, page_size,
                    scale * 1.4426950408889634f, window, splits);
}
}  // namespace

// Items of at most eight (token, head of the group) pairs: tokens * (Hq / Hkv) <= 8.  Arguments as
// llm_attention_flash; with splits > 1 follow with llm_attention_merge.
LLM_EXPORT int llm_attention_decode(const void* q, void* out, float* part_o, float* part_ml,
                                    const void* k_cache, const void* v_cache, long long page_stride,
                                    const int* block_table, int table_stride, const int* items,
                                    const int* row_slot, const int* row_pos, int n_items, int Hq,
                                    int Hkv, int hd, int page_size, float scale, int window,
                                    int splits, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv || splits < 1) return LLM_ERR_ARGUMENT;
  if (splits > 1 && (!part_o || !part_ml)) return LLM_ERR_ARGUMENT;
#define GO(HD)                                                                                       \
  return launch<HD>((const bf16*)q, (bf16*)out, part_o, part_ml, (const bf16*)k_cache,                 \
                    (const bf16*)v_cache, page_stride, block_table, table_stride, items, row_slot,     \
                    row_pos, n_items, Hq, Hkv, page_size, scale, window, splits, stream)
  if (hd == 128) GO(128);
  if (hd == 64) GO(64);
  if (hd == 32) GO(32);
#undef GO
  return LLM_ERR_UNSUPPORTED;
}
