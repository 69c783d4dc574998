// Paged causal attention for bfloat16 with tensor cores: prompt portions and decode rows.
//
// A work item is a run of consecutive tokens of one request (a whole short portion, a slice of
// a long one, or a single decode token).  A CTA takes one item and one KV head; its rows are
// (token, query head of the group) pairs, so the K and V of the group are read once for all of
// its query heads.  Keys are walked in tiles aligned to absolute positions; K and V tiles come
// from the pages named by the block table through cp.async into swizzled shared memory, two
// stages deep.  S = Q K^T and O += P V run on mma.sync m16n8k16 with 32-bit accumulators; the
// softmax keeps a running maximum and sum per row in 32-bit (exp2 of scores pre-multiplied by
// log2 e).  A mask hides keys after the query, keys before the window and keys of other tiles'
// padding.  With splits > 1 the key range of an item is cut across blockIdx.z: every part
// writes an unnormalised sum with its maximum and weight to scratch memory and a second kernel
// merges them.
//
// Head sizes 32, 64 and 128; any number of heads and groups (the rows of a CTA are 16 per warp,
// a group larger than that is refused by the host and served by the generic kernel).
#include "attention_common.cuh"

namespace {

template <int HD, int WARPS, int KT>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 4 ? 3 : 6) flash_paged_kernel(
    const bf16* __restrict__ q, bf16* __restrict__ out, float* __restrict__ part_o,
    float* __restrict__ part_ml, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
    long long page_stride, const int* __restrict__ block_table, int table_stride,
    const int* __restrict__ items, const int* __restrict__ row_slot, const int* __restrict__ row_pos,
    int Hq, int Hkv, int page_size, float scale_log2, int window, int splits) {
  constexpr int CPR = HD / 8;            // 16-byte chunks per key row
  constexpr int KS = HD / 16;            // k-steps of Q K^T
  constexpr int NT = KT / 8;             // key n-tiles of S
  constexpr int DT = HD / 8;             // dim n-tiles of O
  extern __shared__ __align__(128) uint8_t smem_raw[];
  pdl_trigger();
  pdl_wait();
  bf16* ks = reinterpret_cast<bf16*>(smem_raw);               // [2][KT][HD]
  bf16* vs = ks + 2 * KT * HD;                                 // [2][KT][HD]

  // without a list of items every row of the step is an item of one token
  const Item it = items ? reinterpret_cast<const Item*>(items)[blockIdx.x]
                        : Item{(int)blockIdx.x, 1, row_slot[blockIdx.x], row_pos[blockIdx.x]};
  const int kvh = blockIdx.y, z = blockIdx.z;
  const int G = Hq / Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rows_valid = it.tokens * G;
  const int hi = it.pos_start + it.tokens - 1;
  const int lo = (window > 0 && it.pos_start + 1 > window) ? it.pos_start + 1 - window : 0;
  const int tile_first = lo / KT, tile_last = hi / KT;
  const int ntiles = tile_last - tile_first + 1;
  const int per = (ntiles + splits - 1) / splits;
  const int tb0 = tile_first + z * per;
  const int tb1 = min(tile_last + 1, tb0 + per);
  const int* table = block_table + (size_t)it.slot * table_stride;

  // this thread's two rows: r0 = warp*16 + g, r1 = r0 + 8
  int rtok[2], rhead[2], rpos[2], rlo[2];
  bool rvalid[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = warp * 16 + g + 8 * i;
    rvalid[i] = r < rows_valid;
    rtok[i] = rvalid[i] ? r / G : 0;
    rhead[i] = kvh * G + (rvalid[i] ? r % G : 0);
    rpos[i] = it.pos_start + rtok[i];
    rlo[i] = (window > 0 && rpos[i] + 1 > window) ? rpos[i] + 1 - window : 0;
  }

  // Q fragments, kept for the whole kernel
  uint32_t qf[KS][4];
#pragma unroll
  for (int k = 0; k < KS; ++k) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const bf16* src = q + ((size_t)(it.row_start + rtok[i]) * Hq + rhead[i]) * HD + k * 16 + 2 * t;
      qf[k][i] = rvalid[i] ? *reinterpret_cast<const uint32_t*>(src) : 0u;
      qf[k][i + 2] = rvalid[i] ? *reinterpret_cast<const uint32_t*>(src + 8) : 0u;
    }
  }

  float o[DT][4];
#pragma unroll
  for (int d = 0; d < DT; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  // A tile is filled page by page: one look-up in the block table per page, then the rows of
  // that page and KV head (consecutive positions, contiguous) in 16-byte pieces.  Rows outside the item's key range are cleared: their scores are masked,
  // but their values must be finite.
  auto load_tile = [&](int tb, int stage) {
    bf16* kd = ks + stage * KT * HD;
    bf16* vd = vs + stage * KT * HD;
    const int base = tb * KT;
    const int first = max(lo, base), last = min(hi, base + KT - 1);
    if (first > base || last < base + KT - 1) {
      for (int id = threadIdx.x; id < KT * CPR; id += WARPS * 32) {
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
      for (int id = threadIdx.x; id < run * CPR; id += WARPS * 32) {
        const int j = id / CPR, c = id % CPR;
        const int src = j * HD + c * 8;
        const int dst = (j0 + j) * HD + swizzle<CPR>(j0 + j, c) * 8;
        cp_async16(kd + dst, ksrc + src, true);
        cp_async16(vd + dst, vsrc + src, true);
      }
      p0 += run;
    }
  };

  if (tb0 < tb1) load_tile(tb0, 0);
  cp_async_commit();
  for (int tb = tb0; tb < tb1; ++tb) {
    const int stage = (tb - tb0) & 1;
    if (tb + 1 < tb1) load_tile(tb + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const bf16* kt = ks + stage * KT * HD;
    const bf16* vt = vs + stage * KT * HD;

    if (warp * 16 < rows_valid) {
      // ---- S = Q K^T
      float s[NT][4];
#pragma unroll
      for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
      // one ldmatrix feeds two key tiles at one k-step, so that consecutive MMAs write
      // different accumulators
#pragma unroll
      for (int k = 0; k < KS; ++k) {
#pragma unroll
        for (int n2 = 0; n2 < NT / 2; ++n2) {
          uint32_t b[4];
          const int mi = lane >> 3;
          const int row = (2 * n2 + (mi >> 1)) * 8 + (lane & 7), chunk = 2 * k + (mi & 1);
          ldmatrix_x4(b, kt + row * HD + swizzle<CPR>(row, chunk) * 8);
          mma_bf16(s[2 * n2], qf[k], b[0], b[1]);
          mma_bf16(s[2 * n2 + 1], qf[k], b[2], b[3]);
        }
      }
      // ---- mask, running maximum, exponentials
      const int base = tb * KT;
      const bool upper = warp * 16 + 8 < rows_valid;   // rows g + 8 of this warp hold queries
      // a tile that every row of this warp sees completely needs no mask
      const int wr0 = warp * 16, wr1 = min(rows_valid, wr0 + 16) - 1;
      const int min_pos = it.pos_start + wr0 / G, max_pos = it.pos_start + wr1 / G;
      const bool interior = base + KT - 1 <= min_pos &&
                            (window <= 0 || base >= max_pos + 1 - window) && wr1 - wr0 == 15;
      float tmax[2] = {-INFINITY, -INFINITY};
      if (interior) {
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s[n][e] *= scale_log2;
            tmax[e >> 1] = fmaxf(tmax[e >> 1], s[n][e]);
          }
      } else {
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = e >> 1;
            const int p = base + n * 8 + 2 * t + (e & 1);
            const bool vis = rvalid[i] && p <= rpos[i] && p >= rlo[i];
            s[n][e] = vis ? s[n][e] * scale_log2 : -INFINITY;
            tmax[i] = fmaxf(tmax[i], s[n][e]);
          }
      }
      float corr[2], muse[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 1));
        tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 2));
        const float mnew = fmaxf(m[i], tmax[i]);
        muse[i] = mnew == -INFINITY ? 0.f : mnew;
        corr[i] = fast_exp2(m[i] - muse[i]);   // m = -inf gives 0
        m[i] = mnew;
        l[i] *= corr[i];
      }
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pexp = (e < 2 || upper) ? fast_exp2(s[n][e] - muse[e >> 1]) : 0.f;
          s[n][e] = pexp;
          l[e >> 1] += pexp;
        }
      if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
        for (int d = 0; d < DT; ++d) {
          o[d][0] *= corr[0]; o[d][1] *= corr[0];
          o[d][2] *= corr[1]; o[d][3] *= corr[1];
        }
      }
      // ---- O += P V
#pragma unroll
      for (int kk = 0; kk < KT / 16; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int d2 = 0; d2 < DT / 2; ++d2) {
          uint32_t b[4];
          const int mi = lane >> 3;
          const int row = kk * 16 + (mi & 1) * 8 + (lane & 7), chunk = d2 * 2 + (mi >> 1);
          ldmatrix_x4_trans(b, vt + row * HD + swizzle<CPR>(row, chunk) * 8);
          mma_bf16(o[2 * d2], a, b[0], b[1]);
          mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  // ---- finish: the row sums are spread over the four threads of a row
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!rvalid[i]) continue;
    const size_t rowhead = (size_t)(it.row_start + rtok[i]) * Hq + rhead[i];
    if (splits == 1) {
      const float inv = 1.0f / l[i];
      bf16* dst = out + rowhead * HD;
#pragma unroll
      for (int d = 0; d < DT; ++d)
        *reinterpret_cast<uint32_t*>(dst + d * 8 + 2 * t) =
            pack_bf16(o[d][2 * i] * inv, o[d][2 * i + 1] * inv);
    } else {
      float* dst = part_o + (rowhead * splits + z) * HD;
#pragma unroll
      for (int d = 0; d < DT; ++d)
        *reinterpret_cast<float2*>(dst + d * 8 + 2 * t) = make_float2(o[d][2 * i], o[d][2 * i + 1]);
      if (t == 0) {
        part_ml[(rowhead * splits + z) * 2] = m[i];
        part_ml[(rowhead * splits + z) * 2 + 1] = l[i];
      }
    }
  }
}

// out[row][head] = sum_z 2^(m_z - m*) o_z / sum_z 2^(m_z - m*) l_z   over the parts of a row
template <int HD>
__global__ void merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                             bf16* __restrict__ out, const int* __restrict__ rows, int Hq, int splits,
                             float* __restrict__ clear, int clear_stride) {
  pdl_trigger();
  pdl_wait();
  const int row = rows ? rows[blockIdx.x] : (int)blockIdx.x;
  const size_t rowhead = (size_t)row * Hq + blockIdx.y;
  if (clear)      // the head's queries in the projection buffer, which every part has read by now
    for (int d = threadIdx.x; d < HD; d += blockDim.x)
      clear[(size_t)row * clear_stride + blockIdx.y * HD + d] = 0.f;
  float mstar = -INFINITY;
  for (int z = 0; z < splits; ++z) mstar = fmaxf(mstar, part_ml[(rowhead * splits + z) * 2]);
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float acc = 0.f, lsum = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float mz = part_ml[(rowhead * splits + z) * 2];
      if (mz == -INFINITY) continue;      // a part without keys: what lies in its place is not read
      const float w = exp2f(mz - mstar);
      acc += w * part_o[(rowhead * splits + z) * HD + d];
      lsum += w * part_ml[(rowhead * splits + z) * 2 + 1];
    }
    out[rowhead * HD + d] = __float2bfloat16_rn(acc / lsum);
  }
}

template <int HD, int WARPS, int KT>
int launch(const bf16* q, bf16* out, float* part_o, float* part_ml, const bf16* kc, const bf16* vc,
           long long page_stride, const int* table, int table_stride, const int* items,
           const int* row_slot, const int* row_pos, int n_items, int Hq, int Hkv, int page_size,
           float scale, int window, int splits, cudaStream_t s) {
  auto kernel = flash_paged_kernel<HD, WARPS, KT>;
  constexpr int smem = 4 * KT * HD * 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(n_items, Hkv, splits);
  return launch_pdl(kernel, grid, WARPS * 32, smem, s, q, out, part_o, part_ml, kc, vc, page_stride, table,
                    table_stride, items, row_slot, row_pos, Hq, Hkv, page_size,
                    scale * 1.4426950408889634f, window, splits);
}
}  // namespace

// items: n_items x (first row, tokens, request slot, first position) int32 on the device; when
// null, every one of the n_items rows is an item of one token described by row_slot / row_pos.
// rows_per_cta 16: one warp per CTA (decode rows and very short portions, tokens * group <= 16);
// rows_per_cta 64: four warps (tokens * group <= 64).  splits > 1 needs part_o
// [rows*Hq*splits*hd] and part_ml [rows*Hq*splits*2] float scratch and is followed by
// llm_attention_merge over the same rows.
LLM_EXPORT int llm_attention_flash(const void* q, void* out, float* part_o, float* part_ml,
                                   const void* k_cache, const void* v_cache, long long page_stride,
                                   const int* block_table, int table_stride, const int* items,
                                   const int* row_slot, const int* row_pos, int n_items,
                                   int rows_per_cta, int Hq, int Hkv, int hd,
                                   int page_size, float scale, int window, int splits,
                                   cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (Hkv <= 0 || Hq <= 0 || Hq % Hkv || splits < 1 || splits > 65535 || page_size <= 0 || window < 0)
    return LLM_ERR_ARGUMENT;
  if (splits > 1 && (!part_o || !part_ml)) return LLM_ERR_ARGUMENT;
  // a CTA holds rows_per_cta (token, head) pairs and every head of a group belongs to one CTA:
  // a larger group would leave heads uncomputed
  if (Hq / Hkv > rows_per_cta) return LLM_ERR_UNSUPPORTED;
#define GO(HD, W, KT)                                                                                 \
  return launch<HD, W, KT>((const bf16*)q, (bf16*)out, part_o, part_ml, (const bf16*)k_cache,          \
                           (const bf16*)v_cache, page_stride, block_table, table_stride, items, row_slot, \
                           row_pos, n_items,                                                          \
                           Hq, Hkv, page_size, scale, window, splits, stream)
  if (rows_per_cta == 16) {
    if (hd == 128) GO(128, 1, 32);
    if (hd == 64) GO(64, 1, 32);
    if (hd == 32) GO(32, 1, 32);
  } else if (rows_per_cta == 64) {
    if (hd == 128) GO(128, 4, 64);
    if (hd == 64) GO(64, 4, 64);
    if (hd == 32) GO(32, 4, 64);
  }
#undef GO
  return LLM_ERR_UNSUPPORTED;
}

// Merge of the parts of split keys.  With clear given, also clear[row][head * hd .. + hd) = 0 for
// every merged (row, head): the queries that llm_attention_decode_fused leaves in the projection
// buffer when it splits the keys.
LLM_EXPORT int llm_attention_merge_clear(const float* part_o, const float* part_ml, void* out,
                                         const int* rows, int n_rows, int Hq, int hd, int splits,
                                         float* clear, int clear_stride, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  dim3 grid(n_rows, Hq);
  if (hd == 128) return launch_pdl(merge_kernel<128>, grid, 128, 0, stream, part_o, part_ml, (bf16*)out, rows, Hq, splits, clear, clear_stride);
  if (hd == 64) return launch_pdl(merge_kernel<64>, grid, 64, 0, stream, part_o, part_ml, (bf16*)out, rows, Hq, splits, clear, clear_stride);
  if (hd == 32) return launch_pdl(merge_kernel<32>, grid, 32, 0, stream, part_o, part_ml, (bf16*)out, rows, Hq, splits, clear, clear_stride);
  return LLM_ERR_UNSUPPORTED;
}

LLM_EXPORT int llm_attention_merge(const float* part_o, const float* part_ml, void* out,
                                   const int* rows, int n_rows, int Hq, int hd, int splits,
                                   cudaStream_t stream) {
  return llm_attention_merge_clear(part_o, part_ml, out, rows, n_rows, Hq, hd, splits, nullptr, 0, stream);
}

// ------------------------------------------------------------------------------------------------
// Decode attention with built-in scratch memory (declared in no_alloc.h).
//
// llm_attention_flash with split keys needs two float buffers that its caller allocates.  Some
// callers of this library cannot allocate device memory at the moment they need attention: an
// engine whose memory planner handed out every byte of the GPU before the first token (the
// reference plans every byte before it loads a model, crates/engine/plan), a serving loop that
// may not take the device-wide stall a cudaMalloc can cause, or a host that keeps all CUDA
// allocation inside another framework's pool and forbids it elsewhere.  For them this one entry
// point keeps its partial sums in a fixed array that is part of the library image: every GPU
// that loads the library carries these 8 MiB until the process exits.
//
// * Limit: rows * Hq * splits * (hd + 2) floats must fit NO_ALLOC_SCRATCH_FLOATS (2 Mi floats);
//   a larger request returns LLM_ERR_TOO_LARGE and launches nothing.
// * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//   that device current) and remembers it.  Make that first call outside any stream capture.
// * It calls no cudaMalloc, cudaFree or other allocating routine.
// * All calls share the one array and it keeps what the last call left.  Nothing in it has to
//   start at zero: every (row, head, part) cell that the merge reads is written by the first
//   kernel of the same call, parts without keys included.  Two calls that overlap on the GPU
//   (different streams) race on it: order them.
// * The remembered address (one per device) is written without a lock.  Two host threads that
//   make their first call on a device at the same time both look the address up and store the
//   same value, which is harmless.
// * Refused before anything is launched: more than 16 query heads per KV head (LLM_ERR_UNSUPPORTED;
//   one warp holds a group's heads), a head size other than 32, 64 or 128, a page size or
//   number of parts that is not positive, a negative window, more than 65535 parts.
// ------------------------------------------------------------------------------------------------
#include "no_alloc.h"

static __device__ __align__(256) float g_no_alloc_scratch[NO_ALLOC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_scratch_address[MAX_DEVICES] = {nullptr};

// The array's name is a host-side handle, not a device pointer: a kernel must be given the
// address that the runtime reports for the current device.
int scratch_address(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= MAX_DEVICES) return LLM_ERR_UNSUPPORTED;
  if (!g_scratch_address[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_no_alloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_scratch_address[dev] = p;
  }
  *out = g_scratch_address[dev];
  return 0;
}
}  // namespace

LLM_EXPORT int llm_attention_decode_no_alloc(const void* q, void* out, const void* k_cache,
                                             const void* v_cache, long long page_stride,
                                             const int* block_table, int table_stride,
                                             const int* row_slot, const int* row_pos, int rows,
                                             int Hq, int Hkv, int hd, int page_size, float scale,
                                             int window, int splits, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (Hkv <= 0 || Hq <= 0 || Hq % Hkv || splits < 1 || splits > 65535 || hd <= 0 || page_size <= 0 ||
      window < 0)
    return LLM_ERR_ARGUMENT;
  // one warp per (row, KV head) holds 16 (token, head) pairs: a group of more than 16 query heads
  // on a KV head would leave heads uncomputed, so it is refused before anything is launched
  if (Hq / Hkv > 16 || (hd != 128 && hd != 64 && hd != 32)) return LLM_ERR_UNSUPPORTED;
  const long long need = (long long)rows * Hq * splits * (hd + 2);
  if (need > (long long)NO_ALLOC_SCRATCH_FLOATS) return LLM_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int st = scratch_address(&scratch);
  if (st != 0) return st;
  float* part_o = scratch;                                        // [rows*Hq*splits][hd]
  float* part_ml = scratch + (size_t)rows * Hq * splits * hd;     // [rows*Hq*splits][2]
  int r;
#define GO(HD)                                                                                        \
  r = launch<HD, 1, 32>((const bf16*)q, (bf16*)out, part_o, part_ml, (const bf16*)k_cache,             \
                        (const bf16*)v_cache, page_stride, block_table, table_stride, nullptr, row_slot, \
                        row_pos, rows, Hq, Hkv, page_size, scale, window, splits, stream)
  if (hd == 128) GO(128);
  else if (hd == 64) GO(64);
  else if (hd == 32) GO(32);
  else return LLM_ERR_UNSUPPORTED;
#undef GO
  if (r != 0 || splits == 1) return r;
  return llm_attention_merge(part_o, part_ml, out, nullptr, rows, Hq, hd, splits, stream);
}
