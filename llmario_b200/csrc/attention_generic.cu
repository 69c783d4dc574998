// Paged causal attention over the cache for any mix of rows: one warp per (row, query head).
//   s_p = dot(q, K[p]) * scale for the keys p of the row's own request with lo <= p <= pos,
//   lo = max(0, pos + 1 - window) when a window is set; softmax and the weighted sum of V in
//   32-bit with a running maximum.
// Keys are visited in tiles of 32 aligned to absolute positions, each lane scoring one key, so
// the order of every sum depends only on positions: the result for a row is the same however the
// tokens were cut into steps, whatever else is in the batch and whichever pages hold the keys.
// Any head size up to 256 that is a multiple of 8; any number of heads and groups.
#include "common.cuh"

namespace {
constexpr int MAX_HD = 256;
constexpr int WARPS = 4;

template <typename T> struct Vec8;  // 8 elements of T loaded at once
template <> struct Vec8<float> {
  float v[8];
  __device__ __forceinline__ void load(const float* p) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};
template <> struct Vec8<bf16> {
  float v[8];
  __device__ __forceinline__ void load(const bf16* p) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) attention_generic_kernel(
    const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ k_cache,
    const T* __restrict__ v_cache, long long page_stride, const int* __restrict__ block_table,
    int table_stride, const int* __restrict__ row_slot, const int* __restrict__ row_pos, int rows,
    int Hq, int Hkv, int hd, int page_size, float scale, int window) {
  __shared__ float q_s[WARPS][MAX_HD];
  const int warp_in_block = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + warp_in_block;
  if (item >= (long long)rows * Hq) return;
  const int t = (int)(item / Hq), h = (int)(item % Hq);
  const int kvh = h / (Hq / Hkv);
  const int pos = row_pos[t];
  const int* table = block_table + (size_t)row_slot[t] * table_stride;
  const int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;

  float* qs = q_s[warp_in_block];
  const T* qrow = q + ((size_t)t * Hq + h) * hd;
  for (int i = lane; i < hd; i += 32) qs[i] = to_f32(qrow[i]);
  __syncwarp();

  float m = -INFINITY, l = 0.f;
  float acc[MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) acc[i] = 0.f;

  for (int base = (lo / 32) * 32; base <= pos; base += 32) {
    const int p = base + lane;
    const bool valid = p >= lo && p <= pos;
    long long off = 0;  // element offset of this lane's key row inside the layer's cache
    float s = -INFINITY;
    if (valid) {
      const int page = table[p / page_size];
      off = (long long)page * page_stride + ((long long)kvh * page_size + p % page_size) * hd;
      const T* kr = k_cache + off;
      float d = 0.f;
      for (int i = 0; i < hd; i += 8) {
        Vec8<T> kv;
        kv.load(kr + i);
#pragma unroll
        for (int j = 0; j < 8; ++j) d = fmaf(qs[i + j], kv.v[j], d);
      }
      s = d * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float w = valid ? expf(s - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(w);
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; ++i) acc[i] *= corr;
    m = m_new;
    const unsigned mask = __ballot_sync(0xffffffffu, valid);
    for (int j = 0; j < 32; ++j) {
      if (!((mask >> j) & 1u)) continue;
      const float wj = __shfl_sync(0xffffffffu, w, j);
      const long long oj = __shfl_sync(0xffffffffu, off, j);
      const T* vr = v_cache + oj;
#pragma unroll
      for (int i = 0; i < MAX_HD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(wj, to_f32(vr[d]), acc[i]);
      }
    }
  }
  const float inv = 1.0f / l;
  T* orow = out + ((size_t)t * Hq + h) * hd;
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) orow[d] = from_f32<T>(acc[i] * inv);
  }
}
}  // namespace

LLM_EXPORT int llm_attention_generic(const void* q, void* out, const void* k_cache,
                                     const void* v_cache, int dtype, long long page_stride,
                                     const int* block_table, int table_stride, const int* row_slot,
                                     const int* row_pos, int rows, int Hq, int Hkv, int hd,
                                     int page_size, float scale, int window, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hd > MAX_HD || hd % 8 != 0 || Hkv <= 0 || Hq % Hkv != 0) return LLM_ERR_UNSUPPORTED;
  const long long items = (long long)rows * Hq;
  const int blocks = (int)((items + WARPS - 1) / WARPS);
  if (dtype == LLM_F32)
    attention_generic_kernel<float><<<blocks, WARPS * 32, 0, stream>>>(
        (const float*)q, (float*)out, (const float*)k_cache, (const float*)v_cache, page_stride,
        block_table, table_stride, row_slot, row_pos, rows, Hq, Hkv, hd, page_size, scale, window);
  else if (dtype == LLM_BF16)
    attention_generic_kernel<bf16><<<blocks, WARPS * 32, 0, stream>>>(
        (const bf16*)q, (bf16*)out, (const bf16*)k_cache, (const bf16*)v_cache, page_stride,
        block_table, table_stride, row_slot, row_pos, rows, Hq, Hkv, hd, page_size, scale, window);
  else
    return LLM_ERR_UNSUPPORTED;
  return launch_status();
}
