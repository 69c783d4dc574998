// Per-head RMS norm of queries and keys, half-split rotation by absolute position, and the write
// of keys and values into the paged cache (a page holds, per KV head, its positions one after
// the other), in one pass over the projection output.
//   order per head: norm -> rotation -> store; values are stored as projected.
// All arithmetic is 32-bit; rounding to the cache / activation type happens once, at the store.
// On request the kernel clears the projection values it has consumed, so that the buffer is all
// zeros again when the next split-K product adds its partial sums into it.
#include "common.cuh"

namespace {
// One warp per (row, head).  Heads 0..Hq-1 are queries, Hq..Hq+Hkv-1 keys, then Hkv values.
// proj row layout: [Hq*hd | Hkv*hd | Hkv*hd] (keys and values absent when !has_kv).
template <typename TQ, typename TC>
__global__ void qk_norm_rope_store_kernel(
    const float* __restrict__ proj, int proj_stride, TQ* __restrict__ q_out,
    TC* __restrict__ k_cache, TC* __restrict__ v_cache, long long page_stride,
    const int* __restrict__ block_table, int table_stride, const int* __restrict__ row_slot,
    const int* __restrict__ row_pos, const float* __restrict__ q_norm_w,
    const float* __restrict__ k_norm_w, const float* __restrict__ inv_freq,
    const float2* __restrict__ cos_sin, float attn_factor, int rows, int Hq, int Hkv, int hd, int rot_dim,
    int page_size, float eps, int has_kv, int use_norm, int clear_proj) {
  pdl_trigger();
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int heads = Hq + (has_kv ? 2 * Hkv : 0);
  if (warp >= rows * heads) return;
  const int t = warp / heads, h = warp % heads;
  float* src = const_cast<float*>(proj) + (size_t)t * proj_stride + (size_t)h * hd;
  const int pos = row_pos[t];

  TC* cache_dst = nullptr;
  if (h >= Hq) {
    const int slot = row_slot[t];
    const int page = block_table[(size_t)slot * table_stride + pos / page_size];
    const int in_page = pos % page_size;
    const int kvh = (h - Hq) % Hkv;
    TC* base = (h < Hq + Hkv) ? k_cache : v_cache;
    cache_dst = base + (size_t)page * page_stride + ((size_t)kvh * page_size + in_page) * hd;
  }
  if (h >= Hq + Hkv) {  // value: copy
    for (int i = lane; i < hd; i += 32) {
      cache_dst[i] = from_f32<TC>(src[i]);
      if (clear_proj) src[i] = 0.f;
    }
    return;
  }
  const bool is_q = h < Hq;
  const float* w = is_q ? q_norm_w : k_norm_w;
  float scale = 1.f;
  if (use_norm) {
    float ss = 0.f;
    for (int i = lane; i < hd; i += 32) {
      const float v = src[i];
      ss += v * v;
    }
    ss = warp_sum(ss);
    scale = 1.0f / sqrtf(ss / (float)hd + eps);
  }
  const int half = rot_dim / 2;
  const float fpos = (float)pos;
  for (int i = lane; i < half; i += 32) {
    float a = src[i], b = src[i + half];
    if (clear_proj) src[i] = src[i + half] = 0.f;     // the next split-K product adds into zeros
    if (use_norm) {
      a = a * scale * w[i];
      b = b * scale * w[i + half];
    }
    float sn, cs;
    if (cos_sin) {      // made once per step for all heads and layers
      const float2 t2 = cos_sin[(size_t)t * half + i];
      cs = t2.x;
      sn = t2.y;
    } else {
      sincosf(fpos * inv_freq[i], &sn, &cs);
      sn *= attn_factor;
      cs *= attn_factor;
    }
    const float ra = a * cs - b * sn, rb = a * sn + b * cs;
    if (is_q) {
      q_out[(size_t)t * Hq * hd + (size_t)h * hd + i] = from_f32<TQ>(ra);
      q_out[(size_t)t * Hq * hd + (size_t)h * hd + i + half] = from_f32<TQ>(rb);
    } else {
      cache_dst[i] = from_f32<TC>(ra);
      cache_dst[i + half] = from_f32<TC>(rb);
    }
  }
  for (int i = rot_dim + lane; i < hd; i += 32) {  // dimensions beyond the rotated ones
    float a = src[i];
    if (clear_proj) src[i] = 0.f;
    if (use_norm) a = a * scale * w[i];
    if (is_q)
      q_out[(size_t)t * Hq * hd + (size_t)h * hd + i] = from_f32<TQ>(a);
    else
      cache_dst[i] = from_f32<TC>(a);
  }
}
}  // namespace

LLM_EXPORT int llm_qk_norm_rope_store(
    const float* proj, int proj_stride, void* q_out, void* k_cache, void* v_cache, int dtype,
    long long page_stride, const int* block_table, int table_stride, const int* row_slot,
    const int* row_pos, const float* q_norm_w, const float* k_norm_w, const float* inv_freq,
    const float* cos_sin, float attn_factor, int rows, int Hq, int Hkv, int hd, int rot_dim,
    int page_size, float eps, int has_kv, int use_norm, int clear_proj, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (rot_dim > hd || (rot_dim & 1)) return LLM_ERR_ARGUMENT;
  const int heads = Hq + (has_kv ? 2 * Hkv : 0);
  const long long warps = (long long)rows * heads;
  const int threads = 128;
  const int blocks = (int)((warps * 32 + threads - 1) / threads);
#define ARGS proj, proj_stride, (TQ*)q_out, (TQ*)k_cache, (TQ*)v_cache, page_stride, block_table, \
  table_stride, row_slot, row_pos, q_norm_w, k_norm_w, inv_freq, (const float2*)cos_sin, attn_factor, \
  rows, Hq, Hkv, hd, rot_dim, page_size, eps, has_kv, use_norm, clear_proj
  if (dtype == LLM_F32) {
    typedef float TQ;
    return launch_pdl(qk_norm_rope_store_kernel<float, float>, blocks, threads, 0, stream, ARGS);
  } else if (dtype == LLM_BF16) {
    typedef bf16 TQ;
    return launch_pdl(qk_norm_rope_store_kernel<bf16, bf16>, blocks, threads, 0, stream, ARGS);
  }
#undef ARGS
  return LLM_ERR_UNSUPPORTED;
}

namespace {
// cos_sin[t][i] = attn_factor * (cos, sin)(pos[t] * inv_freq[i]): the angles of a step, in 32-bit,
// computed once and shared by every head of every layer that uses this rotation.
__global__ void rope_table_kernel(const int* __restrict__ row_pos, const float* __restrict__ inv_freq,
                                  float2* __restrict__ cos_sin, int rows, int half, float attn_factor) {
  pdl_trigger();
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * half) return;
  const int t = idx / half, i = idx % half;
  float sn, cs;
  sincosf((float)row_pos[t] * inv_freq[i], &sn, &cs);
  cos_sin[idx] = make_float2(cs * attn_factor, sn * attn_factor);
}
}  // namespace

LLM_EXPORT int llm_rope_table(const int* row_pos, const float* inv_freq, float* cos_sin, int rows,
                              int half, float attn_factor, cudaStream_t stream) {
  const int total = rows * half;
  if (total <= 0) return 0;
  return launch_pdl(rope_table_kernel, (total + 255) / 256, 256, 0, stream, row_pos, inv_freq,
                    (float2*)cos_sin, rows, half, attn_factor);
}
