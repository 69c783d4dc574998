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
  // grid: (rows, groups of four heads); no division on the way to (row, head)
  const int t = blockIdx.x;
  const int h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = Hq + (has_kv ? 2 * Hkv : 0);
  if (h >= heads) return;
  float* src = const_cast<float*>(proj) + (size_t)t * proj_stride + h * hd;
  const int pos = row_pos[t];

  TC* cache_dst = nullptr;
  if (h >= Hq) {
    const int slot = row_slot[t];
    // pages usually hold a power of two of positions: shift and mask then
    const bool pow2 = (page_size & (page_size - 1)) == 0;
    const int page_index = pow2 ? pos >> (31 - __clz(page_size)) : pos / page_size;
    const int in_page = pow2 ? pos & (page_size - 1) : pos - page_index * page_size;
    const int page = block_table[(size_t)slot * table_stride + page_index];
    const bool is_k = h < Hq + Hkv;
    const int kvh = is_k ? h - Hq : h - Hq - Hkv;
    TC* base = is_k ? k_cache : v_cache;
    cache_dst = base + (size_t)page * page_stride + (size_t)(kvh * page_size + in_page) * hd;
  }
  if (h >= Hq + Hkv) {  // value: copy
    if (hd == 128 && sizeof(TC) == 2 && !(proj_stride & 3)) {      // four elements per lane
      const float4 v4 = *reinterpret_cast<const float4*>(src + 4 * lane);
      if (clear_proj) *reinterpret_cast<float4*>(src + 4 * lane) = make_float4(0.f, 0.f, 0.f, 0.f);
      __nv_bfloat162 p0 = __floats2bfloat162_rn(v4.x, v4.y), p1 = __floats2bfloat162_rn(v4.z, v4.w);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&p0);
      packed.y = *reinterpret_cast<uint32_t*>(&p1);
      *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(cache_dst) + 4 * lane) = packed;
      return;
    }
    for (int i = lane; i < hd; i += 32) {
      cache_dst[i] = from_f32<TC>(src[i]);
      if (clear_proj) src[i] = 0.f;
    }
    return;
  }
  const bool is_q = h < Hq;
  const float* w = is_q ? q_norm_w : k_norm_w;
  if (hd == 128 && rot_dim == 128 && cos_sin && sizeof(TQ) == 2 && sizeof(TC) == 2 && !(proj_stride & 1)) {
    // The common shape, two elements per lane and half: lane l holds elements 2l, 2l+1 and
    // 64+2l, 65+2l, i.e. the rotation pairs (2l, 64+2l) and (2l+1, 65+2l); 8-byte loads, one
    // 16-byte load of both pairs' cosine and sine, 4-byte stores of two bfloat16 values.
    const float2 lo = *reinterpret_cast<const float2*>(src + 2 * lane);
    const float2 hi = *reinterpret_cast<const float2*>(src + 64 + 2 * lane);
    if (clear_proj) {
      *reinterpret_cast<float2*>(src + 2 * lane) = make_float2(0.f, 0.f);
      *reinterpret_cast<float2*>(src + 64 + 2 * lane) = make_float2(0.f, 0.f);
    }
    float a0 = lo.x, a1 = lo.y, b0 = hi.x, b1 = hi.y;
    if (use_norm) {
      const float ss = warp_sum(a0 * a0 + a1 * a1 + b0 * b0 + b1 * b1);
      const float scale = 1.0f / sqrtf(ss / 128.0f + eps);
      const float2 wl = *reinterpret_cast<const float2*>(w + 2 * lane);
      const float2 wh = *reinterpret_cast<const float2*>(w + 64 + 2 * lane);
      a0 = a0 * scale * wl.x, a1 = a1 * scale * wl.y, b0 = b0 * scale * wh.x, b1 = b1 * scale * wh.y;
    }
    const float4 cs = *reinterpret_cast<const float4*>(cos_sin + (size_t)t * 64 + 2 * lane);   // (cos, sin) x 2
    const float ra0 = a0 * cs.x - b0 * cs.y, rb0 = a0 * cs.y + b0 * cs.x;
    const float ra1 = a1 * cs.z - b1 * cs.w, rb1 = a1 * cs.w + b1 * cs.z;
    bf16* dst = is_q ? reinterpret_cast<bf16*>(q_out) + (size_t)t * Hq * 128 + (size_t)h * 128
                     : reinterpret_cast<bf16*>(cache_dst);
    *reinterpret_cast<__nv_bfloat162*>(dst + 2 * lane) = __floats2bfloat162_rn(ra0, ra1);
    *reinterpret_cast<__nv_bfloat162*>(dst + 64 + 2 * lane) = __floats2bfloat162_rn(rb0, rb1);
    return;
  }
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

// The same for many rows of the common shape (head size 128 rotated whole, cosines and sines from
// the step's table, 16-bit activations and cache): a warp takes FOUR heads of a row and asks for
// all their values before it works on any, and the row's position, request slot and page are
// looked up once.  With one head per warp the kernel waits on a chain of dependent loads per head
// and moves about 2 TB/s; this form keeps four times as many bytes in flight.
// grid: (rows, groups of 16 heads), 128 threads.
__global__ void __launch_bounds__(128) qk_norm_rope_store_rows_kernel(
    const float* __restrict__ proj, int proj_stride, bf16* __restrict__ q_out, bf16* __restrict__ k_cache,
    bf16* __restrict__ v_cache, long long page_stride, const int* __restrict__ block_table, int table_stride,
    const int* __restrict__ row_slot, const int* __restrict__ row_pos, const float* __restrict__ q_norm_w,
    const float* __restrict__ k_norm_w, const float2* __restrict__ cos_sin, int Hq, int Hkv, int page_size,
    float eps, int has_kv, int use_norm) {
  constexpr int HD = 128;
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int h0 = blockIdx.y * 16 + (threadIdx.x >> 5) * 4;
  const int heads = Hq + (has_kv ? 2 * Hkv : 0);
  if (h0 >= heads) return;
  const float* row = proj + (size_t)t * proj_stride;
  float2 lo[4], hi[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (h0 + j < heads) {
      lo[j] = *reinterpret_cast<const float2*>(row + (h0 + j) * HD + 2 * lane);
      hi[j] = *reinterpret_cast<const float2*>(row + (h0 + j) * HD + 64 + 2 * lane);
    }
  const int pos = row_pos[t];
  const float4 cs = *reinterpret_cast<const float4*>(cos_sin + (size_t)t * 64 + 2 * lane);   // (cos, sin) x 2
  size_t page_off = 0;
  int in_page = 0;
  if (has_kv && h0 + 3 >= Hq) {
    const bool pow2 = (page_size & (page_size - 1)) == 0;
    const int page_index = pow2 ? pos >> (31 - __clz(page_size)) : pos / page_size;
    in_page = pow2 ? pos & (page_size - 1) : pos - page_index * page_size;
    page_off = (size_t)block_table[(size_t)row_slot[t] * table_stride + page_index] * page_stride;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int h = h0 + j;
    if (h >= heads) break;
    float a0 = lo[j].x, a1 = lo[j].y, b0 = hi[j].x, b1 = hi[j].y;
    if (h >= Hq + Hkv) {                                   // a value head: stored as projected
      bf16* dst = v_cache + page_off + (size_t)((h - Hq - Hkv) * page_size + in_page) * HD;
      *reinterpret_cast<__nv_bfloat162*>(dst + 2 * lane) = __floats2bfloat162_rn(a0, a1);
      *reinterpret_cast<__nv_bfloat162*>(dst + 64 + 2 * lane) = __floats2bfloat162_rn(b0, b1);
      continue;
    }
    const bool is_q = h < Hq;
    if (use_norm) {
      const float* w = is_q ? q_norm_w : k_norm_w;
      const float ss = warp_sum(a0 * a0 + a1 * a1 + b0 * b0 + b1 * b1);
      const float scale = 1.0f / sqrtf(ss / 128.0f + eps);
      const float2 wl = *reinterpret_cast<const float2*>(w + 2 * lane);
      const float2 wh = *reinterpret_cast<const float2*>(w + 64 + 2 * lane);
      a0 = a0 * scale * wl.x, a1 = a1 * scale * wl.y, b0 = b0 * scale * wh.x, b1 = b1 * scale * wh.y;
    }
    const float ra0 = a0 * cs.x - b0 * cs.y, rb0 = a0 * cs.y + b0 * cs.x;
    const float ra1 = a1 * cs.z - b1 * cs.w, rb1 = a1 * cs.w + b1 * cs.z;
    bf16* dst = is_q ? q_out + ((size_t)t * Hq + h) * HD
                     : k_cache + page_off + (size_t)((h - Hq) * page_size + in_page) * HD;
    *reinterpret_cast<__nv_bfloat162*>(dst + 2 * lane) = __floats2bfloat162_rn(ra0, ra1);
    *reinterpret_cast<__nv_bfloat162*>(dst + 64 + 2 * lane) = __floats2bfloat162_rn(rb0, rb1);
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
  const int threads = 128;
  if (rows >= 256 && dtype == LLM_BF16 && hd == 128 && rot_dim == 128 && cos_sin && !clear_proj &&
      !(proj_stride & 1) && !(((uintptr_t)proj | (uintptr_t)cos_sin) & 15)) {
    const int rc = launch_pdl(qk_norm_rope_store_rows_kernel, dim3(rows, (heads + 15) / 16), threads, 0, stream,
                              proj, proj_stride, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, page_stride,
                              block_table, table_stride, row_slot, row_pos, q_norm_w, k_norm_w,
                              (const float2*)cos_sin, Hq, Hkv, page_size, eps, has_kv, use_norm);
    g_llm_after_rotation = 1;      // (see common.cuh: a CTA-pair product behind this kernel waits for its end)
    return rc;
  }
  const dim3 blocks(rows, (heads + 3) / 4);
#define ARGS proj, proj_stride, (TQ*)q_out, (TQ*)k_cache, (TQ*)v_cache, page_stride, block_table, \
  table_stride, row_slot, row_pos, q_norm_w, k_norm_w, inv_freq, (const float2*)cos_sin, attn_factor, \
  rows, Hq, Hkv, hd, rot_dim, page_size, eps, has_kv, use_norm, clear_proj
  if (dtype == LLM_F32) {
    typedef float TQ;
    const int rc = launch_pdl(qk_norm_rope_store_kernel<float, float>, blocks, threads, 0, stream, ARGS);
    g_llm_after_rotation = 1;
    return rc;
  } else if (dtype == LLM_BF16) {
    typedef bf16 TQ;
    const int rc = launch_pdl(qk_norm_rope_store_kernel<bf16, bf16>, blocks, threads, 0, stream, ARGS);
    g_llm_after_rotation = 1;
    return rc;
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
