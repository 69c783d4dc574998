// Embedding gather, RMS norm, SiLU gating and small bookkeeping kernels.
#include "common.cuh"

int g_llm_pdl = 1;
int g_llm_after_rotation = 0;
LLM_EXPORT void llm_set_pdl(int on) { g_llm_pdl = on ? 1 : 0; }

// x[t][:] = table[token[t]][:]   (residual stream is 32-bit in every mode)
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                             float* __restrict__ x, int width, int vocab, int* __restrict__ err) {
  // The first kernel of a step's layers waits BEFORE it lets its dependents start: no kernel
  // after it can begin, not even the part before its own wait, until everything ahead of the
  // embedding (the step's token, position and block-table updates) is complete.  Kernels of the
  // layers rely on that when they read block tables and old cache pages before their wait.
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int tok = tokens[t];
  if (tok < 0 || tok >= vocab) {
    if (threadIdx.x == 0) atomicExch(err, 1 + t);
    for (int i = threadIdx.x; i < width; i += blockDim.x) x[(size_t)t * width + i] = 0.f;
    return;
  }
  const T* row = table + (size_t)tok * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) x[(size_t)t * width + i] = to_f32(row[i]);
}

LLM_EXPORT int llm_embed(const int* tokens, const void* table, int table_dtype, float* x, int rows,
                         int width, int vocab, int* err_flag, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  if (table_dtype == LLM_F32)
    return launch_pdl(embed_kernel<float>, rows, threads, 0, stream, tokens, (const float*)table, x, width, vocab, err_flag);
  if (table_dtype == LLM_BF16)
    return launch_pdl(embed_kernel<bf16>, rows, threads, 0, stream, tokens, (const bf16*)table, x, width, vocab, err_flag);
  return LLM_ERR_UNSUPPORTED;
}

// y[r][:] = x[src(r)][:] * rsqrt(mean(x^2) + eps) * w[:]    sums and scale in 32-bit.
// src(r) = rows_index ? rows_index[r] : r.
template <typename TOut>
__global__ void rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                TOut* __restrict__ y, const int* __restrict__ rows_index, int width,
                                float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows_index ? rows_index[r] : r) * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = xr[i];
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    y[(size_t)r * width + i] = from_f32<TOut>(xr[i] * scale * w[i]);
}

// The same for widths that are multiples of four and at most 256 * 4 * VEC_MAX: the row is read
// once with 16-byte loads and kept in registers between the sum and the scaling.
constexpr int VEC_MAX = 8;
template <typename TOut>
__global__ void __launch_bounds__(256) rms_norm_vec_kernel(const float* __restrict__ x,
                                                           const float* __restrict__ w, TOut* __restrict__ y,
                                                           const int* __restrict__ rows_index, int width,
                                                           float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows_index ? rows_index[r] : r) * width);
  const float4* wr = reinterpret_cast<const float4*>(w);
  const int n4 = width >> 2;
  float4 v[VEC_MAX];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VEC_MAX; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < n4) {
      v[k] = xr[i];
      ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
  for (int k = 0; k < VEC_MAX; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < n4) {
      const float4 g = wr[i];
      const float a = v[k].x * scale * g.x, b = v[k].y * scale * g.y, c = v[k].z * scale * g.z,
                  d = v[k].w * scale * g.w;
      TOut* dst = y + (size_t)r * width + 4 * i;
      if (sizeof(TOut) == 4) {
        *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst) = packed;
      }
    }
  }
}

// Many rows of a narrow width (at most 32 * 4 * WARP_VEC values): a warp per row, eight rows per
// block, no block-wide barrier.  With a block per row a row of 1,024 values is one 16-byte load
// per thread and two barriers, and the kernel is bound by launching blocks (8.6 us for 2,048
// rows of 1,024 against 3 us here).
constexpr int WARP_VEC = 16;
template <typename TOut>
__global__ void __launch_bounds__(256) rms_norm_warp_kernel(const float* __restrict__ x,
                                                            const float* __restrict__ w, TOut* __restrict__ y,
                                                            const int* __restrict__ rows_index, int rows,
                                                            int width, float eps) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows_index ? rows_index[r] : r) * width);
  const float4* wr = reinterpret_cast<const float4*>(w);
  const int n4 = width >> 2;
  float4 v[WARP_VEC];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < WARP_VEC; ++k) {
    const int i = lane + k * 32;
    if (i < n4) {
      v[k] = xr[i];
      ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
  }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
  for (int k = 0; k < WARP_VEC; ++k) {
    const int i = lane + k * 32;
    if (i < n4) {
      const float4 g = wr[i];
      const float a = v[k].x * scale * g.x, b = v[k].y * scale * g.y, c = v[k].z * scale * g.z,
                  d = v[k].w * scale * g.w;
      TOut* dst = y + (size_t)r * width + 4 * i;
      if (sizeof(TOut) == 4) {
        *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst) = packed;
      }
    }
  }
}

LLM_EXPORT int llm_rms_norm(const float* x, const float* w, void* y, int out_dtype,
                            const int* rows_index, int rows, int width, float eps,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  const bool vec = width % 4 == 0 && width <= 256 * 4 * VEC_MAX &&
                   (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) == 0;
  if (vec && rows >= 512 && width <= 32 * 4 * WARP_VEC) {
    const int blocks = (rows + 7) / 8;
    if (out_dtype == LLM_F32)
      return launch_pdl(rms_norm_warp_kernel<float>, blocks, 256, 0, stream, x, w, (float*)y, rows_index, rows,
                        width, eps);
    if (out_dtype == LLM_BF16)
      return launch_pdl(rms_norm_warp_kernel<bf16>, blocks, 256, 0, stream, x, w, (bf16*)y, rows_index, rows,
                        width, eps);
    return LLM_ERR_UNSUPPORTED;
  }
  if (vec) {
    if (out_dtype == LLM_F32)
      return launch_pdl(rms_norm_vec_kernel<float>, rows, 256, 0, stream, x, w, (float*)y, rows_index, width, eps);
    if (out_dtype == LLM_BF16)
      return launch_pdl(rms_norm_vec_kernel<bf16>, rows, 256, 0, stream, x, w, (bf16*)y, rows_index, width, eps);
    return LLM_ERR_UNSUPPORTED;
  }
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  if (out_dtype == LLM_F32)
    return launch_pdl(rms_norm_kernel<float>, rows, threads, 0, stream, x, w, (float*)y, rows_index, width, eps);
  if (out_dtype == LLM_BF16)
    return launch_pdl(rms_norm_kernel<bf16>, rows, threads, 0, stream, x, w, (bf16*)y, rows_index, width, eps);
  return LLM_ERR_UNSUPPORTED;
}

// out[t][j] = silu(gu[t][j]) * gu[t][ff + j]   with silu(z) = z / (1 + exp(-z)), in 32-bit.
template <typename TOut>
__global__ void silu_mul_kernel(const float* __restrict__ gate_up, TOut* __restrict__ out,
                                long long total, int ff) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const long long t = idx / ff;
    const int j = (int)(idx - t * ff);
    const float g = gate_up[t * 2 * ff + j];
    const float u = gate_up[t * 2 * ff + ff + j];
    out[idx] = from_f32<TOut>(g / (1.0f + expf(-g)) * u);
  }
}

LLM_EXPORT int llm_silu_mul(const float* gate_up, void* out, int out_dtype, int rows, int ff,
                            cudaStream_t stream) {
  const long long total = (long long)rows * ff;
  if (total <= 0) return 0;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (out_dtype == LLM_F32)
    silu_mul_kernel<float><<<blocks, threads, 0, stream>>>(gate_up, (float*)out, total, ff);
  else if (out_dtype == LLM_BF16)
    silu_mul_kernel<bf16><<<blocks, threads, 0, stream>>>(gate_up, (bf16*)out, total, ff);
  else
    return LLM_ERR_UNSUPPORTED;
  return launch_status();
}

// out[t][j] += bias[j], in 32-bit, rounded once to the type of out: the bias of a projection
// (the reference adds it after the product, crates/engine/model/src/forward.rs:810-830).
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ out, const float* __restrict__ bias, long long total,
                                int width) {
  pdl_trigger();
  pdl_wait();
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) out[idx] = from_f32<T>(to_f32(out[idx]) + bias[idx % width]);
}

LLM_EXPORT int llm_add_bias(void* out, int dtype, const float* bias, int rows, int width,
                            cudaStream_t stream) {
  const long long total = (long long)rows * width;
  if (total <= 0) return 0;
  const int threads = 256;
  const long long want = (total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == LLM_F32)
    return launch_pdl(add_bias_kernel<float>, blocks, threads, 0, stream, (float*)out, bias, total, width);
  if (dtype == LLM_BF16)
    return launch_pdl(add_bias_kernel<bf16>, blocks, threads, 0, stream, (bf16*)out, bias, total, width);
  return LLM_ERR_UNSUPPORTED;
}

// Scatter (row, column, value) triples into a table of block ids kept on the device.
__global__ void table_update_kernel(int* __restrict__ table, int row_stride,
                                    const int* __restrict__ updates, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) table[(size_t)updates[3 * i] * row_stride + updates[3 * i + 1]] = updates[3 * i + 2];
}

// The same with the number of triples read from device memory (at most max_n), so that the
// launch itself does not change from step to step.
__global__ void table_update_counted_kernel(int* __restrict__ table, int row_stride,
                                            const int* __restrict__ updates,
                                            const int* __restrict__ count, int max_n) {
  pdl_trigger();
  pdl_wait();
  const int n = min(*count, max_n);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    table[(size_t)updates[3 * i] * row_stride + updates[3 * i + 1]] = updates[3 * i + 2];
}

LLM_EXPORT int llm_table_update_counted(int* table, int row_stride, const int* updates,
                                        const int* count, int max_n, cudaStream_t stream) {
  if (max_n <= 0) return 0;
  const int blocks = (max_n + 127) / 128 < 8 ? (max_n + 127) / 128 : 8;
  return launch_pdl(table_update_counted_kernel, blocks, 128, 0, stream, table, row_stride, updates, count, max_n);
}

LLM_EXPORT int llm_table_update(int* table, int row_stride, const int* updates, int n,
                                cudaStream_t stream) {
  if (n <= 0) return 0;
  table_update_kernel<<<(n + 127) / 128, 128, 0, stream>>>(table, row_stride, updates, n);
  return launch_status();
}

// tokens[i] = source[index[i]] where index[i] >= 0: rows whose token was drawn by the previous
// step and has not been to the host yet take it from the sampler's output on the device.
__global__ void patch_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ source,
                                    const int* __restrict__ index, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && index[i] >= 0) tokens[i] = source[index[i]];
}

LLM_EXPORT int llm_patch_tokens(int* tokens, const int* source, const int* index, int n,
                                cudaStream_t stream) {
  if (n <= 0) return 0;
  patch_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(tokens, source, index, n);
  return launch_status();
}

// Clear a [rows][cols] float matrix with row stride ld (a kernel rather than a memset, so that it
// can take part in programmatic dependent launch).
__global__ void zero_f32_kernel(float* __restrict__ p, int rows, int cols, int ld) {
  pdl_trigger();
  pdl_wait();
  const long long total = (long long)rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x)
    p[(i / cols) * ld + (i % cols)] = 0.f;
}

int llm_zero_f32(float* p, int rows, int cols, int ld, cudaStream_t stream) {
  const long long total = (long long)rows * cols;
  if (total <= 0) return 0;
  const int blocks = (int)((total + 1023) / 1024 < 592 ? (total + 1023) / 1024 : 592);
  return launch_pdl(zero_f32_kernel, blocks, 256, 0, stream, p, rows, cols, ld);
}

// state[slots[i]][:] = 0 for i < *count (count read on the device, at most max_n): the fixed-size
// state of request slots that were opened for this step, cleared inside the step so that a
// recorded step clears whatever slots its replay names.
__global__ void zero_slots_kernel(unsigned int* __restrict__ state, long long row_words,
                                  const int* __restrict__ slots, const int* __restrict__ count) {
  pdl_wait();
  pdl_trigger();
  if ((int)blockIdx.x >= *count) return;
  unsigned int* row = state + (size_t)slots[blockIdx.x] * row_words;
  for (long long i = (long long)blockIdx.y * blockDim.x + threadIdx.x; i < row_words;
       i += (long long)gridDim.y * blockDim.x)
    row[i] = 0u;
}

LLM_EXPORT int llm_zero_slots(void* state, long long row_bytes, const int* slots, const int* count,
                              int max_n, cudaStream_t stream) {
  if (max_n <= 0 || row_bytes <= 0) return 0;
  if (row_bytes % 4 != 0 || ((uintptr_t)state & 3)) return LLM_ERR_UNSUPPORTED;
  const long long words = row_bytes / 4;
  const int chunks = (int)((words + 4095) / 4096 < 64 ? (words + 4095) / 4096 : 64);
  return launch_pdl(zero_slots_kernel, dim3(max_n, chunks), 256, 0, stream, (unsigned int*)state, words,
                    slots, count);
}

// A wait that runs out, on purpose and harmlessly: one thread waits on an mbarrier at which
// nothing arrives, with a caller-given limit of clock cycles, gives up, records role 99 in the
// status word and returns.  Every bounded wait of the TMA / tcgen05 kernels ends this way when
// its limit passes; tests use this kernel to see the host side of that path (the status word
// reaching the engine, the step's requests failing) without a kernel that misbehaves.
__global__ void selftest_wait_kernel(int* status, long long limit) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!mbar_wait(&bar, 0, limit)) atomicExch(status, 99);
  }
}

LLM_EXPORT int llm_selftest_wait_gives_up(int* status, long long limit_cycles, cudaStream_t stream) {
  if (status == nullptr || limit_cycles <= 0 || limit_cycles > 2000000) return LLM_ERR_ARGUMENT;
  selftest_wait_kernel<<<1, 32, 0, stream>>>(status, limit_cycles);
  return launch_status();
}
