// An entry point of this library that never allocates device memory.
//
// It has no counterpart in mannysinghx/LLMario: the reference's engine sizes every buffer in its
// planner before it loads a model and has no CUDA code at all.  It exists for callers of *this*
// library that cannot call cudaMalloc when they need decode attention: programs that gave the
// whole GPU to their own memory plan at start-up, serving loops that must not risk the
// device-wide synchronisation of an allocation, and hosts that allow allocation only inside
// another framework's pool.
//
//   int llm_attention_decode_no_alloc(q, out, k_cache, v_cache, page_stride, block_table,
//                                     table_stride, row_slot, row_pos, rows, Hq, Hkv, hd,
//                                     page_size, scale, window, splits, stream)
//
// One query row per request (bfloat16, head size 32, 64 or 128) against the paged cache, keys cut
// into `splits` parts and merged: the same result as llm_attention_flash followed by
// llm_attention_merge, with the partial sums kept in an 8 MiB array inside the library instead of
// caller-provided buffers.  The caller still passes inputs and the output.
//
//   * rows * Hq * splits * (hd + 2) must not exceed NO_ALLOC_SCRATCH_FLOATS, else the call
//     returns LLM_ERR_TOO_LARGE (-3) and does nothing.
//   * The first call on each device resolves the array's device address; make it before any
//     stream capture begins.
//   * Calls share the array: do not let two of them overlap on the GPU.
//   * At most 16 query heads per KV head; otherwise, or with another head size, the call returns
//     LLM_ERR_UNSUPPORTED (-1).  A page size or number of parts that is not positive, a negative
//     window or more than 65535 parts return LLM_ERR_ARGUMENT (-2).  Nothing is launched then.
//   * The per-device address is cached without a lock; concurrent first calls store the same
//     value.
#pragma once
#include <cuda_runtime.h>

#define NO_ALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define LLM_ERR_TOO_LARGE (-3)

extern "C" __attribute__((visibility("default"))) int llm_attention_decode_no_alloc(
    const void* q, void* out, const void* k_cache, const void* v_cache, long long page_stride,
    const int* block_table, int table_stride, const int* row_slot, const int* row_pos, int rows,
    int Hq, int Hkv, int hd, int page_size, float scale, int window, int splits,
    cudaStream_t stream);
