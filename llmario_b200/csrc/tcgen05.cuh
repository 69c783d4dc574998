// Device helpers for the tcgen05 / TMEM / TMA kernels, and the host-side cache of tensor maps.
#pragma once
#include <cuda.h>

#include "common.cuh"

constexpr int TILE_M = 128;       // weight rows per CTA
constexpr int TILE_K = 64;        // bf16 elements per stage row: 128 bytes, one swizzle span
constexpr int UMMA_K = 16;


enum Epilogue : int { EPI_STORE = 0, EPI_ACCUM = 1, EPI_GATED = 2 };

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_load_5d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            int c4, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, both operands K-major bf16, accumulate in float32
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Shared-memory matrix descriptor: K-major rows of 128 bytes, 128-byte swizzle, groups of eight
// rows 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// silu(g) * u = g / (1 + exp(-g)) * u in 32-bit; with a 16-bit result the division is the fast
// one (two units in the last place, far below the rounding of the result).
template <typename TC> __device__ __forceinline__ float silu_mul(float g, float u) {
  if (sizeof(TC) == 2) return __fdividef(g, 1.0f + __expf(-g)) * u;
  return g / (1.0f + __expf(-g)) * u;
}
// Gated epilogue of 16 accumulator columns v[0..15].  In each warp lanes 0..15 hold gate rows and
// lanes 16..31 the up rows of the same 16 features.  Both halves of the warp work: lane L < 16
// and lane L + 16 swap half of their columns, so that L computes columns 0..7 of its feature and
// L + 16 columns 8..15.  out[i] is column (lane < 16 ? i : 8 + i).
template <typename TC> __device__ __forceinline__ void gated_columns(const uint32_t* v, int lane, float* out) {
  const bool low = lane < 16;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float keep = __uint_as_float(low ? v[i] : v[8 + i]);
    const float send = __uint_as_float(low ? v[8 + i] : v[i]);
    const float got = __shfl_xor_sync(0xffffffffu, send, 16);
    out[i] = low ? silu_mul<TC>(keep, got) : silu_mul<TC>(got, keep);
  }
}

template <int BN>
constexpr uint32_t instr_desc() {
  // float32 accumulator, bf16 A and B, both K-major, N = BN, M = 128
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
}


// A [rows][cols] matrix with row stride ld (elements), tiled in boxes of box_rows x box_cols.
// kind 0: bf16 operand, 128-byte swizzle; kind 1: bf16 output, no swizzle; kind 2: f32 output.
// Maps are made once per (pointer, shape, box) and cached.  Defined in gemm_tcgen05.cu.
bool llm_tensor_map(const void* ptr, long long rows, long long cols, long long ld, int box_rows, int box_cols,
                    int kind, CUtensorMap* out);
// A bfloat16 tensor of 2 to 5 dimensions (innermost first; strides in bytes of dimensions
// 1 .. rank-1), tiled in boxes with the 128-byte swizzle.  Cached; defined in gemm_tcgen05.cu.
bool llm_tensor_map_tiled(const void* ptr, int rank, const long long* dims, const long long* strides,
                          const int* box, CUtensorMap* out);
