// Shared helpers of the kernels: element types, conversions, warp and block reductions, and the
// status convention of the C interface (0 = launched, otherwise a cudaError_t or a negative code
// of this library).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LLM_EXPORT extern "C" __attribute__((visibility("default")))

// negative status codes of this library (positive ones are cudaError_t values)
#define LLM_ERR_UNSUPPORTED (-1)   // a size or dtype the kernel refuses
#define LLM_ERR_ARGUMENT (-2)      // inconsistent arguments

enum LlmDtype : int { LLM_F32 = 0, LLM_BF16 = 1 };

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// ---- mbarriers (shared by the kernels that move data with the TMA unit)
constexpr long long WAIT_CYCLES = 4000000000LL;   // bound of every wait: about two seconds

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// Bounded wait for the phase with the given parity.  mbarrier.try_wait parks the thread until the
// phase completes or a hardware time limit passes, so waking up costs no polling delay; the loop
// around it gives up after WAIT_CYCLES clock cycles (about two seconds).  Returns false then.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, long long limit = WAIT_CYCLES) {
  const uint32_t addr = smem_u32(bar);
  long long start = 0;
  for (uint32_t i = 0;; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (i == 0) start = clock64();
    else if (clock64() - start > limit) return false;
  }
}
static inline int launch_status() { return (int)cudaGetLastError(); }

// Programmatic dependent launch.  A kernel that starts with pdl_trigger() lets the next kernel
// of the stream be scheduled as soon as all of its own blocks have started; that next kernel may
// do work that does not depend on earlier kernels (fetching weights, setting up barriers) and
// must call pdl_wait() before it touches anything an earlier kernel wrote or still reads.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

extern int g_llm_pdl;   // 1: launch with the programmatic-serialization attribute (llm_set_pdl)
// 1: the last kernel this library launched was the rotation kernel (rope_kv.cu).  The product on
// CTA pairs honours it: it is then launched without the programmatic attribute, i.e. only after
// the rotation kernel has finished.  A measurement once ran the sequence "rotation kernel of 2,048
// rows, then directly the CTA-pair product as its programmatic dependent" (no model has it: the
// attention kernel always comes between them) and it stopped making progress in two of three
// tries, with no bounded wait having given up; reading the kernels did not show why.  The
// sequence is therefore not launched that way by anyone, a part registered by a user included.
extern int g_llm_after_rotation;

// Launch a kernel that calls pdl_wait() itself.
template <typename... KArgs, typename... Args>
static inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, Args... args) {
  g_llm_after_rotation = 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_llm_pdl ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
