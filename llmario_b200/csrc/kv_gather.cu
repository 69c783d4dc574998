// Gather the keys and values of requests from small cache pages into large ones.
//
// The tensor-core attention of prompt portions wants its key and value tiles by TMA boxes of 64
// or 128 positions; with cache pages of 4, 8 or 16 positions it has to copy 16-byte pieces
// instead and runs at half the rate or less.  For a portion of more than a few dozen tokens it
// is cheaper to first copy the request's keys and values of one layer into a scratch cache with
// pages of `D` positions (a plain memory-bound copy, a few microseconds) and let the attention
// kernel read that.  Both caches have the layout [page][...][K|V][kv head][position][head dim].
//
// One thread block copies the K or V rows of one source page and KV head (page_size * hd
// elements, contiguous on both sides).  A source page that the request no longer holds (a window
// has passed it) or whose positions all lie below `lo` is written as zeros: its keys are masked
// by the attention kernel and its values must be finite.
#include "common.cuh"

namespace {
// One request to gather: its chunks are the source pages from position `first_pos` (a multiple of
// D) to the end of the scratch page that holds its last position `hi`.  Chunks wholly below `lo`
// or above `hi` are written as zeros: the attention kernel fetches whole scratch pages, masks
// the keys it may not see and multiplies their values by zero, so they must be finite.
struct GatherItem {
  int slot;          // row of the source block table
  int first_pos;     // position of chunk 0
  int n_chunks;
  int dst_base;      // scratch page that holds position first_pos
  int lo, hi;        // lowest and highest position the attention call will read
  int chunk_start;   // chunks of the items before this one
  int pad_;
};

template <typename T>
__global__ void __launch_bounds__(256) kv_gather_kernel(
    const T* __restrict__ k_src, const T* __restrict__ v_src, long long src_page_stride,
    const int* __restrict__ table, int table_stride, int P, T* __restrict__ k_dst, T* __restrict__ v_dst,
    long long dst_page_stride, int D, int hd, const GatherItem* __restrict__ items, int n_items) {
  pdl_trigger();
  // the list and the block tables are complete before the step's layers start; the source rows
  // of this step's own tokens are written by the kernel just ahead: wait for it
  int a = 0, b = n_items - 1;
  const int chunk = blockIdx.x;
  while (a < b) {                      // the item whose chunks hold `chunk`
    const int mid = (a + b + 1) >> 1;
    if (items[mid].chunk_start <= chunk) a = mid; else b = mid - 1;
  }
  const GatherItem it = items[a];
  const int c = chunk - it.chunk_start;
  if (c >= it.n_chunks) return;
  const int pos = it.first_pos + c * P;
  const int kvh = blockIdx.y;
  const bool value = blockIdx.z != 0;
  const int src_page =
      (pos + P - 1 >= it.lo && pos <= it.hi) ? table[(size_t)it.slot * table_stride + pos / P] : -1;
  T* dst = (value ? v_dst : k_dst) + (size_t)(it.dst_base + (pos - it.first_pos) / D) * dst_page_stride +
           ((size_t)kvh * D + pos % D) * hd;
  const int n16 = P * hd * (int)sizeof(T) / 16;
  uint4* d4 = reinterpret_cast<uint4*>(dst);
  pdl_wait();
  if (src_page < 0) {
    for (int i = threadIdx.x; i < n16; i += blockDim.x) d4[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const T* src = (value ? v_src : k_src) + (size_t)src_page * src_page_stride + (size_t)kvh * P * hd;
  const uint4* s4 = reinterpret_cast<const uint4*>(src);
  for (int i = threadIdx.x; i < n16; i += blockDim.x) d4[i] = s4[i];
}
}  // namespace

// items: n_items x (slot, first_pos, n_chunks, dst_base, lo, hi, chunk_start, 0) int32 on the device;
// total_chunks: the sum of n_chunks.  P must divide D; P * hd elements must be a multiple of 16
// bytes and the planes 16-byte aligned.
LLM_EXPORT int llm_kv_gather(const void* k_src, const void* v_src, long long src_page_stride,
                             const int* block_table, int table_stride, int page_size, void* k_dst,
                             void* v_dst, long long dst_page_stride, int dst_page_size, int Hkv, int hd,
                             int dtype, const int* items, int n_items, int total_chunks,
                             cudaStream_t stream) {
  if (n_items <= 0 || total_chunks <= 0) return 0;
  if (page_size <= 0 || dst_page_size % page_size != 0 || Hkv <= 0 || Hkv > 65535 || hd <= 0)
    return LLM_ERR_ARGUMENT;
  const int es = dtype == LLM_BF16 ? 2 : 4;
  if ((page_size * hd * es) % 16 != 0 || (src_page_stride * es) % 16 != 0 || (dst_page_stride * es) % 16 != 0 ||
      (((uintptr_t)k_src | (uintptr_t)v_src | (uintptr_t)k_dst | (uintptr_t)v_dst) & 15))
    return LLM_ERR_UNSUPPORTED;
  const dim3 grid(total_chunks, Hkv, 2);
  if (dtype == LLM_BF16)
    return launch_pdl(kv_gather_kernel<bf16>, grid, 256, 0, stream, (const bf16*)k_src, (const bf16*)v_src,
                      src_page_stride, block_table, table_stride, page_size, (bf16*)k_dst, (bf16*)v_dst,
                      dst_page_stride, dst_page_size, hd, (const GatherItem*)items, n_items);
  if (dtype == LLM_F32)
    return launch_pdl(kv_gather_kernel<float>, grid, 256, 0, stream, (const float*)k_src, (const float*)v_src,
                      src_page_stride, block_table, table_stride, page_size, (float*)k_dst, (float*)v_dst,
                      dst_page_stride, dst_page_size, hd, (const GatherItem*)items, n_items);
  return LLM_ERR_UNSUPPORTED;
}
