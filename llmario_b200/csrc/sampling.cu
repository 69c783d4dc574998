// Sampling on the device: one thread block per row of logits.
//
// The chain is the reference's (crates/engine/decode/src/sampler.rs:234-362): penalties ->
// greedy? -> top-k -> top-p -> min-p -> temperature -> softmax -> inverse-CDF draw.  Candidates
// are ordered by (logit descending, token id ascending); every filter keeps a prefix of that
// order, so the surviving set is "all tokens whose order key is >= a threshold".  Thresholds are
// found by radix selection over a 64-bit key (32 bits of order-preserving logit, 32 bits of
// inverted id): by count for top-k, by accumulated probability mass for top-p and for the draw.
// Nothing is sorted and no size is limited.
#include "common.cuh"

namespace {
constexpr int THREADS = 512;

__device__ __forceinline__ uint32_t float_key(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // larger float -> larger key
}
__device__ __forceinline__ uint64_t order_key(float v, int id) {
  return ((uint64_t)float_key(v) << 32) | (uint32_t)(~(uint32_t)id);  // ties: lower id first
}
__device__ __forceinline__ uint64_t id_key(float, int id) { return (uint32_t)(~(uint32_t)id); }

struct Shared {
  float red[33];
  float hist_f[256];
  int hist_i[256];
  unsigned long long best;
  unsigned long long prefix;
  float carry_f;
  int carry_i;
  int bin;
};

// Largest order key of the row (the arg max, lowest id among equals).
__device__ uint64_t block_best(const float* row, int V, Shared& s) {
  uint64_t b = 0;
  for (int i = threadIdx.x; i < V; i += THREADS) {
    const uint64_t k = order_key(row[i], i);
    b = k > b ? k : b;
  }
  if (threadIdx.x == 0) s.best = 0;
  __syncthreads();
  atomicMax(&s.best, (unsigned long long)b);
  __syncthreads();
  return s.best;
}

// Radix selection, most significant byte first.  Elements take part when their order key is
// >= low.  BY_MASS = false: the `target`-th largest key (target counts from 1).  BY_MASS = true:
// walking keys downwards, the first key at which the accumulated mass w = exp((l - M) * inv_t)
// reaches the target (`>=` when inclusive, `>` otherwise); if it never does, the smallest key
// with non-zero mass.  ID_ORDER walks by ascending token id instead of by logit.
template <bool BY_MASS, bool ID_ORDER>
__device__ uint64_t radix_select(const float* row, int V, uint64_t low, float M, float inv_t,
                                 float target_f, int target_i, bool inclusive, Shared& s) {
  const int top_byte = ID_ORDER ? 3 : 7;
  if (threadIdx.x == 0) { s.prefix = 0; s.carry_f = 0.f; s.carry_i = 0; }
  __syncthreads();
  for (int b = top_byte; b >= 0; --b) {
    for (int i = threadIdx.x; i < 256; i += THREADS) { s.hist_f[i] = 0.f; s.hist_i[i] = 0; }
    __syncthreads();
    const uint64_t prefix = s.prefix;
    const int shift = 8 * b;
    for (int i = threadIdx.x; i < V; i += THREADS) {
      const float l = row[i];
      if (order_key(l, i) < low) continue;
      const uint64_t k = ID_ORDER ? id_key(l, i) : order_key(l, i);
      if (b < top_byte && (k >> (shift + 8)) != (prefix >> (shift + 8))) continue;
      const int bin = (int)((k >> shift) & 255u);
      if (BY_MASS) {
        const float w = expf((l - M) * inv_t);
        if (w > 0.f) { atomicAdd(&s.hist_f[bin], w); atomicAdd(&s.hist_i[bin], 1); }
      } else {
        atomicAdd(&s.hist_i[bin], 1);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int chosen = -1, last_nonempty = -1;
      if (BY_MASS) {
        float cum = s.carry_f;
        for (int bin = 255; bin >= 0; --bin) {
          if (s.hist_i[bin] == 0) continue;
          last_nonempty = bin;
          const float next = cum + s.hist_f[bin];
          // at the last byte a bin is one element: apply the crossing rule exactly there;
          // before it, descend into the first bin whose end reaches the target
          const bool hit = inclusive ? (next >= target_f) : (next > target_f);
          if (hit) { chosen = bin; break; }
          cum = next;
        }
        // never reached (rounding): stay on the smallest keys that carry mass; the carry is
        // left as it was, so the finer levels do not reach the target either
        if (chosen < 0) chosen = last_nonempty < 0 ? 0 : last_nonempty;
        else s.carry_f = cum;
      } else {
        int cum = s.carry_i;
        for (int bin = 255; bin >= 0; --bin) {
          if (s.hist_i[bin] == 0) continue;
          last_nonempty = bin;
          if (cum + s.hist_i[bin] >= target_i) { chosen = bin; break; }
          cum += s.hist_i[bin];
        }
        if (chosen < 0) chosen = last_nonempty < 0 ? 0 : last_nonempty;
        else s.carry_i = cum;
      }
      s.prefix = prefix | ((uint64_t)chosen << shift);
    }
    __syncthreads();
  }
  return s.prefix;
}

__device__ float block_mass(const float* row, int V, uint64_t low, float M, float inv_t, Shared& s) {
  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += THREADS) {
    const float l = row[i];
    if (order_key(l, i) >= low) z += expf((l - M) * inv_t);
  }
  z = warp_sum(z);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s.red[threadIdx.x >> 5] = z;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < THREADS / 32 ? s.red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) s.red[32] = t;
  }
  __syncthreads();
  return s.red[32];
}

__global__ void __launch_bounds__(THREADS) sample_kernel(
    const float* __restrict__ logits, long long ld, int V, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
    const double* __restrict__ uniform, int* __restrict__ out, const int* __restrict__ status,
    int* __restrict__ status_out) {
  __shared__ Shared s;
  const int r = blockIdx.x;
  // the library's status words travel to the host with the tokens: whoever reads the tokens
  // learns in the same copy whether a kernel of the step gave up a wait or met a bad token id
  if (status != nullptr && r == 0 && threadIdx.x < 4) status_out[threadIdx.x] = status[threadIdx.x];
  const float* row = logits + (size_t)r * ld;
  const uint64_t best = block_best(row, V, s);
  const int best_id = (int)(~(uint32_t)(best & 0xffffffffu));
  const float temp = temperature[r];
  if (!(temp > 0.f)) {  // greedy: first maximum wins
    if (threadIdx.x == 0) out[r] = best_id;
    return;
  }
  const float M = row[best_id];
  if (!isfinite(M)) {
    if (threadIdx.x == 0) out[r] = best_id;
    return;
  }
  uint64_t low = 0;
  bool sorted = false;
  const int k = top_k[r];
  if (k > 0 && k < V) {
    low = radix_select<false, false>(row, V, 0, M, 1.f, 0.f, k, true, s);
    sorted = true;
  }
  const float p = top_p[r];
  if (p < 1.0f && !(k == 1)) {
    const float Z = block_mass(row, V, low, M, 1.f, s);
    const uint64_t t = radix_select<true, false>(row, V, low, M, 1.f, p * Z, 0, true, s);
    low = t > low ? t : low;
    sorted = true;
  }
  const float mp = min_p[r];
  if (mp > 0.f) {
    const float floor_logit = M + logf(mp);
    const uint64_t t = (uint64_t)float_key(floor_logit) << 32;  // every id at or above the floor
    low = t > low ? t : low;
  }
  const float inv_t = 1.0f / temp;
  const float Z = block_mass(row, V, low, M, inv_t, s);
  const float target = (float)(uniform[r] * (double)Z);
  uint64_t pick;
  if (sorted) {
    pick = radix_select<true, false>(row, V, low, M, inv_t, target, 0, false, s);
    if (threadIdx.x == 0) out[r] = (int)(~(uint32_t)(pick & 0xffffffffu));
  } else {
    pick = radix_select<true, true>(row, V, low, M, inv_t, target, 0, false, s);
    if (threadIdx.x == 0) out[r] = (int)(~(uint32_t)(pick & 0xffffffffu));
  }
}

// For every (row, token, count) of the penalty windows: a positive logit is divided by the
// repeat penalty, another multiplied; then count * frequency + presence is subtracted
// (sampler.rs:486-507).
__global__ void penalty_kernel(float* __restrict__ logits, long long ld, const int* __restrict__ triples,
                               int n, const float* __restrict__ repeat, const float* __restrict__ freq,
                               const float* __restrict__ presence, const int* __restrict__ inflight_src,
                               const int* __restrict__ drawn) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int r = triples[3 * i], tok = triples[3 * i + 1];
  int count = triples[3 * i + 2];
  // the token that the step before is still drawing for this row counts once more
  if (inflight_src && inflight_src[r] >= 0 && drawn[inflight_src[r]] == tok) ++count;
  float* l = logits + (size_t)r * ld + tok;
  float v = *l;
  v = v <= 0.f ? v * repeat[r] : v / repeat[r];
  v -= (float)count * freq[r] + presence[r];
  *l = v;
}

// Rows whose window gets a token that the host does not know yet (the step before is still
// drawing it; drawn[inflight_src[row]] will hold it in stream order): when no triple of the row
// names that token, it has been seen once.  One thread per row walks the triples.
__global__ void penalty_inflight_kernel(float* __restrict__ logits, long long ld, int V,
                                        const int* __restrict__ triples, int n, int rows,
                                        const float* __restrict__ repeat, const float* __restrict__ freq,
                                        const float* __restrict__ presence,
                                        const int* __restrict__ inflight_src, const int* __restrict__ drawn) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows || inflight_src[r] < 0) return;
  const int tok = drawn[inflight_src[r]];
  if (tok < 0 || tok >= V) return;
  for (int i = 0; i < n; ++i)
    if (triples[3 * i] == r && triples[3 * i + 1] == tok) return;      // counted by its triple
  float* l = logits + (size_t)r * ld + tok;
  float v = *l;
  v = v <= 0.f ? v * repeat[r] : v / repeat[r];
  v -= 1.0f * freq[r] + presence[r];
  *l = v;
}
}  // namespace

LLM_EXPORT int llm_sample(const float* logits, long long ld, int rows, int V,
                          const float* temperature, const int* top_k, const float* top_p,
                          const float* min_p, const double* uniform, int* out, const int* status,
                          int* status_out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (V <= 0) return LLM_ERR_ARGUMENT;
  sample_kernel<<<rows, THREADS, 0, stream>>>(logits, ld, V, temperature, top_k, top_p, min_p,
                                              uniform, out, status, status_out);
  return launch_status();
}

// triples: n (row, token, count) of the tokens in the rows' penalty windows.  inflight_src (may be
// null): per row of `rows`, the index in `drawn` of a token that enters the row's window but is
// still being drawn by the step before (-1: none); rows with penalties switched off must have -1.
LLM_EXPORT int llm_apply_penalties(float* logits, long long ld, int V, const int* triples, int n,
                                   const float* repeat, const float* freq, const float* presence,
                                   const int* inflight_src, const int* drawn, int rows,
                                   cudaStream_t stream) {
  if (n > 0)
    penalty_kernel<<<(n + 127) / 128, 128, 0, stream>>>(logits, ld, triples, n, repeat, freq, presence,
                                                        inflight_src, drawn);
  if (inflight_src && rows > 0)
    penalty_inflight_kernel<<<(rows + 63) / 64, 64, 0, stream>>>(logits, ld, V, triples, n, rows, repeat, freq,
                                                               presence, inflight_src, drawn);
  return launch_status();
}
