// The native step driver: the launches of a run of standard layers, issued from C++.
//
// A step of the engine runs, per layer, about eight kernels.  Issued one by one from Python they
// cost the host ten microseconds each, which is what bounds the prompt and mixed steps of a small
// model (decode steps are replayed as CUDA graphs and do not feel it).  Here the same launches are
// issued by one call per run of layers: Python describes every layer once, when the model is
// built (LlmLayerDesc: weights, sizes, constants), every run-order entry once, when the cache is
// made (LlmCallDesc: where its keys and values live), and the step each time (LlmStepDesc: rows,
// the step's device arrays, the segments of its requests).
//
// The layer is the reference's pre-norm residual block (crates/engine/model/src/forward.rs:356-362):
// x += Attn(RMSNorm(x)); x += FFN(RMSNorm(x)), attention being projections -> per-head norm ->
// rotation -> cache write -> attention over the cache -> output projection (forward.rs:399-485) and
// the feed-forward down(silu(gate h) * (up h)) (forward.rs:500-530).  Which kernel serves a
// product or an attention call, into how many parts K or the keys are cut, and which rows form
// an attention work item are decided here by the same rules as llmario_b200/kernels.py applies for
// parts that are driven from Python (a test holds the two to the same answers and the same
// tokens).  Temporary buffers come from a grow-only arena of this library; it grows only in steps
// that run eagerly (a recorded step has run eagerly with the same sizes before).
#include <math.h>
#include <algorithm>
#include <stdint.h>
#include <string.h>

#include <deque>
#include <map>
#include <vector>

#include "common.cuh"
#include "step_driver.h"

// ---- the kernels' own entry points (defined in the other files of this library)
extern "C" {
int llm_rms_norm(const float* x, const float* w, void* y, int out_dtype, const int* rows_index, int rows,
                 int width, float eps, cudaStream_t stream);
int llm_silu_mul(const float* gate_up, void* out, int out_dtype, int rows, int ff, cudaStream_t stream);
int llm_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype, int M, int N,
                  int K, int lda, int ldw, int ldc, int accumulate, cudaStream_t stream);
int llm_gemm_tcgen05(const void* X, const void* W, void* C, int c_dtype, int T, int N, int K, int lda, int ldw,
                     int ldc, int mode, int half, int bn, int splits, int out_is_zero, int* status,
                     cudaStream_t stream);
int llm_qk_norm_rope_store(const float* proj, int proj_stride, void* q_out, void* k_cache, void* v_cache,
                           int dtype, long long page_stride, const int* block_table, int table_stride,
                           const int* row_slot, const int* row_pos, const float* q_norm_w,
                           const float* k_norm_w, const float* inv_freq, const float* cos_sin,
                           float attn_factor, int rows, int Hq, int Hkv, int hd, int rot_dim, int page_size,
                           float eps, int has_kv, int use_norm, int clear_proj, cudaStream_t stream);
int llm_rope_table(const int* row_pos, const float* inv_freq, float* cos_sin, int rows, int half,
                   float attn_factor, cudaStream_t stream);
int llm_attention_generic(const void* q, void* out, const void* k_cache, const void* v_cache, int dtype,
                          long long page_stride, const int* block_table, int table_stride,
                          const int* row_slot, const int* row_pos, int rows, int Hq, int Hkv, int hd,
                          int page_size, float scale, int window, cudaStream_t stream);
int llm_attention_flash(const void* q, void* out, float* part_o, float* part_ml, const void* k_cache,
                        const void* v_cache, long long page_stride, const int* block_table, int table_stride,
                        const int* items, const int* row_slot, const int* row_pos, int n_items,
                        int rows_per_cta, int Hq, int Hkv, int hd, int page_size, float scale, int window,
                        int splits, cudaStream_t stream);
int llm_attention_decode(const void* q, void* out, float* part_o, float* part_ml, const void* k_cache,
                         const void* v_cache, long long page_stride, const int* block_table,
                         int table_stride, const int* items, const int* row_slot, const int* row_pos,
                         int n_items, int Hq, int Hkv, int hd, int page_size, float scale, int window,
                         int splits, cudaStream_t stream);
int llm_attention_decode_tma(const void* q, void* out, float* part_o, float* part_ml, const void* storage,
                             long long n_pages, int n_slots, int slot, const int* block_table,
                             int table_stride, const int* items, const int* row_slot, const int* row_pos,
                             int n_items, int Hq, int Hkv, int hd, int page_size, float scale, int window,
                             int splits, int* status, cudaStream_t stream);
int llm_attention_decode_persistent(const void* q, float* part_o, float* part_ml, const void* storage,
                                    long long n_pages, int n_slots, int slot, const int* block_table,
                                    int table_stride, const int* row_slot, const int* row_pos, int rows, int Hq,
                                    int Hkv, int hd, int page_size, float scale, int window, int parts, int ctas,
                                    int* status, cudaStream_t stream);
int llm_attention_decode_fused(float* proj, int proj_stride, void* out, float* part_o, float* part_ml,
                               const void* storage, long long n_pages, int n_slots, int slot, void* k_cache,
                               void* v_cache, long long page_stride, const int* block_table,
                               int table_stride, const int* row_slot, const int* row_pos, int rows,
                               const float* q_norm_w, const float* k_norm_w, const float* cos_sin, float eps,
                               int clear, int Hq, int Hkv, int hd, int page_size, float scale, int window,
                               int splits, int* status, cudaStream_t stream);
int llm_attention_merge_clear(const float* part_o, const float* part_ml, void* out, const int* rows,
                              int n_rows, int Hq, int hd, int splits, float* clear, int clear_stride,
                              cudaStream_t stream);
int llm_attention_tcgen05(const void* q, void* out, int rows, const void* k_cache, const void* v_cache,
                          long long page_stride, long long n_pages, const int* block_table, int table_stride,
                          const int* items, int n_items, int Hq, int Hkv, int hd, int page_size, float scale,
                          int window, int persistent, int* status, cudaStream_t stream);
int llm_kv_gather(const void* k_src, const void* v_src, long long src_page_stride, const int* block_table,
                  int table_stride, int page_size, void* k_dst, void* v_dst, long long dst_page_stride,
                  int dst_page_size, int Hkv, int hd, int dtype, const int* items, int n_items,
                  int total_chunks, cudaStream_t stream);
int llm_attention_tcgen05_x2(const void* q, void* out, int rows, const void* k_cache, const void* v_cache,
                             long long page_stride, long long n_pages, const int* block_table,
                             int table_stride, const int* items, int n_items, int Hq, int Hkv, int hd,
                             int page_size, float scale, int window, int* status, cudaStream_t stream);
}

namespace {

// ------------------------------------------------------------------------------------------------
// policies (the same numbers as llmario_b200/kernels.py)
// ------------------------------------------------------------------------------------------------
constexpr int SPLIT_K_MAX_ROWS = 256;       // up to here the q/k/v destination is kept at zero
constexpr int DECODE_TMA_TILE = 32;         // keys of a tile of attention_decode_tma.cu
constexpr int DECODE_TMA_CTAS_PER_SM = 4;   // its one-warp CTAs that fit an SM at head size 128 (three tiles of 16 KB each)
constexpr int PERSISTENT_ATTENTION_MAX_KEYS = 6144;
// Prompt portions over a cache with small pages: the request's keys and values are first
// gathered into scratch pages of GATHER_PAGE positions when the portion has at least
// GATHER_MIN_PAIRS (token, head of the group) pairs.  (The tcgen05 kernel reaches about twice the
// rate with TMA boxes; the copy costs about as much as the attention of 90 / group tokens.)
constexpr int GATHER_PAGE = 128;
constexpr int GATHER_MIN_PAIRS = 512;
int g_gather = 1;                           // 0: never gather (for measurements)
// The persistent decode kernel (attention_decode_tma.cu: as many one-warp CTAs as fit at once
// share all tiles of a step of single tokens evenly; every (row, head) gets PERSISTENT_PARTS parts,
// some empty, for the merge) is OFF unless llm_set_persistent_decode(1).  Measured, 32 query / 8 KV
// heads of 128: by itself it beats one CTA per part where those make one to five waves (32 rows x
// 1,024 keys 31.0 -> 28.2 us, 64 x 1,024 53.0 -> 49.9, 64 x 4,096 169.5 -> 167.4; not beyond 128
// rows, since every CTA first reads all rows' positions).  Inside the decode step of the 36-layer
// model at batch 64 it gains 1.4 % at best (5.38 -> 5.30 ms with 410 CTAs) and LOSES 16 % with the
// 444 CTAs that fit an idle GPU (6.24 ms): between other kernels not all of them find room at
// once, and a CTA that starts late still has its full share to walk.  Short-lived CTAs do not
// have that cliff, so they stay the default.
constexpr int PERSISTENT_PARTS = 4;
constexpr int PERSISTENT_MAX_ROWS = 128;
constexpr int PERSISTENT_MAX_WAVES = 5;
int g_persistent_decode = 0;
int g_fuse_mode = 0;                        // 0: when few waves, 1: always, 2: never

// how often the driver chose which kernel (llm_driver_counts; tests and statistics read them)
enum Kind : int {
  K_NORM, K_GEMM_TCGEN05, K_GEMM_SIMT, K_ROPE_TABLE, K_ROPE_STORE, K_DECODE_FUSED, K_DECODE_TMA, K_DECODE,
  K_FLASH, K_MERGE, K_TCGEN05, K_TCGEN05_X2, K_GENERIC, K_SILU_MUL, K_KV_GATHER, K_DECODE_PERSISTENT,
  N_KINDS
};
long long g_counts[N_KINDS] = {};

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int esize(int dtype) { return dtype == LLM_BF16 ? 2 : 4; }
inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

bool tc_ok(const void* a, int a_dt, int lda, const void* w, int w_dt, int ldw, int k) {
  return a_dt == LLM_BF16 && w_dt == LLM_BF16 && k % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && aligned16(a) &&
         aligned16(w);
}

// ------------------------------------------------------------------------------------------------
// the arena: named device buffers that live across steps and only grow
// ------------------------------------------------------------------------------------------------
enum BufId : int {
  B_H = 1, B_PROJ, B_ZPROJ /* + width */, B_Q, B_OUT, B_ACT, B_GATE_UP, B_PART_O, B_PART_ML, B_ROPE /* + k */,
  B_ITEMS, B_GATHER
};

struct Buf { void* p = nullptr; size_t bytes = 0; bool kept_zero = false; };

struct Arena {
  std::map<long long, Buf> bufs;
  long long generation = 0;
  // pinned staging for the work items of attention: a few slots in turn, each with the event of
  // the copy that last read it
  static constexpr int SLOTS = 4;
  int* pinned[SLOTS] = {nullptr, nullptr, nullptr, nullptr};
  size_t pinned_ints[SLOTS] = {0, 0, 0, 0};
  cudaEvent_t ev[SLOTS] = {nullptr, nullptr, nullptr, nullptr};
  int turn = 0;

  // a buffer of at least `bytes`; `zero`: it is created holding zeros (its users keep it so)
  int get(long long key, size_t bytes, bool zero, void** out) {
    Buf& b = bufs[key];
    if (b.bytes < bytes || b.p == nullptr) {
      if (b.p) cudaFree(b.p);     // (synchronises: nothing in flight reads it afterwards)
      b.p = nullptr;
      const size_t want = bytes < 256 ? 256 : bytes;
      cudaError_t e = cudaMalloc(&b.p, want);
      if (e != cudaSuccess) { b.bytes = 0; return (int)e; }
      if (zero) {
        e = cudaMemset(b.p, 0, want);
        if (e != cudaSuccess) return (int)e;
      }
      b.bytes = want;
      b.kept_zero = zero;
      ++generation;
    }
    *out = b.p;
    return 0;
  }
  void drop() {
    for (auto& kv : bufs)
      if (kv.second.p) cudaFree(kv.second.p);
    bufs.clear();
    ++generation;
  }
  // ints on the device holding `host[0..n)`, copied in stream order.  `index`: which upload of
  // the step this is; each has a device buffer of its own, so that what an earlier upload of
  // the step left stays valid (across steps the buffers are used again: the copy runs in stream
  // order, after every kernel of the step before).
  int upload(const std::vector<int>& host, int index, int** dev, cudaStream_t stream) {
    const int s = turn;
    turn = (turn + 1) % SLOTS;
    if (ev[s]) {
      cudaError_t e = cudaEventSynchronize(ev[s]);
      if (e != cudaSuccess) return (int)e;
    } else {
      cudaError_t e = cudaEventCreateWithFlags(&ev[s], cudaEventDisableTiming);
      if (e != cudaSuccess) return (int)e;
    }
    if (pinned_ints[s] < host.size()) {
      if (pinned[s]) cudaFreeHost(pinned[s]);
      pinned_ints[s] = host.size() * 2 + 64;
      cudaError_t e = cudaMallocHost((void**)&pinned[s], pinned_ints[s] * sizeof(int));
      if (e != cudaSuccess) { pinned_ints[s] = 0; pinned[s] = nullptr; return (int)e; }
    }
    memcpy(pinned[s], host.data(), host.size() * sizeof(int));
    void* d = nullptr;
    int rc = get(B_ITEMS * 1000000LL + index, host.size() * sizeof(int), false, &d);
    if (rc) return rc;
    cudaError_t e = cudaMemcpyAsync(d, pinned[s], host.size() * sizeof(int), cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return (int)e;
    e = cudaEventRecord(ev[s], stream);
    if (e != cudaSuccess) return (int)e;
    *dev = (int*)d;
    return 0;
  }
};

Arena& arena() {
  static std::map<int, Arena> per_device;
  int dev = 0;
  cudaGetDevice(&dev);
  return per_device[dev];
}

// ------------------------------------------------------------------------------------------------
// one run of layers
// ------------------------------------------------------------------------------------------------
struct Plan {          // the rows of the step as work items for one (group, large_cap)
  int group = 0, large_cap = 0;
  int n_small = 0, n_large = 0;
  bool small_single = false;
  const int* small = nullptr;       // device quadruples (first row, tokens, slot, first position)
  const int* large = nullptr;
  const int* small_rows = nullptr;  // the rows of the small items, for the merge
  std::vector<int> large_host;      // the large items as the host made them
};

// The large items of a plan split for a cache with small pages: requests whose portion is long
// enough are read from gathered scratch pages, the others from the cache as it is.
struct GatherPlan {
  int group = 0, large_cap = 0, page_size = 0, window = 0;
  int n_requests = 0, total_chunks = 0, scratch_pages = 0, table_stride = 0;
  int n_gathered = 0, n_direct = 0;
  const int* list = nullptr;        // device: n_requests x GatherItem
  const int* table = nullptr;       // device: block table of the scratch pages, a row per request
  const int* gathered = nullptr;    // device: items whose "slot" is the row of `table`
  const int* direct = nullptr;      // device: items read from the cache itself
};

// What is made once per step and shared by its layers (and by calls that come one by one from
// Python parts): work items and the tables of cosines and sines.  Keyed by the step's id.
struct StepCache {
  long long step_id = -1;
  int uploads = 0;
  std::deque<Plan> plans;
  std::deque<GatherPlan> gathers;
  std::map<const float*, float*> rope;     // inv_freq table -> cos/sin of this step's rows
};

StepCache& step_cache(long long step_id) {
  static std::map<int, StepCache> per_device;
  int dev = 0;
  cudaGetDevice(&dev);
  StepCache& c = per_device[dev];
  if (c.step_id != step_id || step_id < 0) {
    c.plans.clear();
    c.gathers.clear();
    c.rope.clear();
    c.uploads = 0;
    c.step_id = step_id;
  }
  return c;
}

struct Run {
  const LlmStepDesc& st;
  cudaStream_t stream;
  Arena& ar;
  int launches = 0;
  std::deque<Plan>& plans;
  std::deque<GatherPlan>& gathers;
  std::map<const float*, float*>& rope;
  int& uploads;

  Run(const LlmStepDesc& s, cudaStream_t str, StepCache& c)
      : st(s), stream(str), ar(arena()), plans(c.plans), gathers(c.gathers), rope(c.rope), uploads(c.uploads) {}

  int check(int rc, Kind kind) {
    if (rc == 0) {
      ++launches;
      ++g_counts[kind];
    }
    return rc;
  }

  int buffer(long long key, size_t bytes, void** out, bool zero = false) { return ar.get(key, bytes, zero, out); }

  // out (=|+=) a @ w^T with the fastest kernel that takes the operands (kernels.linear)
  int linear(const void* a, int a_dt, int lda, const void* w, int w_dt, int ldw, void* out, int out_dt, int ldc,
             int rows, int n, int k, bool accumulate, bool out_is_zero) {
    if (tc_ok(a, a_dt, lda, w, w_dt, ldw, k)) {
      const int splits = out_dt == LLM_F32 ? llm_k_splits(rows, n, k) : 1;
      return check(llm_gemm_tcgen05(a, w, out, out_dt, rows, n, k, lda, ldw, ldc, accumulate ? 1 : 0, 0,
                                    llm_token_tile(rows), splits, out_is_zero ? 1 : 0, st.status, stream), K_GEMM_TCGEN05);
    }
    return check(llm_gemm_simt(a, a_dt, w, w_dt, out, out_dt, rows, n, k, lda, ldw, ldc, accumulate ? 1 : 0, stream), K_GEMM_SIMT);
  }

  int rope_table(const LlmLayerDesc& L, const float** out) {
    *out = nullptr;
    if (L.inv_freq == nullptr || L.rot_dim <= 0) return 0;
    auto it = rope.find(L.inv_freq);
    if (it != rope.end()) { *out = it->second; return 0; }
    void* t = nullptr;
    const int half = L.rot_dim / 2;
    int rc = buffer(B_ROPE * 1000000LL + (long long)rope.size(), (size_t)st.rows * half * 2 * sizeof(float), &t);
    if (rc) return rc;
    rc = check(llm_rope_table(st.row_pos, L.inv_freq, (float*)t, st.rows, half, L.attn_factor, stream), K_ROPE_TABLE);
    if (rc) return rc;
    rope[L.inv_freq] = (float*)t;
    *out = (float*)t;
    return 0;
  }

  int plan_for(int group, int large_cap, const Plan** out) {
    if (large_cap < 1) large_cap = 1;
    for (const Plan& p : plans)
      if (p.group == group && p.large_cap == large_cap) { *out = &p; return 0; }
    Plan p;
    p.group = group;
    p.large_cap = large_cap;
    const int small_cap = (group <= 8 ? 8 : 16) / group < 1 ? 1 : (group <= 8 ? 8 : 16) / group;
    if (st.all_single) {
      p.n_small = st.rows;
      p.small_single = true;
    } else {
      std::vector<int> small, large, small_rows;
      bool single = true;
      for (int s = 0; s < st.n_segments; ++s) {
        const int* g = st.segments + 4 * s;   // (first row, rows, slot, first position)
        if (g[1] <= small_cap) {
          small.insert(small.end(), {g[0], g[1], g[2], g[3]});
          small_rows.push_back(g[0]);
          single = single && g[1] == 1;
        } else {
          for (int at = 0; at < g[1]; at += large_cap) {
            const int n = g[1] - at < large_cap ? g[1] - at : large_cap;
            large.insert(large.end(), {g[0] + at, n, g[2], g[3] + at});
          }
        }
      }
      p.n_small = (int)small.size() / 4;
      p.n_large = (int)large.size() / 4;
      p.large_host = large;
      p.small_single = single;
      std::vector<int> flat(small);
      flat.insert(flat.end(), large.begin(), large.end());
      flat.insert(flat.end(), small_rows.begin(), small_rows.end());
      int* dev = nullptr;
      int rc = ar.upload(flat, uploads++, &dev, stream);
      if (rc) return rc;
      if (p.n_small) {
        p.small = dev;
        p.small_rows = dev + 4 * (p.n_small + p.n_large);
      }
      if (p.n_large) p.large = dev + 4 * p.n_small;
    }
    plans.push_back(p);
    *out = &plans.back();
    return 0;
  }

  // Split the large items of `plan` for a cache with pages of `ps` < 32 positions.
  int gather_for(const Plan& plan, int ps, int window, const GatherPlan** out) {
    for (const GatherPlan& g : gathers)
      if (g.group == plan.group && g.large_cap == plan.large_cap && g.page_size == ps && g.window == window) {
        *out = &g;
        return 0;
      }
    GatherPlan g;
    g.group = plan.group, g.large_cap = plan.large_cap, g.page_size = ps, g.window = window;
    const int D = GATHER_PAGE;
    // a request's items follow one another; its portion is theirs together
    struct Req { int slot, pos0, pos1, first_item, n_items; };
    std::vector<Req> reqs;
    const std::vector<int>& L = plan.large_host;
    for (int i = 0; i < plan.n_large; ++i) {
      const int* it = &L[4 * i];
      if (!reqs.empty() && reqs.back().slot == it[2] && reqs.back().pos1 == it[3])
        reqs.back().pos1 += it[1], reqs.back().n_items += 1;
      else
        reqs.push_back(Req{it[2], it[3], it[3] + it[1], i, 1});
    }
    std::vector<int> list, table, gathered, direct;
    int max_pages = 0;
    for (const Req& r : reqs)
      if ((r.pos1 - r.pos0) * plan.group >= GATHER_MIN_PAIRS) max_pages = std::max(max_pages, (r.pos1 + D - 1) / D);
    g.table_stride = max_pages;
    for (const Req& r : reqs) {
      const bool take = (r.pos1 - r.pos0) * plan.group >= GATHER_MIN_PAIRS;
      for (int i = r.first_item; i < r.first_item + r.n_items; ++i) {
        const int* it = &L[4 * i];
        if (take) gathered.insert(gathered.end(), {it[0], it[1], g.n_requests, it[3]});
        else direct.insert(direct.end(), {it[0], it[1], it[2], it[3]});
      }
      if (!take) continue;
      const int lo = window > 0 && r.pos0 + 1 > window ? r.pos0 + 1 - window : 0;
      const int first_page = lo / D;                        // scratch page of the lowest key read
      const int first_pos = first_page * D;
      const int n_pages = (r.pos1 - 1) / D - first_page + 1;
      const int n_chunks = n_pages * (D / ps);          // whole scratch pages: the tail is zeroed
      list.insert(list.end(), {r.slot, first_pos, n_chunks, g.scratch_pages, lo, r.pos1 - 1, g.total_chunks, 0});
      for (int pi = 0; pi < max_pages; ++pi)
        table.push_back(pi >= first_page && pi * D < r.pos1 ? g.scratch_pages + pi - first_page : -1);
      g.scratch_pages += n_pages;
      g.total_chunks += n_chunks;
      ++g.n_requests;
    }
    g.n_gathered = (int)gathered.size() / 4;
    g.n_direct = (int)direct.size() / 4;
    if (g.n_requests) {
      std::vector<int> flat(list);
      const size_t o_table = flat.size();
      flat.insert(flat.end(), table.begin(), table.end());
      const size_t o_gathered = flat.size();
      flat.insert(flat.end(), gathered.begin(), gathered.end());
      const size_t o_direct = flat.size();
      flat.insert(flat.end(), direct.begin(), direct.end());
      int* dev = nullptr;
      int rc = ar.upload(flat, uploads++, &dev, stream);
      if (rc) return rc;
      g.list = dev;
      g.table = dev + o_table;
      g.gathered = dev + o_gathered;
      g.direct = g.n_direct ? dev + o_direct : nullptr;
    }
    gathers.push_back(g);
    *out = &gathers.back();
    return 0;
  }

  bool decode_tma_ok(const LlmCallDesc& c, int hd) const {
    const int ps = c.page_size;
    return c.storage != nullptr && (hd == 64 || hd == 128) && (ps & (ps - 1)) == 0 &&
           c.n_pages * c.n_slots * 2 < (1LL << 31);
  }

  bool fusion_ok(const LlmLayerDesc& L, const LlmCallDesc& c, const float* cos_sin) const {
    if (g_fuse_mode == 2) return false;
    const bool ok = st.dtype == LLM_BF16 && cos_sin != nullptr && L.rot_dim == L.head_dim &&
                    L.num_heads / L.num_kv_heads <= 8 && decode_tma_ok(c, L.head_dim) && st.all_single;
    if (!ok || g_fuse_mode == 1) return ok;
    const int reach = L.window ? (st.max_pos + 1 < L.window ? st.max_pos + 1 : L.window) : st.max_pos + 1;
    const int resident = DECODE_TMA_CTAS_PER_SM * sm_count();
    return (long long)st.rows * L.num_kv_heads *
               llm_decode_splits(st.rows, L.num_kv_heads, reach, resident, DECODE_TMA_TILE) <=
           2LL * resident;
  }

  int parts(int splits, const LlmLayerDesc& L, float** part_o, float** part_ml) {
    *part_o = *part_ml = nullptr;
    if (splits <= 1) return 0;
    void *o = nullptr, *ml = nullptr;
    int rc = buffer(B_PART_O, (size_t)st.rows * L.num_heads * splits * L.head_dim * sizeof(float), &o);
    if (rc) return rc;
    rc = buffer(B_PART_ML, (size_t)st.rows * L.num_heads * splits * 2 * sizeof(float), &ml);
    if (rc) return rc;
    *part_o = (float*)o;
    *part_ml = (float*)ml;
    return 0;
  }

  // causal attention of every row over its own request's cached keys (kernels.attention)
  int attention(const LlmLayerDesc& L, const LlmCallDesc& c, const void* q, void* out) {
    const int Hq = L.num_heads, Hkv = L.num_kv_heads, hd = L.head_dim, group = Hq / Hkv;
    const int window = L.window;
    if (st.dtype != LLM_BF16 || !(hd == 32 || hd == 64 || hd == 128) || group > 16)
      return check(llm_attention_generic(q, out, c.k, c.v, st.dtype, c.page_stride, c.block_table,
                                         c.table_stride, st.row_slot, st.row_pos, st.rows, Hq, Hkv, hd,
                                         c.page_size, L.scale, window, stream), K_GENERIC);
    const int ps = c.page_size;
    const bool tc = (hd == 64 || hd == 128) && 128 % group == 0 && (c.page_stride * 2) % 16 == 0;
    const bool x2 = tc && ps >= 32 && (ps & (ps - 1)) == 0 && c.storage != nullptr && ps < 64 &&
                    (long long)st.rows * Hkv >= 4LL * sm_count() * (128 / group);
    const Plan* plan = nullptr;
    int rc = plan_for(group, (x2 ? 256 : tc ? 128 : 64) / group, &plan);
    if (rc) return rc;
    const int reach = window ? (st.max_pos + 1 < window ? st.max_pos + 1 : window) : st.max_pos + 1;
    if (plan->n_small) {
      const bool tma = group <= 8 && decode_tma_ok(c, hd);
      const int splits = plan->small_single
                             ? llm_decode_splits(plan->n_small, Hkv, reach, (tma ? DECODE_TMA_CTAS_PER_SM : 6) * sm_count(),
                                                 tma ? DECODE_TMA_TILE : 32)
                             : 1;
      float *part_o, *part_ml;
      const int resident = DECODE_TMA_CTAS_PER_SM * sm_count();
      if (g_persistent_decode && tma && plan->small == nullptr && st.rows <= PERSISTENT_MAX_ROWS &&
          (long long)plan->n_small * Hkv * splits > resident &&
          (long long)plan->n_small * Hkv * splits <= (long long)PERSISTENT_MAX_WAVES * resident) {
        rc = parts(PERSISTENT_PARTS, L, &part_o, &part_ml);
        if (rc) return rc;
        rc = check(llm_attention_decode_persistent(q, part_o, part_ml, c.storage, c.n_pages, c.n_slots, c.slot,
                                                   c.block_table, c.table_stride, st.row_slot, st.row_pos,
                                                   plan->n_small, Hq, Hkv, hd, ps, L.scale, window,
                                                   PERSISTENT_PARTS, resident - resident / 12, st.status, stream),
                   K_DECODE_PERSISTENT);
        if (rc) return rc;
        return check(llm_attention_merge_clear(part_o, part_ml, out, nullptr, plan->n_small, Hq, hd,
                                               PERSISTENT_PARTS, nullptr, 0, stream), K_MERGE);
      }
      rc = parts(splits, L, &part_o, &part_ml);
      if (rc) return rc;
      if (tma)
        rc = check(llm_attention_decode_tma(q, out, part_o, part_ml, c.storage, c.n_pages, c.n_slots, c.slot,
                                            c.block_table, c.table_stride, plan->small, st.row_slot,
                                            st.row_pos, plan->n_small, Hq, Hkv, hd, ps, L.scale, window,
                                            splits, st.status, stream), K_DECODE_TMA);
      else if (group <= 8)
        rc = check(llm_attention_decode(q, out, part_o, part_ml, c.k, c.v, c.page_stride, c.block_table,
                                        c.table_stride, plan->small, st.row_slot, st.row_pos, plan->n_small,
                                        Hq, Hkv, hd, ps, L.scale, window, splits, stream), K_DECODE);
      else
        rc = check(llm_attention_flash(q, out, part_o, part_ml, c.k, c.v, c.page_stride, c.block_table,
                                       c.table_stride, plan->small, st.row_slot, st.row_pos, plan->n_small,
                                       16, Hq, Hkv, hd, ps, L.scale, window, splits, stream), K_FLASH);
      if (rc) return rc;
      if (splits > 1) {
        rc = check(llm_attention_merge_clear(part_o, part_ml, out, plan->small_rows, plan->n_small, Hq, hd,
                                             splits, nullptr, 0, stream), K_MERGE);
        if (rc) return rc;
      }
    }
    if (plan->n_large && x2)
      return check(llm_attention_tcgen05_x2(q, out, st.rows, c.k, c.v, c.page_stride, c.n_pages,
                                            c.block_table, c.table_stride, plan->large, plan->n_large, Hq, Hkv,
                                            hd, ps, L.scale, window, st.status, stream), K_TCGEN05_X2);
    if (plan->n_large && tc) {
      const int persistent = reach <= PERSISTENT_ATTENTION_MAX_KEYS ? 1 : 0;
      const int* direct = plan->large;
      int n_direct = plan->n_large;
      if (g_gather && ps < 32 && GATHER_PAGE % ps == 0 && !plan->large_host.empty()) {
        // pages too small for TMA boxes: long portions read gathered copies of their requests' keys
        const GatherPlan* gp = nullptr;
        rc = gather_for(*plan, ps, window, &gp);
        if (rc) return rc;
        if (gp->n_requests) {
          const int D = GATHER_PAGE;
          const long long stride = 2LL * Hkv * D * hd;
          void* scratch = nullptr;
          rc = buffer(B_GATHER, (size_t)gp->scratch_pages * stride * 2, &scratch);
          if (rc) return rc;
          bf16* ks = (bf16*)scratch;
          bf16* vs = ks + (size_t)Hkv * D * hd;
          rc = check(llm_kv_gather(c.k, c.v, c.page_stride, c.block_table, c.table_stride, ps, ks, vs, stride, D,
                                   Hkv, hd, LLM_BF16, gp->list, gp->n_requests, gp->total_chunks, stream),
                     K_KV_GATHER);
          if (rc) return rc;
          rc = check(llm_attention_tcgen05(q, out, st.rows, ks, vs, stride, gp->scratch_pages, gp->table,
                                           gp->table_stride, gp->gathered, gp->n_gathered, Hq, Hkv, hd, D, L.scale,
                                           window, persistent, st.status, stream), K_TCGEN05);
          if (rc) return rc;
          direct = gp->direct;
          n_direct = gp->n_direct;
        }
      }
      if (n_direct == 0) return 0;
      return check(llm_attention_tcgen05(q, out, st.rows, c.k, c.v, c.page_stride,
                                         c.storage != nullptr ? c.n_pages : 0, c.block_table, c.table_stride,
                                         direct, n_direct, Hq, Hkv, hd, ps, L.scale, window, persistent,
                                         st.status, stream), K_TCGEN05);
    }
    if (plan->n_large)
      return check(llm_attention_flash(q, out, nullptr, nullptr, c.k, c.v, c.page_stride, c.block_table,
                                       c.table_stride, plan->large, nullptr, nullptr, plan->n_large, 64, Hq,
                                       Hkv, hd, ps, L.scale, window, 1, stream), K_FLASH);
    return 0;
  }

  // the mixer: projections, per-head norm, rotation, cache write, attention, output projection
  int mixer(const LlmLayerDesc& L, const LlmCallDesc& c, const void* h, float* x) {
    const int rows = st.rows, Hq = L.num_heads, Hkv = L.num_kv_heads, hd = L.head_dim;
    const int q_width = Hq * hd, kv_width = Hkv * hd, dt = st.dtype;
    const int width = q_width + (c.writes_cache ? 2 * kv_width : 0);
    // With few rows the product is cut along K and adds its partial sums into a buffer that is
    // kept at zero: created as zeros, cleared again by the kernel that consumes it.
    const bool kept_zero = rows <= SPLIT_K_MAX_ROWS;
    void* proj = nullptr;
    int rc = buffer(kept_zero ? B_ZPROJ * 1000000LL + width : (long long)B_PROJ, (size_t)rows * width * 4, &proj,
                    kept_zero);
    if (rc) return rc;
    rc = linear(h, dt, L.hidden, L.w_qkv, L.w_qkv_dtype, L.hidden, proj, LLM_F32, width, rows, width, L.hidden,
                false, kept_zero);
    if (rc) return rc;
    const float* cos_sin = nullptr;
    rc = rope_table(L, &cos_sin);
    if (rc) return rc;
    void *out = nullptr, *q = nullptr;
    rc = buffer(B_OUT, (size_t)rows * q_width * esize(dt), &out);
    if (rc) return rc;
    rc = buffer(B_Q, (size_t)rows * q_width * esize(dt), &q);
    if (rc) return rc;
    const bool use_norm = L.q_norm_w != nullptr;
    if (fusion_ok(L, c, cos_sin)) {
      const int reach = L.window ? (st.max_pos + 1 < L.window ? st.max_pos + 1 : L.window) : st.max_pos + 1;
      const int splits = llm_decode_splits(rows, Hkv, reach, DECODE_TMA_CTAS_PER_SM * sm_count(), DECODE_TMA_TILE);
      float *part_o, *part_ml;
      rc = parts(splits, L, &part_o, &part_ml);
      if (rc) return rc;
      rc = check(llm_attention_decode_fused(
          (float*)proj, width, out, part_o, part_ml, c.storage, c.n_pages, c.n_slots, c.slot,
          c.writes_cache ? c.k : nullptr, c.writes_cache ? c.v : nullptr, c.page_stride, c.block_table,
          c.table_stride, st.row_slot, st.row_pos, rows, L.q_norm_w, L.k_norm_w, cos_sin,
          use_norm ? L.qk_norm_eps : 0.f, kept_zero ? 1 : 0, Hq, Hkv, hd, c.page_size, L.scale, L.window, splits,
          st.status, stream), K_DECODE_FUSED);
      if (rc) return rc;
      if (splits > 1) {
        rc = check(llm_attention_merge_clear(part_o, part_ml, out, nullptr, rows, Hq, hd, splits,
                                             kept_zero ? (float*)proj : nullptr, kept_zero ? width : 0, stream), K_MERGE);
        if (rc) return rc;
      }
    } else {
      rc = check(llm_qk_norm_rope_store((const float*)proj, width, q, c.writes_cache ? c.k : nullptr,
                                        c.writes_cache ? c.v : nullptr, dt, c.page_stride, c.block_table,
                                        c.table_stride, st.row_slot, st.row_pos, L.q_norm_w, L.k_norm_w,
                                        L.inv_freq, cos_sin, L.attn_factor, rows, Hq, Hkv, hd, L.rot_dim,
                                        c.page_size, use_norm ? L.qk_norm_eps : 0.f, c.writes_cache ? 1 : 0,
                                        use_norm ? 1 : 0, kept_zero ? 1 : 0, stream), K_ROPE_STORE);
      if (rc) return rc;
      rc = attention(L, c, q, out);
      if (rc) return rc;
    }
    return linear(out, dt, q_width, L.w_o, L.w_o_dtype, q_width, x, LLM_F32, L.hidden, rows, L.hidden, q_width, true,
                  false);
  }

  // down(silu(gate h) * (up h)) added into x (kernels.gate_up_silu and the down product)
  int feed_forward(const LlmLayerDesc& L, const void* h, float* x) {
    const int rows = st.rows, dt = st.dtype, ff = L.intermediate;
    void* act = nullptr;
    int rc = buffer(B_ACT, (size_t)rows * ff * esize(dt), &act);
    if (rc) return rc;
    const bool tc = tc_ok(h, dt, L.hidden, L.w_gate_up, L.w_gate_up_dtype, L.hidden, L.hidden);
    if (L.interleaved && !tc) return LLM_ERR_UNSUPPORTED;
    if (tc) {
      rc = check(llm_gemm_tcgen05(h, L.w_gate_up, act, dt, rows, 2 * ff, L.hidden, L.hidden, L.hidden, ff,
                                  L.interleaved ? 3 : 2, ff, llm_token_tile(rows), 1, 0, st.status, stream), K_GEMM_TCGEN05);
    } else {
      void* gu = nullptr;
      rc = buffer(B_GATE_UP, (size_t)rows * 2 * ff * 4, &gu);
      if (rc) return rc;
      rc = linear(h, dt, L.hidden, L.w_gate_up, L.w_gate_up_dtype, L.hidden, gu, LLM_F32, 2 * ff, rows, 2 * ff,
                  L.hidden, false, false);
      if (rc) return rc;
      rc = check(llm_silu_mul((const float*)gu, act, dt, rows, ff, stream), K_SILU_MUL);
    }
    if (rc) return rc;
    return linear(act, dt, ff, L.w_down, L.w_down_dtype, ff, x, LLM_F32, L.hidden, rows, L.hidden, ff, true, false);
  }

  int layer(const LlmLayerDesc& L, const LlmCallDesc& c) {
    void* h = nullptr;
    int rc = buffer(B_H, (size_t)st.rows * L.hidden * esize(st.dtype), &h);
    if (rc) return rc;
    rc = check(llm_rms_norm(st.x, L.mixer_norm_w, h, st.dtype, nullptr, st.rows, L.hidden, L.mixer_norm_eps, stream), K_NORM);
    if (rc) return rc;
    rc = mixer(L, c, h, st.x);
    if (rc) return rc;
    rc = check(llm_rms_norm(st.x, L.ffn_norm_w, h, st.dtype, nullptr, st.rows, L.hidden, L.ffn_norm_eps, stream), K_NORM);
    if (rc) return rc;
    return feed_forward(L, h, st.x);
  }
};

}  // namespace

// ---- policies, exported so that the Python statement of the same rules can be held to them
LLM_EXPORT int llm_token_tile(int rows) {
  for (int bn = 16; bn <= 128; bn *= 2)
    if (rows <= bn) return bn;
  return rows >= 512 ? 256 : 128;
}

LLM_EXPORT int llm_k_splits(int rows, int out_features, int in_features) {
  const int sms = sm_count();
  const int tiles = ceil_div(out_features, 128) * ceil_div(rows, llm_token_tile(rows));
  if (tiles >= 2 * sms - 40) return 1;
  // two CTAs fit an SM: aim at one full wave of two CTAs per SM, at least 256 of K each
  int s = (int)nearbyint(2.0 * sms / tiles);       // ties to even, as Python's round()
  if (s > 16) s = 16;
  if (s > in_features / 256) s = in_features / 256;
  return s < 1 ? 1 : s;
}

LLM_EXPORT int llm_decode_splits(int n_items, int num_kv_heads, int max_len, int resident, int tile) {
  const int ctas = n_items * num_kv_heads < 1 ? 1 : n_items * num_kv_heads;
  const int tiles = ceil_div(max_len, tile) < 1 ? 1 : ceil_div(max_len, tile);
  int most = max_len / 64 < 1 ? 1 : max_len / 64;
  if (most > 32) most = 32;
  int best = 1;
  double best_cost = -1.0;
  for (int s = 1; s <= most; ++s) {
    const int waves = ceil_div(ctas * s, resident);
    const double cost = waves * (double)(ceil_div(tiles, s) * (tile / 32) + 3) + 0.1 * s;
    if (best_cost < 0 || cost < best_cost - 1e-9) {
      best = s;
      best_cost = cost;
    }
  }
  return best;
}

LLM_EXPORT void llm_set_fuse_decode(int mode) { g_fuse_mode = mode; }

// How often the driver launched which kind of kernel since the library was loaded, in the order
// of `Kind`; returns the number of kinds.
LLM_EXPORT int llm_driver_counts(long long* out, int cap) {
  for (int i = 0; i < N_KINDS && i < cap; ++i) out[i] = g_counts[i];
  return N_KINDS;
}

LLM_EXPORT long long llm_arena_generation() { return arena().generation; }

// Forget every buffer of the arena (after a step that failed: a buffer kept at zero may hold
// partial sums).  Synchronises the device.
LLM_EXPORT int llm_arena_drop() {
  cudaError_t e = cudaDeviceSynchronize();
  arena().drop();
  return (int)e;
}

// Run calls[0..n_calls) in order on the residual stream step->x.  *n_launches: kernels launched.
LLM_EXPORT int llm_run_layers(const LlmLayerDesc* layers, const LlmCallDesc* calls, int n_calls,
                              const LlmStepDesc* step, int* n_launches, cudaStream_t stream) {
  if (n_launches) *n_launches = 0;
  if (n_calls <= 0 || step->rows <= 0) return 0;
  if (!step->all_single && (step->segments == nullptr || step->n_segments <= 0)) return LLM_ERR_ARGUMENT;
  Run run(*step, stream, step_cache(step->step_id));
  int rc = 0;
  for (int i = 0; i < n_calls && rc == 0; ++i) rc = run.layer(layers[calls[i].layer], calls[i]);
  if (n_launches) *n_launches = run.launches;
  return rc;
}

// The attention of one layer call by itself, for mixers that are driven from Python: q and out
// [rows][heads * head_dim] in the step's dtype; of `layer` only the sizes, the scale and the window
// are read.  The same choices as inside llm_run_layers.
LLM_EXPORT int llm_attention_step(const LlmLayerDesc* layer, const LlmCallDesc* call, const LlmStepDesc* step,
                                  const void* q, void* out, int* n_launches, cudaStream_t stream) {
  if (n_launches) *n_launches = 0;
  if (step->rows <= 0) return 0;
  if (!step->all_single && (step->segments == nullptr || step->n_segments <= 0)) return LLM_ERR_ARGUMENT;
  Run run(*step, stream, step_cache(step->step_id));
  const int rc = run.attention(*layer, *call, q, out);
  if (n_launches) *n_launches = run.launches;
  return rc;
}

LLM_EXPORT void llm_set_gather(int on) { g_gather = on ? 1 : 0; }
LLM_EXPORT void llm_set_persistent_decode(int on) { g_persistent_decode = on ? 1 : 0; }

// Fill every temporary buffer of the arena (not those that are kept at zero) with `byte`.  For
// tests: with 0xff every 16- and 32-bit value is a NaN, so a kernel that reads what nothing wrote
// in this step shows up in the result.  Synchronises the device.
LLM_EXPORT int llm_arena_fill(int byte) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return (int)e;
  for (auto& kv : arena().bufs)
    if (kv.second.p && !kv.second.kept_zero) {
      e = cudaMemset(kv.second.p, byte, kv.second.bytes);
      if (e != cudaSuccess) return (int)e;
    }
  return (int)cudaDeviceSynchronize();
}
