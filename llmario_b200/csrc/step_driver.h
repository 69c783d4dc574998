// What the native step driver (step_driver.cu) is told: plain C structures that the Python side
// fills through ctypes (llmario_b200/engine/native.py mirrors them field by field).
#pragma once
#include <cuda_runtime.h>

extern "C" {

// One standard layer: pre-norm residual block of grouped-query attention (optional per-head
// q/k norm, optional half-split rotation) and a gated feed-forward.  Matrices are [out][in],
// row-major; dtypes are LlmDtype values (0 float32, 1 bfloat16).
struct LlmLayerDesc {
  int hidden;
  int num_heads, num_kv_heads, head_dim;
  int window;              // 0: every earlier key
  int rot_dim;             // 0: no rotation
  int intermediate;
  int interleaved;         // gate and up rows stored as alternating blocks of 16
  int w_qkv_dtype, w_o_dtype, w_gate_up_dtype, w_down_dtype;
  float scale, attn_factor;
  float mixer_norm_eps, ffn_norm_eps, qk_norm_eps;
  float pad_;
  const float* mixer_norm_w;
  const float* ffn_norm_w;
  const float* q_norm_w;   // null: no per-head norm
  const float* k_norm_w;
  const float* inv_freq;   // [rot_dim / 2]; layers with the same constants share one table
  const void* w_qkv;       // [(heads + 2 kv heads) * head_dim][hidden]
  const void* w_o;         // [hidden][heads * head_dim]
  const void* w_gate_up;   // [2 * intermediate][hidden]
  const void* w_down;      // [hidden][intermediate]
};

// One run-order entry: which layer, and where its keys and values live.
struct LlmCallDesc {
  int layer;               // index into the layers array
  int writes_cache;        // 0: it reads the cache of an earlier entry and projects only queries
  int table_stride, page_size;
  int n_slots, slot;       // cache slots of the group's storage, and this entry's
  long long page_stride;   // elements from one page to the next
  long long n_pages;
  void* k;                 // this entry's K plane of page 0
  void* v;
  const int* block_table;
  void* storage;           // the group's whole tensor (contiguous), or null
};

// One step.
struct LlmStepDesc {
  int rows;
  int max_pos;             // largest position in the step (its context bucket in a recorded step)
  int n_segments;
  int all_single;          // every request of the step has one row
  int dtype;               // dtype of activations between parts
  int pad_;
  long long step_id;       // names the step: what is made once per step is kept under it (-1: keep nothing)
  const int* segments;     // host: n_segments x (first row, rows, request slot, first position)
  const int* tokens;       // device int32 [rows]
  const int* row_pos;
  const int* row_slot;
  float* x;                // the residual stream, float32 [rows][hidden]
  int* status;             // the library's status words
};

int llm_token_tile(int rows);
int llm_k_splits(int rows, int out_features, int in_features);
int llm_decode_splits(int n_items, int num_kv_heads, int max_len, int resident, int tile);
void llm_set_fuse_decode(int mode);
int llm_driver_counts(long long* out, int cap);
long long llm_arena_generation();
int llm_arena_drop();
int llm_attention_step(const LlmLayerDesc* layer, const LlmCallDesc* call, const LlmStepDesc* step,
                       const void* q, void* out, int* n_launches, cudaStream_t stream);
void llm_set_gather(int on);
void llm_set_persistent_decode(int on);
int llm_arena_fill(int byte);
int llm_run_layers(const LlmLayerDesc* layers, const LlmCallDesc* calls, int n_calls,
                   const LlmStepDesc* step, int* n_launches, cudaStream_t stream);
}
