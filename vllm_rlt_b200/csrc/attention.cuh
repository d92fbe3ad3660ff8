// Argument block and row addressing shared by the attention kernels.
#pragma once

#include "common.cuh"

namespace rlt {

struct AttentionArgs {
  const void* q;
  void* out;
  const void* key_cache;
  const void* value_cache;
  int64_t block_stride;   // elements between consecutive physical blocks of this layer view
  int64_t token_stride;   // elements between consecutive tokens inside a block
  int64_t num_blocks;
  int block_size;
  int q_heads;
  int kv_heads;
  int head_dim;
  int dtype;
  const int32_t* block_tables;  // [table_rows, table_width]
  int table_rows;
  int table_width;
  const int32_t* context_lengths;
  const int32_t* cu_seqlens_q;  // nullptr: one table row per query row
  int rows;
};

// Table row and number of visible keys of query row `row`.
// Unpacked: its own table row and context length.  Packed: the sequence s that contains
// the row, and context_lengths[s] - n_s + i + 1 for its i-th of n_s rows.
// The lengths live on the device (graph replays change them without the host seeing them), so
// a length beyond what the row's table can address (table_width * block_size tokens) is
// clamped here: no kernel ever indexes a table row past its width.  `*clamped` (optional) is
// set when that happened, so that the caller can report it.
__device__ __forceinline__ void resolve_row(const AttentionArgs& a, int row, int* table_row, int* len,
                                            bool* clamped = nullptr) {
  const int64_t capacity64 = static_cast<int64_t>(a.table_width) * a.block_size;
  const int capacity = capacity64 > 0x7fffffff ? 0x7fffffff : static_cast<int>(capacity64);
  int n;
  if (a.cu_seqlens_q == nullptr) {
    *table_row = row;
    n = a.context_lengths[row];
  } else {
    int lo = 0, hi = a.table_rows - 1;  // last s with cu[s] <= row
    while (lo < hi) {
      int mid = (lo + hi + 1) >> 1;
      if (a.cu_seqlens_q[mid] <= row) lo = mid; else hi = mid - 1;
    }
    const int first = a.cu_seqlens_q[lo], count = a.cu_seqlens_q[lo + 1] - first;
    *table_row = lo;
    n = a.context_lengths[lo] - count + (row - first) + 1;
  }
  if (n > capacity) {
    n = capacity;
    if (clamped != nullptr) *clamped = true;
  }
  *len = n > 0 ? n : 0;
}

// attention_generic.cu: any shape, one CTA per (row, head).
int launch_attention_generic(const AttentionArgs& a, cudaStream_t stream, int window = 0);   // window > 0: the row's last `window` keys only

// attention_sm100.cu: head_dim 128, 16-token pages, fp16/bf16 — TMA page streaming,
// request-grouped rows on tensor cores, split-KV with a deterministic merge.
bool attention_sm100_supported(const AttentionArgs& a);        // shape and cache view
bool attention_sm100_shape_supported(const AttentionArgs& a);  // shape only (enough to plan)
size_t attention_sm100_workspace_bytes(int rows, int q_heads, int kv_heads, int head_dim,
                                       int block_size, int table_width);
int launch_attention_sm100(const AttentionArgs& a, void* workspace, size_t workspace_bytes,
                           cudaStream_t stream);
// The two halves of launch_attention_sm100: the plan depends only on the block tables, lengths
// and packing; a run consumes it and leaves it intact for the next layer.
int plan_attention_sm100(const AttentionArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t stream);
int run_attention_sm100(const AttentionArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t stream);
// launch_attention_sm100 on the library's built-in 32 MiB scratch block (no allocation anywhere).
size_t attention_sm100_builtin_scratch_bytes();
int launch_attention_sm100_builtin(const AttentionArgs& a, cudaStream_t stream);
int attention_sm100_builtin_warmup();
// attention_prefill_sm100.cu: packed causal prefill (tcgen05 kernels with 256 / 128 query tokens
// per CTA, an mma.sync one with 64), the same shapes.
bool prefill_sm100_supported(const AttentionArgs& a);
size_t prefill_sm100_workspace_bytes(int rows, int seqs);
int launch_prefill_sm100(const AttentionArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t stream);
// Synchronous read-back of the workspace header of the last tiled call:
// {work items planned, rows of length zero, error bits, claim counter (0 after a clean run)}.
int attention_sm100_read_status(const void* workspace, cudaStream_t stream, unsigned* out4);

}  // namespace rlt
