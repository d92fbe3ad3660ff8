// C-ABI entry of the verify attention: argument checks and kernel selection.
#include "attention.cuh"

namespace rlt {
namespace {

int check_metadata(const AttentionArgs& a) {
  RLT_REQUIRE(dtype_valid(a.dtype), "verify_attention: dtype must be float32, float16 or bfloat16");
  RLT_REQUIRE(a.rows >= 0 && a.q_heads > 0 && a.kv_heads > 0 && a.head_dim > 0 && a.block_size > 0,
              "verify_attention: invalid shape");
  RLT_REQUIRE(a.q_heads % a.kv_heads == 0,
              "verify_attention: query heads must be a positive multiple of KV heads");
  if (a.rows == 0) return RLT_OK;
  RLT_REQUIRE(a.block_tables && a.context_lengths, "verify_attention: null pointer");
  RLT_REQUIRE(a.table_rows > 0 && a.table_width > 0,
              "verify_attention: block tables must be int32 [rows, pages] with pages > 0");
  RLT_REQUIRE(a.cu_seqlens_q != nullptr || a.table_rows == a.rows,
              "verify_attention: one block-table row per query row unless cu_seqlens_q is given");
  return RLT_OK;
}

int check_args(const AttentionArgs& a) {
  RLT_REQUIRE(dtype_valid(a.dtype), "verify_attention: dtype must be float32, float16 or bfloat16");
  RLT_REQUIRE(a.rows >= 0 && a.q_heads > 0 && a.kv_heads > 0 && a.head_dim > 0 && a.block_size > 0,
              "verify_attention: invalid shape");
  RLT_REQUIRE(a.q_heads % a.kv_heads == 0,
              "verify_attention: query heads must be a positive multiple of KV heads");
  if (a.rows == 0) return RLT_OK;
  RLT_REQUIRE(a.q && a.out && a.key_cache && a.value_cache && a.block_tables && a.context_lengths,
              "verify_attention: null pointer");
  RLT_REQUIRE(a.table_rows > 0 && a.table_width > 0 && a.num_blocks > 0,
              "verify_attention: block tables must be int32 [rows, pages] with pages > 0");
  RLT_REQUIRE(a.cu_seqlens_q != nullptr || a.table_rows == a.rows,
              "verify_attention: one block-table row per query row unless cu_seqlens_q is given");
  RLT_REQUIRE(a.token_stride >= static_cast<int64_t>(a.kv_heads) * a.head_dim &&
                  a.block_stride >= a.token_stride * a.block_size,
              "verify_attention: cache view must be [blocks, block_size, kv_heads, head_dim] with a "
              "contiguous [kv_heads, head_dim] tail");
  return RLT_OK;
}

}  // namespace
}  // namespace rlt

extern "C" RLT_API size_t rlt_verify_attention_workspace_bytes(int rows, int q_heads, int kv_heads, int head_dim,
                                                       int block_size, int table_width) {
  if (rows <= 0 || q_heads <= 0 || kv_heads <= 0 || table_width <= 0 || block_size <= 0) return 256;
  return rlt::attention_sm100_workspace_bytes(rows, q_heads, kv_heads, head_dim, block_size, table_width);
}

extern "C" RLT_API int rlt_verify_attention(const void* q, void* out, const void* key_cache, const void* value_cache,
                                    int64_t block_stride, int64_t token_stride, int64_t num_blocks,
                                    int block_size, int q_heads, int kv_heads, int head_dim, int dtype,
                                    const int32_t* block_tables, int table_rows, int table_width,
                                    const int32_t* context_lengths, const int32_t* cu_seqlens_q, int rows,
                                    void* workspace, size_t workspace_bytes, rlt_stream_t stream) {
  using namespace rlt;
  AttentionArgs a;
  a.q = q; a.out = out; a.key_cache = key_cache; a.value_cache = value_cache;
  a.block_stride = block_stride; a.token_stride = token_stride; a.num_blocks = num_blocks;
  a.block_size = block_size; a.q_heads = q_heads; a.kv_heads = kv_heads; a.head_dim = head_dim;
  a.dtype = dtype; a.block_tables = block_tables; a.table_rows = table_rows; a.table_width = table_width;
  a.context_lengths = context_lengths; a.cu_seqlens_q = cu_seqlens_q; a.rows = rows;
  int status = check_args(a);
  if (status != RLT_OK || rows == 0) return status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (attention_sm100_supported(a)) return launch_attention_sm100(a, workspace, workspace_bytes, s);
  return launch_attention_generic(a, s);
}

extern "C" RLT_API int rlt_windowed_attention(const void* q, void* out, const void* key_cache, const void* value_cache,
                                              int64_t block_stride, int64_t token_stride, int64_t num_blocks,
                                              int block_size, int q_heads, int kv_heads, int head_dim, int dtype,
                                              const int32_t* block_tables, int table_width,
                                              const int32_t* context_lengths, int rows, int window,
                                              rlt_stream_t stream) {
  using namespace rlt;
  RLT_REQUIRE(window > 0, "windowed_attention: window must be a positive integer");
  AttentionArgs a;
  a.q = q; a.out = out; a.key_cache = key_cache; a.value_cache = value_cache;
  a.block_stride = block_stride; a.token_stride = token_stride; a.num_blocks = num_blocks;
  a.block_size = block_size; a.q_heads = q_heads; a.kv_heads = kv_heads; a.head_dim = head_dim;
  a.dtype = dtype; a.block_tables = block_tables; a.table_rows = rows; a.table_width = table_width;
  a.context_lengths = context_lengths; a.cu_seqlens_q = nullptr; a.rows = rows;
  int status = check_args(a);
  if (status != RLT_OK || rows == 0) return status;
  return launch_attention_generic(a, static_cast<cudaStream_t>(stream), window);
}

extern "C" RLT_API int rlt_verify_attention_plan(const int32_t* block_tables, int table_rows, int table_width,
                                                 const int32_t* context_lengths, const int32_t* cu_seqlens_q,
                                                 int rows, int q_heads, int kv_heads, int head_dim, int block_size,
                                                 int dtype, void* workspace, size_t workspace_bytes,
                                                 rlt_stream_t stream) {
  using namespace rlt;
  AttentionArgs a = {};
  a.block_tables = block_tables; a.table_rows = table_rows; a.table_width = table_width;
  a.context_lengths = context_lengths; a.cu_seqlens_q = cu_seqlens_q; a.rows = rows;
  a.q_heads = q_heads; a.kv_heads = kv_heads; a.head_dim = head_dim; a.block_size = block_size; a.dtype = dtype;
  int status = check_metadata(a);
  if (status != RLT_OK || rows == 0) return status;
  if (!attention_sm100_shape_supported(a)) {
    set_last_error_text("verify_attention_plan: only the tiled kernel (head_dim 128, 16-token pages, fp16/bf16) plans");
    return RLT_ERR_UNSUPPORTED;
  }
  return plan_attention_sm100(a, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" RLT_API int rlt_verify_attention_run(const void* q, void* out, const void* key_cache,
                                                const void* value_cache, int64_t block_stride, int64_t token_stride,
                                                int64_t num_blocks, int block_size, int q_heads, int kv_heads,
                                                int head_dim, int dtype, const int32_t* block_tables, int table_rows,
                                                int table_width, const int32_t* context_lengths,
                                                const int32_t* cu_seqlens_q, int rows, void* workspace,
                                                size_t workspace_bytes, rlt_stream_t stream) {
  using namespace rlt;
  AttentionArgs a;
  a.q = q; a.out = out; a.key_cache = key_cache; a.value_cache = value_cache;
  a.block_stride = block_stride; a.token_stride = token_stride; a.num_blocks = num_blocks;
  a.block_size = block_size; a.q_heads = q_heads; a.kv_heads = kv_heads; a.head_dim = head_dim;
  a.dtype = dtype; a.block_tables = block_tables; a.table_rows = table_rows; a.table_width = table_width;
  a.context_lengths = context_lengths; a.cu_seqlens_q = cu_seqlens_q; a.rows = rows;
  int status = check_args(a);
  if (status != RLT_OK || rows == 0) return status;
  if (!attention_sm100_supported(a)) {
    set_last_error_text("verify_attention_run: this shape or cache view is not covered by the tiled kernel");
    return RLT_ERR_UNSUPPORTED;
  }
  return run_attention_sm100(a, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" RLT_API int rlt_verify_attention_status(const void* workspace, rlt_stream_t stream, uint32_t* status4) {
  using namespace rlt;
  RLT_REQUIRE(workspace != nullptr && status4 != nullptr, "verify_attention_status: null pointer");
  return attention_sm100_read_status(workspace, static_cast<cudaStream_t>(stream), status4);
}

extern "C" RLT_API int rlt_verify_attention_noalloc(const void* q, void* out, const void* key_cache,
                                                    const void* value_cache, int64_t block_stride,
                                                    int64_t token_stride, int64_t num_blocks, int block_size,
                                                    int q_heads, int kv_heads, int head_dim, int dtype,
                                                    const int32_t* block_tables, int table_rows, int table_width,
                                                    const int32_t* context_lengths, const int32_t* cu_seqlens_q,
                                                    int rows, rlt_stream_t stream) {
  using namespace rlt;
  AttentionArgs a;
  a.q = q; a.out = out; a.key_cache = key_cache; a.value_cache = value_cache;
  a.block_stride = block_stride; a.token_stride = token_stride; a.num_blocks = num_blocks;
  a.block_size = block_size; a.q_heads = q_heads; a.kv_heads = kv_heads; a.head_dim = head_dim;
  a.dtype = dtype; a.block_tables = block_tables; a.table_rows = table_rows; a.table_width = table_width;
  a.context_lengths = context_lengths; a.cu_seqlens_q = cu_seqlens_q; a.rows = rows;
  int status = check_args(a);
  if (status != RLT_OK) return status;
  // A call without rows is the warm-up: it loads the library's device image (and with it the
  // built-in block) and resolves the block's address for the current device, and launches nothing.
  if (rows == 0) return attention_sm100_builtin_warmup();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (attention_sm100_supported(a)) return launch_attention_sm100_builtin(a, s);
  return launch_attention_generic(a, s);  // shapes outside the tiled kernel use no scratch at all
}

extern "C" RLT_API size_t rlt_prefill_attention_workspace_bytes(int rows, int sequences, int q_heads, int kv_heads,
                                                                int head_dim, int block_size, int table_width) {
  if (rows <= 0 || sequences <= 0) return 256;
  // The prompt kernels' own scratch where they are the expected path; the grouped kernel's (which grows with
  // rows x heads x context chunks: gigabytes for a batch of prompts) only for shapes they do not cover.
  if (head_dim == 128 && block_size == 16) return rlt::prefill_sm100_workspace_bytes(rows, sequences);
  return rlt_verify_attention_workspace_bytes(rows, q_heads, kv_heads, head_dim, block_size, table_width);
}

extern "C" RLT_API int rlt_prefill_attention(const void* q, void* out, const void* key_cache, const void* value_cache,
                                             int64_t block_stride, int64_t token_stride, int64_t num_blocks,
                                             int block_size, int q_heads, int kv_heads, int head_dim, int dtype,
                                             const int32_t* block_tables, int sequences, int table_width,
                                             const int32_t* context_lengths, const int32_t* cu_seqlens_q, int rows,
                                             void* workspace, size_t workspace_bytes, rlt_stream_t stream) {
  using namespace rlt;
  AttentionArgs a;
  a.q = q; a.out = out; a.key_cache = key_cache; a.value_cache = value_cache;
  a.block_stride = block_stride; a.token_stride = token_stride; a.num_blocks = num_blocks;
  a.block_size = block_size; a.q_heads = q_heads; a.kv_heads = kv_heads; a.head_dim = head_dim;
  a.dtype = dtype; a.block_tables = block_tables; a.table_rows = sequences; a.table_width = table_width;
  a.context_lengths = context_lengths; a.cu_seqlens_q = cu_seqlens_q; a.rows = rows;
  RLT_REQUIRE(cu_seqlens_q != nullptr || rows == 0, "prefill_attention: cu_seqlens_q is required");
  int status = check_args(a);
  if (status != RLT_OK || rows == 0) return status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (prefill_sm100_supported(a)) {
    status = launch_prefill_sm100(a, workspace, workspace_bytes, s);
    if (status != RLT_ERR_UNSUPPORTED) return status;
  }
  // shapes or cache placements outside the tiled prefill kernel: the grouped verify kernel (which reports
  // RLT_ERR_WORKSPACE when the scratch was sized for the prompt kernels only), or the generic one
  if (attention_sm100_supported(a)) return launch_attention_sm100(a, workspace, workspace_bytes, s);
  return launch_attention_generic(a, s);
}
