/*
 * rlt_verify.h — C ABI of the B200 (sm_100a) self-speculative verify step for
 * looped (Ouro-style) language models.
 *
 * Every entry point takes plain pointers and sizes, launches on the CUDA stream
 * it is given (no host synchronisation, no host read of device data, static
 * launch geometry, so calls can be captured in a CUDA graph), borrows its
 * pointer arguments for the lifetime of the work on that stream, and returns
 * an int status: RLT_OK or a negative RLT_ERR_* code.  No exception crosses
 * this boundary.  The library keeps no mutable global state besides a
 * per-device cache of immutable properties (SM count, driver entry points)
 * and the fixed scratch block of rlt_verify_attention_noalloc, which is the one
 * piece of device memory the library owns (see that entry point).
 *
 * Each declaration cites the reference interface (vllm-rlt v0.2.0, paths
 * relative to that project) it stands in for; the few entry points without a
 * counterpart there say so.
 *
 * Element type codes (`dtype` arguments): see rlt_dtype.
 */
#ifndef RLT_VERIFY_H_
#define RLT_VERIFY_H_

#include <stdint.h>
#include <stddef.h>

#if defined(__GNUC__)
#define RLT_API __attribute__((visibility("default")))
#else
#define RLT_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Opaque CUDA stream handle (cudaStream_t / CUstream); NULL = legacy default stream. */
typedef void* rlt_stream_t;

typedef enum rlt_dtype {
  RLT_F32 = 0,
  RLT_F16 = 1,
  RLT_BF16 = 2
} rlt_dtype;

enum {
  RLT_OK = 0,
  RLT_ERR_INVALID = -1,     /* bad argument (shape, alignment, null pointer, range) */
  RLT_ERR_UNSUPPORTED = -2, /* valid request that this build has no kernel for        */
  RLT_ERR_CUDA = -3,        /* a CUDA runtime / driver call failed (see rlt_last_error) */
  RLT_ERR_WORKSPACE = -4    /* workspace missing or too small                          */
};

/* Per-request status words written by the acceptance kernels. */
enum {
  RLT_ROW_OK = 0,
  RLT_ROW_ZERO_PROPOSAL = 1,    /* q[candidate] == 0: ValueError in worker/speculative.py:53-55      */
  RLT_ROW_INVALID_RESIDUAL = 2, /* residual mass zero / non-finite: RuntimeError, speculative.py:61-62 */
  RLT_ROW_BAD_LOGITS = 3,       /* NaN / +inf in a logits row that had to be normalised               */
  RLT_ROW_SHARED_PAGE = 4,      /* rollback would truncate a page with refcount > 1,
                                   core/kv_cache_manager.py:349-351                                    */
  RLT_ROW_BAD_POSITION = 5      /* position outside the request's block table                         */
};

/* Library / build identification: "rlt_verify <version> sm_100a". */
RLT_API const char* rlt_version(void);
/* Text of the most recent CUDA error seen by this thread in this library ("" if none). */
RLT_API const char* rlt_last_error(void);

/* ------------------------------------------------------------------------
 * SiLU-and-Mul.  out[i] = T(silu_f32(f32(gate[i]))) * up[i], the activation
 * rounded to T before the multiply, the multiply rounded once to T.
 * Replaces: torch.ops.vllm_rlt.silu_and_mul -> vllm_rlt::silu_and_mul_cuda
 *   (csrc/torch_bindings.cpp:7-13, csrc/activation/silu_and_mul.cu:220-247;
 *    arithmetic contract csrc/activation/silu_and_mul.cu:20-22,74-79;
 *    Python reference vllm_rlt/kernels/activation.py:20-28).
 * gate/up/out: `n` contiguous elements of `dtype`, any element alignment;
 * out must not alias the inputs.  n == 0 launches nothing.
 * ---------------------------------------------------------------------- */
RLT_API int rlt_silu_and_mul(const void* gate, const void* up, void* out, int64_t n,
                     int dtype, rlt_stream_t stream);

/* SiLU-and-Mul over the two column halves of one fused gate/up projection:
 *   out[r, c] = T(silu_f32(f32(gate_up[r, c]))) * gate_up[r, cols + c]
 * with the arithmetic of rlt_silu_and_mul (bit-identical results).  The reference's MLP runs gate_proj
 * and up_proj as two GEMMs on the same input (vllm_rlt/models/ouro.py:196-197); running them as one
 * GEMM over the concatenated weights leaves gate and up side by side in one [rows, 2 * cols] tensor,
 * which this entry reads in place.  gate_up: `rows` rows of `row_stride` elements (row_stride >=
 * 2 * cols); out: [rows, cols] contiguous.  No counterpart in the reference (its op takes two
 * contiguous tensors). */
RLT_API int rlt_silu_and_mul_packed(const void* gate_up, int64_t row_stride, void* out, int64_t rows,
                            int64_t cols, int dtype, rlt_stream_t stream);

/* ------------------------------------------------------------------------
 * KV write.  For each active row r: cache[write_blocks[r], write_offsets[r], :, :] = k[r]
 * (and v).  A row is active iff r < *active_rows (when active_rows != NULL) and
 * write_mask[r] != 0 (when write_mask != NULL); inactive rows load no address
 * and write nothing.
 * Replaces: KVCacheManager._write_prepared (vllm_rlt/core/kv_cache_manager.py:675-701),
 *   masked_kv_store (vllm_rlt/kernels/routing.py:180-225),
 *   write_graph_kv (vllm_rlt/kernels/graph_kv.py:6-65).
 * key_cache/value_cache: one layer's view [num_blocks, block_size, kv_heads, head_dim];
 *   block_stride and token_stride are in ELEMENTS; the [kv_heads, head_dim] tail is contiguous.
 * k, v: [rows, kv_heads, head_dim] contiguous.  write_blocks/write_offsets: int64 [rows].
 * write_mask: uint8/bool [rows] or NULL.  active_rows: device int32 scalar or NULL.
 * ---------------------------------------------------------------------- */
RLT_API int rlt_kv_write(void* key_cache, void* value_cache, int64_t block_stride, int64_t token_stride,
                 int64_t num_blocks, int block_size, int kv_heads, int head_dim, int dtype,
                 const void* k, const void* v, const int64_t* write_blocks,
                 const int64_t* write_offsets, const uint8_t* write_mask,
                 const int32_t* active_rows, int rows, rlt_stream_t stream);

/* ------------------------------------------------------------------------
 * Depth-aware paged-KV verify attention.
 *   out[r,h,:] = sum_t softmax_t(q[r,h,:].K[t,h/g,:] / sqrt(D)) V[t,h/g,:],  t in [0, len_r)
 *   K[t] = key_cache[table_r[t / block_size], t % block_size]
 * Rows whose block-table rows are identical (the k+1 rows of one request at
 * one depth plane, or k x depths rows in a shared-plane layout) are detected
 * on the device and scored together, so each K/V page is read from HBM once
 * per group instead of once per row.  A row's result is a function of its
 * own query, length and K/V only (bit-identical alone, in any batch and in
 * any group).  len_r == 0 gives a zero row and never dereferences its table.
 * Table entries at or beyond ceil(len_r / block_size) are never read as page ids
 * for that row.  The lengths are device data the host may never have seen (graph
 * replays), so a length beyond table_width * block_size is clamped to that capacity
 * instead of indexing past the table: the row is scored over the tokens its table
 * can address, and the tiled kernel records the event in the error word that
 * rlt_verify_attention_status reports (bit 1).  The reference's Torch path raises
 * IndexError for such a row; here the run stays in bounds and the host learns of it
 * afterwards.
 * Cache slots behind a context's last token (the rest of its last page, pages nobody owns)
 * may hold anything, NaN and Inf bit patterns included — the reference allocates its pools
 * uninitialised (vllm_rlt/core/kv_cache_manager.py:143-145): no result depends on them, here
 * and in rlt_prefill_attention and rlt_windowed_attention.
 * Replaces: TritonPagedAttention.__call__ / paged_attention
 *   (vllm_rlt/kernels/paged_attention.py:119-120, vllm_rlt/kernels/triton_attention.py:150-202,
 *    kernels :20-147); oracle torch_paged_attention (vllm_rlt/kernels/paged_attention.py:12-36);
 *   dispatch KVCacheManager._attend_prepared (vllm_rlt/core/kv_cache_manager.py:728-770).
 *
 * q, out: [rows, q_heads, head_dim] contiguous.  key_cache/value_cache as in rlt_kv_write.
 * block_tables: int32 [table_rows, table_width] contiguous.
 * context_lengths: int32 [rows] (unpacked) or [table_rows] (packed).
 * cu_seqlens_q: NULL for one table row per query row (table_rows == rows).
 *   Otherwise int32 [table_rows + 1]: query rows cu[s]..cu[s+1]-1 belong to table
 *   row s, are consecutive positions ending at context_lengths[s]-1, and row i of
 *   the n_s rows sees context_lengths[s] - n_s + i + 1 keys (bottom-right causal) —
 *   the packed form of AttentionBackend.prefill (vllm_rlt/attention/backend.py:41-42,
 *   vllm_rlt/kernels/triton_attention.py:314-366).
 * workspace: device scratch of at least rlt_verify_attention_workspace_bytes(...)
 *   bytes, 256-byte aligned, owned by the caller, private to this call until its
 *   work on `stream` completes.  Contents on entry are irrelevant.
 * ---------------------------------------------------------------------- */
RLT_API size_t rlt_verify_attention_workspace_bytes(int rows, int q_heads, int kv_heads, int head_dim,
                                            int block_size, int table_width);

RLT_API int rlt_verify_attention(const void* q, void* out, const void* key_cache, const void* value_cache,
                         int64_t block_stride, int64_t token_stride, int64_t num_blocks,
                         int block_size, int q_heads, int kv_heads, int head_dim, int dtype,
                         const int32_t* block_tables, int table_rows, int table_width,
                         const int32_t* context_lengths, const int32_t* cu_seqlens_q, int rows,
                         void* workspace, size_t workspace_bytes, rlt_stream_t stream);

/* ------------------------------------------------------------------------
 * The two halves of rlt_verify_attention, for callers that score many layers against the
 * same block tables and lengths (every layer of one recurrent depth pass shares them,
 * vllm_rlt/models/ouro.py:283-291): plan once, run once per layer.
 *   rlt_verify_attention_plan  groups the rows and builds the work list in `workspace`.
 *   rlt_verify_attention_run   scores q against one layer's K/V with that plan and leaves the
 *                              plan intact.  The block tables, lengths and packing must be the
 *                              ones that were planned (same contents, same workspace).
 * Both return RLT_ERR_UNSUPPORTED for shapes outside the tiled kernel (head_dim 128, 16-token
 * pages, fp16 / bf16, GQA ratio 1/2/4/8/16); use rlt_verify_attention for those.
 * rlt_verify_attention(...) == plan(...) followed by run(...).
 * ---------------------------------------------------------------------- */
RLT_API int rlt_verify_attention_plan(const int32_t* block_tables, int table_rows, int table_width,
                              const int32_t* context_lengths, const int32_t* cu_seqlens_q, int rows,
                              int q_heads, int kv_heads, int head_dim, int block_size, int dtype,
                              void* workspace, size_t workspace_bytes, rlt_stream_t stream);

RLT_API int rlt_verify_attention_run(const void* q, void* out, const void* key_cache, const void* value_cache,
                             int64_t block_stride, int64_t token_stride, int64_t num_blocks,
                             int block_size, int q_heads, int kv_heads, int head_dim, int dtype,
                             const int32_t* block_tables, int table_rows, int table_width,
                             const int32_t* context_lengths, const int32_t* cu_seqlens_q, int rows,
                             void* workspace, size_t workspace_bytes, rlt_stream_t stream);

/* ------------------------------------------------------------------------
 * rlt_verify_attention for hosts that are not allowed to allocate device memory.
 * It has no counterpart in the reference.
 *
 * Who needs it: an engine that gives every free byte of HBM to its KV pool at start-up can
 * find cudaMalloc failing for the rest of its life; a serving loop that must never stall
 * cannot afford the device-wide synchronisation an allocation implies; and a plugin that
 * runs under someone else's memory pool may simply have no allocator to call.  Such a caller
 * cannot provide the scratch workspace rlt_verify_attention asks for.  This entry point takes
 * the same inputs and outputs and no workspace: the scratch is a fixed 32 MiB block that is
 * part of the library image (so every GPU that loads the library holds those 32 MiB until
 * the process exits).  It calls no cudaMalloc, cudaFree or any other allocating routine.
 *
 * Limits and rules:
 *   - The batch must fit the block: rlt_verify_attention_workspace_bytes(rows, q_heads,
 *     kv_heads, head_dim, block_size, table_width) <= 32 MiB (for 16 heads x 128 that is,
 *     e.g., 64 rows with tables of up to 512 pages, or 400 rows with up to 64 pages).
 *     Anything larger is refused with RLT_ERR_WORKSPACE and a message in rlt_last_error();
 *     nothing is launched.
 *   - The first call on each device looks up the block's device address (with that device
 *     current); under CUDA's lazy module loading that is also when the 32 MiB are taken from
 *     the device.  A call with rows == 0 is a valid warm-up: it does this set-up and launches
 *     nothing.  Make it once per device at start-up, BEFORE the host gives its remaining
 *     device memory away (afterwards the set-up itself would fail with RLT_ERR_CUDA, out of
 *     memory) and outside any stream capture.
 *   - All calls on a device share the one block, and it keeps whatever the previous call
 *     left; each call re-initialises the words that must start at zero.  Two calls whose
 *     work can overlap on the GPU (different streams, no ordering between them) race on
 *     the block and corrupt each other: order them, or give one of them its own workspace
 *     through rlt_verify_attention.
 * Results are bit-identical to rlt_verify_attention on the same inputs.
 * ---------------------------------------------------------------------- */
RLT_API int rlt_verify_attention_noalloc(const void* q, void* out, const void* key_cache,
                                 const void* value_cache, int64_t block_stride, int64_t token_stride,
                                 int64_t num_blocks, int block_size, int q_heads, int kv_heads,
                                 int head_dim, int dtype, const int32_t* block_tables, int table_rows,
                                 int table_width, const int32_t* context_lengths,
                                 const int32_t* cu_seqlens_q, int rows, rlt_stream_t stream);

/* ----------------------------------------------------------------------
 * Sliding-window attention: query row r (one block-table row per query row, no packing) attends
 * only its last `window` keys, positions max(0, context_lengths[r] - window) .. context_lengths[r] - 1,
 * its own included; keys outside the window stay stored and are not read.  A row of length 0 is
 * zeros.  Any head_dim <= 256, block size and GQA ratio, fp32 / fp16 / bf16; no workspace; safe
 * under CUDA-graph capture.
 * Replaces: AttentionBackend.windowed (vllm_rlt/attention/backend.py:44-50) as served by
 *   TritonPagedAttention.windowed / torch_paged_attention_windowed
 *   (vllm_rlt/kernels/paged_attention.py:39-70,122-125), called from
 *   KVCacheManager._attend_windowed (vllm_rlt/core/kv_cache_manager.py:773-803).
 * RLT_ERR_INVALID when window <= 0 (the reference raises ValueError).
 * ---------------------------------------------------------------------- */
RLT_API int rlt_windowed_attention(const void* q, void* out, const void* key_cache, const void* value_cache,
                                   int64_t block_stride, int64_t token_stride, int64_t num_blocks,
                                   int block_size, int q_heads, int kv_heads, int head_dim, int dtype,
                                   const int32_t* block_tables, int table_width,
                                   const int32_t* context_lengths, int rows, int window, rlt_stream_t stream);

/* ------------------------------------------------------------------------
 * Packed causal prefill: the same result as rlt_verify_attention with cu_seqlens_q (query i of
 * the n_s new tokens of sequence s sees keys 0 .. context_lengths[s] - n_s + i), computed for
 * prompt-sized n_s: one CTA per 64 query tokens and query head walks the sequence's pages
 * once (head_dim 128, 16-token pages, fp16 / bf16, both caches addressable through one tensor
 * map).  Other shapes, and cache placements the map cannot express, are scored by the kernels
 * behind rlt_verify_attention.  The results agree with rlt_verify_attention to the tolerance
 * of the dtype, not bit for bit (no split-KV merge here), so verification rows that must match
 * decode rows exactly stay on rlt_verify_attention.
 * Replaces: paged_prefill_attention (vllm_rlt/kernels/triton_attention.py:205-366) behind
 *   AttentionBackend.prefill (vllm_rlt/attention/backend.py:30-55).
 * block_tables: int32 [sequences, table_width]; context_lengths: int32 [sequences] (keys in the
 * cache including the new tokens); cu_seqlens_q: int32 [sequences + 1].  workspace: device
 * scratch of rlt_prefill_attention_workspace_bytes(...) bytes, 256-byte aligned; its second
 * 32-bit word is nonzero after a run in which a bounded device-side wait gave up.
 * For head_dim 128 with 16-token pages that is the prompt kernels' tile list (tens of bytes per
 * 256 query tokens).  Where such a call has to fall back to the kernels behind rlt_verify_attention
 * (a 32-bit dtype, or caches the tensor map cannot express) it needs their scratch instead, which
 * grows with rows x heads x context chunks: the call then returns RLT_ERR_WORKSPACE if the workspace
 * is smaller than rlt_verify_attention_workspace_bytes(rows, ...), and is to be repeated with that.
 * ---------------------------------------------------------------------- */
RLT_API size_t rlt_prefill_attention_workspace_bytes(int rows, int sequences, int q_heads, int kv_heads,
                                             int head_dim, int block_size, int table_width);

RLT_API int rlt_prefill_attention(const void* q, void* out, const void* key_cache, const void* value_cache,
                          int64_t block_stride, int64_t token_stride, int64_t num_blocks, int block_size,
                          int q_heads, int kv_heads, int head_dim, int dtype, const int32_t* block_tables,
                          int sequences, int table_width, const int32_t* context_lengths,
                          const int32_t* cu_seqlens_q, int rows, void* workspace, size_t workspace_bytes,
                          rlt_stream_t stream);

/* Diagnostics for the tiled kernel (head_dim 128, 16-token pages, fp16/bf16): waits for
 * `stream` and copies four words of the workspace header to the host —
 * status4[0] = work items planned by the last call (groups x context chunks x kv heads; shows
 * whether rows were grouped), status4[1] = rows of length zero, status4[2] = error bits
 * (nonzero: a bounded device-side wait gave up and the output is invalid), status4[3] = claim
 * counter (0 after a clean run).
 * Synchronises; not for the hot path.  No counterpart in the reference. */
RLT_API int rlt_verify_attention_status(const void* workspace, rlt_stream_t stream, uint32_t* status4);

/* ------------------------------------------------------------------------
 * Row argmax: targets[r] = argmax_v logits[r, v], lowest index on ties, a NaN
 * counts as the maximum (first NaN wins), as torch.argmax does.
 * Replaces: logits.argmax(-1) in SpeculativeRunner._collect_round
 *   (vllm_rlt/worker/speculative.py:469) and AsyncSpeculativeRunner._verify
 *   (vllm_rlt/worker/async_speculative.py:415).
 * logits: [rows, vocab] of `dtype`, row stride in elements.
 * ---------------------------------------------------------------------- */
RLT_API int rlt_argmax_rows(const void* logits, int64_t row_stride, int rows, int vocab, int dtype,
                    int64_t* targets, rlt_stream_t stream);

/* ------------------------------------------------------------------------
 * Greedy acceptance + device state update for n requests whose verification
 * rows are request-major: request i owns rows cu_rows[i] .. cu_rows[i+1]-1
 * (c_i = that count >= 1; column 0 of `tokens` is the committed input token,
 * columns 1..c_i-1 the drafts).
 *   targets[row]       = argmax(logits[row])                       (as rlt_argmax_rows)
 *   accepted[i]        = #leading j < c_i-1 with tokens[i, j+1] == targets[cu_rows[i]+j]
 *   next_token[i]      = targets[cu_rows[i] + accepted[i]]
 *   next_position[i]   = starts[i] + accepted[i] + 1
 *   result             = [targets (rows) | accepted (n) | next_position (n)]   int64
 *   slot_values[slots[i]] = (next_token[i], next_position[i])      (when slots != NULL)
 * Replaces: greedy_accept (vllm_rlt/worker/speculative.py:32-44) and
 *   AsyncSpeculativeRunner._accept_and_update_state
 *   (vllm_rlt/worker/async_speculative.py:417-447; wire layout :62-77).
 * tokens: int64 [n, tokens_width].  slot_values: int64 [*, 2].
 * row_counts: NULL, or int32 [n] for rounds of a fixed shape (one CUDA graph per batch size):
 *   every request then owns the same span of rows, cu_rows[i] .. cu_rows[i+1]-1, of which only
 *   the first row_counts[i] are real; the padding rows are never compared and get -1 in
 *   `result`.  A request with no rows (row_counts[i] <= 0, or an empty span) is left alone:
 *   accepted 0, next_position = starts[i], no slot update.
 * ---------------------------------------------------------------------- */
RLT_API int rlt_accept_greedy(const void* logits, int64_t row_stride, int rows, int vocab, int dtype,
                      const int32_t* cu_rows, int n, const int32_t* row_counts, const int64_t* tokens,
                      int tokens_width, const int64_t* starts, const int64_t* slots, int64_t* slot_values,
                      int64_t* result, rlt_stream_t stream);

/* ------------------------------------------------------------------------
 * Sampling distribution of every row: softmax(float(logits) / temperature) restricted to
 * the strict top-k tokens (by rank, ties broken by the lower token index) and then to the
 * top-p nucleus (rank i stays iff the probability mass of the ranks before it is <= top_p,
 * probabilities taken over the top-k support), renormalised.  probs: float32 [rows, vocab],
 * zero outside the support.  top_k (int32 [rows]) and top_p (float [rows]) may be NULL;
 * top_k[r] <= 0 or >= vocab and top_p[r] >= 1 switch that filter off.  The host validates
 * temperature > 0 and 0 < top_p <= 1 (vllm_rlt/sampling_params.py:30-35); a row with
 * temperature <= 0, NaN / +inf logits or all -inf logits gets status RLT_ROW_BAD_LOGITS and
 * zeros.  Arithmetic: include/rlt_canonical.h (same bits as the CPU oracle).
 * Replaces: Sampler.probabilities (vllm_rlt/worker/sampler.py:27-55).
 * ---------------------------------------------------------------------- */
RLT_API int rlt_probabilities(const void* logits, int64_t row_stride, int rows, int vocab, int dtype,
                      const float* temperature, const int32_t* top_k, const float* top_p,
                      float* probs, int32_t* status, rlt_stream_t stream);

/* ------------------------------------------------------------------------
 * Token draw from the row's sampling distribution (see rlt_probabilities) with a supplied
 * uniform:
 *   tokens[r] = first index whose inclusive fixed-point prefix mass exceeds
 *   floor(u[r] * total)   (see rlt_accept_rejection for the arithmetic).
 * temperature[r] == 0 gives argmax.  top_k / top_p: per row, may be NULL.
 * Used for draft proposals and bonus draws.
 * Replaces: Sampler.sample / Sampler.draw (vllm_rlt/worker/sampler.py:57-81) with the
 *   generator replaced by an explicit uniform.
 * ---------------------------------------------------------------------- */
RLT_API int rlt_sample_rows(const void* logits, int64_t row_stride, int rows, int vocab, int dtype,
                    const float* temperature, const int32_t* top_k, const float* top_p,
                    const float* uniforms, int64_t* tokens, int32_t* status, rlt_stream_t stream);

/* ------------------------------------------------------------------------
 * Rejection-sampling acceptance (sequential per request, parallel over requests).
 * For request i with rows cu_rows[i]..cu_rows[i+1]-1 (c_i rows, c_i-1 drafts) and
 * temperature T_i > 0:
 *   p_j = softmax(target_logits[row_j] / T_i),  q_j = softmax(draft_logits[row_j] / T_i),
 *         both restricted to top_k[i] / top_p[i] as rlt_probabilities does (NULL: no filter)
 *   for j = 0 .. c_i-2, d = tokens[i, j+1]:
 *       accept iff  u_accept[row_j] * q_j[d] < p_j[d]          (fp32, strict)
 *       on the first rejection emit a draw from max(p_j - q_j, 0) / sum with u_final[i]; stop
 *   if every draft was accepted emit a draw from p_{c_i-1} with u_final[i].
 * T_i == 0 selects greedy acceptance for that request (as rlt_accept_greedy).
 * Outputs as rlt_accept_greedy, except result[row] holds the EMITTED tokens of each
 * request at cu_rows[i] .. cu_rows[i]+accepted[i] (later rows of the request: -1),
 * and status[i] is an RLT_ROW_* code (on error accepted/next_* describe the prefix
 * emitted before the failing draft, and the request's slot keeps its old value, so a
 * device-driven next round does not start from an invalid token).  row_counts as in
 * rlt_accept_greedy.
 *
 * Arithmetic (identical in the CPU oracle, so results are bit-exact):
 *   t = x / T (IEEE);  m = max t;  e = rlt_expf(t - m);  Zfix = sum (u64)(e * 2^40);
 *   Z = (float)Zfix * 2^-40;  p[v] = e / Z (IEEE).  Draw weights w[v] = (u64)(mass[v] * 2^40) with
 *   mass[v] = e_p * (1/Z_p) for a plain draw and (e_p * Z_q - e_q * Z_p) * (1/(Z_p * Z_q)) clamped
 *   at 0 for a residual draw; threshold = (u64)((double)u * (double)sum w), token = first v with
 *   prefix(v) > threshold.  Integer sums make every result independent of summation order.
 * workspace: device scratch of rlt_accept_rejection_workspace_bytes(rows) bytes, 16-byte aligned
 *   (per-row normalisers, filled by the first of the call's two launches).
 * Replaces: rejection_sample (vllm_rlt/worker/speculative.py:47-63), the loop in
 *   SpeculativeRunner._collect_round (:483-510), Sampler.probabilities
 *   (vllm_rlt/worker/sampler.py:27-55).
 * target_logits, draft_logits: [rows, vocab]; draft row j of a request holds the logits
 *   draft j+1 was sampled from (its last row is unused).
 * ---------------------------------------------------------------------- */
RLT_API size_t rlt_accept_rejection_workspace_bytes(int rows);

RLT_API int rlt_accept_rejection(const void* target_logits, const void* draft_logits, int64_t row_stride,
                         int rows, int vocab, int dtype, const int32_t* cu_rows, int n,
                         const int32_t* row_counts, const int64_t* tokens, int tokens_width,
                         const int64_t* starts, const float* temperature, const int32_t* top_k, const float* top_p,
                         const float* u_accept, const float* u_final, const int64_t* slots,
                         int64_t* slot_values, int64_t* result, int32_t* status, void* workspace,
                         size_t workspace_bytes, rlt_stream_t stream);

/* ------------------------------------------------------------------------
 * Uniforms of one speculative round for n requests: u_draft[i, o] (the draw of draft o+1),
 * u_accept[i, j] (the accept test of verification row j) and u_final[i] (the residual or bonus
 * draw), each in [0, 1) with 24 random bits, from the counter-based generator of
 * include/rlt_canonical.h (Philox4x32-10 keyed by seeds[i], counter = (index, stream, rounds[i])).
 * A request's uniforms depend on its seed and round number only, not on its batch.
 * Replaces: the per-request torch.Generator of RngRegistry (vllm_rlt/worker/sampler.py:84-119) as
 *   SpeculativeRunner consumes it (vllm_rlt/worker/speculative.py:439-444, 483-510); the
 *   reference's device-resident runner has no sampling at all (engine/stage_engine.py:327-332).
 * seeds, rounds: int64 [n].  u_draft, u_accept: float32 [n, width].  u_final: float32 [n].
 * ---------------------------------------------------------------------- */
RLT_API int rlt_round_uniforms(const int64_t* seeds, const int64_t* rounds, int n, int width, float* u_draft,
                       float* u_accept, float* u_final, rlt_stream_t stream);

/* ------------------------------------------------------------------------
 * Device rollback of rejected positions.  For request i with round start
 * starts[i] and emitted[i] committed tokens (accepted + 1):
 *   frontier[i]             = starts[i] + emitted[i]
 *   written_prefix[i,p,l]   = min(written_prefix[i,p,l], frontier[i])      (all planes, layers)
 *   context_lengths[i]      = frontier[i] + 1
 *   write_offsets[i]        = frontier[i] % block_size
 *   write_blocks[i,p]       = tables[i, p, frontier[i] / block_size]
 *                             (-1 when frontier[i] == table_width * block_size: the allocation is
 *                             full, the rollback itself is valid)
 * A frontier below 0 or beyond table_width * block_size gives RLT_ROW_BAD_POSITION.
 * Block tables and physical pages are not modified (the reservation is kept).
 * If refcounts != NULL and any page of request i at or after frontier[i] / block_size
 * (within pages_used[i]) has refcounts[page] > 1 the request is left untouched and
 * status[i] = RLT_ROW_SHARED_PAGE.
 * Replaces: KVCacheManager.truncate_suffix (vllm_rlt/core/kv_cache_manager.py:338-356)
 *   called from Scheduler.update_from_output (vllm_rlt/core/scheduler.py:1386-1394), and the
 *   device slot mapping of AsyncSpeculativeRunner._execute_recurrent_step
 *   (vllm_rlt/worker/async_speculative.py:267-281).
 * tables: int32 [n, planes, table_width].  written_prefix: int64 [n, planes, layers] or NULL.
 * pages_used: int32 [n] (table entries that are real pages) or NULL (= all table_width).
 * ---------------------------------------------------------------------- */
RLT_API int rlt_rollback(const int64_t* starts, const int64_t* emitted, int n, const int32_t* tables,
                 int planes, int table_width, int block_size, const int32_t* pages_used,
                 const int32_t* refcounts, int64_t num_blocks, int64_t* written_prefix, int layers,
                 int64_t* frontier, int32_t* context_lengths, int64_t* write_blocks,
                 int64_t* write_offsets, int32_t* status, rlt_stream_t stream);

/* ------------------------------------------------------------------------
 * Early-exit finalisation.  For each row (slot, exit depth e, position): copy the token's K/V
 * of every layer from plane e's page into the pages of planes e+1 .. planes-1, so that later
 * tokens attending at deeper loops find it.
 * Replaces: KVCacheManager.finalize_token (vllm_rlt/core/kv_cache_manager.py:805-831) and the
 *   Triton finalize_kernel (vllm_rlt/kernels/routing.py:147-177).
 * key_pool / value_pool: the WHOLE pool [num_blocks, layers, block_size, kv_heads, head_dim];
 *   block_stride, layer_stride, token_stride in elements.  tables: int32 [slots, planes, width].
 * slots / depths / positions: int64 [rows].  Rows must not overlap each other's destinations
 * (one row per token).  A shared-plane layout (planes == 1) is a no-op.
 * ---------------------------------------------------------------------- */
RLT_API int rlt_finalize_tokens(void* key_pool, void* value_pool, int64_t block_stride, int64_t layer_stride,
                        int64_t token_stride, int64_t num_blocks, int layers, int block_size, int kv_heads,
                        int head_dim, int dtype, const int32_t* tables, int planes, int table_width,
                        const int64_t* slots, const int64_t* depths, const int64_t* positions, int rows,
                        rlt_stream_t stream);

/* ------------------------------------------------------------------------
 * Pipeline-mode self-speculation: device state update of every request after one pipeline step
 * (the retained-hidden-state rollback).  Request i keeps `width` oldest-first slots
 * (tokens, depths, candidates, active, hidden rows); the step advanced its first widths[i] slots
 * by draft_loops loops and produced, request-major from row row_starts[i], the LM-head argmax
 * `choices` and the hidden rows `step_hidden`.  The head slot that reached target_loops is
 * emitted and compared with its draft candidate: on a match the slots (and their hidden rows)
 * shift down and a new draft slot is born at the tail; on a mismatch all descendants are dropped
 * and the pipeline restarts from the corrected token; nothing is born at or beyond limits[i].
 * result[6i .. 6i+5] = prediction, accepted, emitted, next position, drafted count, verified count.
 * Replaces: the per-request tensor program of AsyncSpeculativeRunner._pipeline_step
 *   (vllm_rlt/worker/async_speculative.py:527-580; wire layout :62-77).
 * tokens / depths / candidates: int64 [n, width]; active: uint8/bool [n, width];
 * hidden: [n, width, hidden_size] of `dtype`; state_token / state_position / limits: int64 [n];
 * widths / row_starts: int32 [n]; choices: int64 [rows]; step_hidden: [rows, hidden_size].
 * All state arrays are updated in place.  width <= 64.
 * ---------------------------------------------------------------------- */
RLT_API int rlt_pipeline_shift(int64_t* tokens, int64_t* depths, int64_t* candidates, uint8_t* active,
                       void* hidden, int64_t* state_token, int64_t* state_position, const int32_t* widths,
                       const int32_t* row_starts, const int64_t* choices, const void* step_hidden,
                       const int64_t* limits, int n, int width, int hidden_size, int dtype, int draft_loops,
                       int target_loops, int64_t* result, rlt_stream_t stream);

/* ------------------------------------------------------------------------
 * Rotary embedding of q and k fused with the KV write of one layer.
 *   q_out[r]              = q[r] * cos[r] + rotate_half(q[r]) * sin[r]      (per head)
 *   cache_k[block, off]   = k[r] * cos[r] + rotate_half(k[r]) * sin[r]
 *   cache_v[block, off]   = v[r]
 * with rotate_half(x) = (-x[d/2:], x[:d/2]) and every product and sum rounded to `dtype`
 * as the tensor expression rounds, so the results are bit-identical to it.  Rows that
 * rlt_kv_write would skip (mask, active_rows, out-of-pool address) write nothing to the
 * cache; q_out is written for every row.
 * Replaces: apply_rotary_pos_emb (vllm_rlt/layers/rotary_embedding.py:15-24) followed by
 *   KVCacheManager._write_prepared in OuroAttention.forward (vllm_rlt/models/ouro.py:179-186).
 * q: [rows, q_heads, head_dim] with row stride q_row_stride (elements; the [heads, head_dim]
 *   tail contiguous, so slices of one fused QKV projection are accepted); k, v likewise.
 * cos_table / sin_table: [rows, head_dim] of `dtype`, contiguous (RotaryEmbedding.forward,
 *   rotary_embedding.py:54-64, computed once per pass).  q_out: [rows, q_heads, head_dim]
 *   contiguous.  Cache arguments as rlt_kv_write.  head_dim must be even.
 * ---------------------------------------------------------------------- */
RLT_API int rlt_rope_kv_write(const void* q, int64_t q_row_stride, const void* k, int64_t k_row_stride,
                      const void* v, int64_t v_row_stride, const void* cos_table, const void* sin_table,
                      void* q_out, void* key_cache, void* value_cache, int64_t block_stride,
                      int64_t token_stride, int64_t num_blocks, int block_size, int q_heads, int kv_heads,
                      int head_dim, int dtype, const int64_t* write_blocks, const int64_t* write_offsets,
                      const uint8_t* write_mask, const int32_t* active_rows, int rows, rlt_stream_t stream);

/* ------------------------------------------------------------------------
 * RMSNorm of a sandwich-norm sublayer, optionally fused with the residual add and with the
 * norm that opens the next sublayer.  Per row:
 *   y = weight * T(x * rsqrt(mean(x^2) + eps))           (T: round to `dtype`)
 *   s = residual + y        (s = y when residual is NULL)         -> sum_out  (if not NULL)
 *   n = weight2 * T(s * rsqrt(mean(s^2) + eps))                   -> norm_out (if weight2 not NULL)
 * The squares are fp32, their sum is accumulated in double, the reciprocal square root is
 * correctly rounded; products and sums round to `dtype` where the tensor expressions round.
 * (PyTorch's fp32 mean sums in an unspecified order, so agreement with it is to the last
 * place of `dtype`, not bit for bit.)
 * Replaces: RMSNorm.forward (vllm_rlt/layers/normalization.py:20-23) and the residual adds of
 *   OuroDecoderLayer.forward (vllm_rlt/models/ouro.py:217-221).
 * x, residual, sum_out, norm_out: [rows, hidden] contiguous; weight, weight2: [hidden].
 * sum_out may alias residual (in-place residual stream); x must not alias an output.
 * hidden <= 8192.
 * ---------------------------------------------------------------------- */
RLT_API int rlt_sandwich_norm(const void* x, const void* weight, const void* residual, void* sum_out,
                      const void* weight2, void* norm_out, int rows, int hidden, float eps, int dtype,
                      rlt_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* RLT_VERIFY_H_ */
