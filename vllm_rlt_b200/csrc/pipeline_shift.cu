// Pipeline-mode self-speculation: per-request device state update after one pipeline step.
//
// Each request keeps up to W oldest-first token slots on the device (token, loop depth reached,
// retained hidden row, draft candidate, active flag).  After a step that advanced every active
// slot by `draft_loops` loops, the slot at the head may have reached the target depth: its
// prediction is emitted, compared with the candidate drafted for it, and on a match the slots
// shift down by one (the retained hidden rows with them) and a new slot is born at the tail; on
// a mismatch every speculative descendant is dropped and the pipeline restarts from the
// corrected token.  This is the retained-hidden-state rollback of the verify path.  One CTA
// per request: a few dozen integers of bookkeeping by one thread, then all threads move the
// hidden rows (W x hidden_size elements, 16-byte vectors).  Latency-bound.
#include "common.cuh"

namespace rlt {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxWidth = 64;

template <typename V>  // V: copy granule (uint4 or uint16_t)
__global__ void __launch_bounds__(kThreads)
pipeline_shift_kernel(int64_t* __restrict__ tokens, int64_t* __restrict__ depths, int64_t* __restrict__ candidates,
                      uint8_t* __restrict__ active, char* __restrict__ hidden, int64_t* __restrict__ state_token,
                      int64_t* __restrict__ state_position, const int32_t* __restrict__ widths,
                      const int32_t* __restrict__ row_starts, const int64_t* __restrict__ choices,
                      const char* __restrict__ step_hidden, const int64_t* __restrict__ limits, int width,
                      int64_t row_bytes, int draft_loops, int target_loops, int64_t* __restrict__ result) {
  const int i = blockIdx.x;
  __shared__ int s_emitted, s_w;
  int64_t* tok = tokens + static_cast<int64_t>(i) * width;
  int64_t* dep = depths + static_cast<int64_t>(i) * width;
  int64_t* cand = candidates + static_cast<int64_t>(i) * width;
  uint8_t* act = active + static_cast<int64_t>(i) * width;
  const int w = min(widths[i], width);
  const int start = row_starts[i];
  if (threadIdx.x == 0) {
    int64_t old_tok[kMaxWidth], new_dep[kMaxWidth], pred[kMaxWidth], new_cand[kMaxWidth];
    bool valid[kMaxWidth], drafted[kMaxWidth];
    int nvalid = 0;
    int64_t ndrafted = 0;
    for (int j = 0; j < width; ++j) {
      valid[j] = act[j] != 0 && j < w;
      nvalid += valid[j];
      new_dep[j] = dep[j] + (valid[j] ? draft_loops : 0);
      pred[j] = j < w ? choices[start + j] : 0;
      drafted[j] = valid[j] && new_dep[j] == draft_loops;
      ndrafted += drafted[j];
      new_cand[j] = drafted[j] ? pred[j] : cand[j];
      old_tok[j] = tok[j];
    }
    const bool emitted = valid[0] && new_dep[0] == target_loops;
    const bool accepted = emitted && new_cand[0] == pred[0];
    const bool reject = emitted && !accepted;
    int64_t token = state_token[i];
    if (emitted) token = pred[0];
    const int64_t position = state_position[i] + (emitted ? 1 : 0);
    const int remaining = nvalid - (emitted ? 1 : 0);
    const int tail = max(nvalid - 1, 0);
    const bool append = drafted[tail] && !reject;
    const bool restart = reject || (emitted && remaining == 0);
    const int64_t born_token = restart ? token : new_cand[tail];
    const int64_t limit = limits[i];
    for (int j = 0; j < width; ++j) {
      const int src = min(j + (emitted ? 1 : 0), width - 1);
      const bool surviving = j < remaining && !reject;
      bool newborn = restart ? j == 0 : (j == remaining && append);
      newborn = newborn && j < w && position + j < limit;
      tok[j] = newborn ? born_token : old_tok[src];
      dep[j] = newborn ? 0 : new_dep[src];
      cand[j] = new_cand[src];
      act[j] = (surviving || newborn) && position + j < limit;
    }
    state_token[i] = token;
    state_position[i] = position;
    int64_t* out = result + 6 * static_cast<int64_t>(i);
    out[0] = pred[0];
    out[1] = accepted;
    out[2] = emitted;
    out[3] = position;
    out[4] = ndrafted;
    out[5] = emitted;
    s_emitted = emitted;
    s_w = w;
  }
  __syncthreads();
  // hidden[j] = next[min(j + emitted, W - 1)], next[j] = the step's row for j < w, else the old row.
  // Ascending j: the row read in iteration j (j + emitted) is overwritten only in a later one.
  const int shift = s_emitted;
  const int64_t vectors = row_bytes / static_cast<int64_t>(sizeof(V));
  char* mine = hidden + static_cast<int64_t>(i) * width * row_bytes;
  for (int j = 0; j < width; ++j) {
    const int src = min(j + shift, width - 1);
    const char* from = src < s_w ? step_hidden + static_cast<int64_t>(start + src) * row_bytes : mine + src * row_bytes;
    if (!(from == mine + j * row_bytes)) {
      for (int64_t x = threadIdx.x; x < vectors; x += kThreads)
        reinterpret_cast<V*>(mine + j * row_bytes)[x] = reinterpret_cast<const V*>(from)[x];
    }
    __syncthreads();
  }
}

}  // namespace
}  // namespace rlt

extern "C" RLT_API int rlt_pipeline_shift(int64_t* tokens, int64_t* depths, int64_t* candidates, uint8_t* active,
                                          void* hidden, int64_t* state_token, int64_t* state_position,
                                          const int32_t* widths, const int32_t* row_starts, const int64_t* choices,
                                          const void* step_hidden, const int64_t* limits, int n, int width,
                                          int hidden_size, int dtype, int draft_loops, int target_loops,
                                          int64_t* result, rlt_stream_t stream) {
  using namespace rlt;
  RLT_REQUIRE(dtype_valid(dtype), "pipeline_shift: hidden dtype must be float32, float16 or bfloat16");
  RLT_REQUIRE(n >= 0 && width > 0 && width <= kMaxWidth && hidden_size > 0, "pipeline_shift: invalid shape (width <= 64)");
  RLT_REQUIRE(draft_loops > 0 && target_loops > draft_loops, "pipeline_shift: draft_loops must be smaller than target_loops");
  if (n == 0) return RLT_OK;
  RLT_REQUIRE(tokens && depths && candidates && active && hidden && state_token && state_position && widths &&
                  row_starts && choices && step_hidden && limits && result,
              "pipeline_shift: null pointer");
  const int64_t row_bytes = static_cast<int64_t>(hidden_size) * static_cast<int64_t>(dtype_size(dtype));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool wide = row_bytes % 16 == 0 && aligned16(hidden) && aligned16(step_hidden);
#define RLT_SHIFT_LAUNCH(V)                                                                                     \
  pipeline_shift_kernel<V><<<n, kThreads, 0, s>>>(tokens, depths, candidates, active, static_cast<char*>(hidden), \
                                                  state_token, state_position, widths, row_starts, choices,     \
                                                  static_cast<const char*>(step_hidden), limits, width,         \
                                                  row_bytes, draft_loops, target_loops, result)
  if (wide) RLT_SHIFT_LAUNCH(uint4);
  else RLT_SHIFT_LAUNCH(uint16_t);
#undef RLT_SHIFT_LAUNCH
  return launch_status("pipeline_shift_kernel");
}
