// Device rollback of the positions a verify round rejected.
//
// One warp per request.  Pure integer work on O(planes * pages) table entries and
// O(planes * layers) validity words per request: latency-bound, not bandwidth-bound.
// Block tables and pages are never modified — rejected slots keep their stale bytes and
// are hidden by the frontier, exactly as the reference's truncate_suffix leaves them.
#include "common.cuh"

namespace rlt {
namespace {

constexpr int kWarpsPerCta = 4;

__global__ void __launch_bounds__(kWarpsPerCta * 32)
rollback_kernel(const int64_t* __restrict__ starts, const int64_t* __restrict__ emitted, int n,
                const int32_t* __restrict__ tables, int planes, int table_width, int block_size,
                const int32_t* __restrict__ pages_used, const int32_t* __restrict__ refcounts,
                int64_t num_blocks, int64_t* __restrict__ written_prefix, int layers,
                int64_t* __restrict__ frontier, int32_t* __restrict__ context_lengths,
                int64_t* __restrict__ write_blocks, int64_t* __restrict__ write_offsets,
                int32_t* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (i >= n) return;
  const int64_t f = starts[i] + emitted[i];
  const int64_t page = f / block_size;
  if (lane == 0) frontier[i] = f;
  // truncate_suffix accepts 0 <= frontier <= max_tokens: a request that filled its allocation to
  // the last token of its last page is rolled back like any other; only the page of its NEXT
  // token does not exist (write_blocks = -1).
  const bool full = f == static_cast<int64_t>(table_width) * block_size;
  if (f < 0 || (page >= table_width && !full)) {
    if (lane == 0) status[i] = RLT_ROW_BAD_POSITION;
    return;
  }
  const int32_t* mine = tables + static_cast<int64_t>(i) * planes * table_width;
  if (refcounts != nullptr) {
    const int used = pages_used != nullptr ? min(pages_used[i], table_width) : table_width;
    const int span = used - static_cast<int>(page);
    int shared = 0;
    for (int x = lane; x < planes * max(span, 0); x += 32) {
      const int p = x / span, w = static_cast<int>(page) + x % span;
      const int32_t id = mine[static_cast<int64_t>(p) * table_width + w];
      if (id >= 0 && id < num_blocks && refcounts[id] > 1) shared = 1;
    }
    if (__any_sync(0xffffffffu, shared)) {
      if (lane == 0) status[i] = RLT_ROW_SHARED_PAGE;
      return;
    }
  }
  if (written_prefix != nullptr) {
    int64_t* w = written_prefix + static_cast<int64_t>(i) * planes * layers;
    for (int x = lane; x < planes * layers; x += 32)
      if (w[x] > f) w[x] = f;
  }
  for (int p = lane; p < planes; p += 32)
    write_blocks[static_cast<int64_t>(i) * planes + p] = full ? -1 : mine[static_cast<int64_t>(p) * table_width + page];
  if (lane == 0) {
    context_lengths[i] = static_cast<int32_t>(f + 1);
    write_offsets[i] = f % block_size;
    status[i] = RLT_ROW_OK;
  }
}

}  // namespace
}  // namespace rlt

extern "C" RLT_API int rlt_rollback(const int64_t* starts, const int64_t* emitted, int n, const int32_t* tables,
                            int planes, int table_width, int block_size, const int32_t* pages_used,
                            const int32_t* refcounts, int64_t num_blocks, int64_t* written_prefix, int layers,
                            int64_t* frontier, int32_t* context_lengths, int64_t* write_blocks,
                            int64_t* write_offsets, int32_t* status, rlt_stream_t stream) {
  using namespace rlt;
  RLT_REQUIRE(n >= 0 && planes > 0 && table_width > 0 && block_size > 0 && layers >= 0,
              "rollback: invalid shape");
  if (n == 0) return RLT_OK;
  RLT_REQUIRE(starts && emitted && tables && frontier && context_lengths && write_blocks && write_offsets &&
                  status,
              "rollback: null pointer");
  RLT_REQUIRE(written_prefix == nullptr || layers > 0, "rollback: written_prefix needs layers > 0");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  rollback_kernel<<<(n + kWarpsPerCta - 1) / kWarpsPerCta, kWarpsPerCta * 32, 0, s>>>(
      starts, emitted, n, tables, planes, table_width, block_size, pages_used, refcounts, num_blocks,
      written_prefix, layers, frontier, context_lengths, write_blocks, write_offsets, status);
  return launch_status("rollback_kernel");
}
