// Scatter of the new K/V rows of one layer into their pages.
//
// One CTA column per (row, K|V): the row is kv_heads * head_dim contiguous elements
// (4 KiB for 16 x 128 bf16) copied as 16-byte vectors.  Inactive rows (masked, or at or
// beyond *active_rows) return before reading their write address, so padding rows of a
// captured graph can carry arbitrary addresses.  Addresses outside the pool are skipped.
#include "common.cuh"

namespace rlt {
namespace {

constexpr int kThreads = 128;

template <int kBytes>  // copy granule: 16, 4 or 2 bytes
struct Granule;
template <> struct Granule<16> { using type = uint4; };
template <> struct Granule<4> { using type = uint32_t; };
template <> struct Granule<2> { using type = uint16_t; };

template <int kBytes>
__global__ void __launch_bounds__(kThreads)
kv_write_kernel(char* __restrict__ key_cache, char* __restrict__ value_cache,
                int64_t block_stride_bytes, int64_t token_stride_bytes, int64_t num_blocks,
                int block_size, int64_t row_bytes, const char* __restrict__ k,
                const char* __restrict__ v, const int64_t* __restrict__ write_blocks,
                const int64_t* __restrict__ write_offsets, const uint8_t* __restrict__ write_mask,
                const int32_t* __restrict__ active_rows, int rows) {
  using G = typename Granule<kBytes>::type;
  const int row = blockIdx.x;
  if (active_rows != nullptr && row >= *active_rows) return;
  if (write_mask != nullptr && write_mask[row] == 0) return;
  const int64_t block = write_blocks[row];
  const int64_t offset = write_offsets[row];
  if (block < 0 || block >= num_blocks || offset < 0 || offset >= block_size) return;
  const char* src = (blockIdx.y == 0 ? k : v) + static_cast<int64_t>(row) * row_bytes;
  char* dst = (blockIdx.y == 0 ? key_cache : value_cache) + block * block_stride_bytes +
              offset * token_stride_bytes;
  const int64_t count = row_bytes / kBytes;
  for (int64_t i = threadIdx.x; i < count; i += kThreads)
    reinterpret_cast<G*>(dst)[i] = reinterpret_cast<const G*>(src)[i];
}

}  // namespace
}  // namespace rlt

extern "C" RLT_API int rlt_kv_write(void* key_cache, void* value_cache, int64_t block_stride,
                            int64_t token_stride, int64_t num_blocks, int block_size, int kv_heads,
                            int head_dim, int dtype, const void* k, const void* v,
                            const int64_t* write_blocks, const int64_t* write_offsets,
                            const uint8_t* write_mask, const int32_t* active_rows, int rows,
                            rlt_stream_t stream) {
  using namespace rlt;
  RLT_REQUIRE(dtype_valid(dtype), "kv_write: KV dtype must be float32, float16, or bfloat16");
  RLT_REQUIRE(rows >= 0 && kv_heads > 0 && head_dim > 0 && block_size > 0 && num_blocks > 0,
              "kv_write: invalid shape");
  if (rows == 0) return RLT_OK;
  RLT_REQUIRE(key_cache && value_cache && k && v && write_blocks && write_offsets,
              "kv_write: null pointer");
  RLT_REQUIRE(token_stride >= static_cast<int64_t>(kv_heads) * head_dim && block_stride > 0,
              "kv_write: the [kv_heads, head_dim] tail of the cache view must be contiguous");
  const int64_t es = static_cast<int64_t>(dtype_size(dtype));
  const int64_t row_bytes = static_cast<int64_t>(kv_heads) * head_dim * es;
  const int64_t bsb = block_stride * es, tsb = token_stride * es;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(static_cast<unsigned>(rows), 2);
  auto all_multiple = [&](int64_t m) {
    return row_bytes % m == 0 && bsb % m == 0 && tsb % m == 0 &&
           reinterpret_cast<uintptr_t>(key_cache) % m == 0 &&
           reinterpret_cast<uintptr_t>(value_cache) % m == 0 &&
           reinterpret_cast<uintptr_t>(k) % m == 0 && reinterpret_cast<uintptr_t>(v) % m == 0;
  };
#define RLT_KV_LAUNCH(B)                                                                         \
  kv_write_kernel<B><<<grid, kThreads, 0, s>>>(                                                  \
      static_cast<char*>(key_cache), static_cast<char*>(value_cache), bsb, tsb, num_blocks,      \
      block_size, row_bytes, static_cast<const char*>(k), static_cast<const char*>(v),           \
      write_blocks, write_offsets, write_mask, active_rows, rows)
  if (all_multiple(16)) RLT_KV_LAUNCH(16);
  else if (all_multiple(4)) RLT_KV_LAUNCH(4);
  else RLT_KV_LAUNCH(2);
#undef RLT_KV_LAUNCH
  return launch_status("kv_write_kernel");
}
