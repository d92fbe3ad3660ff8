// Early-exit finalisation: copy a token's K/V of its exit depth into every deeper plane.
//
// A request that leaves the recurrence at depth e never writes planes e+1 .. P-1 for that
// token, but later tokens attend at those depths; the reference fills the gap by copying the
// exit plane's K/V (all layers) into the deeper planes.  One CTA per (row, target plane):
// layers x kv_heads*head_dim elements moved as 16-byte vectors, both K and V.  Pure copy,
// 2 * 2 * layers * channels * sizeof bytes per (row, plane); latency-bound at decode sizes.
#include "common.cuh"

namespace rlt {
namespace {

constexpr int kThreads = 256;

template <int kBytes> struct Granule;
template <> struct Granule<16> { using type = uint4; };
template <> struct Granule<4> { using type = uint32_t; };
template <> struct Granule<2> { using type = uint16_t; };

template <int kBytes>
__global__ void __launch_bounds__(kThreads)
finalize_kernel(char* __restrict__ key_pool, char* __restrict__ value_pool, int64_t block_stride_bytes,
                int64_t layer_stride_bytes, int64_t token_stride_bytes, int64_t num_blocks, int layers,
                int block_size, int64_t channel_bytes, const int32_t* __restrict__ tables, int planes,
                int table_width, const int64_t* __restrict__ slots, const int64_t* __restrict__ depths,
                const int64_t* __restrict__ positions, int rows) {
  using G = typename Granule<kBytes>::type;
  const int row = blockIdx.x, target = blockIdx.y;
  const int64_t slot = slots[row], depth = depths[row], pos = positions[row];
  if (target <= depth || depth < 0 || pos < 0 || pos / block_size >= table_width) return;
  const int32_t* mine = tables + slot * planes * table_width;
  const int64_t source = mine[depth * table_width + pos / block_size];
  const int64_t dest = mine[static_cast<int64_t>(target) * table_width + pos / block_size];
  if (source < 0 || source >= num_blocks || dest < 0 || dest >= num_blocks) return;
  const int64_t within = (pos % block_size) * token_stride_bytes;
  const int64_t per_layer = channel_bytes / kBytes;
  for (int64_t i = threadIdx.x; i < per_layer * layers; i += kThreads) {
    const int64_t layer = i / per_layer, x = i % per_layer;
    const int64_t offset = layer * layer_stride_bytes + within + x * kBytes;
    *reinterpret_cast<G*>(key_pool + dest * block_stride_bytes + offset) =
        *reinterpret_cast<const G*>(key_pool + source * block_stride_bytes + offset);
    *reinterpret_cast<G*>(value_pool + dest * block_stride_bytes + offset) =
        *reinterpret_cast<const G*>(value_pool + source * block_stride_bytes + offset);
  }
}

}  // namespace
}  // namespace rlt

extern "C" RLT_API int rlt_finalize_tokens(void* key_pool, void* value_pool, int64_t block_stride,
                                           int64_t layer_stride, int64_t token_stride, int64_t num_blocks,
                                           int layers, int block_size, int kv_heads, int head_dim, int dtype,
                                           const int32_t* tables, int planes, int table_width,
                                           const int64_t* slots, const int64_t* depths, const int64_t* positions,
                                           int rows, rlt_stream_t stream) {
  using namespace rlt;
  RLT_REQUIRE(dtype_valid(dtype), "finalize_tokens: KV dtype must be float32, float16, or bfloat16");
  RLT_REQUIRE(rows >= 0 && layers > 0 && block_size > 0 && kv_heads > 0 && head_dim > 0 && planes > 0 &&
                  table_width > 0 && num_blocks > 0,
              "finalize_tokens: invalid shape");
  if (rows == 0 || planes == 1) return RLT_OK;
  RLT_REQUIRE(key_pool && value_pool && tables && slots && depths && positions, "finalize_tokens: null pointer");
  const int64_t es = static_cast<int64_t>(dtype_size(dtype));
  const int64_t channel_bytes = static_cast<int64_t>(kv_heads) * head_dim * es;
  RLT_REQUIRE(token_stride * es >= channel_bytes, "finalize_tokens: the [kv_heads, head_dim] tail must be contiguous");
  const int64_t bsb = block_stride * es, lsb = layer_stride * es, tsb = token_stride * es;
  auto all_multiple = [&](int64_t m) {
    return channel_bytes % m == 0 && bsb % m == 0 && lsb % m == 0 && tsb % m == 0 &&
           reinterpret_cast<uintptr_t>(key_pool) % m == 0 && reinterpret_cast<uintptr_t>(value_pool) % m == 0;
  };
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(static_cast<unsigned>(rows), static_cast<unsigned>(planes));
#define RLT_FINALIZE_LAUNCH(B)                                                                          \
  finalize_kernel<B><<<grid, kThreads, 0, s>>>(static_cast<char*>(key_pool), static_cast<char*>(value_pool), \
                                                bsb, lsb, tsb, num_blocks, layers, block_size, channel_bytes, \
                                                tables, planes, table_width, slots, depths, positions, rows)
  if (all_multiple(16)) RLT_FINALIZE_LAUNCH(16);
  else if (all_multiple(4)) RLT_FINALIZE_LAUNCH(4);
  else RLT_FINALIZE_LAUNCH(2);
#undef RLT_FINALIZE_LAUNCH
  return launch_status("finalize_kernel");
}
