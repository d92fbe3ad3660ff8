// Shape-generic paged attention: any head_dim <= 256, any block size, any GQA ratio,
// fp32 / fp16 / bf16.  One CTA per (query row, query head); four warps stride over the
// row's tokens with an fp32 online softmax each and are merged in warp order, so a row's
// result depends on nothing but its own query, length and K/V.  This is the path for
// shapes the tiled sm_100a kernel (attention_sm100.cu) does not cover — the fp32 tiny
// model and the odd head sizes the reference's tests use; it reads K/V once per row.
// With window > 0 a row attends only its last `window` keys (sliding-window layers).
#include <math.h>

#include "attention.cuh"

namespace rlt {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxPerLane = 8;  // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(kThreads)
attention_generic_kernel(AttentionArgs a, float scale, int window) {
  const int row = blockIdx.x / a.q_heads;
  const int head = blockIdx.x % a.q_heads;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int D = a.head_dim;
  const T* q = static_cast<const T*>(a.q);
  T* out = static_cast<T*>(a.out) + (static_cast<int64_t>(row) * a.q_heads + head) * D;

  int table_row, len;
  resolve_row(a, row, &table_row, &len);
  if (len <= 0) {
    for (int d = threadIdx.x; d < D; d += kThreads) out[d] = Elem<T>::from_float(0.0f);
    return;
  }
  const int32_t* table = a.block_tables + static_cast<int64_t>(table_row) * a.table_width;
  const int kv_head = head / (a.q_heads / a.kv_heads);
  const T* kc = static_cast<const T*>(a.key_cache);
  const T* vc = static_cast<const T*>(a.value_cache);

  float qr[kMaxPerLane], o[kMaxPerLane];
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    int d = lane + 32 * j;
    qr[j] = d < D ? Elem<T>::to_float(q[(static_cast<int64_t>(row) * a.q_heads + head) * D + d]) : 0.0f;
    o[j] = 0.0f;
  }
  float m = -INFINITY, l = 0.0f;
  const int first = window > 0 && len > window ? len - window : 0;
  for (int t = first + warp; t < len; t += kWarps) {
    const int64_t page = table[t / a.block_size];
    if (page < 0 || page >= a.num_blocks) continue;  // corrupt table entry: never dereferenced
    const int64_t base = page * a.block_stride + static_cast<int64_t>(t % a.block_size) * a.token_stride +
                         static_cast<int64_t>(kv_head) * D;
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      int d = lane + 32 * j;
      if (d < D) s = fmaf(qr[j], Elem<T>::to_float(kc[base + d]), s);
    }
#pragma unroll
    for (int x = 16; x > 0; x >>= 1) s += __shfl_xor_sync(0xffffffffu, s, x);
    s *= scale;
    const float m_new = fmaxf(m, s);
    const float alpha = m == -INFINITY ? 0.0f : expf(m - m_new);
    const float p = expf(s - m_new);
    l = fmaf(l, alpha, p);
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      int d = lane + 32 * j;
      if (d < D) o[j] = fmaf(o[j], alpha, p * Elem<T>::to_float(vc[base + d]));
    }
    m = m_new;
  }

  __shared__ float sm_m[kWarps], sm_l[kWarps];
  __shared__ float sm_o[kWarps][32 * kMaxPerLane];
  if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) sm_o[warp][lane + 32 * j] = o[j];
  __syncthreads();
  float big = -INFINITY;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) big = fmaxf(big, sm_m[w]);
  for (int d = threadIdx.x; d < D; d += kThreads) {
    float total = 0.0f, acc = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      if (sm_m[w] == -INFINITY) continue;
      const float f = expf(sm_m[w] - big);
      total = fmaf(sm_l[w], f, total);
      acc = fmaf(sm_o[w][d], f, acc);
    }
    out[d] = Elem<T>::from_float(total > 0.0f ? acc / total : 0.0f);
  }
}

}  // namespace

int launch_attention_generic(const AttentionArgs& a, cudaStream_t stream, int window) {
  if (a.head_dim > 32 * kMaxPerLane) {
    set_last_error_text("verify_attention supports head_dim <= 256");
    return RLT_ERR_UNSUPPORTED;
  }
  const int64_t ctas = static_cast<int64_t>(a.rows) * a.q_heads;
  if (ctas > 0x7fffffff) {
    set_last_error_text("verify_attention: rows * q_heads exceeds the grid limit");
    return RLT_ERR_INVALID;
  }
  const float scale = static_cast<float>(1.0 / sqrt(static_cast<double>(a.head_dim)));
  RLT_DISPATCH_DTYPE(a.dtype, T,
                     (attention_generic_kernel<T><<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(a, scale, window)));
  return launch_status("attention_generic_kernel");
}

}  // namespace rlt
