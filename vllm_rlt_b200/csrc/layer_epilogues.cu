// Elementwise work around the attention call of a decoder layer, fused so that a layer of a
// verify pass is GEMMs plus four launches instead of GEMMs plus about forty:
//
//   rope_kv_write_kernel   q, k -> rotary embedding; rotated k and v scattered into their
//                          pages; rotated q to a contiguous buffer for the attention call
//   sandwich_norm_kernel   y = w * T(rmsnorm(x)); optionally s = residual + y; optionally a
//                          second norm n = w2 * T(rmsnorm(s)) — the tail of one sandwich-norm
//                          sublayer and the head of the next in one pass over the row
//
// Both are HBM-bound streaming kernels (a row is hidden * sizeof(T) bytes, read once and
// written once per output).  Every product and sum is rounded to the storage type T exactly
// where the PyTorch expressions they replace round, so rope_kv_write is bit-identical to them.
#include "common.cuh"

namespace rlt {
namespace {

constexpr int kNormThreads = 256;
constexpr int kRopeThreads = 256;

__device__ __forceinline__ double block_sum_double(double v, double* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int x = 16; x > 0; x >>= 1) v += __shfl_xor_sync(0xffffffffu, v, x);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  v = lane < kNormThreads / 32 ? scratch[lane] : 0.0;
#pragma unroll
  for (int x = 16; x > 0; x >>= 1) v += __shfl_xor_sync(0xffffffffu, v, x);
  return v;
}

// 1 / sqrt(mean(x^2) + eps) with fp32 squares summed in double: independent of the thread
// count up to the last bit of a double.
__device__ __forceinline__ float inverse_rms(double sum_squares, int hidden, float eps) {
  const float mean = static_cast<float>(sum_squares / static_cast<double>(hidden));
  return __frsqrt_rn(__fadd_rn(mean, eps));
}

template <typename T>
__global__ void __launch_bounds__(kNormThreads)
sandwich_norm_kernel(const T* __restrict__ x, const T* __restrict__ weight, const T* residual,
                     T* sum_out, const T* __restrict__ weight2, T* __restrict__ norm_out,
                     int hidden, float eps) {
  extern __shared__ float row_values[];
  __shared__ double scratch[32];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * hidden;
  double ss = 0.0;
  for (int i = threadIdx.x; i < hidden; i += kNormThreads) {
    const float v = Elem<T>::to_float(x[base + i]);
    row_values[i] = v;
    ss += static_cast<double>(__fmul_rn(v, v));
  }
  float r = inverse_rms(block_sum_double(ss, scratch), hidden, eps);
  ss = 0.0;
  for (int i = threadIdx.x; i < hidden; i += kNormThreads) {
    const float normed = Elem<T>::to_float(Elem<T>::from_float(__fmul_rn(row_values[i], r)));
    float s = Elem<T>::to_float(Elem<T>::from_float(__fmul_rn(Elem<T>::to_float(weight[i]), normed)));
    if (residual != nullptr) s = Elem<T>::to_float(Elem<T>::from_float(__fadd_rn(Elem<T>::to_float(residual[base + i]), s)));
    if (sum_out != nullptr) sum_out[base + i] = Elem<T>::from_float(s);
    row_values[i] = s;
    ss += static_cast<double>(__fmul_rn(s, s));
  }
  if (weight2 == nullptr) return;
  r = inverse_rms(block_sum_double(ss, scratch), hidden, eps);
  for (int i = threadIdx.x; i < hidden; i += kNormThreads) {
    const float normed = Elem<T>::to_float(Elem<T>::from_float(__fmul_rn(row_values[i], r)));
    norm_out[base + i] = Elem<T>::from_float(__fmul_rn(Elem<T>::to_float(weight2[i]), normed));
  }
}

// The same arithmetic with the row held in registers: thread i owns kPer 16-byte vectors of the
// row (hidden = 256 * kPer * 16 / sizeof(T)), every global access is one 16-byte vector, and the
// weight / residual loads are issued before the first reduction so that the kernel is two block
// reductions long.
template <typename T, int kPer>
__global__ void __launch_bounds__(kNormThreads)
sandwich_norm_vec_kernel(const T* __restrict__ x, const T* __restrict__ weight, const T* residual, T* sum_out,
                         const T* __restrict__ weight2, T* __restrict__ norm_out, int hidden, float eps) {
  constexpr int kVec = 16 / sizeof(T);
  struct alignas(16) Vec { T e[kVec]; };
  __shared__ double scratch[32];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * hidden;
  Vec xv[kPer], wv[kPer], rv[kPer], w2v[kPer];
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    const int i = (k * kNormThreads + threadIdx.x) * kVec;
    xv[k] = *reinterpret_cast<const Vec*>(x + base + i);
    wv[k] = *reinterpret_cast<const Vec*>(weight + i);
    if (residual != nullptr) rv[k] = *reinterpret_cast<const Vec*>(residual + base + i);
    if (weight2 != nullptr) w2v[k] = *reinterpret_cast<const Vec*>(weight2 + i);
  }
  double ss = 0.0;
#pragma unroll
  for (int k = 0; k < kPer; ++k)
#pragma unroll
    for (int e = 0; e < kVec; ++e) {
      const float v = Elem<T>::to_float(xv[k].e[e]);
      ss += static_cast<double>(__fmul_rn(v, v));
    }
  float r = inverse_rms(block_sum_double(ss, scratch), hidden, eps);
  float sv[kPer][kVec];
  ss = 0.0;
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    Vec out;
#pragma unroll
    for (int e = 0; e < kVec; ++e) {
      const float normed = Elem<T>::to_float(Elem<T>::from_float(__fmul_rn(Elem<T>::to_float(xv[k].e[e]), r)));
      float s = Elem<T>::to_float(Elem<T>::from_float(__fmul_rn(Elem<T>::to_float(wv[k].e[e]), normed)));
      if (residual != nullptr) s = Elem<T>::to_float(Elem<T>::from_float(__fadd_rn(Elem<T>::to_float(rv[k].e[e]), s)));
      out.e[e] = Elem<T>::from_float(s);
      sv[k][e] = s;
      ss += static_cast<double>(__fmul_rn(s, s));
    }
    if (sum_out != nullptr) *reinterpret_cast<Vec*>(sum_out + base + (k * kNormThreads + threadIdx.x) * kVec) = out;
  }
  if (weight2 == nullptr) return;
  r = inverse_rms(block_sum_double(ss, scratch), hidden, eps);
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    Vec out;
#pragma unroll
    for (int e = 0; e < kVec; ++e) {
      const float normed = Elem<T>::to_float(Elem<T>::from_float(__fmul_rn(sv[k][e], r)));
      out.e[e] = Elem<T>::from_float(__fmul_rn(Elem<T>::to_float(w2v[k].e[e]), normed));
    }
    *reinterpret_cast<Vec*>(norm_out + base + (k * kNormThreads + threadIdx.x) * kVec) = out;
  }
}

// out = T(T(a * cos) + T(rot * sin)): the two products and the sum round separately, as
// `x * cos + rotate_half(x) * sin` does on tensors of type T.
template <typename T>
__device__ __forceinline__ T rotary(T a, T rot, T c, T s, bool negate) {
  const float first = Elem<T>::to_float(Elem<T>::from_float(__fmul_rn(Elem<T>::to_float(a), Elem<T>::to_float(c))));
  const float r = negate ? -Elem<T>::to_float(rot) : Elem<T>::to_float(rot);
  const float second = Elem<T>::to_float(Elem<T>::from_float(__fmul_rn(r, Elem<T>::to_float(s))));
  return Elem<T>::from_float(__fadd_rn(first, second));
}

// One CTA per row.  A work item is one (head, j < head_dim / 2) pair of elements j and
// j + head_dim / 2, kVec pairs at a time; heads 0 .. q_heads-1 are q, the rest are k.
template <typename T, int kVec>
__global__ void __launch_bounds__(kRopeThreads)
rope_kv_write_kernel(const T* __restrict__ q, int64_t q_stride, const T* __restrict__ k, int64_t k_stride,
                     const T* __restrict__ v, int64_t v_stride, const T* __restrict__ cos_table,
                     const T* __restrict__ sin_table, T* __restrict__ q_out, T* __restrict__ key_cache,
                     T* __restrict__ value_cache, int64_t block_stride, int64_t token_stride, int64_t num_blocks,
                     int block_size, int q_heads, int kv_heads, int head_dim,
                     const int64_t* __restrict__ write_blocks, const int64_t* __restrict__ write_offsets,
                     const uint8_t* __restrict__ write_mask, const int32_t* __restrict__ active_rows) {
  struct alignas(sizeof(T) * kVec) Vec { T e[kVec]; };
  const int row = blockIdx.x;
  const int half = head_dim / 2, per_half = half / kVec;
  bool store = !(active_rows != nullptr && row >= *active_rows) && !(write_mask != nullptr && write_mask[row] == 0);
  T* key_row = nullptr;
  T* value_row = nullptr;
  if (store) {
    const int64_t block = write_blocks[row], offset = write_offsets[row];
    store = block >= 0 && block < num_blocks && offset >= 0 && offset < block_size;
    if (store) {
      key_row = key_cache + block * block_stride + offset * token_stride;
      value_row = value_cache + block * block_stride + offset * token_stride;
    }
  }
  const T* cos_row = cos_table + static_cast<int64_t>(row) * head_dim;
  const T* sin_row = sin_table + static_cast<int64_t>(row) * head_dim;
  const int items = (q_heads + kv_heads) * per_half;
  for (int item = threadIdx.x; item < items; item += kRopeThreads) {
    const int head = item / per_half, j = (item % per_half) * kVec;
    const bool is_q = head < q_heads;
    if (!is_q && !store) continue;
    const T* src = is_q ? q + static_cast<int64_t>(row) * q_stride + static_cast<int64_t>(head) * head_dim
                        : k + static_cast<int64_t>(row) * k_stride + static_cast<int64_t>(head - q_heads) * head_dim;
    T* dst = is_q ? q_out + (static_cast<int64_t>(row) * q_heads + head) * head_dim
                  : key_row + static_cast<int64_t>(head - q_heads) * head_dim;
    const Vec lo = *reinterpret_cast<const Vec*>(src + j), hi = *reinterpret_cast<const Vec*>(src + j + half);
    const Vec cl = *reinterpret_cast<const Vec*>(cos_row + j), ch = *reinterpret_cast<const Vec*>(cos_row + j + half);
    const Vec sl = *reinterpret_cast<const Vec*>(sin_row + j), sh = *reinterpret_cast<const Vec*>(sin_row + j + half);
    Vec out_lo, out_hi;
#pragma unroll
    for (int e = 0; e < kVec; ++e) {
      out_lo.e[e] = rotary(lo.e[e], hi.e[e], cl.e[e], sl.e[e], true);    // rotate_half: (-second, first)
      out_hi.e[e] = rotary(hi.e[e], lo.e[e], ch.e[e], sh.e[e], false);
    }
    *reinterpret_cast<Vec*>(dst + j) = out_lo;
    *reinterpret_cast<Vec*>(dst + j + half) = out_hi;
  }
  if (!store) return;
  const int v_items = kv_heads * head_dim / kVec;
  const T* v_row = v + static_cast<int64_t>(row) * v_stride;
  for (int item = threadIdx.x; item < v_items; item += kRopeThreads)
    reinterpret_cast<Vec*>(value_row)[item] = reinterpret_cast<const Vec*>(v_row)[item];
}

}  // namespace
}  // namespace rlt

extern "C" RLT_API int rlt_sandwich_norm(const void* x, const void* weight, const void* residual, void* sum_out,
                                         const void* weight2, void* norm_out, int rows, int hidden, float eps,
                                         int dtype, rlt_stream_t stream) {
  using namespace rlt;
  RLT_REQUIRE(dtype_valid(dtype), "sandwich_norm: dtype must be float32, float16 or bfloat16");
  RLT_REQUIRE(rows >= 0 && hidden > 0 && eps >= 0.0f, "sandwich_norm: invalid shape or eps");
  if (rows == 0) return RLT_OK;
  RLT_REQUIRE(x && weight, "sandwich_norm: null input");
  RLT_REQUIRE(sum_out || (weight2 && norm_out), "sandwich_norm: no output requested");
  RLT_REQUIRE((weight2 == nullptr) == (norm_out == nullptr), "sandwich_norm: weight2 and norm_out go together");
  const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
  if (smem > 32u * 1024u) {
    set_last_error_text("sandwich_norm: hidden size above 8192 is not supported");
    return RLT_ERR_UNSUPPORTED;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // rows that are a whole number of 16-byte vectors per thread stay in registers
  const int per_thread = hidden * static_cast<int>(dtype_size(dtype)) / (kNormThreads * 16);
  const bool vectors = hidden * static_cast<int>(dtype_size(dtype)) == per_thread * kNormThreads * 16 &&
                       (per_thread == 1 || per_thread == 2 || per_thread == 4) && aligned16(x) && aligned16(weight) &&
                       aligned16(residual) && aligned16(sum_out) && aligned16(weight2) && aligned16(norm_out);
  if (vectors) {
#define RLT_NORM_LAUNCH(T, P)                                                                                   \
  sandwich_norm_vec_kernel<T, P><<<rows, kNormThreads, 0, s>>>(                                                 \
      static_cast<const T*>(x), static_cast<const T*>(weight), static_cast<const T*>(residual),                 \
      static_cast<T*>(sum_out), static_cast<const T*>(weight2), static_cast<T*>(norm_out), hidden, eps)
    RLT_DISPATCH_DTYPE(dtype, T, {
      if (per_thread == 1) RLT_NORM_LAUNCH(T, 1);
      else if (per_thread == 2) RLT_NORM_LAUNCH(T, 2);
      else RLT_NORM_LAUNCH(T, 4);
    });
#undef RLT_NORM_LAUNCH
    return launch_status("sandwich_norm_vec_kernel");
  }
  RLT_DISPATCH_DTYPE(dtype, T, (sandwich_norm_kernel<T><<<rows, kNormThreads, smem, s>>>(
                                   static_cast<const T*>(x), static_cast<const T*>(weight),
                                   static_cast<const T*>(residual), static_cast<T*>(sum_out),
                                   static_cast<const T*>(weight2), static_cast<T*>(norm_out), hidden, eps)));
  return launch_status("sandwich_norm_kernel");
}

extern "C" RLT_API int rlt_rope_kv_write(const void* q, int64_t q_row_stride, const void* k, int64_t k_row_stride,
                                         const void* v, int64_t v_row_stride, const void* cos_table,
                                         const void* sin_table, void* q_out, void* key_cache, void* value_cache,
                                         int64_t block_stride, int64_t token_stride, int64_t num_blocks,
                                         int block_size, int q_heads, int kv_heads, int head_dim, int dtype,
                                         const int64_t* write_blocks, const int64_t* write_offsets,
                                         const uint8_t* write_mask, const int32_t* active_rows, int rows,
                                         rlt_stream_t stream) {
  using namespace rlt;
  RLT_REQUIRE(dtype_valid(dtype), "rope_kv_write: dtype must be float32, float16 or bfloat16");
  RLT_REQUIRE(rows >= 0 && q_heads > 0 && kv_heads > 0 && head_dim > 0 && head_dim % 2 == 0 && block_size > 0 &&
                  num_blocks > 0,
              "rope_kv_write: invalid shape (head_dim must be even)");
  if (rows == 0) return RLT_OK;
  RLT_REQUIRE(q && k && v && cos_table && sin_table && q_out && key_cache && value_cache && write_blocks &&
                  write_offsets,
              "rope_kv_write: null pointer");
  RLT_REQUIRE(q_row_stride >= static_cast<int64_t>(q_heads) * head_dim &&
                  k_row_stride >= static_cast<int64_t>(kv_heads) * head_dim &&
                  v_row_stride >= static_cast<int64_t>(kv_heads) * head_dim,
              "rope_kv_write: row strides smaller than a row");
  RLT_REQUIRE(token_stride >= static_cast<int64_t>(kv_heads) * head_dim && block_stride > 0,
              "rope_kv_write: the [kv_heads, head_dim] tail of the cache view must be contiguous");
  const int64_t es = static_cast<int64_t>(dtype_size(dtype));
  const int vec = static_cast<int>(16 / es);
  auto multiple = [&](int64_t elements) { return elements % vec == 0; };
  const bool wide = (head_dim / 2) % vec == 0 && multiple(q_row_stride) && multiple(k_row_stride) &&
                    multiple(v_row_stride) && multiple(block_stride) && multiple(token_stride) && aligned16(q) &&
                    aligned16(k) && aligned16(v) && aligned16(cos_table) && aligned16(sin_table) && aligned16(q_out) &&
                    aligned16(key_cache) && aligned16(value_cache);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define RLT_ROPE_LAUNCH(T, V)                                                                                 \
  rope_kv_write_kernel<T, V><<<rows, kRopeThreads, 0, s>>>(                                                   \
      static_cast<const T*>(q), q_row_stride, static_cast<const T*>(k), k_row_stride, static_cast<const T*>(v), \
      v_row_stride, static_cast<const T*>(cos_table), static_cast<const T*>(sin_table), static_cast<T*>(q_out), \
      static_cast<T*>(key_cache), static_cast<T*>(value_cache), block_stride, token_stride, num_blocks,        \
      block_size, q_heads, kv_heads, head_dim, write_blocks, write_offsets, write_mask, active_rows)
  if (dtype == RLT_F32) { if (wide) RLT_ROPE_LAUNCH(float, 4); else RLT_ROPE_LAUNCH(float, 1); }
  else if (dtype == RLT_F16) { if (wide) RLT_ROPE_LAUNCH(__half, 8); else RLT_ROPE_LAUNCH(__half, 1); }
  else { if (wide) RLT_ROPE_LAUNCH(__nv_bfloat16, 8); else RLT_ROPE_LAUNCH(__nv_bfloat16, 1); }
#undef RLT_ROPE_LAUNCH
  return launch_status("rope_kv_write_kernel");
}
