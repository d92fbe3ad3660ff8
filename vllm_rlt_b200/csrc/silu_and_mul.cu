// SiLU-and-Mul for the Ouro MLP: out = T(silu_f32(gate)) * up.
//
// Pure streaming op (3 * n * sizeof(T) bytes of traffic, ~12 flops per element).  At the path's sizes
// (4 - 35 MB per call) a call lasts a few microseconds, so what counts is how quickly the whole chip has
// its loads in flight and how little tail it leaves: every thread handles ONE 16-byte vector of each
// input and the grid covers the array without a grid-stride loop.  (Measured on B200 at [128 .. 1024,
// 5632] bf16: four vectors per thread were 35 - 60 % slower, two 15 - 25 %, 32-byte `ld.global.v8.b32`
// vectors 4 % slower from HBM.)  One launch covers the vector body and the scalar edges (unaligned
// head, tail).
//
// Arithmetic contract (bit-exact with F.silu(gate) * up on the same GPU):
//   silu(x) = x / (1 + expf(-x)) in fp32, rounded to T, then one multiply in T.
#include "common.cuh"

namespace rlt {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + expf(-x)); }

template <typename T> struct Pack;  // 16 bytes of T

template <> struct Pack<float> {
  __device__ __forceinline__ static uint4 apply(uint4 g, uint4 u) {
    float4 gf = *reinterpret_cast<float4*>(&g), uf = *reinterpret_cast<float4*>(&u), o;
    o.x = __fmul_rn(silu_f32(gf.x), uf.x);
    o.y = __fmul_rn(silu_f32(gf.y), uf.y);
    o.z = __fmul_rn(silu_f32(gf.z), uf.z);
    o.w = __fmul_rn(silu_f32(gf.w), uf.w);
    return *reinterpret_cast<uint4*>(&o);
  }
  __device__ __forceinline__ static float scalar(float g, float u) { return __fmul_rn(silu_f32(g), u); }
};

template <> struct Pack<__half> {
  __device__ __forceinline__ static uint32_t pair(uint32_t g, uint32_t u) {
    float2 gf = __half22float2(*reinterpret_cast<__half2*>(&g));
    __half2 act = __floats2half2_rn(silu_f32(gf.x), silu_f32(gf.y));
    __half2 r = __hmul2(act, *reinterpret_cast<__half2*>(&u));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  __device__ __forceinline__ static uint4 apply(uint4 g, uint4 u) {
    return make_uint4(pair(g.x, u.x), pair(g.y, u.y), pair(g.z, u.z), pair(g.w, u.w));
  }
  __device__ __forceinline__ static __half scalar(__half g, __half u) {
    return __hmul(__float2half_rn(silu_f32(__half2float(g))), u);
  }
};

template <> struct Pack<__nv_bfloat16> {
  __device__ __forceinline__ static uint32_t pair(uint32_t g, uint32_t u) {
    float2 gf = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&g));
    __nv_bfloat162 act = __floats2bfloat162_rn(silu_f32(gf.x), silu_f32(gf.y));
    __nv_bfloat162 r = __hmul2(act, *reinterpret_cast<__nv_bfloat162*>(&u));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  __device__ __forceinline__ static uint4 apply(uint4 g, uint4 u) {
    return make_uint4(pair(g.x, u.x), pair(g.y, u.y), pair(g.z, u.z), pair(g.w, u.w));
  }
  __device__ __forceinline__ static __nv_bfloat16 scalar(__nv_bfloat16 g, __nv_bfloat16 u) {
    return __hmul(__float2bfloat16_rn(silu_f32(__bfloat162float(g))), u);
  }
};

// The vector body of one contiguous run: `nvec` 16-byte vectors starting at (g, u, o), spread over
// `nthreads` threads of which this one is `tid`.
template <typename T>
__device__ __forceinline__ void vector_body(const T* __restrict__ g, const T* __restrict__ u, T* __restrict__ o,
                                            int64_t nvec, int64_t tid, int64_t nthreads) {
  const uint4* gv = reinterpret_cast<const uint4*>(g);
  const uint4* uv = reinterpret_cast<const uint4*>(u);
  uint4* ov = reinterpret_cast<uint4*>(o);
  for (int64_t i = tid; i < nvec; i += nthreads) ov[i] = Pack<T>::apply(__ldg(gv + i), __ldg(uv + i));
}

// head: leading elements handled one by one so that the vector body starts 16-byte aligned
// in all three arrays (head == n sends everything through the scalar loop).
template <typename T>
__global__ void __launch_bounds__(kThreads)
silu_and_mul_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out,
                    int64_t n, int64_t head) {
  constexpr int kElems = 16 / sizeof(T);
  const int64_t nvec = (n - head) / kElems;
  const int64_t tail_start = head + nvec * kElems;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * kThreads;
  vector_body<T>(gate + head, up + head, out + head, nvec, tid, nthreads);
  const int64_t edges = head + (n - tail_start);
  for (int64_t e = tid; e < edges; e += nthreads) {
    int64_t i = e < head ? e : tail_start + (e - head);
    out[i] = Pack<T>::scalar(gate[i], up[i]);
  }
}

// Most CTAs per SM a launch asks for: the vector body gets one vector per thread up to this many (beyond
// it a grid-stride loop takes over); the all-scalar path (arrays with different misalignments) does better
// with fewer, longer-lived threads.
constexpr int kVectorCtasPerSm = 32, kScalarCtasPerSm = 8;

template <typename T>
int launch(const void* gate, const void* up, void* out, int64_t n, cudaStream_t stream) {
  constexpr int kElems = 16 / sizeof(T);
  DeviceInfo info;
  int status = current_device_info(&info);
  if (status != RLT_OK) return status;
  const uintptr_t ga = reinterpret_cast<uintptr_t>(gate) & 15u;
  const uintptr_t ua = reinterpret_cast<uintptr_t>(up) & 15u;
  const uintptr_t oa = reinterpret_cast<uintptr_t>(out) & 15u;
  int64_t head = n;  // all scalar unless the three arrays share one misalignment
  if (ga == ua && ga == oa && ga % sizeof(T) == 0) {
    head = ga == 0 ? 0 : static_cast<int64_t>((16 - ga) / sizeof(T));
    if (head > n) head = n;
  }
  const int64_t nvec = (n - head) / kElems;
  const int64_t scalar_work = n - nvec * kElems;
  int64_t work = nvec > scalar_work ? nvec : scalar_work;
  int64_t blocks = (work + kThreads - 1) / kThreads;
  const int64_t cap = static_cast<int64_t>(info.sm_count) * (nvec > 0 ? kVectorCtasPerSm : kScalarCtasPerSm);
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  silu_and_mul_kernel<T><<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(
      static_cast<const T*>(gate), static_cast<const T*>(up), static_cast<T*>(out), n, head);
  return launch_status("silu_and_mul_kernel");
}

// Row-strided form: gate and up are [rows, cols] views with their own row strides (the two column
// halves of one fused gate/up projection), out is contiguous.  A row is covered by `row_ctas` CTAs
// (blockIdx.x = row * row_ctas + part), every thread handling one 16-byte vector; rows whose
// pointers are not 16-byte aligned go through the scalar loop.
template <typename T>
__global__ void __launch_bounds__(kThreads)
silu_and_mul_rows_kernel(const T* __restrict__ gate, int64_t gate_stride, const T* __restrict__ up, int64_t up_stride,
                         T* __restrict__ out, int64_t cols, int row_ctas, int vector_ok) {
  constexpr int kElems = 16 / sizeof(T);
  const int64_t row = blockIdx.x / row_ctas;
  const int part = blockIdx.x % row_ctas;
  const T* g = gate + row * gate_stride;
  const T* u = up + row * up_stride;
  T* o = out + row * cols;
  const int64_t nvec = vector_ok ? cols / kElems : 0;
  const int64_t tid = static_cast<int64_t>(part) * kThreads + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(row_ctas) * kThreads;
  vector_body<T>(g, u, o, nvec, tid, nthreads);
  for (int64_t i = nvec * kElems + tid; i < cols; i += nthreads) o[i] = Pack<T>::scalar(g[i], u[i]);
}

template <typename T>
int launch_rows(const void* gate, int64_t gate_stride, const void* up, int64_t up_stride, void* out, int64_t rows,
                int64_t cols, cudaStream_t stream) {
  constexpr int kElems = 16 / sizeof(T);
  const bool vector_ok = aligned16(gate) && aligned16(up) && aligned16(out) && gate_stride % kElems == 0 &&
                         up_stride % kElems == 0 && cols % kElems == 0;
  const int64_t per_row = vector_ok ? cols / kElems : cols;
  int64_t row_ctas = (per_row + kThreads - 1) / kThreads;
  if (row_ctas < 1) row_ctas = 1;
  if (row_ctas > 64) row_ctas = 64;
  if (rows * row_ctas > 0x7fffffffll) {
    set_last_error_text("silu_and_mul_packed: too many rows for one launch");
    return RLT_ERR_INVALID;
  }
  silu_and_mul_rows_kernel<T><<<static_cast<unsigned>(rows * row_ctas), kThreads, 0, stream>>>(
      static_cast<const T*>(gate), gate_stride, static_cast<const T*>(up), up_stride, static_cast<T*>(out), cols,
      static_cast<int>(row_ctas), vector_ok ? 1 : 0);
  return launch_status("silu_and_mul_rows_kernel");
}

}  // namespace
}  // namespace rlt

extern "C" RLT_API int rlt_silu_and_mul_packed(const void* gate_up, int64_t row_stride, void* out, int64_t rows,
                                               int64_t cols, int dtype, rlt_stream_t stream) {
  using namespace rlt;
  RLT_REQUIRE(dtype_valid(dtype), "silu_and_mul_packed supports float32, float16 and bfloat16");
  RLT_REQUIRE(rows >= 0 && cols >= 0 && row_stride >= 2 * cols, "silu_and_mul_packed: invalid shape");
  if (rows == 0 || cols == 0) return RLT_OK;
  RLT_REQUIRE(gate_up && out, "silu_and_mul_packed: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int status = RLT_OK;
  RLT_DISPATCH_DTYPE(dtype, T, status = launch_rows<T>(gate_up, row_stride, static_cast<const T*>(gate_up) + cols,
                                                       row_stride, out, rows, cols, s));
  return status;
}

extern "C" RLT_API int rlt_silu_and_mul(const void* gate, const void* up, void* out, int64_t n, int dtype,
                                rlt_stream_t stream) {
  using namespace rlt;
  RLT_REQUIRE(dtype_valid(dtype), "silu_and_mul supports float32, float16 and bfloat16");
  RLT_REQUIRE(n >= 0, "silu_and_mul: negative element count");
  if (n == 0) return RLT_OK;
  RLT_REQUIRE(gate && up && out, "silu_and_mul: null pointer");
  RLT_REQUIRE(out != gate && out != up, "silu_and_mul: output must not alias an input");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int status = RLT_OK;
  RLT_DISPATCH_DTYPE(dtype, T, status = launch<T>(gate, up, out, n, s));
  return status;
}
