// Building blocks shared by the sm_100a attention kernels: shared-memory barriers, TMA page
// copies and their tensor maps, ldmatrix / mma.sync wrappers.
#pragma once

#include <cuda.h>
#include <math.h>

#include <mutex>
#include <type_traits>

#include "attention.cuh"

namespace rlt {

constexpr int kHeadDim = 128;
constexpr int kPage = 16;
constexpr int kTileBytes = kPage * kHeadDim * 2;  // one page of one head: 4 KiB
constexpr int kStageBytes = 2 * kTileBytes;       // K page + V page
constexpr long long kWaitCycles = 4000000000ll;   // bounded waits (about 2 s): give up instead of hanging

// ---- PTX wrappers -----------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false if the phase did not complete within kWaitCycles clock cycles.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > kWaitCycles) return false;
  }
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
// One [64 dims x 16 tokens] box of one page: coordinates (element in token row, token, block).
__device__ __forceinline__ void tma_load_page_half(uint32_t dst, const CUtensorMap* map, int x, int block,
                                                   uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3, %4}], [%5], %6;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(0), "r"(block), "r"(bar), "l"(policy)
      : "memory");
}
// Both 64-dim halves of one head of one page in a single copy: coordinates (element in half,
// token, half-head index, block); lands as [half][token][64 dims], the layout two half copies give.
__device__ __forceinline__ void tma_load_page(uint32_t dst, const CUtensorMap* map, int half_head, int block,
                                              uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3, %4, %5}], [%6], %7;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(0), "r"(half_head), "r"(block), "r"(bar),
        "l"(policy)
      : "memory");
}
// K and V head slices of one page in a single copy through a map whose fourth dimension steps
// from one cache to the other: coordinates (element, token, half-head index, cache, block).
__device__ __forceinline__ void tma_load_page_kv(uint32_t dst, const CUtensorMap* map, int half_head, int block,
                                                 uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3, %4, %5, %6}], [%7], %8;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(0), "r"(half_head), "r"(0), "r"(block), "r"(bar),
        "l"(policy)
      : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <bool kBF16>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (kBF16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Zero token rows [first_row, end_row) of a K or V operand block in shared memory — two halves of 128-byte rows
// (64 dims each), swizzled within the row, so a whole row can be cleared without knowing the swizzle.  Done by the
// whole warp.  Cache slots behind a context's last token were never written: the caller's allocation may hold
// anything there (NaN and Inf bit patterns included), the scores of such keys are masked by assignment, but in
// P V a probability of zero times a NaN is a NaN, so those rows of V are cleared before they are multiplied.
// Ends with the proxy fence the block's next asynchronous reader (an MMA) or writer (the next copy) needs.
__device__ __forceinline__ void zero_rows_warp(unsigned char* half0, unsigned char* half1, int first_row, int end_row, int lane) {
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  const int pieces = (end_row - first_row) * 16;   // eight 16-byte pieces per row and half
  for (int x = lane; x < pieces; x += 32) {
    const int r = first_row + (x >> 4), piece = x & 15;
    *reinterpret_cast<uint4*>(((piece & 8) ? half1 : half0) + r * 128 + ((piece & 7) << 4)) = zero;
  }
  fence_async_proxy();
  __syncwarp();
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <bool kBF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kBF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// ---- tensor maps (host) -------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Tensor map over one layer's cache view as [num_blocks][16 tokens][kv_heads * 128] elements,
// box = 64 elements x 16 tokens x 1 block, 128-byte swizzle.
inline int make_page_map(CUtensorMap* map, const void* base, const AttentionArgs& a) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) {
    set_last_error_text("cuTensorMapEncodeTiled is not available from this driver");
    return RLT_ERR_CUDA;
  }
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(a.kv_heads) * kHeadDim, kPage,
                              static_cast<cuuint64_t>(a.num_blocks)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(a.token_stride) * 2,
                                 static_cast<cuuint64_t>(a.block_stride) * 2};
  const cuuint32_t box[3] = {64, kPage, 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = fn(map, a.dtype == RLT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        3, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error_text("cuTensorMapEncodeTiled rejected the KV cache view");
    return RLT_ERR_CUDA;
  }
  return RLT_OK;
}

// The same view as [num_blocks][kv_heads * 2 half-heads][16 tokens][64] elements: box = 64
// elements x 16 tokens x 2 halves x 1 block.  The half-head stride (128 bytes) is smaller than
// the token stride before it; returns RLT_ERR_UNSUPPORTED if the driver refuses that order.
inline int make_head_map(CUtensorMap* map, const void* base, const AttentionArgs& a) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return RLT_ERR_UNSUPPORTED;
  const cuuint64_t dims[4] = {64, kPage, static_cast<cuuint64_t>(a.kv_heads) * 2,
                              static_cast<cuuint64_t>(a.num_blocks)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(a.token_stride) * 2, 128,
                                 static_cast<cuuint64_t>(a.block_stride) * 2};
  const cuuint32_t box[4] = {64, kPage, 2, 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  const CUresult r = fn(map, a.dtype == RLT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        4, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? RLT_OK : RLT_ERR_UNSUPPORTED;
}

// Both caches as one tensor [num_blocks][2 caches][kv_heads * 2][16 tokens][64]: the cache
// dimension's stride is the distance between the two base addresses, so it exists only when
// that distance is a positive multiple of 16 below 2^40 from `base` (the lower of the two).
inline int make_joint_map(CUtensorMap* map, const AttentionArgs& a, bool* k_first) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return RLT_ERR_UNSUPPORTED;
  const uintptr_t k = reinterpret_cast<uintptr_t>(a.key_cache), v = reinterpret_cast<uintptr_t>(a.value_cache);
  *k_first = k < v;
  const uintptr_t lower = k < v ? k : v, distance = k < v ? v - k : k - v;
  if (distance == 0 || distance % 16 != 0 || distance >= (1ull << 40)) return RLT_ERR_UNSUPPORTED;
  const cuuint64_t dims[5] = {64, kPage, static_cast<cuuint64_t>(a.kv_heads) * 2, 2,
                              static_cast<cuuint64_t>(a.num_blocks)};
  const cuuint64_t strides[4] = {static_cast<cuuint64_t>(a.token_stride) * 2, 128, distance,
                                 static_cast<cuuint64_t>(a.block_stride) * 2};
  const cuuint32_t box[5] = {64, kPage, 2, 2, 1};
  const cuuint32_t elem[5] = {1, 1, 1, 1, 1};
  const CUresult r = fn(map, a.dtype == RLT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        5, reinterpret_cast<void*>(lower), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? RLT_OK : RLT_ERR_UNSUPPORTED;
}

}  // namespace rlt
