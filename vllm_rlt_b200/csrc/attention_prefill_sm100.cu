// Packed causal prefill over the paged KV cache for sm_100a: head_dim 128, 16-token pages,
// fp16 / bf16.  The verify kernel scores at most 16 query rows per pass over a context, which
// is right for verification rows and wrong for a prompt: a prompt of n tokens would read its
// K/V n / 16 times.  Here a CTA owns 64 consecutive query tokens of one sequence and one query
// head and walks that sequence's pages once, 64 tokens (four pages) per shared-memory stage.
//
//   plan kernel   one CTA turns cu_seqlens_q into a list of (sequence, first query, count)
//                 tiles, the last tile of a sequence first (it sees the longest context).
//   main kernel   four warps of 16 query rows each.  Thread 0 copies the next four pages with
//                 TMA (one copy per page through the 5-D map over both caches, 128-byte
//                 swizzle) into a two-stage ring guarded by full / empty mbarriers; every warp
//                 scores a stage (up to 64 keys) with 64 + 64 m16n8k16 tensor-core instructions
//                 around one fp32 online-softmax step in the log2 domain, skipping pages that lie
//                 entirely in its rows' causal future and masking only the stages its diagonal
//                 crosses.
//
// Causality is bottom-right aligned (`vllm_rlt/kernels/triton_attention.py:205-366` of the
// reference): query i of the n_s new tokens of sequence s sees positions 0 .. len_s - n_s + i.
// This is GEMM-shaped work: 4 * D flops per (query, key) pair against 2 * D * sizeof bytes per
// key read once per 64 queries, about 128 flop/byte — tensor-bound, unlike the verify path.
#include <cuda.h>
#include <math.h>

#include "attention.cuh"
#include "sm100_primitives.cuh"

namespace rlt {
namespace {

constexpr int kTileRows = 64;                  // query tokens per CTA
constexpr int kTilePages = 4;                  // pages per stage (64 keys)
#ifndef RLT_PREFILL_STAGES
#define RLT_PREFILL_STAGES 2
#endif
constexpr int kPrefillStages = RLT_PREFILL_STAGES;
constexpr int kPrefillWarps = kTileRows / 16;
constexpr int kPrefillPlanThreads = 1024;

struct PrefillHeader {
  unsigned tiles;
  unsigned error;
};
struct PrefillTile {
  int seq;
  int first;   // first query of the tile, counted from the sequence's first new token
  int count;   // 1 .. 64
  int pad;
};

struct __align__(1024) PrefillShared {
  unsigned char stages[kPrefillStages][kTilePages][kStageBytes];  // per page: K lo | K hi | V lo | V hi
  unsigned long long full[kPrefillStages];
  unsigned long long empty[kPrefillStages];
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Tile list: sequence s contributes ceil(n_s / 64) tiles, written last tile first.
__global__ void __launch_bounds__(kPrefillPlanThreads)
prefill_plan_kernel(const int32_t* __restrict__ cu_seqlens_q, int seqs, PrefillHeader* header,
                    PrefillTile* tiles) {
  __shared__ int warp_totals[32];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int base = 0; base < seqs; base += kPrefillPlanThreads) {
    __syncthreads();
    const int s = base + threadIdx.x;
    const int n = s < seqs ? max(cu_seqlens_q[s + 1] - cu_seqlens_q[s], 0) : 0;
    const int mine = (n + kTileRows - 1) / kTileRows;
    int inc = mine;
#pragma unroll
    for (int x = 1; x < 32; x <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, inc, x);
      if (lane >= x) inc += o;
    }
    if (lane == 31) warp_totals[warp] = inc;
    __syncthreads();
    int before = carry;
    for (int w = 0; w < warp; ++w) before += warp_totals[w];
    const int start = before + inc - mine;
    for (int t = 0; t < mine; ++t) {
      const int first = (mine - 1 - t) * kTileRows;
      tiles[start + t] = PrefillTile{s, first, min(kTileRows, n - first), 0};
    }
    __syncthreads();
    if (threadIdx.x == kPrefillPlanThreads - 1) carry = before + inc;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    header->tiles = static_cast<unsigned>(carry);
    header->error = 0;
  }
}

template <bool kBF16>
__global__ void __launch_bounds__(kPrefillWarps * 32)
prefill_attention_kernel(const __grid_constant__ CUtensorMap kv_map, AttentionArgs a, const PrefillHeader* header,
                         const PrefillTile* tiles, unsigned* error, float scale_log2, int k_first) {
  using T = typename std::conditional<kBF16, __nv_bfloat16, __half>::type;
  if (blockIdx.x >= header->tiles) return;
  extern __shared__ unsigned char smem_raw[];
  PrefillShared& sm = *reinterpret_cast<PrefillShared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const PrefillTile tile = tiles[blockIdx.x];
  const int q_head = blockIdx.y, kv_head = q_head / (a.q_heads / a.kv_heads);
  const int seq_first = a.cu_seqlens_q[tile.seq];
  const int n_new = a.cu_seqlens_q[tile.seq + 1] - seq_first;
  const int base_len = a.context_lengths[tile.seq] - n_new + 1;   // keys visible to the sequence's first new token
  // visible keys of fragment rows g and g + 8 of this warp (0 for rows beyond the tile)
  const int row0 = warp * 16 + g, row1 = row0 + 8;
  const int len0 = row0 < tile.count ? max(base_len + tile.first + row0, 0) : 0;
  const int len1 = row1 < tile.count ? max(base_len + tile.first + row1, 0) : 0;
  const int warp_rows = min(max(tile.count - warp * 16, 0), 16);
  const int warp_max = warp_rows > 0 ? max(base_len + tile.first + warp * 16 + warp_rows - 1, 0) : 0;
  const int warp_min = warp_rows > 0 ? max(base_len + tile.first + warp * 16, 0) : 0;
  const int kv_end = max(base_len + tile.first + tile.count - 1, 0);   // keys the tile's last row sees
  const int total_pages = (kv_end + kPage - 1) / kPage;
  const int kv_tiles = (total_pages + kTilePages - 1) / kTilePages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPrefillStages; ++s) {
      mbar_init(smem_u32(&sm.full[s]), 1);
      mbar_init(smem_u32(&sm.empty[s]), kPrefillWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const uint64_t policy = policy_evict_first();
  const int32_t* table = a.block_tables + static_cast<int64_t>(tile.seq) * a.table_width;
  auto issue = [&](int jt) {   // thread 0: the pages of key tile jt into stage jt % kPrefillStages
    const int stage = jt % kPrefillStages;
    const int pages = min(kTilePages, total_pages - jt * kTilePages);
    const uint32_t bar = smem_u32(&sm.full[stage]);
    mbar_expect_tx(bar, pages * kStageBytes);
    for (int p = 0; p < pages; ++p)
      tma_load_page_kv(smem_u32(&sm.stages[stage][p][0]), &kv_map, kv_head * 2, table[jt * kTilePages + p], bar, policy);
  };
  if (threadIdx.x == 0)
    for (int jt = 0; jt < min(kPrefillStages, kv_tiles); ++jt) issue(jt);

  // ldmatrix source offsets inside a page (see the verify kernel: same stage layout)
  uint32_t koff[8], voff[8];
  {
    const int mi = lane >> 3;
    const int ktoken = ((mi >> 1) << 3) + (lane & 7), vtoken = ((mi & 1) << 3) + (lane & 7);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int chunk16 = ((ks & 3) << 1) + (mi & 1);
      koff[ks] = (k_first ? 0 : kTileBytes) + ((ks >> 2) << 11) + ktoken * 128 + ((chunk16 ^ (ktoken & 7)) << 4);
    }
#pragma unroll
    for (int jp = 0; jp < 8; ++jp) {
      const int c = 2 * jp + (mi >> 1);
      voff[jp] = (k_first ? kTileBytes : 0) + ((c >> 3) << 11) + vtoken * 128 + (((c & 7) ^ (vtoken & 7)) << 4);
    }
  }

  // Q fragments of this warp's 16 rows
  const int64_t q0 = ((static_cast<int64_t>(seq_first) + tile.first + row0) * a.q_heads + q_head) * kHeadDim;
  const int64_t q1 = ((static_cast<int64_t>(seq_first) + tile.first + row1) * a.q_heads + q_head) * kHeadDim;
  const uint32_t* qp = reinterpret_cast<const uint32_t*>(a.q);
  uint32_t qa[8][4];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const int c = ks * 16 + 2 * t;
    qa[ks][0] = len0 > 0 ? __ldg(qp + ((q0 + c) >> 1)) : 0u;
    qa[ks][1] = len1 > 0 ? __ldg(qp + ((q1 + c) >> 1)) : 0u;
    qa[ks][2] = len0 > 0 ? __ldg(qp + ((q0 + c + 8) >> 1)) : 0u;
    qa[ks][3] = len1 > 0 ? __ldg(qp + ((q1 + c + 8) >> 1)) : 0u;
  }
  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) { o[j][0] = 0.f; o[j][1] = 0.f; o[j][2] = 0.f; o[j][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  bool failed = false;

  for (int jt = 0; jt < kv_tiles && !failed; ++jt) {
    const int stage = jt % kPrefillStages;
    const uint32_t parity = (jt / kPrefillStages) & 1;
    if (!mbar_wait(smem_u32(&sm.full[stage]), parity)) { failed = true; break; }
    const int pages = min(kTilePages, total_pages - jt * kTilePages);
    const int tile_start = jt * kTilePages * kPage;
    // pages of this stage that hold a key some row of this warp can see (the rest is its causal future)
    const int mine = min(pages, max(warp_max - tile_start + kPage - 1, 0) / kPage);
    if (mine > 0) {
      // S = Q K^T for up to 64 keys: one softmax step per stage
      float s[2 * kTilePages][4];
#pragma unroll
      for (int p = 0; p < kTilePages; ++p) {
        if (p < mine) {
          const uint32_t base = smem_u32(&sm.stages[stage][p][0]);
          float sa[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
          float sb[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            uint32_t b[4];
            ldmatrix_x4(base + koff[ks], b);
            if (ks & 1) {
              mma_16816<kBF16>(sb[0], qa[ks], b[0], b[1]);
              mma_16816<kBF16>(sb[1], qa[ks], b[2], b[3]);
            } else {
              mma_16816<kBF16>(sa[0], qa[ks], b[0], b[1]);
              mma_16816<kBF16>(sa[1], qa[ks], b[2], b[3]);
            }
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) { s[2 * p][e] = sa[0][e] + sb[0][e]; s[2 * p + 1][e] = sa[1][e] + sb[1][e]; }
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) { s[2 * p][e] = -INFINITY; s[2 * p + 1][e] = -INFINITY; }
        }
      }
      if (tile_start + mine * kPage > warp_min || warp_rows < 16) {   // the diagonal crosses this stage
#pragma unroll
        for (int nt = 0; nt < 2 * kTilePages; ++nt) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int pos = tile_start + nt * 8 + 2 * t + e;
            if (pos >= len0) s[nt][e] = -INFINITY;
            if (pos >= len1) s[nt][2 + e] = -INFINITY;
          }
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 2 * kTilePages; ++nt) {
        mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
        mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0 * scale_log2), mn1 = fmaxf(m1, mx1 * scale_log2);
      const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
      const bool moved = (mn0 != m0) || (mn1 != m1);
      const float al0 = fast_exp2(m0 - mu0), al1 = fast_exp2(m1 - mu1);
      m0 = mn0; m1 = mn1;
      uint32_t pa[kTilePages][4];
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int p = 0; p < kTilePages; ++p) {
        const float p00 = fast_exp2(fmaf(s[2 * p][0], scale_log2, -mu0)), p01 = fast_exp2(fmaf(s[2 * p][1], scale_log2, -mu0));
        const float p02 = fast_exp2(fmaf(s[2 * p][2], scale_log2, -mu1)), p03 = fast_exp2(fmaf(s[2 * p][3], scale_log2, -mu1));
        const float p10 = fast_exp2(fmaf(s[2 * p + 1][0], scale_log2, -mu0)), p11 = fast_exp2(fmaf(s[2 * p + 1][1], scale_log2, -mu0));
        const float p12 = fast_exp2(fmaf(s[2 * p + 1][2], scale_log2, -mu1)), p13 = fast_exp2(fmaf(s[2 * p + 1][3], scale_log2, -mu1));
        sum0 += (p00 + p01) + (p10 + p11);
        sum1 += (p02 + p03) + (p12 + p13);
        pa[p][0] = pack2<kBF16>(p00, p01);
        pa[p][1] = pack2<kBF16>(p02, p03);
        pa[p][2] = pack2<kBF16>(p10, p11);
        pa[p][3] = pack2<kBF16>(p12, p13);
      }
      l0 = l0 * al0 + sum0;
      l1 = l1 * al1 + sum1;
      if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
        for (int jn = 0; jn < 16; ++jn) { o[jn][0] *= al0; o[jn][1] *= al0; o[jn][2] *= al1; o[jn][3] *= al1; }
      }
      // O += P V, page by page
#pragma unroll
      for (int p = 0; p < kTilePages; ++p) {
        if (p < mine) {
          const uint32_t base = smem_u32(&sm.stages[stage][p][0]);
#pragma unroll
          for (int jp = 0; jp < 8; ++jp) {
            uint32_t b[4];
            ldmatrix_x4_trans(base + voff[jp], b);
            mma_16816<kBF16>(o[2 * jp], pa[p], b[0], b[1]);
            mma_16816<kBF16>(o[2 * jp + 1], pa[p], b[2], b[3]);
          }
        }
      }
    }
    // this warp is done with the stage; thread 0 refills it once all four warps are
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&sm.empty[stage]));
    if (threadIdx.x == 0 && jt + kPrefillStages < kv_tiles) {
      if (!mbar_wait(smem_u32(&sm.empty[stage]), parity)) failed = true;
      else issue(jt + kPrefillStages);
    }
    failed = __shfl_sync(0xffffffffu, failed ? 1 : 0, 0) != 0;
  }
  if (failed) {
    if (lane == 0) atomicOr(error, 1u);
    return;
  }

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  T* out = static_cast<T*>(a.out);
  if (row0 < tile.count) {
    const float inv = l0 > 0.f ? 1.0f / l0 : 0.f;
    uint32_t* dst = reinterpret_cast<uint32_t*>(out + q0);
#pragma unroll
    for (int jn = 0; jn < 16; ++jn) dst[jn * 4 + t] = pack2<kBF16>(o[jn][0] * inv, o[jn][1] * inv);
  }
  if (row1 < tile.count) {
    const float inv = l1 > 0.f ? 1.0f / l1 : 0.f;
    uint32_t* dst = reinterpret_cast<uint32_t*>(out + q1);
#pragma unroll
    for (int jn = 0; jn < 16; ++jn) dst[jn * 4 + t] = pack2<kBF16>(o[jn][2] * inv, o[jn][3] * inv);
  }
}

size_t tile_capacity(int rows, int seqs) { return static_cast<size_t>(rows) / kTileRows + static_cast<size_t>(seqs) + 1; }

}  // namespace

bool prefill_sm100_supported(const AttentionArgs& a) {
  return a.cu_seqlens_q != nullptr && attention_sm100_supported(a);
}

size_t prefill_sm100_workspace_bytes(int rows, int seqs) {
  return 256 + sizeof(PrefillTile) * tile_capacity(rows, seqs);
}

// RLT_ERR_UNSUPPORTED when the two caches cannot share one tensor map (the caller then scores
// the rows with the verify kernel).
int launch_prefill_sm100(const AttentionArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  if (workspace == nullptr || workspace_bytes < prefill_sm100_workspace_bytes(a.rows, a.table_rows) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) {
    set_last_error_text("prefill_attention: workspace missing, misaligned or too small");
    return RLT_ERR_WORKSPACE;
  }
  CUtensorMap kv_map;
  bool k_first = true;
  if (make_joint_map(&kv_map, a, &k_first) != RLT_OK) return RLT_ERR_UNSUPPORTED;
  PrefillHeader* header = static_cast<PrefillHeader*>(workspace);
  PrefillTile* tiles = reinterpret_cast<PrefillTile*>(static_cast<unsigned char*>(workspace) + 256);
  prefill_plan_kernel<<<1, kPrefillPlanThreads, 0, stream>>>(a.cu_seqlens_q, a.table_rows, header, tiles);
  int status = launch_status("prefill_plan_kernel");
  if (status != RLT_OK) return status;
  const size_t smem = sizeof(PrefillShared) + 1024;
  const float scale_log2 = static_cast<float>(1.4426950408889634 / sqrt(static_cast<double>(kHeadDim)));
  const dim3 grid(static_cast<unsigned>(tile_capacity(a.rows, a.table_rows)), static_cast<unsigned>(a.q_heads));
  if (a.dtype == RLT_BF16) {
    auto kernel = prefill_attention_kernel<true>;
    RLT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    kernel<<<grid, kPrefillWarps * 32, smem, stream>>>(kv_map, a, header, tiles, &header->error, scale_log2, k_first ? 1 : 0);
  } else {
    auto kernel = prefill_attention_kernel<false>;
    RLT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    kernel<<<grid, kPrefillWarps * 32, smem, stream>>>(kv_map, a, header, tiles, &header->error, scale_log2, k_first ? 1 : 0);
  }
  return launch_status("prefill_attention_kernel");
}

}  // namespace rlt
