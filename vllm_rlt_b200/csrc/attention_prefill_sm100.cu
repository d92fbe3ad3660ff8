// Packed causal prefill over the paged KV cache for sm_100a: head_dim 128, 16-token pages,
// fp16 / bf16.  The verify kernel scores at most 16 query rows per pass over a context, which
// is right for verification rows and wrong for a prompt: a prompt of n tokens would read its
// K/V n / 16 times.  Here a CTA owns a tile of consecutive query tokens of one sequence and one
// query head and walks that sequence's pages once, 64 keys (four pages) per shared-memory stage.
//
//   plan kernel     one CTA turns cu_seqlens_q into a list of (sequence, first query, count)
//                   tiles, the last tile of a sequence first (it sees the longest context).
//   pair kernel     tcgen05 / TMEM, two 128-row query tiles per CTA that share every K / V stage;
//                   Q and P are TMEM operands of the MMAs, separate warps copy, issue and do the
//                   softmax (see the comment above prefill_pair_kernel).  Default for prompts.
//   one-tile kernel tcgen05 / TMEM, one 128-row tile per CTA and two CTAs per SM (above
//                   prefill_umma_kernel).  The pair kernel's predecessor; selectable, no longer a default.
//   mma.sync kernel 64-row tiles, four warps of 16 query rows each.  Thread 0 copies the next four
//                   pages with TMA (one copy per page through the 5-D map over both caches, 128-byte
//                   swizzle) into a two-stage ring guarded by full / empty mbarriers; every warp
//                   scores a stage with 64 + 64 m16n8k16 tensor-core instructions around one fp32
//                   online-softmax step in the log2 domain, skipping pages that lie entirely in
//                   its rows' causal future and masking only the stages its diagonal crosses.
//
// Causality is bottom-right aligned (`vllm_rlt/kernels/triton_attention.py:205-366` of the
// reference): query i of the n_s new tokens of sequence s sees positions 0 .. len_s - n_s + i.
// This is GEMM-shaped work: 4 * D flops per (query, key) pair against 2 * D * sizeof bytes per
// key read once per 64 queries, about 128 flop/byte — tensor-bound, unlike the verify path.
#include <cuda.h>
#include <math.h>
#include <stdlib.h>

#include "attention.cuh"
#include "sm100_primitives.cuh"

namespace rlt {
namespace {

constexpr int kTileRows = 64;                  // query tokens per CTA of the mma.sync kernel
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
  int first;     // first query of the tile, counted from the sequence's first new token
  int count;     // rows of the tile
  int visible;   // keys the tile's first row sees: min(context, table capacity) - new tokens + 1 + first (may be <= 0)
  int q_row;     // the first row's index in the packed query tensor
  int pad[3];
};

struct __align__(1024) PrefillShared {
  unsigned char stages[kPrefillStages][kTilePages][kStageBytes];  // per page: K lo | K hi | V lo | V hi
  unsigned long long full[kPrefillStages];
  unsigned long long empty[kPrefillStages];
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Tile list: sequence s contributes ceil(n_s / tile_rows) tiles, written last tile first.
__global__ void __launch_bounds__(kPrefillPlanThreads)
prefill_plan_kernel(const int32_t* __restrict__ cu_seqlens_q, const int32_t* __restrict__ context_lengths, int table_width,
                    int seqs, int tile_rows, PrefillHeader* header, PrefillTile* tiles) {
  __shared__ int warp_totals[32];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int base = 0; base < seqs; base += kPrefillPlanThreads) {
    __syncthreads();
    const int s = base + threadIdx.x;
    const int seq_first = s < seqs ? cu_seqlens_q[s] : 0;
    const int n = s < seqs ? max(cu_seqlens_q[s + 1] - seq_first, 0) : 0;
    const int base_len = s < seqs ? min(context_lengths[s], table_width * kPage) - n + 1 : 0;   // keys the first new token sees
    const int mine = (n + tile_rows - 1) / tile_rows;
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
      const int first = (mine - 1 - t) * tile_rows;
      tiles[start + t] = PrefillTile{s, first, min(tile_rows, n - first), base_len + first, seq_first + first, {0, 0, 0}};
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
  const int base_len = min(a.context_lengths[tile.seq], a.table_width * kPage) - n_new + 1;   // keys visible to the sequence's first new token
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
    if (jt == kv_tiles - 1 && kv_end < tile_start + pages * kPage) {
      // slots of the last page behind the last key any row of the tile sees (every warp clears them before its own
      // reads: the same zeros from each)
      unsigned char* v_page = &sm.stages[stage][pages - 1][0] + (k_first ? kTileBytes : 0);
      zero_rows_warp(v_page, v_page + 2048, kv_end - tile_start - (pages - 1) * kPage, kPage, lane);
    }
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

// ---- the same tile on the 5th-generation tensor cores (tcgen05 / TMEM) ----------------------
// 128 query tokens of one query head per CTA, 64 keys per stage, five warps.  Q sits in shared
// memory as two K-major 64-dim halves; every K / V page lands as four 2 KiB TMA copies so that a
// stage holds K as [half][64 keys][64 dims] (K-major B operand of S = Q K^T) and V in the same
// shape, which is the MN-major B operand of O += P V.
//   warp 4       issues the copies and, from one thread, every MMA.  Scores are double-buffered
//                in tensor memory (columns 0..63 and 64..127) and the output tile accumulates in
//                columns 128..255.  In steady state it waits for P(j), issues O += P(j) V(j) and
//                right behind it S(j + 2) = Q K(j + 2)^T into the buffer P(j) is read from.
//   warps 0..3   one query row per thread (the row that is its TMEM lane): tcgen05.ld of S(j),
//                online softmax without any shuffle, P(j) as packed bf16 pairs stored with
//                tcgen05.st over the first 32 columns of the same buffer — the A operand of the
//                P V MMA is read from tensor memory — then an arrival on the buffer's barrier.
//                S(j + 1) is complete by then, so these warps never wait for an MMA in steady
//                state.  A row of the output tile is rescaled in place only when its running
//                maximum is raised, after the previous P V product has been committed.
// 97 KiB of shared memory and 256 TMEM columns per CTA: two CTAs per SM.
constexpr int kUmmaRows = 128;
constexpr int kUmmaThreads = 160;
constexpr int kUmmaKeys = 64;
constexpr int kUmmaStages = 2;
constexpr uint32_t kTmemColumns = 256;
constexpr uint32_t kTmemOut = 128;       // first column of the output tile

struct __align__(1024) UmmaShared {
  unsigned char q[2][kUmmaRows * 128];                   // [half][row][64 dims], 128-byte swizzle
  unsigned char k[kUmmaStages][2][kUmmaKeys * 128];      // [half][key][64 dims]
  unsigned char v[kUmmaStages][2][kUmmaKeys * 128];      // [half][key][64 dims]
  unsigned long long full_k[kUmmaStages], full_v[kUmmaStages];
  unsigned long long s_ready[2], p_ready[2], pv_done[2];
  uint32_t tmem_base;
};

// Shared-memory matrix descriptor, 128-byte swizzle: start address, leading and stride byte
// offsets in 16-byte units, descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t leading_bytes, uint32_t stride_bytes) {
  return static_cast<uint64_t>((saddr >> 4) & 0x3fffu) | (static_cast<uint64_t>((leading_bytes >> 4) & 0x3fffu) << 16) |
         (static_cast<uint64_t>((stride_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (2ull << 61);
}
// D[tmem] (+)= A[smem] * B[smem], one elected thread.
__device__ __forceinline__ void umma_issue(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
               "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_store32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
               "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                 "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                 "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                 "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
               : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem]: A as packed 16-bit pairs, one row per lane.
__device__ __forceinline__ void umma_issue_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
               ::"r"(tmem_d), "r"(tmem_a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}

template <bool kBF16>
__global__ void __launch_bounds__(kUmmaThreads, 2)
prefill_umma_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                    AttentionArgs a, const PrefillHeader* header, const PrefillTile* tiles, unsigned* error,
                    float scale_log2) {
  using T = typename std::conditional<kBF16, __nv_bfloat16, __half>::type;
  if (blockIdx.x >= header->tiles) return;
  extern __shared__ unsigned char smem_raw[];
  UmmaShared& sm = *reinterpret_cast<UmmaShared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, row = threadIdx.x & (kUmmaRows - 1);
  const bool issuer = warp == 4;
  const PrefillTile tile = tiles[blockIdx.x];
  const int q_head = blockIdx.y, kv_head = q_head / (a.q_heads / a.kv_heads);
  const int seq_first = a.cu_seqlens_q[tile.seq];
  const int n_new = a.cu_seqlens_q[tile.seq + 1] - seq_first;
  const int base_len = min(a.context_lengths[tile.seq], a.table_width * kPage) - n_new + 1;
  const int len = (!issuer && row < tile.count) ? max(base_len + tile.first + row, 0) : 0;   // keys this thread's row sees
  const int kv_end = max(base_len + tile.first + tile.count - 1, 0);
  const int total_pages = (kv_end + kPage - 1) / kPage;
  const int kv_tiles = (total_pages + 3) / 4;
  const int64_t q_offset = ((static_cast<int64_t>(seq_first) + tile.first + row) * a.q_heads + q_head) * kHeadDim;

  // ---- prologue: barriers, tensor memory, Q into its swizzled halves, V stages zeroed (a partial
  // last stage multiplies P = 0 with whatever lies behind its last page: that must be finite) ----
  if (threadIdx.x == 0) {
    for (int s = 0; s < kUmmaStages; ++s) {
      mbar_init(smem_u32(&sm.full_k[s]), 1);
      mbar_init(smem_u32(&sm.full_v[s]), 1);
      mbar_init(smem_u32(&sm.s_ready[s]), 1);
      mbar_init(smem_u32(&sm.p_ready[s]), kUmmaRows);
      mbar_init(smem_u32(&sm.pv_done[s]), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (issuer) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(kTmemColumns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  {
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    uint4* vz = reinterpret_cast<uint4*>(&sm.v[0][0][0]);
    for (int i = threadIdx.x; i < static_cast<int>(sizeof(sm.v) / 16); i += kUmmaThreads) vz[i] = zero;
    if (!issuer) {
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const T*>(a.q) + q_offset);
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const uint4 value = len > 0 ? __ldg(src + c) : zero;
        *reinterpret_cast<uint4*>(&sm.q[c >> 3][row * 128 + (((c & 7) ^ (row & 7)) << 4)]) = value;
      }
    }
  }
  fence_async_proxy();
  tcgen05_before_sync();
  __syncthreads();
  tcgen05_after_sync();
  const uint32_t tmem = sm.tmem_base;
  constexpr uint32_t kFormat = kBF16 ? 1u : 0u;
  constexpr uint32_t kIdesc = (1u << 4) | (kFormat << 7) | (kFormat << 10) | (static_cast<uint32_t>(kUmmaRows >> 4) << 24);
  constexpr uint32_t kIdescQK = kIdesc | (static_cast<uint32_t>(kUmmaKeys >> 3) << 17);            // N = 64 keys
  constexpr uint32_t kIdescPV = kIdesc | (static_cast<uint32_t>(kHeadDim >> 3) << 17) | (1u << 16);  // N = 128 dims, B MN-major
  bool failed = false;

  if (issuer) {
    const uint64_t policy = policy_evict_first();
    const int32_t* table = a.block_tables + static_cast<int64_t>(tile.seq) * a.table_width;
    // the eight 2 KiB copies of one operand of key tile jt (4 pages x low / high half), one per lane
    auto issue_copies = [&](int jt, bool keys) {
      const int stage = jt % kUmmaStages;
      const int pages = min(4, total_pages - jt * 4);
      const uint32_t bar = smem_u32(keys ? &sm.full_k[stage] : &sm.full_v[stage]);
      if (lane == 0) mbar_expect_tx(bar, pages * kTileBytes);
      __syncwarp();
      const int page = lane >> 1, half = lane & 1;
      if (lane < 8 && page < pages) {
        unsigned char* dst = (keys ? &sm.k[stage][half][0] : &sm.v[stage][half][0]) + page * 2048;
        tma_load_page_half(smem_u32(dst), keys ? &k_map : &v_map, kv_head * kHeadDim + half * 64, table[jt * 4 + page], bar, policy);
      }
    };
    // lane 0: S(jt) = Q K(jt)^T over the 128 dims in eight K = 16 steps, into score buffer jt & 1
    auto issue_qk = [&](int jt) {
      const int stage = jt % kUmmaStages;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t da = umma_desc(smem_u32(&sm.q[ks >> 2][0]) + (ks & 3) * 32, 16, 1024);
        const uint64_t db = umma_desc(smem_u32(&sm.k[stage][ks >> 2][0]) + (ks & 3) * 32, 16, 1024);
        umma_issue(tmem + (jt & 1) * kUmmaKeys, da, db, kIdescQK, ks > 0);
      }
      umma_commit(smem_u32(&sm.s_ready[jt & 1]));
    };
    // lane 0 waits, the warp learns the outcome
    auto warp_wait = [&](unsigned long long* bar, int parity) {
      bool ok = true;
      if (lane == 0) ok = mbar_wait(smem_u32(bar), parity);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) failed = true;
      return ok;
    };
    for (int jt = 0; jt < min(kUmmaStages, kv_tiles); ++jt) { issue_copies(jt, true); issue_copies(jt, false); }
    for (int jt = 0; jt < min(2, kv_tiles) && !failed; ++jt) {
      if (!warp_wait(&sm.full_k[jt], 0)) break;
      if (lane == 0) { tcgen05_after_sync(); issue_qk(jt); }
    }
    for (int jt = 0; jt < kv_tiles && !failed; ++jt) {
      const int b = jt & 1, phase = (jt >> 1) & 1;
      if (jt + 2 < kv_tiles) {           // S(jt) is complete: its K stage takes key tile jt + 2
        if (!warp_wait(&sm.s_ready[b], phase)) break;
        issue_copies(jt + 2, true);
      }
      if (jt >= 1 && jt + 1 < kv_tiles) {   // P(jt - 1) V(jt - 1) is complete: its V stage takes key tile jt + 1
        if (!warp_wait(&sm.pv_done[b ^ 1], ((jt - 1) >> 1) & 1)) break;
        issue_copies(jt + 1, false);
      }
      if (!warp_wait(&sm.p_ready[b], phase)) break;
      if (!warp_wait(&sm.full_v[b], phase)) break;
      if (jt == kv_tiles - 1 && kv_end < jt * kUmmaKeys + min(4, total_pages - jt * 4) * kPage)   // slots behind the last visible key
        zero_rows_warp(&sm.v[b][0][0], &sm.v[b][1][0], kv_end - jt * kUmmaKeys, min(4, total_pages - jt * 4) * kPage, lane);
      if (lane == 0) {
        tcgen05_after_sync();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {   // O += P V over the 64 keys in four K = 16 steps
          const uint64_t db = umma_desc(smem_u32(&sm.v[b][0][0]) + ks * 2048, 8192, 1024);
          umma_issue_ts(tmem + kTmemOut, tmem + b * kUmmaKeys + ks * 8, db, kIdescPV, (jt > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&sm.pv_done[b]));
      }
      if (jt + 2 < kv_tiles) {           // the scores of key tile jt + 2 follow into the buffer P(jt) was read from
        if (!warp_wait(&sm.full_k[b], ((jt + 2) >> 1) & 1)) break;
        if (lane == 0) { tcgen05_after_sync(); issue_qk(jt + 2); }
      }
    }
  } else {
    const uint32_t tmem_row = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    // The output tile stays in tensor memory.  A row's running maximum m is raised — and its TMEM
    // row rescaled by 2^(m_old - m_new) — only when the stage's maximum exceeds it by more than 8
    // (log2 units): until then P is taken against the old m (values up to 2^8, exact in the fp32
    // sums), and l follows the same m.
    constexpr float kRaise = 8.0f;
    float m = -INFINITY, l = 0.f;
    for (int jt = 0; jt < kv_tiles; ++jt) {
      const int b = jt & 1, phase = (jt >> 1) & 1;
      if (!mbar_wait(smem_u32(&sm.s_ready[b]), phase)) { failed = true; break; }
      tcgen05_after_sync();
      float s[kUmmaKeys];
      {
        uint32_t r0[32], r1[32];
        tmem_load32(tmem_row + b * kUmmaKeys, r0);
        tmem_load32(tmem_row + b * kUmmaKeys + 32, r1);
        tmem_load_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) { s[j] = __uint_as_float(r0[j]); s[32 + j] = __uint_as_float(r1[j]); }
      }
      const int first_key = jt * kUmmaKeys;
      if (first_key + kUmmaKeys > len) {
#pragma unroll
        for (int j = 0; j < kUmmaKeys; ++j)
          if (first_key + j >= len) s[j] = -INFINITY;
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < kUmmaKeys; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], s[j]);
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float candidate = mx * scale_log2;
      const bool raise = candidate > m + kRaise || (m == -INFINITY && candidate > -INFINITY);
      const float alpha = (raise && m != -INFINITY) ? fast_exp2(m - candidate) : 1.0f;
      if (raise) m = candidate;
      const float mu = m == -INFINITY ? 0.f : m;
      if (jt > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {   // rescale this warp's 32 output rows in place
        if (!mbar_wait(smem_u32(&sm.pv_done[b ^ 1]), ((jt - 1) >> 1) & 1)) { failed = true; break; }
        tcgen05_after_sync();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_load32(tmem_row + kTmemOut + c * 32, r);
          tmem_load_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
          tmem_store32(tmem_row + kTmemOut + c * 32, r);
        }
      }
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t packed[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const float p0 = fast_exp2(fmaf(s[2 * e], scale_log2, -mu));
        const float p1 = fast_exp2(fmaf(s[2 * e + 1], scale_log2, -mu));
        sum4[e & 3] += p0 + p1;
        packed[e] = pack2<kBF16>(p0, p1);
      }
      l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      tmem_store32(tmem_row + b * kUmmaKeys, packed);   // P(jt) over the first half of S(jt)
      tmem_store_wait();
      tcgen05_before_sync();
      mbar_arrive(smem_u32(&sm.p_ready[b]));
    }
    if (!failed && kv_tiles > 0 && !mbar_wait(smem_u32(&sm.pv_done[(kv_tiles - 1) & 1]), ((kv_tiles - 1) >> 1) & 1)) failed = true;
    tcgen05_after_sync();
    failed = __any_sync(0xffffffffu, failed);
    if (!failed) {
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      uint4* dst = reinterpret_cast<uint4*>(static_cast<T*>(a.out) + q_offset);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        if (kv_tiles > 0) {
          tmem_load32(tmem_row + kTmemOut + c * 32, r);
          tmem_load_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (row < tile.count) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const float* f = reinterpret_cast<const float*>(&r[q4 * 8]);
            dst[c * 4 + q4] = make_uint4(pack2<kBF16>(f[0] * inv, f[1] * inv), pack2<kBF16>(f[2] * inv, f[3] * inv),
                                         pack2<kBF16>(f[4] * inv, f[5] * inv), pack2<kBF16>(f[6] * inv, f[7] * inv));
          }
        }
      }
    }
  }
  if (failed && lane == 0) atomicOr(error, 1u);
  tcgen05_before_sync();
  __syncthreads();
  if (issuer) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemColumns) : "memory");
}

// Packed fp32 pairs and the three-input maximum of sm_100: half the instructions for the scaling,
// the sums and the row maximum of the softmax, whose warps are bound by issue slots and latency.
__device__ __forceinline__ float2 fma_pair(float2 a, float2 b, float2 c) {
  unsigned long long ra, rb, rc, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
__device__ __forceinline__ float2 add_pair(float2 a, float2 b) {
  unsigned long long ra, rb, rd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Non-blocking probe of a barrier phase (try_wait may suspend the thread for a while).
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}

// ---- two query tiles per CTA: K / V stages shared, A operands in tensor memory -----------------
// 256 query tokens of one query head per CTA (one CTA per SM, all 512 TMEM columns), ten warps:
//   warps 0..3 / 4..7  the softmax rows of query tile 0 / 1 (row = TMEM lane),
//   warps 8, 9         issue the Q K^T MMAs of tile 0 / 1 (the warp runs the loop, an elected lane issues),
//   warps 10, 11       issue the P V MMAs of tile 0 / 1,
//   warp 12            the TMA copies, kPairStages stages of 64 keys ahead.
// Per tile the scores S (64 columns) and the probabilities P (32 columns of packed 16-bit pairs)
// have separate TMEM columns, so S(j + 1) = Q K(j + 1)^T is issued as soon as the rows have read
// S(j) into registers, runs under their softmax, and O += P(j) V(j) follows when P(j) is stored:
// in steady state neither the rows nor the tensor cores wait for each other.  P is always a TMEM
// operand; Q of tile 0 is one too (each thread stores its row with tcgen05.st), Q of tile 1 sits in
// shared memory (the 512 columns are used up).  Every copied stage serves both tiles.
// TMEM columns: Q0 0..63 | S0 64..127, P0 128..159 | S1 160..223, P1 224..255 | O0 256..383 | O1 384..511.
constexpr int kPairRows = 2 * kUmmaRows;
constexpr int kPairThreads = 416;
constexpr int kPairStages = 5;
constexpr uint32_t kPairTmemColumns = 512;

struct __align__(1024) PairShared {
  unsigned char q[2][kUmmaRows * 128];                   // tile 1: [half][row][64 dims], 128-byte swizzle
  unsigned char k[kPairStages][2][kUmmaKeys * 128];      // [half][key][64 dims]
  unsigned char v[kPairStages][2][kUmmaKeys * 128];
  unsigned char rows[2 * kUmmaRows / 32][32 * 128];      // per softmax warp: its 32 rows, 64 columns of 16 bits, 16-byte pieces swizzled
  unsigned long long full_k[kPairStages], full_v[kPairStages], free_k[kPairStages], free_v[kPairStages];
  unsigned long long s_ready[2], s_free[2], p_ready[2], pv_done[2];
  unsigned long long turn[kUmmaRows / 32][2];            // [scheduler][tile]: the other tile's warp has left its exponentials
  uint32_t tmem_base;
};

__device__ __forceinline__ bool elect_one() {
  uint32_t leader;
  asm volatile("{\n.reg .pred e;\nelect.sync _|e, 0xffffffff;\nselp.u32 %0, 1, 0, e;\n}\n" : "=r"(leader));
  return leader != 0;
}

constexpr uint32_t kColQ = 0, kColS = 64, kTileCols = 96, kColP = 64, kColO = 256;   // P: offset inside a tile's S / P block

// The issue loop of one warp: the scores (kScores) or the output product of query tile kTile, `mine` stages
// (`other`: the stages of the other tile).  The whole warp runs the loop, so that the barrier probes, the
// stage arithmetic and the operand descriptors stay warp-uniform; one elected lane issues the MMAs and their
// commits.
//   S(j):  Q announced (first phase of p_ready) for j = 0, else S(j - 1) read (s_free) — and K(j)
//   O(j):  P(j) stored (p_ready) — and V(j)
// The two products of a tile touch different TMEM columns, so their warps need no order between
// them.  A stage is released to the copy warp by the commits of both tiles' warps; for a tile that
// does not read the stage the other tile's warp arrives by hand.  Returns true when a wait gave up.
template <bool kScores, int kTile>
__device__ __forceinline__ bool pair_issue(PairShared& sm, uint32_t tmem, int mine, int other, uint32_t idesc,
                                           int kv_end, int total_pages, int lane) {
  const uint32_t s_col = tmem + kColS + kTile * kTileCols, o_col = tmem + kColO + kTile * kHeadDim;
  // Q announced: from here on p_ready has completed its first phase, so a parity probe of it is unambiguous
  if (mine > 0 && !__all_sync(0xffffffffu, mbar_wait(smem_u32(&sm.p_ready[kTile]), 0))) return true;
  const uint64_t q_desc = umma_desc(smem_u32(&sm.q[0][0]), 16, 1024);
  long long last_progress = clock64();
  unsigned probes = 0;
  int stage = 0;
  uint32_t ring_parity = 0;
  for (int j = 0; j < mine;) {
    bool go;
    if (kScores) go = (j == 0 || mbar_test(smem_u32(&sm.s_free[kTile]), (j - 1) & 1)) && mbar_test(smem_u32(&sm.full_k[stage]), ring_parity);
    else go = mbar_test(smem_u32(&sm.p_ready[kTile]), (j + 1) & 1) && mbar_test(smem_u32(&sm.full_v[stage]), ring_parity);
    if (!__all_sync(0xffffffffu, go)) {
      if ((++probes & 255u) == 0 && clock64() - last_progress > kWaitCycles) return true;
      continue;
    }
    tcgen05_after_sync();
    if (kScores) {   // S(j) = Q K(j)^T over the 128 dims
      const uint64_t k_desc = umma_desc(smem_u32(&sm.k[stage][0][0]), 16, 1024);
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t step = static_cast<uint64_t>(((ks >> 2) * (kUmmaKeys * 128) + (ks & 3) * 32) >> 4);   // address field, 16-byte units
          if (kTile == 0) umma_issue_ts(s_col, tmem + kColQ + ks * 8, k_desc + step, idesc, ks > 0);
          else umma_issue(s_col, q_desc + static_cast<uint64_t>(((ks >> 2) * (kUmmaRows * 128) + (ks & 3) * 32) >> 4), k_desc + step, idesc, ks > 0);
        }
        umma_commit(smem_u32(&sm.s_ready[kTile]));
        umma_commit(smem_u32(&sm.free_k[stage]));
        if (j >= other) mbar_arrive(smem_u32(&sm.free_k[stage]));
      }
    } else {         // O += P(j) V(j) over the 64 keys
      const int rows = min(4, total_pages - j * 4) * kPage;
      if (kv_end - j * kUmmaKeys < rows)   // the last stage: slots behind the last key any row sees (both tiles' warps may clear them)
        zero_rows_warp(&sm.v[stage][0][0], &sm.v[stage][1][0], kv_end - j * kUmmaKeys, rows, lane);
      const uint64_t v_desc = umma_desc(smem_u32(&sm.v[stage][0][0]), 8192, 1024);
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_issue_ts(o_col, s_col + kColP + ks * 8, v_desc + static_cast<uint64_t>((ks * 2048) >> 4), idesc, (j > 0 || ks > 0) ? 1u : 0u);
        umma_commit(smem_u32(&sm.pv_done[kTile]));
        umma_commit(smem_u32(&sm.free_v[stage]));
        if (j >= other) mbar_arrive(smem_u32(&sm.free_v[stage]));
      }
    }
    __syncwarp();
    ++j;
    if (++stage == kPairStages) { stage = 0; ring_parity ^= 1u; }
    last_progress = clock64();
    probes = 0;
  }
  return false;
}

template <bool kBF16>
__global__ void __launch_bounds__(kPairThreads, 1)
prefill_pair_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                    AttentionArgs a, const PrefillHeader* header, const PrefillTile* tiles, unsigned* error,
                    float scale_log2, int take_turns) {
  using T = typename std::conditional<kBF16, __nv_bfloat16, __half>::type;
  if (blockIdx.x >= header->tiles) return;
  extern __shared__ unsigned char smem_raw[];
  PairShared& sm = *reinterpret_cast<PairShared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int lane = threadIdx.x & 31, warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);   // warp-uniform for the compiler too
  const PrefillTile tile = tiles[blockIdx.x];   // everything the CTA needs to know about its rows: one load
  const int q_head = blockIdx.y, kv_head = q_head / (a.q_heads / a.kv_heads);
  const int seq_first = tile.q_row - tile.first;
  const int base_len = tile.visible - tile.first;
  // key stages of the two query tiles: tile 1 (the later rows) sees every stage tile 0 does
  const int count0 = min(tile.count, kUmmaRows), count1 = max(tile.count - kUmmaRows, 0);
  const int stages0 = (max(base_len + tile.first + count0 - 1, 0) + kUmmaKeys - 1) / kUmmaKeys;
  const int stages1 = count1 > 0 ? (max(base_len + tile.first + kUmmaRows + count1 - 1, 0) + kUmmaKeys - 1) / kUmmaKeys : 0;
  const int all_stages = max(stages0, stages1);
  const int total_pages = (max(base_len + tile.first + tile.count - 1, 0) + kPage - 1) / kPage;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(smem_u32(&sm.full_k[s]), 1);
      mbar_init(smem_u32(&sm.full_v[s]), 1);
      mbar_init(smem_u32(&sm.free_k[s]), 2);   // one arrival per query tile
      mbar_init(smem_u32(&sm.free_v[s]), 2);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(smem_u32(&sm.s_ready[t]), 1);
      mbar_init(smem_u32(&sm.s_free[t]), kUmmaRows / 32);    // one arrival per softmax warp
      mbar_init(smem_u32(&sm.p_ready[t]), kUmmaRows / 32);
      mbar_init(smem_u32(&sm.pv_done[t]), 1);
      for (int w = 0; w < kUmmaRows / 32; ++w) mbar_init(smem_u32(&sm.turn[w][t]), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(kPairTmemColumns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // A partial last stage multiplies P = 0 with what lies behind its last page of V: that has to be
  // finite.  Once the ring has wrapped it is an earlier stage's data; before that it is whatever
  // the shared memory held, so the tail of that one stage is zeroed.
  if (all_stages > 0 && all_stages <= kPairStages) {
    const int pages_last = total_pages - (all_stages - 1) * 4;   // 1 .. 4
    const int tail = (4 - pages_last) * 2048 / 16;               // 16-byte words per half
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int i = threadIdx.x; i < 2 * tail; i += kPairThreads) {
      const int half = i / tail, word = i - half * tail;
      reinterpret_cast<uint4*>(&sm.v[all_stages - 1][half][pages_last * 2048])[word] = zero;
    }
  }
  fence_async_proxy();
  tcgen05_before_sync();
  __syncthreads();
  tcgen05_after_sync();
  const uint32_t tmem = sm.tmem_base;
  constexpr uint32_t kFormat = kBF16 ? 1u : 0u;
  constexpr uint32_t kIdesc = (1u << 4) | (kFormat << 7) | (kFormat << 10) | (static_cast<uint32_t>(kUmmaRows >> 4) << 24);
  constexpr uint32_t kIdescQK = kIdesc | (static_cast<uint32_t>(kUmmaKeys >> 3) << 17);            // N = 64 keys
  constexpr uint32_t kIdescPV = kIdesc | (static_cast<uint32_t>(kHeadDim >> 3) << 17) | (1u << 16);  // N = 128 dims, B MN-major
  bool failed = false;

  if (warp == 12) {
    // ---- copies: stage j takes key tile j once both of its operands' readers have committed ----
    const uint64_t policy = policy_evict_first();
    const int32_t* table = a.block_tables + static_cast<int64_t>(tile.seq) * a.table_width;
    for (int j = 0; j < all_stages && !failed; ++j) {
      const int stage = j % kPairStages, use = j / kPairStages;
      const int pages = min(4, total_pages - j * 4);
      const int page = (lane & 7) >> 1, half = lane & 1;
      const int block = (lane < 8 && page < pages) ? table[j * 4 + page] : 0;
#pragma unroll
      for (int operand = 0; operand < 2; ++operand) {
        bool ok = true;
        if (lane == 0 && use > 0) ok = mbar_wait(smem_u32(operand == 0 ? &sm.free_k[stage] : &sm.free_v[stage]), (use - 1) & 1);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) { failed = true; break; }
        const uint32_t bar = smem_u32(operand == 0 ? &sm.full_k[stage] : &sm.full_v[stage]);
        if (lane == 0) mbar_expect_tx(bar, pages * kTileBytes);
        __syncwarp();
        if (lane < 8 && page < pages) {
          unsigned char* dst = (operand == 0 ? &sm.k[stage][half][0] : &sm.v[stage][half][0]) + page * 2048;
          tma_load_page_half(smem_u32(dst), operand == 0 ? &k_map : &v_map, kv_head * kHeadDim + half * 64, block, bar, policy);
        }
      }
    }
  } else if (warp >= 8) {
    // ---- MMA issue: one warp per query tile and product ----
    const int kv_end = max(base_len + tile.first + tile.count - 1, 0);   // keys the pair's last row sees
    if (warp == 8) failed = pair_issue<true, 0>(sm, tmem, stages0, stages1, kIdescQK, kv_end, total_pages, lane);
    else if (warp == 9) failed = pair_issue<true, 1>(sm, tmem, stages1, stages0, kIdescQK, kv_end, total_pages, lane);
    else if (warp == 10) failed = pair_issue<false, 0>(sm, tmem, stages0, stages1, kIdescPV, kv_end, total_pages, lane);
    else failed = pair_issue<false, 1>(sm, tmem, stages1, stages0, kIdescPV, kv_end, total_pages, lane);
  } else {
    // ---- softmax rows ----
    const int t = warp >> 2, row = threadIdx.x & (kUmmaRows - 1);
    const int count = t == 0 ? count0 : count1;
    const int len = row < count ? max(base_len + tile.first + t * kUmmaRows + row, 0) : 0;
    const int my_stages = t == 0 ? stages0 : stages1;
    const uint32_t tmem_row = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    // This warp's 32 rows of the query and of the output are read and written as 128-byte pieces by eight lanes
    // each (a thread that moved its own 256-byte row would touch 32 lines per instruction, and the eight warps
    // together would keep the load / store unit busy for thousands of cycles); a thread's own row goes through the
    // warp's staging rows in shared memory, whose 16-byte pieces are swizzled by the row.
    const int warp_row = (warp & 3) * 32, warp_count = min(max(count - warp_row, 0), 32);
    const int64_t row_stride = static_cast<int64_t>(a.q_heads) * kHeadDim;
    const int64_t warp_offset = ((static_cast<int64_t>(seq_first) + tile.first + t * kUmmaRows + warp_row) * a.q_heads + q_head) * kHeadDim;
    unsigned char* staging = &sm.rows[warp][0];
    if (my_stages > 0) {   // Q: tile 0 into tensor memory (two 16-bit values per column, a thread stores its row), tile 1 into shared memory
      const T* src = static_cast<const T*>(a.q) + warp_offset;
      const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
      if (t == 0) {
        uint4 piece[2][8];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = 4 * i + (lane >> 3);
            piece[h][i] = r < warp_count ? __ldg(reinterpret_cast<const uint4*>(src + r * row_stride + h * 64) + (lane & 7)) : zero;
          }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = 4 * i + (lane >> 3);
            *reinterpret_cast<uint4*>(staging + r * 128 + (((lane & 7) ^ (r & 7)) << 4)) = piece[h][i];
          }
          __syncwarp();
          uint32_t q[32];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 value = *reinterpret_cast<const uint4*>(staging + lane * 128 + ((c ^ (lane & 7)) << 4));
            q[c * 4] = value.x; q[c * 4 + 1] = value.y; q[c * 4 + 2] = value.z; q[c * 4 + 3] = value.w;
          }
          tmem_store32(tmem_row + kColQ + h * 32, q);
          __syncwarp();
        }
        tmem_store_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int r = 2 * i + (lane >> 4), c = lane & 15;
          const uint4 value = r < warp_count ? __ldg(reinterpret_cast<const uint4*>(src + r * row_stride) + c) : zero;
          *reinterpret_cast<uint4*>(&sm.q[c >> 3][(warp_row + r) * 128 + (((c & 7) ^ (r & 7)) << 4)]) = value;
        }
        fence_async_proxy();
      }
      tcgen05_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm.p_ready[t]));
    }
    constexpr float kRaise = 8.0f;
    const bool alternate = take_turns != 0 && stages0 > 0 && stages1 > 0;
    float m = -INFINITY, l = 0.f;
    const uint32_t s_col = tmem_row + kColS + t * kTileCols, p_col = s_col + kColP, o_col = tmem_row + kColO + t * kHeadDim;
    for (int j = 0; j < my_stages; ++j) {
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sm.s_ready[t]), j & 1))) { failed = true; break; }   // warp-uniform exit
      tcgen05_after_sync();
      float s[kUmmaKeys];
      {
        uint32_t r0[32], r1[32];
        tmem_load32(s_col, r0);
        tmem_load32(s_col + 32, r1);
        tmem_load_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) { s[i] = __uint_as_float(r0[i]); s[32 + i] = __uint_as_float(r1[i]); }
      }
      tcgen05_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm.s_free[t]));   // the scores are in registers: the next stage's may be written
      const int first_key = j * kUmmaKeys;
      if (first_key + kUmmaKeys > len) {
#pragma unroll
        for (int i = 0; i < kUmmaKeys; ++i)
          if (first_key + i >= len) s[i] = -INFINITY;
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < kUmmaKeys; i += 8) {
#pragma unroll
        for (int c = 0; c < 4; ++c) mx4[c] = max3(mx4[c], s[i + 2 * c], s[i + 2 * c + 1]);
      }
      const float candidate = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
      const bool raise = candidate > m + kRaise || (m == -INFINITY && candidate > -INFINITY);
      const float alpha = (raise && m != -INFINITY) ? fast_exp2(m - candidate) : 1.0f;
      if (raise) m = candidate;
      const float mu = m == -INFINITY ? 0.f : m;
      float2 sum4[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
      uint32_t packed[32];
      const float2 scale2 = make_float2(scale_log2, scale_log2), shift2 = make_float2(-mu, -mu);
      // On long prompts the two tiles' warps of one scheduler take turns at its exponential unit (tile 0 first
      // in every stage): left alone they fall into step, and one warp's loads, maxima and stores then no
      // longer run under the other's exponentials.
      if (alternate) {
        const bool wait = t == 0 ? j > 0 : j < stages0;
        if (wait && !__all_sync(0xffffffffu, mbar_wait(smem_u32(&sm.turn[warp & 3][t]), (t == 0 ? j - 1 : j) & 1))) { failed = true; break; }
      }
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const float2 x = fma_pair(make_float2(s[2 * e], s[2 * e + 1]), scale2, shift2);
        const float2 p = make_float2(fast_exp2(x.x), fast_exp2(x.y));
        sum4[e & 3] = add_pair(sum4[e & 3], p);
        packed[e] = pack2<kBF16>(p.x, p.y);
      }
      if (alternate) {
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm.turn[warp & 3][t ^ 1]));
      }
      const float2 sum2 = add_pair(add_pair(sum4[0], sum4[1]), add_pair(sum4[2], sum4[3]));
      l = l * alpha + (sum2.x + sum2.y);
      if (j > 0) {   // P(j - 1) has been read and the output tile is at rest once the previous product is complete
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sm.pv_done[t]), (j - 1) & 1))) { failed = true; break; }
        tcgen05_after_sync();
        if (__any_sync(0xffffffffu, alpha != 1.0f)) {   // rescale this warp's 32 output rows in place
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_load32(o_col + c * 32, r);
            tmem_load_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_store32(o_col + c * 32, r);
          }
        }
      }
      tmem_store32(p_col, packed);
      tmem_store_wait();
      tcgen05_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm.p_ready[t]));
    }
    if (!failed && my_stages > 0 && !mbar_wait(smem_u32(&sm.pv_done[t]), (my_stages - 1) & 1)) failed = true;
    tcgen05_after_sync();
    failed = __any_sync(0xffffffffu, failed);
    if (!failed && count > 0) {
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      T* dst = static_cast<T*>(a.out) + warp_offset;
#pragma unroll
      for (int h = 0; h < 2; ++h) {   // 64 output columns at a time
        uint32_t lo[32], hi[32];
        if (my_stages > 0) {
          tmem_load32(o_col + h * 64, lo);
          tmem_load32(o_col + h * 64 + 32, hi);
          tmem_load_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) lo[i] = hi[i] = 0u;
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const float* f = reinterpret_cast<const float*>(c < 4 ? &lo[c * 8] : &hi[(c - 4) * 8]);
          *reinterpret_cast<uint4*>(staging + lane * 128 + ((c ^ (lane & 7)) << 4)) =
              make_uint4(pack2<kBF16>(f[0] * inv, f[1] * inv), pack2<kBF16>(f[2] * inv, f[3] * inv),
                         pack2<kBF16>(f[4] * inv, f[5] * inv), pack2<kBF16>(f[6] * inv, f[7] * inv));
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = 4 * i + (lane >> 3);
          if (r < warp_count)
            reinterpret_cast<uint4*>(dst + r * row_stride + h * 64)[lane & 7] =
                *reinterpret_cast<const uint4*>(staging + r * 128 + (((lane & 7) ^ (r & 7)) << 4));
        }
        __syncwarp();
      }
    }
  }
  if (failed && lane == 0) atomicOr(error, 1u);
  tcgen05_before_sync();
  __syncthreads();
  if (warp == 8) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kPairTmemColumns) : "memory");
}

size_t tile_capacity(int rows, int seqs) { return static_cast<size_t>(rows) / kTileRows + static_cast<size_t>(seqs) + 1; }

}  // namespace

bool prefill_sm100_supported(const AttentionArgs& a) {
  return a.cu_seqlens_q != nullptr && attention_sm100_supported(a);
}

size_t prefill_sm100_workspace_bytes(int rows, int seqs) {
  return 256 + sizeof(PrefillTile) * tile_capacity(rows, seqs);
}

// The tcgen05 kernels by default; RLT_PREFILL_KERNEL=pair|umma|mma forces one of the three.
// RLT_ERR_UNSUPPORTED when no tiled prefill kernel can address the caches (the caller then scores
// the rows with the verify kernel).
int launch_prefill_sm100(const AttentionArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  if (workspace == nullptr || workspace_bytes < prefill_sm100_workspace_bytes(a.rows, a.table_rows) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) {
    set_last_error_text("prefill_attention: workspace missing, misaligned or too small");
    return RLT_ERR_WORKSPACE;
  }
  // 'p'air, 'u'mma (one tile per CTA) or 'm'ma.sync; unset: the pair kernel.  It is the fastest of the three also
  // where its second tile stays empty (chunks of 128 new tokens per sequence: 48 against 66 and 80 us at 16 sequences
  // on 1024-token contexts, 70 against 138 and 147 us at 4 sequences on 4096-token ones).
  const char* forced = getenv("RLT_PREFILL_KERNEL");
  const char kernel_choice = forced != nullptr && forced[0] != 0 ? forced[0] : 'p';
  const bool use_mma_sync = kernel_choice == 'm';
  PrefillHeader* header = static_cast<PrefillHeader*>(workspace);
  PrefillTile* tiles = reinterpret_cast<PrefillTile*>(static_cast<unsigned char*>(workspace) + 256);
  const float scale_log2 = static_cast<float>(1.4426950408889634 / sqrt(static_cast<double>(kHeadDim)));
  CUtensorMap k_map, v_map;
  if (kernel_choice == 'p' && make_page_map(&k_map, a.key_cache, a) == RLT_OK && make_page_map(&v_map, a.value_cache, a) == RLT_OK) {
    prefill_plan_kernel<<<1, kPrefillPlanThreads, 0, stream>>>(a.cu_seqlens_q, a.context_lengths, a.table_width, a.table_rows, kPairRows, header, tiles);
    int status = launch_status("prefill_plan_kernel");
    if (status != RLT_OK) return status;
    const size_t smem = sizeof(PairShared) + 1024;
    const int take_turns = static_cast<int64_t>(a.rows) >= 2048ll * a.table_rows ? 1 : 0;   // prompts of 2048 tokens and more on average
    const dim3 grid(static_cast<unsigned>(static_cast<size_t>(a.rows) / kPairRows + static_cast<size_t>(a.table_rows) + 1),
                    static_cast<unsigned>(a.q_heads));
    if (a.dtype == RLT_BF16) {
      auto kernel = prefill_pair_kernel<true>;
      RLT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
      kernel<<<grid, kPairThreads, smem, stream>>>(k_map, v_map, a, header, tiles, &header->error, scale_log2, take_turns);
    } else {
      auto kernel = prefill_pair_kernel<false>;
      RLT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
      kernel<<<grid, kPairThreads, smem, stream>>>(k_map, v_map, a, header, tiles, &header->error, scale_log2, take_turns);
    }
    return launch_status("prefill_pair_kernel");
  }
  if (!use_mma_sync && make_page_map(&k_map, a.key_cache, a) == RLT_OK && make_page_map(&v_map, a.value_cache, a) == RLT_OK) {
    prefill_plan_kernel<<<1, kPrefillPlanThreads, 0, stream>>>(a.cu_seqlens_q, a.context_lengths, a.table_width, a.table_rows, kUmmaRows, header, tiles);
    int status = launch_status("prefill_plan_kernel");
    if (status != RLT_OK) return status;
    const size_t smem = sizeof(UmmaShared) + 1024;
    const dim3 grid(static_cast<unsigned>(tile_capacity(a.rows, a.table_rows)), static_cast<unsigned>(a.q_heads));
    if (a.dtype == RLT_BF16) {
      auto kernel = prefill_umma_kernel<true>;
      RLT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
      kernel<<<grid, kUmmaThreads, smem, stream>>>(k_map, v_map, a, header, tiles, &header->error, scale_log2);
    } else {
      auto kernel = prefill_umma_kernel<false>;
      RLT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
      kernel<<<grid, kUmmaThreads, smem, stream>>>(k_map, v_map, a, header, tiles, &header->error, scale_log2);
    }
    return launch_status("prefill_umma_kernel");
  }
  CUtensorMap kv_map;
  bool k_first = true;
  if (make_joint_map(&kv_map, a, &k_first) != RLT_OK) return RLT_ERR_UNSUPPORTED;
  prefill_plan_kernel<<<1, kPrefillPlanThreads, 0, stream>>>(a.cu_seqlens_q, a.context_lengths, a.table_width, a.table_rows, kTileRows, header, tiles);
  int status = launch_status("prefill_plan_kernel");
  if (status != RLT_OK) return status;
  const size_t smem = sizeof(PrefillShared) + 1024;
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
