// Verify attention for sm_100a: head_dim 128, 16-token pages, fp16 / bf16.
//
// Data flow
//   plan kernel   one warp per query row finds the rows that share a block-table row (the k+1
//                 rows of one request at one depth plane; k x depths rows in a shared-plane
//                 layout) and zero-fills empty rows; the last CTA to finish turns the groups
//                 into a work list of (group, context chunk, kv head) items, full-size chunks
//                 first and then the ragged last chunk of every group, longest first.
//   main kernel   persistent, one CTA per SM, every warp an independent worker.  A warp claims
//                 an item and streams that head's K/V pages through its own ring of shared
//                 memory stages with TMA (cp.async.bulk.tensor, 128-byte swizzle, page id =
//                 TMA block coordinate), always kStages-1 pages ahead of the page it is
//                 scoring, across item boundaries.  Each page is scored for up to 16 query
//                 rows at once on tensor cores (m16n8k16; Q in registers, K/V fragments by
//                 ldmatrix) with an fp32 online softmax, so a page is read from HBM once per
//                 group instead of once per row.  A row whose context fits one chunk is
//                 finished from registers; otherwise the warp stores an fp32 partial.
//   merge kernel  one warp per (row, query head) whose context spans more than one chunk folds
//                 that row's partials in chunk order.  The kernel boundary is the only ordering
//                 between the partial stores and their readers: a device-scope fence inside the
//                 streaming kernel waits for the warp's pages in flight, a full memory latency
//                 per work item, which costs more than this launch.
//
// The main kernel has no cross-warp reduction, no CTA-wide barrier after start-up and no
// atomics besides the work-item claim; its only synchronisation is each warp's mbarrier ring.
//
// Batch invariance: chunk boundaries and the merge order are functions of absolute token
// positions only, and a tensor-core output row depends only on its own input row, so a row's
// bits do not depend on its group or batch.
//
// HBM traffic per call = each group's K/V once + Q + O (+ fp32 partials for contexts of more
// than one chunk), which is what the roofline of this kernel is measured against.
#include <cuda.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include <mutex>
#include <type_traits>

#include "attention.cuh"
#include "sm100_primitives.cuh"

namespace rlt {
namespace {

constexpr int kPartialStride = 132;               // floats per stored partial: O[128], m, l, pad
constexpr int kPlanThreads = 1024;
constexpr int kMaxGroupRows = 16;
constexpr unsigned kErrorWaitGaveUp = 1u, kErrorLengthClamped = 2u;
constexpr int kSizeClasses = 64;                  // list B is bucketed by pages in the last chunk (64 or more share a class)

// ---- context chunks -------------------------------------------------------------------
// Fixed, position-only chunk boundaries: sixteen 512-token chunks up to 8192, then every
// power-of-two octave [8192 * 2^k, 8192 * 2^(k+1)) in four equal chunks.
__host__ __device__ inline int floor_log2(unsigned x) {
#ifdef __CUDA_ARCH__
  return 31 - __clz(x);
#else
  return 31 - __builtin_clz(x);
#endif
}

__host__ __device__ inline int chunk_count(int len) {
  if (len <= 0) return 0;
  if (len <= 8192) return (len + 511) >> 9;
  const int k = floor_log2(static_cast<unsigned>((len - 1) >> 13));
  return 16 + 4 * k + (len - 1 - (8192 << k)) / (2048 << k) + 1;
}

__host__ __device__ inline void chunk_range(int c, int* start, int* end) {
  if (c < 16) {
    *start = c << 9;
    *end = *start + 512;
  } else {
    const int k = (c - 16) >> 2, j = (c - 16) & 3;
    *start = (8192 << k) + j * (2048 << k);
    *end = *start + (2048 << k);
  }
}

// ---- workspace ------------------------------------------------------------------------
struct Header {
  unsigned full_items;   // items of list A (full-size chunks)
  unsigned last_items;   // items of list B (last chunk of every group)
  unsigned next_item;    // claim counter of the main kernel
  unsigned error;        // bit 0: a bounded wait gave up; bit 1: a context length exceeded its table and was clamped
  unsigned plan_done;    // CTAs of the plan kernel that finished phase 1
  unsigned zero_rows;    // rows of length 0 (their output is zero-filled by every run)
  unsigned exited;       // warps of the running main kernel that have finished
};

struct Item {
  int row_start;
  int table_row;
  int nrows_head;  // nrows | kv_head << 16
  int chunk;
};

struct Layout {
  size_t header, row_len, row_table, link, zero_list, items_a, items_b, partials, total;
  int max_chunks;
};

inline size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

Layout make_layout(int rows, int q_heads, int kv_heads, int block_size, int table_width) {
  Layout l;
  const long long max_len = static_cast<long long>(table_width) * block_size;
  l.max_chunks = chunk_count(static_cast<int>(max_len > (1 << 26) ? (1 << 26) : max_len));
  if (l.max_chunks < 1) l.max_chunks = 1;
  size_t off = 0;
  l.header = off; off += 256;
  l.row_len = off; off += align256(sizeof(int) * rows);
  l.row_table = off; off += align256(sizeof(int) * rows);
  l.link = off; off += align256(sizeof(int) * rows);
  l.zero_list = off; off += align256(sizeof(int) * rows);
  l.items_a = off; off += align256(sizeof(Item) * static_cast<size_t>(rows) * kv_heads * (l.max_chunks - 1) + 16);
  l.items_b = off; off += align256(sizeof(Item) * static_cast<size_t>(rows) * kv_heads);
  l.partials = off;
  off += align256(sizeof(float) * kPartialStride * static_cast<size_t>(rows) * q_heads * l.max_chunks);
  l.total = off;
  return l;
}

struct Workspace {
  Header* header;
  int* row_len;
  int* row_table;
  int* link;
  int* zero_list;
  Item* items_a;
  Item* items_b;
  float* partials;
  int max_chunks;
};

// ---- plan kernel ------------------------------------------------------------------------
// Inclusive block scans over kPlanThreads threads (warp shuffles + one shared array).
__device__ __forceinline__ int block_scan_max(int v, int* warp_totals) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int x = 1; x < 32; x <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, v, x);
    if (lane >= x) v = max(v, o);
  }
  __syncthreads();
  if (lane == 31) warp_totals[warp] = v;
  __syncthreads();
  int before = -1;
  for (int w = 0; w < warp; ++w) before = max(before, warp_totals[w]);
  return max(v, before);
}
__device__ __forceinline__ unsigned long long block_scan_sum(unsigned long long v, unsigned long long* warp_totals) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int x = 1; x < 32; x <<= 1) {
    const unsigned long long o = __shfl_up_sync(0xffffffffu, v, x);
    if (lane >= x) v += o;
  }
  __syncthreads();
  if (lane == 31) warp_totals[warp] = v;
  __syncthreads();
  unsigned long long before = 0;
  for (int w = 0; w < warp; ++w) before += warp_totals[w];
  return v + before;
}

// Rows r-1 and r are linked when both are non-empty and their table rows agree on every
// page any of the last `cap` rows can need (that window makes agreement transitive inside
// a group of at most `cap` rows).  Packed input states its groups through cu_seqlens_q.
__global__ void __launch_bounds__(kPlanThreads)
plan_kernel(AttentionArgs a, Workspace ws, int cap) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x * (kPlanThreads / 32) + warp;
  if (row < a.rows) {
    int table_row, len;
    bool clamped = false;
    resolve_row(a, row, &table_row, &len, &clamped);
    if (clamped && lane == 0) atomicOr(&ws.header->error, kErrorLengthClamped);
    int link = 0;
    if (len > 0 && row > 0) {
      int prev_table, prev_len;
      resolve_row(a, row - 1, &prev_table, &prev_len);
      if (prev_len > 0) {
        if (a.cu_seqlens_q != nullptr) {
          link = prev_table == table_row;
        } else {
          const int other = (lane >= 1 && lane < cap && row - lane >= 0) ? a.context_lengths[row - lane] : 0;
          int longest = max(len, other);
#pragma unroll
          for (int x = 16; x > 0; x >>= 1) longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, x));
          const int pages = min((longest + a.block_size - 1) / a.block_size, a.table_width);
          const int32_t* mine = a.block_tables + static_cast<int64_t>(row) * a.table_width;
          const int32_t* prev = mine - a.table_width;
          int same = 1;
          for (int p = lane; p < pages; p += 32) same &= mine[p] == prev[p];
          link = __all_sync(0xffffffffu, same);
        }
      }
    }
    if (lane == 0) {
      if (len <= 0) ws.zero_list[atomicAdd(&ws.header->zero_rows, 1u)] = row;  // empty row: never in a group
      ws.row_len[row] = len > 0 ? len : 0;
      ws.row_table[row] = table_row;
      ws.link[row] = link;
    }
  }

  // The last CTA to get here builds the work lists.
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned done = atomicAdd(&ws.header->plan_done, 1u);
    s_last = done == gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();

  __shared__ int s_link[kPlanThreads + kMaxGroupRows];
  __shared__ int s_len[kPlanThreads + kMaxGroupRows];
  __shared__ int s_imax[32];
  __shared__ unsigned long long s_usum[32];
  __shared__ int s_carry_start;
  __shared__ unsigned s_base_full, s_base_last;
  // List B is ordered longest first (a counting sort of the groups by the pages of their last
  // chunk): the schedule then ends with the smallest items and the warps finish together.
  // Phase 0 counts the groups per size class, phase 1 writes the items.
  __shared__ unsigned s_class[kSizeClasses];
  for (int i = threadIdx.x; i < kSizeClasses; i += kPlanThreads) s_class[i] = 0u;
  for (int phase = 0; phase < 2; ++phase) {
  __syncthreads();
  if (threadIdx.x == 0) {
    s_carry_start = 0; s_base_full = 0; s_base_last = 0;
    if (phase == 1) {  // counts -> first slot of every class, largest class first
      unsigned running = 0;
      for (int c = 0; c < kSizeClasses; ++c) { const unsigned n = s_class[c]; s_class[c] = running; running += n; }
    }
  }
  for (int base = 0; base < a.rows; base += kPlanThreads) {
    __syncthreads();
    for (int i = threadIdx.x; i < kPlanThreads + kMaxGroupRows; i += kPlanThreads) {
      const int r = base + i;
      s_link[i] = r < a.rows ? __ldcg(&ws.link[r]) : 0;
      s_len[i] = r < a.rows ? __ldcg(&ws.row_len[r]) : 0;
    }
    __syncthreads();
    const int r = base + threadIdx.x;
    const bool in = r < a.rows;
    const int len = s_len[threadIdx.x];
    int run_start = block_scan_max((in && !s_link[threadIdx.x]) ? r : -1, s_imax);
    if (run_start < 0) run_start = s_carry_start;
    const bool leader = in && len > 0 && ((r - run_start) % cap == 0);
    int nrows = 0, longest = 0, longest_row = r;
    if (leader) {
      nrows = 1;
      longest = len;
      while (nrows < cap && s_link[threadIdx.x + nrows]) {  // rows beyond a.rows read as unlinked
        const int other = s_len[threadIdx.x + nrows];
        if (other > longest) { longest = other; longest_row = r + nrows; }
        ++nrows;
      }
    }
    const int chunks = leader ? chunk_count(longest) : 0;
    unsigned last_slot = 0;
    if (leader) {
      int last_start, last_end;
      chunk_range(chunks - 1, &last_start, &last_end);
      const int pages = (longest - last_start + kPage - 1) / kPage;
      const int size_class = kSizeClasses - 1 - min(pages - 1, kSizeClasses - 1);
      last_slot = atomicAdd(&s_class[size_class], static_cast<unsigned>(a.kv_heads));  // phase 0: count; phase 1: slot
    }
    const unsigned long long mine = leader ? ((static_cast<unsigned long long>(a.kv_heads) << 32) |
                                              static_cast<unsigned>((chunks - 1) * a.kv_heads))
                                           : 0ull;
    const unsigned long long inclusive = block_scan_sum(mine, s_usum);
    const unsigned long long exclusive = inclusive - mine;
    // Work items are written by the whole warp of each leader, 32 consecutive items per step.
    // Pages are addressed through the table row of the group's longest member: the link
    // window guarantees every member agrees with it on all pages that member can need.
    const int table_row = leader ? __ldcg(&ws.row_table[longest_row]) : 0;
    unsigned leaders = __ballot_sync(0xffffffffu, leader && phase == 1);
    while (leaders != 0u) {
      const int src = __ffs(leaders) - 1;
      leaders &= leaders - 1;
      Item it;
      it.row_start = __shfl_sync(0xffffffffu, r, src);
      it.table_row = __shfl_sync(0xffffffffu, table_row, src);
      const int l_nrows = __shfl_sync(0xffffffffu, nrows, src);
      const int l_chunks = __shfl_sync(0xffffffffu, chunks, src);
      const unsigned l_full = s_base_full + __shfl_sync(0xffffffffu, static_cast<unsigned>(exclusive & 0xffffffffu), src);
      const unsigned l_last = __shfl_sync(0xffffffffu, last_slot, src);
      const int full_count = (l_chunks - 1) * a.kv_heads;
      for (int i = lane; i < full_count; i += 32) {
        it.nrows_head = l_nrows | ((i % a.kv_heads) << 16);
        it.chunk = i / a.kv_heads;
        ws.items_a[l_full + i] = it;
      }
      for (int h = lane; h < a.kv_heads; h += 32) {
        it.nrows_head = l_nrows | (h << 16);
        it.chunk = l_chunks - 1;
        ws.items_b[l_last + h] = it;
      }
    }
    __syncthreads();
    if (threadIdx.x == kPlanThreads - 1) {
      s_carry_start = run_start;
      s_base_full += static_cast<unsigned>(inclusive & 0xffffffffu);
      s_base_last += static_cast<unsigned>(inclusive >> 32);
    }
  }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    ws.header->full_items = s_base_full;
    ws.header->last_items = s_base_last;
    ws.header->next_item = 0;   // `error` keeps what phase 1 recorded (the header is zeroed before every plan)
    ws.header->plan_done = 0;
    ws.header->exited = 0;
  }
}

// ---- main kernel ------------------------------------------------------------------------
// Per-warp view of one claimed work item.  Scalars are warp-uniform; `len` is lane-indexed
// (lane i < nrows: visible length of group row i) and `page` holds the page id of the item's
// tile `lane` (the first 32 tiles).
struct ItemCtx {
  int valid;
  int row_start;
  int table_row;
  int nrows;
  int kv_head;
  int chunk;
  int chunk_start;
  int ntiles;
  int len;
  int page;
};

template <int kWarps, int kStages>
struct __align__(1024) SharedStorage {
  unsigned char stages[kWarps][kStages][kStageBytes];  // per stage: K lo | K hi | V lo | V hi, 2 KiB each
  unsigned long long full[kWarps][kStages];
};

// Claiming a work item is a chain of dependent global accesses (the atomic that hands out the index,
// the item record, then the rows' lengths and the first page ids).  It is split into stages that the
// main loop issues an item ahead of their use, each stage only after the previous one has had a page's
// time to arrive, so that none of them is waited for:
//   claim_index   the atomic; result first used one whole item later
//   fetch_item    the 16-byte item record
//   fetch_rows    lane-indexed: the group's row lengths and the chunk's first 32 page ids
//   finish_item   warp reductions over what fetch_rows loaded
struct Pending {
  int valid;
  Item it;
  int len;
  int page;
};

__device__ __forceinline__ unsigned claim_index(const Workspace& ws, int lane) {
  unsigned idx = 0;
  if (lane == 0) idx = atomicAdd(&ws.header->next_item, 1u);
  return __shfl_sync(0xffffffffu, idx, 0);
}

__device__ __forceinline__ Pending fetch_item(const Workspace& ws, unsigned idx) {
  Pending p;
  const unsigned full = ws.header->full_items, last = ws.header->last_items;
  p.valid = idx < full + last;
  p.len = 0;
  p.page = -1;
  p.it.row_start = p.it.table_row = p.it.nrows_head = p.it.chunk = 0;
  if (p.valid) {
    const int4 raw = *reinterpret_cast<const int4*>(idx < full ? &ws.items_a[idx] : &ws.items_b[idx - full]);
    p.it.row_start = raw.x; p.it.table_row = raw.y; p.it.nrows_head = raw.z; p.it.chunk = raw.w;
  }
  return p;
}

__device__ __forceinline__ void fetch_rows(const AttentionArgs& a, const Workspace& ws, Pending& p, int lane) {
  if (!p.valid) return;
  const int nrows = p.it.nrows_head & 0xffff;
  p.len = lane < nrows ? ws.row_len[p.it.row_start + lane] : 0;
  int cstart, cend;
  chunk_range(p.it.chunk, &cstart, &cend);
  // Page ids are fetched for every lane whose entry lies inside the table row: entries beyond the
  // group's pages are padding, loaded but never used as addresses (finish_item discards them).
  const int first = cstart / kPage;
  const int32_t* table = a.block_tables + static_cast<int64_t>(p.it.table_row) * a.table_width;
  p.page = first + lane < a.table_width ? table[first + lane] : -1;
}

__device__ __forceinline__ ItemCtx finish_item(const Pending& p, int lane) {
  ItemCtx c;
  c.valid = p.valid;
  c.row_start = p.it.row_start;
  c.table_row = p.it.table_row;
  c.nrows = p.it.nrows_head & 0xffff;
  c.kv_head = p.it.nrows_head >> 16;
  c.chunk = p.it.chunk;
  c.len = p.len;
  c.chunk_start = c.ntiles = 0;
  c.page = -1;
  if (!c.valid) return c;
  int longest = c.len;
#pragma unroll
  for (int x = 16; x > 0; x >>= 1) longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, x));
  int cend;
  chunk_range(c.chunk, &c.chunk_start, &cend);
  const int visible = min(cend, longest) - c.chunk_start;
  c.ntiles = visible > 0 ? (visible + kPage - 1) / kPage : 0;
  c.page = lane < c.ntiles ? p.page : -1;
  return c;
}

__device__ __forceinline__ ItemCtx claim_item(const AttentionArgs& a, const Workspace& ws, int lane) {
  Pending p = fetch_item(ws, claim_index(ws, lane));
  fetch_rows(a, ws, p, lane);
  return finish_item(p, lane);
}

// Merge of one row's per-chunk partials, one warp per (row, query head), lane l owning dims
// 4l .. 4l+3:  out = sum_c O_c * 2^(m_c - M) / sum_c l_c * 2^(m_c - M), folded in chunk order with
// M the maximum over the first eight chunks (all chunks, for contexts up to 4096 tokens), raised
// and the sums rescaled when a later group of eight chunks brings a larger one.  Rows of one chunk were finished by the main kernel and are skipped.  The
// partials were written moments ago and are read from L2.
constexpr int kMergeWarps = 4;

template <bool kBF16>
__global__ void __launch_bounds__(kMergeWarps * 32)
merge_kernel(AttentionArgs a, Workspace ws) {
  using T = typename std::conditional<kBF16, __nv_bfloat16, __half>::type;
  const int lane = threadIdx.x & 31;
  const int64_t pair = static_cast<int64_t>(blockIdx.x) * kMergeWarps + (threadIdx.x >> 5);
  if (pair >= static_cast<int64_t>(a.rows) * a.q_heads) return;
  const int64_t row = pair / a.q_heads;
  const int chunks = chunk_count(ws.row_len[row]);
  if (chunks < 2) return;
  const float* part = ws.partials + pair * ws.max_chunks * kPartialStride;
  // Eight chunks per step, all sixteen loads of a step in flight together: a context of up to
  // 4096 tokens is one L2 round trip.  Across steps the running maximum M only grows, and the
  // accumulators are rescaled by 2^(M_old - M_new) — exactly 1 when it did not grow.
  float big = -INFINITY, total = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int c0 = 0; c0 < chunks; c0 += 8) {
    float2 ml[8];
    float4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float* pc = part + min(c0 + i, chunks - 1) * kPartialStride;
      ml[i] = __ldcg(reinterpret_cast<const float2*>(pc + kHeadDim));
      v[i] = __ldcg(reinterpret_cast<const float4*>(pc) + lane);
    }
    float step_big = big;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (c0 + i < chunks) step_big = fmaxf(step_big, ml[i].x);
    if (step_big != big) {
      const float r = big == -INFINITY ? 0.f : fast_exp2(big - step_big);
      acc.x *= r; acc.y *= r; acc.z *= r; acc.w *= r;
      total *= r;
      big = step_big;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (c0 + i < chunks) {
        const float f = ml[i].x == -INFINITY ? 0.f : fast_exp2(ml[i].x - big);
        acc.x = fmaf(v[i].x, f, acc.x); acc.y = fmaf(v[i].y, f, acc.y);
        acc.z = fmaf(v[i].z, f, acc.z); acc.w = fmaf(v[i].w, f, acc.w);
        total = fmaf(ml[i].y, f, total);
      }
    }
  }
  const float inv = 1.0f / total;
  uint2 packed;
  packed.x = pack2<kBF16>(acc.x * inv, acc.y * inv);
  packed.y = pack2<kBF16>(acc.z * inv, acc.w * inv);
  reinterpret_cast<uint2*>(static_cast<T*>(a.out) + pair * kHeadDim)[lane] = packed;
}

// kCopies: TMA copies per page.  4: 3-D maps, one copy per 64-dim half of K and of V.  2: 4-D
// maps, one copy per K or V head slice.  1: one 5-D map over both caches (k_map; v_map unused),
// one copy per page; `k_first` tells which cache lies at the lower address and therefore lands
// in the first half of a stage.
template <bool kBF16, int kWarps, int kStages, int kCopies>
__global__ void __launch_bounds__(kWarps * 32, 1)
verify_attention_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                        AttentionArgs a, Workspace ws, float scale_log2, int k_first) {
  using T = typename std::conditional<kBF16, __nv_bfloat16, __half>::type;
  using Storage = SharedStorage<kWarps, kStages>;
  extern __shared__ unsigned char smem_raw[];
  Storage& sm = *reinterpret_cast<Storage*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gqa = a.q_heads / a.kv_heads;
  const int g = lane >> 2, t = lane & 3;  // fragment row within 8, column pair

  if (lane == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(smem_u32(&sm.full[warp][s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  // Rows of length zero: zeros, their block table is never read.
  {
    const unsigned zero_rows = ws.header->zero_rows;
    const int row_elems = a.q_heads * kHeadDim;  // multiple of 4 elements = 8 bytes
    for (unsigned z = blockIdx.x * kWarps + warp; z < zero_rows; z += gridDim.x * kWarps) {
      uint2* dst = reinterpret_cast<uint2*>(static_cast<T*>(a.out) + static_cast<int64_t>(ws.zero_list[z]) * row_elems);
      for (int i = lane; i < row_elems / 4; i += 32) dst[i] = make_uint2(0u, 0u);
    }
  }
  const uint64_t policy = policy_evict_first();
  const uint32_t stage_base = smem_u32(&sm.stages[warp][0][0]);
  const uint32_t bar_base = smem_u32(&sm.full[warp][0]);

  // ldmatrix source offsets inside a stage (lane dependent, item independent).
  // K: matrix mi of an x4 load = (tokens 8*(mi>>1).., 8-dim chunk 2*(ks&3) + (mi&1)) of half ks>>2.
  // V: matrix mi = (tokens 8*(mi&1).., 8-dim chunk jn + (mi>>1)), transposed on load.
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

  unsigned issued = 0, consumed = 0;  // tiles of this warp's ring
  bool failed = false;
  // A warp holds two items: `cur` is being scored and `nxt` is the one it will score next (claiming
  // further ahead costs more in the schedule's tail than it saves).  nxt is claimed when cur starts,
  // one stage of the chain per page of cur, so it is complete — record, rows, Q fragments — after
  // cur's third page and the issue side can run on into its pages as before.
  ItemCtx cur = claim_item(a, ws, lane);
  ItemCtx nxt = cur;
  nxt.valid = 0;

  // Q rows of an item as mma A-fragments (fragment rows g and g + 8 -> group row and query head).
  auto load_q = [&](const ItemCtx& it, uint32_t (&q)[8][4]) {
    const int rows = it.nrows * gqa;
    const int r0 = g, r1 = g + 8;
    const int l0 = __shfl_sync(0xffffffffu, it.len, (r0 < rows ? r0 : 0) / gqa);
    const int l1 = __shfl_sync(0xffffffffu, it.len, (r1 < rows ? r1 : 0) / gqa);
    const bool live0 = it.valid && r0 < rows && l0 > 0, live1 = it.valid && r1 < rows && l1 > 0;
    const int64_t row0 = it.row_start + r0 / gqa, row1 = it.row_start + r1 / gqa;
    const int head0 = it.kv_head * gqa + r0 % gqa, head1 = it.kv_head * gqa + r1 % gqa;
    const int64_t e0 = (row0 * a.q_heads + head0) * kHeadDim, e1 = (row1 * a.q_heads + head1) * kHeadDim;
    const uint32_t* qp = reinterpret_cast<const uint32_t*>(a.q);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int c = ks * 16 + 2 * t;
      q[ks][0] = live0 ? __ldg(qp + ((e0 + c) >> 1)) : 0u;
      q[ks][1] = live1 ? __ldg(qp + ((e1 + c) >> 1)) : 0u;
      q[ks][2] = live0 ? __ldg(qp + ((e0 + c + 8) >> 1)) : 0u;
      q[ks][3] = live1 ? __ldg(qp + ((e1 + c + 8) >> 1)) : 0u;
    }
  };
  uint32_t qa[8][4];
  load_q(cur, qa);

  // Issue side state, all in registers: the item whose pages are being requested.
  int iss_valid = cur.valid, iss_ntiles = cur.ntiles, iss_x0 = cur.kv_head * kHeadDim;
  int iss_page = cur.page, iss_page_base = 0, iss_tile = 0;
  const int32_t* iss_table = a.block_tables + static_cast<int64_t>(cur.table_row) * a.table_width + cur.chunk_start / kPage;
  bool iss_on_next = false;  // the issue side has moved on to `nxt`
  bool nxt_ready = false;    // nxt's claim is complete (it may still be the invalid end marker)

  // Keep every stage that is not being scored in flight.  Called when all tiles below
  // `consumed` are finished, so tile n may go into stage n % kStages as long as
  // n - consumed < kStages (the tile at `consumed` keeps its own stage while it is scored).
  auto top_up = [&]() {
    while (issued - consumed < static_cast<unsigned>(kStages)) {
      if (!iss_valid) break;
      if (iss_tile >= iss_ntiles) {
        if (iss_on_next || !nxt_ready) break;  // at most one item ahead of the one being scored
        iss_on_next = true;
        iss_valid = nxt.valid; iss_ntiles = nxt.ntiles; iss_x0 = nxt.kv_head * kHeadDim;
        iss_page = nxt.page; iss_page_base = 0; iss_tile = 0;
        iss_table = a.block_tables + static_cast<int64_t>(nxt.table_row) * a.table_width + nxt.chunk_start / kPage;
        continue;
      }
      if (iss_tile >= iss_page_base + 32) {  // next batch of 32 page ids
        iss_page = iss_tile + lane < iss_ntiles ? iss_table[iss_tile + lane] : -1;
        iss_page_base = iss_tile;
      }
      const int block = __shfl_sync(0xffffffffu, iss_page, iss_tile - iss_page_base);
      if (lane == 0) {
        const int stage = issued % kStages;
        const uint32_t bar = bar_base + stage * 8;
        const uint32_t dst = stage_base + stage * kStageBytes;
        mbar_expect_tx(bar, kStageBytes);
        if constexpr (kCopies == 1) {
          tma_load_page_kv(dst, &k_map, iss_x0 >> 6, block, bar, policy);
        } else if constexpr (kCopies == 2) {
          tma_load_page(dst, &k_map, iss_x0 >> 6, block, bar, policy);
          tma_load_page(dst + 4096, &v_map, iss_x0 >> 6, block, bar, policy);
        } else {
          tma_load_page_half(dst, &k_map, iss_x0, block, bar, policy);
          tma_load_page_half(dst + 2048, &k_map, iss_x0 + 64, block, bar, policy);
          tma_load_page_half(dst + 4096, &v_map, iss_x0, block, bar, policy);
          tma_load_page_half(dst + 6144, &v_map, iss_x0 + 64, block, bar, policy);
        }
      }
      ++issued;
      ++iss_tile;
    }
  };

  while (cur.valid && !failed) {
    const int mrows = cur.nrows * gqa;
    const int r0 = g, r1 = g + 8;  // fragment rows -> (group row, query head)
    const int shuffled0 = __shfl_sync(0xffffffffu, cur.len, (r0 < mrows ? r0 : 0) / gqa);
    const int shuffled1 = __shfl_sync(0xffffffffu, cur.len, (r1 < mrows ? r1 : 0) / gqa);
    const int len0 = r0 < mrows ? shuffled0 : 0, len1 = r1 < mrows ? shuffled1 : 0;
    // tiles that end at or before the shortest member's length need no masking
    int shortest = lane < cur.nrows ? cur.len : 0x7fffffff;
#pragma unroll
    for (int x = 16; x > 0; x >>= 1) shortest = min(shortest, __shfl_xor_sync(0xffffffffu, shortest, x));
    const bool padded_rows = mrows < 16;
    nxt_ready = false;  // `nxt` still names this item until the new claim below completes
    top_up();

    const int64_t qrow0 = cur.row_start + r0 / gqa, qrow1 = cur.row_start + r1 / gqa;
    const int qhead0 = cur.kv_head * gqa + r0 % gqa, qhead1 = cur.kv_head * gqa + r1 % gqa;
    const int64_t q0 = (qrow0 * a.q_heads + qhead0) * kHeadDim, q1 = (qrow1 * a.q_heads + qhead1) * kHeadDim;
    // nxt: the atomic now, its record after cur's first page, its rows after the second, the warp
    // reductions and the Q fragments after the third (or at the end of a shorter item).
    uint32_t qb[8][4];
    const unsigned nxt_index = claim_index(ws, lane);
    Pending pending;
    int stage_done = 0;
    auto advance_claim = [&]() {
      if (stage_done == 0) {
        pending = fetch_item(ws, nxt_index);
      } else if (stage_done == 1) {
        fetch_rows(a, ws, pending, lane);
      } else if (stage_done == 2) {
        nxt = finish_item(pending, lane);
        load_q(nxt, qb);
        nxt_ready = true;
      }
      ++stage_done;
    };

    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) { o[j][0] = 0.f; o[j][1] = 0.f; o[j][2] = 0.f; o[j][3] = 0.f; }
    // m: running maximum of score * scale_log2; l: running sum of exp2(score * scale_log2 - m)
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int j = 0; j < cur.ntiles; ++j) {
      const int stage = consumed % kStages;
      if (!mbar_wait(bar_base + stage * 8, (consumed / kStages) & 1)) { failed = true; break; }
      const uint32_t base = stage_base + stage * kStageBytes;
      if (j == cur.ntiles - 1) {   // the page that may end behind the group's longest context: clear V of the slots nobody sees
        int longest = cur.len;
#pragma unroll
        for (int x = 16; x > 0; x >>= 1) longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, x));
        const int seen = longest - (cur.chunk_start + j * kPage);
        if (seen < kPage) {
          unsigned char* v_page = &sm.stages[warp][stage][0] + (k_first ? kTileBytes : 0);
          zero_rows_warp(v_page, v_page + 2048, max(seen, 0), kPage, lane);
        }
      }

      // S = Q K^T for the 16 tokens of this page (two n8 tiles, two accumulator chains each)
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      float s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t b[4];
        ldmatrix_x4(base + koff[ks], b);
        if (ks & 1) {
          mma_16816<kBF16>(s2[0], qa[ks], b[0], b[1]);
          mma_16816<kBF16>(s2[1], qa[ks], b[2], b[3]);
        } else {
          mma_16816<kBF16>(s[0], qa[ks], b[0], b[1]);
          mma_16816<kBF16>(s[1], qa[ks], b[2], b[3]);
        }
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] += s2[nt][e];
      }
      // mask by each row's own length (only tiles that reach past the shortest member)
      const int tile_start = cur.chunk_start + j * kPage;
      if (padded_rows || tile_start + kPage > shortest) {
        const int tok = tile_start + 2 * t;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int pos = tok + nt * 8 + e;
            if (pos >= len0) s[nt][e] = -INFINITY;
            if (pos >= len1) s[nt][2 + e] = -INFINITY;
          }
        }
      }
      float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
      float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0 * scale_log2), mn1 = fmaxf(m1, mx1 * scale_log2);
      const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
      const bool moved = (mn0 != m0) || (mn1 != m1);
      const float al0 = fast_exp2(m0 - mu0), al1 = fast_exp2(m1 - mu1);
      m0 = mn0; m1 = mn1;
      uint32_t pa[4];
      {
        const float p00 = fast_exp2(fmaf(s[0][0], scale_log2, -mu0)), p01 = fast_exp2(fmaf(s[0][1], scale_log2, -mu0));
        const float p02 = fast_exp2(fmaf(s[0][2], scale_log2, -mu1)), p03 = fast_exp2(fmaf(s[0][3], scale_log2, -mu1));
        const float p10 = fast_exp2(fmaf(s[1][0], scale_log2, -mu0)), p11 = fast_exp2(fmaf(s[1][1], scale_log2, -mu0));
        const float p12 = fast_exp2(fmaf(s[1][2], scale_log2, -mu1)), p13 = fast_exp2(fmaf(s[1][3], scale_log2, -mu1));
        l0 = l0 * al0 + ((p00 + p01) + (p10 + p11));
        l1 = l1 * al1 + ((p02 + p03) + (p12 + p13));
        pa[0] = pack2<kBF16>(p00, p01);
        pa[1] = pack2<kBF16>(p02, p03);
        pa[2] = pack2<kBF16>(p10, p11);
        pa[3] = pack2<kBF16>(p12, p13);
      }
      // Rescale O only when some row's running maximum moved (a factor of exactly 1 otherwise).
      if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
        for (int jn = 0; jn < 16; ++jn) { o[jn][0] *= al0; o[jn][1] *= al0; o[jn][2] *= al1; o[jn][3] *= al1; }
      }
      // O += P V
#pragma unroll
      for (int jp = 0; jp < 8; ++jp) {
        uint32_t b[4];
        ldmatrix_x4_trans(base + voff[jp], b);
        mma_16816<kBF16>(o[2 * jp], pa, b[0], b[1]);
        mma_16816<kBF16>(o[2 * jp + 1], pa, b[2], b[3]);
      }
      ++consumed;
      if (j < 3) advance_claim();
      // The stage just read is free.  Every lane's ldmatrix results have been consumed by its
      // MMAs, so the reads are complete before lane 0 passes this barrier and issues the copy
      // that overwrites the stage (the consumer-release step of a TMA pipeline needs no
      // proxy fence: only generic WRITES must be fenced before async-proxy accesses).
      __syncwarp();
      top_up();
    }
    if (failed) break;
    while (stage_done < 3) advance_claim();  // items of fewer than three pages

    // ---- epilogue: straight from registers ----
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const int chunks0 = chunk_count(len0), chunks1 = chunk_count(len1);
    T* out = static_cast<T*>(a.out);
    if (cur.chunk < chunks0) {
      if (chunks0 == 1) {
        const float inv = 1.0f / l0;
        uint32_t* dst = reinterpret_cast<uint32_t*>(out + q0);
#pragma unroll
        for (int jn = 0; jn < 16; ++jn) dst[jn * 4 + t] = pack2<kBF16>(o[jn][0] * inv, o[jn][1] * inv);
      } else {
        float* part = ws.partials + ((qrow0 * a.q_heads + qhead0) * ws.max_chunks + cur.chunk) * kPartialStride;
#pragma unroll
        for (int jn = 0; jn < 16; ++jn) *reinterpret_cast<float2*>(part + jn * 8 + 2 * t) = make_float2(o[jn][0], o[jn][1]);
        if (t == 0) { part[kHeadDim] = m0; part[kHeadDim + 1] = l0; }
      }
    }
    if (cur.chunk < chunks1) {
      if (chunks1 == 1) {
        const float inv = 1.0f / l1;
        uint32_t* dst = reinterpret_cast<uint32_t*>(out + q1);
#pragma unroll
        for (int jn = 0; jn < 16; ++jn) dst[jn * 4 + t] = pack2<kBF16>(o[jn][2] * inv, o[jn][3] * inv);
      } else {
        float* part = ws.partials + ((qrow1 * a.q_heads + qhead1) * ws.max_chunks + cur.chunk) * kPartialStride;
#pragma unroll
        for (int jn = 0; jn < 16; ++jn) *reinterpret_cast<float2*>(part + jn * 8 + 2 * t) = make_float2(o[jn][2], o[jn][3]);
        if (t == 0) { part[kHeadDim] = m1; part[kHeadDim + 1] = l1; }
      }
    }
    // ---- next item ----
    cur = nxt;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) { qa[ks][0] = qb[ks][0]; qa[ks][1] = qb[ks][1]; qa[ks][2] = qb[ks][2]; qa[ks][3] = qb[ks][3]; }
    if (iss_on_next) {
      iss_on_next = false;  // the issue side is already inside the new `cur`
    } else {                // (re)start the issue side at the first page of the new item
      iss_valid = cur.valid; iss_ntiles = cur.ntiles; iss_x0 = cur.kv_head * kHeadDim;
      iss_page = cur.page; iss_page_base = 0; iss_tile = 0;
      iss_table = a.block_tables + static_cast<int64_t>(cur.table_row) * a.table_width + cur.chunk_start / kPage;
    }
  }

  if (failed) {
    if (lane == 0) atomicOr(&ws.header->error, kErrorWaitGaveUp);
    // let copies already in flight land before the shared memory is released
    for (unsigned n = consumed + 1; n < issued; ++n) mbar_wait(bar_base + (n % kStages) * 8, (n / kStages) & 1);
  }
  // The last warp to finish rewinds the claim counter: the plan in the workspace stays valid
  // for further runs over the same block tables and lengths (other layers of the same pass).
  if (lane == 0) {
    const unsigned before = atomicAdd(&ws.header->exited, 1u);
    if (before == gridDim.x * kWarps - 1) {
      ws.header->next_item = 0;
      ws.header->exited = 0;
    }
  }
}

// ---- host side ----------------------------------------------------------------------------
int gqa_cap(const AttentionArgs& a) { return kMaxGroupRows / (a.q_heads / a.kv_heads); }

template <bool kBF16, int kWarps, int kStages, int kCopies>
int launch_main(const CUtensorMap& k_map, const CUtensorMap& v_map, const AttentionArgs& a, const Workspace& ws,
                int sm_count, cudaStream_t stream, bool k_first = true) {
  const size_t smem = sizeof(SharedStorage<kWarps, kStages>) + 1024;
  const float scale_log2 = static_cast<float>(1.4426950408889634 / sqrt(static_cast<double>(kHeadDim)));
  auto kernel = verify_attention_kernel<kBF16, kWarps, kStages, kCopies>;
  RLT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  kernel<<<sm_count, kWarps * 32, smem, stream>>>(k_map, v_map, a, ws, scale_log2, k_first ? 1 : 0);
  int status = launch_status("verify_attention_kernel");
  if (status != RLT_OK || ws.max_chunks < 2) return status;  // no context can span two chunks
  const int64_t pairs = static_cast<int64_t>(a.rows) * a.q_heads;
  merge_kernel<kBF16><<<static_cast<unsigned>((pairs + kMergeWarps - 1) / kMergeWarps), kMergeWarps * 32, 0, stream>>>(a, ws);
  return launch_status("merge_kernel");
}

}  // namespace

bool attention_sm100_shape_supported(const AttentionArgs& a) {
  if (a.dtype != RLT_BF16 && a.dtype != RLT_F16) return false;
  if (a.head_dim != kHeadDim || a.block_size != kPage) return false;
  if (a.kv_heads <= 0 || a.q_heads % a.kv_heads != 0) return false;
  const int gqa = a.q_heads / a.kv_heads;
  if (gqa != 1 && gqa != 2 && gqa != 4 && gqa != 8 && gqa != 16) return false;
  if (a.kv_heads > 32767) return false;
  if (static_cast<long long>(a.table_width) * a.block_size > (1 << 26)) return false;
  return true;
}

bool attention_sm100_supported(const AttentionArgs& a) {
  if (!attention_sm100_shape_supported(a)) return false;
  if (a.token_stride < static_cast<int64_t>(a.kv_heads) * kHeadDim) return false;
  if ((a.token_stride * 2) % 16 != 0 || (a.block_stride * 2) % 16 != 0) return false;
  if (a.block_stride < a.token_stride * kPage) return false;
  if (!aligned16(a.key_cache) || !aligned16(a.value_cache)) return false;
  if ((reinterpret_cast<uintptr_t>(a.q) & 3u) != 0 || (reinterpret_cast<uintptr_t>(a.out) & 15u) != 0) return false;
  if (a.num_blocks > 0xffffffffll) return false;
  return true;
}

size_t attention_sm100_workspace_bytes(int rows, int q_heads, int kv_heads, int head_dim, int block_size,
                                       int table_width) {
  (void)head_dim;
  return make_layout(rows, q_heads, kv_heads, block_size, table_width).total;
}

int attention_sm100_read_status(const void* workspace, cudaStream_t stream, unsigned* out4) {
  Header h;
  RLT_CUDA_TRY(cudaMemcpyAsync(&h, workspace, sizeof(Header), cudaMemcpyDeviceToHost, stream));
  RLT_CUDA_TRY(cudaStreamSynchronize(stream));
  out4[0] = h.full_items + h.last_items; out4[1] = h.zero_rows; out4[2] = h.error; out4[3] = h.next_item;
  return RLT_OK;
}

namespace {

int bind_workspace(const AttentionArgs& a, void* workspace, size_t workspace_bytes, Workspace* ws) {
  const Layout l = make_layout(a.rows, a.q_heads, a.kv_heads, a.block_size, a.table_width);
  if (workspace == nullptr || workspace_bytes < l.total || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) {
    set_last_error_text("verify_attention: workspace missing, misaligned or too small");
    return RLT_ERR_WORKSPACE;
  }
  char* base = static_cast<char*>(workspace);
  ws->header = reinterpret_cast<Header*>(base + l.header);
  ws->row_len = reinterpret_cast<int*>(base + l.row_len);
  ws->row_table = reinterpret_cast<int*>(base + l.row_table);
  ws->link = reinterpret_cast<int*>(base + l.link);
  ws->zero_list = reinterpret_cast<int*>(base + l.zero_list);
  ws->items_a = reinterpret_cast<Item*>(base + l.items_a);
  ws->items_b = reinterpret_cast<Item*>(base + l.items_b);
  ws->partials = reinterpret_cast<float*>(base + l.partials);
  ws->max_chunks = l.max_chunks;
  return RLT_OK;
}

}  // namespace

// Builds the work lists for (block_tables, context_lengths, cu_seqlens_q) in the workspace.
int plan_attention_sm100(const AttentionArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  Workspace ws;
  int status = bind_workspace(a, workspace, workspace_bytes, &ws);
  if (status != RLT_OK) return status;
  RLT_CUDA_TRY(cudaMemsetAsync(ws.header, 0, sizeof(Header), stream));
  const int plan_ctas = (a.rows + kPlanThreads / 32 - 1) / (kPlanThreads / 32);
  plan_kernel<<<plan_ctas, kPlanThreads, 0, stream>>>(a, ws, gqa_cap(a));
  return launch_status("plan_kernel");
}

// Scores q against one layer's K/V with the plan already in the workspace.
int run_attention_sm100(const AttentionArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  Workspace ws;
  int status = bind_workspace(a, workspace, workspace_bytes, &ws);
  if (status != RLT_OK) return status;
  DeviceInfo info;
  status = current_device_info(&info);
  if (status != RLT_OK) return status;
  // RLT_ATTENTION_COPIES (4, 2 or 1 TMA copies per page) pins a variant for tuning runs.  By
  // default the fewest copies the driver accepts a map for are used.
  static const int pinned = [] {
    const char* e = getenv("RLT_ATTENTION_COPIES");
    return e ? atoi(e) : 0;
  }();
  CUtensorMap k_map, v_map;
  bool k_first = true;
  int copies = 4;
  if ((pinned == 0 || pinned == 1) && make_joint_map(&k_map, a, &k_first) == RLT_OK) {
    copies = 1;
    v_map = k_map;
  } else if (pinned != 4 && make_head_map(&k_map, a.key_cache, a) == RLT_OK &&
             make_head_map(&v_map, a.value_cache, a) == RLT_OK) {
    copies = 2;
    k_first = true;
  } else {
    k_first = true;
    status = make_page_map(&k_map, a.key_cache, a);
    if (status != RLT_OK) return status;
    status = make_page_map(&v_map, a.value_cache, a);
    if (status != RLT_OK) return status;
  }
  if (a.dtype == RLT_BF16) {
    if (copies == 1) return launch_main<true, 8, 3, 1>(k_map, v_map, a, ws, info.sm_count, stream, k_first);
    if (copies == 2) return launch_main<true, 8, 3, 2>(k_map, v_map, a, ws, info.sm_count, stream);
    return launch_main<true, 8, 3, 4>(k_map, v_map, a, ws, info.sm_count, stream);
  }
  if (copies == 1) return launch_main<false, 8, 3, 1>(k_map, v_map, a, ws, info.sm_count, stream, k_first);
  if (copies == 2) return launch_main<false, 8, 3, 2>(k_map, v_map, a, ws, info.sm_count, stream);
  return launch_main<false, 8, 3, 4>(k_map, v_map, a, ws, info.sm_count, stream);
}

int launch_attention_sm100(const AttentionArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  const int status = plan_attention_sm100(a, workspace, workspace_bytes, stream);
  if (status != RLT_OK) return status;
  return run_attention_sm100(a, workspace, workspace_bytes, stream);
}

// ---- built-in scratch for callers that must not allocate ------------------------------------
// A fixed 32 MiB block of device memory that is part of the library image: every GPU context
// that loads the library holds it until the process exits.  In host code the array's name is
// only a handle; the device address the kernels need is looked up once per device.
constexpr size_t kBuiltinScratchBytes = 32u << 20;
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];

namespace {

int builtin_scratch_address(void** address) {
  constexpr int kMaxDevices = 64;
  static std::mutex mutex;
  static void* cached[kMaxDevices] = {};
  int device = 0;
  RLT_CUDA_TRY(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) {
    set_last_error_text("device index out of range");
    return RLT_ERR_INVALID;
  }
  std::lock_guard<std::mutex> lock(mutex);
  if (cached[device] == nullptr) {
    void* found = nullptr;
    RLT_CUDA_TRY(cudaGetSymbolAddress(&found, g_builtin_scratch));  // for the current device
    cached[device] = found;
  }
  *address = cached[device];
  return RLT_OK;
}

}  // namespace

size_t attention_sm100_builtin_scratch_bytes() { return kBuiltinScratchBytes; }

// Looks the block up for the current device without launching anything: the one-time set-up a
// host performs before it hands its remaining device memory to something else.
int attention_sm100_builtin_warmup() {
  void* scratch = nullptr;
  return builtin_scratch_address(&scratch);
}

int launch_attention_sm100_builtin(const AttentionArgs& a, cudaStream_t stream) {
  const size_t need = make_layout(a.rows, a.q_heads, a.kv_heads, a.block_size, a.table_width).total;
  if (need > kBuiltinScratchBytes) {
    char text[256];
    snprintf(text, sizeof(text),
             "verify_attention_noalloc: this batch needs %zu bytes of scratch but the built-in scratch holds %zu; "
             "use rlt_verify_attention with a caller-owned workspace",
             need, kBuiltinScratchBytes);
    set_last_error_text(text);
    return RLT_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  const int status = builtin_scratch_address(&scratch);
  if (status != RLT_OK) return status;
  return launch_attention_sm100(a, scratch, kBuiltinScratchBytes, stream);
}


}  // namespace rlt
