// Verify attention for sm_100a: head_dim 128, 16-token pages, fp16 / bf16.
//
// Data flow
//   plan kernel   one warp per query row: finds the rows that share a block-table row
//                 (the k+1 rows of one request at one depth plane; k x depths rows in a
//                 shared-plane layout), zero-fills empty rows, and the last CTA to finish
//                 turns the groups into a work list of (group, context chunk, kv head).
//   main kernel   persistent, 2 CTAs per SM.  A producer warp pulls work items and streams
//                 the item's K/V pages into a ring of shared-memory stages with TMA
//                 (cp.async.bulk.tensor, 128-byte swizzle, page id = TMA block coordinate,
//                 so every page is read from HBM once per group, not once per row).  Four
//                 consumer warps score up to 16 query rows against each page on tensor
//                 cores (m16n8k16, Q in registers, K/V fragments by ldmatrix) with an fp32
//                 online softmax, are merged in warp order, and either finish the row or
//                 store an fp32 partial; the CTA that stores the last partial of a group
//                 merges the chunks in chunk order.
//
// Batch invariance: tile -> warp assignment, chunk boundaries and both merge orders are
// functions of absolute token positions only, and a tensor-core output row depends only on
// its own input row, so a row's bits do not depend on its group or batch.
//
// HBM traffic per call = each group's K/V once + Q + O (+ fp32 partials for contexts of more
// than one chunk), which is what the roofline of this kernel is measured against.
#include <cuda.h>
#include <math.h>

#include <mutex>
#include <type_traits>

#include "attention.cuh"

namespace rlt {
namespace {

constexpr int kHeadDim = 128;
constexpr int kPage = 16;
constexpr int kStages = 8;                    // ring of (K page, V page) tiles
constexpr int kTileBytes = kPage * kHeadDim * 2;  // one page of one head: 4 KiB
constexpr int kStageBytes = 2 * kTileBytes;
constexpr int kConsumerWarps = 4;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kItemSlots = 4;
constexpr int kMergeStride = 132;             // floats per merged row (128 + pad)
constexpr int kPartialStride = 132;           // floats per stored partial: O[128], m, l, pad
constexpr int kPlanWarps = 8;
constexpr long long kWaitCycles = 4000000000ll;  // bounded waits (about 2 s): give up instead of hanging

// ---- context chunks -------------------------------------------------------------------
// Fixed, position-only chunk boundaries: eight 512-token chunks up to 4096, then every
// power-of-two octave [4096 * 2^k, 4096 * 2^(k+1)) in four equal chunks.
__host__ __device__ inline int floor_log2(unsigned x) {
#ifdef __CUDA_ARCH__
  return 31 - __clz(x);
#else
  return 31 - __builtin_clz(x);
#endif
}

__host__ __device__ inline int chunk_count(int len) {
  if (len <= 0) return 0;
  if (len <= 4096) return (len + 511) >> 9;
  const int k = floor_log2(static_cast<unsigned>((len - 1) >> 12));
  return 8 + 4 * k + (len - 1 - (4096 << k)) / (1024 << k) + 1;
}

__host__ __device__ inline void chunk_range(int c, int* start, int* end) {
  if (c < 8) {
    *start = c << 9;
    *end = *start + 512;
  } else {
    const int k = (c - 8) >> 2, j = (c - 8) & 3;
    *start = (4096 << k) + j * (1024 << k);
    *end = *start + (1024 << k);
  }
}

// ---- workspace ------------------------------------------------------------------------
struct Header {
  unsigned item_count;
  unsigned next_item;
  unsigned error;      // nonzero: a bounded wait gave up (bit 0 producer, bit 1 consumer)
  unsigned plan_done;  // CTAs of the plan kernel that finished phase 1
};

struct Item {
  int row_start;
  int table_row;
  int nrows_head;  // nrows | kv_head << 16
  int chunk;
};

struct Layout {
  size_t header, row_len, row_table, link, counters, items, partials, total;
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
  l.counters = off; off += align256(sizeof(unsigned) * rows * kv_heads);
  l.items = off; off += align256(sizeof(Item) * static_cast<size_t>(rows) * kv_heads * l.max_chunks);
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
  unsigned* counters;
  Item* items;
  float* partials;
  int max_chunks;
};

// ---- PTX wrappers -----------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
__device__ __forceinline__ void consumer_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}

// ---- plan kernel ------------------------------------------------------------------------
// Rows r-1 and r are linked when both are non-empty and their table rows agree on every
// page any of the last `cap` rows can need (that window makes agreement transitive inside
// a group of at most `cap` rows).  Packed input states its groups through cu_seqlens_q.
template <typename T>
__global__ void __launch_bounds__(kPlanWarps * 32)
plan_kernel(AttentionArgs a, Workspace ws, int cap) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x * kPlanWarps + warp;
  if (row < a.rows) {
    int table_row, len;
    resolve_row(a, row, &table_row, &len);
    int link = 0;
    if (len > 0 && row > 0) {
      int prev_table, prev_len;
      resolve_row(a, row - 1, &prev_table, &prev_len);
      if (prev_len > 0) {
        if (a.cu_seqlens_q != nullptr) {
          link = prev_table == table_row;
        } else {
          int longest = len;
          for (int back = 1; back < cap && row - back >= 0; ++back) {
            const int other = a.context_lengths[row - back];
            longest = other > longest ? other : longest;
          }
          const int pages = (longest + a.block_size - 1) / a.block_size;
          const int32_t* mine = a.block_tables + static_cast<int64_t>(row) * a.table_width;
          const int32_t* prev = mine - a.table_width;
          int same = 1;
          for (int p = lane; p < pages && p < a.table_width; p += 32) same &= mine[p] == prev[p];
          link = __all_sync(0xffffffffu, same);
        }
      }
    }
    if (len <= 0) {  // empty row: zeros, never part of a group
      T* out = static_cast<T*>(a.out) + static_cast<int64_t>(row) * a.q_heads * a.head_dim;
      for (int i = lane; i < a.q_heads * a.head_dim; i += 32) out[i] = Elem<T>::from_float(0.0f);
    }
    if (lane == 0) {
      ws.row_len[row] = len > 0 ? len : 0;
      ws.row_table[row] = table_row;
      ws.link[row] = link;
    }
    for (int h = lane; h < a.kv_heads; h += 32) ws.counters[static_cast<int64_t>(row) * a.kv_heads + h] = 0;
  }

  // The last CTA to get here builds the work list.
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

  constexpr int kT = kPlanWarps * 32;
  __shared__ int s_scan[kT];
  __shared__ int s_carry_start;   // start of the run that reaches into this tile
  __shared__ unsigned s_item_base;
  if (threadIdx.x == 0) { s_carry_start = 0; s_item_base = 0; }
  __syncthreads();
  volatile int* vlink = ws.link;
  volatile int* vlen = ws.row_len;
  for (int base = 0; base < a.rows; base += kT) {
    const int r = base + threadIdx.x;
    const bool in = r < a.rows;
    const int linked = in ? vlink[r] : 0;
    const int len = in ? vlen[r] : 0;
    // run start of every row: max-scan of (start ? r : carry)
    s_scan[threadIdx.x] = (in && !linked) ? r : -1;
    __syncthreads();
    for (int step = 1; step < kT; step <<= 1) {
      int v = s_scan[threadIdx.x];
      if (threadIdx.x >= step) v = max(v, s_scan[threadIdx.x - step]);
      __syncthreads();
      s_scan[threadIdx.x] = v;
      __syncthreads();
    }
    int run_start = s_scan[threadIdx.x];
    if (run_start < 0) run_start = s_carry_start;
    __syncthreads();
    if (threadIdx.x == kT - 1) s_carry_start = run_start;
    const bool leader = in && len > 0 && ((r - run_start) % cap == 0);
    int nrows = 0, longest = 0, longest_row = r;
    if (leader) {
      nrows = 1;
      longest = len;
      while (nrows < cap && r + nrows < a.rows && vlink[r + nrows]) {
        const int other = vlen[r + nrows];
        if (other > longest) { longest = other; longest_row = r + nrows; }
        ++nrows;
      }
    }
    const int chunks = leader ? chunk_count(longest) : 0;
    const int count = chunks * a.kv_heads;
    // exclusive scan of item counts
    s_scan[threadIdx.x] = count;
    __syncthreads();
    for (int step = 1; step < kT; step <<= 1) {
      int v = s_scan[threadIdx.x];
      if (threadIdx.x >= step) v += s_scan[threadIdx.x - step];
      __syncthreads();
      s_scan[threadIdx.x] = v;
      __syncthreads();
    }
    const unsigned first = s_item_base + static_cast<unsigned>(s_scan[threadIdx.x] - count);
    if (leader) {
      // Pages are addressed through the table row of the group's longest member: the link
      // window guarantees every member agrees with it on all pages that member can need.
      const int table_row = __ldcg(&ws.row_table[longest_row]);
      unsigned i = first;
      for (int c = chunks - 1; c >= 0; --c)        // last (largest / ragged) chunks first
        for (int h = 0; h < a.kv_heads; ++h) {
          Item it;
          it.row_start = r;
          it.table_row = table_row;
          it.nrows_head = nrows | (h << 16);
          it.chunk = c;
          ws.items[i++] = it;
        }
    }
    __syncthreads();
    if (threadIdx.x == kT - 1) s_item_base += static_cast<unsigned>(s_scan[kT - 1]);
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    ws.header->item_count = s_item_base;
    ws.header->next_item = 0;
    ws.header->error = 0;
    ws.header->plan_done = 0;
  }
}

// ---- main kernel ------------------------------------------------------------------------
struct ItemSlot {
  int valid;
  int row_start;
  int nrows;
  int kv_head;
  int chunk;
  int chunk_start;
  int ntiles;
  int group_chunks;
  int lens[16];
};

struct __align__(1024) SharedStorage {
  unsigned char stages[kStages][kStageBytes];         // K lo | K hi | V lo | V hi, 2 KiB each
  float merge_o[kConsumerWarps][16][kMergeStride];
  float merge_m[kConsumerWarps][16];
  float merge_l[kConsumerWarps][16];
  ItemSlot slots[kItemSlots];
  unsigned long long full[kStages];
  unsigned long long empty[kStages];
  unsigned long long item_full[kItemSlots];
  unsigned long long item_empty[kItemSlots];
  int last_flag;
};

template <bool kBF16>
__global__ void __launch_bounds__(kThreads, 2)
verify_attention_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                        AttentionArgs a, Workspace ws, float scale_log2) {
  using T = typename std::conditional<kBF16, __nv_bfloat16, __half>::type;
  extern __shared__ unsigned char smem_raw[];
  SharedStorage& sm = *reinterpret_cast<SharedStorage*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gqa = a.q_heads / a.kv_heads;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(smem_u32(&sm.full[s]), 1); mbar_init(smem_u32(&sm.empty[s]), 1); }
    for (int s = 0; s < kItemSlots; ++s) {
      mbar_init(smem_u32(&sm.item_full[s]), 1);
      mbar_init(smem_u32(&sm.item_empty[s]), kConsumerWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ===================== producer warp =====================
    const uint64_t policy = policy_evict_first();
    unsigned tile_counter = 0;  // tiles issued so far by this CTA (ring position)
    unsigned item_counter = 0;
    bool failed = false;
    for (;;) {
      unsigned idx = 0;
      if (lane == 0) idx = atomicAdd(&ws.header->next_item, 1u);
      idx = __shfl_sync(0xffffffffu, idx, 0);
      const unsigned total = ws.header->item_count;
      const int slot = item_counter % kItemSlots;
      const unsigned use = item_counter / kItemSlots;
      if (use > 0 && !mbar_wait(smem_u32(&sm.item_empty[slot]), (use - 1) & 1)) { failed = true; break; }
      if (idx >= total) {
        if (lane == 0) { sm.slots[slot].valid = 0; mbar_arrive(smem_u32(&sm.item_full[slot])); }
        break;
      }
      const Item it = ws.items[idx];
      const int nrows = it.nrows_head & 0xffff, kv_head = it.nrows_head >> 16;
      int len = (lane < nrows) ? ws.row_len[it.row_start + lane] : 0;
      int longest = len;
#pragma unroll
      for (int x = 16; x > 0; x >>= 1) longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, x));
      int cstart, cend;
      chunk_range(it.chunk, &cstart, &cend);
      const int visible = min(cend, longest) - cstart;
      const int ntiles = visible > 0 ? (visible + kPage - 1) / kPage : 0;
      if (lane < 16) sm.slots[slot].lens[lane] = len;
      if (lane == 0) {
        ItemSlot& s = sm.slots[slot];
        s.valid = 1; s.row_start = it.row_start; s.nrows = nrows; s.kv_head = kv_head;
        s.chunk = it.chunk; s.chunk_start = cstart; s.ntiles = ntiles;
        s.group_chunks = chunk_count(longest);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm.item_full[slot]));
      ++item_counter;

      const int32_t* table = a.block_tables + static_cast<int64_t>(it.table_row) * a.table_width + cstart / kPage;
      const int x0 = kv_head * kHeadDim;
      for (int tbase = 0; tbase < ntiles && !failed; tbase += 32) {
        const int mine = tbase + lane;
        const int page = mine < ntiles ? table[mine] : -1;
        const int batch = min(32, ntiles - tbase);
        for (int j = 0; j < batch; ++j) {
          const int block = __shfl_sync(0xffffffffu, page, j);
          if (lane == 0) {
            const int stage = tile_counter % kStages;
            const unsigned suse = tile_counter / kStages;
            if (suse > 0 && !mbar_wait(smem_u32(&sm.empty[stage]), (suse - 1) & 1)) failed = true;
            if (!failed) {
              const uint32_t bar = smem_u32(&sm.full[stage]);
              const uint32_t dst = smem_u32(&sm.stages[stage][0]);
              mbar_expect_tx(bar, kStageBytes);
              tma_load_page_half(dst, &k_map, x0, block, bar, policy);
              tma_load_page_half(dst + 2048, &k_map, x0 + 64, block, bar, policy);
              tma_load_page_half(dst + 4096, &v_map, x0, block, bar, policy);
              tma_load_page_half(dst + 6144, &v_map, x0 + 64, block, bar, policy);
            }
          }
          ++tile_counter;
          failed = __shfl_sync(0xffffffffu, failed ? 1 : 0, 0) != 0;
          if (failed) break;
        }
      }
      if (failed) break;
    }
    if (failed && lane == 0) {
      atomicOr(&ws.header->error, 1u);
      // Tell the consumers to stop, then let copies already in flight land before the
      // shared memory is released.
      for (int s = 0; s < kItemSlots; ++s) sm.slots[s].valid = 0;
      __threadfence_block();
      for (int s = 0; s < kItemSlots; ++s) mbar_arrive(smem_u32(&sm.item_full[s]));
      const unsigned issued = tile_counter;
      for (unsigned n = issued > kStages ? issued - kStages : 0; n < issued; ++n)
        mbar_wait(smem_u32(&sm.full[n % kStages]), (n / kStages) & 1);
    }
    return;
  }

  // ===================== consumer warps =====================
  const int g = lane >> 2, t = lane & 3;  // fragment row within 8, column pair
  unsigned tile_counter = 0, item_counter = 0;
  for (;;) {
    const int slot = item_counter % kItemSlots;
    if (!mbar_wait(smem_u32(&sm.item_full[slot]), (item_counter / kItemSlots) & 1)) {
      if (lane == 0) atomicOr(&ws.header->error, 2u);
      break;
    }
    const ItemSlot& is = sm.slots[slot];
    if (!is.valid) break;
    const int row_start = is.row_start, nrows = is.nrows, kv_head = is.kv_head;
    const int chunk = is.chunk, chunk_start = is.chunk_start, ntiles = is.ntiles;
    const int group_chunks = is.group_chunks;
    // fragment rows g and g+8 -> (query row, query head, visible length)
    const int mrows = nrows * gqa;
    const int r0 = g, r1 = g + 8;
    const int len0 = r0 < mrows ? is.lens[r0 / gqa] : 0;
    const int len1 = r1 < mrows ? is.lens[r1 / gqa] : 0;
    ++item_counter;

    const int64_t q0 = (static_cast<int64_t>(row_start + r0 / gqa) * a.q_heads + kv_head * gqa + r0 % gqa) * kHeadDim;
    const int64_t q1 = (static_cast<int64_t>(row_start + r1 / gqa) * a.q_heads + kv_head * gqa + r1 % gqa) * kHeadDim;
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

    for (int j = warp; j < ntiles; j += kConsumerWarps) {
      const unsigned n = tile_counter + j;
      const int stage = n % kStages;
      if (!mbar_wait(smem_u32(&sm.full[stage]), (n / kStages) & 1)) { failed = true; break; }
      const uint32_t kbase = smem_u32(&sm.stages[stage][0]);
      const uint32_t vbase = kbase + kTileBytes;

      // S = Q K^T for the 16 tokens of this page (two n8 tiles)
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      {
        const int mi = lane >> 3, token = ((mi >> 1) << 3) + (lane & 7);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const int chunk16 = ((ks & 3) << 1) + (mi & 1);
          const uint32_t addr = kbase + ((ks >> 2) << 11) + token * 128 + ((chunk16 ^ (token & 7)) << 4);
          uint32_t b[4];
          ldmatrix_x4(addr, b);
          mma_16816<kBF16>(s[0], qa[ks], b[0], b[1]);
          mma_16816<kBF16>(s[1], qa[ks], b[2], b[3]);
        }
      }
      // mask by each row's own length, move to the log2 domain
      const int tok = chunk_start + j * kPage + 2 * t;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int pos = tok + nt * 8 + e;
          s[nt][e] = pos < len0 ? s[nt][e] * scale_log2 : -INFINITY;
          s[nt][2 + e] = pos < len1 ? s[nt][2 + e] * scale_log2 : -INFINITY;
        }
      }
      float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
      float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
      const float al0 = fast_exp2(m0 - mu0), al1 = fast_exp2(m1 - mu1);
      m0 = mn0; m1 = mn1;
      uint32_t pa[4];
      {
        const float p00 = fast_exp2(s[0][0] - mu0), p01 = fast_exp2(s[0][1] - mu0);
        const float p02 = fast_exp2(s[0][2] - mu1), p03 = fast_exp2(s[0][3] - mu1);
        const float p10 = fast_exp2(s[1][0] - mu0), p11 = fast_exp2(s[1][1] - mu0);
        const float p12 = fast_exp2(s[1][2] - mu1), p13 = fast_exp2(s[1][3] - mu1);
        l0 = l0 * al0 + ((p00 + p01) + (p10 + p11));
        l1 = l1 * al1 + ((p02 + p03) + (p12 + p13));
        pa[0] = pack2<kBF16>(p00, p01);
        pa[1] = pack2<kBF16>(p02, p03);
        pa[2] = pack2<kBF16>(p10, p11);
        pa[3] = pack2<kBF16>(p12, p13);
      }
#pragma unroll
      for (int jn = 0; jn < 16; ++jn) { o[jn][0] *= al0; o[jn][1] *= al0; o[jn][2] *= al1; o[jn][3] *= al1; }
      // O += P V
      {
        const int mi = lane >> 3, token = ((mi & 1) << 3) + (lane & 7);
#pragma unroll
        for (int jn = 0; jn < 16; jn += 2) {
          const int c = jn + (mi >> 1);
          const uint32_t addr = vbase + ((c >> 3) << 11) + token * 128 + (((c & 7) ^ (token & 7)) << 4);
          uint32_t b[4];
          ldmatrix_x4_trans(addr, b);
          mma_16816<kBF16>(o[jn], pa, b[0], b[1]);
          mma_16816<kBF16>(o[jn + 1], pa, b[2], b[3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm.empty[stage]));
    }
    tile_counter += ntiles;
    if (failed) {
      if (lane == 0) atomicOr(&ws.header->error, 2u);
      break;
    }

    // ---- merge the four warps in warp order ----
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (t == 0) {
      sm.merge_m[warp][r0] = m0; sm.merge_l[warp][r0] = l0;
      sm.merge_m[warp][r1] = m1; sm.merge_l[warp][r1] = l1;
    }
#pragma unroll
    for (int jn = 0; jn < 16; ++jn) {
      *reinterpret_cast<float2*>(&sm.merge_o[warp][r0][jn * 8 + 2 * t]) = make_float2(o[jn][0], o[jn][1]);
      *reinterpret_cast<float2*>(&sm.merge_o[warp][r1][jn * 8 + 2 * t]) = make_float2(o[jn][2], o[jn][3]);
    }
    consumer_barrier();
    const int d = threadIdx.x;  // one head dimension per consumer thread
    bool stored_partial = false;
    for (int r = 0; r < mrows; ++r) {
      const int len = is.lens[r / gqa];
      const int row_chunks = chunk_count(len);
      if (chunk >= row_chunks) continue;  // this row ends before the chunk
      float big = -INFINITY;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) big = fmaxf(big, sm.merge_m[w][r]);
      float acc = 0.f, total = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) {
        const float mw = sm.merge_m[w][r];
        const float f = mw == -INFINITY ? 0.f : fast_exp2(mw - big);
        acc = fmaf(sm.merge_o[w][r][d], f, acc);
        total = fmaf(sm.merge_l[w][r], f, total);
      }
      const int64_t qrow = row_start + r / gqa;
      const int qhead = kv_head * gqa + r % gqa;
      if (row_chunks == 1) {
        static_cast<T*>(a.out)[(qrow * a.q_heads + qhead) * kHeadDim + d] = Elem<T>::from_float(acc / total);
      } else {
        float* part = ws.partials + ((qrow * a.q_heads + qhead) * ws.max_chunks + chunk) * kPartialStride;
        part[d] = acc;
        if (d == 0) { part[kHeadDim] = big; part[kHeadDim + 1] = total; }
        stored_partial = true;
      }
    }
    // ---- the CTA that stores a group's last partial merges its chunks in chunk order ----
    if (group_chunks > 1) {
      (void)stored_partial;
      __threadfence();
      consumer_barrier();
      if (threadIdx.x == 0) {
        const unsigned prior = atomicAdd(&ws.counters[static_cast<int64_t>(row_start) * a.kv_heads + kv_head], 1u);
        sm.last_flag = prior == static_cast<unsigned>(group_chunks - 1);
      }
      consumer_barrier();
      if (sm.last_flag) {
        __threadfence();
        for (int r = 0; r < mrows; ++r) {
          const int row_chunks = chunk_count(is.lens[r / gqa]);
          if (row_chunks < 2) continue;
          const int64_t qrow = row_start + r / gqa;
          const int qhead = kv_head * gqa + r % gqa;
          const float* part = ws.partials + ((qrow * a.q_heads + qhead) * ws.max_chunks) * kPartialStride;
          float big = -INFINITY;
          for (int c = 0; c < row_chunks; ++c) big = fmaxf(big, __ldcg(part + c * kPartialStride + kHeadDim));
          float acc = 0.f, total = 0.f;
          for (int c = 0; c < row_chunks; ++c) {
            const float mc = __ldcg(part + c * kPartialStride + kHeadDim);
            const float f = mc == -INFINITY ? 0.f : fast_exp2(mc - big);
            acc = fmaf(__ldcg(part + c * kPartialStride + d), f, acc);
            total = fmaf(__ldcg(part + c * kPartialStride + kHeadDim + 1), f, total);
          }
          static_cast<T*>(a.out)[(qrow * a.q_heads + qhead) * kHeadDim + d] = Elem<T>::from_float(acc / total);
        }
      }
    }
    consumer_barrier();  // merge buffers and the item slot are free again
    if (lane == 0) mbar_arrive(smem_u32(&sm.item_empty[slot]));
  }
}

// ---- host side ----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
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
int make_page_map(CUtensorMap* map, const void* base, const AttentionArgs& a) {
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

int gqa_cap(const AttentionArgs& a) { return 16 / (a.q_heads / a.kv_heads); }

}  // namespace

bool attention_sm100_supported(const AttentionArgs& a) {
  if (a.dtype != RLT_BF16 && a.dtype != RLT_F16) return false;
  if (a.head_dim != kHeadDim || a.block_size != kPage) return false;
  if (a.kv_heads <= 0 || a.q_heads % a.kv_heads != 0) return false;
  const int gqa = a.q_heads / a.kv_heads;
  if (gqa != 1 && gqa != 2 && gqa != 4 && gqa != 8 && gqa != 16) return false;
  if (a.kv_heads > 32767) return false;
  if (static_cast<long long>(a.table_width) * a.block_size > (1 << 26)) return false;
  if (a.token_stride < static_cast<int64_t>(a.kv_heads) * kHeadDim) return false;
  if ((a.token_stride * 2) % 16 != 0 || (a.block_stride * 2) % 16 != 0) return false;
  if (a.block_stride < a.token_stride * kPage) return false;
  if (!aligned16(a.key_cache) || !aligned16(a.value_cache)) return false;
  if ((reinterpret_cast<uintptr_t>(a.q) & 3u) != 0) return false;
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
  out4[0] = h.item_count; out4[1] = h.next_item; out4[2] = h.error; out4[3] = h.plan_done;
  return RLT_OK;
}

int launch_attention_sm100(const AttentionArgs& a, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  const Layout l = make_layout(a.rows, a.q_heads, a.kv_heads, a.block_size, a.table_width);
  if (workspace == nullptr || workspace_bytes < l.total || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) {
    set_last_error_text("verify_attention: workspace missing, misaligned or too small");
    return RLT_ERR_WORKSPACE;
  }
  DeviceInfo info;
  int status = current_device_info(&info);
  if (status != RLT_OK) return status;
  char* base = static_cast<char*>(workspace);
  Workspace ws;
  ws.header = reinterpret_cast<Header*>(base + l.header);
  ws.row_len = reinterpret_cast<int*>(base + l.row_len);
  ws.row_table = reinterpret_cast<int*>(base + l.row_table);
  ws.link = reinterpret_cast<int*>(base + l.link);
  ws.counters = reinterpret_cast<unsigned*>(base + l.counters);
  ws.items = reinterpret_cast<Item*>(base + l.items);
  ws.partials = reinterpret_cast<float*>(base + l.partials);
  ws.max_chunks = l.max_chunks;

  CUtensorMap k_map, v_map;
  status = make_page_map(&k_map, a.key_cache, a);
  if (status != RLT_OK) return status;
  status = make_page_map(&v_map, a.value_cache, a);
  if (status != RLT_OK) return status;

  RLT_CUDA_TRY(cudaMemsetAsync(ws.header, 0, sizeof(Header), stream));
  const int plan_ctas = (a.rows + kPlanWarps - 1) / kPlanWarps;
  const int cap = gqa_cap(a);
  if (a.dtype == RLT_BF16)
    plan_kernel<__nv_bfloat16><<<plan_ctas, kPlanWarps * 32, 0, stream>>>(a, ws, cap);
  else
    plan_kernel<__half><<<plan_ctas, kPlanWarps * 32, 0, stream>>>(a, ws, cap);
  status = launch_status("plan_kernel");
  if (status != RLT_OK) return status;

  const size_t smem = sizeof(SharedStorage) + 1024;
  const float scale_log2 = static_cast<float>(1.4426950408889634 / sqrt(static_cast<double>(kHeadDim)));
  const int grid = info.sm_count * 2;
  if (a.dtype == RLT_BF16) {
    RLT_CUDA_TRY(cudaFuncSetAttribute(verify_attention_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
    RLT_CUDA_TRY(cudaFuncSetAttribute(verify_attention_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                      cudaSharedmemCarveoutMaxShared));
    verify_attention_kernel<true><<<grid, kThreads, smem, stream>>>(k_map, v_map, a, ws, scale_log2);
  } else {
    RLT_CUDA_TRY(cudaFuncSetAttribute(verify_attention_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
    RLT_CUDA_TRY(cudaFuncSetAttribute(verify_attention_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                      cudaSharedmemCarveoutMaxShared));
    verify_attention_kernel<false><<<grid, kThreads, smem, stream>>>(k_map, v_map, a, ws, scale_log2);
  }
  return launch_status("verify_attention_kernel");
}

}  // namespace rlt
