// Acceptance sampler of the verify step: row argmax, greedy prefix acceptance with the
// device state update, token draws with explicit uniforms and rejection sampling with
// residual resampling.
//
// All of these are streaming reductions over [rows, vocab] logits (HBM-bound: rows * vocab *
// sizeof(T) bytes, a few flops per byte).  Argmax is exact and order independent (a packed
// (value, lowest index) key reduced with max).  The probabilistic kernels use the canonical
// arithmetic of include/rlt_canonical.h — an exp built from IEEE fused multiply-adds and
// 2^-40 fixed-point integer sums — so their results are identical to the CPU oracle's for
// any thread count or reduction shape.
#include "common.cuh"

#include "../../include/rlt_canonical.h"

namespace rlt {
namespace {

constexpr int kArgmaxThreads = 512;
constexpr int kSampleThreads = 1024;

// ---- packed argmax key ------------------------------------------------------------------
// Larger key = better candidate: NaN above every number, then by value (-0 == +0), then the
// LOWER index.  max() over keys therefore reproduces torch.argmax.
__device__ __forceinline__ unsigned long long argmax_key(float x, int index) {
  uint32_t bits;
  if (x != x) {
    bits = 0xffffffffu;
  } else {
    if (x == 0.0f) x = 0.0f;  // -0 -> +0
    bits = __float_as_uint(x);
    bits = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
  }
  return (static_cast<unsigned long long>(bits) << 32) | (0xffffffffu - static_cast<uint32_t>(index));
}
__device__ __forceinline__ int key_index(unsigned long long key) {
  return static_cast<int>(0xffffffffu - static_cast<uint32_t>(key & 0xffffffffu));
}

__device__ __forceinline__ unsigned long long warp_max(unsigned long long v) {
#pragma unroll
  for (int x = 16; x > 0; x >>= 1) {
    const unsigned long long o = __shfl_xor_sync(0xffffffffu, v, x);
    v = o > v ? o : v;
  }
  return v;
}
__device__ __forceinline__ unsigned long long warp_sum(unsigned long long v) {
#pragma unroll
  for (int x = 16; x > 0; x >>= 1) v += __shfl_xor_sync(0xffffffffu, v, x);
  return v;
}

// Block-wide reductions for kThreads threads; every thread receives the result.
template <int kThreads>
__device__ __forceinline__ unsigned long long block_max(unsigned long long v, unsigned long long* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  v = lane < kThreads / 32 ? scratch[lane] : 0ull;
  return warp_max(v);
}
template <int kThreads>
__device__ __forceinline__ unsigned long long block_sum(unsigned long long v, unsigned long long* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  v = lane < kThreads / 32 ? scratch[lane] : 0ull;
  return warp_sum(v);
}

// Packed (value, lowest index) maximum of one row by the whole CTA.  16-byte loads when the row
// allows them, four in flight per thread (a row is only a few hundred KB: latency, not issue
// rate, decides how fast one CTA can stream it).
// kPlain: `row` may point to shared memory (a staged row), so no global-only load forms.
template <typename T, int kThreads, bool kPlain = false>
__device__ __forceinline__ unsigned long long block_max_key(const T* __restrict__ row, int vocab,
                                                           unsigned long long* scratch) {
  constexpr int kVec = 16 / sizeof(T);
  constexpr int kDepth = 4;
  unsigned long long best = 0ull;
  if ((reinterpret_cast<uintptr_t>(row) & 15u) == 0 && vocab % kVec == 0) {
    const uint4* rv = reinterpret_cast<const uint4*>(row);
    const int nvec = vocab / kVec;
    for (int base = threadIdx.x; base < nvec; base += kThreads * kDepth) {
      uint4 raw[kDepth];
#pragma unroll
      for (int k = 0; k < kDepth; ++k) {
        const int i = base + k * kThreads;
        if (i < nvec) raw[k] = kPlain ? rv[i] : __ldcs(rv + i);
      }
#pragma unroll
      for (int k = 0; k < kDepth; ++k) {
        const int i = base + k * kThreads;
        if (i < nvec) {
          const T* e = reinterpret_cast<const T*>(&raw[k]);
#pragma unroll
          for (int j = 0; j < kVec; ++j) {
            const unsigned long long key = argmax_key(Elem<T>::to_float(e[j]), i * kVec + j);
            best = key > best ? key : best;
          }
        }
      }
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += kThreads) {
      const unsigned long long key = argmax_key(Elem<T>::to_float(row[i]), i);
      best = key > best ? key : best;
    }
  }
  return block_max<kThreads>(best, scratch);
}

template <typename T, int kThreads>
__device__ __forceinline__ int block_argmax(const T* __restrict__ row, int vocab, unsigned long long* scratch) {
  return key_index(block_max_key<T, kThreads>(row, vocab, scratch));
}

template <typename T>
__global__ void __launch_bounds__(kArgmaxThreads)
argmax_rows_kernel(const T* __restrict__ logits, int64_t row_stride, int vocab, int64_t* __restrict__ targets) {
  __shared__ unsigned long long scratch[32];
  const int index = block_argmax<T, kArgmaxThreads>(logits + static_cast<int64_t>(blockIdx.x) * row_stride, vocab, scratch);
  if (threadIdx.x == 0) targets[blockIdx.x] = index;
}

// Rows of request i: the span cu_rows[i] .. cu_rows[i+1]-1, of which only the first
// row_counts[i] are real when row_counts is given (a fixed-shape round pads every request to the
// same span).  Zero rows: the request is left alone (accepted 0, next position = its start, no
// slot update).
__device__ __forceinline__ int request_rows(const int32_t* __restrict__ cu_rows, const int32_t* __restrict__ row_counts,
                                            int i, int* first, int* span) {
  *first = cu_rows[i];
  *span = cu_rows[i + 1] - cu_rows[i];
  const int c = row_counts != nullptr ? min(row_counts[i], *span) : *span;
  return c > 0 ? c : 0;
}

// One thread per request: matching prefix, next token / position, slot update, wire buffer.
__global__ void greedy_finish_kernel(const int32_t* __restrict__ cu_rows, int n, int rows,
                                     const int32_t* __restrict__ row_counts,
                                     const int64_t* __restrict__ tokens, int tokens_width,
                                     const int64_t* __restrict__ starts, const int64_t* __restrict__ slots,
                                     int64_t* __restrict__ slot_values, int64_t* __restrict__ result) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int a, span;
  const int c = request_rows(cu_rows, row_counts, i, &a, &span);
  for (int j = c; j < span; ++j) result[a + j] = -1;  // padding rows carry no target
  if (c == 0) {
    result[rows + i] = 0;
    result[rows + n + i] = starts[i];
    return;
  }
  const int64_t* tok = tokens + static_cast<int64_t>(i) * tokens_width;
  int accepted = 0;
  while (accepted < c - 1 && tok[accepted + 1] == result[a + accepted]) ++accepted;
  const int64_t next_token = result[a + accepted];
  const int64_t next_pos = starts[i] + accepted + 1;
  result[rows + i] = accepted;
  result[rows + n + i] = next_pos;
  if (slots != nullptr && slot_values != nullptr) {
    slot_values[2 * slots[i]] = next_token;
    slot_values[2 * slots[i] + 1] = next_pos;
  }
}

// ---- canonical distributions ----------------------------------------------------------
// Support of a row after top-k / top-p: the prefix of the ranking (scaled logit descending,
// token index ascending) that ends at (key, limit); see rlt_in_support.
struct Cut {
  uint32_t key;
  int limit;
};
__device__ __forceinline__ Cut whole_row() { return Cut{0u, 0x7fffffff}; }

struct RowNorm {
  float m;   // max of logits / T
  float z;   // normaliser over the support (from the fixed-point sum)
  int ok;    // 0: NaN / +inf / all -inf
  Cut cut;   // support of the distribution
};

template <typename T>
__device__ __forceinline__ float scaled_logit(const T* row, int v, float temperature) {
  return RLT_DIV(Elem<T>::to_float(row[v]), temperature);
}

// max of row / temperature.  Division by a positive temperature is monotonic, so
// max_v (x_v / T) == (max_v x_v) / T exactly: the pass is a plain maximum over the raw logits
// (NaN counts as the maximum and is then reported), one division at the end.
template <typename T, int kThreads, bool kPlain = false>
__device__ __forceinline__ RowNorm block_row_max(const T* __restrict__ row, int vocab, float temperature,
                                                 unsigned long long* scratch) {
  const unsigned long long best = block_max_key<T, kThreads, kPlain>(row, vocab, scratch);
  RowNorm n;
  uint32_t bits = static_cast<uint32_t>(best >> 32);
  bits = (bits & 0x80000000u) ? (bits & 0x7fffffffu) : ~bits;
  const float raw_max = __uint_as_float(bits);
  n.m = RLT_DIV(raw_max, temperature);
  n.ok = best != 0ull && raw_max == raw_max && n.m != INFINITY && n.m != -INFINITY;
  n.z = 0.0f;
  n.cut = whole_row();
  return n;
}

// Normaliser of softmax(row / temperature) over the whole row.
template <typename T, int kThreads, bool kPlain = false>
__device__ __forceinline__ float block_full_sum(const T* __restrict__ row, int vocab, float temperature, float m,
                                                unsigned long long* scratch) {
  unsigned long long zfix = 0ull;
  constexpr int kVec = 16 / sizeof(T);
  if ((reinterpret_cast<uintptr_t>(row) & 15u) == 0 && vocab % kVec == 0) {
    const uint4* rv = reinterpret_cast<const uint4*>(row);
    const int nvec = vocab / kVec;
    for (int base = threadIdx.x; base < nvec; base += kThreads * 2) {
      uint4 raw[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int i = base + k * kThreads;
        if (i < nvec) raw[k] = kPlain ? rv[i] : __ldg(rv + i);
      }
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int i = base + k * kThreads;
        if (i < nvec) {
          const T* e = reinterpret_cast<const T*>(&raw[k]);
#pragma unroll
          for (int j = 0; j < kVec; ++j)
            zfix += rlt_fix_weight(rlt_expf(RLT_SUB(RLT_DIV(Elem<T>::to_float(e[j]), temperature), m)));
        }
      }
    }
  } else {
    for (int v = threadIdx.x; v < vocab; v += kThreads)
      zfix += rlt_fix_weight(rlt_expf(RLT_SUB(scaled_logit(row, v, temperature), m)));
  }
  return rlt_fix_to_float(block_sum<kThreads>(zfix, scratch));
}

// Normaliser over the tokens inside `cut`.
template <typename T, int kThreads>
__device__ __forceinline__ float block_cut_sum(const T* __restrict__ row, int vocab, float temperature, float m,
                                               Cut cut, unsigned long long* scratch) {
  unsigned long long zfix = 0ull;
  for (int v = threadIdx.x; v < vocab; v += kThreads) {
    const float t = scaled_logit(row, v, temperature);
    if (rlt_in_support(rlt_order_key(t), v, cut.key, cut.limit)) zfix += rlt_fix_weight(rlt_expf(RLT_SUB(t, m)));
  }
  return rlt_fix_to_float(block_sum<kThreads>(zfix, scratch));
}

// ---- top-k / top-p: radix select over the ranking ------------------------------------------
// Both filters keep the ranks whose exclusive prefix WEIGHT is <= a limit: weight 1 per token
// and limit k - 1 for top-k, the fixed-point probability mass and rlt_top_p_limit for top-p.
// The cut is found digit by digit (four 8-bit digits of the order key, most significant first):
// a histogram of weight per digit over the tokens that match the digits chosen so far, then the
// digit in which the running weight, accumulated from the top, first exceeds the limit.  Equal
// keys have equal weights, so inside the final tie group the kept count follows by division and
// the cut index is the n-th matching token in index order.  A row is a few hundred KB and stays
// in L2 between the passes.
struct SelectScratch {
  unsigned long long mass[256];
  unsigned int count[256];
  unsigned long long above;
  int digit;
  int found;
  int warp_counts[32];
};

// One shared-memory atomic per distinct digit in the warp: lanes with the same digit find each
// other with match.any and add their weights with two integer warp reductions (a weight is below
// 2^41: 20 low and 21 high bits, so 32 of them cannot overflow a 32-bit partial sum).  The leading
// byte of the key has only a few populated values, so plain per-lane atomics would serialise.
template <bool kByMass>
__device__ __forceinline__ void hist_add(SelectScratch& h, int bucket, unsigned long long w, bool valid) {
  const int lane = threadIdx.x & 31;
  const unsigned peers = __match_any_sync(0xffffffffu, valid ? bucket : 0x7fff);
  const bool leader = valid && lane == __ffs(peers) - 1;
  if (kByMass) {
    const unsigned low = __reduce_add_sync(peers, static_cast<unsigned>(w & 0xfffffu));
    const unsigned high = __reduce_add_sync(peers, static_cast<unsigned>(w >> 20));
    if (leader) atomicAdd(&h.mass[bucket], (static_cast<unsigned long long>(high) << 20) + low);
  }
  if (leader) atomicAdd(&h.count[bucket], static_cast<unsigned int>(__popc(peers)));
}

// Index of the n-th (1-based) token in ascending index order with order key `key` inside `outer`.
template <typename T, int kThreads>
__device__ __forceinline__ int block_nth_index(const T* __restrict__ row, int vocab, float temperature,
                                               uint32_t key, Cut outer, unsigned int n, SelectScratch& h) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) h.found = 0x7fffffff;
  unsigned int running = 0;
  for (int base = 0; base < vocab; base += kThreads) {
    const int v = base + static_cast<int>(threadIdx.x);
    bool flag = false;
    if (v < vocab) {
      const uint32_t k = rlt_order_key(scaled_logit(row, v, temperature));
      flag = k == key && rlt_in_support(k, v, outer.key, outer.limit);
    }
    const unsigned ballot = __ballot_sync(0xffffffffu, flag);
    __syncthreads();
    if (lane == 0) h.warp_counts[warp] = __popc(ballot);
    __syncthreads();
    unsigned int before = running, total = 0;
    for (int w = 0; w < kThreads / 32; ++w) {
      const unsigned int c = h.warp_counts[w];
      if (w < warp) before += c;
      total += c;
    }
    if (flag && before + __popc(ballot & ((1u << lane) - 1u)) + 1u == n) h.found = v;
    running += total;
    if (running >= n) break;  // uniform: every thread computes the same totals
  }
  __syncthreads();
  return h.found;
}

template <typename T, int kThreads, bool kByMass>
__device__ __forceinline__ Cut block_select(const T* __restrict__ row, int vocab, float temperature, float m,
                                            float inv, Cut outer, unsigned long long limit, SelectScratch& h) {
  uint32_t prefix = 0u;
  unsigned long long above = 0ull;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    __syncthreads();
    for (int i = threadIdx.x; i < 256; i += kThreads) { h.mass[i] = 0ull; h.count[i] = 0u; }
    __syncthreads();
    for (int base = 0; base < vocab; base += kThreads) {
      const int v = base + static_cast<int>(threadIdx.x);
      bool valid = false;
      int bucket = 0;
      unsigned long long w = 0ull;
      if (v < vocab) {
        const float t = scaled_logit(row, v, temperature);
        const uint32_t key = rlt_order_key(t);
        valid = rlt_in_support(key, v, outer.key, outer.limit) &&
                (pass == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8)));
        bucket = static_cast<int>((key >> shift) & 255u);
        if (kByMass && valid) w = rlt_fix_weight(rlt_draw_mass(rlt_expf(RLT_SUB(t, m)), inv));
      }
      hist_add<kByMass>(h, bucket, w, valid);
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // lane l scans digits 255 - 8l down to 248 - 8l
      const int lane = threadIdx.x, hi = 255 - 8 * lane;
      unsigned long long local = 0ull;
#pragma unroll
      for (int j = 0; j < 8; ++j) local += kByMass ? h.mass[hi - j] : static_cast<unsigned long long>(h.count[hi - j]);
      unsigned long long inc = local;
#pragma unroll
      for (int x = 1; x < 32; x <<= 1) {
        const unsigned long long o = __shfl_up_sync(0xffffffffu, inc, x);
        if (lane >= x) inc += o;
      }
      const unsigned crossing = __ballot_sync(0xffffffffu, above + inc > limit);
      if (crossing == 0u) {
        if (lane == 0) h.digit = -1;
      } else if (lane == __ffs(crossing) - 1) {
        unsigned long long acc = above + inc - local;
        int digit = hi;
        for (int j = 0; j < 8; ++j) {
          const unsigned long long wd = kByMass ? h.mass[hi - j] : static_cast<unsigned long long>(h.count[hi - j]);
          digit = hi - j;
          if (acc + wd > limit) break;
          acc += wd;
        }
        h.digit = digit;
        h.above = acc;
      }
    }
    __syncthreads();
    if (h.digit < 0) return outer;  // the whole of `outer` stays (its weight never exceeds the limit)
    prefix |= static_cast<uint32_t>(h.digit) << shift;
    above = h.above;
  }
  const unsigned int ties = h.count[prefix & 255u];
  const unsigned long long each = kByMass ? h.mass[prefix & 255u] / ties : 1ull;
  const unsigned long long keep = (limit - above) / each + 1ull;
  __syncthreads();
  if (keep >= ties) return Cut{prefix, prefix == outer.key ? outer.limit : 0x7fffffff};
  return Cut{prefix, block_nth_index<T, kThreads>(row, vocab, temperature, prefix, outer,
                                                  static_cast<unsigned int>(keep), h)};
}

// max, support and normaliser of the distribution Sampler.probabilities builds for one row
// (vllm_rlt/worker/sampler.py:37-55): softmax(row / T) restricted to top-k, then to top-p.
// top_k <= 0 or >= vocab and top_p >= 1 switch the filters off.
template <typename T, int kThreads, bool kPlain = false>
__device__ __forceinline__ RowNorm block_normalise(const T* __restrict__ row, int vocab, float temperature,
                                                   int top_k, float top_p, unsigned long long* scratch,
                                                   SelectScratch& h) {
  RowNorm n = block_row_max<T, kThreads, kPlain>(row, vocab, temperature, scratch);
  if (!n.ok) return n;
  const bool use_k = top_k > 0 && top_k < vocab, use_p = top_p < 1.0f;
  if (use_k) {
    n.cut = block_select<T, kThreads, false>(row, vocab, temperature, n.m, 0.0f, whole_row(),
                                             static_cast<unsigned long long>(top_k - 1), h);
    n.z = block_cut_sum<T, kThreads>(row, vocab, temperature, n.m, n.cut, scratch);
  } else {
    n.z = block_full_sum<T, kThreads, kPlain>(row, vocab, temperature, n.m, scratch);
  }
  if (use_p) {
    const Cut outer = n.cut;
    n.cut = block_select<T, kThreads, true>(row, vocab, temperature, n.m, RLT_DIV(1.0f, n.z), outer,
                                            rlt_top_p_limit(top_p), h);
    if (n.cut.key != outer.key || n.cut.limit != outer.limit)
      n.z = block_cut_sum<T, kThreads>(row, vocab, temperature, n.m, n.cut, scratch);
  }
  return n;
}

// A row copied to shared memory as fp32 (exact for all three storage types).  The filters make a
// dozen passes over a row; from shared memory a pass costs a few microseconds instead of one L2
// round trip per element and thread.  Used when the caller passes filters and the row fits.
template <typename T, int kThreads>
__device__ __forceinline__ const float* stage_row(const T* __restrict__ row, int vocab, float* staged) {
  for (int v = threadIdx.x; v < vocab; v += kThreads) staged[v] = Elem<T>::to_float(row[v]);
  __syncthreads();
  return staged;
}

// exp(t_v - max) for a token of the support, 0 outside it.
template <typename T>
__device__ __forceinline__ float exp_at(const T* row, int v, float temperature, const RowNorm& n) {
  const float t = scaled_logit(row, v, temperature);
  if (!rlt_in_support(rlt_order_key(t), v, n.cut.key, n.cut.limit)) return 0.0f;
  return rlt_expf(RLT_SUB(t, n.m));
}

template <typename T>
__device__ __forceinline__ float prob_at(const T* row, int v, float temperature, const RowNorm& n) {
  return RLT_DIV(exp_at(row, v, temperature, n), n.z);
}

// Fixed-point draw weight of token v: p[v] (plain) or max(p[v] - q[v], 0) (residual), in the
// division-free form of rlt_canonical.h; `inv` is 1/zp or 1/(zp*zq).
template <typename T>
__device__ __forceinline__ unsigned long long draw_weight(const T* prow, const RowNorm& pn, const T* qrow,
                                                          const RowNorm& qn, bool residual, int v,
                                                          float temperature, float inv) {
  const float ep = exp_at(prow, v, temperature, pn);
  if (!residual) return rlt_fix_weight(rlt_draw_mass(ep, inv));
  return rlt_fix_weight(rlt_residual_mass(ep, exp_at(qrow, v, temperature, qn), pn.z, qn.z, inv));
}

// Inverse-CDF draw over fixed-point weights in ascending token index; -1 if the mass is zero.
// Thread t owns the contiguous tokens [t*span, (t+1)*span); its weights stay in registers
// between the sum and the search when the span is small enough.
template <typename T, int kThreads>
__device__ __forceinline__ int block_draw(const T* __restrict__ prow, const RowNorm& pn,
                                          const T* __restrict__ qrow, const RowNorm& qn, bool residual,
                                          int vocab, float temperature, float u, unsigned long long* scratch,
                                          int* token_slot) {
  const float inv = residual ? RLT_DIV(1.0f, RLT_MUL(pn.z, qn.z)) : RLT_DIV(1.0f, pn.z);
  const int span = (vocab + kThreads - 1) / kThreads;
  const int begin = min(static_cast<int>(threadIdx.x) * span, vocab), end = min(begin + span, vocab);
  unsigned long long local = 0ull;
  for (int v = begin; v < end; ++v) local += draw_weight(prow, pn, qrow, qn, residual, v, temperature, inv);
  // exclusive scan over threads: inclusive warp scan, then warp totals
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned long long inc = local;
#pragma unroll
  for (int x = 1; x < 32; x <<= 1) {
    const unsigned long long o = __shfl_up_sync(0xffffffffu, inc, x);
    if (lane >= x) inc += o;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = inc;
  if (threadIdx.x == 0) *token_slot = -1;
  __syncthreads();
  unsigned long long before = 0ull, total = 0ull;
  for (int w = 0; w < kThreads / 32; ++w) {
    const unsigned long long s = scratch[w];
    if (w < warp) before += s;
    total += s;
  }
  if (total != 0ull) {
    const unsigned long long threshold = rlt_draw_threshold(u, total);
    unsigned long long prefix = before + inc - local;
    if (prefix <= threshold && threshold < prefix + local) {
      for (int v = begin; v < end; ++v) {
        prefix += draw_weight(prow, pn, qrow, qn, residual, v, temperature, inv);
        if (prefix > threshold) { *token_slot = v; break; }
      }
    }
  }
  __syncthreads();
  return *token_slot;
}

template <typename T, bool kStaged>
__global__ void __launch_bounds__(kSampleThreads)
sample_rows_kernel(const T* __restrict__ logits, int64_t row_stride, int vocab,
                   const float* __restrict__ temperature, const int32_t* __restrict__ top_k,
                   const float* __restrict__ top_p, const float* __restrict__ uniforms,
                   int64_t* __restrict__ tokens, int32_t* __restrict__ status) {
  __shared__ unsigned long long scratch[32];
  __shared__ SelectScratch select;
  __shared__ int token_slot;
  const int r = blockIdx.x;
  const T* row = logits + static_cast<int64_t>(r) * row_stride;
  const float temp = temperature[r];
  int st = RLT_ROW_OK;
  int token = -1;
  if (temp == 0.0f) {
    token = block_argmax<T, kSampleThreads>(row, vocab, scratch);
  } else if constexpr (kStaged) {
    extern __shared__ __align__(16) float staged[];
    const float* frow = stage_row<T, kSampleThreads>(row, vocab, staged);
    const RowNorm n = block_normalise<float, kSampleThreads, true>(frow, vocab, temp, top_k ? top_k[r] : -1,
                                                                   top_p ? top_p[r] : 1.0f, scratch, select);
    if (!n.ok) {
      st = RLT_ROW_BAD_LOGITS;
    } else {
      token = block_draw<float, kSampleThreads>(frow, n, frow, n, false, vocab, temp, uniforms[r], scratch, &token_slot);
      if (token < 0) st = RLT_ROW_INVALID_RESIDUAL;
    }
  } else {
    const RowNorm n = block_normalise<T, kSampleThreads>(row, vocab, temp, top_k ? top_k[r] : -1,
                                                         top_p ? top_p[r] : 1.0f, scratch, select);
    if (!n.ok) {
      st = RLT_ROW_BAD_LOGITS;
    } else {
      token = block_draw<T, kSampleThreads>(row, n, row, n, false, vocab, temp, uniforms[r], scratch, &token_slot);
      if (token < 0) st = RLT_ROW_INVALID_RESIDUAL;
    }
  }
  if (threadIdx.x == 0) { tokens[r] = token; status[r] = st; }
}

// Sampler.probabilities for every row: fp32 [rows, vocab], zero outside the support.
template <typename T, bool kStaged>
__global__ void __launch_bounds__(kSampleThreads)
probabilities_kernel(const T* __restrict__ logits, int64_t row_stride, int vocab,
                     const float* __restrict__ temperature, const int32_t* __restrict__ top_k,
                     const float* __restrict__ top_p, float* __restrict__ probs, int32_t* __restrict__ status) {
  __shared__ unsigned long long scratch[32];
  __shared__ SelectScratch select;
  const int r = blockIdx.x;
  const T* row = logits + static_cast<int64_t>(r) * row_stride;
  float* out = probs + static_cast<int64_t>(r) * vocab;
  const float temp = temperature[r];
  RowNorm n;
  n.ok = 0;
  if constexpr (kStaged) {
    extern __shared__ __align__(16) float staged[];
    const float* frow = stage_row<T, kSampleThreads>(row, vocab, staged);
    if (temp > 0.0f)
      n = block_normalise<float, kSampleThreads, true>(frow, vocab, temp, top_k ? top_k[r] : -1,
                                                       top_p ? top_p[r] : 1.0f, scratch, select);
    for (int v = threadIdx.x; v < vocab; v += kSampleThreads) out[v] = n.ok ? prob_at(frow, v, temp, n) : 0.0f;
  } else {
    if (temp > 0.0f)
      n = block_normalise<T, kSampleThreads>(row, vocab, temp, top_k ? top_k[r] : -1, top_p ? top_p[r] : 1.0f,
                                             scratch, select);
    for (int v = threadIdx.x; v < vocab; v += kSampleThreads) out[v] = n.ok ? prob_at(row, v, temp, n) : 0.0f;
  }
  if (threadIdx.x == 0) status[r] = n.ok ? RLT_ROW_OK : RLT_ROW_BAD_LOGITS;
}

// ---- rejection sampling in two launches -------------------------------------------------
// 1. row_stats_kernel, one CTA per (verification row, target | draft): everything about a
//    row that does not depend on earlier accept decisions — max, normaliser and the
//    probability of the row's draft token (or the argmax for a greedy request) — so the
//    streaming over [rows, vocab] runs at full width instead of request by request.
// 2. decide_kernel, one CTA per request: the sequential accept walk over those few numbers,
//    then the single residual or bonus draw the request needs.
struct RowStats {
  float m;
  float z;
  float prob;  // probability of the row's draft token under this row's distribution
  int info;    // bit 0: distribution valid; greedy requests: argmax index << 1
  Cut cut;     // support after top-k / top-p
};

constexpr int kStatsThreads = 512;

__device__ __forceinline__ int request_of_row(const int32_t* cu_rows, int n, int row) {
  int lo = 0, hi = n - 1;  // last i with cu_rows[i] <= row
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_rows[mid] <= row) lo = mid; else hi = mid - 1;
  }
  return lo;
}

template <typename T, int kThreads, bool kStaged>
__global__ void __launch_bounds__(kThreads)
row_stats_kernel(const T* __restrict__ target_logits, const T* __restrict__ draft_logits, int64_t row_stride,
                 int vocab, const int32_t* __restrict__ cu_rows, int n, const int32_t* __restrict__ row_counts,
                 const int64_t* __restrict__ tokens, int tokens_width, const float* __restrict__ temperature,
                 const int32_t* __restrict__ top_k, const float* __restrict__ top_p, RowStats* __restrict__ stats) {
  __shared__ unsigned long long scratch[32];
  __shared__ SelectScratch select;
  const int row = blockIdx.x, side = blockIdx.y;  // side 0: target, 1: draft
  const int i = request_of_row(cu_rows, n, row);
  int first, span;
  const int count = request_rows(cu_rows, row_counts, i, &first, &span);
  const int j = row - first;
  if (j >= count) return;  // a padding row: nothing reads its statistics
  const float temp = temperature[i];
  RowStats out = {0.0f, 0.0f, 0.0f, 0, whole_row()};
  if (temp == 0.0f) {
    if (side == 1) return;
    out.info = block_argmax<T, kThreads>(target_logits + static_cast<int64_t>(row) * row_stride, vocab, scratch) << 1;
  } else {
    if (side == 1 && j == count - 1) return;  // the bonus row has no draft distribution
    const T* logits = (side == 0 ? target_logits : draft_logits) + static_cast<int64_t>(row) * row_stride;
    RowNorm norm;
    if constexpr (kStaged) {
      extern __shared__ __align__(16) float staged[];
      norm = block_normalise<float, kThreads, true>(stage_row<T, kThreads>(logits, vocab, staged), vocab, temp,
                                                    top_k ? top_k[i] : -1, top_p ? top_p[i] : 1.0f, scratch, select);
    } else {
      norm = block_normalise<T, kThreads>(logits, vocab, temp, top_k ? top_k[i] : -1, top_p ? top_p[i] : 1.0f,
                                          scratch, select);
    }
    const int64_t d = j < count - 1 ? tokens[static_cast<int64_t>(i) * tokens_width + j + 1] : -1;
    out.m = norm.m;
    out.z = norm.z;
    out.info = norm.ok ? 1 : 0;
    out.cut = norm.cut;
    if (norm.ok && d >= 0 && d < vocab) out.prob = prob_at(logits, static_cast<int>(d), temp, norm);
  }
  if (threadIdx.x == 0) stats[2 * row + side] = out;
}

template <typename T>
__global__ void __launch_bounds__(kSampleThreads)
decide_kernel(const T* __restrict__ target_logits, const T* __restrict__ draft_logits, int64_t row_stride, int rows,
              int vocab, const int32_t* __restrict__ cu_rows, int n, const int32_t* __restrict__ row_counts,
              const int64_t* __restrict__ tokens, int tokens_width, const int64_t* __restrict__ starts,
              const float* __restrict__ temperature, const float* __restrict__ u_accept,
              const float* __restrict__ u_final, const int64_t* __restrict__ slots,
              int64_t* __restrict__ slot_values, const RowStats* __restrict__ stats,
              int64_t* __restrict__ result, int32_t* __restrict__ status) {
  __shared__ unsigned long long scratch[32];
  __shared__ int token_slot;
  const int i = blockIdx.x;
  int a, span;
  const int c = request_rows(cu_rows, row_counts, i, &a, &span);
  const int64_t* tok = tokens + static_cast<int64_t>(i) * tokens_width;
  const float temp = temperature[i];
  for (int j = threadIdx.x; j < span; j += kSampleThreads) result[a + j] = -1;
  if (c == 0) {  // no rows: the request is left alone
    if (threadIdx.x == 0) {
      result[rows + i] = 0;
      result[rows + n + i] = starts[i];
      status[i] = RLT_ROW_OK;
    }
    return;
  }
  __syncthreads();

  int accepted = 0, st = RLT_ROW_OK;
  int64_t final_token = -1;
  if (temp == 0.0f) {
    for (int j = 0; j < c; ++j) {
      const int target = stats[2 * (a + j)].info >> 1;
      if (threadIdx.x == 0) result[a + j] = target;
      final_token = target;
      if (j < c - 1 && tok[j + 1] == target) { ++accepted; continue; }
      break;
    }
  } else {
    int j = 0;
    for (; j < c - 1; ++j) {
      const RowStats ps = stats[2 * (a + j)], qs = stats[2 * (a + j) + 1];
      const int64_t d = tok[j + 1];
      if (!(ps.info & 1) || !(qs.info & 1) || d < 0 || d >= vocab) { st = RLT_ROW_BAD_LOGITS; break; }
      if (!(qs.prob > 0.0f)) { st = RLT_ROW_ZERO_PROPOSAL; break; }
      if (RLT_MUL(u_accept[a + j], qs.prob) < ps.prob) {
        if (threadIdx.x == 0) result[a + j] = d;
        ++accepted;
        continue;
      }
      const RowNorm pn = {ps.m, ps.z, 1, ps.cut}, qn = {qs.m, qs.z, 1, qs.cut};
      final_token = block_draw<T, kSampleThreads>(target_logits + static_cast<int64_t>(a + j) * row_stride, pn,
                                                  draft_logits + static_cast<int64_t>(a + j) * row_stride, qn, true,
                                                  vocab, temp, u_final[i], scratch, &token_slot);
      if (final_token < 0) st = RLT_ROW_INVALID_RESIDUAL;
      break;
    }
    if (st == RLT_ROW_OK && j == c - 1) {
      const RowStats ps = stats[2 * (a + c - 1)];
      if (!(ps.info & 1)) {
        st = RLT_ROW_BAD_LOGITS;
      } else {
        const RowNorm pn = {ps.m, ps.z, 1, ps.cut};
        const T* prow = target_logits + static_cast<int64_t>(a + c - 1) * row_stride;
        final_token = block_draw<T, kSampleThreads>(prow, pn, prow, pn, false, vocab, temp, u_final[i], scratch,
                                                    &token_slot);
        if (final_token < 0) st = RLT_ROW_INVALID_RESIDUAL;
      }
    }
  }
  if (threadIdx.x == 0) {
    if (temp != 0.0f && st == RLT_ROW_OK) result[a + accepted] = final_token;
    const int64_t next_pos = starts[i] + accepted + 1;
    result[rows + i] = accepted;
    result[rows + n + i] = next_pos;
    status[i] = st;
    // A failed request keeps its slot: the next round must not start from token -1.
    if (st == RLT_ROW_OK && slots != nullptr && slot_values != nullptr) {
      slot_values[2 * slots[i]] = final_token;
      slot_values[2 * slots[i] + 1] = next_pos;
    }
  }
}

// Filters were passed and an fp32 copy of a row fits beside the kernels' static shared memory.
bool stage_rows(const int32_t* top_k, const float* top_p, int vocab) {
  return (top_k != nullptr || top_p != nullptr) && static_cast<size_t>(vocab) * sizeof(float) <= 200u * 1024u;
}

int check_logits(const void* logits, int64_t row_stride, int rows, int vocab, int dtype) {
  RLT_REQUIRE(dtype_valid(dtype), "acceptance: logits must be float32, float16 or bfloat16");
  RLT_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "acceptance: invalid logits shape");
  RLT_REQUIRE(rows == 0 || logits != nullptr, "acceptance: null logits");
  return RLT_OK;
}

}  // namespace
}  // namespace rlt

extern "C" RLT_API int rlt_argmax_rows(const void* logits, int64_t row_stride, int rows, int vocab, int dtype,
                               int64_t* targets, rlt_stream_t stream) {
  using namespace rlt;
  int status = check_logits(logits, row_stride, rows, vocab, dtype);
  if (status != RLT_OK || rows == 0) return status;
  RLT_REQUIRE(targets != nullptr, "argmax_rows: null output");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  RLT_DISPATCH_DTYPE(dtype, T, (argmax_rows_kernel<T><<<rows, kArgmaxThreads, 0, s>>>(
                                   static_cast<const T*>(logits), row_stride, vocab, targets)));
  return launch_status("argmax_rows_kernel");
}

extern "C" RLT_API int rlt_accept_greedy(const void* logits, int64_t row_stride, int rows, int vocab, int dtype,
                                 const int32_t* cu_rows, int n, const int32_t* row_counts, const int64_t* tokens,
                                 int tokens_width, const int64_t* starts, const int64_t* slots,
                                 int64_t* slot_values, int64_t* result, rlt_stream_t stream) {
  using namespace rlt;
  int status = check_logits(logits, row_stride, rows, vocab, dtype);
  if (status != RLT_OK) return status;
  RLT_REQUIRE(n >= 0 && tokens_width >= 1, "accept_greedy: invalid request count or token width");
  if (n == 0 && rows == 0) return RLT_OK;
  RLT_REQUIRE(cu_rows && tokens && starts && result, "accept_greedy: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rows > 0) {
    RLT_DISPATCH_DTYPE(dtype, T, (argmax_rows_kernel<T><<<rows, kArgmaxThreads, 0, s>>>(
                                     static_cast<const T*>(logits), row_stride, vocab, result)));
    status = launch_status("argmax_rows_kernel");
    if (status != RLT_OK) return status;
  }
  if (n > 0) {
    greedy_finish_kernel<<<(n + 127) / 128, 128, 0, s>>>(cu_rows, n, rows, row_counts, tokens, tokens_width, starts,
                                                         slots, slot_values, result);
    status = launch_status("greedy_finish_kernel");
  }
  return status;
}

extern "C" RLT_API int rlt_sample_rows(const void* logits, int64_t row_stride, int rows, int vocab, int dtype,
                               const float* temperature, const int32_t* top_k, const float* top_p,
                               const float* uniforms, int64_t* tokens, int32_t* status_out, rlt_stream_t stream) {
  using namespace rlt;
  int status = check_logits(logits, row_stride, rows, vocab, dtype);
  if (status != RLT_OK || rows == 0) return status;
  RLT_REQUIRE(temperature && uniforms && tokens && status_out, "sample_rows: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (stage_rows(top_k, top_p, vocab)) {
    const size_t smem = static_cast<size_t>(vocab) * sizeof(float);
    RLT_DISPATCH_DTYPE(dtype, T, {
      auto kernel = sample_rows_kernel<T, true>;
      RLT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
      kernel<<<rows, kSampleThreads, smem, s>>>(static_cast<const T*>(logits), row_stride, vocab, temperature, top_k,
                                                top_p, uniforms, tokens, status_out);
    });
  } else {
    RLT_DISPATCH_DTYPE(dtype, T, (sample_rows_kernel<T, false><<<rows, kSampleThreads, 0, s>>>(
                                     static_cast<const T*>(logits), row_stride, vocab, temperature, top_k, top_p,
                                     uniforms, tokens, status_out)));
  }
  return launch_status("sample_rows_kernel");
}

extern "C" RLT_API int rlt_probabilities(const void* logits, int64_t row_stride, int rows, int vocab, int dtype,
                                         const float* temperature, const int32_t* top_k, const float* top_p,
                                         float* probs, int32_t* status_out, rlt_stream_t stream) {
  using namespace rlt;
  int status = check_logits(logits, row_stride, rows, vocab, dtype);
  if (status != RLT_OK || rows == 0) return status;
  RLT_REQUIRE(temperature && probs && status_out, "probabilities: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (stage_rows(top_k, top_p, vocab)) {
    const size_t smem = static_cast<size_t>(vocab) * sizeof(float);
    RLT_DISPATCH_DTYPE(dtype, T, {
      auto kernel = probabilities_kernel<T, true>;
      RLT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
      kernel<<<rows, kSampleThreads, smem, s>>>(static_cast<const T*>(logits), row_stride, vocab, temperature, top_k,
                                                top_p, probs, status_out);
    });
  } else {
    RLT_DISPATCH_DTYPE(dtype, T, (probabilities_kernel<T, false><<<rows, kSampleThreads, 0, s>>>(
                                     static_cast<const T*>(logits), row_stride, vocab, temperature, top_k, top_p,
                                     probs, status_out)));
  }
  return launch_status("probabilities_kernel");
}

namespace rlt {
namespace {
__global__ void round_uniforms_kernel(const int64_t* __restrict__ seeds, const int64_t* __restrict__ rounds, int n,
                                      int width, float* __restrict__ u_draft, float* __restrict__ u_accept,
                                      float* __restrict__ u_final) {
  const int x = blockIdx.x * blockDim.x + threadIdx.x;
  if (x >= n * (2 * width + 1)) return;
  const int i = x / (2 * width + 1), j = x % (2 * width + 1);
  const uint64_t seed = static_cast<uint64_t>(seeds[i]), round = static_cast<uint64_t>(rounds[i]);
  if (j < width) u_draft[i * width + j] = rlt_uniform(seed, round, RLT_STREAM_DRAFT, j);
  else if (j < 2 * width) u_accept[i * width + j - width] = rlt_uniform(seed, round, RLT_STREAM_ACCEPT, j - width);
  else u_final[i] = rlt_uniform(seed, round, RLT_STREAM_FINAL, 0);
}
}  // namespace
}  // namespace rlt

extern "C" RLT_API int rlt_round_uniforms(const int64_t* seeds, const int64_t* rounds, int n, int width,
                                          float* u_draft, float* u_accept, float* u_final, rlt_stream_t stream) {
  using namespace rlt;
  RLT_REQUIRE(n >= 0 && width >= 1 && width <= 4096, "round_uniforms: invalid request count or width");
  if (n == 0) return RLT_OK;
  RLT_REQUIRE(seeds && rounds && u_draft && u_accept && u_final, "round_uniforms: null pointer");
  const int total = n * (2 * width + 1);
  round_uniforms_kernel<<<(total + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      seeds, rounds, n, width, u_draft, u_accept, u_final);
  return launch_status("round_uniforms_kernel");
}

extern "C" RLT_API size_t rlt_accept_rejection_workspace_bytes(int rows) {
  return rows > 0 ? static_cast<size_t>(rows) * 2 * sizeof(rlt::RowStats) : 32;
}

extern "C" RLT_API int rlt_accept_rejection(const void* target_logits, const void* draft_logits, int64_t row_stride,
                                            int rows, int vocab, int dtype, const int32_t* cu_rows, int n,
                                            const int32_t* row_counts, const int64_t* tokens, int tokens_width,
                                            const int64_t* starts,
                                            const float* temperature, const int32_t* top_k, const float* top_p,
                                            const float* u_accept, const float* u_final, const int64_t* slots,
                                            int64_t* slot_values, int64_t* result, int32_t* status_out,
                                            void* workspace, size_t workspace_bytes,
                                            rlt_stream_t stream) {
  using namespace rlt;
  int status = check_logits(target_logits, row_stride, rows, vocab, dtype);
  if (status != RLT_OK) return status;
  RLT_REQUIRE(n >= 0 && tokens_width >= 1, "accept_rejection: invalid request count or token width");
  if (n == 0) return RLT_OK;
  RLT_REQUIRE(draft_logits && cu_rows && tokens && starts && temperature && u_accept && u_final && result &&
                  status_out,
              "accept_rejection: null pointer");
  if (workspace == nullptr || workspace_bytes < rlt_accept_rejection_workspace_bytes(rows) ||
      (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) {
    set_last_error_text("accept_rejection: workspace missing, misaligned or too small");
    return RLT_ERR_WORKSPACE;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  RowStats* stats = static_cast<RowStats*>(workspace);
  if (stage_rows(top_k, top_p, vocab)) {
    const size_t smem = static_cast<size_t>(vocab) * sizeof(float);
    RLT_DISPATCH_DTYPE(dtype, T, {
      auto kernel = row_stats_kernel<T, kSampleThreads, true>;
      RLT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
      kernel<<<dim3(rows, 2), kSampleThreads, smem, s>>>(static_cast<const T*>(target_logits),
                                                         static_cast<const T*>(draft_logits), row_stride, vocab, cu_rows,
                                                         n, row_counts, tokens, tokens_width, temperature, top_k, top_p,
                                                         stats);
    });
  } else {
    RLT_DISPATCH_DTYPE(dtype, T, (row_stats_kernel<T, kStatsThreads, false><<<dim3(rows, 2), kStatsThreads, 0, s>>>(
                                     static_cast<const T*>(target_logits), static_cast<const T*>(draft_logits),
                                     row_stride, vocab, cu_rows, n, row_counts, tokens, tokens_width, temperature,
                                     top_k, top_p, stats)));
  }
  status = launch_status("row_stats_kernel");
  if (status != RLT_OK) return status;
  RLT_DISPATCH_DTYPE(dtype, T, (decide_kernel<T><<<n, kSampleThreads, 0, s>>>(
                                   static_cast<const T*>(target_logits), static_cast<const T*>(draft_logits),
                                   row_stride, rows, vocab, cu_rows, n, row_counts, tokens, tokens_width, starts,
                                   temperature, u_accept, u_final, slots, slot_values, stats, result, status_out)));
  return launch_status("decide_kernel");
}
