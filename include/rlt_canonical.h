/*
 * rlt_canonical.h — arithmetic that must give the same bits on the host and on
 * the GPU.  Included by the CUDA acceptance kernels and by the CPU oracle.
 *
 * The acceptance sampler compares u*q[c] against p[c] in fp32
 * (vllm-rlt: vllm_rlt/worker/speculative.py:56-58) and draws from fp32
 * distributions (vllm_rlt/worker/sampler.py:57-60); accepted-token sequences
 * must be identical for identical logits and uniforms.  To make that hold on
 * any machine and for any parallel decomposition:
 *   - exp is evaluated by rlt_expf below, built only from IEEE-754 fused
 *     multiply-adds, multiplies and adds in a fixed order (no library exp,
 *     no hardware approximation);
 *   - every sum over the vocabulary is an integer sum of 2^-40 fixed-point
 *     terms, so it does not depend on summation order;
 *   - divisions are IEEE round-to-nearest.
 * Build host code that includes this file with -ffp-contract=off.
 */
#ifndef RLT_CANONICAL_H_
#define RLT_CANONICAL_H_

#include <stdint.h>

#if defined(__CUDA_ARCH__)
#define RLT_HD __host__ __device__ __forceinline__
#define RLT_FMA(a, b, c) __fmaf_rn((a), (b), (c))
#define RLT_MUL(a, b) __fmul_rn((a), (b))
#define RLT_ADD(a, b) __fadd_rn((a), (b))
#define RLT_SUB(a, b) __fsub_rn((a), (b))
#define RLT_DIV(a, b) __fdiv_rn((a), (b))
#define RLT_F2ULL(x) __float2ull_rz((x))
#define RLT_ULL2F(x) __ull2float_rn((x))
#define RLT_DMUL(a, b) __dmul_rn((a), (b))
#define RLT_D2ULL(x) __double2ull_rz((x))
#else
#include <math.h>
#if defined(__CUDACC__)
#define RLT_HD __host__ __device__ inline
#else
#define RLT_HD static inline
#endif
#define RLT_FMA(a, b, c) fmaf((a), (b), (c))
#define RLT_MUL(a, b) ((float)(a) * (float)(b))
#define RLT_ADD(a, b) ((float)(a) + (float)(b))
#define RLT_SUB(a, b) ((float)(a) - (float)(b))
#define RLT_DIV(a, b) ((float)(a) / (float)(b))
#define RLT_F2ULL(x) ((unsigned long long)(x))
#define RLT_ULL2F(x) ((float)(long long)(x))
#define RLT_DMUL(a, b) ((double)(a) * (double)(b))
#define RLT_D2ULL(x) ((unsigned long long)(x))
#endif

/* 2^40: one unit of probability mass in fixed point. */
#define RLT_FIX_ONE 1099511627776.0f
#define RLT_FIX_INV 9.094947017729282e-13f /* 2^-40, exact */

RLT_HD float rlt_bits_to_float(uint32_t b) {
  union { uint32_t u; float f; } c;
  c.u = b;
  return c.f;
}
RLT_HD uint32_t rlt_float_to_bits(float f) {
  union { uint32_t u; float f; } c;
  c.f = f;
  return c.u;
}

/*
 * exp(d) for the softmax numerator.  d <= 0 in every use (d = t - max t); the
 * function is defined for any float:
 *   NaN -> NaN;  d < -86 -> 0;  d > 88 -> +inf;
 *   otherwise k = round(d*log2 e), r = d - k*ln2 (two-constant Cody-Waite),
 *   exp(r) = 1 + r + r^2 * P(r) with the degree-5 polynomial of Cephes expf,
 *   result = exp(r) * 2^k by exponent-field addition.  Max error about 1 ulp.
 */
RLT_HD float rlt_expf(float d) {
  if (d != d) return d;
  if (d < -86.0f) return 0.0f;
  if (d > 88.0f) return rlt_bits_to_float(0x7f800000u);
  const float magic = 12582912.0f; /* 1.5 * 2^23: adding and subtracting rounds to nearest integer */
  float k = RLT_SUB(RLT_FMA(d, 1.44269504088896341f, magic), magic);
  float r = RLT_FMA(k, -0.693359375f, d);
  r = RLT_FMA(k, 2.12194440e-4f, r);
  float p = 1.9875691500e-4f;
  p = RLT_FMA(p, r, 1.3981999507e-3f);
  p = RLT_FMA(p, r, 8.3334519073e-3f);
  p = RLT_FMA(p, r, 4.1665795894e-2f);
  p = RLT_FMA(p, r, 1.6666665459e-1f);
  p = RLT_FMA(p, r, 5.0000001201e-1f);
  float r2 = RLT_MUL(r, r);
  float y = RLT_ADD(RLT_FMA(p, r2, r), 1.0f);
  int32_t ki = (int32_t)k;
  return rlt_bits_to_float(rlt_float_to_bits(y) + ((uint32_t)ki << 23));
}

/* Fixed-point weight of a probability-like value in [0, 1]; NaN and negatives give 0. */
RLT_HD unsigned long long rlt_fix_weight(float mass) {
  if (!(mass > 0.0f)) return 0ull;
  return RLT_F2ULL(RLT_MUL(mass, RLT_FIX_ONE));
}

/* Normaliser as a float from the fixed-point sum of exp terms (sum < 2^57). */
RLT_HD float rlt_fix_to_float(unsigned long long zfix) {
  return RLT_MUL(RLT_ULL2F(zfix), RLT_FIX_INV);
}

/* Mass of token v in a plain draw from p = e / z:  e * (1 / z). */
RLT_HD float rlt_draw_mass(float e, float inv_z) { return RLT_MUL(e, inv_z); }

/* Mass of token v in a residual draw, max(p - q, 0) with p = ep / zp and q = eq / zq, written
 * without a division per token: (ep * zq - eq * zp) * (1 / (zp * zq)).  Negative values and
 * NaN get weight zero in rlt_fix_weight. */
RLT_HD float rlt_residual_mass(float ep, float eq, float zp, float zq, float inv_zpzq) {
  return RLT_MUL(RLT_SUB(RLT_MUL(ep, zq), RLT_MUL(eq, zp)), inv_zpzq);
}

/* Draw threshold: floor(u * total), u in [0, 1), total < 2^53. */
RLT_HD unsigned long long rlt_draw_threshold(float u, unsigned long long total) {
  return RLT_D2ULL(RLT_DMUL((double)u, (double)total));
}

/*
 * Support filters (strict top-k by index, then top-p;
 * vllm_rlt/worker/sampler.py:40-54).  Tokens are ranked by (scaled logit descending, token
 * index ascending); both filters keep a prefix of that ranking, so the support of a row is
 * described by one cut (key, limit): token v with scaled logit t is kept iff
 *     rlt_order_key(t) > key  ||  (rlt_order_key(t) == key && v <= limit).
 * The reference leaves the order among tied logits unspecified; this definition fixes it.
 * top-k keeps the first k ranks.  top-p keeps rank i iff the probability mass of the ranks
 * before it (exclusive prefix, as 2^-40 fixed-point integers of e * (1 / z) with z the
 * normaliser over the top-k support) is <= rlt_top_p_limit(top_p) — the integer form of the
 * reference's "drop a token once the cumulative probability before it exceeds top_p".
 */
RLT_HD uint32_t rlt_order_key(float t) {
  if (t == 0.0f) t = 0.0f; /* -0 ranks with +0 */
  uint32_t b = rlt_float_to_bits(t);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

RLT_HD unsigned long long rlt_top_p_limit(float top_p) {
  if (!(top_p > 0.0f)) return 0ull;
  return RLT_D2ULL(RLT_DMUL((double)top_p, 1099511627776.0));
}

RLT_HD int rlt_in_support(uint32_t order_key, int v, uint32_t cut_key, int cut_limit) {
  return order_key > cut_key || (order_key == cut_key && v <= cut_limit);
}

/*
 * Uniforms of a speculative round.  The reference draws them from one torch.Generator per
 * request (vllm_rlt/worker/sampler.py:84-119), on the host, in the order: the round's draft
 * draws, then per verified row the accept test, then the final residual / bonus draw
 * (vllm_rlt/worker/speculative.py:439-444, 483-510).  A device-resident round cannot consult host
 * generators, so the same three streams are defined as a counter-based generator: Philox4x32-10
 * (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11) keyed by the request's
 * seed, with the counter (index, stream, round).  A request's uniforms therefore depend on its
 * seed and on how many rounds it has run, never on the batch it shares a round with.
 */
#define RLT_STREAM_DRAFT 0u
#define RLT_STREAM_ACCEPT 1u
#define RLT_STREAM_FINAL 2u

RLT_HD void rlt_philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
    c[0] = n0;
    c[1] = (uint32_t)p1;
    c[2] = n2;
    c[3] = (uint32_t)p0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

/* U[0, 1) with 24 random bits: exact in fp32, never 1. */
RLT_HD float rlt_uniform(uint64_t seed, uint64_t round, uint32_t stream, uint32_t index) {
  uint32_t c[4];
  c[0] = index;
  c[1] = stream;
  c[2] = (uint32_t)round;
  c[3] = (uint32_t)(round >> 32);
  rlt_philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
  return RLT_MUL((float)(c[0] >> 8), 5.9604644775390625e-08f); /* 2^-24 */
}

#endif /* RLT_CANONICAL_H_ */
