/*
 * TEST INFRASTRUCTURE — CPU side of the counter-based random stream.
 *
 * Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3",
 * SC'11).  The reference draws from cuRAND's Philox4_32_10 / XORWOW with a hard-coded seed
 * (src/cuda/sampling.cu:20-21, src/cuda/fusion/slice_sampling.cu:19-20,
 * src/cuda/fusion/random_walk.cu:23-25); no reference test pins a sampled value, so the exact
 * stream is free.  This library keys one Philox block by (seed, item, slot/4, stream) so that
 * any sample can be regenerated in isolation; the CUDA kernels use the same function, which
 * makes the stochastic kernels bit-comparable with this restatement.
 */
#ifndef GS_ORACLE_PHILOX_H_
#define GS_ORACLE_PHILOX_H_
#include <stdint.h>

typedef struct {
  uint32_t v[4];
} gso_u32x4;

static inline gso_u32x4 gso_philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                          uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
  for (int r = 0; r < 10; ++r) {
    uint64_t p0 = (uint64_t)M0 * c0;
    uint64_t p1 = (uint64_t)M1 * c2;
    uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
    uint32_t n1 = (uint32_t)p1;
    uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    uint32_t n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += W0; k1 += W1;
  }
  gso_u32x4 out = {{c0, c1, c2, c3}};
  return out;
}

/* Stream tags: which operator consumes the block (keeps operators statistically independent
 * when they share a seed). */
enum {
  GSO_STREAM_UNIFORM = 1,
  GSO_STREAM_WEIGHTED = 2,
  GSO_STREAM_WALK = 3,
  GSO_STREAM_LIST = 4,
  GSO_STREAM_LIST_WEIGHTED = 5
};

/* 32-bit word number `slot` of the stream (seed, item, stream). */
static inline uint32_t gso_rand_u32(uint64_t seed, uint64_t item, uint64_t slot, uint32_t stream) {
  gso_u32x4 r = gso_philox4x32_10((uint32_t)item, (uint32_t)(item >> 32), (uint32_t)(slot >> 2),
                                  stream, (uint32_t)seed, (uint32_t)(seed >> 32));
  return r.v[slot & 3];
}

/* Map a 32-bit word to [0, n) by multiply-high (bias <= n / 2^32, as small as the
 * reference's `curand() % n`).  For n >= 2^32 two words are combined. */
static inline uint64_t gso_bounded(uint64_t seed, uint64_t item, uint64_t slot, uint32_t stream,
                                   uint64_t n) {
  uint32_t r = gso_rand_u32(seed, item, slot, stream);
  if (n <= 0xFFFFFFFFull) return ((uint64_t)r * n) >> 32;
  uint64_t r64 = ((uint64_t)r << 32) | gso_rand_u32(seed, item, slot, stream ^ 0x80u);
  return (uint64_t)(((unsigned __int128)r64 * n) >> 64);
}

/* Uniform float in (0, 1], 24 bits (exact in fp32). */
static inline float gso_uniform01(uint32_t r) { return (float)((r >> 8) + 1u) * (1.0f / 16777216.0f); }

/* log2(x) for normal x > 0 built only from IEEE add / mul / div / fma, so the CPU and the
 * CUDA kernels (which spell the same operations with __f*_rn intrinsics) produce identical
 * bits.  |relative error| < 3e-7.  Efraimidis-Spirakis keys u^(1/w) are ranked through the
 * monotone transform log2(u) / w. */
static inline float gso_log2f(float x) {
  union { float f; uint32_t u; } cv;
  cv.f = x;
  int32_t e = (int32_t)(cv.u >> 23) - 127;
  cv.u = (cv.u & 0x007FFFFFu) | 0x3F800000u; /* mantissa in [1, 2) */
  float m = cv.f;
  if (m > 1.41421356f) { m = m * 0.5f; e += 1; }
  float s = (m - 1.0f) / (m + 1.0f);
  float z = s * s;
  float p = __builtin_fmaf(z, 0.11111111f, 0.14285714f);
  p = __builtin_fmaf(z, p, 0.2f);
  p = __builtin_fmaf(z, p, 0.33333333f);
  p = __builtin_fmaf(z, p, 1.0f);
  float ln_m_over_2 = s * p; /* = ln(m) / 2 */
  return __builtin_fmaf(ln_m_over_2, 2.88539008f, (float)e); /* 2 / ln 2 */
}

/* A-Res ranking key (larger wins).  Weights <= 0 (and NaN) can never beat a positive weight,
 * which is the guard the reference applies in list sampling
 * (src/cuda/list_sampling_probs.cu:70-73). */
static inline float gso_ares_key(uint32_t r, float w) {
  if (!(w > 0.0f)) return -__builtin_inff();
  return gso_log2f(gso_uniform01(r)) / w;
}

#endif
