// Counter-based random stream of the sampling kernels: Philox4x32-10 (Salmon et al., SC'11) keyed
// by the call's 64-bit seed, with the counter holding (item, slot / 4, operator tag).  Any draw can
// be regenerated in isolation from (seed, item, slot), so results do not depend on how work is
// spread over threads, CTAs or GPUs.  (The reference seeds cuRAND with constants and keys the
// stream by block / thread index: src/cuda/sampling.cu:20-21.)
#pragma once
#include <stdint.h>

namespace gsb {

enum : uint32_t {
  STREAM_UNIFORM = 1,
  STREAM_WEIGHTED = 2,
  STREAM_WALK = 3,
  STREAM_LIST = 4,
  STREAM_LIST_WEIGHTED = 5
};

struct U32x4 {
  uint32_t v[4];
};

__device__ __forceinline__ U32x4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                               uint32_t k0, uint32_t k1) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
    const uint32_t hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0;
    const uint32_t n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += W0; k1 += W1;
  }
  U32x4 out;
  out.v[0] = c0; out.v[1] = c1; out.v[2] = c2; out.v[3] = c3;
  return out;
}

__device__ __forceinline__ U32x4 rand_block(uint64_t seed, uint64_t item, uint64_t block, uint32_t stream) {
  return philox4x32_10((uint32_t)item, (uint32_t)(item >> 32), (uint32_t)block, stream, (uint32_t)seed,
                       (uint32_t)(seed >> 32));
}

// 32-bit word number `slot` of the stream (seed, item, stream).
__device__ __forceinline__ uint32_t rand_u32(uint64_t seed, uint64_t item, uint64_t slot, uint32_t stream) {
  const U32x4 b = rand_block(seed, item, slot >> 2, stream);
  const uint32_t s = (uint32_t)slot & 3u;
  return s == 0 ? b.v[0] : s == 1 ? b.v[1] : s == 2 ? b.v[2] : b.v[3];
}

// Uniform integer in [0, n) by multiply-high; two words when n does not fit 32 bits.
__device__ __forceinline__ uint64_t rand_bounded(uint64_t seed, uint64_t item, uint64_t slot, uint32_t stream,
                                                 uint64_t n) {
  const uint32_t r = rand_u32(seed, item, slot, stream);
  if (n <= 0xFFFFFFFFull) return ((uint64_t)r * n) >> 32;
  const uint64_t r64 = ((uint64_t)r << 32) | rand_u32(seed, item, slot, stream ^ 0x80u);
  return __umul64hi(r64, n);
}

__device__ __forceinline__ uint64_t bounded_from_word(uint32_t r, uint64_t n) { return ((uint64_t)r * n) >> 32; }

// Uniform float in (0, 1] with 24 random bits (exact in fp32).
__device__ __forceinline__ float uniform01(uint32_t r) {
  return __fmul_rn((float)((r >> 8) + 1u), 1.0f / 16777216.0f);
}

// log2(x), x normal and positive, from IEEE add / mul / div / fma only (explicitly rounded
// intrinsics, never contracted), so a host implementation spelling the same operations returns
// the same bits.  |relative error| < 3e-7.
__device__ __forceinline__ float det_log2f(float x) {
  uint32_t u = __float_as_uint(x);
  int e = (int)(u >> 23) - 127;
  float m = __uint_as_float((u & 0x007FFFFFu) | 0x3F800000u);
  if (m > 1.41421356f) {
    m = __fmul_rn(m, 0.5f);
    e += 1;
  }
  const float s = __fdiv_rn(__fsub_rn(m, 1.0f), __fadd_rn(m, 1.0f));
  const float z = __fmul_rn(s, s);
  float p = __fmaf_rn(z, 0.11111111f, 0.14285714f);
  p = __fmaf_rn(z, p, 0.2f);
  p = __fmaf_rn(z, p, 0.33333333f);
  p = __fmaf_rn(z, p, 1.0f);
  return __fmaf_rn(__fmul_rn(s, p), 2.88539008f, (float)e);
}

// Efraimidis-Spirakis ranking key: the k largest u^(1/w) win; ranked through the monotone
// transform log2(u) / w.  w <= 0 or NaN ranks below every positive weight.
__device__ __forceinline__ float ares_key(uint32_t r, float w) {
  if (!(w > 0.0f)) return __uint_as_float(0xFF800000u);  // -inf
  return __fdiv_rn(det_log2f(uniform01(r)), w);
}

}  // namespace gsb
