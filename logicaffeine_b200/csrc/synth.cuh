// Counter-based synthetic-input generator, device side.
//
// Every value is a pure function of (seed, stream, index), so any shard of any
// tensor can be produced on the GPU that owns it and 38 GB of weights never
// cross PCIe.  All floating-point steps use the explicitly rounded intrinsics
// (__fmul_rn / __fadd_rn / __fdiv_rn / __fsqrt_rn), which the compiler never
// contracts into FMAs, and hand-written polynomial log / sin / cos, so a CPU
// build with contraction off reproduces the same bits.
//
// Mixer: the SplitMix64 finaliser, the generator the reference seeds its own
// runtime with (crates/logicaffeine_runtime/src/seed.rs:15-28).
#pragma once
#include <stdint.h>

namespace logos {
namespace synth {

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z ^= z >> 30;
  z *= 0xBF58476D1CE4E5B9ull;
  z ^= z >> 27;
  z *= 0x94D049BB133111EBull;
  z ^= z >> 31;
  return z;
}

__host__ __device__ __forceinline__ uint64_t ctr_hash(uint64_t seed, uint64_t stream, uint64_t idx) {
  const uint64_t G = 0x9E3779B97F4A7C15ull;
  return mix64(mix64(seed + G * (stream + 1)) + G * (idx + 1));
}

__device__ __forceinline__ int uniform_i8(uint64_t seed, uint64_t stream, uint64_t idx) {
  uint32_t r = (uint32_t)(ctr_hash(seed, stream, idx) >> 32);
  return (int)(r % 255u) - 127;
}

__device__ __forceinline__ int uniform_i32(uint64_t seed, uint64_t stream, uint64_t idx, uint32_t n) {
  uint32_t r = (uint32_t)(ctr_hash(seed, stream, idx) >> 32);
  return (int)(r % n);
}

__device__ __forceinline__ float uniform_f32(uint64_t seed, uint64_t stream, uint64_t idx, float a, float b) {
  uint32_t r = (uint32_t)(ctr_hash(seed, stream, idx) >> 40);  // 24 bits
  float u = __fmul_rn((float)r, 5.9604644775390625e-08f);      // * 2^-24, exact
  return __fadd_rn(a, __fmul_rn(u, __fsub_rn(b, a)));
}

// Standard normal by Box-Muller; one hash feeds a pair (index>>1), bit 0 of the
// index picks the cosine or the sine branch.
__device__ __forceinline__ float normal_f32(uint64_t seed, uint64_t stream, uint64_t idx) {
  uint64_t h = ctr_hash(seed, stream, idx >> 1);
  uint32_t k1 = (uint32_t)(h >> 40);             // 24 bits
  uint32_t k2 = (uint32_t)(h >> 16) & 0xFFFFFFu; // 24 bits

  // ln(u1), u1 = (k1+1) * 2^-24 in (0,1]
  uint32_t v = k1 + 1u;                 // [1, 2^24]
  int e = 31 - __clz((int)v);           // floor(log2 v)
  float m = __fmul_rn((float)v, __int_as_float((127 - e) << 23));  // v * 2^-e in [1,2), exact
  if (m > 1.41421354f) {
    m = __fmul_rn(m, 0.5f);
    e += 1;
  }
  float t = __fdiv_rn(__fsub_rn(m, 1.0f), __fadd_rn(m, 1.0f));
  float t2 = __fmul_rn(t, t);
  float p = 0.111111111f;                                   // 1/9
  p = __fadd_rn(__fmul_rn(p, t2), 0.142857143f);            // 1/7
  p = __fadd_rn(__fmul_rn(p, t2), 0.2f);
  p = __fadd_rn(__fmul_rn(p, t2), 0.333333343f);
  p = __fadd_rn(__fmul_rn(p, t2), 1.0f);
  float ln_m = __fmul_rn(__fmul_rn(2.0f, t), p);
  float ln_u = __fadd_rn(ln_m, __fmul_rn((float)(e - 24), 0.693147182f));
  float r = __fsqrt_rn(__fmul_rn(-2.0f, ln_u));

  // angle 2*pi*u2 = quadrant*(pi/2) + f*(pi/2), f in [0,1)
  uint32_t quad = k2 >> 22;
  float f = __fmul_rn((float)(k2 & 0x3FFFFFu), 2.384185791015625e-07f);  // * 2^-22, exact
  float x = __fmul_rn(f, 1.57079637f);
  float x2 = __fmul_rn(x, x);
  // cos x, Taylor to x^12
  float c = 2.08767570e-09f;
  c = __fadd_rn(__fmul_rn(c, x2), -2.75573192e-07f);
  c = __fadd_rn(__fmul_rn(c, x2), 2.48015873e-05f);
  c = __fadd_rn(__fmul_rn(c, x2), -1.38888889e-03f);
  c = __fadd_rn(__fmul_rn(c, x2), 4.16666667e-02f);
  c = __fadd_rn(__fmul_rn(c, x2), -0.5f);
  c = __fadd_rn(__fmul_rn(c, x2), 1.0f);
  // sin x, Taylor to x^13
  float s = 1.60590438e-10f;
  s = __fadd_rn(__fmul_rn(s, x2), -2.50521084e-08f);
  s = __fadd_rn(__fmul_rn(s, x2), 2.75573192e-06f);
  s = __fadd_rn(__fmul_rn(s, x2), -1.98412698e-04f);
  s = __fadd_rn(__fmul_rn(s, x2), 8.33333333e-03f);
  s = __fadd_rn(__fmul_rn(s, x2), -1.66666667e-01f);
  s = __fadd_rn(__fmul_rn(s, x2), 1.0f);
  s = __fmul_rn(s, x);
  float cq, sq;
  switch (quad) {
    case 0: cq = c; sq = s; break;
    case 1: cq = -s; sq = c; break;
    case 2: cq = -c; sq = -s; break;
    default: cq = s; sq = -c; break;
  }
  return __fmul_rn(r, (idx & 1ull) ? sq : cq);
}

// ln of a positive normal float: the exponent comes off by bits, the mantissa (folded into
// (0.707, 1.414]) goes through the same atanh series as above.
__device__ __forceinline__ float ln_pos(float x) {
  const int bits = __float_as_int(x);
  int e = (bits >> 23) - 127;
  float m = __int_as_float((bits & 0x007FFFFF) | 0x3F800000);
  if (m > 1.41421354f) {
    m = __fmul_rn(m, 0.5f);
    e += 1;
  }
  float t = __fdiv_rn(__fsub_rn(m, 1.0f), __fadd_rn(m, 1.0f));
  float t2 = __fmul_rn(t, t);
  float p = 0.111111111f;
  p = __fadd_rn(__fmul_rn(p, t2), 0.142857143f);
  p = __fadd_rn(__fmul_rn(p, t2), 0.2f);
  p = __fadd_rn(__fmul_rn(p, t2), 0.333333343f);
  p = __fadd_rn(__fmul_rn(p, t2), 1.0f);
  float ln_m = __fmul_rn(__fmul_rn(2.0f, t), p);
  return __fadd_rn(ln_m, __fmul_rn((float)e, 0.693147182f));
}

// Standard Gumbel variate -ln(-ln u) with u = (2k + 1) * 2^-24 for a 23-bit k, so u lies strictly
// inside (0, 1) and both logarithms see a positive normal number.  argmax(logit / T + gumbel)
// draws from softmax(logit / T).
__device__ __forceinline__ float gumbel_f32(uint64_t seed, uint64_t stream, uint64_t idx) {
  const uint32_t k = (uint32_t)(ctr_hash(seed, stream, idx) >> 41);
  const float u = __fmul_rn((float)(2u * k + 1u), 5.9604644775390625e-08f);  // * 2^-24, exact
  const float l = -ln_pos(u);
  return -ln_pos(l);
}

__device__ __forceinline__ float normal_scaled(uint64_t seed, uint64_t stream, uint64_t idx, float mean, float std) {
  return __fadd_rn(mean, __fmul_rn(std, normal_f32(seed, stream, idx)));
}

}  // namespace synth
}  // namespace logos
