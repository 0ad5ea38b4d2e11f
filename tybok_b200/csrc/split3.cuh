// Exact three-term e5m2 decomposition of bf16/fp32 activations.
//
// x * 2^shift = h1 + h2 + h3 with every term an e5m2 number: h1 = rn(x'), h2 = rn(x' - h1),
// h3 = rn(x' - h1 - h2).  Three terms of 3 significant bits each carry the 8 significant bits
// of a bf16 value, so the sum is exact whenever |x'| lies in [2^-7, 57344]; below that the
// absolute error is at most 2^-17 + 2^-25, above it the terms saturate.  A weight-stationary fp8
// tensor-core GEMM over the three planes therefore reproduces the bf16-activation product
// exactly while the weights stay e4m3 in shared memory.
#pragma once

#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace tb {

// The residuals are formed in packed fp16: a bf16 value inside the window is an fp16 number
// (8 significant bits, exponent in range), each e5m2 term is the upper byte of an fp16, and
// every difference x' - h1 (- h2) is again an fp16 number, so the arithmetic is exact there and
// needs two conversions and two packed subtractions fewer per pair than an fp32 formulation.
__device__ __forceinline__ uint32_t f16x2_from_floats(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t e5m2x2_from_f16x2(uint32_t h2) {
  uint16_t r;
  asm("cvt.rn.satfinite.e5m2x2.f16x2 %0, %1;" : "=h"(r) : "r"(h2));
  return r;
}
__device__ __forceinline__ uint32_t f16x2_sub(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Two values -> three byte pairs (low byte = first value).
__device__ __forceinline__ void split3_pair(float x0, float x1, uint32_t& p1, uint32_t& p2, uint32_t& p3) {
  uint32_t x = f16x2_from_floats(x0, x1);
  p1 = e5m2x2_from_f16x2(x);
  x = f16x2_sub(x, __byte_perm(p1, 0, 0x1404));  // e5m2 bytes -> the upper bytes of the two halves
  p2 = e5m2x2_from_f16x2(x);
  x = f16x2_sub(x, __byte_perm(p2, 0, 0x1404));
  p3 = e5m2x2_from_f16x2(x);
}

// Four values -> one 32-bit word per plane (byte i = value i).
__device__ __forceinline__ void split3_quad(const float (&x)[4], uint32_t& w1, uint32_t& w2, uint32_t& w3) {
  uint32_t a1, a2, a3, b1, b2, b3;
  split3_pair(x[0], x[1], a1, a2, a3);
  split3_pair(x[2], x[3], b1, b2, b3);
  w1 = a1 | (b1 << 16);
  w2 = a2 | (b2 << 16);
  w3 = a3 | (b3 << 16);
}

// ------------------------------------------------------------------------------------------
// Two-term e4m3 decomposition with a per-row power-of-two scale, for producers that see a whole
// activation row (the norm kernels): x * 2^k = g1 + g2 with g1 = rn(x'), g2 = rn(x' - g1) in e4m3,
// where k puts the row's largest magnitude into (224, 448].  Two terms of 4 significant bits carry
// the 8 significant bits of a bf16 value exactly whenever |x'| >= 2^-2, i.e. for every element
// within 2^-10.8 of the row maximum; smaller elements err by at most 2^-10 in scaled units
// (4e-6 of the row maximum).  The GEMM multiplies its accumulator column of that token by 2^-k.
// Two planes instead of three: a third less tensor work and operand traffic, token tiles to 128.
__device__ __forceinline__ uint32_t e4m3x2_from_f16x2(uint32_t h2) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(r) : "r"(h2));
  return r;
}
__device__ __forceinline__ uint32_t f16x2_from_e4m3x2(uint32_t p) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(static_cast<uint16_t>(p)));
  return r;
}
// Four scaled values -> one 32-bit word per plane (byte i = value i).
__device__ __forceinline__ void split2_quad(const float (&x)[4], uint32_t& w1, uint32_t& w2) {
  uint32_t a = f16x2_from_floats(x[0], x[1]), b = f16x2_from_floats(x[2], x[3]);
  const uint32_t a1 = e4m3x2_from_f16x2(a), b1 = e4m3x2_from_f16x2(b);
  a = f16x2_sub(a, f16x2_from_e4m3x2(a1));
  b = f16x2_sub(b, f16x2_from_e4m3x2(b1));
  w1 = a1 | (b1 << 16);
  w2 = e4m3x2_from_f16x2(a) | (e4m3x2_from_f16x2(b) << 16);
}
// Exponent k with amax * 2^k in (224, 448] (0 for an all-zero row), returned as the two exact
// powers of two: up = 2^k for the producer, down = 2^-k for the consumer.
__device__ __forceinline__ void row_pow2(float amax, float& up, float& down) {
  const uint32_t bits = __float_as_uint(amax);
  int k = 0;
  if (amax > 1e-30f && amax < 1e30f) {
    const int e = static_cast<int>((bits >> 23) & 0xffu) - 127;          // amax = f * 2^e, f in [1, 2)
    const float f = __uint_as_float((bits & 0x7fffffu) | 0x3f800000u);
    k = 8 - e - (f > 1.75f ? 1 : 0);                                     // 448 = 1.75 * 2^8
  }
  up = __uint_as_float(static_cast<uint32_t>(k + 127) << 23);
  down = __uint_as_float(static_cast<uint32_t>(127 - k) << 23);
}

}  // namespace tb
