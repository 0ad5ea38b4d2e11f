// Exact three-term e5m2 decomposition of bf16/fp32 activations.
//
// x * 2^shift = h1 + h2 + h3 with every term an e5m2 number: h1 = rn(x'), h2 = rn(x' - h1),
// h3 = rn(x' - h1 - h2).  Three terms of 3 significant bits each carry the 8 significant bits
// of a bf16 value, so the sum is exact whenever |x'| lies in [2^-7, 57344]; below that the
// absolute error is at most 2^-17, above it the terms saturate.  A weight-stationary fp8
// tensor-core GEMM over the three planes therefore reproduces the bf16-activation product
// exactly while the weights stay e4m3 in shared memory.
#pragma once

#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace tb {

__device__ __forceinline__ float2 e5m2x2_to_float2(uint32_t pair) {
  // e5m2 is the upper byte of an fp16: shift each byte into the high half of a 16-bit lane.
  const uint32_t h = ((pair & 0xFFu) << 8) | ((pair & 0xFF00u) << 16);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

// Two values -> three byte pairs (low byte = first value).
__device__ __forceinline__ void split3_pair(float x0, float x1, uint32_t& p1, uint32_t& p2, uint32_t& p3) {
  p1 = __nv_cvt_float2_to_fp8x2(make_float2(x0, x1), __NV_SATFINITE, __NV_E5M2);
  float2 f = e5m2x2_to_float2(p1);
  x0 -= f.x;
  x1 -= f.y;
  p2 = __nv_cvt_float2_to_fp8x2(make_float2(x0, x1), __NV_SATFINITE, __NV_E5M2);
  f = e5m2x2_to_float2(p2);
  x0 -= f.x;
  x1 -= f.y;
  p3 = __nv_cvt_float2_to_fp8x2(make_float2(x0, x1), __NV_SATFINITE, __NV_E5M2);
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

}  // namespace tb
