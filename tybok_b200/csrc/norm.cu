// RMS normalisation that feeds a W8 GEMM: one warp per token row, fp32 statistics, output as
// the three e5m2 activation planes (and/or bf16).
//
// Two forms, both from tybok/policies/pi05/models/layers.py:34-84:
//   plain Gemma norm   y = bf16( x * rsqrt(mean(x^2) + eps) * (1 + weight) )
//   AdaRMS norm        y = bf16( x * rsqrt(mean(x^2) + eps) * (1 + scale) + shift )
// where scale/shift are the first two thirds of a precomputed dense(cond) row
// ([groups, 3*W] or [groups, 2*W], fp32), one row per group of `rows_per_group` tokens.
// Algorithmic bytes per row: 2*W read, 3*W (+2*W) written.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/tybok_b200.h"
#include "host_util.h"
#include "ptx.cuh"
#include "split3.cuh"

namespace tb {

constexpr int NORM_MAX_VEC = 16;  // 16 vectors of 8 elements per lane: W <= 4096

struct NormParams {
  const __nv_bfloat16* x;
  long long ldx;
  const float* weight;  // [W] or NULL
  const float* mod;     // [groups, ldmod] or NULL; scale at [0,W), shift at [W,2W)
  const __nv_bfloat16* ln_scale;  // [W] bf16: LayerNorm + modulate form when set
  const __nv_bfloat16* ln_shift;  // [W] bf16
  int ln_affine;  // 1: ln_scale / ln_shift are an affine LayerNorm's weight / bias, y = bf16(LN(x) * w + b) in fp32
  long long ldmod;
  int rows_per_group;
  int M, W;
  float eps;
  float plane_scale;
  uint8_t* planes;       // [3][M][W] or NULL
  uint8_t* planes2;      // [2][M][W] e4m3 planes of y * 2^k(row) or NULL, with row_scale[M] = 2^-k(row)
  float* row_scale;
  __nv_bfloat16* y;      // [M, ldy] or NULL
  long long ldy;
  int pdl;
  int* dbg;  // debugging aid: stage counters, NULL in production
};

// VEC = 8-element vectors per lane; FULL = every lane owns exactly VEC vectors (W == 256 * VEC),
// which removes the bounds predicates so that the loads can be hoisted and overlapped.
template <int VEC, bool FULL>
__global__ void __launch_bounds__(128) rmsnorm_kernel(const NormParams p) {
  // Let the next kernel in the stream start its preamble (weight prefetch) right away; it still
  // waits for this grid to finish before it reads what is written here.
  if (p.pdl) pdl_launch_dependents();
  if (threadIdx.x == 0) dbg_stage(p.dbg, 8, 0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x * 4 + warp;
  const int nvec = p.W / 8;  // 8-element vectors per row
  // Scale / shift are constants of the step: fetch them before waiting for the previous kernel.
  const float* mod = (p.mod && m < p.M) ? p.mod + static_cast<long long>(m / p.rows_per_group) * p.ldmod : nullptr;
  constexpr bool PRE = VEC <= 8;  // wider rows would not fit the constants in registers
  float4 csc[PRE ? VEC : 1][2], csh[PRE ? VEC : 1][2];
  if (PRE && !p.ln_scale && m < p.M) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = lane + 32 * i;
      if (FULL || c < nvec) {
        const float* a = mod ? mod + c * 8 : p.weight + c * 8;
        csc[PRE ? i : 0][0] = *reinterpret_cast<const float4*>(a);
        csc[PRE ? i : 0][1] = *reinterpret_cast<const float4*>(a + 4);
        if (mod) {
          csh[PRE ? i : 0][0] = *reinterpret_cast<const float4*>(a + p.W);
          csh[PRE ? i : 0][1] = *reinterpret_cast<const float4*>(a + p.W + 4);
        }
      }
    }
  }
  if (p.pdl) pdl_wait();
  if (threadIdx.x == 0) dbg_stage(p.dbg, 8, 2);
  if (m < p.M) {
    const __nv_bfloat16* row = p.x + m * p.ldx;
    float v[VEC][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = lane + 32 * i;
      if (FULL || c < nvec) {
        const uint4 raw = *reinterpret_cast<const uint4*>(row + c * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[i][2 * e] = __bfloat162float(h[e].x);
          v[i][2 * e + 1] = __bfloat162float(h[e].y);
          ss += v[i][2 * e] * v[i][2 * e] + v[i][2 * e + 1] * v[i][2 * e + 1];
        }
      }
    }
    float mean = 0.f;
    if (p.ln_scale) {  // LayerNorm: centre first, then the variance of the centred values
      float sm = 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i)
        if (FULL || lane + 32 * i < nvec) {
#pragma unroll
          for (int e = 0; e < 8; ++e) sm += v[i][e];
        }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, o);
      mean = sm / static_cast<float>(p.W);
      ss = 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i)
        if (FULL || lane + 32 * i < nvec) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            v[i][e] -= mean;
            ss += v[i][e] * v[i][e];
          }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss / static_cast<float>(p.W) + p.eps);
    const long long plane = static_cast<long long>(p.M) * p.W;
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = lane + 32 * i;
      if (FULL || c < nvec) {
        float o[8];
        if (p.ln_scale) {
          // modulate(LN(x)) with every step rounded to bf16, as the reference's bf16 tensor ops
          // do: n = bf16(LN), t = bf16(1 + scale), out = bf16(bf16(n * t) + shift).
          const uint4 rs = *reinterpret_cast<const uint4*>(p.ln_scale + c * 8);
          const uint4 rh = *reinterpret_cast<const uint4*>(p.ln_shift + c * 8);
          const __nv_bfloat16* ps = reinterpret_cast<const __nv_bfloat16*>(&rs);
          const __nv_bfloat16* ph = reinterpret_cast<const __nv_bfloat16*>(&rh);
          if (p.ln_affine) {  // fp32 statistics and fp32 affine, one rounding (wan_base.py:141-148)
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = v[i][e] * rstd * __bfloat162float(ps[e]) + __bfloat162float(ph[e]);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float nrm = bf16_round(v[i][e] * rstd);
              const float t = bf16_round(1.0f + __bfloat162float(ps[e]));
              o[e] = bf16_round(nrm * t) + __bfloat162float(ph[e]);
            }
          }
        } else {
        // x * rstd is formed in fp32 (the bf16 x promotes), as in the reference's _norm
        float4 q0, q1, h0 = make_float4(0.f, 0.f, 0.f, 0.f), h1 = h0;
        if (PRE) {
          q0 = csc[PRE ? i : 0][0]; q1 = csc[PRE ? i : 0][1];
          if (mod) { h0 = csh[PRE ? i : 0][0]; h1 = csh[PRE ? i : 0][1]; }
        } else {
          const float* a = mod ? mod + c * 8 : p.weight + c * 8;
          q0 = *reinterpret_cast<const float4*>(a); q1 = *reinterpret_cast<const float4*>(a + 4);
          if (mod) { h0 = *reinterpret_cast<const float4*>(a + p.W); h1 = *reinterpret_cast<const float4*>(a + p.W + 4); }
        }
        const float sc[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const float sh[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float t = v[i][e] * rstd * (1.0f + sc[e]);
          if (mod) t = v[i][e] * rstd * (1.0f + sc[e]) + sh[e];
          o[e] = t;
        }
        }
        __nv_bfloat162 b[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) b[e] = __floats2bfloat162_rn(o[2 * e], o[2 * e + 1]);
        if (p.y) *reinterpret_cast<uint4*>(p.y + m * p.ldy + c * 8) = *reinterpret_cast<const uint4*>(b);
        if (p.planes) {
          const float lo[4] = {__bfloat162float(b[0].x) * p.plane_scale, __bfloat162float(b[0].y) * p.plane_scale,
                               __bfloat162float(b[1].x) * p.plane_scale, __bfloat162float(b[1].y) * p.plane_scale};
          const float hi[4] = {__bfloat162float(b[2].x) * p.plane_scale, __bfloat162float(b[2].y) * p.plane_scale,
                               __bfloat162float(b[3].x) * p.plane_scale, __bfloat162float(b[3].y) * p.plane_scale};
          uint2 w1, w2, w3;
          split3_quad(lo, w1.x, w2.x, w3.x);
          split3_quad(hi, w1.y, w2.y, w3.y);
          uint8_t* dst = p.planes + static_cast<long long>(m) * p.W + c * 8;
          *reinterpret_cast<uint2*>(dst) = w1;
          *reinterpret_cast<uint2*>(dst + plane) = w2;
          *reinterpret_cast<uint2*>(dst + 2 * plane) = w3;
        }
        if (p.planes2) {  // keep the rounded row (over v, which is dead now) until its maximum is known
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            v[i][2 * e] = __bfloat162float(b[e].x);
            v[i][2 * e + 1] = __bfloat162float(b[e].y);
            amax = fmaxf(amax, fmaxf(fabsf(v[i][2 * e]), fabsf(v[i][2 * e + 1])));
          }
        }
      }
    }
    if (p.planes2) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      float up, down;
      row_pow2(amax, up, down);
      if (lane == 0) p.row_scale[m] = down;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const int c = lane + 32 * i;
        if (FULL || c < nvec) {
          const float lo[4] = {v[i][0] * up, v[i][1] * up, v[i][2] * up, v[i][3] * up};
          const float hi[4] = {v[i][4] * up, v[i][5] * up, v[i][6] * up, v[i][7] * up};
          uint2 w1, w2;
          split2_quad(lo, w1.x, w2.x);
          split2_quad(hi, w1.y, w2.y);
          uint8_t* dst = p.planes2 + static_cast<long long>(m) * p.W + c * 8;
          *reinterpret_cast<uint2*>(dst) = w1;
          *reinterpret_cast<uint2*>(dst + plane) = w2;
        }
      }
    }
  }
}

// The RMS forms with one CTA per row and eight elements per thread (rows of 512..4096
// elements): one load in flight per thread instead of W / 256 per lane, an eighth of the
// per-thread arithmetic, and the sum of squares crosses the warps through shared memory.
__global__ void __launch_bounds__(512) rmsnorm_row_kernel(const NormParams p) {
  __shared__ float red[16];
  __shared__ float red_max[16];
  if (p.pdl) pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int m = blockIdx.x, c = threadIdx.x;
  const bool live = c < p.W / 8;
  // Scale / shift are constants of the step: fetch them before waiting for the previous kernel.
  const float* mod = p.mod ? p.mod + static_cast<long long>(m / p.rows_per_group) * p.ldmod : nullptr;
  float4 q0 = {}, q1 = {}, h0 = {}, h1 = {};
  if (live) {
    const float* a = mod ? mod + c * 8 : p.weight + c * 8;
    q0 = *reinterpret_cast<const float4*>(a);
    q1 = *reinterpret_cast<const float4*>(a + 4);
    if (mod) {
      h0 = *reinterpret_cast<const float4*>(a + p.W);
      h1 = *reinterpret_cast<const float4*>(a + p.W + 4);
    }
  }
  if (p.pdl) pdl_wait();
  float v[8];
  float ss = 0.f;
  if (live) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p.x + m * p.ldx + c * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      v[2 * e] = __bfloat162float(h[e].x);
      v[2 * e + 1] = __bfloat162float(h[e].y);
      ss += v[2 * e] * v[2 * e] + v[2 * e + 1] * v[2 * e + 1];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < nwarps; ++w) tot += red[w];
  const float rstd = rsqrtf(tot / static_cast<float>(p.W) + p.eps);
  if (live) {
    // x * rstd is formed in fp32 (the bf16 x promotes), as in the reference's _norm
    const float sc[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    const float sh[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float t = v[e] * rstd * (1.0f + sc[e]);
      if (mod) t = v[e] * rstd * (1.0f + sc[e]) + sh[e];
      o[e] = t;
    }
    __nv_bfloat162 b[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) b[e] = __floats2bfloat162_rn(o[2 * e], o[2 * e + 1]);
    if (p.y) *reinterpret_cast<uint4*>(p.y + m * p.ldy + c * 8) = *reinterpret_cast<const uint4*>(b);
    if (p.planes) {
      const float lo[4] = {__bfloat162float(b[0].x) * p.plane_scale, __bfloat162float(b[0].y) * p.plane_scale,
                           __bfloat162float(b[1].x) * p.plane_scale, __bfloat162float(b[1].y) * p.plane_scale};
      const float hi[4] = {__bfloat162float(b[2].x) * p.plane_scale, __bfloat162float(b[2].y) * p.plane_scale,
                           __bfloat162float(b[3].x) * p.plane_scale, __bfloat162float(b[3].y) * p.plane_scale};
      uint2 w1, w2, w3;
      split3_quad(lo, w1.x, w2.x, w3.x);
      split3_quad(hi, w1.y, w2.y, w3.y);
      const long long plane = static_cast<long long>(p.M) * p.W;
      uint8_t* dst = p.planes + static_cast<long long>(m) * p.W + c * 8;
      *reinterpret_cast<uint2*>(dst) = w1;
      *reinterpret_cast<uint2*>(dst + plane) = w2;
      *reinterpret_cast<uint2*>(dst + 2 * plane) = w3;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {  // the rounded values, for the two-plane form below
      v[2 * e] = __bfloat162float(b[e].x);
      v[2 * e + 1] = __bfloat162float(b[e].y);
    }
  }
  if (p.planes2) {  // CTA-uniform: the row maximum crosses the warps like the sum of squares did
    float amax = 0.f;
    if (live) {
#pragma unroll
      for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) red_max[warp] = amax;
    __syncthreads();
    amax = 0.f;
    for (int w = 0; w < nwarps; ++w) amax = fmaxf(amax, red_max[w]);
    float up, down;
    row_pow2(amax, up, down);
    if (threadIdx.x == 0) p.row_scale[m] = down;
    if (live) {
      const float lo[4] = {v[0] * up, v[1] * up, v[2] * up, v[3] * up};
      const float hi[4] = {v[4] * up, v[5] * up, v[6] * up, v[7] * up};
      uint2 w1, w2;
      split2_quad(lo, w1.x, w2.x);
      split2_quad(hi, w1.y, w2.y);
      uint8_t* dst = p.planes2 + static_cast<long long>(m) * p.W + c * 8;
      *reinterpret_cast<uint2*>(dst) = w1;
      *reinterpret_cast<uint2*>(dst + static_cast<long long>(p.M) * p.W) = w2;
    }
  }
}

// ------------------------------------------------------------------------------------------
// Residual add + affine LayerNorm of the vision tower (tybok/policies/pi05/models/vision.py:
// x = x + sublayer(x); h = LayerNorm(x)): x_out = bf16(x + y), h = bf16(LN_fp32(x_out) * w + b).
// One warp per row; the two bf16 adds and the norm that torch runs as two kernels are one.
struct AddLnParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* y;  // or NULL: plain LayerNorm of x
  const __nv_bfloat16* w;
  const __nv_bfloat16* b;
  __nv_bfloat16* x_out;    // or NULL
  __nv_bfloat16* h;
  int M, W;
  float eps;
  int pdl;
};

template <int VEC>
__global__ void __launch_bounds__(128) add_layernorm_kernel(const AddLnParams p) {
  if (p.pdl) pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x * 4 + warp;
  if (p.pdl) pdl_wait();
  if (m >= p.M) return;
  const int nvec = p.W / 8;
  const long long base = static_cast<long long>(m) * p.W;
  float v[VEC][8];
  uint4 rw[VEC], rb[VEC];  // scale and bias: requested with the row, not after its two reductions
  float sm = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      rw[i] = *reinterpret_cast<const uint4*>(p.w + c * 8);
      rb[i] = *reinterpret_cast<const uint4*>(p.b + c * 8);
    }
  }
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      const uint4 rx = *reinterpret_cast<const uint4*>(p.x + base + c * 8);
      const __nv_bfloat162* hx = reinterpret_cast<const __nv_bfloat162*>(&rx);
      __nv_bfloat162 s2[4];
      if (p.y) {
        const uint4 ry = *reinterpret_cast<const uint4*>(p.y + base + c * 8);
        const __nv_bfloat162* hy = reinterpret_cast<const __nv_bfloat162*>(&ry);
#pragma unroll
        for (int e = 0; e < 4; ++e)  // bf16 + bf16 -> bf16, as the residual add of the bf16 modules
          s2[e] = __floats2bfloat162_rn(__bfloat162float(hx[e].x) + __bfloat162float(hy[e].x),
                                        __bfloat162float(hx[e].y) + __bfloat162float(hy[e].y));
        if (p.x_out) *reinterpret_cast<uint4*>(p.x_out + base + c * 8) = *reinterpret_cast<const uint4*>(s2);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) s2[e] = hx[e];
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[i][2 * e] = __bfloat162float(s2[e].x);
        v[i][2 * e + 1] = __bfloat162float(s2[e].y);
        sm += v[i][2 * e] + v[i][2 * e + 1];
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, o);
  const float mean = sm / static_cast<float>(p.W);
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i)
    if (lane + 32 * i < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        v[i][e] -= mean;
        ss += v[i][e] * v[i][e];
      }
    }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float rstd = rsqrtf(ss / static_cast<float>(p.W) + p.eps);
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      const __nv_bfloat16* pw = reinterpret_cast<const __nv_bfloat16*>(&rw[i]);
      const __nv_bfloat16* pb = reinterpret_cast<const __nv_bfloat16*>(&rb[i]);
      __nv_bfloat162 o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        o[e] = __floats2bfloat162_rn(v[i][2 * e] * rstd * __bfloat162float(pw[2 * e]) + __bfloat162float(pb[2 * e]),
                                     v[i][2 * e + 1] * rstd * __bfloat162float(pw[2 * e + 1]) + __bfloat162float(pb[2 * e + 1]));
      *reinterpret_cast<uint4*>(p.h + base + c * 8) = *reinterpret_cast<const uint4*>(o);
    }
  }
}

// The same operation with one CTA per row and eight elements per thread: for rows of a thousand
// elements and a few hundred rows the warp-per-row form leaves most of the machine idle and each
// lane walks five dependent-latency loads; here every thread has one load in flight and the two
// reductions cross the warps through shared memory.
__global__ void __launch_bounds__(256) add_layernorm_row_kernel(const AddLnParams p) {
  __shared__ float red[2][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int c = threadIdx.x, nvec = p.W / 8;
  const bool live = c < nvec;
  const long long base = static_cast<long long>(blockIdx.x) * p.W;
  uint4 rw = {}, rb = {};
  float v[8];
  float sm = 0.f;
  if (live) {
    rw = *reinterpret_cast<const uint4*>(p.w + c * 8);
    rb = *reinterpret_cast<const uint4*>(p.b + c * 8);
    const uint4 rx = *reinterpret_cast<const uint4*>(p.x + base + c * 8);
    const __nv_bfloat162* hx = reinterpret_cast<const __nv_bfloat162*>(&rx);
    __nv_bfloat162 s2[4];
    if (p.y) {
      const uint4 ry = *reinterpret_cast<const uint4*>(p.y + base + c * 8);
      const __nv_bfloat162* hy = reinterpret_cast<const __nv_bfloat162*>(&ry);
#pragma unroll
      for (int e = 0; e < 4; ++e)  // bf16 + bf16 -> bf16, as the residual add of the bf16 modules
        s2[e] = __floats2bfloat162_rn(__bfloat162float(hx[e].x) + __bfloat162float(hy[e].x),
                                      __bfloat162float(hx[e].y) + __bfloat162float(hy[e].y));
      if (p.x_out) *reinterpret_cast<uint4*>(p.x_out + base + c * 8) = *reinterpret_cast<const uint4*>(s2);
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) s2[e] = hx[e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      v[2 * e] = __bfloat162float(s2[e].x);
      v[2 * e + 1] = __bfloat162float(s2[e].y);
      sm += v[2 * e] + v[2 * e + 1];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, o);
  if (lane == 0) red[0][warp] = sm;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < nwarps; ++w) tot += red[0][w];
  const float mean = tot / static_cast<float>(p.W);
  float ss = 0.f;
  if (live) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      v[e] -= mean;
      ss += v[e] * v[e];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) red[1][warp] = ss;
  __syncthreads();
  tot = 0.f;
  for (int w = 0; w < nwarps; ++w) tot += red[1][w];
  const float rstd = rsqrtf(tot / static_cast<float>(p.W) + p.eps);
  if (live) {
    const __nv_bfloat16* pw = reinterpret_cast<const __nv_bfloat16*>(&rw);
    const __nv_bfloat16* pb = reinterpret_cast<const __nv_bfloat16*>(&rb);
    __nv_bfloat162 o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      o[e] = __floats2bfloat162_rn(v[2 * e] * rstd * __bfloat162float(pw[2 * e]) + __bfloat162float(pb[2 * e]),
                                   v[2 * e + 1] * rstd * __bfloat162float(pw[2 * e + 1]) + __bfloat162float(pb[2 * e + 1]));
    *reinterpret_cast<uint4*>(p.h + base + c * 8) = *reinterpret_cast<const uint4*>(o);
  }
}

// Mixed form for a bf16 tower whose residual stream stays in fp32: x and x_out fp32, the sublayer
// output y, weight, bias and the normalised h bf16.  The stream is then never rounded to bf16
// (only the GEMM inputs are), which is where a bf16 tower loses most of its accuracy: the stream is
// several times larger than what a sublayer adds to it.  One CTA per row, eight elements per thread.
// T16 = __nv_bfloat16 or __half: the 16-bit type of the sublayer output, the norm's weight / bias and h.
template <typename T16>
struct AddLnMixedParams {
  const float* x;
  const T16* y;  // or NULL
  const T16* w;
  const T16* b;
  float* x_out;  // or NULL
  T16* h;
  int M, W;
  float eps;
};
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ uint32_t pack2(float a, float b, __nv_bfloat16) {
  const __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&t);
}
__device__ __forceinline__ uint32_t pack2(float a, float b, __half) {
  const __half2 t = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&t);
}

template <typename T16>
__global__ void __launch_bounds__(256) add_layernorm_mixed_kernel(const AddLnMixedParams<T16> p) {
  __shared__ float red[2][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int c = threadIdx.x * 8;
  const bool live = c < p.W;
  const long long base = static_cast<long long>(blockIdx.x) * p.W;
  uint4 rw = {}, rb = {};
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  float sm = 0.f;
  if (live) {
    rw = *reinterpret_cast<const uint4*>(p.w + c);
    rb = *reinterpret_cast<const uint4*>(p.b + c);
    const float4 a0 = *reinterpret_cast<const float4*>(p.x + base + c);
    const float4 a1 = *reinterpret_cast<const float4*>(p.x + base + c + 4);
    v[0] = a0.x; v[1] = a0.y; v[2] = a0.z; v[3] = a0.w; v[4] = a1.x; v[5] = a1.y; v[6] = a1.z; v[7] = a1.w;
    if (p.y) {
      const uint4 ry = *reinterpret_cast<const uint4*>(p.y + base + c);
      const T16* hy = reinterpret_cast<const T16*>(&ry);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += to_f32(hy[e]);
      if (p.x_out) {
        *reinterpret_cast<float4*>(p.x_out + base + c) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p.x_out + base + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) sm += v[e];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, o);
  if (lane == 0) red[0][warp] = sm;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < nwarps; ++w) tot += red[0][w];
  const float mean = tot / static_cast<float>(p.W);
  float ss = 0.f;
  if (live) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      v[e] -= mean;
      ss += v[e] * v[e];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) red[1][warp] = ss;
  __syncthreads();
  tot = 0.f;
  for (int w = 0; w < nwarps; ++w) tot += red[1][w];
  const float rstd = rsqrtf(tot / static_cast<float>(p.W) + p.eps);
  if (live) {
    const T16* pw = reinterpret_cast<const T16*>(&rw);
    const T16* pb = reinterpret_cast<const T16*>(&rb);
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      o[e] = pack2(v[2 * e] * rstd * to_f32(pw[2 * e]) + to_f32(pb[2 * e]),
                   v[2 * e + 1] * rstd * to_f32(pw[2 * e + 1]) + to_f32(pb[2 * e + 1]), T16());
    *reinterpret_cast<uint4*>(p.h + base + c) = *reinterpret_cast<const uint4*>(o);
  }
}

// fp32 form of add_layernorm_row_kernel for the tower run in fp32 / TF32: x, y, weight, bias,
// x_out and h are fp32; one CTA per row, four elements per thread.
struct AddLnF32Params {
  const float* x;
  const float* y;  // or NULL
  const float* w;
  const float* b;
  float* x_out;    // or NULL
  float* h;
  int M, W;
  float eps;
};

__global__ void __launch_bounds__(512) add_layernorm_f32_kernel(const AddLnF32Params p) {
  __shared__ float red[2][16];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int c = threadIdx.x * 4;
  const bool live = c < p.W;
  const long long base = static_cast<long long>(blockIdx.x) * p.W;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f), rw = v, rb = v;
  if (live) {
    rw = *reinterpret_cast<const float4*>(p.w + c);
    rb = *reinterpret_cast<const float4*>(p.b + c);
    v = *reinterpret_cast<const float4*>(p.x + base + c);
    if (p.y) {
      const float4 u = *reinterpret_cast<const float4*>(p.y + base + c);
      v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
      if (p.x_out) *reinterpret_cast<float4*>(p.x_out + base + c) = v;
    }
  }
  float sm = v.x + v.y + v.z + v.w;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, o);
  if (lane == 0) red[0][warp] = sm;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < nwarps; ++w) tot += red[0][w];
  const float mean = tot / static_cast<float>(p.W);
  float ss = 0.f;
  if (live) {
    v.x -= mean; v.y -= mean; v.z -= mean; v.w -= mean;
    ss = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) red[1][warp] = ss;
  __syncthreads();
  tot = 0.f;
  for (int w = 0; w < nwarps; ++w) tot += red[1][w];
  const float rstd = rsqrtf(tot / static_cast<float>(p.W) + p.eps);
  if (live)
    *reinterpret_cast<float4*>(p.h + base + c) = make_float4(v.x * rstd * rw.x + rb.x, v.y * rstd * rw.y + rb.y,
                                                              v.z * rstd * rw.z + rb.z, v.w * rstd * rw.w + rb.w);
}

}  // namespace tb

namespace tb {
static int launch_norm(const void* x, int64_t ldx, const float* weight, const float* mod, int64_t ldmod,
                       int rows_per_group, const void* ln_scale, const void* ln_shift, int M, int W, float eps, void* y,
                       int64_t ldy, void* y_planes, int out_shift, void* stream, int ln_affine = 0,
                       void* y_planes2 = nullptr, float* row_scale = nullptr) {
  if (!x || (!y && !y_planes && !y_planes2) || (!weight && !mod && !ln_scale)) return host::fail(TYBOK_ERR_ARG, "rmsnorm: null pointer argument");
  if ((y_planes2 != nullptr) != (row_scale != nullptr) || (reinterpret_cast<uintptr_t>(y_planes2) & 7))
    return host::fail(TYBOK_ERR_ARG, "norm: two-plane output needs both planes (8-byte aligned) and row_scale");
  if (M <= 0 || W <= 0 || W % 8 != 0 || W > NORM_MAX_VEC * 256)
    return host::fail(TYBOK_ERR_ARG, "rmsnorm: W must be a multiple of 8 and <= 4096");
  if (ldx % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (y && ((reinterpret_cast<uintptr_t>(y) & 15) || ldy % 8 != 0)) ||
      (y_planes && (reinterpret_cast<uintptr_t>(y_planes) & 7)) ||
      ((reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(mod)) & 15) || (mod && ldmod % 4 != 0))
    return host::fail(TYBOK_ERR_ARG, "rmsnorm: rows must be 16-byte aligned (ld % 8 == 0)");
  if (mod && rows_per_group <= 0) return host::fail(TYBOK_ERR_ARG, "rmsnorm: rows_per_group must be positive");
  if (out_shift < -60 || out_shift > 60) return host::fail(TYBOK_ERR_ARG, "rmsnorm: exponent shift out of range");
  if (int rc = host::require_sm100()) return rc;
  NormParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x); p.ldx = ldx; p.weight = weight; p.mod = mod; p.ldmod = ldmod;
  p.ln_scale = static_cast<const __nv_bfloat16*>(ln_scale); p.ln_shift = static_cast<const __nv_bfloat16*>(ln_shift);
  p.ln_affine = ln_affine;
  p.rows_per_group = rows_per_group > 0 ? rows_per_group : 1; p.M = M; p.W = W; p.eps = eps;
  p.plane_scale = ldexpf(1.0f, out_shift); p.planes = static_cast<uint8_t*>(y_planes);
  p.planes2 = static_cast<uint8_t*>(y_planes2); p.row_scale = row_scale;
  p.y = static_cast<__nv_bfloat16*>(y); p.ldy = ldy; p.pdl = host::pdl_enabled() ? 1 : 0;
  p.dbg = host::counter_buffer();
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((M + 3) / 4);
  cfg.blockDim = dim3(128);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl;
  const int per_lane = (W / 8 + 31) / 32;
  const bool full = W % 256 == 0 && W / 256 == per_lane && (per_lane & (per_lane - 1)) == 0;
  cudaError_t e;
  if (!ln_scale && per_lane >= 2) {  // one CTA per row
    cfg.gridDim = dim3(M);
    cfg.blockDim = dim3(per_lane * 32);
    e = cudaLaunchKernelEx(&cfg, rmsnorm_row_kernel, p);
  } else if (full && per_lane == 4) e = cudaLaunchKernelEx(&cfg, rmsnorm_kernel<4, true>, p);
  else if (full && per_lane == 8) e = cudaLaunchKernelEx(&cfg, rmsnorm_kernel<8, true>, p);
  else if (full && per_lane == 1) e = cudaLaunchKernelEx(&cfg, rmsnorm_kernel<1, true>, p);
  else if (full && per_lane == 2) e = cudaLaunchKernelEx(&cfg, rmsnorm_kernel<2, true>, p);
  else if (per_lane <= 1) e = cudaLaunchKernelEx(&cfg, rmsnorm_kernel<1, false>, p);
  else if (per_lane <= 2) e = cudaLaunchKernelEx(&cfg, rmsnorm_kernel<2, false>, p);
  else if (per_lane <= 4) e = cudaLaunchKernelEx(&cfg, rmsnorm_kernel<4, false>, p);
  else if (per_lane <= 8) e = cudaLaunchKernelEx(&cfg, rmsnorm_kernel<8, false>, p);
  else e = cudaLaunchKernelEx(&cfg, rmsnorm_kernel<NORM_MAX_VEC, false>, p);
  if (e != cudaSuccess) return host::fail_cuda("launch rmsnorm_kernel");
  host::count_launch();
  return TYBOK_OK;
}
}  // namespace tb

extern "C" {

int tybok_rmsnorm(const void* x, int64_t ldx, const float* weight, const float* mod, int64_t ldmod, int rows_per_group,
                  int M, int W, float eps, void* y, int64_t ldy, void* y_planes, int out_shift, void* stream) {
  return tb::launch_norm(x, ldx, weight, mod, ldmod, rows_per_group, nullptr, nullptr, M, W, eps, y, ldy, y_planes,
                         out_shift, stream);
}

int tybok_add_layernorm(const void* x, const void* y, const void* weight, const void* bias, int M, int W, float eps,
                        void* x_out, void* h, void* stream) {
  using namespace tb;
  if (!x || !weight || !bias || !h) return host::fail(TYBOK_ERR_ARG, "add_layernorm: null pointer argument");
  if (M <= 0 || W <= 0 || W % 8 != 0 || W > 8 * 256) return host::fail(TYBOK_ERR_ARG, "add_layernorm: W must be a multiple of 8 and <= 2048");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(weight) |
       reinterpret_cast<uintptr_t>(bias) | reinterpret_cast<uintptr_t>(x_out) | reinterpret_cast<uintptr_t>(h)) & 15)
    return host::fail(TYBOK_ERR_ARG, "add_layernorm: tensors must be 16-byte aligned");
  if (int rc = host::require_sm100()) return rc;
  AddLnParams p{static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(y),
                static_cast<const __nv_bfloat16*>(weight), static_cast<const __nv_bfloat16*>(bias),
                static_cast<__nv_bfloat16*>(x_out), static_cast<__nv_bfloat16*>(h), M, W, eps, host::pdl_enabled() ? 1 : 0};
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((M + 3) / 4);
  cfg.blockDim = dim3(128);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 0;  // neighbours are library kernels that know nothing of programmatic launches
  p.pdl = 0;
  const int per_lane = (W / 8 + 31) / 32;
  cudaError_t e;
  if (per_lane >= 2 && M >= 64) {  // one CTA per row
    cfg.gridDim = dim3(M);
    cfg.blockDim = dim3(per_lane * 32);
    e = cudaLaunchKernelEx(&cfg, add_layernorm_row_kernel, p);
  } else if (per_lane <= 1) e = cudaLaunchKernelEx(&cfg, add_layernorm_kernel<1>, p);
  else if (per_lane <= 2) e = cudaLaunchKernelEx(&cfg, add_layernorm_kernel<2>, p);
  else if (per_lane <= 5) e = cudaLaunchKernelEx(&cfg, add_layernorm_kernel<5>, p);
  else e = cudaLaunchKernelEx(&cfg, add_layernorm_kernel<8>, p);
  if (e != cudaSuccess) return host::fail_cuda("launch add_layernorm_kernel");
  host::count_launch();
  return TYBOK_OK;
}

static int launch_add_layernorm_mixed(const float* x, const void* y, const void* weight, const void* bias, int M, int W,
                                      float eps, float* x_out, void* h, void* stream, bool half) {
  using namespace tb;
  if (!x || !weight || !bias || !h) return host::fail(TYBOK_ERR_ARG, "add_layernorm_mixed: null pointer argument");
  if (M <= 0 || W <= 0 || W % 8 != 0 || W > 2048) return host::fail(TYBOK_ERR_ARG, "add_layernorm_mixed: W must be a multiple of 8 and <= 2048");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(weight) |
       reinterpret_cast<uintptr_t>(bias) | reinterpret_cast<uintptr_t>(x_out) | reinterpret_cast<uintptr_t>(h)) & 15)
    return host::fail(TYBOK_ERR_ARG, "add_layernorm_mixed: tensors must be 16-byte aligned");
  if (int rc = host::require_sm100()) return rc;
  const int threads = ((W / 8) + 31) / 32 * 32;
  if (half) {
    AddLnMixedParams<__half> p{x, static_cast<const __half*>(y), static_cast<const __half*>(weight),
                               static_cast<const __half*>(bias), x_out, static_cast<__half*>(h), M, W, eps};
    add_layernorm_mixed_kernel<__half><<<M, threads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  } else {
    AddLnMixedParams<__nv_bfloat16> p{x, static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(weight),
                                      static_cast<const __nv_bfloat16*>(bias), x_out, static_cast<__nv_bfloat16*>(h), M, W, eps};
    add_layernorm_mixed_kernel<__nv_bfloat16><<<M, threads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  }
  if (cudaGetLastError() != cudaSuccess) return host::fail_cuda("launch add_layernorm_mixed_kernel");
  host::count_launch();
  return TYBOK_OK;
}

int tybok_add_layernorm_mixed(const float* x, const void* y, const void* weight, const void* bias, int M, int W, float eps,
                              float* x_out, void* h, void* stream) {
  return launch_add_layernorm_mixed(x, y, weight, bias, M, W, eps, x_out, h, stream, false);
}

int tybok_add_layernorm_mixed_f16(const float* x, const void* y, const void* weight, const void* bias, int M, int W,
                                  float eps, float* x_out, void* h, void* stream) {
  return launch_add_layernorm_mixed(x, y, weight, bias, M, W, eps, x_out, h, stream, true);
}

int tybok_add_layernorm_f32(const float* x, const float* y, const float* weight, const float* bias, int M, int W,
                            float eps, float* x_out, float* h, void* stream) {
  using namespace tb;
  if (!x || !weight || !bias || !h) return host::fail(TYBOK_ERR_ARG, "add_layernorm_f32: null pointer argument");
  if (M <= 0 || W <= 0 || W % 4 != 0 || W > 2048) return host::fail(TYBOK_ERR_ARG, "add_layernorm_f32: W must be a multiple of 4 and <= 2048");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(weight) |
       reinterpret_cast<uintptr_t>(bias) | reinterpret_cast<uintptr_t>(x_out) | reinterpret_cast<uintptr_t>(h)) & 15)
    return host::fail(TYBOK_ERR_ARG, "add_layernorm_f32: tensors must be 16-byte aligned");
  if (int rc = host::require_sm100()) return rc;
  AddLnF32Params p{x, y, weight, bias, x_out, h, M, W, eps};
  add_layernorm_f32_kernel<<<M, ((W / 4) + 31) / 32 * 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  if (cudaGetLastError() != cudaSuccess) return host::fail_cuda("launch add_layernorm_f32_kernel");
  host::count_launch();
  return TYBOK_OK;
}

int tybok_layernorm_modulate(const void* x, int64_t ldx, const void* shift, const void* scale, int M, int W, float eps,
                             void* y, int64_t ldy, void* y_planes, int out_shift, void* stream) {
  if (!shift || !scale) return tb::host::fail(TYBOK_ERR_ARG, "layernorm_modulate: null shift/scale");
  if ((reinterpret_cast<uintptr_t>(shift) | reinterpret_cast<uintptr_t>(scale)) & 15)
    return tb::host::fail(TYBOK_ERR_ARG, "layernorm_modulate: shift/scale must be 16-byte aligned");
  return tb::launch_norm(x, ldx, nullptr, nullptr, 0, 1, scale, shift, M, W, eps, y, ldy, y_planes, out_shift, stream);
}


int tybok_layernorm_affine(const void* x, int64_t ldx, const void* weight, const void* bias, int M, int W, float eps,
                           void* y, int64_t ldy, void* y_planes, int out_shift, void* stream) {
  if (!weight || !bias) return tb::host::fail(TYBOK_ERR_ARG, "layernorm_affine: null weight/bias");
  if ((reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(bias)) & 15)
    return tb::host::fail(TYBOK_ERR_ARG, "layernorm_affine: weight/bias must be 16-byte aligned");
  return tb::launch_norm(x, ldx, nullptr, nullptr, 0, 1, weight, bias, M, W, eps, y, ldy, y_planes, out_shift, stream, 1);
}

int tybok_norm_planes2(const void* x, int64_t ldx, int mode, const void* a, const void* b, int64_t ldmod, int rows_per_group,
                       int M, int W, float eps, void* y_planes2, float* row_scale, void* stream) {
  using namespace tb;
  switch (mode) {
    case TYBOK_NORM_RMS:
      return launch_norm(x, ldx, static_cast<const float*>(a), nullptr, 0, 1, nullptr, nullptr, M, W, eps, nullptr, 0, nullptr,
                         0, stream, 0, y_planes2, row_scale);
    case TYBOK_NORM_ADARMS:
      return launch_norm(x, ldx, nullptr, static_cast<const float*>(a), ldmod, rows_per_group, nullptr, nullptr, M, W, eps,
                         nullptr, 0, nullptr, 0, stream, 0, y_planes2, row_scale);
    case TYBOK_NORM_LN_MODULATE:  // a = shift, b = scale (bf16 [W])
    case TYBOK_NORM_LN_AFFINE:    // a = weight, b = bias (bf16 [W])
      if (!a || !b || ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15))
        return host::fail(TYBOK_ERR_ARG, "norm_planes2: the two bf16 vectors must be given, 16-byte aligned");
      return mode == TYBOK_NORM_LN_MODULATE
                 ? launch_norm(x, ldx, nullptr, nullptr, 0, 1, b, a, M, W, eps, nullptr, 0, nullptr, 0, stream, 0, y_planes2, row_scale)
                 : launch_norm(x, ldx, nullptr, nullptr, 0, 1, a, b, M, W, eps, nullptr, 0, nullptr, 0, stream, 1, y_planes2, row_scale);
    default:
      return host::fail(TYBOK_ERR_ARG, "norm_planes2: unknown mode");
  }
}

}  // extern "C"
