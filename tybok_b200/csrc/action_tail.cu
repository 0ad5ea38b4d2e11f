// Per-step tail of the action-expert loop in one launch, one CTA per action token:
//   y   = bf16( AdaRMS(x; scale, shift) )                    final norm, scale/shift-only modulation
//   v   = W_out . float(y) + b_out                           fp32 velocity, [A] per token
//   x_t = x_t + dt * v                                       forward-Euler update, fp32
//   h   = bf16( W_in . x_t + b_in )                          next step's suffix embedding
// following tybok/policies/pi05/models/flow_matching.py:193-254,464-502,505-556 (eager branch) and
// the reference's fused final-norm + out-projection kernel (flow_matching.py:41-150).  With
// `x == NULL` only the last line runs (the first step's embedding of the initial noise).
// All projections are true fp32 (weights fp32, fp32 FMA), like the reference's fp32 modules.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/tybok_b200.h"
#include "host_util.h"
#include "ptx.cuh"

namespace tb {

constexpr int TAIL_A = 32;        // padded action dimension (one output per lane)
constexpr int TAIL_MAX_W = 2048;  // expert width limit: 64 elements per lane

struct TailParams {
  const __nv_bfloat16* x;  // [M, W] last expert hidden state, or NULL
  long long ldx;
  const float* mod;        // [groups, ldmod]: scale at [0,W), shift at [W,2W)
  long long ldmod;
  int rows_per_group;
  float eps;
  const float* w_out;      // [A, W]
  const float* b_out;      // [A]
  float* x_t;              // [M, A] fp32, updated in place
  float dt;
  const float* w_in;       // [W, A]
  const float* b_in;       // [W]
  __nv_bfloat16* h;        // [M, W] next suffix embedding, or NULL
  int M, W, pdl;
};

// One CTA (4 warps) per token: every warp normalises the row (2 KB, cheap), warp w produces the
// 8 outputs a = 8w..8w+7 with lane-interleaved k (coalesced weight rows), the 32 new x_t values
// meet in shared memory, and all 128 threads compute the next embedding.
template <int PER_LANE>  // W / 32: a compile-time trip count keeps every load unpredicated and hoistable
__global__ void __launch_bounds__(128) action_tail_kernel(const TailParams p) {
  __shared__ float xt_s[TAIL_A];
  if (p.pdl) pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x;
  if (p.pdl) pdl_wait();
  if (threadIdx.x < TAIL_A) xt_s[threadIdx.x] = p.x_t[static_cast<long long>(m) * TAIL_A + threadIdx.x];
  __syncthreads();
  if (p.x) {
    // k = lane + 32 * i
    const __nv_bfloat16* row = p.x + m * p.ldx;
    float xv[PER_LANE];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      xv[i] = __bfloat162float(row[lane + 32 * i]);
      ss += xv[i] * xv[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss / static_cast<float>(p.W) + p.eps);
    const float* mod = p.mod + static_cast<long long>(m / p.rows_per_group) * p.ldmod;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int k = lane + 32 * i;
      xv[i] = bf16_round(xv[i] * rstd * (1.0f + mod[k]) + mod[p.W + k]);
    }
    float mine = 0.f;
    // Fully unrolled: all weight loads of the 8 outputs are in flight together.
#pragma unroll
    for (int j = 0; j < TAIL_A / 4; ++j) {
      const int a = warp * (TAIL_A / 4) + j;
      const float* wr = p.w_out + static_cast<long long>(a) * p.W;
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) s += xv[i] * wr[lane + 32 * i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == j) mine = s;
    }
    __syncthreads();  // everyone has read the old x_t
    if (lane < TAIL_A / 4) {
      const int a = warp * (TAIL_A / 4) + lane;
      const float nx = xt_s[a] + p.dt * (mine + p.b_out[a]);
      xt_s[a] = nx;
      p.x_t[static_cast<long long>(m) * TAIL_A + a] = nx;
    }
    __syncthreads();
  }
  if (p.h) {
#pragma unroll
    for (int kk = 0; kk < PER_LANE / 4; ++kk) {
      const int k = threadIdx.x + 128 * kk;  // h[k] = sum_a W_in[k, a] * x_t[a] + b_in[k]
      const float4* wr = reinterpret_cast<const float4*>(p.w_in + static_cast<long long>(k) * TAIL_A);
      float s = 0.f;
#pragma unroll
      for (int a4 = 0; a4 < TAIL_A / 4; ++a4) {
        const float4 w = wr[a4];
        s += w.x * xt_s[4 * a4] + w.y * xt_s[4 * a4 + 1] + w.z * xt_s[4 * a4 + 2] + w.w * xt_s[4 * a4 + 3];
      }
      p.h[static_cast<long long>(m) * p.W + k] = __float2bfloat16_rn(s + p.b_in[k]);
    }
  }
}

}  // namespace tb

extern "C" int tybok_action_tail(const void* x, int64_t ldx, const float* mod, int64_t ldmod, int rows_per_group,
                                 float eps, const float* w_out, const float* b_out, float* x_t, float dt,
                                 const float* w_in, const float* b_in, void* h, int M, int W, int A, void* stream) {
  using namespace tb;
  if (!x_t || (!x && !h)) return host::fail(TYBOK_ERR_ARG, "action_tail: null pointer argument");
  if (x && (!mod || !w_out || !b_out)) return host::fail(TYBOK_ERR_ARG, "action_tail: norm/out-projection inputs missing");
  if (h && (!w_in || !b_in)) return host::fail(TYBOK_ERR_ARG, "action_tail: in-projection inputs missing");
  if (A != TAIL_A) return host::fail(TYBOK_ERR_ARG, "action_tail: the padded action dimension must be 32");
  if (M <= 0 || (W != 128 && W != 256 && W != 512 && W != 1024 && W != 2048))
    return host::fail(TYBOK_ERR_ARG, "action_tail: W must be 128, 256, 512, 1024 or 2048");
  if (x && rows_per_group <= 0) return host::fail(TYBOK_ERR_ARG, "action_tail: rows_per_group must be positive");
  if (w_in && (reinterpret_cast<uintptr_t>(w_in) & 15)) return host::fail(TYBOK_ERR_ARG, "action_tail: w_in must be 16-byte aligned");
  if (int rc = host::require_sm100()) return rc;
  TailParams p{static_cast<const __nv_bfloat16*>(x), ldx, mod, ldmod, rows_per_group > 0 ? rows_per_group : 1, eps, w_out,
               b_out, x_t, dt, w_in, b_in, static_cast<__nv_bfloat16*>(h), M, W, host::pdl_enabled() ? 1 : 0};
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(M);
  cfg.blockDim = dim3(128);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl;
  cudaError_t e;
  switch (W) {
    case 128: e = cudaLaunchKernelEx(&cfg, action_tail_kernel<4>, p); break;
    case 256: e = cudaLaunchKernelEx(&cfg, action_tail_kernel<8>, p); break;
    case 512: e = cudaLaunchKernelEx(&cfg, action_tail_kernel<16>, p); break;
    case 1024: e = cudaLaunchKernelEx(&cfg, action_tail_kernel<32>, p); break;
    default: e = cudaLaunchKernelEx(&cfg, action_tail_kernel<64>, p); break;
  }
  if (e != cudaSuccess) return host::fail_cuda("launch action_tail_kernel");
  host::count_launch();
  return TYBOK_OK;
}
