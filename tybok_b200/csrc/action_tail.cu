// Per-step tail of the action-expert loop in one launch (a cluster of CTAs per four action tokens,
// each CTA owning a slice of the expert width):
//   y   = bf16( AdaRMS(x; scale, shift) )                    final norm, scale/shift-only modulation
//   v   = W_out . float(y) + b_out                           fp32 velocity, [A] per token
//   x_t = x_t + dt * v                                       forward-Euler update, fp32
//   h   = bf16( W_in . x_t + b_in )                          next step's suffix embedding
// following tybok/policies/pi05/models/flow_matching.py:193-254,464-502,505-556 (eager branch) and
// the reference's fused final-norm + out-projection kernel (flow_matching.py:41-150).  With
// `x == NULL` only the last line runs (the first step's embedding of the initial noise).
// All projections are true fp32 (weights fp32, fp32 FMA), like the reference's fp32 modules.
#include <algorithm>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/tybok_b200.h"
#include "host_util.h"
#include "ptx.cuh"

namespace tb {

constexpr int TAIL_A = 32;        // padded action dimension
constexpr int TAIL_T = 4;         // action tokens per cluster
constexpr int TAIL_THREADS = 256;

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

struct __align__(16) TailShared {
  float xn[TAIL_T][256];       // this CTA's column slice of the normalised rows (bf16-rounded values)
  float red[TAIL_T][2];
  float part_ss[TAIL_T];       // sum of squares over this slice
  float vp[TAIL_T][TAIL_A];    // out-projection partial sums over this slice
  float xt[TAIL_T][TAIL_A];    // x_t of the group's tokens, old then updated
};

__device__ __forceinline__ float tail_peer_f32(const float* local, uint32_t rank, bool clustered) {
  if (!clustered) return *local;
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(dsmem_addr(smem_u32(local), rank)));
  return v;
}

// A cluster of C CTAs per group of TAIL_T tokens; CTA r owns columns [r*KS, (r+1)*KS) of the expert
// width: it reads that slice of the hidden rows and of both fp32 projection matrices (32 KB
// instead of the 256 KB a CTA per token reads), and the slices meet through distributed shared
// memory twice: the row sums of squares, and the 32 partial dot products per token.
template <int KS>
__global__ void __launch_bounds__(TAIL_THREADS) action_tail_kernel(const TailParams p) {
  __shared__ TailShared sh;
  if (p.pdl) pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int C = gridDim.x;
  const bool clustered = C > 1;
  const uint32_t rank = clustered ? cluster_ctarank() : 0u;
  const int m0 = blockIdx.y * TAIL_T;
  const int k0 = static_cast<int>(rank) * KS;
  constexpr int NI = KS / 128;

  // Projection weights depend on nothing that runs before this kernel: fetch them first.
  float4 wo[4][NI], wi[NI][4];
  if (p.x) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < NI; ++i)
        wo[j][i] = *reinterpret_cast<const float4*>(p.w_out + static_cast<long long>(warp * 4 + j) * p.W + k0 + lane * 4 + 128 * i);
  }
  if (p.h) {
#pragma unroll
    for (int i = 0; i < NI; ++i)
#pragma unroll
      for (int q = 0; q < 4; ++q)
        wi[i][q] = *reinterpret_cast<const float4*>(p.w_in + static_cast<long long>(k0 + (tid >> 1) + 128 * i) * TAIL_A + (tid & 1) * 16 + 4 * q);
  }
  // The modulation row, like the biases, is a per-step constant nobody has touched since the
  // last chunk (cold in L2): fetch it before waiting as well.
  constexpr int PT = KS / 64;
  float msc[PT], msh[PT];
  float bo = 0.f;
  if (p.x) {
    const int t = tid >> 6, c = (tid & 63) * PT;
    const float* mod = p.mod + static_cast<long long>(m0 + t < p.M ? (m0 + t) / p.rows_per_group : 0) * p.ldmod + k0 + c;
#pragma unroll
    for (int e = 0; e < PT; ++e) { msc[e] = mod[e]; msh[e] = mod[p.W + e]; }
    bo = p.b_out[lane];
  }
  float bi[NI];
  if (p.h) {
#pragma unroll
    for (int i = 0; i < NI; ++i) bi[i] = p.b_in[k0 + (tid >> 1) + 128 * i];
  }
  if (p.pdl) pdl_wait();
  if (tid < TAIL_T * TAIL_A) {
    const int t = tid >> 5;
    sh.xt[t][lane] = m0 + t < p.M ? p.x_t[static_cast<long long>(m0 + t) * TAIL_A + lane] : 0.f;
  }
  if (p.x) {
    // ---- final AdaRMS norm of this slice: 64 threads per token, KS/64 consecutive columns each
    const int t = tid >> 6, c = (tid & 63) * PT;
    const bool live = m0 + t < p.M;
    float xv[PT];
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < PT; ++e) {
      xv[e] = live ? __bfloat162float(p.x[static_cast<long long>(m0 + t) * p.ldx + k0 + c + e]) : 0.f;
      ss += xv[e] * xv[e];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) sh.red[t][warp & 1] = ss;
    __syncthreads();
    if (tid < TAIL_T) sh.part_ss[tid] = sh.red[tid][0] + sh.red[tid][1];
    if (clustered) cluster_sync_all(); else __syncthreads();
    float tot = 0.f;
    for (int r = 0; r < C; ++r) tot += tail_peer_f32(&sh.part_ss[t], r, clustered);  // rank order: reproducible
    const float rstd = rsqrtf(tot / static_cast<float>(p.W) + p.eps);
#pragma unroll
    for (int e = 0; e < PT; ++e) sh.xn[t][c + e] = live ? bf16_round(xv[e] * rstd * (1.0f + msc[e]) + msh[e]) : 0.f;
    __syncthreads();
    // ---- out-projection partials: warp w owns outputs 4w..4w+3, lane covers 4 columns per 128
    float acc[4][TAIL_T];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int tt = 0; tt < TAIL_T; ++tt) acc[j][tt] = 0.f;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
#pragma unroll
      for (int tt = 0; tt < TAIL_T; ++tt) {
        const float4 xq = *reinterpret_cast<const float4*>(&sh.xn[tt][lane * 4 + 128 * i]);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          acc[j][tt] += wo[j][i].x * xq.x + wo[j][i].y * xq.y + wo[j][i].z * xq.z + wo[j][i].w * xq.w;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int tt = 0; tt < TAIL_T; ++tt) {
        float v = acc[j][tt];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) sh.vp[tt][warp * 4 + j] = v;
      }
    if (clustered) cluster_sync_all(); else __syncthreads();
    // ---- Euler update: every CTA of the cluster forms the same 4 x 32 new values
    if (tid < TAIL_T * TAIL_A) {
      const int tt = tid >> 5;
      float v = 0.f;
      for (int r = 0; r < C; ++r) v += tail_peer_f32(&sh.vp[tt][lane], r, clustered);
      const float nx = sh.xt[tt][lane] + p.dt * (v + bo);
      sh.xt[tt][lane] = nx;
      if (rank == 0 && m0 + tt < p.M) p.x_t[static_cast<long long>(m0 + tt) * TAIL_A + lane] = nx;
    }
    if (clustered) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");  // done reading the peers
  }
  __syncthreads();
  if (p.h) {
    // ---- next suffix embedding of this slice: a thread pair per output column, 16 actions each
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int kl = (tid >> 1) + 128 * i, half = tid & 1;
      float s[TAIL_T];
#pragma unroll
      for (int tt = 0; tt < TAIL_T; ++tt) {
        s[tt] = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 xq = *reinterpret_cast<const float4*>(&sh.xt[tt][half * 16 + 4 * q]);
          s[tt] += wi[i][q].x * xq.x + wi[i][q].y * xq.y + wi[i][q].z * xq.z + wi[i][q].w * xq.w;
        }
        s[tt] += __shfl_xor_sync(0xffffffffu, s[tt], 1);
      }
      const float bias = bi[i];
#pragma unroll
      for (int tt = 0; tt < TAIL_T / 2; ++tt) {  // each thread of the pair stores two of the four tokens
        const int tk = half * (TAIL_T / 2) + tt;
        const float val = half == 0 ? s[tt] : s[TAIL_T / 2 + tt];
        if (m0 + tk < p.M) p.h[static_cast<long long>(m0 + tk) * p.W + k0 + kl] = __float2bfloat16_rn(val + bias);
      }
    }
  }
  if (p.x && clustered) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
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
  if ((reinterpret_cast<uintptr_t>(w_in) | reinterpret_cast<uintptr_t>(w_out)) & 15)
    return host::fail(TYBOK_ERR_ARG, "action_tail: projection weights must be 16-byte aligned");
  if (int rc = host::require_sm100()) return rc;
  TailParams p{static_cast<const __nv_bfloat16*>(x), ldx, mod, ldmod, rows_per_group > 0 ? rows_per_group : 1, eps, w_out,
               b_out, x_t, dt, w_in, b_in, static_cast<__nv_bfloat16*>(h), M, W, host::pdl_enabled() ? 1 : 0};
  const int slices = std::min(8, W / 128);  // cluster size; 128 or 256 columns per CTA
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(slices, (M + TAIL_T - 1) / TAIL_T);
  cfg.blockDim = dim3(TAIL_THREADS);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (p.pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (slices > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = slices;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  const cudaError_t e = W / slices == 128 ? cudaLaunchKernelEx(&cfg, action_tail_kernel<128>, p)
                                          : cudaLaunchKernelEx(&cfg, action_tail_kernel<256>, p);
  if (e != cudaSuccess) return host::fail_cuda("launch action_tail_kernel");
  host::count_launch();
  return TYBOK_OK;
}
