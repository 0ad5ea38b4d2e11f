// W8A16 linear for sm_100a: e4m3 weights with per-output-channel fp32 scales, bf16
// activations, fp32 accumulation in tensor memory.
//
// Orientation ("swap-AB"): the weight tile is the 128-row M side of the UMMA and the tokens
// are its N side, D[n, m] = sum_k W[n,k] x[m,k], so any token count from 1 to 256 fills the
// 128 tensor-memory lanes and the output channel of a thread is fixed (scale/bias are
// per-thread scalars in the epilogue).
//
// Data flow per CTA (one 128 x token_tile output tile, one K range when split-K is on):
//   warp 0      TMA producer: weight tiles (128 rows x 128 e4m3 bytes, 128B swizzle) and the
//               matching bf16 activation tile into an n-stage shared-memory ring.
//   warps 2-9   expand e4m3 -> bf16 exactly (bit placement + one multiply by 2^120) and write
//               the result into tensor memory as the A operand (tcgen05.st); the weights never
//               take a second trip through shared memory.
//   warp 1      one thread issues tcgen05.mma (A from TMEM, B = activations from shared memory).
//   warps 2-9   epilogue: tcgen05.ld the accumulator, apply scale/bias and the fused epilogue,
//               store bf16; with split-K, store fp32 partials and let the last-arriving CTA of
//               a tile add them in split order (deterministic; no CTA ever waits for another).
//
// Algorithmic HBM bytes per launch: N*K (weights) + 4*N (scales) + 2*M*K (x) + 2*M*N (y).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstring>

#include "../../include/tybok_b200.h"
#include "host_util.h"
#include "ptx.cuh"

namespace tb {

constexpr int BN = 128;          // weight rows per tile = UMMA M
constexpr int BK = 128;          // K per pipeline stage (one 128-byte swizzle row of e4m3)
constexpr int W_TILE_BYTES = BN * BK;
constexpr int MAX_STAGES = 8;
constexpr int A_SLOTS = 4;       // tensor-memory A slots, 64 columns (128 bf16 of K) each
constexpr int A_COL0 = 256;      // accumulators live in columns [0,256), A slots in [256,512)
constexpr int TMEM_COLS = 512;
constexpr int CVT_WARPS = 8;
constexpr int THREADS = 32 * (2 + CVT_WARPS);
constexpr int DYN_SMEM_MAX = 226 * 1024;  // 227 KB per CTA minus 1 KB left for static shared memory

enum : int { EPI_NONE = 0, EPI_GELU = 1, EPI_RESIDUAL = 2, EPI_GEGLU = 3 };

struct GemmParams {
  int M, N, K;
  int bt;            // token tile (UMMA N), multiple of 16, <= 256 (<= 128 when nw == 2)
  int nw;            // weight matrices per CTA: 1, or 2 for the gated form
  int splits;        // split-K factor
  int kb_total;      // ceil(K / BK)
  int kb_per_split;
  int nstages;
  int epi;
  int pdl;
  const float* scale0;
  const float* scale1;
  const __nv_bfloat16* bias0;
  __nv_bfloat16* y;
  long long ldy;
  const __nv_bfloat16* res;
  long long ldres;
  const void* gate;
  long long ldgate;
  int rows_per_gate;
  int gate_bf16;
  float* partials;
  int* counters;
  int* status;
};

struct __align__(8) Barriers {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t a_full[A_SLOTS];
  uint64_t a_empty[A_SLOTS];
  uint64_t tmem_full;
  uint64_t epi;  // epilogue warps meet here (bounded), twice per split-K tile
  uint32_t tmem_base;
  volatile int abort;
  int is_last;
};


__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitLimitCycles) return false;
  }
  return true;
}

__device__ __forceinline__ void fail(Barriers* b, int* status, int code) {
  b->abort = 1;
  if (status) atomicCAS(status, 0, code);
}

// Meeting point of the epilogue warps (one arrival per warp), with the same bounded wait as
// every other barrier here. `phase` is 0 for the first meeting of a launch, 1 for the second.
__device__ __forceinline__ bool epi_sync(Barriers* b, uint32_t phase, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(&b->epi);
  return wait_or_abort(&b->epi, phase, &b->abort);
}

__device__ __forceinline__ float load_gate(const GemmParams& p, int m, int n) {
  if (!p.gate) return 1.0f;
  const long long g = static_cast<long long>(m / p.rows_per_gate) * p.ldgate + n;
  if (p.gate_bf16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p.gate)[g]);
  return bf16_round(static_cast<const float*>(p.gate)[g]);
}

// Final value of one output element from its accumulator(s); every rounding point is the one
// the bf16 torch modules of the reference have (linear output, GELU output, product, sum).
__device__ __forceinline__ float finish(const GemmParams& p, float acc0, float acc1, float s0, float s1, float b0,
                                        int m, int n) {
  float v = bf16_round(acc0 * s0 + b0);
  if (p.epi == EPI_GELU) {
    v = gelu_tanh_f(v);
  } else if (p.epi == EPI_GEGLU) {
    const float u = bf16_round(acc1 * s1);
    v = bf16_round(gelu_tanh_f(v)) * u;
  } else if (p.epi == EPI_RESIDUAL) {
    if (p.gate) v = bf16_round(v * load_gate(p, m, n));
    v = __bfloat162float(p.res[static_cast<long long>(m) * p.ldres + n]) + v;
  }
  return v;
}

__global__ void __launch_bounds__(THREADS, 1)
w8a16_gemm_kernel(const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w1,
                  const __grid_constant__ CUtensorMap tm_x, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ Barriers bars;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int ns = p.nstages;
  const int stage_bytes = p.nw * W_TILE_BYTES + p.bt * 256;
  const int x_off = p.nw * W_TILE_BYTES;  // activation tile offset inside a stage
  const int a_stages = A_SLOTS / p.nw;

  const int t_tile = blockIdx.x, n_tile = blockIdx.y, split = blockIdx.z;
  const int kb0 = split * p.kb_per_split;
  const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
  const int nkb = kb1 - kb0;

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_w0);
    if (p.nw == 2) tma_prefetch_desc(&tm_w1);
    tma_prefetch_desc(&tm_x);
    for (int i = 0; i < MAX_STAGES; ++i) {
      mbar_init(&bars.full[i], 1);
      mbar_init(&bars.empty[i], 1);
    }
    for (int i = 0; i < A_SLOTS; ++i) {
      mbar_init(&bars.a_full[i], CVT_WARPS);
      mbar_init(&bars.a_empty[i], 1);
    }
    mbar_init(&bars.tmem_full, 1);
    mbar_init(&bars.epi, CVT_WARPS);
    bars.abort = 0;
    bars.is_last = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars.tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars.tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int issued = 0;
      bool ok = true;
      // Weights do not depend on the previous kernel in the stream: start streaming them
      // before waiting for it; activations are loaded after the dependency has resolved.
      const int pre = min(ns, nkb);
      for (int i = 0; i < pre; ++i) {
        uint8_t* st = smem + i * stage_bytes;
        mbar_arrive_expect_tx(&bars.full[i], stage_bytes);
        const int k0 = (kb0 + i) * BK;
        tma_load_2d(st, &tm_w0, &bars.full[i], k0, n_tile * BN);
        if (p.nw == 2) tma_load_2d(st + W_TILE_BYTES, &tm_w1, &bars.full[i], k0, n_tile * BN);
      }
      if (p.pdl) pdl_wait();
      for (int i = 0; i < pre; ++i) {
        uint8_t* st = smem + i * stage_bytes + x_off;
        const int k0 = (kb0 + i) * BK;
        tma_load_2d(st, &tm_x, &bars.full[i], k0, t_tile * p.bt);
        tma_load_2d(st + p.bt * 128, &tm_x, &bars.full[i], k0 + 64, t_tile * p.bt);
      }
      issued = pre;
      for (int i = pre; i < nkb && ok; ++i) {
        const int s = i % ns;
        const uint32_t ph = (i / ns) & 1;
        if (!wait_or_abort(&bars.empty[s], ph ^ 1, &bars.abort)) {
          fail(&bars, p.status, TYBOK_DEV_TIMEOUT_PRODUCER);
          ok = false;
          break;
        }
        uint8_t* st = smem + s * stage_bytes;
        mbar_arrive_expect_tx(&bars.full[s], stage_bytes);
        const int k0 = (kb0 + i) * BK;
        tma_load_2d(st, &tm_w0, &bars.full[s], k0, n_tile * BN);
        if (p.nw == 2) tma_load_2d(st + W_TILE_BYTES, &tm_w1, &bars.full[s], k0, n_tile * BN);
        tma_load_2d(st + x_off, &tm_x, &bars.full[s], k0, t_tile * p.bt);
        tma_load_2d(st + x_off + p.bt * 128, &tm_x, &bars.full[s], k0 + 64, t_tile * p.bt);
        issued = i + 1;
      }
      if (p.pdl) pdl_launch_dependents();
      if (!ok || bars.abort) {
        // Unwinding: do not leave the CTA while its own bulk copies may still land in its
        // shared memory. Wait (bounded) for the newest copy of every stage.
        for (int i = max(0, issued - ns); i < issued; ++i) mbar_wait(&bars.full[i % ns], (i / ns) & 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = idesc_bf16_f32(BN, p.bt);
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % ns;
        const uint32_t ph = (i / ns) & 1;
        const int a = i % a_stages;
        const uint32_t aph = (i / a_stages) & 1;
        if (!wait_or_abort(&bars.full[s], ph, &bars.abort) || !wait_or_abort(&bars.a_full[a], aph, &bars.abort)) {
          fail(&bars, p.status, TYBOK_DEV_TIMEOUT_MMA);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t x_base = smem_u32(smem + s * stage_bytes + x_off);
        for (int w = 0; w < p.nw; ++w) {
          const uint32_t a_col = A_COL0 + (a * p.nw + w) * 64;
          const uint32_t d_col = w * p.bt;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t b_addr = x_base + (j >> 2) * (p.bt * 128) + (j & 3) * 32;
            umma_ts_bf16(tmem + d_col, tmem + a_col + j * 8, smem_desc_sw128(b_addr), idesc, (i > 0 || j > 0) ? 1u : 0u);
          }
        }
        tc_commit(&bars.empty[s]);
        tc_commit(&bars.a_empty[a]);
      }
      if (ok) tc_commit(&bars.tmem_full);
    }
  } else {
    // ------------------------------------------------------------ e4m3 -> bf16 expansion into TMEM
    const int cw = warp - 2;
    const int q = warp & 3;       // TMEM lane quadrant this warp may access
    const int half = cw >> 2;     // which 64-byte half of the 128-byte K row
    const int row = q * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    bool ok = true;
    for (int i = 0; i < nkb && ok; ++i) {
      const int s = i % ns;
      const uint32_t ph = (i / ns) & 1;
      const int a = i % a_stages;
      const uint32_t aph = (i / a_stages) & 1;
      // Warp-uniform outcome: the tcgen05.st below is warp-collective.
      const bool ready = wait_or_abort(&bars.a_empty[a], aph ^ 1, &bars.abort) && wait_or_abort(&bars.full[s], ph, &bars.abort);
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) fail(&bars, p.status, TYBOK_DEV_TIMEOUT_CONVERT);
        ok = false;
        break;
      }
      for (int w = 0; w < p.nw; ++w) {
        const uint8_t* rowp = smem + s * stage_bytes + w * W_TILE_BYTES + row * 128;
        uint32_t v[32];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int chunk = half * 4 + c;
          const uint4 d = *reinterpret_cast<const uint4*>(rowp + ((chunk ^ (row & 7)) << 4));
          e4m3x4_to_bf16x4(d.x, v[c * 8 + 0], v[c * 8 + 1]);
          e4m3x4_to_bf16x4(d.y, v[c * 8 + 2], v[c * 8 + 3]);
          e4m3x4_to_bf16x4(d.z, v[c * 8 + 4], v[c * 8 + 5]);
          e4m3x4_to_bf16x4(d.w, v[c * 8 + 6], v[c * 8 + 7]);
        }
        tmem_st32(tmem + lane_addr + A_COL0 + (a * p.nw + w) * 64 + half * 32, v);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.a_full[a]);
    }

    // ------------------------------------------------------------ epilogue
    if (ok) {  // `ok` is warp-uniform here; keep it so: tcgen05.ld below is warp-collective
      ok = __all_sync(0xffffffffu, wait_or_abort(&bars.tmem_full, 0, &bars.abort));
      if (!ok && lane == 0) fail(&bars, p.status, TYBOK_DEV_TIMEOUT_EPILOGUE);
    }
    if (ok) {
      tc_fence_after();
      if (p.pdl) pdl_wait();  // y / residual / workspace may still be in use by the previous kernel
      const int n = n_tile * BN + row;
      const bool n_ok = n < p.N;
      const float s0 = n_ok ? p.scale0[n] : 0.f;
      const float s1 = (n_ok && p.nw == 2) ? p.scale1[n] : 0.f;
      const float b0 = (n_ok && p.bias0) ? __bfloat162float(p.bias0[n]) : 0.f;
      const int nchunks = p.bt / 8;
      const int m_base = t_tile * p.bt;
      if (p.splits == 1) {
        for (int c = half; c < nchunks; c += 2) {
          uint32_t a0[8], a1[8];
          tmem_ld8(tmem + lane_addr + c * 8, a0);
          if (p.nw == 2) tmem_ld8(tmem + lane_addr + p.bt + c * 8, a1);
          tc_wait_ld();
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int m = m_base + c * 8 + e;
            if (n_ok && m < p.M) {
              const float v = finish(p, __uint_as_float(a0[e]), p.nw == 2 ? __uint_as_float(a1[e]) : 0.f, s0, s1, b0, m, n);
              p.y[static_cast<long long>(m) * p.ldy + n] = __float2bfloat16_rn(v);
            }
          }
        }
      } else {
        // fp32 partials: [tile][split][w][token][128 channels]
        const int tile_id = n_tile * gridDim.x + t_tile;
        const long long tile_stride = static_cast<long long>(p.nw) * p.bt * BN;
        float* mine = p.partials + (static_cast<long long>(tile_id) * p.splits + split) * tile_stride;
        for (int c = half; c < nchunks; c += 2) {
          for (int w = 0; w < p.nw; ++w) {
            uint32_t a0[8];
            tmem_ld8(tmem + lane_addr + w * p.bt + c * 8, a0);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < 8; ++e)
              mine[(static_cast<long long>(w) * p.bt + c * 8 + e) * BN + row] = __uint_as_float(a0[e]);
          }
        }
        __threadfence();
        bool met = __all_sync(0xffffffffu, epi_sync(&bars, 0, lane));
        if (met && cw == 0 && lane == 0) {
          const int old = atomicAdd(&p.counters[tile_id], 1);
          bars.is_last = (old == p.splits - 1) ? 1 : 0;
        }
        met = met && __all_sync(0xffffffffu, epi_sync(&bars, 1, lane));
        if (!met && lane == 0) fail(&bars, p.status, TYBOK_DEV_TIMEOUT_EPILOGUE);
        if (met && bars.is_last) {
          __threadfence();
          const float* base = p.partials + static_cast<long long>(tile_id) * p.splits * tile_stride;
          for (int c = half; c < nchunks; c += 2) {
#pragma unroll 2
            for (int e = 0; e < 8; ++e) {
              const int t = c * 8 + e;
              const int m = m_base + t;
              if (!(n_ok && m < p.M)) continue;
              float acc0 = 0.f, acc1 = 0.f;
              for (int sp = 0; sp < p.splits; ++sp) {  // fixed order: bit-reproducible
                const float* ps = base + sp * tile_stride;
                acc0 += __ldcg(ps + static_cast<long long>(t) * BN + row);
                if (p.nw == 2) acc1 += __ldcg(ps + (static_cast<long long>(p.bt) + t) * BN + row);
              }
              const float v = finish(p, acc0, acc1, s0, s1, b0, m, n);
              p.y[static_cast<long long>(m) * p.ldy + n] = __float2bfloat16_rn(v);
            }
          }
          if (cw == 0 && lane == 0) p.counters[tile_id] = 0;  // ready for the next launch
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------ host
struct Plan {
  int bt, t_tiles, n_tiles, splits, kb_total, kb_per_split, nstages, smem_bytes;
};

static int round_up(int a, int b) { return (a + b - 1) / b * b; }

static bool make_plan(int M, int N, int K, int nw, int force_bt, int force_splits, Plan& pl) {
  const int max_bt = nw == 2 ? 128 : 256;
  int bt;
  if (force_bt > 0) {
    bt = force_bt;
  } else {
    const int cap = nw == 2 ? 128 : 192;
    const int tiles = (M + cap - 1) / cap;
    bt = round_up((M + tiles - 1) / tiles, 16);
  }
  if (bt % 16 != 0 || bt < 16 || bt > max_bt) return false;
  pl.bt = bt;
  pl.t_tiles = (M + bt - 1) / bt;
  pl.n_tiles = (N + BN - 1) / BN;
  pl.kb_total = (K + BK - 1) / BK;
  int splits = force_splits;
  if (splits <= 0) {
    const int sms = host::sm_count();
    const int tiles = pl.t_tiles * pl.n_tiles;
    splits = 1;
    if (tiles * 2 <= sms) {
      splits = sms / tiles;
      splits = std::min(splits, std::max(1, pl.kb_total / 2));  // keep >= 2 K blocks per split
    }
  }
  splits = std::max(1, std::min(splits, pl.kb_total));
  pl.kb_per_split = (pl.kb_total + splits - 1) / splits;
  pl.splits = (pl.kb_total + pl.kb_per_split - 1) / pl.kb_per_split;  // no empty split
  const int stage_bytes = nw * W_TILE_BYTES + bt * 256;
  pl.nstages = std::min(MAX_STAGES, (DYN_SMEM_MAX - 1024) / stage_bytes);  // 1 KB of alignment slack
  pl.nstages = std::min(pl.nstages, std::max(2, pl.kb_per_split));
  if (pl.nstages < 2) return false;
  pl.smem_bytes = pl.nstages * stage_bytes + 1024;
  return true;
}

static size_t workspace_bytes_for(int M, int N, int K, int nw) {
  // Upper bound over every plan the heuristic can choose: partials are written only when
  // splits > 1, which happens only when tiles * 2 <= SM count.
  Plan pl;
  if (!make_plan(M, N, K, nw, 0, 0, pl)) return TYBOK_COUNTER_BYTES;
  const size_t per_tile = static_cast<size_t>(nw) * pl.bt * BN * sizeof(float);
  const size_t tiles = static_cast<size_t>(pl.t_tiles) * pl.n_tiles;
  // Allow forced split factors up to 32 in tests and tuning runs.
  const size_t splits = std::max(pl.splits, 32);
  return TYBOK_COUNTER_BYTES + tiles * splits * per_tile;
}

static int launch_gemm(const void* x, const void* w0, const void* w1, const float* s0, const float* s1,
                       const void* bias, void* y, int M, int N, int K, long long ldx, long long ldy, int epi,
                       const void* res, long long ldres, const void* gate, long long ldgate, int rows_per_gate,
                       int gate_bf16, int force_bt, int force_splits, void* ws, size_t ws_bytes, int* status,
                       cudaStream_t stream) {
  const int nw = w1 ? 2 : 1;
  if (!x || !w0 || !s0 || !y) return host::fail(TYBOK_ERR_ARG, "w8a16: null pointer argument");
  if (M <= 0 || N <= 0 || K <= 0) return host::fail(TYBOK_ERR_ARG, "w8a16: M, N, K must be positive");
  if (K % 16 != 0) return host::fail(TYBOK_ERR_ARG, "w8a16: K must be a multiple of 16 (TMA row pitch)");
  if (ldx % 8 != 0 || ldx < K) return host::fail(TYBOK_ERR_ARG, "w8a16: ldx must be >= K and a multiple of 8");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w0) | reinterpret_cast<uintptr_t>(w1)) & 15)
    return host::fail(TYBOK_ERR_ARG, "w8a16: x and w8 must be 16-byte aligned");
  if (epi == EPI_RESIDUAL && !res) return host::fail(TYBOK_ERR_ARG, "w8a16: residual epilogue without residual");
  if (gate && rows_per_gate <= 0) return host::fail(TYBOK_ERR_ARG, "w8a16: rows_per_gate must be positive");
  if (int rc = host::require_sm100()) return rc;

  Plan pl;
  if (!make_plan(M, N, K, nw, force_bt, force_splits, pl))
    return host::fail(TYBOK_ERR_ARG, "w8a16: unsupported token tile (multiple of 16, <= 256, <= 128 when gated)");
  if (pl.n_tiles > 65535 || pl.splits > 65535) return host::fail(TYBOK_ERR_ARG, "w8a16: grid too large");
  const size_t tiles = static_cast<size_t>(pl.t_tiles) * pl.n_tiles;
  if (pl.splits > 1) {
    const size_t need = TYBOK_COUNTER_BYTES + tiles * pl.splits * nw * pl.bt * BN * sizeof(float);
    if (!ws || ws_bytes < need) return host::fail(TYBOK_ERR_WORKSPACE, "w8a16: split-K needs a larger workspace");
    if (tiles * sizeof(int) > TYBOK_COUNTER_BYTES) return host::fail(TYBOK_ERR_WORKSPACE, "w8a16: too many tiles for the counter block");
  }

  CUtensorMap tm_w0, tm_w1, tm_x;
  if (int rc = host::tensor_map_2d(&tm_w0, w0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, N, K, BK, BN)) return rc;
  tm_w1 = tm_w0;
  if (nw == 2)
    if (int rc = host::tensor_map_2d(&tm_w1, w1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, N, K, BK, BN)) return rc;
  if (int rc = host::tensor_map_2d(&tm_x, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, ldx * 2, 64, pl.bt)) return rc;

  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.bt = pl.bt; p.nw = nw; p.splits = pl.splits; p.kb_total = pl.kb_total; p.kb_per_split = pl.kb_per_split;
  p.nstages = pl.nstages; p.epi = epi; p.pdl = host::pdl_enabled() ? 1 : 0;
  p.scale0 = s0; p.scale1 = s1; p.bias0 = static_cast<const __nv_bfloat16*>(bias);
  p.y = static_cast<__nv_bfloat16*>(y); p.ldy = ldy;
  p.res = static_cast<const __nv_bfloat16*>(res); p.ldres = ldres;
  p.gate = gate; p.ldgate = ldgate; p.rows_per_gate = rows_per_gate > 0 ? rows_per_gate : 1; p.gate_bf16 = gate_bf16;
  p.counters = static_cast<int*>(ws);
  p.partials = ws ? reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + TYBOK_COUNTER_BYTES) : nullptr;
  p.status = status;

  static bool attr_set[64] = {};
  const int dev = host::current_device();
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(w8a16_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DYN_SMEM_MAX) != cudaSuccess)
      return host::fail_cuda("cudaFuncSetAttribute(w8a16_gemm_kernel)");
    attr_set[dev] = true;
  }

  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(pl.t_tiles, pl.n_tiles, pl.splits);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = pl.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 1 : 0;
  if (cudaLaunchKernelEx(&cfg, w8a16_gemm_kernel, tm_w0, tm_w1, tm_x, p) != cudaSuccess)
    return host::fail_cuda("launch w8a16_gemm_kernel");
  host::count_launch();
  return TYBOK_OK;
}

}  // namespace tb

extern "C" {

size_t tybok_w8a16_workspace_bytes(int M, int N, int K, int dual) {
  return tb::workspace_bytes_for(M, N, K, dual ? 2 : 1);
}

int tybok_w8a16_linear(const void* x, const void* w8, const float* scale, const void* bias, void* y, int M, int N,
                       int K, int64_t ldx, int64_t ldy, int epilogue, const void* residual, int64_t ldres,
                       const void* gate, int64_t ldgate, int rows_per_gate, int gate_is_bf16, int token_tile,
                       int splits, void* workspace, size_t workspace_bytes, int* status_word, void* stream) {
  if (epilogue != TYBOK_EPI_NONE && epilogue != TYBOK_EPI_GELU && epilogue != TYBOK_EPI_RESIDUAL)
    return tb::host::fail(TYBOK_ERR_ARG, "w8a16_linear: unknown epilogue");
  return tb::launch_gemm(x, w8, nullptr, scale, nullptr, bias, y, M, N, K, ldx, ldy, epilogue, residual, ldres, gate,
                         ldgate, rows_per_gate, gate_is_bf16, token_tile, splits, workspace, workspace_bytes,
                         status_word, static_cast<cudaStream_t>(stream));
}

int tybok_w8a16_geglu(const void* x, const void* w8_gate, const float* scale_gate, const void* w8_up,
                      const float* scale_up, void* h, int M, int I, int K, int64_t ldx, int64_t ldh, int token_tile,
                      int splits, void* workspace, size_t workspace_bytes, int* status_word, void* stream) {
  if (!w8_up || !scale_up) return tb::host::fail(TYBOK_ERR_ARG, "w8a16_geglu: null up-projection");
  return tb::launch_gemm(x, w8_gate, w8_up, scale_gate, scale_up, nullptr, h, M, I, K, ldx, ldh, tb::EPI_GEGLU, nullptr,
                         0, nullptr, 0, 1, 0, token_tile, splits, workspace, workspace_bytes, status_word,
                         static_cast<cudaStream_t>(stream));
}

}  // extern "C"
