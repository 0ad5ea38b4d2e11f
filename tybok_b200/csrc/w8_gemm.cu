// W8A16 linear for sm_100a: e4m3 weights with per-output-channel fp32 scales, bf16
// activations, fp32 accumulation in tensor memory -- with no per-weight ALU work.
//
// The activations arrive as three e5m2 planes whose sum is the bf16 value exactly
// (split3.cuh).  The weight tile goes TMA -> shared memory -> tcgen05.mma (kind::f8f6f4,
// A = e4m3, B = e5m2) untouched; each 32-wide K slice is multiplied by the three planes into
// the same fp32 accumulator.  Products of an e4m3 and an e5m2 number are exact in fp32, so
// the result is the bf16-activation x e4m3-weight dot product up to fp32 summation order.
//
// Orientation: the weight tile is the 128-row M side of the UMMA and the tokens are its N
// side, D[n, m] = sum_k W[n,k] x[m,k], so any token count from 1 to 256 fills all 128
// tensor-memory lanes.
//
// Per CTA (one 128 x token_tile output tile, one K range when split-K is on):
//   warp 0     TMA producer: weight tile(s) (128 rows x 128 bytes, 128B swizzle) and the three
//              activation planes of the same K range into an n-stage shared-memory ring.
//              Weights are requested before the programmatic-dependency wait, activations after.
//   warp 1     one elected lane issues the MMAs (12 per weight tile and K block) and one
//              tcgen05.commit per K block.
//   warps 2-9  epilogue: accumulator -> fp32 staging tile in shared memory; then, 4 channels
//              per thread: split-K sum, scale/bias, activation, gate/residual and 8-byte stores
//              (bf16, and/or the three e5m2 planes the next GEMM consumes).
// Split-K runs as a thread-block cluster along z: every CTA stages its partial tile in its
// own shared memory, the cluster meets at a hardware barrier, and CTA r sums token rows
// r*R..(r+1)*R-1 over all ranks in rank order through distributed shared memory.  No global
// scratch, no atomics, bit-reproducible.
//
// Algorithmic HBM bytes per launch: N*K (weights) + 4*N (scales) + 2*M*K (x) + 2*M*N (y).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "../../include/tybok_b200.h"
#include "host_util.h"
#include "ptx.cuh"
#include "split3.cuh"

namespace tb {

constexpr int BN = 128;  // weight rows per tile = UMMA M
constexpr int BK = 128;  // K per pipeline stage (one 128-byte swizzle row of 8-bit elements)
constexpr int W_TILE_BYTES = BN * BK;
constexpr int MAX_STAGES = 8;
constexpr int EPI_WARPS = 8;       // epilogue warps of the full-K forms (two CTAs share an SM)
constexpr int EPI_WARPS_WIDE = 16; // ... of the split-K form: four warps per tensor-memory lane quadrant
constexpr int THREADS = 32 * (2 + EPI_WARPS);
constexpr int THREADS_WIDE = 32 * (2 + EPI_WARPS_WIDE);
constexpr int DYN_SMEM_MAX = 226 * 1024;  // 227 KB per CTA minus 1 KB left for static shared memory
constexpr int CORESIDENT_SMEM = 112 * 1024;  // dynamic shared memory of a CTA when two share an SM (228 KB)
constexpr int MAX_SPLITS = 8;             // portable cluster size

// EPI_GEGLU_PACKED: one weight matrix whose 128-row tiles hold 64 gate rows followed by the 64
// up rows of the same channels; the tile yields 64 output channels gelu(gate) * up.
// EPI_QKV_ROPE: packed q/k/v projection whose 128-row tiles hold 64 head dimensions followed by
// their rotate-half partners (d, d + D/2); the tile is rotated and stored as q rows / cache rows.
enum : int { EPI_NONE = 0, EPI_GELU = 1, EPI_RESIDUAL = 2, EPI_GEGLU = 3, EPI_GEGLU_PACKED = 4, EPI_QKV_ROPE = 5 };

struct RopeEpi {
  const int* pos;              // [M] position of every token row
  const __nv_bfloat16* cos;    // [max_pos][D]
  const __nv_bfloat16* sin;
  __nv_bfloat16* q;            // [M][H*D]
  __nv_bfloat16* kcache;       // [B][G][Lcap][D]
  __nv_bfloat16* vcache;
  int L, H, G, D, Lcap, key_off;
};

struct GemmParams {
  int M, N, K;
  int n_out;     // width of the output rows: N, or N / 2 for EPI_GEGLU_PACKED
  int bt;        // token tile (UMMA N), multiple of 16, <= 256 (<= 128 when nw == 2)
  int nw;        // weight matrices per CTA: 1, or 2 for the gated form
  int splits;    // split-K factor == cluster size along z
  int kb_total;  // ceil(K / BK)
  int kb_per_split;
  int nstages;
  int tmem_cols;
  int stage_off;  // byte offset of the epilogue staging tile: 0 (over the idle ring) without split-K,
                  // behind the ring with split-K, because peers write into it while this CTA still streams
  int np;        // activation planes: 3 (e5m2, fixed exponent shift) or 2 (e4m3, per-token scale row_scale[m])
  const float* row_scale;  // [M] 2^-k of every token row (two-plane form), else NULL
  // AdaRMS norm folded into its neighbours (action expert below the two-plane threshold).  The GEMM
  // that writes the residual stream also writes planes of bf16(x * (1 + scale_next)) and, per channel
  // tile, the row sums of squares of x; the GEMM that follows multiplies its accumulator rows by
  // rsqrt(mean(x^2) + eps) and adds W * shift as an fp32 bias: y = W (x r (1 + scale) + shift).
  const float* nn_scale;  // producer: [N] fp32 scale row of the next norm, or NULL
  float* nn_part;         // producer: [N / 128][M] partial sums of squares of the bf16 output rows
  const float* dn_part;   // consumer: [dn_tiles][M] partial sums written by the producer, or NULL
  int dn_tiles;
  float dn_inv_w, dn_eps;
  const float* bias_f32;  // consumer: [N] fp32 bias in weight-row order, or NULL
  int merge;     // 1: the planes are one UMMA of N = np*bt whose column groups the epilogue adds
  int pair;      // 1: CTA pairs (cluster of 2 along the channel tiles) run one UMMA of M = 256; each CTA
                 // loads its own weight tile and half of the activation planes (tm_w1 = half-tile map)
  int epi;
  int pdl;
  float out_scale;   // 2^-x_shift: undoes the power-of-two pre-scale of the activation planes
  float plane_scale; // 2^out_shift applied to the values written as output planes
  const float* scale0;
  const float* scale1;
  const __nv_bfloat16* bias0;
  __nv_bfloat16* y;  // bf16 output or NULL
  long long ldy;
  uint8_t* y_planes;  // [3][M][N] e5m2 output planes or NULL
  const __nv_bfloat16* res;
  long long ldres;
  const void* gate;
  long long ldgate;
  int rows_per_gate;
  int gate_bf16;
  int* status;
  long long* trace;  // tuning aid: [CTA][16] SM-clock samples, NULL in production
  int* dbg;          // debugging aid: stage counters, NULL in production
  long long epi_wait_limit;  // SM clocks the epilogue waits for the accumulator (kWaitLimitCycles in production)
  RopeEpi rope;      // EPI_QKV_ROPE only
};

struct __align__(8) Barriers {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t tmem_full;
  uint64_t mma_done;  // every tensor-core instruction this CTA (or its pair) issued has retired
  uint32_t tmem_base;
  volatile int abort;
};

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                              long long limit = kWaitLimitCycles) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > limit) return false;
  }
  return true;
}

__device__ __forceinline__ void fail(Barriers* b, int* status, int code) {
  b->abort = 1;
  if (status) atomicCAS(status, 0, code);
}

// Bounded for two CTAs per SM: multi-wave full-K launches run with a shallow ring so that one
// tile's epilogue overlaps the other's main loop (register budget 64K / 640 threads).
// PAIR: the CTA-pair form (cta_group::2 instructions oblige every launch of a kernel that holds
// them to use clusters of two, so it is an instantiation of its own).
// EW: epilogue warps.  A split-K CTA has the SM to itself and a long serial epilogue per thread
// (accumulator groups to push, rows to finish): sixteen warps halve both.
// rsqrt(mean(x^2) + eps) of token row m from the producer's per-channel-tile partial sums (fixed order).
// The partial sums were written by other SMs a moment ago (an L2 round trip each), so eight loads are
// in flight at a time.
__device__ __forceinline__ float deferred_rstd(const GemmParams& p, int m) {
  float t = 0.f;
  for (int i0 = 0; i0 < p.dn_tiles; i0 += 8) {
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      v[i] = i0 + i < p.dn_tiles ? __ldcg(p.dn_part + static_cast<long long>(i0 + i) * p.M + m) : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += v[i];
  }
  return rsqrtf(t * p.dn_inv_w + p.dn_eps);
}

template <bool PAIR, int EW = EPI_WARPS>
__global__ void __launch_bounds__(32 * (2 + EW), EW == EPI_WARPS ? 2 : 1)
w8_gemm_kernel(const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w1,
               const __grid_constant__ CUtensorMap tm_x, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ Barriers bars;

  const long long t_start = clock64();
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int KID = PAIR ? 2 : (EW == EPI_WARPS ? 0 : 1);
  if (tid == 0) dbg_stage(p.dbg, KID, 0);

  const int ns = p.nstages;
  const int x_bytes = PAIR ? p.np * p.bt * 64 : p.np * p.bt * 128;  // np planes of bt rows x 128 bytes (a pair: half each)
  const int x_off = p.nw * W_TILE_BYTES;              // activation planes follow the weight tile(s)
  const int stage_bytes = x_off + x_bytes;

  // A pair is two neighbouring channel tiles; pairs lie along x of the grid (and of the cluster).
  const int t_tile = PAIR ? blockIdx.y : blockIdx.x, n_tile = PAIR ? blockIdx.x : blockIdx.y, split = blockIdx.z;
  const uint32_t pair_rank = PAIR ? cluster_ctarank() : 0u;  // 0 issues the pair's UMMAs
  const int kb0 = split * p.kb_per_split;
  const int nkb = min(p.kb_total, kb0 + p.kb_per_split) - kb0;

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_w0);
    if (p.nw == 2 || PAIR) tma_prefetch_desc(&tm_w1);
    if (!PAIR) tma_prefetch_desc(&tm_x);
    for (int i = 0; i < MAX_STAGES; ++i) {
      mbar_init(&bars.full[i], 1);
      mbar_init(&bars.empty[i], 1);
    }
    mbar_init(&bars.tmem_full, 1);
    mbar_init(&bars.mma_done, 1);
    bars.abort = 0;
    fence_barrier_init();
    // Weights depend on nothing that runs before this kernel: request the first stages now,
    // before the rest of the CTA has even finished its set-up.  (A pair first has to know that
    // the partner's barriers exist: it requests them after the cluster has met.)
    if (!PAIR) {
      const int pre = min(ns, nkb);
      for (int i = 0; i < pre; ++i) {
        uint8_t* st = smem + i * stage_bytes;
        mbar_arrive_expect_tx(&bars.full[i], stage_bytes);
        const int k0 = (kb0 + i) * BK;
        tma_load_2d(st, &tm_w0, &bars.full[i], k0, n_tile * BN);
        if (p.nw == 2) tma_load_2d(st + W_TILE_BYTES, &tm_w1, &bars.full[i], k0, n_tile * BN);
      }
    }
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(&bars.tmem_base, p.tmem_cols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&bars.tmem_base, p.tmem_cols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if (PAIR) {
    __syncwarp();
    cluster_sync_all();
  } else {
    __syncthreads();
  }
  tc_fence_after();
  if (tid == 0) dbg_stage(p.dbg, KID, 1);
  const uint32_t tmem = bars.tmem_base;
  // Per-thread epilogue constants (4 consecutive channels), fetched while the main loop runs.
  float s0[4] = {0, 0, 0, 0}, s1[4] = {0, 0, 0, 0}, b0[4] = {0, 0, 0, 0};
  float b1[4] = {0, 0, 0, 0};   // bias of the second half tile (packed forms, fp32 bias only)
  float nsc[4] = {0, 0, 0, 0};  // 1 + scale of the next norm for this thread's channels (producer form)
  float rs_pf = 1.0f;           // deferred norm: rstd of this thread's first token row
  uint2 res_pf[4] = {};  // residual of this thread's first four token rows, fetched early
  float4 gate_pf = make_float4(0.f, 0.f, 0.f, 0.f);  // gate values of the first token row's group (fp32 form)
  int gate_pf_group = -1;
  // Split-K ownership: the tile's real token rows are divided evenly over the cluster ranks.
  const int m_base = t_tile * p.bt;
  const int nvalid = min(p.bt, p.M - m_base);
  const int rpr = (nvalid + p.splits - 1) / p.splits;
  const int rank = p.splits > 1 ? static_cast<int>(cluster_ctarank()) : 0;
  const int own_rows = max(0, min(nvalid, rank * rpr + rpr) - rank * rpr);
  long long* tr = p.trace ? p.trace + 16ll * ((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) : nullptr;
  if (tr && tid == 0) { tr[0] = t_start; tr[1] = clock64(); }

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int issued = 0;
      bool ok = true;
      // Dependents may start their own preamble (their weight prefetch) as soon as every CTA of
      // this grid is running; they still wait for this grid to complete before touching its output.
      if (p.pdl) pdl_launch_dependents();
      const int pre = min(ns, nkb);
      if (PAIR) {
        // CTA pair: both CTAs load their own weight tile and their half of the activation planes
        // (three boxes of bt/2 token rows of one plane); every byte is credited to the full
        // barrier of the even-ranked CTA, which issues the UMMAs for both.
        const int hrows = p.bt >> 1;
        auto pair_stage = [&](int i, bool weights, bool acts) {
          uint8_t* st = smem + (i % ns) * stage_bytes;
          const uint32_t bar = dsmem_addr(smem_u32(&bars.full[i % ns]), 0);
          const int k0 = (kb0 + i) * BK;
          if (weights) {
            if (pair_rank == 0) mbar_arrive_expect_tx(&bars.full[i % ns], 2 * stage_bytes);
            tma_load_2d_pair(st, &tm_w0, bar, k0, n_tile * BN);
          }
          if (acts) {
            for (int j = 0; j < p.np; ++j) {
              const int u = static_cast<int>(pair_rank) * p.np + j;  // half-plane index 0 .. 2 np - 1
              tma_load_3d_pair(st + x_off + j * hrows * 128, &tm_w1, bar, k0, t_tile * p.bt + (u & 1) * hrows, u >> 1);
            }
          }
        };
        for (int i = 0; i < pre; ++i) pair_stage(i, true, false);
        if (p.pdl) pdl_wait();
        dbg_stage(p.dbg, KID, 2);
        for (int i = 0; i < pre; ++i) pair_stage(i, false, true);
        int armed = pre;
        for (int i = pre; i < nkb; ++i) {
          if (!wait_or_abort(&bars.empty[i % ns], ((i / ns) & 1) ^ 1, &bars.abort)) {
            fail(&bars, p.status, TYBOK_DEV_TIMEOUT_PRODUCER);
            break;
          }
          pair_stage(i, true, true);
          armed = i + 1;
        }
        // Unwinding (completion is observed through the issuing CTA's barriers only): the even CTA
        // waits for the newest copy of every stage it armed; the pair leaves together at the
        // closing cluster barrier.
        if (bars.abort && pair_rank == 0)
          for (int i = max(0, armed - ns); i < armed; ++i) mbar_wait(&bars.full[i % ns], (i / ns) & 1);
        issued = 0;
        ok = true;
      } else {
      // The weight tiles of the first stages were requested during set-up; the activation planes
      // are requested once the programmatic dependency has resolved.
      if (p.pdl) pdl_wait();
      dbg_stage(p.dbg, KID, 2);
      for (int i = 0; i < pre; ++i)
        tma_load_3d(smem + i * stage_bytes + x_off, &tm_x, &bars.full[i], (kb0 + i) * BK, t_tile * p.bt, 0);
      issued = pre;
      for (int i = pre; i < nkb; ++i) {
        const int s = i % ns;
        if (!wait_or_abort(&bars.empty[s], ((i / ns) & 1) ^ 1, &bars.abort)) {
          fail(&bars, p.status, TYBOK_DEV_TIMEOUT_PRODUCER);
          ok = false;
          break;
        }
        uint8_t* st = smem + s * stage_bytes;
        mbar_arrive_expect_tx(&bars.full[s], stage_bytes);
        const int k0 = (kb0 + i) * BK;
        tma_load_2d(st, &tm_w0, &bars.full[s], k0, n_tile * BN);
        if (p.nw == 2) tma_load_2d(st + W_TILE_BYTES, &tm_w1, &bars.full[s], k0, n_tile * BN);
        tma_load_3d(st + x_off, &tm_x, &bars.full[s], k0, t_tile * p.bt, 0);
        issued = i + 1;
      }
      }
      if (!PAIR && (!ok || bars.abort)) {
        // Unwinding: do not leave the CTA while its own bulk copies may still land in its
        // shared memory. Wait (bounded) for the newest copy of every stage.
        for (int i = max(0, issued - ns); i < issued; ++i) mbar_wait(&bars.full[i % ns], (i / ns) & 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp runs the loop, so every operand is warp-uniform; one elected lane issues.
    const bool leader = elect_one();
    // Small token tiles: the three planes are contiguous rows in shared memory, so one UMMA
    // with N = 3*bt multiplies a K slice by all of them (one column group per plane) -- 4
    // instead of 12 instructions per weight tile and K block.  Larger tiles issue one UMMA per
    // plane into the same accumulator.
    const int mma_n = p.merge ? p.np * p.bt : p.bt;
    const uint32_t idesc = p.np == 2 ? idesc_e4m3_e4m3_f32(PAIR ? 2 * BN : BN, mma_n) : idesc_e4m3_e5m2_f32(PAIR ? 2 * BN : BN, mma_n);
    const int nkb_mma = (PAIR && pair_rank != 0) ? 0 : nkb;  // the odd CTA of a pair issues nothing
    const uint64_t desc_const = smem_desc_sw128(0);
    const uint32_t plane16 = static_cast<uint32_t>(p.bt * 128) >> 4;  // plane pitch in 16-byte units
    const int acc_cols = p.merge ? p.np * p.bt : p.bt;
    bool ok = true;
    for (int i = 0; i < nkb_mma; ++i) {
      const int s = i % ns;
      const long long c0 = tr ? clock64() : 0;
      const bool ready = wait_or_abort(&bars.full[s], (i / ns) & 1, &bars.abort);
      if (tr && leader) { const long long c1 = clock64(); tr[8] += c1 - c0; if (i == 0) tr[2] = c1; }
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) fail(&bars, p.status, TYBOK_DEV_TIMEOUT_MMA);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t st16 = (smem_u32(smem + s * stage_bytes) & 0x3FFFFu) >> 4;
      const uint32_t x16 = st16 + (x_off >> 4);
      for (int w = 0; w < p.nw; ++w) {
        const uint32_t w16 = st16 + w * (W_TILE_BYTES >> 4);
        const uint32_t d_addr = tmem + w * acc_cols;
        if (p.merge) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // K = 32 per instruction: 32 bytes = 2 sixteen-byte units
            const uint64_t a_desc = desc_const | (w16 + j * 2);
            const uint64_t b_desc = desc_const | (x16 + j * 2);
            if (leader) {
              if (PAIR) umma_ss_f8_pair(d_addr, a_desc, b_desc, idesc, (i > 0 || j > 0) ? 1u : 0u);
              else umma_ss_f8(d_addr, a_desc, b_desc, idesc, (i > 0 || j > 0) ? 1u : 0u);
            }
          }
        } else {
          for (int pl = 0; pl < p.np; ++pl) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint64_t a_desc = desc_const | (w16 + j * 2);
              const uint64_t b_desc = desc_const | (x16 + pl * plane16 + j * 2);
              if (leader) umma_ss_f8(d_addr, a_desc, b_desc, idesc, (i > 0 || pl > 0 || j > 0) ? 1u : 0u);
            }
          }
        }
      }
      if (leader) {  // frees the stage (in both CTAs of a pair) once these MMAs have read it
        if (PAIR) tc_commit_pair(&bars.empty[s], 3);
        else tc_commit(&bars.empty[s]);
      }
      __syncwarp();
    }
    if (ok && leader && nkb_mma > 0) {
      if (PAIR) tc_commit_pair(&bars.tmem_full, 3);
      else tc_commit(&bars.tmem_full);
    }
    if (tr && leader) tr[3] = clock64();
    // Whatever happened above, and whatever the other warps decide: this warp frees the tensor
    // memory at the end, so it first sees every instruction it issued retire (in a pair the even
    // CTA's commit arrives in both CTAs).  On the normal path this completes together with
    // tmem_full; the warp has nothing else to do until the CTA meets.
    if (leader && (!PAIR || pair_rank == 0)) {
      if (PAIR) tc_commit_pair(&bars.mma_done, 3);
      else tc_commit(&bars.mma_done);
    }
    __syncwarp();
    if (!mbar_wait(&bars.mma_done, 0) && lane == 0) fail(&bars, p.status, TYBOK_DEV_TIMEOUT_MMA);
  } else {
    // ------------------------------------------------------------ epilogue, phase A
    // Accumulator (lane = channel, column = token) -> fp32 staging tile [w][token][128 channels]
    // at the start of the (by now idle) stage ring.
    const int ew = warp - 2;
    const int q = warp & 3;   // TMEM lane quadrant this warp may access
    const int half = ew >> 2;  // which of the EW / 4 warps of this lane quadrant
    const int row = q * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    {
      const bool packed = p.epi == EPI_GEGLU_PACKED || p.epi == EPI_QKV_ROPE;  // paired half tiles
      const int v4p = (tid - 64) & 31;
      const int col0 = packed ? (v4p & 15) * 4 : v4p * 4;
      const int n = p.epi == EPI_GEGLU_PACKED ? n_tile * (BN / 2) + col0 : n_tile * BN + col0;  // first output channel
      if (n < p.n_out) {  // weights-side data: independent of the previous kernel in the stream
        const float4 t = *reinterpret_cast<const float4*>(p.scale0 + n_tile * BN + col0);
        s0[0] = t.x * p.out_scale; s0[1] = t.y * p.out_scale; s0[2] = t.z * p.out_scale; s0[3] = t.w * p.out_scale;
        if (p.nw == 2 || packed) {
          const float4 u = packed ? *reinterpret_cast<const float4*>(p.scale0 + n_tile * BN + BN / 2 + col0)
                                  : *reinterpret_cast<const float4*>(p.scale1 + n);
          s1[0] = u.x * p.out_scale; s1[1] = u.y * p.out_scale; s1[2] = u.z * p.out_scale; s1[3] = u.w * p.out_scale;
        }
        if (p.bias0) {
#pragma unroll
          for (int e = 0; e < 4; ++e) b0[e] = __bfloat162float(p.bias0[n + e]);
        }
        if (p.bias_f32) {  // weight-row order: the second half tile of a packed form has its own rows
          const float4 t0 = *reinterpret_cast<const float4*>(p.bias_f32 + n_tile * BN + col0);
          b0[0] = t0.x; b0[1] = t0.y; b0[2] = t0.z; b0[3] = t0.w;
          if (packed) {
            const float4 t1 = *reinterpret_cast<const float4*>(p.bias_f32 + n_tile * BN + BN / 2 + col0);
            b1[0] = t1.x; b1[1] = t1.y; b1[2] = t1.z; b1[3] = t1.w;
          }
        }
        if (p.nn_scale) {
          const float4 t0 = *reinterpret_cast<const float4*>(p.nn_scale + n);
          nsc[0] = 1.0f + t0.x; nsc[1] = 1.0f + t0.y; nsc[2] = 1.0f + t0.z; nsc[3] = 1.0f + t0.w;
        }
        if (p.epi == EPI_RESIDUAL && p.gate && !p.gate_bf16) {
          // fp32 gates are per-step constants (precomputed modulations), touched once per chunk
          // and therefore cold in L2: fetch them now, not between the accumulator and the stores.
          gate_pf_group = (m_base + rank * rpr) / p.rows_per_gate;
          gate_pf = *reinterpret_cast<const float4*>(static_cast<const float*>(p.gate) +
                                                     static_cast<long long>(gate_pf_group) * p.ldgate + n);
        }
        if (p.epi == EPI_QKV_ROPE) {
          // Positions and tables are constants: fetch the cos/sin of this thread's first row now.
          const RopeEpi& r = p.rope;
          const int tps = r.D >> 7;
          const int rl = ((tid - 64) >> 5) * 2 + (v4p >> 4);
          if (rl < own_rows && n_tile / tps < r.H + r.G) {
            const long long tb = static_cast<long long>(r.pos[m_base + rank * rpr + rl]) * r.D + (n_tile % tps) * 64 + col0;
            res_pf[0] = *reinterpret_cast<const uint2*>(r.cos + tb);
            res_pf[1] = *reinterpret_cast<const uint2*>(r.cos + tb + (r.D >> 1));
            res_pf[2] = *reinterpret_cast<const uint2*>(r.sin + tb);
            res_pf[3] = *reinterpret_cast<const uint2*>(r.sin + tb + (r.D >> 1));
          }
        }
      }
      // These warps are idle until the accumulator is complete, so they wait for the previous
      // kernel now, under the main loop, not between the accumulator and the stores.
      if (p.pdl) pdl_wait();
      if (n < p.n_out) {
        if (p.dn_part) {  // written by the previous GEMM: this thread's first row, under the main loop
          const int rl = packed ? ((tid - 64) >> 5) * 2 + (v4p >> 4) : (tid - 64) >> 5;
          if (rl < own_rows) rs_pf = deferred_rstd(p, m_base + rank * rpr + rl);
        }
        if (p.epi == EPI_RESIDUAL) {
          // The residual was written by an earlier kernel: fetch the rows this thread will finish
          // first, long before the accumulator is ready.
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int rl = ((tid - 64) >> 5) + EW * u;
            if (rl < own_rows)
              res_pf[u] = *reinterpret_cast<const uint2*>(
                  p.res + static_cast<long long>(m_base + rank * rpr + rl) * p.ldres + n);
          }
        }
      }
    }
    bool ok = __all_sync(0xffffffffu, wait_or_abort(&bars.tmem_full, 0, &bars.abort, p.epi_wait_limit));
    if (!ok && lane == 0) fail(&bars, p.status, TYBOK_DEV_TIMEOUT_EPILOGUE);
    if (tr && ew == 0 && lane == 0) tr[4] = clock64();
    if (ok) {
      tc_fence_after();
      // Every token row is written straight into the staging tile of the CTA that owns it
      // (slot [split][w][row within owner][128 channels], through distributed shared memory when
      // the owner is another rank), so that after the meeting point each owner only reads its
      // own shared memory.
      const uint32_t stage_addr = smem_u32(smem + p.stage_off);
      const int ngroups = (nvalid + 15) / 16;
      const int acc_cols = p.merge ? p.np * p.bt : p.bt;
      for (int w = 0; w < p.nw; ++w) {
        for (int g = half; g < ngroups; g += EW / 4) {
          uint32_t v[16];
          const uint32_t col = tmem + lane_addr + w * acc_cols + g * 16;
          tmem_ld16(col, v);
          if (p.merge && p.np == 2) {  // add the per-plane column groups in plane order
            uint32_t v2[16];
            tmem_ld16(col + p.bt, v2);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) + __uint_as_float(v2[e]));
          } else if (p.merge) {
            uint32_t v2[16], v3[16];
            tmem_ld16(col + p.bt, v2);
            tmem_ld16(col + 2 * p.bt, v3);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e)
              v[e] = __float_as_uint((__uint_as_float(v[e]) + __uint_as_float(v2[e])) + __uint_as_float(v3[e]));
          } else {
            tc_wait_ld();
          }
          if (p.splits == 1) {
            // Own tile, row = token: up to 16 stores at fixed 512-byte steps.
            float* dst = reinterpret_cast<float*>(smem + p.stage_off) + (w * rpr + g * 16) * BN + row;
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (g * 16 + e < nvalid) dst[e * BN] = __uint_as_float(v[e]);
          } else {
            // Up to three owners per group of 16 tokens; an owner's window is linear, so one
            // address translation per owner and 512-byte steps inside it.
            const int t0 = g * 16;
            int owner = t0 / rpr, rl = t0 - owner * rpr;
            const uint32_t slot = stage_addr + (((split * p.nw + w) * rpr) * BN + row) * 4;
            uint32_t base = dsmem_addr(slot, owner);
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              if (t0 + e < nvalid)
                asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(base + rl * (BN * 4)), "f"(__uint_as_float(v[e])));
              if (++rl == rpr) {
                rl = 0;
                ++owner;
                if (owner < p.splits) base = dsmem_addr(slot, owner);
              }
            }
          }
        }
      }
    }
  }

  // ------------------------------------------------------------ meet: staging tiles complete
  if (tr && tid == 64) tr[5] = clock64();
  tc_fence_before();
  if (p.splits > 1) {
    __syncwarp();
    cluster_sync_all();
  } else {
    __syncthreads();
  }

  if (tr && tid == 64) tr[6] = clock64();
  if (tid == 0) dbg_stage(p.dbg, KID, 3);
  if (warp >= 2 && !bars.abort) {
    // ---------------------------------------------------------- epilogue, phase B
    // 4 consecutive channels per thread, 8 token rows per pass; with split-K, rank r owns token
    // rows [r*R, (r+1)*R) and sums them over all ranks in rank order.
    if (tr && tid == 64) tr[9] = clock64();
    const int et = tid - 64;
    const int v4 = et & 31;
    const int rgrp = et >> 5;
    // Packed gated form: 16 lanes cover the 64 output channels of a row, so a warp takes two
    // rows per pass; otherwise 32 lanes cover the 128 channels of one row.
    const bool packed = p.epi == EPI_GEGLU_PACKED || p.epi == EPI_QKV_ROPE;
    const int col0 = packed ? (v4 & 15) * 4 : v4 * 4;
    const int n = p.epi == EPI_GEGLU_PACKED ? n_tile * (BN / 2) + col0 : n_tile * BN + col0;
    const bool n_ok = n < p.n_out;  // n_out % 4 == 0, so all four channels are valid together
    const int row0 = packed ? rgrp * 2 + (v4 >> 4) : rgrp;
    const int rstep = packed ? 2 * EW : EW;
    const float* stage = reinterpret_cast<const float*>(smem + p.stage_off);
    const long long plane = static_cast<long long>(p.M) * p.n_out;
    if (tr && tid == 64) tr[10] = clock64();
#pragma unroll 1
    for (int rl = row0; rl < own_rows && n_ok; rl += rstep) {
      const int m = m_base + rank * rpr + rl;
      float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
      for (int sp = 0; sp < p.splits; ++sp) {  // split order: bit-reproducible
        const float* r0p = stage + ((sp * p.nw) * rpr + rl) * BN;
        const float4 f = *reinterpret_cast<const float4*>(r0p + col0);
        a0.x += f.x; a0.y += f.y; a0.z += f.z; a0.w += f.w;
        if (p.nw == 2 || packed) {
          const float4 g = packed ? *reinterpret_cast<const float4*>(r0p + BN / 2 + col0)
                                  : *reinterpret_cast<const float4*>(stage + ((sp * p.nw + 1) * rpr + rl) * BN + col0);
          a1.x += g.x; a1.y += g.y; a1.z += g.z; a1.w += g.w;
        }
      }
      if (p.row_scale || p.dn_part) {
        // two-plane form: undo the token's power-of-two pre-scale (exact); deferred norm: the row's rstd
        const float rs = p.row_scale ? p.row_scale[m] : (rl == row0 ? rs_pf : deferred_rstd(p, m));
        a0.x *= rs; a0.y *= rs; a0.z *= rs; a0.w *= rs;
        a1.x *= rs; a1.y *= rs; a1.z *= rs; a1.w *= rs;
      }
      {
      // Every rounding point is the one the reference's bf16 torch modules have: linear output,
      // GELU output, product, gated value, residual sum.
      float o[4] = {bf16_round(a0.x * s0[0] + b0[0]), bf16_round(a0.y * s0[1] + b0[1]),
                    bf16_round(a0.z * s0[2] + b0[2]), bf16_round(a0.w * s0[3] + b0[3])};
      if (p.epi == EPI_GELU) {
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = gelu_tanh_fast(o[e]);
      } else if (p.epi == EPI_GEGLU || p.epi == EPI_GEGLU_PACKED) {
        const float u[4] = {bf16_round(a1.x * s1[0] + b1[0]), bf16_round(a1.y * s1[1] + b1[1]),
                            bf16_round(a1.z * s1[2] + b1[2]), bf16_round(a1.w * s1[3] + b1[3])};
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = bf16_round(gelu_tanh_fast(o[e])) * u[e];
      } else if (p.epi == EPI_QKV_ROPE) {
        // o = dimensions d..d+3 of one head slot, u = their partners d + D/2; rotate q and k
        // slots (bf16 rounding points of rope.py:67-75), pass v through, store both halves.
        const RopeEpi& r = p.rope;
        float u[4] = {bf16_round(a1.x * s1[0] + b1[0]), bf16_round(a1.y * s1[1] + b1[1]),
                      bf16_round(a1.z * s1[2] + b1[2]), bf16_round(a1.w * s1[3] + b1[3])};
        const int tps = r.D >> 7;  // 128-row tiles per head slot
        const int slot = n_tile / tps;
        const int d = (n_tile - slot * tps) * 64 + col0;
        const int half = r.D >> 1;
        if (slot < r.H + r.G) {
          uint2 c0 = res_pf[0], c1 = res_pf[1], n0 = res_pf[2], n1 = res_pf[3];
          if (rl != row0) {
            const long long tb = static_cast<long long>(r.pos[m]) * r.D + d;
            c0 = *reinterpret_cast<const uint2*>(r.cos + tb); c1 = *reinterpret_cast<const uint2*>(r.cos + tb + half);
            n0 = *reinterpret_cast<const uint2*>(r.sin + tb); n1 = *reinterpret_cast<const uint2*>(r.sin + tb + half);
          }
          const __nv_bfloat16* pc0 = reinterpret_cast<const __nv_bfloat16*>(&c0);
          const __nv_bfloat16* pc1 = reinterpret_cast<const __nv_bfloat16*>(&c1);
          const __nv_bfloat16* pn0 = reinterpret_cast<const __nv_bfloat16*>(&n0);
          const __nv_bfloat16* pn1 = reinterpret_cast<const __nv_bfloat16*>(&n1);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float lo = o[e], hi = u[e];  // rotate_half(x) = (-x2, x1)
            o[e] = rope1(lo, -hi, __bfloat162float(pc0[e]), __bfloat162float(pn0[e]));
            u[e] = rope1(hi, lo, __bfloat162float(pc1[e]), __bfloat162float(pn1[e]));
          }
        }
        __nv_bfloat16* dst;
        if (slot < r.H) {
          dst = r.q + (static_cast<long long>(m) * r.H + slot) * r.D;
        } else {
          const int g = (slot - r.H) % r.G;
          const int b = m / r.L, t = m - b * r.L;
          dst = (slot < r.H + r.G ? r.kcache : r.vcache) +
                ((static_cast<long long>(b) * r.G + g) * r.Lcap + r.key_off + t) * r.D;
        }
        const __nv_bfloat162 l01 = __floats2bfloat162_rn(o[0], o[1]), l23 = __floats2bfloat162_rn(o[2], o[3]);
        const __nv_bfloat162 h01 = __floats2bfloat162_rn(u[0], u[1]), h23 = __floats2bfloat162_rn(u[2], u[3]);
        uint2 st;
        st.x = *reinterpret_cast<const uint32_t*>(&l01); st.y = *reinterpret_cast<const uint32_t*>(&l23);
        *reinterpret_cast<uint2*>(dst + d) = st;
        st.x = *reinterpret_cast<const uint32_t*>(&h01); st.y = *reinterpret_cast<const uint32_t*>(&h23);
        *reinterpret_cast<uint2*>(dst + half + d) = st;
        continue;
      } else if (p.epi == EPI_RESIDUAL) {
        if (p.gate) {
          const long long gi = static_cast<long long>(m / p.rows_per_gate) * p.ldgate + n;
          float gv[4];
          if (p.gate_bf16) {
            const uint2 gr = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p.gate) + gi);
            const __nv_bfloat162 g01 = *reinterpret_cast<const __nv_bfloat162*>(&gr.x);
            const __nv_bfloat162 g23 = *reinterpret_cast<const __nv_bfloat162*>(&gr.y);
            gv[0] = __bfloat162float(g01.x); gv[1] = __bfloat162float(g01.y);
            gv[2] = __bfloat162float(g23.x); gv[3] = __bfloat162float(g23.y);
          } else {
            const float4 gr = m / p.rows_per_gate == gate_pf_group
                                  ? gate_pf
                                  : *reinterpret_cast<const float4*>(static_cast<const float*>(p.gate) + gi);
            gv[0] = bf16_round(gr.x); gv[1] = bf16_round(gr.y); gv[2] = bf16_round(gr.z); gv[3] = bf16_round(gr.w);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) o[e] = bf16_round(o[e] * gv[e]);
        }
        const int u = (rl - rgrp) / EW;
        const uint2 rr = u < 4 ? res_pf[u < 4 ? u : 0]
                               : *reinterpret_cast<const uint2*>(p.res + static_cast<long long>(m) * p.ldres + n);
        const __nv_bfloat162 r01 = *reinterpret_cast<const __nv_bfloat162*>(&rr.x);
        const __nv_bfloat162 r23 = *reinterpret_cast<const __nv_bfloat162*>(&rr.y);
        o[0] += __bfloat162float(r01.x); o[1] += __bfloat162float(r01.y);
        o[2] += __bfloat162float(r23.x); o[3] += __bfloat162float(r23.y);
      }
      const __nv_bfloat162 o01 = __floats2bfloat162_rn(o[0], o[1]);
      const __nv_bfloat162 o23 = __floats2bfloat162_rn(o[2], o[3]);
      if (p.y) {
        uint2 st;
        st.x = *reinterpret_cast<const uint32_t*>(&o01);
        st.y = *reinterpret_cast<const uint32_t*>(&o23);
        *reinterpret_cast<uint2*>(p.y + static_cast<long long>(m) * p.ldy + n) = st;
      }
      if (p.y_planes) {
        // The next GEMM's activation planes, from the bf16-rounded values just produced.
        float xs[4] = {__bfloat162float(o01.x), __bfloat162float(o01.y), __bfloat162float(o23.x), __bfloat162float(o23.y)};
        if (p.nn_scale) {
          // Next norm folded in: this tile's share of the row's sum of squares (the warp holds the 128
          // channels of one row) and planes of bf16(x * (1 + scale)) instead of planes of x.
          float ss = (xs[0] * xs[0] + xs[1] * xs[1]) + (xs[2] * xs[2] + xs[3] * xs[3]);
#pragma unroll
          for (int sh = 16; sh > 0; sh >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sh);
          if (v4 == 0) p.nn_part[static_cast<long long>(n_tile) * p.M + m] = ss;
#pragma unroll
          for (int e = 0; e < 4; ++e) xs[e] = bf16_round(xs[e] * nsc[e]);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) xs[e] *= p.plane_scale;
        uint32_t w1, w2, w3;
        split3_quad(xs, w1, w2, w3);
        uint8_t* dst = p.y_planes + static_cast<long long>(m) * p.n_out + n;
        *reinterpret_cast<uint32_t*>(dst) = w1;
        *reinterpret_cast<uint32_t*>(dst + plane) = w2;
        *reinterpret_cast<uint32_t*>(dst + 2 * plane) = w3;
      }
      }
    }
  }

  if (tr && tid == 64) tr[7] = clock64();
  // After the meeting point nobody touches another CTA's shared memory: CTAs leave on their own.
  if (PAIR) {  // tensor memory of a pair is released together, once both CTAs have read theirs
    tc_fence_before();
    __syncwarp();
    cluster_sync_all();
  } else {
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem, p.tmem_cols);
    else tmem_dealloc(tmem, p.tmem_cols);
  }
  if (tid == 0) dbg_stage(p.dbg, KID, 4);
}

// ------------------------------------------------------------------------------------ split kernel
// x[M,K] (bf16, row stride ldx) -> three e5m2 planes [3][M][K] holding x * 2^shift.
__global__ void split3_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ planes, int M,
                              int K, float mult, int pdl) {
  if (pdl) pdl_launch_dependents();  // the next kernel may start its preamble now
  if (pdl) pdl_wait();
  const long long plane = static_cast<long long>(M) * K;
  const int kv = K / 8;  // 8 elements per thread
  const long long total = static_cast<long long>(M) * kv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int m = static_cast<int>(i / kv), c = static_cast<int>(i % kv);
    const uint4 raw = *reinterpret_cast<const uint4*>(x + m * ldx + c * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float lo[4] = {__bfloat162float(h[0].x) * mult, __bfloat162float(h[0].y) * mult, __bfloat162float(h[1].x) * mult,
                   __bfloat162float(h[1].y) * mult};
    float hi[4] = {__bfloat162float(h[2].x) * mult, __bfloat162float(h[2].y) * mult, __bfloat162float(h[3].x) * mult,
                   __bfloat162float(h[3].y) * mult};
    uint2 w1, w2, w3;
    split3_quad(lo, w1.x, w2.x, w3.x);
    split3_quad(hi, w1.y, w2.y, w3.y);
    uint8_t* dst = planes + static_cast<long long>(m) * K + c * 8;
    *reinterpret_cast<uint2*>(dst) = w1;
    *reinterpret_cast<uint2*>(dst + plane) = w2;
    *reinterpret_cast<uint2*>(dst + 2 * plane) = w3;
  }
}

// ------------------------------------------------------------------------------------ host
struct Plan {
  int bt, t_tiles, n_tiles, splits, kb_total, kb_per_split, nstages, smem_bytes, tmem_cols, merge, stage_off, pair;
};

static int round_up(int a, int b) { return (a + b - 1) / b * b; }

// How many clusters of `splits` CTAs of the GEMM kernel the device runs at once (a cluster lives
// inside one GPC, so this is less than SMs / splits: 15 clusters of 8 on a B200).  A launch with
// more clusters than that runs its last ones as a second wave.
static int max_active_clusters(int splits) {
  static int cached[MAX_SPLITS + 1] = {};
  if (splits <= 1) return 1 << 30;
  if (cached[splits] == 0) {
    cudaFuncSetAttribute(w8_gemm_kernel<false, EPI_WARPS_WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, DYN_SMEM_MAX);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1, 1, splits);
    cfg.blockDim = dim3(THREADS_WIDE);
    cfg.dynamicSmemBytes = DYN_SMEM_MAX;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = splits;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, w8_gemm_kernel<false, EPI_WARPS_WIDE>, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = host::sm_count() / (2 * splits);  // conservative guess
    }
    cached[splits] = std::max(1, n);
  }
  return cached[splits];
}

static bool make_plan(int M, int N, int K, int nw, int force_bt, int force_splits, Plan& pl, int np = 3) {
  const int max_bt = nw == 2 ? 128 : 256;
  int bt;
  if (force_bt > 0) {
    bt = force_bt;
  } else {
    // Token tiles of at most 80 keep 3*bt <= 256, so the three planes are one UMMA per K slice
    // (measured on 544 x 2048 x 16384: 733 vs 447 TFLOP/s against 112-token tiles).
    // Between caps of 80 and 64 tokens take the one with the cheaper wave count: a wave costs
    // about bt + 24 token-columns of MMA time (544 x 2048 x 16384: 112 tiles of 80 -> 54 us,
    // 144 tiles of 64 -> 51 us; 544 x 2560 x 2048: 140 tiles of 80 -> 13.5 us, 180 of 64 -> 23 us).
    const int sms = host::sm_count();
    const int n_tiles = (N + BN - 1) / BN;
    long long best_cost = 0;
    bt = 0;
    // Two planes: np * bt <= 256 allows token tiles up to 128 (caps 128 / 112 / 96 / 80 / 64).  Their
    // cost model knows the two launch forms: up to 2 * SMs tiles run one CTA per SM in whole waves; from
    // there on (CTA pairs, two CTAs per SM, one tile's epilogue under the other's main loop) CTAs start
    // as others finish, a "wave" of 2 * SMs tiles costs 1.5 single waves and fractions of it count.
    // Measured against forced tiles of 64 .. 128 the pick is within a few percent of the best from 544
    // tokens up; between 256 and 800 tokens with short K the spread between tiles is inside the noise.
    const int caps3[5] = {80, 64, 0, 0, 0}, caps2[5] = {128, 112, 96, 80, 64};
    double best2 = 0.0;
    for (int ci = 0; ci < 5; ++ci) {
      const int cap = np == 2 ? caps2[ci] : caps3[ci];
      if (cap == 0) break;
      if (ci > 0 && M <= (np == 2 ? 128 : 80)) break;  // one tile already: do not stream the weights twice
      const int tiles = (M + cap - 1) / cap;
      const int cand = round_up((M + tiles - 1) / tiles, 16);
      const long long ctas = static_cast<long long>((M + cand - 1) / cand) * n_tiles;
      if (np == 2) {
        const bool multi = ctas >= 2 * sms && nw == 1;
        const double waves = multi ? std::max(1.0, static_cast<double>(ctas) / (2.0 * sms)) * 1.5
                                   : static_cast<double>((ctas + sms - 1) / sms);
        const double cost = waves * (cand + 24);
        if (bt == 0 || cost < best2) { bt = cand; best2 = cost; }
      } else {
        const long long waves = (ctas + sms - 1) / sms;
        const long long cost = waves * (cand + 24);
        if (bt == 0 || cost < best_cost) { bt = cand; best_cost = cost; }
      }
    }
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
    if (tiles * 2 <= sms) splits = std::min(sms / tiles, std::max(1, pl.kb_total / 2));  // >= 2 K blocks per split
    splits = std::max(1, std::min(std::min(splits, MAX_SPLITS), pl.kb_total));
    // every cluster must be resident at once (2048 x 16384, 16 tiles: 8 splits 17 us, 6 splits 11 us)
    while (splits > 1 && tiles > max_active_clusters(splits)) --splits;
  }
  splits = std::max(1, std::min(std::min(splits, MAX_SPLITS), pl.kb_total));
  // Multi-wave full-K launches run as CTA pairs (one UMMA of 256 weight rows per two CTAs): each
  // CTA then loads half of the activation planes, a third less shared-memory fill per MMA and a
  // third stage in the same shared memory (4146 x 3072 x 14336: 503 -> 409 us; 544 x 32768 x 2048:
  // unchanged; single-wave launches lose a microsecond to the pair's set-up, so they stay single).
  pl.pair = (splits == 1 && nw == 1 && np * bt <= 256 && pl.n_tiles % 2 == 0 &&
             pl.t_tiles * pl.n_tiles >= 2 * host::sm_count()) ? 1 : 0;
  const int stage_bytes = pl.pair ? W_TILE_BYTES + np * bt * 64 : nw * W_TILE_BYTES + np * bt * 128;
  for (;; --splits) {  // fewer splits if the split-K staging tile does not fit beside the ring
    pl.kb_per_split = (pl.kb_total + splits - 1) / splits;
    pl.splits = (pl.kb_total + pl.kb_per_split - 1) / pl.kb_per_split;  // no empty split
    // Staging tile of the epilogue: [splits][nw][rows per rank][128] fp32.
    const int rpr = (bt + pl.splits - 1) / pl.splits;
    const int staging = round_up(pl.splits * nw * rpr * BN * 4, 1024);
    const int extra = pl.splits > 1 ? staging : 0;
    pl.nstages = std::min(MAX_STAGES, (DYN_SMEM_MAX - 1024 - extra) / stage_bytes);  // 1 KB of alignment slack
    pl.nstages = std::min(pl.nstages, std::max(2, pl.kb_per_split));
    // Several waves of full-K tiles: a shallower ring lets two CTAs share an SM, so one tile's
    // epilogue runs under the other's main loop (measured on 544 x 32768 x 2048: 117 vs 156 us).
    if (pl.splits == 1 && pl.t_tiles * pl.n_tiles >= 2 * host::sm_count() && nw * np * bt <= 256) {
      const int shared = (CORESIDENT_SMEM - 1024) / stage_bytes;
      if (shared >= 2) pl.nstages = std::min(pl.nstages, shared);
    }
    while (pl.splits == 1 && pl.nstages * stage_bytes < staging) ++pl.nstages;  // the ring doubles as the tile
    pl.stage_off = pl.splits > 1 ? pl.nstages * stage_bytes : 0;
    pl.smem_bytes = pl.nstages * stage_bytes + extra + 1024;
    if (pl.nstages >= 2 && pl.nstages <= MAX_STAGES && pl.smem_bytes <= DYN_SMEM_MAX) break;
    if (splits == 1) return false;
  }
  pl.merge = (np * bt <= 256 && nw * np * bt <= 512) ? 1 : 0;
  pl.tmem_cols = 32;
  while (pl.tmem_cols < nw * bt * (pl.merge ? np : 1)) pl.tmem_cols *= 2;
  return true;
}

// AdaRMS norm folded into the GEMMs on either side of it (see GemmParams).
struct NormFold {
  const float* next_scale = nullptr;  // producer
  float* part_out = nullptr;
  const float* part_in = nullptr;     // consumer
  int part_tiles = 0;
  int norm_width = 0;
  float eps = 0.f;
  const float* bias_rows = nullptr;
};

static int launch_gemm(const uint8_t* planes, const void* w0, const void* w1, const float* s0, const float* s1,
                       const void* bias, void* y, void* y_planes, int M, int N, int K, long long ldy, int epi,
                       const void* res, long long ldres, const void* gate, long long ldgate, int rows_per_gate,
                       int gate_bf16, int x_shift, int out_shift, int force_bt, int force_splits, int* status,
                       cudaStream_t stream, const RopeEpi* rope = nullptr, bool check_only = false,
                       const float* row_scale = nullptr, const NormFold* fold = nullptr) {
  const int np = row_scale ? 2 : 3;  // two e4m3 planes with a per-token scale, or three e5m2 planes
  const int nw = w1 ? 2 : 1;
  if (!planes || !w0 || !s0 || (!y && !y_planes && !rope)) return host::fail(TYBOK_ERR_ARG, "w8 gemm: null pointer argument");
  if (M <= 0 || N <= 0 || K <= 0) return host::fail(TYBOK_ERR_ARG, "w8 gemm: M, N, K must be positive");
  if (K % 16 != 0) return host::fail(TYBOK_ERR_ARG, "w8 gemm: K must be a multiple of 16 (TMA row pitch)");
  if (N % 4 != 0) return host::fail(TYBOK_ERR_ARG, "w8 gemm: N must be a multiple of 4 (vector epilogue)");
  if (epi == EPI_GEGLU_PACKED && (N % BN != 0 || w1)) return host::fail(TYBOK_ERR_ARG, "w8 gemm: packed gate/up needs 2*I % 128 == 0");
  const int n_out = epi == EPI_GEGLU_PACKED ? N / 2 : N;
  if ((reinterpret_cast<uintptr_t>(planes) | reinterpret_cast<uintptr_t>(w0) | reinterpret_cast<uintptr_t>(w1) |
       reinterpret_cast<uintptr_t>(s0) | reinterpret_cast<uintptr_t>(s1)) & 15)
    return host::fail(TYBOK_ERR_ARG, "w8 gemm: planes, w8 and scale must be 16-byte aligned");
  if (y && ((reinterpret_cast<uintptr_t>(y) & 7) || ldy % 4 != 0 || ldy < n_out))
    return host::fail(TYBOK_ERR_ARG, "w8 gemm: y must be 8-byte aligned with ldy >= N, ldy % 4 == 0");
  if (y_planes && (reinterpret_cast<uintptr_t>(y_planes) & 3))
    return host::fail(TYBOK_ERR_ARG, "w8 gemm: output planes must be 4-byte aligned");
  if (epi == EPI_RESIDUAL && (!res || (reinterpret_cast<uintptr_t>(res) & 7) || ldres % 4 != 0))
    return host::fail(TYBOK_ERR_ARG, "w8 gemm: residual epilogue needs an 8-byte aligned residual, ldres % 4 == 0");
  if (gate && rows_per_gate <= 0) return host::fail(TYBOK_ERR_ARG, "w8 gemm: rows_per_gate must be positive");
  if (x_shift < -60 || x_shift > 60 || out_shift < -60 || out_shift > 60)
    return host::fail(TYBOK_ERR_ARG, "w8 gemm: exponent shift out of range");
  if (fold && (fold->next_scale || fold->part_out)) {
    if (!fold->next_scale || !fold->part_out || epi != EPI_RESIDUAL || !y_planes || N % BN != 0 || w1)
      return host::fail(TYBOK_ERR_ARG, "w8 gemm: the next-norm form needs the residual epilogue, output planes, N % 128 == 0");
    if ((reinterpret_cast<uintptr_t>(fold->next_scale) & 15) || (reinterpret_cast<uintptr_t>(fold->part_out) & 3))
      return host::fail(TYBOK_ERR_ARG, "w8 gemm: next_scale must be 16-byte aligned");
  }
  if (fold && (fold->part_in || fold->bias_rows)) {
    if (!fold->part_in || !fold->bias_rows || fold->part_tiles <= 0 || fold->norm_width <= 0 || row_scale || w1 || bias ||
        (epi != EPI_QKV_ROPE && epi != EPI_GEGLU_PACKED && epi != EPI_NONE))
      return host::fail(TYBOK_ERR_ARG, "w8 gemm: the folded-norm form takes row sums, their tile count, the norm width and an fp32 bias");
    if (reinterpret_cast<uintptr_t>(fold->bias_rows) & 15)
      return host::fail(TYBOK_ERR_ARG, "w8 gemm: bias_rows must be 16-byte aligned");
  }
  if (int rc = host::require_sm100()) return rc;

  Plan pl;
  if (!make_plan(M, N, K, nw, force_bt, force_splits, pl, np))
    return host::fail(TYBOK_ERR_ARG, "w8 gemm: unsupported token tile (multiple of 16, <= 256, <= 128 when gated)");
  if (force_splits > MAX_SPLITS) return host::fail(TYBOK_ERR_ARG, "w8 gemm: at most 8 K splits (cluster size)");
  if ((pl.pair ? pl.t_tiles : pl.n_tiles) > 65535) return host::fail(TYBOK_ERR_ARG, "w8 gemm: grid too large");
  if (check_only) return TYBOK_OK;  // every argument check has passed; nothing was launched

  CUtensorMap tm_w0, tm_w1, tm_x;
  if (int rc = host::tensor_map_2d(&tm_w0, w0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, N, K, BK, BN)) return rc;
  tm_w1 = tm_w0;
  if (nw == 2)
    if (int rc = host::tensor_map_2d(&tm_w1, w1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, N, K, BK, BN)) return rc;
  if (pl.pair)  // half-plane boxes of the activation planes: bt/2 token rows of one plane
    if (int rc = host::tensor_map_3d(&tm_w1, planes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, M, np, K,
                                     static_cast<uint64_t>(M) * K, BK, pl.bt / 2, 1))
      return rc;
  if (int rc = host::tensor_map_3d(&tm_x, planes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, M, np, K,
                                   static_cast<uint64_t>(M) * K, BK, pl.bt, np))
    return rc;

  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.n_out = n_out;
  p.bt = pl.bt; p.nw = nw; p.splits = pl.splits; p.kb_total = pl.kb_total; p.kb_per_split = pl.kb_per_split;
  p.nstages = pl.nstages; p.tmem_cols = pl.tmem_cols; p.merge = pl.merge; p.pair = pl.pair; p.stage_off = pl.stage_off; p.epi = epi; p.pdl = host::pdl_enabled() ? 1 : 0;
  p.np = np; p.row_scale = row_scale;
  p.out_scale = row_scale ? 1.0f : ldexpf(1.0f, -x_shift);
  p.plane_scale = ldexpf(1.0f, out_shift);
  p.scale0 = s0; p.scale1 = s1; p.bias0 = static_cast<const __nv_bfloat16*>(bias);
  p.y = static_cast<__nv_bfloat16*>(y); p.ldy = ldy; p.y_planes = static_cast<uint8_t*>(y_planes);
  p.res = static_cast<const __nv_bfloat16*>(res); p.ldres = ldres;
  p.gate = gate; p.ldgate = ldgate; p.rows_per_gate = rows_per_gate > 0 ? rows_per_gate : 1; p.gate_bf16 = gate_bf16;
  p.status = status;
  p.trace = host::trace_buffer();
  p.dbg = host::counter_buffer();
  p.epi_wait_limit = host::epilogue_wait_limit() > 0 ? host::epilogue_wait_limit() : kWaitLimitCycles;
  if (rope) p.rope = *rope;
  if (fold) {
    p.nn_scale = fold->next_scale; p.nn_part = fold->part_out;
    p.dn_part = fold->part_in; p.dn_tiles = fold->part_tiles;
    p.dn_inv_w = fold->norm_width > 0 ? 1.0f / static_cast<float>(fold->norm_width) : 0.f;
    p.dn_eps = fold->eps; p.bias_f32 = fold->bias_rows;
  }

  static bool attr_set[64] = {};
  const int dev = host::current_device();
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(w8_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DYN_SMEM_MAX) != cudaSuccess ||
        cudaFuncSetAttribute(w8_gemm_kernel<false, EPI_WARPS_WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, DYN_SMEM_MAX) != cudaSuccess ||
        cudaFuncSetAttribute(w8_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DYN_SMEM_MAX) != cudaSuccess)
      return host::fail_cuda("cudaFuncSetAttribute(w8_gemm_kernel)");
    attr_set[dev] = true;
  }

  cudaLaunchConfig_t cfg{};
  cfg.gridDim = pl.pair ? dim3(pl.n_tiles, pl.t_tiles, 1) : dim3(pl.t_tiles, pl.n_tiles, pl.splits);
  // sixteen epilogue warps wherever a CTA has its SM to itself: split-K, and full-K grids of one wave
  const bool wide = !pl.pair && (pl.splits > 1 || pl.t_tiles * pl.n_tiles <= host::sm_count());
  cfg.blockDim = dim3(wide ? THREADS_WIDE : THREADS);
  cfg.dynamicSmemBytes = pl.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (p.pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (pl.splits > 1 || pl.pair) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = pl.pair ? 2 : 1;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = pl.pair ? 1 : pl.splits;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  if ((pl.pair         ? cudaLaunchKernelEx(&cfg, w8_gemm_kernel<true>, tm_w0, tm_w1, tm_x, p)
       : wide          ? cudaLaunchKernelEx(&cfg, w8_gemm_kernel<false, EPI_WARPS_WIDE>, tm_w0, tm_w1, tm_x, p)
                       : cudaLaunchKernelEx(&cfg, w8_gemm_kernel<false>, tm_w0, tm_w1, tm_x, p)) != cudaSuccess)
    return host::fail_cuda("launch w8_gemm_kernel");
  host::count_launch();
  return TYBOK_OK;
}

static int launch_split3(const void* x, long long ldx, void* planes, int M, int K, int shift, cudaStream_t stream) {
  if (!x || !planes) return host::fail(TYBOK_ERR_ARG, "split3: null pointer argument");
  if (M <= 0 || K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldx < K)
    return host::fail(TYBOK_ERR_ARG, "split3: K and ldx must be multiples of 8, ldx >= K");
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(planes) & 15) ||
      (static_cast<long long>(M) * K) % 8 != 0)
    return host::fail(TYBOK_ERR_ARG, "split3: x and planes must be 16-byte aligned");
  if (shift < -60 || shift > 60) return host::fail(TYBOK_ERR_ARG, "split3: exponent shift out of range");
  const long long total = static_cast<long long>(M) * (K / 8);
  const int threads = 256;
  const int blocks = static_cast<int>(std::min<long long>((total + threads - 1) / threads, 4 * host::sm_count()));
  const int pdl = host::pdl_enabled() ? 1 : 0;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(threads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl;
  if (cudaLaunchKernelEx(&cfg, split3_kernel, static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(planes),
                         M, K, ldexpf(1.0f, shift), pdl) != cudaSuccess)
    return host::fail_cuda("launch split3_kernel");
  host::count_launch();
  return TYBOK_OK;
}

// The argument checks of tybok_w8x3_linear without its launch (for the two-launch entry points,
// which must not start their first kernel when the second would be refused).
static int check_linear_args(const void* planes, const void* w8, const float* scale, const void* bias, void* y,
                             long long ldy, int M, int N, int K, int epilogue, const void* residual, long long ldres,
                             const void* gate, long long ldgate, int rows_per_gate, int gate_is_bf16, int token_tile,
                             int splits) {
  if (epilogue != TYBOK_EPI_NONE && epilogue != TYBOK_EPI_GELU && epilogue != TYBOK_EPI_RESIDUAL)
    return host::fail(TYBOK_ERR_ARG, "w8x3_linear: unknown epilogue");
  return launch_gemm(static_cast<const uint8_t*>(planes), w8, nullptr, scale, nullptr, bias, y, nullptr, M, N, K, ldy,
                     epilogue, residual, ldres, gate, ldgate, rows_per_gate, gate_is_bf16, TYBOK_DEFAULT_X_SHIFT, 0,
                     token_tile, splits, nullptr, nullptr, nullptr, true);
}

}  // namespace tb

extern "C" {

size_t tybok_w8a16_workspace_bytes(int M, int N, int K, int dual) {
  (void)N;
  (void)dual;
  return static_cast<size_t>(3) * static_cast<size_t>(M > 0 ? M : 0) * static_cast<size_t>(K > 0 ? K : 0);
}

int tybok_split3(const void* x, int64_t ldx, void* planes, int M, int K, int x_shift, void* stream) {
  return tb::launch_split3(x, ldx, planes, M, K, x_shift, static_cast<cudaStream_t>(stream));
}

int tybok_w8x3_linear(const void* x_planes, int x_shift, const void* w8, const float* scale, const void* bias, void* y,
                      int64_t ldy, void* y_planes, int out_shift, int M, int N, int K, int epilogue,
                      const void* residual, int64_t ldres, const void* gate, int64_t ldgate, int rows_per_gate,
                      int gate_is_bf16, int token_tile, int splits, int* status_word, void* stream) {
  if (epilogue != TYBOK_EPI_NONE && epilogue != TYBOK_EPI_GELU && epilogue != TYBOK_EPI_RESIDUAL)
    return tb::host::fail(TYBOK_ERR_ARG, "w8x3_linear: unknown epilogue");
  return tb::launch_gemm(static_cast<const uint8_t*>(x_planes), w8, nullptr, scale, nullptr, bias, y, y_planes, M, N, K,
                         ldy, epilogue, residual, ldres, gate, ldgate, rows_per_gate, gate_is_bf16, x_shift, out_shift,
                         token_tile, splits, status_word, static_cast<cudaStream_t>(stream));
}

int tybok_w8x3_geglu(const void* x_planes, int x_shift, const void* w8_gate, const float* scale_gate, const void* w8_up,
                     const float* scale_up, void* h, int64_t ldh, void* h_planes, int out_shift, int M, int I, int K,
                     int token_tile, int splits, int* status_word, void* stream) {
  if (!w8_up || !scale_up) return tb::host::fail(TYBOK_ERR_ARG, "w8x3_geglu: null up-projection");
  return tb::launch_gemm(static_cast<const uint8_t*>(x_planes), w8_gate, w8_up, scale_gate, scale_up, nullptr, h,
                         h_planes, M, I, K, ldh, tb::EPI_GEGLU, nullptr, 0, nullptr, 0, 1, 0, x_shift, out_shift,
                         token_tile, splits, status_word, static_cast<cudaStream_t>(stream));
}

int tybok_w8x3_geglu_packed(const void* x_planes, int x_shift, const void* w8_packed, const float* scale_packed, void* h,
                            int64_t ldh, void* h_planes, int out_shift, int M, int I, int K, int token_tile, int splits,
                            int* status_word, void* stream) {
  return tb::launch_gemm(static_cast<const uint8_t*>(x_planes), w8_packed, nullptr, scale_packed, nullptr, nullptr, h,
                         h_planes, M, 2 * I, K, ldh, tb::EPI_GEGLU_PACKED, nullptr, 0, nullptr, 0, 1, 0, x_shift,
                         out_shift, token_tile, splits, status_word, static_cast<cudaStream_t>(stream));
}

int tybok_w8x3_qkv_rope(const void* x_planes, int x_shift, const void* w8_paired, const float* scale_paired,
                        const int* pos, const void* cos_table, const void* sin_table, void* q_out, void* k_cache,
                        void* v_cache, int B, int L, int H, int G, int D, int Lcap, int key_off, int K, int token_tile,
                        int splits, int* status_word, void* stream) {
  if (!pos || !cos_table || !sin_table || !q_out || !k_cache || !v_cache)
    return tb::host::fail(TYBOK_ERR_ARG, "qkv_rope: null pointer argument");
  if (B <= 0 || L <= 0 || H <= 0 || G <= 0 || D <= 0 || D % 128 != 0 || key_off < 0 || key_off + L > Lcap)
    return tb::host::fail(TYBOK_ERR_ARG, "qkv_rope: needs head_dim % 128 == 0 and key_off + L <= Lcap");
  if ((reinterpret_cast<uintptr_t>(cos_table) | reinterpret_cast<uintptr_t>(sin_table) |
       reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 7)
    return tb::host::fail(TYBOK_ERR_ARG, "qkv_rope: tables, q and caches must be 8-byte aligned");
  tb::RopeEpi r{};
  r.pos = pos; r.cos = static_cast<const __nv_bfloat16*>(cos_table); r.sin = static_cast<const __nv_bfloat16*>(sin_table);
  r.q = static_cast<__nv_bfloat16*>(q_out); r.kcache = static_cast<__nv_bfloat16*>(k_cache);
  r.vcache = static_cast<__nv_bfloat16*>(v_cache);
  r.L = L; r.H = H; r.G = G; r.D = D; r.Lcap = Lcap; r.key_off = key_off;
  return tb::launch_gemm(static_cast<const uint8_t*>(x_planes), w8_paired, nullptr, scale_paired, nullptr, nullptr,
                         nullptr, nullptr, B * L, (H + 2 * G) * D, K, 0, tb::EPI_QKV_ROPE, nullptr, 0, nullptr, 0, 1, 0,
                         x_shift, 0, token_tile, splits, status_word, static_cast<cudaStream_t>(stream), &r);
}

int tybok_w8x2_gemm(const void* x_planes2, const float* row_scale, const void* w8, const float* scale, const void* bias,
                    void* y, int64_t ldy, void* y_planes, int out_shift, int M, int N, int K, int epilogue,
                    const void* residual, int64_t ldres, const void* gate, int64_t ldgate, int rows_per_gate,
                    int gate_is_bf16, int token_tile, int splits, int* status_word, void* stream) {
  if (!row_scale) return tb::host::fail(TYBOK_ERR_ARG, "w8x2_gemm: null row_scale");
  if (epilogue != TYBOK_EPI_NONE && epilogue != TYBOK_EPI_GELU && epilogue != TYBOK_EPI_RESIDUAL &&
      epilogue != TYBOK_EPI_GEGLU_PACKED)
    return tb::host::fail(TYBOK_ERR_ARG, "w8x2_gemm: unknown epilogue");
  // the packed gated form takes N = 2*I weight rows and writes I output columns
  return tb::launch_gemm(static_cast<const uint8_t*>(x_planes2), w8, nullptr, scale, nullptr, bias, y, y_planes, M, N, K,
                         ldy, epilogue == TYBOK_EPI_GEGLU_PACKED ? tb::EPI_GEGLU_PACKED : epilogue, residual, ldres, gate,
                         ldgate, rows_per_gate, gate_is_bf16, 0, out_shift, token_tile, splits, status_word,
                         static_cast<cudaStream_t>(stream), nullptr, false, row_scale);
}

int tybok_w8x2_qkv_rope(const void* x_planes2, const float* row_scale, const void* w8_paired, const float* scale_paired,
                        const int* pos, const void* cos_table, const void* sin_table, void* q_out, void* k_cache,
                        void* v_cache, int B, int L, int H, int G, int D, int Lcap, int key_off, int K, int token_tile,
                        int splits, int* status_word, void* stream) {
  if (!row_scale || !pos || !cos_table || !sin_table || !q_out || !k_cache || !v_cache)
    return tb::host::fail(TYBOK_ERR_ARG, "w8x2_qkv_rope: null pointer argument");
  if (B <= 0 || L <= 0 || H <= 0 || G <= 0 || D <= 0 || D % 128 != 0 || key_off < 0 || key_off + L > Lcap)
    return tb::host::fail(TYBOK_ERR_ARG, "w8x2_qkv_rope: needs head_dim % 128 == 0 and key_off + L <= Lcap");
  if ((reinterpret_cast<uintptr_t>(cos_table) | reinterpret_cast<uintptr_t>(sin_table) |
       reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 7)
    return tb::host::fail(TYBOK_ERR_ARG, "w8x2_qkv_rope: tables, q and caches must be 8-byte aligned");
  tb::RopeEpi r{};
  r.pos = pos; r.cos = static_cast<const __nv_bfloat16*>(cos_table); r.sin = static_cast<const __nv_bfloat16*>(sin_table);
  r.q = static_cast<__nv_bfloat16*>(q_out); r.kcache = static_cast<__nv_bfloat16*>(k_cache);
  r.vcache = static_cast<__nv_bfloat16*>(v_cache);
  r.L = L; r.H = H; r.G = G; r.D = D; r.Lcap = Lcap; r.key_off = key_off;
  return tb::launch_gemm(static_cast<const uint8_t*>(x_planes2), w8_paired, nullptr, scale_paired, nullptr, nullptr,
                         nullptr, nullptr, B * L, (H + 2 * G) * D, K, 0, tb::EPI_QKV_ROPE, nullptr, 0, nullptr, 0, 1, 0, 0,
                         0, token_tile, splits, status_word, static_cast<cudaStream_t>(stream), &r, false, row_scale);
}

int tybok_w8x3_residual_next_adarms(const void* x_planes, int x_shift, const void* w8, const float* scale, void* y,
                                    int64_t ldy, const void* residual, int64_t ldres, const float* gate,
                                    const float* next_scale, void* u_planes, int u_shift, float* ss_part, int M, int N,
                                    int K, int token_tile, int splits, int* status_word, void* stream) {
  if (!y || !gate || !next_scale || !u_planes || !ss_part)
    return tb::host::fail(TYBOK_ERR_ARG, "w8x3_residual_next_adarms: null pointer argument");
  tb::NormFold f;
  f.next_scale = next_scale; f.part_out = ss_part;
  return tb::launch_gemm(static_cast<const uint8_t*>(x_planes), w8, nullptr, scale, nullptr, nullptr, y, u_planes, M, N, K,
                         ldy, tb::EPI_RESIDUAL, residual, ldres, gate, 0, M, 0, x_shift, u_shift, token_tile, splits,
                         status_word, static_cast<cudaStream_t>(stream), nullptr, false, nullptr, &f);
}

int tybok_w8x3_geglu_packed_adarms(const void* u_planes, int u_shift, const float* ss_part, int ss_tiles, float eps,
                                   const float* bias_rows, const void* w8_packed, const float* scale_packed, void* h,
                                   int64_t ldh, void* h_planes, int out_shift, int M, int I, int K, int token_tile,
                                   int splits, int* status_word, void* stream) {
  tb::NormFold f;
  f.part_in = ss_part; f.part_tiles = ss_tiles; f.norm_width = K; f.eps = eps; f.bias_rows = bias_rows;
  if (!ss_part || !bias_rows) return tb::host::fail(TYBOK_ERR_ARG, "w8x3_geglu_packed_adarms: null pointer argument");
  return tb::launch_gemm(static_cast<const uint8_t*>(u_planes), w8_packed, nullptr, scale_packed, nullptr, nullptr, h,
                         h_planes, M, 2 * I, K, ldh, tb::EPI_GEGLU_PACKED, nullptr, 0, nullptr, 0, 1, 0, u_shift,
                         out_shift, token_tile, splits, status_word, static_cast<cudaStream_t>(stream), nullptr, false,
                         nullptr, &f);
}

int tybok_w8x3_qkv_rope_adarms(const void* u_planes, int u_shift, const float* ss_part, int ss_tiles, float eps,
                               const float* bias_rows, const void* w8_paired, const float* scale_paired, const int* pos,
                               const void* cos_table, const void* sin_table, void* q_out, void* k_cache, void* v_cache,
                               int B, int L, int H, int G, int D, int Lcap, int key_off, int K, int token_tile,
                               int splits, int* status_word, void* stream) {
  if (!ss_part || !bias_rows || !pos || !cos_table || !sin_table || !q_out || !k_cache || !v_cache)
    return tb::host::fail(TYBOK_ERR_ARG, "w8x3_qkv_rope_adarms: null pointer argument");
  if (B <= 0 || L <= 0 || H <= 0 || G <= 0 || D <= 0 || D % 128 != 0 || key_off < 0 || key_off + L > Lcap)
    return tb::host::fail(TYBOK_ERR_ARG, "w8x3_qkv_rope_adarms: needs head_dim % 128 == 0 and key_off + L <= Lcap");
  if ((reinterpret_cast<uintptr_t>(cos_table) | reinterpret_cast<uintptr_t>(sin_table) |
       reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 7)
    return tb::host::fail(TYBOK_ERR_ARG, "w8x3_qkv_rope_adarms: tables, q and caches must be 8-byte aligned");
  tb::RopeEpi r{};
  r.pos = pos; r.cos = static_cast<const __nv_bfloat16*>(cos_table); r.sin = static_cast<const __nv_bfloat16*>(sin_table);
  r.q = static_cast<__nv_bfloat16*>(q_out); r.kcache = static_cast<__nv_bfloat16*>(k_cache);
  r.vcache = static_cast<__nv_bfloat16*>(v_cache);
  r.L = L; r.H = H; r.G = G; r.D = D; r.Lcap = Lcap; r.key_off = key_off;
  tb::NormFold f;
  f.part_in = ss_part; f.part_tiles = ss_tiles; f.norm_width = K; f.eps = eps; f.bias_rows = bias_rows;
  return tb::launch_gemm(static_cast<const uint8_t*>(u_planes), w8_paired, nullptr, scale_paired, nullptr, nullptr,
                         nullptr, nullptr, B * L, (H + 2 * G) * D, K, 0, tb::EPI_QKV_ROPE, nullptr, 0, nullptr, 0, 1, 0,
                         u_shift, 0, token_tile, splits, status_word, static_cast<cudaStream_t>(stream), &r, false,
                         nullptr, &f);
}

int tybok_w8a16_linear(const void* x, const void* w8, const float* scale, const void* bias, void* y, int M, int N,
                       int K, int64_t ldx, int64_t ldy, int epilogue, const void* residual, int64_t ldres,
                       const void* gate, int64_t ldgate, int rows_per_gate, int gate_is_bf16, int token_tile,
                       int splits, void* workspace, size_t workspace_bytes, int* status_word, void* stream) {
  if (!workspace || workspace_bytes < tybok_w8a16_workspace_bytes(M, N, K, 0))
    return tb::host::fail(TYBOK_ERR_WORKSPACE, "w8a16_linear: workspace must hold 3*M*K bytes of activation planes");
  const int shift = TYBOK_DEFAULT_X_SHIFT;
  // Refuse a bad GEMM argument before the split kernel has written anything.
  if (int rc = tb::check_linear_args(workspace, w8, scale, bias, y, ldy, M, N, K, epilogue, residual, ldres, gate, ldgate,
                                     rows_per_gate, gate_is_bf16, token_tile, splits))
    return rc;
  if (int rc = tybok_split3(x, ldx, workspace, M, K, shift, stream)) return rc;
  return tybok_w8x3_linear(workspace, shift, w8, scale, bias, y, ldy, nullptr, 0, M, N, K, epilogue, residual, ldres,
                           gate, ldgate, rows_per_gate, gate_is_bf16, token_tile, splits, status_word, stream);
}

// ---- W8A16 linear for callers that may not allocate ------------------------------------------
// Some hosts of this library cannot hand it a workspace: a plugin running inside a serving
// process whose memory pool is owned (and fully reserved) by another runtime, a real-time
// control loop that forbids allocator calls after start-up, or a foreign-language binding that
// has no device allocator at all.  For them the activation planes of tybok_w8a16_linear live in
// this fixed device array instead of a caller-provided buffer.  Every GPU that loads the
// library holds the array until the process exits.
static __device__ __align__(256) uint8_t g_static_planes[TYBOK_STATIC_PLANES_BYTES];

// Host code must not pass `g_static_planes` itself to a kernel or a tensor map: on the host
// that name is only a stand-in for the symbol.  Its device address is looked up once per
// device, with that device current.
static void* static_planes_ptr(int* rc) {
  static std::atomic<void*> ptr[64];  // zero-initialised; two threads racing on a first call store the same address
  *rc = TYBOK_OK;
  const int dev = tb::host::current_device();
  if (dev < 0 || dev >= 64) {
    *rc = tb::host::fail(TYBOK_ERR_CUDA, "w8a16_linear_noalloc: no current CUDA device");
    return nullptr;
  }
  void* p = ptr[dev].load(std::memory_order_acquire);
  if (!p) {
    if (cudaGetSymbolAddress(&p, g_static_planes) != cudaSuccess || !p) {
      *rc = tb::host::fail_cuda("w8a16_linear_noalloc: cudaGetSymbolAddress(g_static_planes)");
      return nullptr;
    }
    ptr[dev].store(p, std::memory_order_release);
  }
  return p;
}

int tybok_w8a16_linear_noalloc(const void* x, const void* w8, const float* scale, const void* bias, void* y, int M,
                               int N, int K, int64_t ldx, int64_t ldy, int epilogue, const void* residual,
                               int64_t ldres, const void* gate, int64_t ldgate, int rows_per_gate, int gate_is_bf16,
                               int* status_word, void* stream) {
  if (M <= 0 || K <= 0) return tb::host::fail(TYBOK_ERR_ARG, "w8a16_linear_noalloc: M and K must be positive");
  const size_t need = static_cast<size_t>(3) * static_cast<size_t>(M) * static_cast<size_t>(K);
  if (need > TYBOK_STATIC_PLANES_BYTES)
    return tb::host::fail(TYBOK_ERR_WORKSPACE,
                          "w8a16_linear_noalloc: 3*M*K exceeds TYBOK_STATIC_PLANES_BYTES (1.5 MiB); use "
                          "tybok_w8a16_linear with a caller-owned workspace for larger problems");
  int rc = TYBOK_OK;
  void* planes = static_planes_ptr(&rc);
  if (!planes) return rc;
  // Nothing in the array has to start at zero: split3 overwrites all 3*M*K bytes the GEMM reads.
  const int shift = TYBOK_DEFAULT_X_SHIFT;
  // A call the GEMM would refuse must leave the shared array as it found it.
  if (int r = tb::check_linear_args(planes, w8, scale, bias, y, ldy, M, N, K, epilogue, residual, ldres, gate, ldgate,
                                    rows_per_gate, gate_is_bf16, 0, 0))
    return r;
  if (int r = tybok_split3(x, ldx, planes, M, K, shift, stream)) return r;
  return tybok_w8x3_linear(planes, shift, w8, scale, bias, y, ldy, nullptr, 0, M, N, K, epilogue, residual, ldres,
                           gate, ldgate, rows_per_gate, gate_is_bf16, 0, 0, status_word, stream);
}

int tybok_w8a16_geglu(const void* x, const void* w8_gate, const float* scale_gate, const void* w8_up,
                      const float* scale_up, void* h, int M, int I, int K, int64_t ldx, int64_t ldh, int token_tile,
                      int splits, void* workspace, size_t workspace_bytes, int* status_word, void* stream) {
  if (!workspace || workspace_bytes < tybok_w8a16_workspace_bytes(M, I, K, 1))
    return tb::host::fail(TYBOK_ERR_WORKSPACE, "w8a16_geglu: workspace must hold 3*M*K bytes of activation planes");
  const int shift = TYBOK_DEFAULT_X_SHIFT;
  if (!w8_up || !scale_up) return tb::host::fail(TYBOK_ERR_ARG, "w8a16_geglu: null up-projection");
  if (int rc = tb::launch_gemm(static_cast<const uint8_t*>(workspace), w8_gate, w8_up, scale_gate, scale_up, nullptr, h,
                               nullptr, M, I, K, ldh, tb::EPI_GEGLU, nullptr, 0, nullptr, 0, 1, 0, shift, 0, token_tile,
                               splits, nullptr, nullptr, nullptr, true))
    return rc;
  if (int rc = tybok_split3(x, ldx, workspace, M, K, shift, stream)) return rc;
  return tybok_w8x3_geglu(workspace, shift, w8_gate, scale_gate, w8_up, scale_up, h, ldh, nullptr, 0, M, I, K,
                          token_tile, splits, status_word, stream);
}

}  // extern "C"
