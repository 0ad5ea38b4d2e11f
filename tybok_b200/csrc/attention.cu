// GQA/MQA attention over [prefix KV cache ; own keys] for sm_100a, plus the RoPE/KV-store
// kernel that feeds it.
//
// rope_store_kernel: packed qkv rows (the qkv GEMM output) -> rotated q [tokens, H*D], rotated k
// and v appended to the per-layer cache at key offset `key_off` (0 for the prefix prefill,
// prefix length for the action suffix), so the attention kernel sees one contiguous key range
// and nothing is ever concatenated or expanded per head.
//
// attention_kernel: one CTA per (128-query tile of one head, 128-key block, batch element).
//   warp 0     TMA: Q tile, K block, V block (four 64-wide swizzled column chunks each).
//   warp 1     tcgen05.mma: S = Q K^T (128x128x256), then O = P V (128x256x128) with P read from
//              tensor memory and V as an MN-major shared-memory operand.
//   warps 2-9  softmax on S straight out of tensor memory (two threads per query row, 64 keys
//              each, fp32, key-validity mask), P written back to tensor memory as bf16; epilogue.
// The key blocks of one query tile form a thread-block cluster and CTA r merges query rows
// r*R..(r+1)*R-1 over all key blocks in block order (bit-reproducible).  Two exchange forms:
// short suffixes in the split-column form push every partial row straight into the shared
// memory of the CTA that merges it (bulk copies credited to the receiver's barrier); everything
// else stages its rows in a global workspace that stays in L2, meets at the cluster barrier
// and pulls.  Sequences of more than 128 queries, and every head_dim 128 call, take the
// key-loop kernel further down, which exchanges nothing.
//
// Algorithmic bytes: Q + O once per (layer, step), K + V once per (batch, kv head).
// Flops: 4 * Mq * Lk * D * H.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/tybok_b200.h"
#include "host_util.h"
#include "ptx.cuh"
#include "split3.cuh"

namespace tb {

constexpr int AT_D = 256;        // head dimension this kernel is built for
constexpr int AT_BQ = 128;       // query rows per CTA (UMMA M)
constexpr int AT_BK = 128;       // keys per CTA
constexpr int AT_CHUNK = 16384;  // one 64-column chunk of a 128-row bf16 tile (128 rows x 128 bytes)
constexpr int AT_TILE = 4 * AT_CHUNK;
constexpr int AT_THREADS = 320;
constexpr int AT_WS_PER_CTA = AT_BQ * AT_D * 4 + AT_BQ * 8;  // workspace per CTA: O rows (fp32) + (max, sum) per row
constexpr int AT_MAX_SPLITS = 8;
constexpr int AT_MERGE_BATCH = 3;  // query rows a merging thread has in flight
constexpr int AT_SMEM = 3 * AT_TILE + 1024;
// Push form: the receive area is the half of the V tile that the split-column form leaves idle;
// partial rows of 128 fp32 first, then 16 bytes of statistics per row.
constexpr int AT_PUSH_RECV = 2 * AT_CHUNK;    // offset inside the V tile
constexpr int AT_PUSH_STATS = 28 * 1024;      // offset of the statistics inside the receive area
constexpr int AT_PUSH_MAX_ROWS = 56;          // nsplit * rows per rank: 56 * 512 B = 28 KB, 56 * 16 B < 4 KB

struct RopeParams {
  const __nv_bfloat16* qkv;
  long long ldq;
  const int* pos;
  const __nv_bfloat16* cos;
  const __nv_bfloat16* sin;
  __nv_bfloat16* q_out;
  __nv_bfloat16* kcache;
  __nv_bfloat16* vcache;
  int B, L, H, G, D, Lcap, key_off, pdl;
};

__global__ void rope_store_kernel(const RopeParams p) {
  if (p.pdl) pdl_launch_dependents();  // the next kernel may start its preamble now
  if (p.pdl) pdl_wait();
  const int vec_per_head = p.D / 16;  // each thread: 8 elements of the first half + their partners
  const int slots = p.H + 2 * p.G;
  const long long total = static_cast<long long>(p.B) * p.L * slots * vec_per_head;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % vec_per_head);
    const int s = static_cast<int>((i / vec_per_head) % slots);
    const int m = static_cast<int>(i / (static_cast<long long>(vec_per_head) * slots));
    const int b = m / p.L, t = m % p.L;
    const __nv_bfloat16* src = p.qkv + m * p.ldq + s * p.D;
    const int half = p.D / 2;
    uint4 lo = *reinterpret_cast<const uint4*>(src + c * 8);
    uint4 hi = *reinterpret_cast<const uint4*>(src + half + c * 8);
    if (s < p.H + p.G) {
      const int ps = p.pos[m];
      const uint4 cl = *reinterpret_cast<const uint4*>(p.cos + static_cast<long long>(ps) * p.D + c * 8);
      const uint4 sl = *reinterpret_cast<const uint4*>(p.sin + static_cast<long long>(ps) * p.D + c * 8);
      const uint4 ch = *reinterpret_cast<const uint4*>(p.cos + static_cast<long long>(ps) * p.D + half + c * 8);
      const uint4 sh = *reinterpret_cast<const uint4*>(p.sin + static_cast<long long>(ps) * p.D + half + c * 8);
      __nv_bfloat16* xl = reinterpret_cast<__nv_bfloat16*>(&lo);
      __nv_bfloat16* xh = reinterpret_cast<__nv_bfloat16*>(&hi);
      const __nv_bfloat16* pcl = reinterpret_cast<const __nv_bfloat16*>(&cl);
      const __nv_bfloat16* psl = reinterpret_cast<const __nv_bfloat16*>(&sl);
      const __nv_bfloat16* pch = reinterpret_cast<const __nv_bfloat16*>(&ch);
      const __nv_bfloat16* psh = reinterpret_cast<const __nv_bfloat16*>(&sh);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float a = __bfloat162float(xl[e]), bb = __bfloat162float(xh[e]);
        // rotate_half(x) = (-x2, x1)
        const float ol = rope1(a, -bb, __bfloat162float(pcl[e]), __bfloat162float(psl[e]));
        const float oh = rope1(bb, a, __bfloat162float(pch[e]), __bfloat162float(psh[e]));
        xl[e] = __float2bfloat16_rn(ol);
        xh[e] = __float2bfloat16_rn(oh);
      }
    }
    __nv_bfloat16* dst;
    if (s < p.H) {
      dst = p.q_out + (static_cast<long long>(m) * p.H + s) * p.D;
    } else {
      const int g = (s - p.H) % p.G;
      __nv_bfloat16* cache = (s < p.H + p.G) ? p.kcache : p.vcache;
      dst = cache + ((static_cast<long long>(b) * p.G + g) * p.Lcap + p.key_off + t) * p.D;
    }
    *reinterpret_cast<uint4*>(dst + c * 8) = lo;
    *reinterpret_cast<uint4*>(dst + half + c * 8) = hi;
  }
}

// qk-norm + rotary embedding + KV store of a DiT block (tybok/policies/fastwam/models/dit_block.py:
// 246-273, wan_base.py:97-128): per token row, q and k are RMS-normalised over ALL heads' channels
// together (fp32 statistics, the normalised value rounded to bf16, then times a bf16 weight), rotated
// pair-wise ((x[2i], x[2i+1]) times a complex table entry, fp32, rounded to bf16) and stored: q as
// rows [M, H*D], k and the untouched v head-major into the caches [B, H, Lcap, D] at key_off.
// One CTA per row, eight channels per thread.
struct QkNormParams {
  const __nv_bfloat16* src;
  long long ld;
  int q_off, k_off, v_off;     // column of q / k / v inside a source row; negative = absent
  const __nv_bfloat16* wq;     // [H*D] norm weights
  const __nv_bfloat16* wk;
  const float* cos;            // [L][D/2] or NULL (no rotation)
  const float* sin;
  __nv_bfloat16* q_out;        // [M][H*D]
  __nv_bfloat16* kcache;       // [B][H][Lcap][D]
  __nv_bfloat16* vcache;
  int M, L, H, D, Lcap, key_off;
  float eps;
  int pdl;
  int* dbg;
};

__global__ void __launch_bounds__(512) qknorm_rope_store_kernel(const QkNormParams p) {
  __shared__ float red[2][16];
  if (p.pdl) pdl_launch_dependents();
  if (threadIdx.x == 0) dbg_stage(p.dbg, 7, 0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int m = blockIdx.x, c = threadIdx.x * 8, A = p.H * p.D;
  const bool live = c < A;
  const int b = m / p.L, t = m - b * p.L;
  const int head = live ? c / p.D : 0, d0 = live ? c - head * p.D : 0;
  // norm weights and rotary table entries are constants: fetch them before waiting for the producer
  uint4 wq = {}, wk = {};
  float4 cs = make_float4(1.f, 1.f, 1.f, 1.f), sn = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) {
    if (p.q_off >= 0) wq = *reinterpret_cast<const uint4*>(p.wq + c);
    if (p.k_off >= 0) wk = *reinterpret_cast<const uint4*>(p.wk + c);
    if (p.cos) {
      cs = *reinterpret_cast<const float4*>(p.cos + static_cast<long long>(t) * (p.D >> 1) + (d0 >> 1));
      sn = *reinterpret_cast<const float4*>(p.sin + static_cast<long long>(t) * (p.D >> 1) + (d0 >> 1));
    }
  }
  if (p.pdl) pdl_wait();
  if (threadIdx.x == 0) dbg_stage(p.dbg, 7, 2);
  const __nv_bfloat16* row = p.src + static_cast<long long>(m) * p.ld;
  uint4 rq = {}, rk = {}, rv = {};
  float ssq = 0.f, ssk = 0.f;
  if (live) {
    if (p.q_off >= 0) rq = *reinterpret_cast<const uint4*>(row + p.q_off + c);
    if (p.k_off >= 0) rk = *reinterpret_cast<const uint4*>(row + p.k_off + c);
    if (p.v_off >= 0) rv = *reinterpret_cast<const uint4*>(row + p.v_off + c);
    const __nv_bfloat16* hq = reinterpret_cast<const __nv_bfloat16*>(&rq);
    const __nv_bfloat16* hk = reinterpret_cast<const __nv_bfloat16*>(&rk);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float a = __bfloat162float(hq[e]), kk = __bfloat162float(hk[e]);
      ssq += a * a;
      ssk += kk * kk;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
    ssk += __shfl_xor_sync(0xffffffffu, ssk, o);
  }
  if (lane == 0) {
    red[0][warp] = ssq;
    red[1][warp] = ssk;
  }
  __syncthreads();
  float tq = 0.f, tk = 0.f;
  for (int w = 0; w < nwarps; ++w) {
    tq += red[0][w];
    tk += red[1][w];
  }
  if (!live) return;
  const float cosv[4] = {cs.x, cs.y, cs.z, cs.w}, sinv[4] = {sn.x, sn.y, sn.z, sn.w};
  auto finish = [&](const uint4& raw, const uint4& wraw, float total) {
    const float rstd = rsqrtf(total / static_cast<float>(A) + p.eps);
    const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&raw);
    const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(&wraw);
    float n[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) n[e] = bf16_round(bf16_round(__bfloat162float(h[e]) * rstd) * __bfloat162float(w[e]));
    uint4 out;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = n[2 * j], bb = n[2 * j + 1];
      o2[j] = p.cos ? __floats2bfloat162_rn(a * cosv[j] - bb * sinv[j], a * sinv[j] + bb * cosv[j])
                    : __floats2bfloat162_rn(a, bb);
    }
    return out;
  };
  const long long crow = ((static_cast<long long>(b) * p.H + head) * p.Lcap + p.key_off + t) * p.D + d0;
  if (p.q_off >= 0) *reinterpret_cast<uint4*>(p.q_out + static_cast<long long>(m) * A + c) = finish(rq, wq, tq);
  if (p.k_off >= 0) *reinterpret_cast<uint4*>(p.kcache + crow) = finish(rk, wk, tk);
  if (p.v_off >= 0) *reinterpret_cast<uint4*>(p.vcache + crow) = rv;
  if (threadIdx.x == 0) dbg_stage(p.dbg, 7, 4);
}

struct AttnParams {
  int B, L, H, G, Lk, Lcap;
  int nsplit;
  float scale_log2e;  // softmax scale * log2(e)
  const uint8_t* key_valid;  // [B][Lk] or NULL (all keys valid)
  __nv_bfloat16* out;        // [B*L][H*D] or NULL
  uint8_t* out_planes;       // [3][B*L][H*D] or NULL
  float plane_scale;
  int* status;
  int pdl;
  uint8_t* ws;       // [CTA][AT_WS_PER_CTA] exchange workspace (nsplit > 1)
  int q_rows;        // query rows per bulk copy: 128, or 64 when all real rows fit (the rest of the tile is never read back)
  int dsplit;        // 1, or 2: two CTAs per (query tile, key block), each producing half of the output columns
  long long* trace;  // tuning aid: [CTA][16] SM-clock samples, NULL in production
  int* dbg;          // debugging aid: stage counters, NULL in production
};

struct __align__(16) AttnBars {
  float4 stat[AT_BQ];    // push form: (max, sum of keys 0..63, sum of keys 64..127, -) of every query row of this block
  uint64_t qk_full[4];  // one per 64-column chunk of Q and K: S = Q K^T starts when the first pair has landed
  uint64_t v_full, s_full, p_full, o_full;
  uint64_t recv;         // push form: the peers' partial rows of the query rows this CTA merges have arrived
  uint64_t recv_stat;    // push form: the statistics of those rows have arrived (sent ahead, while P.V runs)
  uint64_t mma_done;     // every tensor-core instruction of this CTA has retired (awaited before the tensor memory is freed)
  uint32_t tmem_base;
  volatile int abort;
  uint32_t valid[4];     // key-validity bits of this CTA's 128 keys
  float row_max[AT_BQ];  // per query row: maximum (log2 domain) and sum of this key block
  float row_sum[AT_BQ];
  float hmax[2][AT_BQ];  // the same per half of the key block (one half per thread of a row)
  float hsum[2][AT_BQ];
  float wn[AT_MAX_SPLITS][AT_BQ];  // merge weights of the rows this CTA owns: exp2(m_s - m) / denominator
};

__device__ __forceinline__ bool at_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitLimitCycles) return false;
  }
  return true;
}

// MN-major shared-memory operand with the 128-byte swizzle: 64-element (128-byte) runs along
// N, 8 K-rows per 1024-byte group; [16,30) leading byte offset >> 4 = distance between 64-wide
// N chunks, [32,46) stride byte offset >> 4 = distance between 8-row K groups.
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// PUSH: short suffixes in the split-column form.  Every CTA sends the partial rows a peer will
// merge straight into that peer's shared memory (the idle half of its V tile) with bulk copies
// credited to the peer's barrier, so the merge starts when the rows land: no trip through L2,
// no cluster-wide meeting point before it.
template <bool PUSH>
__global__ void __launch_bounds__(AT_THREADS, 1)
attention_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ AttnBars bars;
  const long long t_start = clock64();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sq = smem;
  uint8_t* sk = smem + AT_TILE;
  uint8_t* sv = smem + 2 * AT_TILE;

  const int sp = blockIdx.x;  // key block == rank in the cluster
  const int n_qt = (p.L + AT_BQ - 1) / AT_BQ;
  // Small grids split the value / output columns over two CTAs (both compute the full S and
  // softmax; each multiplies P by its half of V): half the exchange volume per CTA.
  const int dh = blockIdx.y % p.dsplit;
  const int h = (blockIdx.y / p.dsplit) / n_qt, qt = (blockIdx.y / p.dsplit) % n_qt;
  const int dv = AT_D / p.dsplit;  // output columns of this CTA
  const int b = blockIdx.z;
  const int g = h / (p.H / p.G);
  const int key0 = sp * AT_BK;

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    for (int c = 0; c < 4; ++c) mbar_init(&bars.qk_full[c], 1);
    mbar_init(&bars.v_full, 1);
    mbar_init(&bars.s_full, 1);
    mbar_init(&bars.p_full, 8);
    mbar_init(&bars.o_full, 1);
    mbar_init(&bars.mma_done, 1);
    bars.abort = 0;
    if (PUSH) {
      mbar_init(&bars.recv, 1);
      mbar_init(&bars.recv_stat, 1);
      const int rpr = (min(AT_BQ, p.L) + p.nsplit - 1) / p.nsplit;
      const int mine = max(0, min(min(AT_BQ, p.L), (sp + 1) * rpr) - sp * rpr);
      fence_barrier_init();
      mbar_arrive_expect_tx(&bars.recv, (p.nsplit - 1) * mine * (AT_D / 2 * 4));
      mbar_arrive_expect_tx(&bars.recv_stat, (p.nsplit - 1) * mine * 16);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars.tmem_base, 512);
    tmem_relinquish();
  }
  if (warp == 2) {  // validity bits of this block's keys: the four loads in flight together
    bool ok[4];
    if (p.key_valid && p.pdl) pdl_wait();
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const int j = key0 + w * 32 + lane;
      ok[w] = j < p.Lk;
      if (ok[w] && p.key_valid) ok[w] = p.key_valid[static_cast<long long>(b) * p.Lk + j] != 0;
    }
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint32_t bits = __ballot_sync(0xffffffffu, ok[w]);
      if (lane == 0) bars.valid[w] = bits;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (PUSH) cluster_arrive_relaxed();  // this CTA's receive barrier is armed
  const uint32_t tmem = bars.tmem_base;
  const uint32_t t_s = tmem, t_p = tmem + 128, t_o = tmem + 256;
  const int nvalid = min(AT_BQ, p.L - qt * AT_BQ);  // real query rows of this tile
  uint8_t* my_ws = p.ws + static_cast<long long>((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * AT_WS_PER_CTA;
  long long* tr = p.trace ? p.trace + 16ll * ((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) : nullptr;
  if (tr && tid == 0) { tr[0] = t_start; tr[1] = clock64(); }

  if (warp == 0) {
    if (lane == 0) {
      if (p.pdl) pdl_launch_dependents();  // the o-projection GEMM may start prefetching its weights
      if (p.pdl) pdl_wait();
      const int qrow = b * p.L + qt * AT_BQ;
      const int krow = (b * p.G + g) * p.Lcap + key0;
      for (int c = 0; c < 4; ++c) {
        mbar_arrive_expect_tx(&bars.qk_full[c], AT_CHUNK + p.q_rows * 128);
        tma_load_2d(sq + c * AT_CHUNK, &tm_q, &bars.qk_full[c], h * AT_D + c * 64, qrow);
        tma_load_2d(sk + c * AT_CHUNK, &tm_k, &bars.qk_full[c], c * 64, krow);
      }
      const int nvc = dv / 64;  // 64-column chunks of V this CTA multiplies
      mbar_arrive_expect_tx(&bars.v_full, nvc * AT_CHUNK);
      for (int c = 0; c < nvc; ++c) tma_load_2d(sv + c * AT_CHUNK, &tm_v, &bars.v_full, dh * dv + c * 64, krow);
    }
  } else if (warp == 1) {
    const bool leader = elect_one();
    const uint64_t dk = smem_desc_sw128(0);
    bool ok = true;
    {
      const uint32_t idesc_s = idesc_bf16_f32(AT_BQ, AT_BK);
      const uint32_t q16 = (smem_u32(sq) & 0x3FFFFu) >> 4, k16 = (smem_u32(sk) & 0x3FFFFu) >> 4;
#pragma unroll
      for (int ks = 0; ks < 16; ++ks) {  // D = 256 in steps of 16: chunk ks/4, 32 bytes per step
        if ((ks & 3) == 0 && ok) {
          ok = __all_sync(0xffffffffu, at_wait(&bars.qk_full[ks >> 2], 0, &bars.abort));
          tc_fence_after();
        }
        const uint32_t off = (ks >> 2) * (AT_CHUNK >> 4) + (ks & 3) * 2;
        if (ok && leader) umma_ss_bf16(t_s, dk | (q16 + off), dk | (k16 + off), idesc_s, ks > 0 ? 1u : 0u);
      }
    }
    if (ok) {
      if (leader) tc_commit(&bars.s_full);
      __syncwarp();
      ok = __all_sync(0xffffffffu, at_wait(&bars.v_full, 0, &bars.abort) && at_wait(&bars.p_full, 0, &bars.abort));
    }
    if (ok) {
      tc_fence_after();
      // O[128 x 256] = P[128 x 128 keys] . V[keys x 256]: B operand N = D (MN-major), K = keys.
      const uint32_t idesc_o = idesc_bf16_f32(AT_BQ, dv) | (1u << 16);
      const uint32_t v_addr = smem_u32(sv);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {  // 16 keys per step: 16 rows x 128 bytes inside every chunk
        const uint64_t bd = smem_desc_sw128_mn(v_addr + ks * 2048, AT_CHUNK);
        if (leader) umma_ts_bf16(t_o, t_p + ks * 8, bd, idesc_o, ks > 0 ? 1u : 0u);
      }
      if (leader) tc_commit(&bars.o_full);
      __syncwarp();
    } else if (lane == 0) {
      bars.abort = 1;
      if (p.status) atomicCAS(p.status, 0, TYBOK_DEV_TIMEOUT_MMA);
    }
    // This warp frees the tensor memory at the end, whatever the other warps decide: it first sees
    // every instruction it issued retire (on the normal path this completes together with o_full).
    if (leader) tc_commit(&bars.mma_done);
    __syncwarp();
    mbar_wait(&bars.mma_done, 0);
  } else {
    // ------------------------------------------------------------ softmax, two threads per row
    const int q = warp & 3;          // tensor-memory lane quadrant of this warp
    const int hf = (warp - 2) >> 2;  // which 64 keys of the block / which 128 output columns
    const int row = q * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const bool live = q * 32 < nvalid;  // warp-uniform: this quadrant holds real query rows
    // Every named barrier below is reached by all eight warps whatever the waits returned.
    bool ok = __all_sync(0xffffffffu, at_wait(&bars.s_full, 0, &bars.abort));
    if (tr && tid == 128) tr[2] = clock64();
    uint32_t v0[32], v1[32];
    float mx = -1e30f;
    if (ok && live) {
      tc_fence_after();
      tmem_ld32(t_s + lane_addr + (hf * 2) * 32, v0);
      tmem_ld32(t_s + lane_addr + (hf * 2 + 1) * 32, v1);
      tc_wait_ld();
      const uint32_t b0 = bars.valid[hf * 2], b1 = bars.valid[hf * 2 + 1];
      // per 32-key chunk: all valid -> no per-element selects; none valid -> nothing to do
      if (b0 == 0xffffffffu) {
#pragma unroll
        for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(v0[e]));
      } else if (b0 != 0u) {
#pragma unroll
        for (int e = 0; e < 32; ++e)
          if ((b0 >> e) & 1u) mx = fmaxf(mx, __uint_as_float(v0[e]));
      }
      if (b1 == 0xffffffffu) {
#pragma unroll
        for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(v1[e]));
      } else if (b1 != 0u) {
#pragma unroll
        for (int e = 0; e < 32; ++e)
          if ((b1 >> e) & 1u) mx = fmaxf(mx, __uint_as_float(v1[e]));
      }
    }
    bars.hmax[hf][row] = mx;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    const float m2 = fmaxf(bars.hmax[0][row], bars.hmax[1][row]) * p.scale_log2e;  // scale > 0
    float sum = 0.f;
    if (ok && live) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint32_t bits = bars.valid[hf * 2 + c];
        uint32_t pk[16];
        if (bits == 0xffffffffu) {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float s0 = __uint_as_float(c == 0 ? v0[e] : v1[e]), s1 = __uint_as_float(c == 0 ? v0[e + 1] : v1[e + 1]);
            const float p0 = exp2f(s0 * p.scale_log2e - m2), p1 = exp2f(s1 * p.scale_log2e - m2);
            sum += p0 + p1;
            const __nv_bfloat162 pp = __floats2bfloat162_rn(p0, p1);
            pk[e >> 1] = *reinterpret_cast<const uint32_t*>(&pp);
          }
        } else if (bits == 0u) {
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = 0u;
        } else {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float s0 = __uint_as_float(c == 0 ? v0[e] : v1[e]), s1 = __uint_as_float(c == 0 ? v0[e + 1] : v1[e + 1]);
            const float p0 = ((bits >> e) & 1u) ? exp2f(s0 * p.scale_log2e - m2) : 0.f;
            const float p1 = ((bits >> (e + 1)) & 1u) ? exp2f(s1 * p.scale_log2e - m2) : 0.f;
            sum += p0 + p1;
            const __nv_bfloat162 pp = __floats2bfloat162_rn(p0, p1);
            pk[e >> 1] = *reinterpret_cast<const uint32_t*>(&pp);
          }
        }
        tmem_st16(t_p + lane_addr + (hf * 2 + c) * 16, pk);
      }
      tc_wait_st();
    }
    tc_fence_before();
    bars.hsum[hf][row] = sum;
    if (hf == 0) bars.row_max[row] = m2;
    __syncwarp();
    if (ok && lane == 0) mbar_arrive(&bars.p_full);
    if (tr && tid == 128) tr[3] = clock64();
    if (PUSH) {
      // The statistics are final here: send them to the merging peers while P.V runs, so that
      // the merge weights are ready before the partial rows arrive.
      if (row < nvalid) {
        if (hf == 0) {
          bars.stat[row].x = m2;
          bars.stat[row].y = sum;
        } else {
          bars.stat[row].z = sum;
        }
      }
      fence_proxy_async();  // the statistics stores, for the bulk copy engine
      asm volatile("bar.sync 1, 256;" ::: "memory");
      cluster_wait_acquire();  // every peer's receive barriers are armed
      if (ok && warp == 2 && lane < p.nsplit && lane != sp) {
        const int rpr = (nvalid + p.nsplit - 1) / p.nsplit;
        const int rs = lane * rpr, ns = min(nvalid, rs + rpr) - rs;
        if (ns > 0)
          bulk_copy_to_peer(dsmem_addr(smem_u32(sv + AT_PUSH_RECV + AT_PUSH_STATS) + sp * rpr * 16, lane), &bars.stat[rs],
                            ns * 16, dsmem_addr(smem_u32(&bars.recv_stat), lane));
      }
    }
    // ---------------------------------------------------------- stage O (un-normalised), fp32
    ok = ok && __all_sync(0xffffffffu, at_wait(&bars.o_full, 0, &bars.abort));
    if (tr && tid == 128) tr[4] = clock64();
    if (ok && live) {
      tc_fence_after();
      // Staging tile over the (no longer needed) Q and K tiles: [row][64 float4], the float4
      // index XORed with (row & 7) so that a warp's 16-byte stores spread over all banks.
      // Only the tile's real query rows are staged.
      float4* stage = reinterpret_cast<float4*>(smem);
      const int q4 = dv / 4;      // float4 per staged row
      const int nch = dv / 64;    // 32-column chunks per thread (this thread's half of the row)
#pragma unroll 1
      for (int c = 0; c < nch; ++c) {
        uint32_t v[32];
        tmem_ld32(t_o + lane_addr + (hf * nch + c) * 32, v);
        tc_wait_ld();
        if (row < nvalid) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            stage[row * q4 + (((hf * nch + c) * 8 + j) ^ (row & 7))] =
                make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                            __uint_as_float(v[4 * j + 3]));
        }
      }
    }
    if (!ok && lane == 0) {
      bars.abort = 1;
      if (p.status) atomicCAS(p.status, 0, TYBOK_DEV_TIMEOUT_EPILOGUE);
    }
    if (PUSH) {
      // Send every peer the staged partial rows it merges: one bulk copy per peer, one lane each.
      fence_proxy_async();  // the staging stores, for the bulk copy engine
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (!bars.abort && warp == 2 && lane < p.nsplit && lane != sp) {
        const int rpr = (nvalid + p.nsplit - 1) / p.nsplit;
        const int rs = lane * rpr, ns = min(nvalid, rs + rpr) - rs;
        if (ns > 0) {
          const uint32_t recv = smem_u32(sv + AT_PUSH_RECV), bar = dsmem_addr(smem_u32(&bars.recv), lane);
          bulk_copy_to_peer(dsmem_addr(recv + sp * rpr * (AT_D / 2 * 4), lane), smem + rs * (AT_D / 2 * 4),
                            ns * (AT_D / 2 * 4), bar);
        }
      }
    } else if (p.nsplit > 1) {
      // Publish this block's rows: statistics by plain stores, the staged O rows by one bulk copy
      // out of shared memory.  Every softmax warp reaches this point, aborted or not.
      fence_proxy_async();  // the staging stores, for the bulk copy engine
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (!bars.abort) {
        if (hf == 0 && row < nvalid)
          reinterpret_cast<float2*>(my_ws + AT_BQ * AT_D * 4)[row] =
              make_float2(bars.row_max[row], bars.hsum[0][row] + bars.hsum[1][row]);
        if (tid == 64) {
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(my_ws), "r"(smem_u32(smem)),
                       "r"(nvalid * dv * 4)
                       : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // written, not merely read out of shared memory
          fence_proxy_async();
        }
      }
    } else {
      bars.row_sum[row] = bars.hsum[0][row] + bars.hsum[1][row];
    }
  }

  // ------------------------------------------------------------ meet: every key block published
  if (tr && tid == 64) tr[5] = clock64();
  tc_fence_before();
  if (PUSH) {
    if (warp < 2) {  // the two service warps only keep the cluster barrier's books
      cluster_wait_acquire();
      cluster_arrive_release();
    }
  } else if (p.nsplit > 1) {
    __syncwarp();
    cluster_sync_all();  // release / acquire at cluster scope: the peers' workspace rows are visible
  } else {
    __syncthreads();
  }

  if (tr && tid == 64) tr[6] = clock64();
  // One merged quad of output columns: bf16 row-major and / or the three e5m2 planes.
  const long long hd = static_cast<long long>(p.H) * AT_D;
  const long long plane = static_cast<long long>(p.B) * p.L * hd;
  auto emit = [&](int r, int c4, const float4& acc) {
    const int t = qt * AT_BQ + r;
    const __nv_bfloat162 o01 = __floats2bfloat162_rn(acc.x, acc.y);
    const __nv_bfloat162 o23 = __floats2bfloat162_rn(acc.z, acc.w);
    const long long off = (static_cast<long long>(b) * p.L + t) * hd + static_cast<long long>(h) * AT_D + dh * dv + c4 * 4;
    if (p.out) {
      uint2 st;
      st.x = *reinterpret_cast<const uint32_t*>(&o01);
      st.y = *reinterpret_cast<const uint32_t*>(&o23);
      *reinterpret_cast<uint2*>(p.out + off) = st;
    }
    if (p.out_planes) {
      const float xs[4] = {__bfloat162float(o01.x) * p.plane_scale, __bfloat162float(o01.y) * p.plane_scale,
                           __bfloat162float(o23.x) * p.plane_scale, __bfloat162float(o23.y) * p.plane_scale};
      uint32_t w1, w2, w3;
      split3_quad(xs, w1, w2, w3);
      uint8_t* dst = p.out_planes + off;
      *reinterpret_cast<uint32_t*>(dst) = w1;
      *reinterpret_cast<uint32_t*>(dst + plane) = w2;
      *reinterpret_cast<uint32_t*>(dst + 2 * plane) = w3;
    }
  };
  // Normalised merge weights of one owned query row from every block's (max, sum).
  auto merge_weights = [&](int et, const float (&w_in)[AT_MAX_SPLITS], const float (&l)[AT_MAX_SPLITS]) {
    float w[AT_MAX_SPLITS];
    float mx = -1e30f;
#pragma unroll
    for (int s = 0; s < AT_MAX_SPLITS; ++s) mx = fmaxf(mx, w_in[s]);
    float denom = 0.f;
#pragma unroll
    for (int s = 0; s < AT_MAX_SPLITS; ++s) {
      w[s] = s < p.nsplit ? exp2f(w_in[s] - mx) : 0.f;  // 0 for a block without valid keys
      denom += w[s] * l[s];
    }
    const float inv = denom > 0.f ? 1.0f / denom : 0.f;
#pragma unroll
    for (int s = 0; s < AT_MAX_SPLITS; ++s) bars.wn[s][et] = w[s] * inv;
  };

  if (PUSH && warp >= 2) {
    const int et = tid - 64;
    constexpr int q4 = AT_D / 2 / 4, rstep = 256 / q4;
    const int c4 = et % q4, rsub = et / q4;
    const int rpr = (nvalid + p.nsplit - 1) / p.nsplit;
    const int r0 = sp * rpr, r1 = min(nvalid, r0 + rpr);
    const float4* stage = reinterpret_cast<const float4*>(smem);
    const float4* recv = reinterpret_cast<const float4*>(sv + AT_PUSH_RECV);
    const float4* rstat = reinterpret_cast<const float4*>(sv + AT_PUSH_RECV + AT_PUSH_STATS);
    bool got = true;
    if (r0 + et < r1) {  // one thread per owned row: its weights, while the partial rows are in flight
      got = at_wait(&bars.recv_stat, 0, &bars.abort);
      float w[AT_MAX_SPLITS], l[AT_MAX_SPLITS];
#pragma unroll
      for (int s = 0; s < AT_MAX_SPLITS; ++s) {
        w[s] = -1e30f;
        l[s] = 0.f;
        if (s < p.nsplit) {
          const float4 st = s == sp ? bars.stat[r0 + et] : rstat[s * rpr + et];
          w[s] = st.x;
          l[s] = st.y + st.z;
        }
      }
      merge_weights(et, w, l);
    }
    if (tr && tid == 64) tr[9] = clock64();
    got = at_wait(&bars.recv, 0, &bars.abort) && got;
    cluster_arrive_release();  // this thread needs nothing more from the peers
    if (tr && tid == 64) tr[6] = clock64();
    if (!got) {
      bars.abort = 1;
      if (p.status) atomicCAS(p.status, 0, TYBOK_DEV_TIMEOUT_EPILOGUE);
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (tr && tid == 64) tr[7] = clock64();
    if (!bars.abort) {
      for (int r = r0 + rsub; r < r1; r += rstep) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const int sw = c4 ^ (r & 7);
#pragma unroll
        for (int s = 0; s < AT_MAX_SPLITS; ++s) {  // block order: bit-reproducible
          if (s < p.nsplit) {
            const float ws = bars.wn[s][r - r0];
            const float4 v = s == sp ? stage[r * q4 + sw] : recv[(s * rpr + r - r0) * q4 + sw];
            acc.x += ws * v.x; acc.y += ws * v.y; acc.z += ws * v.z; acc.w += ws * v.w;
          }
        }
        emit(r, c4, acc);
      }
    }
  }

  if (!PUSH && warp >= 2 && !bars.abort) {
    // Merge: this CTA owns query rows [r0, r1) of the tile; thread = (4 output columns, row phase).
    const int et = tid - 64;
    const int q4 = dv / 4;          // float4 per row: 64, or 32 with split columns
    const int rstep = 256 / q4;     // rows per pass of the 256 merging threads
    const int c4 = et % q4, rsub = et / q4;
    const int rpr = (nvalid + p.nsplit - 1) / p.nsplit;
    const int r0 = sp * rpr, r1 = min(nvalid, r0 + rpr);
    const float4* stage = reinterpret_cast<const float4*>(smem);
    const uint8_t* ws0 = my_ws - static_cast<long long>(sp) * AT_WS_PER_CTA;  // block 0 of this cluster
    // The partial rows come out of L2 (about a microsecond away), so a thread requests a batch of
    // rows -- every key block of each -- before it needs any of them; the first batch is in
    // flight while the merge weights are worked out.
    float4 buf[AT_MERGE_BATCH][AT_MAX_SPLITS];
    auto fetch = [&](int rb) {
#pragma unroll
      for (int j = 0; j < AT_MERGE_BATCH; ++j) {
        const int r = rb + rstep * j;
        if (r < r1) {
          const int idx = r * q4 + (c4 ^ (r & 7));
#pragma unroll
          for (int s = 0; s < AT_MAX_SPLITS; ++s)
            if (s < p.nsplit)
              buf[j][s] = s == sp ? stage[idx]
                                  : __ldcg(reinterpret_cast<const float4*>(ws0 + static_cast<long long>(s) * AT_WS_PER_CTA) + idx);
        }
      }
    };
    int rb = r0 + rsub;
    fetch(rb);
    if (tr && tid == 64) tr[9] = clock64();
    if (r0 + et < r1) {  // one thread per owned row: normalised weight of every key block
      const int r = r0 + et;
      float w[AT_MAX_SPLITS], l[AT_MAX_SPLITS];
      float mx = -1e30f;
#pragma unroll
      for (int s = 0; s < AT_MAX_SPLITS; ++s) {
        w[s] = -1e30f;
        l[s] = 0.f;
        if (s < p.nsplit) {
          if (p.nsplit > 1) {
            const float2 st = __ldcg(reinterpret_cast<const float2*>(ws0 + static_cast<long long>(s) * AT_WS_PER_CTA +
                                                                      AT_BQ * AT_D * 4) + r);
            w[s] = st.x;
            l[s] = st.y;
          } else {
            w[s] = bars.row_max[r];
            l[s] = bars.row_sum[r];
          }
        }
        mx = fmaxf(mx, w[s]);
      }
      if (tr && tid == 64) tr[10] = clock64() + (mx == 12345.f);
      float denom = 0.f;
#pragma unroll
      for (int s = 0; s < AT_MAX_SPLITS; ++s) {
        w[s] = s < p.nsplit ? exp2f(w[s] - mx) : 0.f;  // 0 for a block without valid keys
        denom += w[s] * l[s];
      }
      const float inv = denom > 0.f ? 1.0f / denom : 0.f;
#pragma unroll
      for (int s = 0; s < AT_MAX_SPLITS; ++s) bars.wn[s][et] = w[s] * inv;
      if (tr && tid == 64) tr[11] = clock64() + (inv == 12345.f);
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (tr && tid == 64) tr[7] = clock64();
#pragma unroll 1
    for (; rb < r1; rb += rstep * AT_MERGE_BATCH) {
#pragma unroll
      for (int j = 0; j < AT_MERGE_BATCH; ++j) {
        const int r = rb + rstep * j;
        if (r < r1) {
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int s = 0; s < AT_MAX_SPLITS; ++s) {  // block order: bit-reproducible
            if (s < p.nsplit) {
              const float ws = bars.wn[s][r - r0];
              const float4 v = buf[j][s];
              acc.x += ws * v.x; acc.y += ws * v.y; acc.z += ws * v.z; acc.w += ws * v.w;
            }
          }
          emit(r, c4, acc);
        }
      }
      if (rb + rstep * AT_MERGE_BATCH < r1) fetch(rb + rstep * AT_MERGE_BATCH);
    }
  }

  if (tr && tid == 64) tr[8] = clock64();
  // Pull form: nothing after the meeting point touches a peer's shared memory, CTAs leave on
  // their own.  Push form: a CTA stays until every peer holds the rows it was sent, which is
  // when the copies have finished reading this CTA's shared memory.
  if (PUSH) cluster_wait_acquire();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}


// ------------------------------------------------------------------------------ prefill form
// Long query sequences (more than one query tile): one CTA per (query tile, head, batch) walks
// over the keys in blocks (64 keys at head_dim 256, 128 at head_dim 128) and keeps the running
// output in tensor memory, so nothing is exchanged between CTAs.  Warp 0 streams K and V blocks
// through two-deep rings, warp 1 issues S_j = Q K_j^T one block ahead and O += P_j V_j, warps 2..9
// hold two threads per query row (half of a block's keys each): block maximum,
// P_j = exp2(s * c - m) as bf16 over the S_j columns, row sum.  The reference
// maximum m of a row only moves when the block maximum exceeds it by more than 2^8 (P stays
// below 256, exact enough in bf16 and fp32); then the thread rescales its O row and its sum.
// All eight epilogue warps normalise and write the output at the end.
// Keys per block: 64 at head_dim 256 (two K and two V blocks of 32 KB each beside the Q tile), 128 at
// head_dim 128, where the same shared memory holds blocks twice as long: every block pays one chain of
// tensor-memory round trips and one named barrier whatever its length, and at 64 keys that chain,
// not the special-function unit, set the pace of the DiT self-attention (65 blocks per CTA).
__host__ __device__ constexpr int pf_bk(int d) { return d == 128 ? 128 : 64; }
__host__ __device__ constexpr int pf_kchunk(int d) { return pf_bk(d) * 128; }  // one 64-column chunk of a K or V block
constexpr int PF_MAX_KEYS = 8192;
// Shared memory of the key-loop kernel: the Q tile and two K and two V blocks, D / 64 chunks each.
constexpr int pf_smem(int d) { return (d / 64) * (AT_CHUNK + 4 * pf_kchunk(d)) + 1024; }
constexpr float PF_RESCALE = 8.0f;
// 2^x by the special-function unit alone (results below 2^-126 flush to zero).
__device__ __forceinline__ float pf_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct __align__(8) PrefillBars {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full[2], p_full[2];
  uint64_t o_done;    // one phase per P.V product.  S_j is issued after P.V of block j-2, so a thread that
                      // holds S_j and waits for phase j-1 is never more than one phase behind
  uint64_t all_done;  // the last P.V product has landed
  uint64_t mma_done;  // unwinding: whatever was issued before a failed wait has retired
  uint32_t tmem_base;
  volatile int abort;
  uint32_t valid[PF_MAX_KEYS / 32];
  float hmax[2][2][AT_BQ];  // [block parity][half of the block's keys][row]: maximum of the valid scores
  float hsum[2][AT_BQ];     // [half][row]: sum of that half's probabilities over all blocks
};

// HD = head dimension, 128 or 256.  Either way a CTA takes ALL 512 tensor-memory columns of its SM
// and therefore has the SM's tensor memory to itself.  (At HD = 128 two CTAs of 256 columns each
// would fit, and ran, but chains that alternate this kernel with the CTA-pair GEMM -- whose two CTAs
// allocate 256 columns collectively on two SMs -- then stalled once in some 10^5 launches with one
// GEMM pair waiting for tensor memory on an otherwise idle device.  Whole-SM allocations next to
// the pair GEMM are the combination that has run the pi0.5 prefix 10^6 launches without a stall.)
template <int HD>
__global__ void __launch_bounds__(AT_THREADS, 1)
attention_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                         const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ PrefillBars bars;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int KID = HD == 256 ? 5 : 6;
  if (tid == 0) dbg_stage(p.dbg, KID, 0);
  constexpr int NCH = HD / 64;              // 64-column chunks of a Q, K or V row
  constexpr int PF_BK = pf_bk(HD);          // keys per block
  constexpr int PF_KCHUNK = pf_kchunk(HD);
  constexpr int PF_KV = NCH * PF_KCHUNK;    // one K or V block: PF_BK keys x HD
  constexpr int KW = PF_BK / 64;            // 32-key words per thread and block (two threads per query row)
  constexpr int Q_TILE = NCH * AT_CHUNK;    // 128 query rows x HD
  constexpr int T_COLS = 512;               // tensor memory: S / P at columns 0 and PF_BK, O from column 256
  constexpr int OCH = HD / 64;              // 32-column chunks of O per thread (its half of the row)
  uint8_t* sq = smem;
  uint8_t* sk = smem + Q_TILE;               // two K blocks
  uint8_t* sv = smem + Q_TILE + 2 * PF_KV;   // two V blocks

  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int g = h / (p.H / p.G);
  const int nkb = (p.Lk + PF_BK - 1) / PF_BK;
  const int nvalid = min(AT_BQ, p.L - qt * AT_BQ);

  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    mbar_init(&bars.q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars.k_full[i], 1);
      mbar_init(&bars.k_empty[i], 1);
      mbar_init(&bars.v_full[i], 1);
      mbar_init(&bars.v_empty[i], 1);
      mbar_init(&bars.s_full[i], 1);
      mbar_init(&bars.p_full[i], 8);
    }
    mbar_init(&bars.o_done, 1);
    mbar_init(&bars.all_done, 1);
    mbar_init(&bars.mma_done, 1);
    bars.abort = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars.tmem_base, T_COLS);
    tmem_relinquish();
  }
  if (warp >= 2 && warp < 6) {  // validity bits of every key, 32 per word
    if (p.key_valid && p.pdl) pdl_wait();
    for (int w = warp - 2; w < (PF_BK / 32) * nkb; w += 4) {
      const int j = w * 32 + lane;
      bool ok = j < p.Lk;
      if (ok && p.key_valid) ok = p.key_valid[static_cast<long long>(b) * p.Lk + j] != 0;
      const uint32_t bits = __ballot_sync(0xffffffffu, ok);
      if (lane == 0) bars.valid[w] = bits;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars.tmem_base;
  const uint32_t t_o = tmem + 256;  // S_j (and P_j over it) at columns PF_BK * (j & 1)
  if (tid == 0) dbg_stage(p.dbg, KID, 1);
  long long* tr = p.trace ? p.trace + 16ll * ((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) : nullptr;
  const long long t_start = clock64();
  if (tr && tid == 0) tr[0] = t_start;

  if (warp == 0) {
    if (lane == 0) {
      if (p.pdl) pdl_launch_dependents();
      if (p.pdl) pdl_wait();
      dbg_stage(p.dbg, KID, 2);
      mbar_arrive_expect_tx(&bars.q_full, Q_TILE);
      for (int c = 0; c < NCH; ++c) tma_load_2d(sq + c * AT_CHUNK, &tm_q, &bars.q_full, h * HD + c * 64, b * p.L + qt * AT_BQ);
      for (int j = 0; j < nkb; ++j) {
        const int s = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;  // the ring slot's previous use
        const int krow = (b * p.G + g) * p.Lcap + j * PF_BK;
        if (j >= 2 && !at_wait(&bars.k_empty[s], par, &bars.abort)) break;
        mbar_arrive_expect_tx(&bars.k_full[s], PF_KV);
        for (int c = 0; c < NCH; ++c) tma_load_2d(sk + s * PF_KV + c * PF_KCHUNK, &tm_k, &bars.k_full[s], c * 64, krow);
        if (j >= 2 && !at_wait(&bars.v_empty[s], par, &bars.abort)) break;
        mbar_arrive_expect_tx(&bars.v_full[s], PF_KV);
        for (int c = 0; c < NCH; ++c) tma_load_2d(sv + s * PF_KV + c * PF_KCHUNK, &tm_v, &bars.v_full[s], c * 64, krow);
      }
    }
  } else if (warp == 1) {
    const bool leader = elect_one();
    const uint64_t dk = smem_desc_sw128(0);
    const uint32_t idesc_s = idesc_bf16_f32(AT_BQ, PF_BK);
    const uint32_t idesc_o = idesc_bf16_f32(AT_BQ, HD) | (1u << 16);
    const uint32_t q16 = (smem_u32(sq) & 0x3FFFFu) >> 4;
    bool ok = __all_sync(0xffffffffu, at_wait(&bars.q_full, 0, &bars.abort));
    auto issue_s = [&](int j) {  // S_j = Q K_j^T into columns PF_BK * (j & 1); frees the K slot when done
      const int s = j & 1;
      ok = ok && __all_sync(0xffffffffu, at_wait(&bars.k_full[s], (j >> 1) & 1, &bars.abort));
      if (!ok) return;
      tc_fence_after();
      const uint32_t k16 = (smem_u32(sk + s * PF_KV) & 0x3FFFFu) >> 4;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {  // the head dimension in steps of 16: chunk ks / 4, 32 bytes per step
        const uint32_t qo = (ks >> 2) * (AT_CHUNK >> 4) + (ks & 3) * 2, ko = (ks >> 2) * (PF_KCHUNK >> 4) + (ks & 3) * 2;
        if (leader) umma_ss_bf16(tmem + s * PF_BK, dk | (q16 + qo), dk | (k16 + ko), idesc_s, ks > 0 ? 1u : 0u);
      }
      if (leader) {
        tc_commit(&bars.k_empty[s]);
        tc_commit(&bars.s_full[s]);
      }
      __syncwarp();
    };
    if (ok) issue_s(0);
    if (ok && nkb > 1) issue_s(1);
#pragma unroll 1
    for (int j = 0; j < nkb && ok; ++j) {
      const int s = j & 1;
      const uint32_t par = (j >> 1) & 1;
      ok = __all_sync(0xffffffffu, at_wait(&bars.p_full[s], par, &bars.abort) && at_wait(&bars.v_full[s], par, &bars.abort));
      if (!ok) break;
      tc_fence_after();
      const uint32_t v_addr = smem_u32(sv + s * PF_KV);
#pragma unroll
      for (int ks = 0; ks < PF_BK / 16; ++ks) {  // 16 keys per step: 16 rows x 128 bytes inside every chunk
        const uint64_t bd = smem_desc_sw128_mn(v_addr + ks * 2048, PF_KCHUNK);
        if (leader) umma_ts_bf16(t_o, tmem + s * PF_BK + ks * 8, bd, idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
      }
      if (leader) {
        tc_commit(&bars.v_empty[s]);
        tc_commit(&bars.o_done);
        if (j == nkb - 1) tc_commit(&bars.all_done);
      }
      __syncwarp();
      if (j + 2 < nkb) issue_s(j + 2);  // over P_j, which the product just issued reads first
    }
    // nothing of this CTA's tensor work may be in flight when it gives up its tensor memory
    ok = ok && __all_sync(0xffffffffu, at_wait(&bars.all_done, 0, &bars.abort));
    if (!ok) {
      if (lane == 0) {
        bars.abort = 1;
        if (p.status) atomicCAS(p.status, 0, TYBOK_DEV_TIMEOUT_MMA);
      }
      // a failed wait left the loop early: see what was issued before it retire
      if (leader) tc_commit(&bars.mma_done);
      __syncwarp();
      mbar_wait(&bars.mma_done, 0);
    }
  }
  else {
    // -------------------------------------------------------------- softmax: two threads per query row
    const int q = warp & 3;          // tensor-memory lane quadrant of this warp
    const int hf = (warp - 2) >> 2;  // which half of a block's keys / which half of the output columns
    const int row = q * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const bool live = q * 32 < nvalid;  // warp-uniform: this quadrant holds real query rows
    // All eight warps walk the blocks in step (one named barrier per block), whatever the waits
    // return: after a failed wait `ok` stays false and the abort flag makes every later wait return.
    bool ok = true;
    float m_ref = -1e30f, l = 0.f;
#pragma unroll 1
    for (int j = 0; j < nkb; ++j) {
      const int s = j & 1;
      if (ok && !__all_sync(0xffffffffu, at_wait(&bars.s_full[s], (j >> 1) & 1, &bars.abort))) {
        ok = false;
        bars.abort = 1;
      }
      if (tr && tid == 128 && j < 6) tr[1 + 2 * j] = clock64();
      uint32_t v[KW][32];
      uint32_t bits[KW];
#pragma unroll
      for (int w = 0; w < KW; ++w) bits[w] = bars.valid[(2 * j + hf) * KW + w];
      float mx = -1e30f;
      if (ok && live) {
        tc_fence_after();
#pragma unroll
        for (int w = 0; w < KW; ++w) tmem_ld32(tmem + lane_addr + s * PF_BK + (hf * KW + w) * 32, v[w]);
        tc_wait_ld();
#pragma unroll
        for (int w = 0; w < KW; ++w) {
          if (bits[w] == 0xffffffffu) {
#pragma unroll
            for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(v[w][e]));
          } else if (bits[w] != 0u) {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if ((bits[w] >> e) & 1u) mx = fmaxf(mx, __uint_as_float(v[w][e]));
          }
        }
      }
      bars.hmax[s][hf][row] = mx;
      tc_fence_before();
      asm volatile("bar.sync 1, 256;" ::: "memory");  // both halves of every row have read S_j
      if (ok && live) {
        tc_fence_after();
        const float m_blk = fmaxf(bars.hmax[s][0][row], bars.hmax[s][1][row]) * p.scale_log2e;  // scale > 0
        if (j == 0) {
          m_ref = m_blk;
        } else {
          const bool grow = m_blk > m_ref + PF_RESCALE;
          if (__any_sync(0xffffffffu, grow)) {
            // Rescale this thread's half of the O row (and its sum) to the new reference maximum;
            // rows of the warp that keep theirs multiply by one.  The previous P.V product must
            // have landed (it is at most one phase away, see PrefillBars::o_done).
            if (!__all_sync(0xffffffffu, at_wait(&bars.o_done, (j - 1) & 1, &bars.abort))) {
              ok = false;
              bars.abort = 1;
            } else {
              tc_fence_after();
              const float f = grow ? pf_exp2(m_ref - m_blk) : 1.0f;
#pragma unroll 1
              for (int c = hf * OCH; c < hf * OCH + OCH; ++c) {
                uint32_t o[32];
                tmem_ld32(t_o + lane_addr + c * 32, o);
                tc_wait_ld();
#pragma unroll
                for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
                tmem_st32(t_o + lane_addr + c * 32, o);
              }
              tc_wait_st();
              l *= f;
              if (grow) m_ref = m_blk;
            }
          }
        }
      }
      if (ok && live) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < KW; ++w) {
          uint32_t pk[16];
          if (bits[w] == 0xffffffffu) {
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              const float p0 = pf_exp2(__uint_as_float(v[w][e]) * p.scale_log2e - m_ref);
              const float p1 = pf_exp2(__uint_as_float(v[w][e + 1]) * p.scale_log2e - m_ref);
              sum += p0 + p1;
              const __nv_bfloat162 pp = __floats2bfloat162_rn(p0, p1);
              pk[e >> 1] = *reinterpret_cast<const uint32_t*>(&pp);
            }
          } else if (bits[w] == 0u) {
#pragma unroll
            for (int e = 0; e < 16; ++e) pk[e] = 0u;
          } else {
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              const float p0 = ((bits[w] >> e) & 1u) ? pf_exp2(__uint_as_float(v[w][e]) * p.scale_log2e - m_ref) : 0.f;
              const float p1 = ((bits[w] >> (e + 1)) & 1u) ? pf_exp2(__uint_as_float(v[w][e + 1]) * p.scale_log2e - m_ref) : 0.f;
              sum += p0 + p1;
              const __nv_bfloat162 pp = __floats2bfloat162_rn(p0, p1);
              pk[e >> 1] = *reinterpret_cast<const uint32_t*>(&pp);
            }
          }
          // P_j as bf16 pairs over the start of S_j: 16 columns per 32 keys (every thread of the row
          // has read its scores before the named barrier above)
          tmem_st16(tmem + lane_addr + s * PF_BK + (hf * KW + w) * 16, pk);
        }
        l += sum;
        tc_wait_st();
      }
      tc_fence_before();
      __syncwarp();
      if (ok && lane == 0) mbar_arrive(&bars.p_full[s]);
      if (tr && tid == 128 && j < 6) tr[2 + 2 * j] = clock64();
    }
    bars.hsum[hf][row] = l;
    if (ok && !__all_sync(0xffffffffu, at_wait(&bars.all_done, 0, &bars.abort))) ok = false;
    if (!ok && lane == 0) {
      bars.abort = 1;
      if (p.status) atomicCAS(p.status, 0, TYBOK_DEV_TIMEOUT_EPILOGUE);
    }
    // ------------------------------------------------------------ output
    // Normalised rows go through shared memory (Q, K and V are idle by now): bf16 rows of 512
    // bytes and three plane rows of 256 bytes, each padded by 16 bytes against bank conflicts,
    // then one warp per row, so that global memory sees whole rows.
    if (tr && tid == 128) tr[13] = clock64();
    if (tid == 64) dbg_stage(p.dbg, KID, 3);
    tc_fence_before();
    asm volatile("bar.sync 1, 256;" ::: "memory");
    constexpr int OB = HD * 2 + 16, OP = HD + 16;  // padded row pitches
    uint8_t* so = smem;
    uint8_t* sp = smem + AT_BQ * OB;
    const bool good = !bars.abort;
    if (good && live) {  // warp-uniform: the tensor-memory loads below are warp-wide
      tc_fence_after();
      const float ls = bars.hsum[0][row] + bars.hsum[1][row];
      const float inv = ls > 0.f ? 1.0f / ls : 0.f;
#pragma unroll 1
      for (int c = hf * OCH; c < hf * OCH + OCH; ++c) {
        uint32_t o[32];
        tmem_ld32(t_o + lane_addr + c * 32, o);
        tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; e += 8) {
          uint32_t ob[4], w1[2], w2[2], w3[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const __nv_bfloat162 o01 = __floats2bfloat162_rn(__uint_as_float(o[e + 4 * u]) * inv, __uint_as_float(o[e + 4 * u + 1]) * inv);
            const __nv_bfloat162 o23 = __floats2bfloat162_rn(__uint_as_float(o[e + 4 * u + 2]) * inv, __uint_as_float(o[e + 4 * u + 3]) * inv);
            ob[2 * u] = *reinterpret_cast<const uint32_t*>(&o01);
            ob[2 * u + 1] = *reinterpret_cast<const uint32_t*>(&o23);
            const float xs[4] = {__bfloat162float(o01.x) * p.plane_scale, __bfloat162float(o01.y) * p.plane_scale,
                                 __bfloat162float(o23.x) * p.plane_scale, __bfloat162float(o23.y) * p.plane_scale};
            split3_quad(xs, w1[u], w2[u], w3[u]);
          }
          const int col = c * 32 + e;
          *reinterpret_cast<uint4*>(so + row * OB + col * 2) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
          *reinterpret_cast<uint2*>(sp + row * OP + col) = make_uint2(w1[0], w1[1]);
          *reinterpret_cast<uint2*>(sp + (AT_BQ + row) * OP + col) = make_uint2(w2[0], w2[1]);
          *reinterpret_cast<uint2*>(sp + (2 * AT_BQ + row) * OP + col) = make_uint2(w3[0], w3[1]);
        }
      }
    }
    if (tr && tid == 128) tr[15] = clock64();
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (good) {
      // one warp per row: every lane moves HD / 32 elements of the bf16 row and of every plane
      const long long hd = static_cast<long long>(p.H) * HD;
      const long long plane = static_cast<long long>(p.B) * p.L * hd;
#pragma unroll 2
      for (int r = warp - 2; r < nvalid; r += 8) {
        const long long off = (static_cast<long long>(b) * p.L + qt * AT_BQ + r) * hd + static_cast<long long>(h) * HD;
        if (HD == 256) {
          if (p.out) *reinterpret_cast<uint4*>(p.out + off + lane * 8) = *reinterpret_cast<const uint4*>(so + r * OB + lane * 16);
          if (p.out_planes) {
            uint8_t* dst = p.out_planes + off + lane * 8;
            *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(sp + r * OP + lane * 8);
            *reinterpret_cast<uint2*>(dst + plane) = *reinterpret_cast<const uint2*>(sp + (AT_BQ + r) * OP + lane * 8);
            *reinterpret_cast<uint2*>(dst + 2 * plane) = *reinterpret_cast<const uint2*>(sp + (2 * AT_BQ + r) * OP + lane * 8);
          }
        } else {
          if (p.out) *reinterpret_cast<uint2*>(p.out + off + lane * 4) = *reinterpret_cast<const uint2*>(so + r * OB + lane * 8);
          if (p.out_planes) {
            uint8_t* dst = p.out_planes + off + lane * 4;
            *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(sp + r * OP + lane * 4);
            *reinterpret_cast<uint32_t*>(dst + plane) = *reinterpret_cast<const uint32_t*>(sp + (AT_BQ + r) * OP + lane * 4);
            *reinterpret_cast<uint32_t*>(dst + 2 * plane) = *reinterpret_cast<const uint32_t*>(sp + (2 * AT_BQ + r) * OP + lane * 4);
          }
        }
      }
    }
  }
  if (tr && tid == 128) tr[14] = clock64();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, T_COLS);
  }
  if (tid == 0) dbg_stage(p.dbg, KID, 4);
}

}  // namespace tb

extern "C" {

int tybok_rope_store(const void* qkv, int64_t ldq, const int* pos, const void* cos_table, const void* sin_table,
                     void* q_out, void* k_cache, void* v_cache, int B, int L, int H, int G, int D, int Lcap,
                     int key_off, void* stream) {
  using namespace tb;
  if (!qkv || !pos || !cos_table || !sin_table || !q_out || !k_cache || !v_cache)
    return host::fail(TYBOK_ERR_ARG, "rope_store: null pointer argument");
  if (B <= 0 || L <= 0 || H <= 0 || G <= 0 || D % 16 != 0 || H % G != 0 || key_off < 0 || key_off + L > Lcap)
    return host::fail(TYBOK_ERR_ARG, "rope_store: bad shape (D % 16 == 0, H % G == 0, key_off + L <= Lcap)");
  if (ldq % 8 != 0 || ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                        reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
                        reinterpret_cast<uintptr_t>(cos_table) | reinterpret_cast<uintptr_t>(sin_table)) & 15))
    return host::fail(TYBOK_ERR_ARG, "rope_store: tensors must be 16-byte aligned, ldq % 8 == 0");
  if (int rc = host::require_sm100()) return rc;
  RopeParams p{static_cast<const __nv_bfloat16*>(qkv), ldq, pos, static_cast<const __nv_bfloat16*>(cos_table),
               static_cast<const __nv_bfloat16*>(sin_table), static_cast<__nv_bfloat16*>(q_out),
               static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), B, L, H, G, D, Lcap, key_off,
               host::pdl_enabled() ? 1 : 0};
  const long long total = static_cast<long long>(B) * L * (H + 2 * G) * (D / 16);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(std::min<long long>((total + 255) / 256, 8 * host::sm_count())));
  cfg.blockDim = dim3(256);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl;
  if (cudaLaunchKernelEx(&cfg, rope_store_kernel, p) != cudaSuccess) return host::fail_cuda("launch rope_store_kernel");
  host::count_launch();
  return TYBOK_OK;
}

int tybok_qknorm_rope_store(const void* src, int64_t ld, int q_off, int k_off, int v_off, const void* norm_q_weight,
                            const void* norm_k_weight, float eps, const float* cos_table, const float* sin_table,
                            void* q_out, void* k_cache, void* v_cache, int B, int L, int H, int D, int Lcap, int key_off,
                            void* stream) {
  using namespace tb;
  if (!src || (q_off < 0 && k_off < 0)) return host::fail(TYBOK_ERR_ARG, "qknorm_rope_store: nothing to do (no q and no k)");
  if ((q_off >= 0 && (!q_out || !norm_q_weight)) || (k_off >= 0 && (!k_cache || !norm_k_weight)) || (v_off >= 0 && !v_cache))
    return host::fail(TYBOK_ERR_ARG, "qknorm_rope_store: null pointer for a requested output");
  if ((cos_table == nullptr) != (sin_table == nullptr)) return host::fail(TYBOK_ERR_ARG, "qknorm_rope_store: cos and sin come together");
  if (B <= 0 || L <= 0 || H <= 0 || D <= 0 || D % 8 != 0 || H * D > 4096 || key_off < 0 ||
      ((k_off >= 0 || v_off >= 0) && key_off + L > Lcap))
    return host::fail(TYBOK_ERR_ARG, "qknorm_rope_store: bad shape (D % 8 == 0, H*D <= 4096, key_off + L <= Lcap)");
  if (ld % 8 != 0 || (q_off >= 0 && q_off % 8) || (k_off >= 0 && k_off % 8) || (v_off >= 0 && v_off % 8))
    return host::fail(TYBOK_ERR_ARG, "qknorm_rope_store: row stride and column offsets must be multiples of 8");
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_cache) |
       reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(norm_q_weight) |
       reinterpret_cast<uintptr_t>(norm_k_weight) | reinterpret_cast<uintptr_t>(cos_table) |
       reinterpret_cast<uintptr_t>(sin_table)) & 15)
    return host::fail(TYBOK_ERR_ARG, "qknorm_rope_store: tensors must be 16-byte aligned");
  if (int rc = host::require_sm100()) return rc;
  QkNormParams p{};
  p.src = static_cast<const __nv_bfloat16*>(src); p.ld = ld; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off;
  p.wq = static_cast<const __nv_bfloat16*>(norm_q_weight); p.wk = static_cast<const __nv_bfloat16*>(norm_k_weight);
  p.cos = cos_table; p.sin = sin_table; p.q_out = static_cast<__nv_bfloat16*>(q_out);
  p.kcache = static_cast<__nv_bfloat16*>(k_cache); p.vcache = static_cast<__nv_bfloat16*>(v_cache);
  p.M = B * L; p.L = L; p.H = H; p.D = D; p.Lcap = Lcap; p.key_off = key_off; p.eps = eps;
  p.pdl = host::pdl_enabled() ? 1 : 0;
  p.dbg = host::counter_buffer();
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(p.M));
  cfg.blockDim = dim3(static_cast<unsigned>(((H * D / 8) + 31) / 32 * 32));
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl;
  if (cudaLaunchKernelEx(&cfg, qknorm_rope_store_kernel, p) != cudaSuccess) return host::fail_cuda("launch qknorm_rope_store_kernel");
  host::count_launch();
  return TYBOK_OK;
}

size_t tybok_attention_workspace_bytes(int B, int L, int H, int Lk) {
  using namespace tb;
  if (B <= 0 || L <= 0 || H <= 0 || Lk <= AT_BK) return 0;  // a single key block merges inside its CTA
  if (L > AT_BQ && Lk <= PF_MAX_KEYS) return 0;             // the key-loop form exchanges nothing
  const size_t nsplit = (static_cast<size_t>(Lk) + AT_BK - 1) / AT_BK, n_qt = (static_cast<size_t>(L) + AT_BQ - 1) / AT_BQ;
  return 2 * nsplit * n_qt * H * B * AT_WS_PER_CTA;  // room for the split-column form of small grids
}

int tybok_attention(const void* q, const void* k_cache, const void* v_cache, const void* key_valid, void* out,
                    void* out_planes, int out_shift, int B, int L, int H, int G, int D, int Lk, int Lcap, float scale,
                    void* workspace, size_t workspace_bytes, int* status_word, void* stream) {
  using namespace tb;
  if (!q || !k_cache || !v_cache || (!out && !out_planes)) return host::fail(TYBOK_ERR_ARG, "attention: null pointer argument");
  if (D != AT_D && D != 128) return host::fail(TYBOK_ERR_ARG, "attention: head_dim must be 128 or 256");
  if (B <= 0 || L <= 0 || H <= 0 || G <= 0 || H % G != 0 || Lk <= 0 || Lk > Lcap)
    return host::fail(TYBOK_ERR_ARG, "attention: bad shape (H % G == 0, 0 < Lk <= Lcap)");
  const int nsplit = (Lk + AT_BK - 1) / AT_BK;
  // several query tiles, or head_dim 128: the key-loop form
  const bool prefill = (L > AT_BQ || D == 128) && Lk <= PF_MAX_KEYS;
  if (D == 128 && !prefill) return host::fail(TYBOK_ERR_ARG, "attention: at most 8192 keys at head_dim 128");
  if (!prefill && nsplit > AT_MAX_SPLITS)
    return host::fail(TYBOK_ERR_ARG, "attention: at most 1024 keys (8 blocks of 128 per cluster) for up to 128 queries, "
                                     "8192 keys beyond");
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
       reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(out_planes)) & 15)
    return host::fail(TYBOK_ERR_ARG, "attention: tensors must be 16-byte aligned");
  if (out_shift < -60 || out_shift > 60) return host::fail(TYBOK_ERR_ARG, "attention: exponent shift out of range");
  const size_t need = prefill ? 0 : tybok_attention_workspace_bytes(B, L, H, Lk);
  if (need && (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15)))
    return host::fail(TYBOK_ERR_WORKSPACE, "attention: workspace must hold tybok_attention_workspace_bytes(), 16-byte aligned");
  if (int rc = host::require_sm100()) return rc;

  CUtensorMap tm_q, tm_k, tm_v;
  const uint64_t hd = static_cast<uint64_t>(H) * D;
  const int q_rows = (L <= 64 && !prefill) ? 64 : AT_BQ;  // short suffixes: half the query tile is enough
  if (int rc = host::tensor_map_2d(&tm_q, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, hd, static_cast<uint64_t>(B) * L, hd * 2, 64, q_rows))
    return rc;
  const uint64_t krows = static_cast<uint64_t>(B) * G * Lcap;
  const int kbox = prefill ? pf_bk(D) : AT_BK;
  if (int rc = host::tensor_map_2d(&tm_k, k_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, D, krows, D * 2, 64, kbox)) return rc;
  if (int rc = host::tensor_map_2d(&tm_v, v_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, D, krows, D * 2, 64, kbox)) return rc;

  AttnParams p{};
  p.B = B; p.L = L; p.H = H; p.G = G; p.Lk = Lk; p.Lcap = Lcap; p.nsplit = nsplit;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.key_valid = static_cast<const uint8_t*>(key_valid);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_planes = static_cast<uint8_t*>(out_planes);
  p.plane_scale = ldexpf(1.0f, out_shift);
  p.status = status_word;
  p.pdl = host::pdl_enabled() ? 1 : 0;
  p.ws = static_cast<uint8_t*>(workspace);
  p.q_rows = q_rows;
  const int n_qt = (L + AT_BQ - 1) / AT_BQ;
  p.dsplit = (nsplit > 1 && 2 * nsplit * H * n_qt * B <= host::sm_count()) ? 2 : 1;
  p.trace = host::trace_buffer();
  p.dbg = host::counter_buffer();
  const int rows_per_rank = (std::min(L, AT_BQ) + nsplit - 1) / nsplit;
  const bool push = p.dsplit == 2 && n_qt == 1 && nsplit * rows_per_rank <= AT_PUSH_MAX_ROWS;

  static bool attr_set[64] = {};
  const int dev = host::current_device();
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(attention_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(attention_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(attention_prefill_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, pf_smem(256)) != cudaSuccess ||
        cudaFuncSetAttribute(attention_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, pf_smem(128)) != cudaSuccess)
      return host::fail_cuda("cudaFuncSetAttribute(attention_kernel)");
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = prefill ? dim3(n_qt, H, B) : dim3(nsplit, H * n_qt * p.dsplit, B);
  cfg.blockDim = dim3(AT_THREADS);
  cfg.dynamicSmemBytes = prefill ? pf_smem(D) : AT_SMEM;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (p.pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (nsplit > 1 && !prefill) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = nsplit;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  if (cudaLaunchKernelEx(&cfg, prefill ? (D == 128 ? attention_prefill_kernel<128> : attention_prefill_kernel<256>)
                                       : push ? attention_kernel<true> : attention_kernel<false>,
                         tm_q, tm_k, tm_v, p) != cudaSuccess)
    return host::fail_cuda("launch attention_kernel");
  host::count_launch();
  return TYBOK_OK;
}

}  // extern "C"
