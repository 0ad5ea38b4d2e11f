/* tybok_b200 -- C ABI of the B200-native fp8 hot path.
 *
 * Every entry point takes plain pointers and sizes (device pointers unless said otherwise),
 * launches on the CUDA stream it is given (a cudaStream_t passed as void*), allocates
 * nothing, and returns a status code: 0 on success, a TYBOK_ERR_* value otherwise, with a
 * message retrievable through tybok_last_error().  Buffers are caller-owned; weights are
 * referenced in place.  Nothing here falls back to a CPU or library path.
 *
 * The interface replaces, for the fp8 FFN/attention path, what the reference binds through
 * its per-kernel extension modules: raw int64 pointers + stream + caller-owned scratch
 * (tybok/policies/fastwam/kernels/adit_fused_bindings.cpp:21-30,121-127,163-206), where a
 * failure is an exception rather than a process exit (kernels/coop_grid.h:20-27).
 */
#ifndef TYBOK_B200_H
#define TYBOK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TYBOK_OK 0
#define TYBOK_ERR_ARG 1       /* bad shape, stride or alignment; nothing was launched */
#define TYBOK_ERR_CUDA 2      /* a CUDA runtime/driver call failed */
#define TYBOK_ERR_WORKSPACE 3 /* workspace missing or too small */
#define TYBOK_ERR_ARCH 4      /* the current device is not sm_100 */

/* Epilogues of the W8A16 linear. */
#define TYBOK_EPI_NONE 0     /* y = bf16(acc*scale + bias) */
#define TYBOK_EPI_GELU 1     /* y = bf16(gelu_tanh(bf16(acc*scale + bias))) */
#define TYBOK_EPI_RESIDUAL 2 /* y = bf16(res + bf16(bf16(acc*scale + bias) * bf16(gate))) ; gate optional */

/* Device-side status word values (written by a kernel whose bounded wait ran out). */
#define TYBOK_DEV_OK 0
#define TYBOK_DEV_TIMEOUT_PRODUCER 101
#define TYBOK_DEV_TIMEOUT_MMA 102
#define TYBOK_DEV_TIMEOUT_CONVERT 103
#define TYBOK_DEV_TIMEOUT_EPILOGUE 104

int tybok_version(void);
/* Host pointer to a thread-local, NUL-terminated description of the last failure. */
const char* tybok_last_error(void);
/* Number of kernels this library has launched in this process (all threads, all streams). */
long long tybok_launch_count(void);

/* ---- activation planes -------------------------------------------------------------------
 * The GEMMs consume activations as three e5m2 byte planes [3][M][K] whose sum is
 * x * 2^x_shift; for bf16 x the sum is exact whenever |x * 2^x_shift| lies in [2^-7, 57344]
 * (below: absolute error <= 2^-17 + 2^-25; above: the terms saturate).  Kernels of this library that
 * produce activations can write the planes directly; tybok_split3 converts a bf16 tensor. */
#define TYBOK_DEFAULT_X_SHIFT 4
int tybok_split3(const void* x, int64_t ldx, void* planes, int M, int K, int x_shift, void* stream);

/* Bytes of scratch tybok_w8a16_linear / tybok_w8a16_geglu need: the activation planes, 3*M*K. */
size_t tybok_w8a16_workspace_bytes(int M, int N, int K, int dual);

/* W8A16 linear: y[M,N] = epilogue(x[M,K] . (W8[N,K] * scale[N])^T + bias[N]).
 *   x        bf16, row stride ldx elements (ldx % 8 == 0, pointer 16-byte aligned)
 *   w8       e4m3 bytes, contiguous [N,K] (K % 16 == 0, N % 4 == 0, pointer 16-byte aligned)
 *   scale    fp32 [N] (16-byte aligned); bias bf16 [N] or NULL
 *   y        bf16, row stride ldy (ldy % 4 == 0, pointer 8-byte aligned)
 *   epilogue TYBOK_EPI_*; residual bf16 [M,N] stride ldres (EPI_RESIDUAL only)
 *   gate     NULL, or per-row-group gate [ceil(M/rows_per_gate), N] with row stride ldgate:
 *            fp32 when gate_is_bf16 == 0 (rounded to bf16 before use), bf16 otherwise
 *   token_tile, splits  0 = choose automatically; otherwise force the token tile
 *            (multiple of 16, <= 256) / the split-K factor (<= 8, one cluster per output tile)
 *   workspace  >= tybok_w8a16_workspace_bytes(...) bytes, 16-byte aligned
 *   status_word  optional device int; set non-zero if a bounded device wait ran out
 * Two launches: tybok_split3 into the workspace, then tybok_w8x3_linear.
 * Replaces the reference's dequant-then-F.linear path
 * (tybok/policies/fastwam/models/policy.py:48-58,127-129) and its W8 GEMM body
 * (tybok/policies/fastwam/kernels/vdit_gemm_core.cu:68, epilogues EPI/RESID). */
int tybok_w8a16_linear(const void* x, const void* w8, const float* scale, const void* bias, void* y, int M, int N,
                       int K, int64_t ldx, int64_t ldy, int epilogue, const void* residual, int64_t ldres,
                       const void* gate, int64_t ldgate, int rows_per_gate, int gate_is_bf16, int token_tile,
                       int splits, void* workspace, size_t workspace_bytes, int* status_word, void* stream);

/* Gated FFN front half: h[M,I] = bf16(bf16(gelu_tanh(g)) * u) with g = bf16(x.Wg^T*sg),
 * u = bf16(x.Wu^T*su); both weight matrices are e4m3 [I,K].  Replaces gate_proj / up_proj /
 * GELU-tanh / multiply of GemmaMLP.forward (tybok/policies/pi05/models/layers.py:87-95) and
 * the reference's fused norm+gate/up kernel
 * (tybok/policies/pi05/models/triton_expert_mlp_fp8.py:54-151) without its activation quantisation. */
int tybok_w8a16_geglu(const void* x, const void* w8_gate, const float* scale_gate, const void* w8_up,
                      const float* scale_up, void* h, int M, int I, int K, int64_t ldx, int64_t ldh, int token_tile,
                      int splits, void* workspace, size_t workspace_bytes, int* status_word, void* stream);

/* tybok_w8a16_linear for callers that cannot allocate device memory and so cannot supply a
 * workspace (a plugin inside a process whose GPU memory pool belongs to another runtime, a
 * control loop that bans allocator calls once it is running, a binding without a device
 * allocator).  It has no counterpart in the reference.  The activation planes live in a fixed
 * 1.5 MiB device array inside the library (TYBOK_STATIC_PLANES_BYTES; held by every GPU that
 * loads the library until exit), so 3*M*K must not exceed that size -- e.g. M = 128 tokens at
 * K = 4096 -- and larger problems are refused with TYBOK_ERR_WORKSPACE.  It calls no
 * cudaMalloc/cudaFree and no allocating library routine.  The first call on each device looks
 * the array's address up (cudaGetSymbolAddress); make that first call before any stream
 * capture.  All calls share the one array, which keeps whatever the previous call left in it
 * (nothing needs clearing: each call overwrites every byte it later reads); two calls that can
 * overlap on the GPU (different streams, or graph branches) race on it -- serialise them.
 * Arguments as tybok_w8a16_linear, minus the workspace, token_tile and splits: the token tile and
 * the split-K factor are always chosen automatically (as token_tile = splits = 0 there).  A call
 * that is refused (bad argument, too large) launches nothing and leaves the array untouched. */
#define TYBOK_STATIC_PLANES_BYTES (3u * 128u * 4096u)
int tybok_w8a16_linear_noalloc(const void* x, const void* w8, const float* scale, const void* bias, void* y, int M,
                               int N, int K, int64_t ldx, int64_t ldy, int epilogue, const void* residual,
                               int64_t ldres, const void* gate, int64_t ldgate, int rows_per_gate, int gate_is_bf16,
                               int* status_word, void* stream);

/* The same two operations on activation planes (one launch each).  Either output may be NULL:
 *   y / h        bf16 result, row stride ldy / ldh
 *   y_planes / h_planes  [3][M][N] planes of result * 2^out_shift, ready for the next GEMM
 * These are what the fused layer chains call: a producer kernel writes planes, so the FFN
 * intermediate reaches the down projection without a bf16 round trip
 * (the role of P3 "requant" in tybok/policies/fastwam/kernels/adit_ffn.cu:65-432). */
int tybok_w8x3_linear(const void* x_planes, int x_shift, const void* w8, const float* scale, const void* bias, void* y,
                      int64_t ldy, void* y_planes, int out_shift, int M, int N, int K, int epilogue,
                      const void* residual, int64_t ldres, const void* gate, int64_t ldgate, int rows_per_gate,
                      int gate_is_bf16, int token_tile, int splits, int* status_word, void* stream);
int tybok_w8x3_geglu(const void* x_planes, int x_shift, const void* w8_gate, const float* scale_gate, const void* w8_up,
                     const float* scale_up, void* h, int64_t ldh, void* h_planes, int out_shift, int M, int I, int K,
                     int token_tile, int splits, int* status_word, void* stream);

/* ---- two-plane activations ---------------------------------------------------------------
 * A producer that sees a whole activation row (the norm kernels) can hand the GEMM two e4m3 planes
 * [2][M][K] of x * 2^k(row) plus row_scale[M] = 2^-k(row), k chosen so that the row's largest
 * magnitude lies in (224, 448]: exact for every element within 2^-10.8 of its row maximum (4e-6 of
 * the maximum below that), a third less tensor work and operand traffic than three e5m2 planes and
 * token tiles up to 128.  tybok_norm_planes2 produces the form for the four norms of this library:
 *   TYBOK_NORM_RMS          a = fp32 weight [W]                       (tybok_rmsnorm, weight form)
 *   TYBOK_NORM_ADARMS       a = fp32 mod [groups, ldmod], rows_per_group (tybok_rmsnorm, mod form)
 *   TYBOK_NORM_LN_MODULATE  a = bf16 shift [W], b = bf16 scale [W]    (tybok_layernorm_modulate)
 *   TYBOK_NORM_LN_AFFINE    a = bf16 weight [W], b = bf16 bias [W]    (tybok_layernorm_affine)
 * (W a multiple of 8, at most 4096, as for the norms themselves; x bf16 with row stride ldx).
 * tybok_w8x2_gemm is tybok_w8x3_linear on that form (epilogue TYBOK_EPI_* or
 * TYBOK_EPI_GEGLU_PACKED: N = 2*I packed gate/up rows in, I columns out, as
 * tybok_w8x3_geglu_packed); tybok_w8x2_qkv_rope is tybok_w8x3_qkv_rope on it.  Outputs are as in
 * the three-plane entry points (bf16 and / or three e5m2 planes for the next GEMM). */
#define TYBOK_NORM_RMS 0
#define TYBOK_NORM_ADARMS 1
#define TYBOK_NORM_LN_MODULATE 2
#define TYBOK_NORM_LN_AFFINE 3
#define TYBOK_EPI_GEGLU_PACKED 4
int tybok_norm_planes2(const void* x, int64_t ldx, int mode, const void* a, const void* b, int64_t ldmod, int rows_per_group,
                       int M, int W, float eps, void* y_planes2, float* row_scale, void* stream);
int tybok_w8x2_gemm(const void* x_planes2, const float* row_scale, const void* w8, const float* scale, const void* bias,
                    void* y, int64_t ldy, void* y_planes, int out_shift, int M, int N, int K, int epilogue,
                    const void* residual, int64_t ldres, const void* gate, int64_t ldgate, int rows_per_gate,
                    int gate_is_bf16, int token_tile, int splits, int* status_word, void* stream);
int tybok_w8x2_qkv_rope(const void* x_planes2, const float* row_scale, const void* w8_paired, const float* scale_paired,
                        const int* pos, const void* cos_table, const void* sin_table, void* q_out, void* k_cache,
                        void* v_cache, int B, int L, int H, int G, int D, int Lcap, int key_off, int K, int token_tile,
                        int splits, int* status_word, void* stream);

/* RMS normalisation feeding a W8 GEMM (fp32 statistics, one warp per row).
 *   weight != NULL: plain Gemma norm    y = bf16(x * rsqrt(mean(x^2)+eps) * (1 + weight))
 *   mod    != NULL: AdaRMS norm         y = bf16(x * rsqrt(mean(x^2)+eps) * (1 + scale) + shift),
 *                   scale = mod[g, 0:W], shift = mod[g, W:2W], g = row / rows_per_group
 *                   (mod is the precomputed dense(cond) output, fp32, row stride ldmod)
 * Outputs: y (bf16, may be NULL) and/or y_planes ([3][M][W] planes of y * 2^out_shift).
 * Replaces GemmaRMSNorm.forward (tybok/policies/pi05/models/layers.py:34-84) and the norm
 * prologues of the reference's fused kernels (triton_expert_mlp.py:29-111). */
int tybok_rmsnorm(const void* x, int64_t ldx, const float* weight, const float* mod, int64_t ldmod,
                  int rows_per_group, int M, int W, float eps, void* y, int64_t ldy, void* y_planes,
                  int out_shift, void* stream);

/* LayerNorm (no affine, fp32 statistics) followed by the DiT modulation x * (1 + scale) + shift
 * with bf16 shift/scale [W] broadcast over rows and every step rounded to bf16, as
 * modulate(apply_norm2(x), shift, scale) of tybok/policies/fastwam/models/dit_block.py:67-69,
 * 392-397 and wan_base.py:131-148.  Outputs as tybok_rmsnorm. */
int tybok_layernorm_modulate(const void* x, int64_t ldx, const void* shift, const void* scale, int M, int W, float eps,
                             void* y, int64_t ldy, void* y_planes, int out_shift, void* stream);

/* Per-step tail of the action-expert loop, one launch: final AdaRMS norm (scale/shift from
 * mod[g, 0:2W]) -> fp32 out-projection [A=32, W] -> x_t += dt * v (fp32, in place) -> next
 * step's suffix embedding h = bf16(W_in . x_t + b_in) with W_in fp32 [W, 32].  x == NULL skips
 * everything but the embedding (first step); h == NULL skips the embedding (last step).
 * Replaces expert.norm + action_out_proj + the Euler update + action_in_proj of
 * tybok/policies/pi05/models/flow_matching.py:193-254,464-502,545-556 and its fused
 * final-norm/out-projection kernel (flow_matching.py:41-150). */
int tybok_action_tail(const void* x, int64_t ldx, const float* mod, int64_t ldmod, int rows_per_group, float eps,
                      const float* w_out, const float* b_out, float* x_t, float dt, const float* w_in,
                      const float* b_in, void* h, int M, int W, int A, void* stream);

/* Residual add + affine LayerNorm of the SigLIP tower in one kernel (all tensors bf16, rows of W
 * contiguous): x_out = x + y (bf16 add; y NULL: x_out = x, nothing stored), h = LayerNorm(x_out)
 * * weight + bias with fp32 statistics.  x_out may alias x.  Replaces the residual adds and
 * nn.LayerNorm calls of tybok/policies/pi05/models/vision.py (encoder layer forward). */
int tybok_add_layernorm(const void* x, const void* y, const void* weight, const void* bias, int M, int W, float eps,
                        void* x_out, void* h, void* stream);

/* The same with the residual stream kept in fp32: x and x_out fp32, y / weight / bias / h bf16
 * (W % 8 == 0, W <= 2048).  A bf16 tower run this way never rounds its stream to bf16. */
int tybok_add_layernorm_mixed(const float* x, const void* y, const void* weight, const void* bias, int M, int W, float eps,
                              float* x_out, void* h, void* stream);
/* The mixed form with y / weight / bias / h in fp16 instead of bf16, for a tower whose GEMMs and attention
 * run on fp16 operands (11 significant bits, as TF32, at the speed of bf16). */
int tybok_add_layernorm_mixed_f16(const float* x, const void* y, const void* weight, const void* bias, int M, int W,
                                  float eps, float* x_out, void* h, void* stream);
/* The same in fp32 (all six tensors fp32; W % 4 == 0, W <= 2048), for a tower run in fp32 / TF32. */
int tybok_add_layernorm_f32(const float* x, const float* y, const float* weight, const float* bias, int M, int W,
                            float eps, float* x_out, float* h, void* stream);

/* LayerNorm with affine weight / bias (bf16 [W]) and fp32 statistics, one rounding at the end:
 * y = bf16(LN(x) * weight + bias), as apply_norm3 of a DiT block
 * (tybok/policies/fastwam/models/dit_block.py:236-237, wan_base.py:141-148).  Outputs as tybok_rmsnorm. */
int tybok_layernorm_affine(const void* x, int64_t ldx, const void* weight, const void* bias, int M, int W, float eps,
                           void* y, int64_t ldy, void* y_planes, int out_shift, void* stream);

/* qk-norm + rotary embedding + KV store of a DiT attention (one launch, one CTA per token row).
 * A source row (bf16, row stride ld) holds q at column q_off, k at k_off, v at v_off, each H*D wide;
 * a negative offset means "absent".  q and k are RMS-normalised over all H*D channels of the row
 * (fp32 statistics, bf16(x * rstd) * bf16 weight -> bf16), then rotated pair-wise by the per-token
 * table cos/sin fp32 [L, D/2] ((x[2i], x[2i+1]) times (cos + i sin), fp32, rounded to bf16; NULL
 * tables = no rotation); q goes to q_out [B*L, H*D], k and the untouched v head-major into the
 * caches [B, H, Lcap, D] at key offset key_off.  H*D <= 4096, D % 8 == 0.
 * Replaces norm_q / norm_k / apply_dense_rope and the K/V concatenation of
 * tybok/policies/fastwam/models/dit_block.py:246-273,255-266 and wan_base.py:97-128 (the reference's fused
 * form: phases P2 of tybok/policies/fastwam/kernels/adit_attn_self.cu:87-783 and adit_attn_cross.cu:77-813). */
int tybok_qknorm_rope_store(const void* src, int64_t ld, int q_off, int k_off, int v_off, const void* norm_q_weight,
                            const void* norm_k_weight, float eps, const float* cos_table, const float* sin_table,
                            void* q_out, void* k_cache, void* v_cache, int B, int L, int H, int D, int Lcap, int key_off,
                            void* stream);

/* RoPE + KV store.  qkv is the packed projection output [B*L, (H+2G)*D] (row stride ldq); q and
 * k are rotated (rotate-half form, bf16 cos/sin tables [max_pos, D], bf16 arithmetic with the
 * reference's rounding points) at positions pos[B*L]; q goes to q_out [B*L, H*D], k and v to the
 * caches [B, G, Lcap, D] at key offset key_off.  Replaces apply_rotary_pos_emb + the K/V
 * concatenation of tybok/policies/pi05/models/layers.py:145-164 and rope.py:67-75. */
int tybok_rope_store(const void* qkv, int64_t ldq, const int* pos, const void* cos_table, const void* sin_table,
                     void* q_out, void* k_cache, void* v_cache, int B, int L, int H, int G, int D, int Lcap,
                     int key_off, void* stream);

/* The packed q/k/v projection with tybok_rope_store as its epilogue: q_out and the caches are
 * written straight from the accumulator, no [B*L, (H+2G)*D] intermediate.  w8_paired is the
 * packed qkv weight [(H+2G)*D, K] with the rows of every head slot reordered so that each block
 * of 128 rows holds dimensions 64t..64t+63 followed by their rotate-half partners D/2+64t..
 * (scale_paired likewise); D % 128 == 0.  Same role as the interleaved q/k rows of the
 * reference's fused qkv+RoPE kernel (tybok/policies/pi05/models/triton_expert_fused_qkv_rope_attn.py:103-251). */
int tybok_w8x3_qkv_rope(const void* x_planes, int x_shift, const void* w8_paired, const float* scale_paired,
                        const int* pos, const void* cos_table, const void* sin_table, void* q_out, void* k_cache,
                        void* v_cache, int B, int L, int H, int G, int D, int Lcap, int key_off, int K, int token_tile,
                        int splits, int* status_word, void* stream);

/* GQA/MQA attention of L query tokens per batch element over the first Lk keys of the caches
 * (head_dim 256: Lk <= 1024 for L <= 128, Lk <= 8192 for longer query sequences; head_dim 128: any L,
 * Lk <= 8192):
 * softmax(q k^T * scale + mask) v with fp32 softmax, bf16 P.
 *   q          [B*L, H*D] bf16 (already rotated);  k_cache / v_cache  [B, G, Lcap, D] bf16, finite
 *   key_valid  NULL or uint8 [B, Lk]: 0 masks a key for every query of that batch element
 *   out        bf16 [B*L, H*D] and/or out_planes [3][B*L][H*D] planes of out * 2^out_shift
 *   workspace  >= tybok_attention_workspace_bytes(B, L, H, Lk) bytes, 16-byte aligned (0 bytes, and
 *              NULL allowed, when Lk <= 128 or L > 128): where the key blocks of a query tile are
 *              spread over a cluster and the partial outputs do not fit the exchange through
 *              shared memory, they pass through it (L2) and merge in block order.  L > 128, and every
 *              head_dim 128 call, runs one CTA per query tile and head over all keys and exchanges nothing.
 * Replaces GemmaAttention._forward_eager (tybok/policies/pi05/models/layers.py:166-191) and the
 * split-K flash kernels of tybok/policies/pi05/models/triton_expert_fused_qkv_rope_attn.py:322-433. */
int tybok_attention(const void* q, const void* k_cache, const void* v_cache, const void* key_valid, void* out,
                    void* out_planes, int out_shift, int B, int L, int H, int G, int D, int Lk, int Lcap, float scale,
                    void* workspace, size_t workspace_bytes, int* status_word, void* stream);
size_t tybok_attention_workspace_bytes(int B, int L, int H, int Lk);

/* tybok_w8x3_geglu on ONE packed weight matrix [2*I, K]: every block of 128 rows holds the 64
 * gate rows of channels 64j..64j+63 followed by their 64 up rows (scale_packed [2*I] likewise),
 * so a CTA streams a single weight tile per K block and its accumulator holds gate and up of
 * the same channels (the role of the interleaved q/k rows in the reference's fused kernels,
 * tybok/policies/pi05/models/triton_expert_fused_qkv_rope_attn.py:103-251).  I % 64 == 0. */
int tybok_w8x3_geglu_packed(const void* x_planes, int x_shift, const void* w8_packed, const float* scale_packed, void* h,
                            int64_t ldh, void* h_planes, int out_shift, int M, int I, int K, int token_tile, int splits,
                            int* status_word, void* stream);

/* AdaRMS norm folded into the GEMMs on either side of it (the action expert below 128 tokens, where
 * a norm kernel between two latency-bound GEMMs costs as much as either of them):
 *   y = W (x r (1 + scale) + shift) = r * W (x (1 + scale)) + W shift,   r = rsqrt(mean(x^2) + eps).
 * tybok_w8x3_residual_next_adarms is tybok_w8x3_linear with the gated residual epilogue
 * (x_new = residual + gate * (W8 a), gate fp32 [N], one group) that also writes the next norm's
 * input in consumable form: u_planes [3][M][N] = planes of bf16(x_new * (1 + next_scale)) * 2^u_shift
 * and ss_part [N / 128][M] = per channel tile, the row sums of squares of the bf16 x_new (N % 128 == 0).
 * tybok_w8x3_qkv_rope_adarms / tybok_w8x3_geglu_packed_adarms are tybok_w8x3_qkv_rope /
 * tybok_w8x3_geglu_packed on those planes: every accumulator row is multiplied by
 * rsqrt(sum_t ss_part[t][m] / K + eps) and bias_rows [weight rows] fp32 = W shift (dequantised weight
 * times the norm's shift row, in the order of the packed / paired weight rows) is added before the
 * first bf16 rounding.  Against the norm kernel followed by the plain GEMM the only difference is
 * the rounding point (x (1 + scale) instead of the normalised value is rounded to bf16).  Same role
 * as the norm prologues of the reference's fused expert kernels
 * (tybok/policies/pi05/models/triton_expert_fused_qkv_rope_attn.py:103-251); math of
 * GemmaRMSNorm.forward with cond (tybok/policies/pi05/models/layers.py:34-84). */
int tybok_w8x3_residual_next_adarms(const void* x_planes, int x_shift, const void* w8, const float* scale, void* y,
                                    int64_t ldy, const void* residual, int64_t ldres, const float* gate,
                                    const float* next_scale, void* u_planes, int u_shift, float* ss_part, int M, int N,
                                    int K, int token_tile, int splits, int* status_word, void* stream);
int tybok_w8x3_geglu_packed_adarms(const void* u_planes, int u_shift, const float* ss_part, int ss_tiles, float eps,
                                   const float* bias_rows, const void* w8_packed, const float* scale_packed, void* h,
                                   int64_t ldh, void* h_planes, int out_shift, int M, int I, int K, int token_tile,
                                   int splits, int* status_word, void* stream);
int tybok_w8x3_qkv_rope_adarms(const void* u_planes, int u_shift, const float* ss_part, int ss_tiles, float eps,
                               const float* bias_rows, const void* w8_paired, const float* scale_paired, const int* pos,
                               const void* cos_table, const void* sin_table, void* q_out, void* k_cache, void* v_cache,
                               int B, int L, int H, int G, int D, int Lcap, int key_off, int K, int token_tile,
                               int splits, int* status_word, void* stream);

/* Enable (1) / disable (0) programmatic dependent launch for every kernel of this library
 * (process-wide; default 1).  With it, a kernel's weight prefetch overlaps the tail of the
 * previous kernel in the stream. */
void tybok_set_pdl(int enabled);

/* Tuning aid: with a device buffer of 16 int64 per CTA of the following GEMM launches, the
 * kernels record SM clock samples at their phase boundaries into it.  NULL (default) = off. */
void tybok_debug_set_trace(void* device_buffer);

/* Debugging aid: with a zeroed device buffer of 128 ints, every CTA of the following launches bumps
 * counter [kernel * 8 + stage] at its stage boundaries (stage 0 entered, 1 set-up done / tensor memory
 * held, 2 predecessor awaited, 3 main loop done, 4 leaving; kernels: 0-2 w8_gemm_kernel (8 warps, 16
 * warps, pair), 5 / 6 attention_prefill_kernel<256> / <128>, 7 qknorm_rope_store_kernel, 8 norm
 * kernels).  Read from another stream, it tells where a stalled chain stands.  NULL (default) = off. */
void tybok_debug_set_counters(void* device_buffer);

/* Test aid: how many SM clocks the epilogue warps of the following GEMM launches wait for their
 * accumulator before they give up, record TYBOK_DEV_TIMEOUT_EPILOGUE in the status word and skip
 * their stores (the producer, the MMA warp and the unwinding keep the production limit of about a
 * second).  0 (default) restores the production limit.  The error contract it lets a test
 * exercise is the reference's "error instead of exit" rule for its cooperative kernels
 * (tybok/policies/fastwam/kernels/coop_grid.h:20-27). */
void tybok_debug_set_epilogue_wait_limit(long long sm_clocks);

#ifdef __cplusplus
}
#endif
#endif /* TYBOK_B200_H */
